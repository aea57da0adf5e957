"""GPU parity tests of the prefill path, through the op surface and the C ABI.

Tolerance: atol = rtol = 2e-3 against the fp32 oracle (see _util.check_close)."""
import pytest
import torch

from _util import (bf16_tolerance_counts, check_close, check_close_bf16_by_keys, check_close_bf16_rows, load_prefill,
                   seeded_qkv)
from oracle import oracle as O

pytestmark = pytest.mark.gpu

F16 = (1, 1, 2)  # qtype F16, qblock_size, qtype_size: what the reference's callers pass


def run_masked(kerns, q, k, v, mask):
    out = torch.full(q.shape, float("nan"), dtype=q.dtype, device="cuda")
    kerns.flash_attn(*F16, q.cuda(), k.cuda(), v.cuda(), mask.cuda(), out)
    from minfer.kernels.torch_ext.ops import check_status
    check_status()
    return out


def run_causal(kerns, q, k, v):
    out = torch.full(q.shape, float("nan"), dtype=q.dtype, device="cuda")
    kerns.flash_attn_causal(q.cuda(), k.cuda(), v.cuda(), out)
    from minfer.kernels.torch_ext.ops import check_status
    check_status()
    return out


@pytest.mark.parametrize("name", ["prefill_causal_g4_d128", "prefill_window_g6_d128", "prefill_random_g1_d64",
                                  "prefill_causal_bf16_g8_d128", "prefill_causal_g4_d64"])
def test_golden_vectors_dense_mask(kerns, name):
    q, k, v, mask, want = load_prefill(name)
    got = run_masked(kerns, q, k, v, mask)
    check_close(got, want, name, bf16=q.dtype == torch.bfloat16)


@pytest.mark.parametrize("name", ["prefill_causal_g4_d128", "prefill_causal_bf16_g8_d128", "prefill_causal_g4_d64"])
def test_golden_vectors_causal_fast_path(kerns, name):
    q, k, v, mask, want = load_prefill(name)
    got = run_causal(kerns, q, k, v)
    check_close(got, want, name, bf16=q.dtype == torch.bfloat16)


def test_config1_shape_fp16_cast(kerns):
    """The fp32 CPU self-check configuration, run on the GPU on a float16 cast of its inputs."""
    q, k, v = seeded_qkv(0, 1, 8, 8, 256, 256, 64, torch.float16)
    want = O.prefill_oracle(q, k, v, causal=True)
    check_close(run_causal(kerns, q, k, v), want, "config1")


@pytest.mark.parametrize("L", [1, 5, 127, 128, 129, 383, 640])
@pytest.mark.parametrize("D,H,Hkv", [(128, 4, 1), (64, 6, 1), (128, 3, 3)])
def test_ragged_lengths_causal_and_mask_agree(kerns, L, D, H, Hkv):
    q, k, v = seeded_qkv(100 + L, 2, H, Hkv, L, L, D, torch.float16)
    want = O.prefill_oracle(q, k, v, causal=True)
    got_c = run_causal(kerns, q, k, v)
    got_m = run_masked(kerns, q, k, v, O.causal_mask(2, L))
    check_close(got_c, want, f"causal L={L}")
    check_close(got_m, want, f"masked L={L}")
    check_close(got_m, got_c.float().cpu(), f"masked vs causal L={L}")


@pytest.mark.parametrize("H,Hkv", [(4, 2), (3, 3)])
def test_block_sparse_mask_with_empty_tiles_and_rows(kerns, H, Hkv):
    """A mask whose 128 x 128 tiles are a mix of empty, full and ragged ones, with some query
    tiles that see nothing at all: exercises tile skipping for both slot pairings (two heads of
    a group / two row tiles of one head)."""
    B, L, D = 2, 700, 128
    g = torch.Generator().manual_seed(40 + H)
    q, k, v = seeded_qkv(41 + H, B, H, Hkv, L, L, D, torch.float16)
    nt = (L + 127) // 128
    kind = torch.randint(0, 3, (B, nt, nt), generator=g)          # 0 empty, 1 full, 2 ragged
    kind[:, 2, :] = 0                                              # a query tile that sees nothing
    kind[:, 4, :] = 0
    kind[:, 4, 1] = 2
    mask = torch.zeros(B, 1, L, L, dtype=torch.bool)
    for b in range(B):
        for i in range(nt):
            for j in range(nt):
                r, c = slice(i * 128, min(L, (i + 1) * 128)), slice(j * 128, min(L, (j + 1) * 128))
                if kind[b, i, j] == 1:
                    mask[b, 0, r, c] = True
                elif kind[b, i, j] == 2:
                    blk = torch.rand(r.stop - r.start, c.stop - c.start, generator=g) < 0.3
                    mask[b, 0, r, c] = blk
    want = O.attention_f64(q, k, v, mask=mask)
    got = run_masked(kerns, q, k, v, mask)
    check_close(got, want, "block sparse")
    assert torch.count_nonzero(got[:, :, 256:384]) == 0


@pytest.mark.parametrize("D", [128, 64])
def test_sparse_mask_over_many_key_tiles(kerns, D):
    """70 key tiles (three 32-tile groups of the kernel's tile flags): a band that leaves whole groups
    unvisited, query tiles that see far-away groups only or as well, rows that see nothing, and query
    heads of one kv head that fall into different work items (odd GQA group)."""
    B, H, Hkv, L = 1, 3, 1, 70 * 128 - 37
    q, k, v = seeded_qkv(91 + D, B, H, Hkv, L, L, D, torch.float16)
    rows = torch.arange(L)[:, None]
    cols = torch.arange(L)[None, :]
    m = (cols - rows).abs() <= 120                                                        # band around the diagonal
    m[128:256] = (cols >= 66 * 128 + 5) & (cols < 69 * 128 + 77) & ((rows[128:256] + cols) % 3 != 0)  # last group only
    m[300:310] = False                                                                    # rows without any visible key
    m[384:512] |= cols < 40                                                               # group 0 twice
    m[5000:5128] |= (cols < 130) | (cols >= L - 200)                                      # groups 0, 1 and 2 for one query tile
    mask = m[None, None].expand(B, 1, L, L).contiguous()
    want = O.attention_f64(q, k, v, mask=mask)
    got = run_masked(kerns, q, k, v, mask)
    check_close(got, want, f"sparse 70 tiles D={D}")
    assert torch.count_nonzero(got[:, :, 300:310]) == 0


def test_dense_mask_without_workspace_matches(kerns):
    """Through the C ABI: the same masked call with and without the tile-class workspace."""
    import ctypes
    from minfer.kernels.torch_ext import _lib
    B, H, Hkv, L, D = 1, 4, 2, 512, 128
    q, k, v = seeded_qkv(77, B, H, Hkv, L, L, D, torch.float16)
    mask = O.window_mask(B, L, 100)
    qd, kd, vd, md = q.cuda(), k.cuda(), v.cuda(), mask.cuda().contiguous()
    outs = []
    for use_ws in (True, False):
        out = torch.full((B, H, L, D), float("nan"), dtype=torch.float16, device="cuda")
        p = _lib.PrefillParams()
        p.q, p.k, p.v, p.out, p.mask = qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), out.data_ptr(), md.data_ptr()
        for i in range(3):
            p.q_stride[i], p.kv_stride[i], p.out_stride[i] = qd.stride(i), kd.stride(i), out.stride(i)
        p.batch, p.n_heads, p.n_kv_heads, p.seq_q, p.seq_k, p.head_dim = B, H, Hkv, L, L, D
        p.dtype, p.causal, p.softmax_scale, p.flags = _lib.F16, 0, 0.0, 0
        if use_ws:
            need = _lib.lib.minfer_attn_prefill_workspace_bytes(B, L, L)
            assert need == 16 + 16  # work-item counter + 4 x 4 tile classes
            ws = torch.empty(need, dtype=torch.uint8, device="cuda")
            p.workspace, p.workspace_bytes = ws.data_ptr(), need
        rc = _lib.lib.minfer_attn_prefill(ctypes.byref(p), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        assert rc == 0, _lib.strerror(rc)
        torch.cuda.synchronize()
        outs.append(out)
    check_close(outs[0], O.attention_f64(q, k, v, mask=mask), "window with workspace")
    assert torch.equal(outs[0], outs[1])


def _c_abi_call(q, k, v, out, mask=None, causal=True, ws=None, max_ctas=0, flags=0):
    import ctypes
    from minfer.kernels.torch_ext import _lib
    B, H, L, D = q.shape
    p = _lib.PrefillParams()
    p.q, p.k, p.v, p.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
    if mask is not None:
        p.mask = mask.data_ptr()
    for i in range(3):
        p.q_stride[i], p.kv_stride[i], p.out_stride[i] = q.stride(i), k.stride(i), out.stride(i)
    p.batch, p.n_heads, p.n_kv_heads, p.seq_q, p.seq_k, p.head_dim = B, H, k.size(1), L, k.size(2), D
    p.dtype = _lib.F16 if q.dtype == torch.float16 else _lib.BF16
    p.causal, p.softmax_scale, p.flags, p.max_ctas = int(causal), 0.0, flags, max_ctas
    if ws is not None:
        p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel()
    return _lib.lib.minfer_attn_prefill(ctypes.byref(p), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


@pytest.mark.parametrize("D,H,Hkv", [(128, 4, 2), (64, 3, 1)])
def test_grid_limit_and_workspace_do_not_change_the_result(kerns, D, H, Hkv):
    """max_ctas (a grid smaller than the SM count, which the multi-GPU harness uses to leave SMs to a
    collective) and the presence of a workspace (dynamic or static dealing of work items; tile classes
    of a dense mask) change the schedule only: every variant meets the tolerance and all are bitwise
    equal.  A non-zero reserved `flags` word is refused."""
    from minfer.kernels.torch_ext import _lib
    B, L = 2, 640
    q, k, v = seeded_qkv(78 + D, B, H, Hkv, L, L, D, torch.float16)
    mask = O.window_mask(B, L, 200).clone()
    mask[:, :, 130:140] = False
    wants = {"causal": O.prefill_oracle(q, k, v, causal=True), "mask": O.attention_f64(q, k, v, mask=mask)}
    qd, kd, vd, md = q.cuda(), k.cuda(), v.cuda(), mask.cuda().contiguous()
    ws = torch.empty(_lib.lib.minfer_attn_prefill_workspace_bytes(B, L, L), dtype=torch.uint8, device="cuda")
    for kind in ("causal", "mask"):
        outs = []
        for max_ctas in (0, 1, 5, 100000):
            for use_ws in (False, True):
                out = torch.full((B, H, L, D), float("nan"), dtype=torch.float16, device="cuda")
                rc = _c_abi_call(qd, kd, vd, out, mask=md if kind == "mask" else None, causal=kind == "causal",
                                 ws=ws if use_ws else None, max_ctas=max_ctas)
                assert rc == 0, _lib.strerror(rc)
                torch.cuda.synchronize()
                check_close(out, wants[kind], f"{kind} max_ctas={max_ctas} workspace={use_ws}")
                outs.append(out)
        assert all(torch.equal(outs[0], o) for o in outs[1:])
    out = torch.zeros(B, H, L, D, dtype=torch.float16, device="cuda")
    assert _c_abi_call(qd, kd, vd, out, flags=1) == 2      # MINFER_ATTN_EUNSUPPORTED
    assert _c_abi_call(qd, kd, vd, out, max_ctas=-1) == 1  # MINFER_ATTN_EINVAL


@pytest.mark.parametrize("D,dtype", [(64, torch.bfloat16), (128, torch.bfloat16), (64, torch.float16)])
def test_rows_without_a_visible_key_inside_mixed_tiles_are_zero(kerns, D, dtype):
    """Padding rows of a serving mask: rows with no True entry that sit inside tiles other rows do see.
    They must come out as exact zeros in every output type (a tiny positive exponential of a masked
    score is a normal bfloat16 number, so the sum of such a row is not zero by itself)."""
    B, H, Hkv, L = 2, 4, 2, 400
    q, k, v = seeded_qkv(300 + D, B, H, Hkv, L, L, D, dtype)
    g = torch.Generator().manual_seed(301)
    mask = torch.rand(B, 1, L, L, generator=g) < 0.4
    dead = torch.tensor([0, 5, 127, 128, 200, 201, 202, 399])
    mask[:, :, dead] = False
    mask[1, :, 256:384] = False                     # and a whole query tile
    want = O.attention_f64(q, k, v, mask=mask)
    for use_ws in (True, False):
        out = torch.full((B, H, L, D), float("nan"), dtype=dtype, device="cuda")
        if use_ws:
            kerns.flash_attn(*F16, q.cuda(), k.cuda(), v.cuda(), mask.cuda(), out)
        else:
            assert _c_abi_call(q.cuda(), k.cuda(), v.cuda(), out, mask=mask.cuda().contiguous(), causal=False) == 0
        torch.cuda.synchronize()
        check_close(out, want, f"dead rows D={D} ws={use_ws}", bf16=dtype == torch.bfloat16)
        assert torch.count_nonzero(out[:, :, dead]) == 0
        assert torch.count_nonzero(out[1, :, 256:384]) == 0


@pytest.mark.parametrize("Lq,Lk,H,Hkv,D", [(200, 712, 4, 2, 128), (1, 300, 3, 3, 64), (384, 385, 8, 1, 128)])
def test_causal_with_more_keys_than_queries(kerns, Lq, Lk, H, Hkv, D):
    """Chunked prefill: the queries are the LAST Lq positions of a length-Lk sequence (key j visible to
    query i iff j <= i + Lk - Lq)."""
    g = torch.Generator().manual_seed(Lq + Lk)
    q = torch.randn(2, H, Lq, D, generator=g).half()
    k = torch.randn(2, Hkv, Lk, D, generator=g).half()
    v = torch.randn(2, Hkv, Lk, D, generator=g).half()
    want = O.attention_f64(q, k, v, causal=True)
    check_close(run_causal(kerns, q, k, v), want, f"Lq={Lq} Lk={Lk}")


def test_explicit_softmax_scale_through_the_c_abi():
    import ctypes
    from minfer.kernels.torch_ext import _lib
    B, H, Hkv, L, D, scale = 1, 4, 2, 300, 128, 0.05
    q, k, v = seeded_qkv(91, B, H, Hkv, L, L, D, torch.float16)
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    out = torch.full((B, H, L, D), float("nan"), dtype=torch.float16, device="cuda")
    p = _lib.PrefillParams()
    p.q, p.k, p.v, p.out = qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), out.data_ptr()
    for i in range(3):
        p.q_stride[i], p.kv_stride[i], p.out_stride[i] = qd.stride(i), kd.stride(i), out.stride(i)
    p.batch, p.n_heads, p.n_kv_heads, p.seq_q, p.seq_k, p.head_dim = B, H, Hkv, L, L, D
    p.dtype, p.causal, p.softmax_scale, p.flags = _lib.F16, 1, scale, 0
    assert _lib.lib.minfer_attn_prefill(ctypes.byref(p), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)) == 0
    torch.cuda.synchronize()
    check_close(out, O.attention_f64(q, k, v, causal=True, scale=scale), "explicit scale")


def test_adversarial_score_growth(kerns):
    """Scores that grow by far more than 2^8 from one key tile to the next force the reference maximum to
    move (and O to be rescaled) on every tile; and a huge early outlier must not poison later tiles."""
    B, H, Hkv, L, D = 1, 2, 1, 640, 128
    g = torch.Generator().manual_seed(17)
    q = torch.randn(B, H, L, D, generator=g).half()
    k = torch.randn(B, Hkv, L, D, generator=g).half()
    v = torch.randn(B, Hkv, L, D, generator=g).half()
    k *= (1 + torch.arange(L) // 128 * 6).view(1, 1, L, 1).half()      # later key tiles score much higher
    k[0, 0, 3] *= 40                                                    # an early outlier
    want = O.attention_f64(q, k, v, causal=True)
    check_close(run_causal(kerns, q, k, v), want, "growing scores")
    check_close(run_masked(kerns, q, k, v, O.causal_mask(B, L)), want, "growing scores, dense mask")


@pytest.mark.parametrize("D,dtype", [(128, torch.float16), (64, torch.float16), (128, torch.bfloat16)])
def test_scores_that_jump_late_in_a_row(kerns, D, dtype):
    """A few keys far into the sequence carry scores tens of units above everything before them - for some
    rows only, positive for some and negative for others - in the first half, the second half and the last
    chunk of their 128-key tiles: whatever reference the kernel keeps for a row has to move in the middle of
    a tile, after part of the tile's P may already have been consumed."""
    B, H, Hkv, L = 1, 4, 2, 768
    q, k, v = seeded_qkv(55 + D, B, H, Hkv, L, L, D, dtype)
    k = k.float()
    for pos, gain in ((128 + 10, 40.0), (128 + 100, 25.0), (256 + 127, 60.0), (512 + 64, 30.0), (640 + 3, 80.0)):
        k[:, :, pos] *= gain
    k = k.to(dtype)
    want = O.prefill_oracle(q, k, v, causal=True)
    check_close(run_causal(kerns, q, k, v), want, "late jumps, causal entry", bf16=dtype == torch.bfloat16)
    check_close(run_masked(kerns, q, k, v, O.causal_mask(B, L)), want, "late jumps, dense mask",
                bf16=dtype == torch.bfloat16)


def test_bf16_medium(kerns, record_property):
    q, k, v = seeded_qkv(7, 1, 8, 1, 1024, 1024, 128, torch.bfloat16)
    want = O.prefill_oracle(q, k, v, causal=True)
    got = run_causal(kerns, q, k, v)
    counts = bf16_tolerance_counts(got, want)
    print("bf16 L=1024:", counts)
    record_property("bf16_counts", counts)
    check_close_bf16_rows(got, want, 0, "bf16 L=1024")
    assert counts["fail_plain_2e-3"] <= 1e-4 * counts["elements"]


def test_config4_long_context_bf16_shard_and_full(kerns, record_property):
    """The long-context configuration: B=1, 64 query / 8 kv heads, D=128, L=32768, bfloat16, seed 3.
    One GPU's share under the kv-head-group partition (kv head g, query heads 8g..8g+7) is run as its own
    call and must equal the same heads of the full 64-head call bit for bit; row blocks at the start, around
    rows 2-3 k, in the middle and at the end are checked against the fp64-accumulating oracle.  The three
    bfloat16 tolerance counts are printed for each block."""
    B, H, Hkv, L, D, g_shard = 1, 64, 8, 32768, 128, 5
    gen = torch.Generator().manual_seed(3)
    q = torch.randn(B, H, L, D, generator=gen).bfloat16()
    k = torch.randn(B, Hkv, L, D, generator=gen).bfloat16()
    v = torch.randn(B, Hkv, L, D, generator=gen).bfloat16()
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    full = torch.full((B, H, L, D), float("nan"), dtype=torch.bfloat16, device="cuda")
    kerns.flash_attn_causal(qc, kc, vc, full)
    hs = slice(8 * g_shard, 8 * g_shard + 8)
    part = torch.full((B, 8, L, D), float("nan"), dtype=torch.bfloat16, device="cuda")
    kerns.flash_attn_causal(qc[:, hs], kc[:, g_shard:g_shard + 1], vc[:, g_shard:g_shard + 1], part)
    from minfer.kernels.torch_ext.ops import check_status
    check_status()
    assert torch.isfinite(full).all()
    assert torch.equal(part, full[:, hs]), "a kv-head-group shard differs from the same heads of the full call"
    assert torch.equal(full[:, :, 0], vc[:, :, 0].repeat_interleave(H // Hkv, dim=1))
    totals = {"elements": 0, "fail_plain_2e-3": 0, "fail_with_half_ulp": 0, "rounded_oracle_fails_plain": 0}
    qs, ks, vs = q[:, hs], k[:, g_shard:g_shard + 1], v[:, g_shard:g_shard + 1]
    for rows in ((0, 128), (2048, 2112), (2976, 3040), (16352, 16416), (L - 128, L)):
        want = O.attention_f64(qs, ks, vs, causal=True, rows=rows)
        got = part[:, :, rows[0]:rows[1]]
        counts = bf16_tolerance_counts(got, want)
        print(f"config4 shard rows {rows}:", counts)
        for key in totals:
            totals[key] += counts[key]
        check_close_bf16_rows(got, want, rows[0], f"config4 rows={rows}")
    # the first rows of two other heads of the full call, where |out| is largest
    for h in (0, 63):
        want = O.attention_f64(q[:, h:h + 1], k[:, h // 8:h // 8 + 1], v[:, h // 8:h // 8 + 1], causal=True, rows=(0, 256))
        counts = bf16_tolerance_counts(full[:, h:h + 1, :256], want)
        print(f"config4 full head {h} rows (0, 256):", counts)
        for key in totals:
            totals[key] += counts[key]
        check_close_bf16_rows(full[:, h:h + 1, :256], want, 0, f"config4 head {h}")
    record_property("bf16_counts", totals)
    print("config4 totals:", totals)
    assert totals["fail_with_half_ulp"] <= 1e-5 * totals["elements"]
    assert totals["fail_plain_2e-3"] <= 1e-4 * totals["elements"]


def test_strided_views_as_the_reference_callers_pass(kerns):
    """[B, L, H*D] storage viewed as [B, H, L, D] (test/kernels.py:230-237 of the reference)."""
    B, L, H, Hkv, D = 2, 512, 12, 2, 128
    g = torch.Generator().manual_seed(5)
    q = torch.randn(B, L, H * D, generator=g).half().view(B, L, H, D).transpose(1, 2)
    k = torch.randn(B, L, Hkv * D, generator=g).half().view(B, L, Hkv, D).transpose(1, 2)
    v = torch.randn(B, L, Hkv * D, generator=g).half().view(B, L, Hkv, D).transpose(1, 2)
    assert not q.is_contiguous()
    want = O.prefill_oracle(q, k, v, causal=True)
    out = torch.zeros(B, H, L, D, dtype=torch.float16, device="cuda")
    kerns.flash_attn(*F16, q.cuda(), k.cuda(), v.cuda(), O.causal_mask(B, L).cuda(), out)
    check_close(out, want, "strided")
    # strided output too
    out2 = torch.zeros(B, L, H * D, dtype=torch.float16, device="cuda").view(B, L, H, D).transpose(1, 2)
    kerns.flash_attn_causal(q.cuda(), k.cuda(), v.cuda(), out2)
    check_close(out2, want, "strided out")


def test_head_slices_for_kv_group_sharding(kerns):
    """A shard of heads (a strided slice) gives the same rows as the full call."""
    q, k, v = seeded_qkv(9, 1, 16, 4, 384, 384, 128, torch.float16)
    full = run_causal(kerns, q, k, v)
    qs, ks, vs = q.cuda()[:, 8:12], k.cuda()[:, 2:3], v.cuda()[:, 2:3]
    part = torch.zeros(1, 4, 384, 128, dtype=torch.float16, device="cuda")
    kerns.flash_attn_causal(qs, ks, vs, part)
    assert torch.equal(part, full[:, 8:12])


def test_reference_test_flash_attn_shapes():
    """The reference's own test of this op (test/kernels.py:222-298) with its imports, its argument
    passing (the qtype as the enum member, sizes from GGML_QUANT_SIZES), its shapes (B=8 L=4096 48/8 heads
    D=128, inputs as transposed views, K/V scaled by 1/sqrt(D)) and its two masks (causal, sliding window
    256): expected values through refs.flash_attn on expanded K/V at its atol = 3e-1 - and then, because
    that tolerance is as large as the values themselves, sampled row blocks at this path's own tolerance
    against the fp32 oracle."""
    from minfer.kernels import refs
    from minfer.kernels import KernelBackend
    from minfer.const import GGMLQuantizationType, GGML_QUANT_SIZES
    import minfer.kernels.torch_ext  # noqa: F401  (what the reference's conftest.py imports)

    kerns = KernelBackend("torch_ext")
    B, L, H, Hkv, D = 8, 4096, 48, 8, 128
    qtype = GGMLQuantizationType.F16
    qblock_size, qtype_size = GGML_QUANT_SIZES[qtype]
    g = torch.Generator().manual_seed(1234)
    q = torch.randn(B, L, H * D, generator=g).half().cuda().view(B, L, H, D).transpose(1, 2)
    k = ((1 / D ** 0.5) * torch.randn(B, L, Hkv * D, generator=g)).half().cuda().view(B, L, Hkv, D).transpose(1, 2)
    v = ((1 / D ** 0.5) * torch.randn(B, L, Hkv * D, generator=g)).half().cuda().view(B, L, Hkv, D).transpose(1, 2)
    for kind in ("causal", "window"):
        mask = (O.causal_mask(B, L) if kind == "causal" else O.window_mask(B, L, 256)).cuda()
        out = torch.zeros(B, H, L, D, dtype=torch.float16).cuda()
        kerns.flash_attn(qtype, qblock_size, qtype_size, q, k, v, mask, out)
        torch.cuda.synchronize()
        n_rep = H // Hkv
        expected = refs.flash_attn(q, k.repeat_interleave(n_rep, dim=1), v.repeat_interleave(n_rep, dim=1), mask)
        assert torch.allclose(expected.cpu(), out.cpu(), atol=3e-1), "flash_attn"
        del expected
        for b, rows in ((0, (0, 64)), (3, (2000, 2032)), (7, (4064, 4096))):
            want = O.attention_f64(q[b:b + 1].cpu(), k[b:b + 1].cpu(), v[b:b + 1].cpu(), mask=mask[b:b + 1].cpu(), rows=rows)
            check_close(out[b:b + 1, :, rows[0]:rows[1]], want, f"{kind} b={b} rows={rows}")
        del mask, out
        torch.cuda.empty_cache()


def test_config2_full_size_properties(kerns):
    """Llama-3-8B-shaped prefill at full size: sampled row blocks against the oracle, plus
    size-independent properties: row 0 reproduces V's first row, a permutation of the batch
    permutes the output, and the run is bitwise repeatable."""
    B, H, Hkv, L, D = 4, 32, 8, 4096, 128
    q, k, v = seeded_qkv(1, B, H, Hkv, L, L, D, torch.float16)
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    out = torch.full((B, H, L, D), float("nan"), dtype=torch.float16, device="cuda")
    kerns.flash_attn_causal(qc, kc, vc, out)
    from minfer.kernels.torch_ext.ops import check_status
    check_status()
    assert torch.isfinite(out).all()
    for b, rows in ((0, (0, 40)), (1, (1000, 1024)), (2, (2040, 2060)), (3, (4080, 4096))):
        want = O.attention_f64(q[b:b + 1], k[b:b + 1], v[b:b + 1], causal=True, rows=rows)
        check_close(out[b:b + 1, :, rows[0]:rows[1]], want, f"config2 b={b} rows={rows}")
    # the first token attends only itself
    assert torch.equal(out[:, :, 0, :], vc[:, :, 0, :].repeat_interleave(H // Hkv, dim=1))
    perm = torch.tensor([2, 0, 3, 1], device="cuda")
    out_p = torch.empty_like(out)
    kerns.flash_attn_causal(qc[perm].contiguous(), kc[perm].contiguous(), vc[perm].contiguous(), out_p)
    assert torch.equal(out_p, out[perm])
    out_r = torch.empty_like(out)
    kerns.flash_attn_causal(qc, kc, vc, out_r)
    assert torch.equal(out_r, out)


def test_argument_errors_raise(kerns):
    q = torch.zeros(1, 4, 128, 128, dtype=torch.float16, device="cuda")
    k = torch.zeros(1, 2, 128, 128, dtype=torch.float16, device="cuda")
    m = torch.ones(1, 1, 128, 128, dtype=torch.bool, device="cuda")
    out = torch.zeros_like(q)
    with pytest.raises(RuntimeError):
        kerns.flash_attn(*F16, q.float(), k.float(), k.float(), m, out.float())      # dtype
    with pytest.raises(RuntimeError):
        kerns.flash_attn(*F16, q, k, k[:, :, :64], m, out)                            # k/v shapes differ
    with pytest.raises(RuntimeError):
        kerns.flash_attn(*F16, q, k, k, m[..., :64], out)                             # mask shape
    with pytest.raises(RuntimeError):
        kerns.flash_attn(*F16, q, k, k, m.to(torch.uint8), out)                       # mask dtype
    q96 = torch.zeros(1, 4, 128, 96, dtype=torch.float16, device="cuda")
    with pytest.raises(RuntimeError):
        kerns.flash_attn_causal(q96, q96, q96, torch.zeros_like(q96))                 # head_dim
    with pytest.raises(RuntimeError):
        kerns.flash_attn_causal(q, k[:, :, :64], k[:, :, :64], out)                   # fewer keys than queries


def test_opcheck(kerns):
    """torch.library.opcheck on the ops (the reference does this for gemm only, test/kernels.py:167-170)."""
    q, k, v = seeded_qkv(3, 1, 4, 2, 128, 128, 64, torch.float16)
    q, k, v = q.cuda(), k.cuda(), v.cuda()
    out = torch.zeros_like(q)
    mask = O.causal_mask(1, 128).cuda()
    torch.library.opcheck(torch.ops.minfer.flash_attn.default, (1, 1, 2, q, k, v, mask, out),
                          test_utils=("test_schema", "test_faketensor"))
    torch.library.opcheck(torch.ops.minfer.flash_attn_causal.default, (q, k, v, out),
                          test_utils=("test_schema", "test_faketensor"))


@pytest.mark.parametrize("seed", range(12))
def test_random_shapes_against_the_oracle(kerns, seed):
    """Seeded random draws of everything a caller may vary - batch, heads, GQA group (powers of two or not),
    sequence lengths (ragged against the 128-row tiles, more keys than queries), head_dim, type, layout
    (contiguous or the reference callers' transposed views), causal entry or a random dense mask."""
    g = torch.Generator().manual_seed(9000 + seed)
    r = lambda lo, hi: int(torch.randint(lo, hi + 1, (1,), generator=g))  # noqa: E731
    B, Hkv, group = r(1, 3), r(1, 3), [1, 2, 3, 4, 6, 8][r(0, 5)]
    H, D = Hkv * group, [64, 128][r(0, 1)]
    dtype = [torch.float16, torch.bfloat16][r(0, 1)]
    Lq = r(1, 700)
    causal = r(0, 1) == 1
    Lk = Lq + (r(0, 300) if causal and r(0, 1) else 0)
    transposed = r(0, 1) == 1
    if transposed:
        q = torch.randn(B, Lq, H * D, generator=g).to(dtype).view(B, Lq, H, D).transpose(1, 2)
        k = torch.randn(B, Lk, Hkv * D, generator=g).to(dtype).view(B, Lk, Hkv, D).transpose(1, 2)
        v = torch.randn(B, Lk, Hkv * D, generator=g).to(dtype).view(B, Lk, Hkv, D).transpose(1, 2)
    else:
        q = torch.randn(B, H, Lq, D, generator=g).to(dtype)
        k = torch.randn(B, Hkv, Lk, D, generator=g).to(dtype)
        v = torch.randn(B, Hkv, Lk, D, generator=g).to(dtype)
    what = f"seed {seed}: B={B} H={H} Hkv={Hkv} D={D} Lq={Lq} Lk={Lk} {dtype} causal={causal} transposed={transposed}"
    if causal:
        want = O.attention_f64(q, k, v, causal=True)
        got = run_causal(kerns, q, k, v)
        n_keys = (torch.arange(Lq) + 1 + Lk - Lq).view(1, 1, Lq, 1)
    else:
        mask = torch.rand(B, 1, Lq, Lk, generator=g) < [0.05, 0.5, 0.95][r(0, 2)]
        mask[:, :, :, 0] |= torch.rand(B, 1, Lq, generator=g) < 0.9      # most rows see at least one key, some none
        want = O.attention_f64(q, k, v, mask=mask)
        got = run_masked(kerns, q, k, v, mask)
        n_keys = mask.sum(-1, keepdim=True)
    if dtype == torch.bfloat16:
        check_close_bf16_by_keys(got, want, n_keys, what)    # a sparse random mask makes every row a short one
    else:
        check_close(got, want, what)
