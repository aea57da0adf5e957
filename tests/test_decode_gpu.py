"""GPU parity tests of the split-KV decode path.  Tolerance: atol = rtol = 2e-3 vs the fp32 oracle."""
import ctypes

import pytest
import torch

from _util import check_close, load_decode
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def run_decode(kerns, q, kc, vc, lens):
    out = torch.full(q.shape, float("nan"), dtype=q.dtype, device="cuda")
    kerns.flash_attn_decode(q.cuda(), kc.cuda(), vc.cuda(), lens.cuda().to(torch.int32), out)
    torch.cuda.synchronize()
    return out


@pytest.mark.parametrize("name", ["decode_g4_d128", "decode_g1_d64_bf16", "decode_g6_d128"])
def test_golden_vectors(kerns, name):
    q, k, v, lens, want = load_decode(name)
    check_close(run_decode(kerns, q, k, v, lens), want, name, bf16=q.dtype == torch.bfloat16)


@pytest.mark.parametrize("D,H,Hkv,dtype", [(128, 32, 8, torch.float16), (64, 32, 8, torch.float16),
                                            (128, 16, 2, torch.bfloat16), (128, 5, 5, torch.float16),
                                            (64, 32, 2, torch.float16)])
def test_ragged_lengths(kerns, D, H, Hkv, dtype):
    B, Lmax = 9, 2100
    g = torch.Generator().manual_seed(31 + D + H)
    q = torch.randn(B, H, 1, D, generator=g).to(dtype)
    kc = torch.randn(B, Hkv, Lmax, D, generator=g).to(dtype)
    vc = torch.randn(B, Hkv, Lmax, D, generator=g).to(dtype)
    lens = torch.tensor([1, 2, 15, 16, 17, 511, 512, 513, 2100], dtype=torch.int32)
    want = O.decode_oracle(q, kc, vc, lens)
    check_close(run_decode(kerns, q, kc, vc, lens), want, "ragged", bf16=dtype == torch.bfloat16)


def test_padding_is_never_read(kerns):
    """NaN beyond lens[b] must not reach the output; a zero-length sequence yields zeros."""
    B, H, Hkv, Lmax, D = 3, 8, 2, 700, 128
    g = torch.Generator().manual_seed(77)
    q = torch.randn(B, H, 1, D, generator=g).half()
    kc = torch.randn(B, Hkv, Lmax, D, generator=g).half()
    vc = torch.randn(B, Hkv, Lmax, D, generator=g).half()
    lens = torch.tensor([0, 300, 641], dtype=torch.int32)
    want = O.decode_oracle(q, kc, vc, torch.tensor([1, 300, 641]))
    for b in range(B):
        kc[b, :, int(lens[b]):] = float("nan")
        vc[b, :, int(lens[b]):] = float("nan")
    got = run_decode(kerns, q, kc, vc, lens)
    assert torch.count_nonzero(got[0]) == 0
    check_close(got[1:], want[1:], "padding")


def test_strided_cache_views(kerns):
    """Cache stored [B, Lmax, Hkv, D] and viewed as [B, Hkv, Lmax, D]; batch-sliced shard."""
    B, H, Hkv, Lmax, D = 4, 8, 2, 600, 128
    g = torch.Generator().manual_seed(78)
    q = torch.randn(B, H, 1, D, generator=g).half()
    kc = torch.randn(B, Lmax, Hkv, D, generator=g).half().transpose(1, 2)
    vc = torch.randn(B, Lmax, Hkv, D, generator=g).half().transpose(1, 2)
    lens = torch.tensor([600, 77, 512, 130], dtype=torch.int32)
    want = O.decode_oracle(q, kc, vc, lens)
    qd, kd, vd, ld = q.cuda(), kc.cuda(), vc.cuda(), lens.cuda()
    assert not kd.is_contiguous()
    out = torch.zeros(B, H, 1, D, dtype=torch.float16, device="cuda")
    kerns.flash_attn_decode(qd, kd, vd, ld, out)
    check_close(out, want, "strided cache")
    part = torch.zeros(2, H, 1, D, dtype=torch.float16, device="cuda")
    kerns.flash_attn_decode(qd[2:], kd[2:], vd[2:], ld[2:].contiguous(), part)
    assert torch.equal(part, out[2:])


@pytest.mark.parametrize("chunk", [64, 256, 1024, 8192])
def test_chunk_sizes_through_the_c_abi(chunk):
    """Any chunk (split) size gives the same answer within tolerance: called through the C ABI directly."""
    from minfer.kernels.torch_ext import _lib
    B, H, Hkv, Lmax, D = 5, 8, 2, 1500, 128
    g = torch.Generator().manual_seed(79)
    q = torch.randn(B, H, 1, D, generator=g).half()
    kc = torch.randn(B, Hkv, Lmax, D, generator=g).half()
    vc = torch.randn(B, Hkv, Lmax, D, generator=g).half()
    lens = torch.tensor([1500, 3, 1024, 1025, 64], dtype=torch.int32)
    want = O.decode_oracle(q, kc, vc, lens)
    qd, kd, vd, ld = q.cuda(), kc.cuda(), vc.cuda(), lens.cuda()
    out = torch.zeros(B, H, 1, D, dtype=torch.float16, device="cuda")
    need = _lib.lib.minfer_attn_decode_workspace_bytes(B, H, Lmax, D, chunk)
    ws = torch.full((need,), 0xFF, dtype=torch.uint8, device="cuda")   # the workspace may hold anything
    p = _lib.DecodeParams()
    p.q, p.k_cache, p.v_cache, p.lens, p.out = qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), ld.data_ptr(), out.data_ptr()
    p.workspace, p.workspace_bytes = ws.data_ptr(), need
    p.batch, p.n_heads, p.n_kv_heads, p.max_len, p.head_dim = B, H, Hkv, Lmax, D
    p.dtype, p.chunk, p.softmax_scale = _lib.F16, chunk, 0.0
    for i in range(2):
        p.q_stride[i], p.out_stride[i] = qd.stride(i), out.stride(i)
    for i in range(3):
        p.kv_stride[i] = kd.stride(i)
    rc = _lib.lib.minfer_attn_decode(ctypes.byref(p), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, _lib.strerror(rc)
    torch.cuda.synchronize()
    check_close(out, want, f"chunk={chunk}")
    # repeated calls, back to back on the same workspace, give the same bits
    first = out.clone()
    for _ in range(20):
        out.fill_(float("nan"))
        assert _lib.lib.minfer_attn_decode(ctypes.byref(p), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)) == 0
        assert torch.equal(out, first)
    p.workspace_bytes = need - 1
    assert _lib.lib.minfer_attn_decode(ctypes.byref(p), None) == 5


def test_config3_full_size(kerns):
    """Batch 64, 32/8 heads, D=128, lengths uniform in [512, 8192], cache padded to 8192 and
    filled everywhere (so an over-read would show): every sequence against the oracle."""
    B, H, Hkv, Lmax, D = 64, 32, 8, 8192, 128
    g = torch.Generator().manual_seed(2)
    lens = torch.randint(512, 8193, (B,), generator=g, dtype=torch.int32)
    lens[0], lens[1] = 512, 8192
    q = torch.randn(B, H, 1, D, generator=g).half()
    kd = torch.randn(B, Hkv, Lmax, D, device="cuda", dtype=torch.float16)
    vd = torch.randn(B, Hkv, Lmax, D, device="cuda", dtype=torch.float16)
    out = torch.full((B, H, 1, D), float("nan"), dtype=torch.float16, device="cuda")
    kerns.flash_attn_decode(q.cuda(), kd, vd, lens.cuda(), out)
    torch.cuda.synchronize()
    for b0 in range(0, B, 16):
        want = O.decode_oracle(q[b0:b0 + 16], kd[b0:b0 + 16].cpu(), vd[b0:b0 + 16].cpu(), lens[b0:b0 + 16])
        check_close(out[b0:b0 + 16], want, f"config3 b={b0}")
    out2 = torch.empty_like(out)
    kerns.flash_attn_decode(q.cuda(), kd, vd, lens.cuda(), out2)
    assert torch.equal(out, out2)


def test_argument_errors_raise(kerns):
    q = torch.zeros(2, 8, 1, 128, dtype=torch.float16, device="cuda")
    kc = torch.zeros(2, 2, 256, 128, dtype=torch.float16, device="cuda")
    lens = torch.tensor([5, 6], dtype=torch.int32, device="cuda")
    out = torch.zeros_like(q)
    with pytest.raises(RuntimeError):
        kerns.flash_attn_decode(q, kc, kc, lens.long(), out)
    with pytest.raises(RuntimeError):
        kerns.flash_attn_decode(q, kc, kc, lens[:1], out)
    with pytest.raises(RuntimeError):
        kerns.flash_attn_decode(q.expand(2, 8, 2, 128), kc, kc, lens, out.expand(2, 8, 2, 128))


@pytest.mark.parametrize("seed", range(8))
def test_random_shapes_against_the_oracle(kerns, seed):
    """Seeded random batch, heads, GQA group up to 16, head_dim, type, padded length and lengths (empty sequences
    included), contiguous or [B, Lmax, Hkv, D]-stored caches."""
    g = torch.Generator().manual_seed(7000 + seed)
    r = lambda lo, hi: int(torch.randint(lo, hi + 1, (1,), generator=g))  # noqa: E731
    B, Hkv, group = r(1, 9), r(1, 4), [1, 2, 3, 4, 5, 8, 16][r(0, 6)]
    H, D = Hkv * group, [64, 128][r(0, 1)]
    dtype = [torch.float16, torch.bfloat16][r(0, 1)]
    Lmax = r(1, 3000)
    lens = torch.randint(0, Lmax + 1, (B,), generator=g, dtype=torch.int32)
    lens[r(0, B - 1)] = Lmax
    q = torch.randn(B, H, 1, D, generator=g).to(dtype)
    if r(0, 1):
        kc = torch.randn(B, Lmax, Hkv, D, generator=g).to(dtype).transpose(1, 2)
        vc = torch.randn(B, Lmax, Hkv, D, generator=g).to(dtype).transpose(1, 2)
    else:
        kc = torch.randn(B, Hkv, Lmax, D, generator=g).to(dtype)
        vc = torch.randn(B, Hkv, Lmax, D, generator=g).to(dtype)
    want = O.attention_f64(q, kc, vc, lens=lens)
    got = run_decode(kerns, q, kc, vc, lens)
    assert torch.count_nonzero(got[lens == 0]) == 0
    live = lens > 0
    what = f"seed {seed}: B={B} H={H} Hkv={Hkv} D={D} Lmax={Lmax} {dtype}"
    if dtype == torch.bfloat16:
        from _util import check_close_bf16_by_keys
        check_close_bf16_by_keys(got[live], want[live], lens[live].view(-1, 1, 1, 1), what)
    else:
        check_close(got[live], want[live], what)
