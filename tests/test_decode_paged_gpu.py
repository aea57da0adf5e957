"""GPU parity tests of decode over a paged KV cache.

The oracle is the contiguous decode oracle run on the cache gathered from the pages; the paged kernel must
also agree bit for bit with the contiguous kernel on that gathered cache (same arithmetic, other addresses).
Tolerance against the oracle: atol = rtol = 2e-3."""
import ctypes

import pytest
import torch

from _util import check_close
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def make_paged(B, Hkv, D, page, lens, dtype, seed, spare=7):
    """Random pools with a shuffled page assignment; returns pools, table and the gathered contiguous caches."""
    g = torch.Generator().manual_seed(seed)
    max_pages = (int(max(lens)) + page - 1) // page + 1        # one table column is never needed
    n_pages = B * max_pages + spare
    kp = torch.randn(n_pages, Hkv, page, D, generator=g).to(dtype)
    vp = torch.randn(n_pages, Hkv, page, D, generator=g).to(dtype)
    perm = torch.randperm(n_pages, generator=g)[: B * max_pages].reshape(B, max_pages).to(torch.int32)
    table = perm.clone()
    for b in range(B):                                         # entries past the sequence are garbage on purpose
        used = (int(lens[b]) + page - 1) // page
        table[b, used:] = 2 ** 30
    kc = kp[perm.long()].permute(0, 2, 1, 3, 4).reshape(B, Hkv, max_pages * page, D).contiguous()
    vc = vp[perm.long()].permute(0, 2, 1, 3, 4).reshape(B, Hkv, max_pages * page, D).contiguous()
    return kp, vp, table, kc, vc


@pytest.mark.parametrize("D,H,Hkv,page,dtype", [(128, 32, 8, 16, torch.float16), (128, 8, 2, 64, torch.bfloat16),
                                                 (64, 12, 2, 256, torch.float16), (128, 5, 5, 48, torch.float16)])
def test_paged_matches_oracle_and_contiguous_kernel(kerns, D, H, Hkv, page, dtype):
    lens = torch.tensor([1, 16, 17, 700, 1025, 2048, 333], dtype=torch.int32)
    B = lens.numel()
    kp, vp, table, kc, vc = make_paged(B, Hkv, D, page, lens, dtype, seed=5 + D + page)
    g = torch.Generator().manual_seed(99)
    q = torch.randn(B, H, 1, D, generator=g).to(dtype)
    want = O.decode_paged_oracle(q, kp, vp, table, lens)
    out_p = torch.full(q.shape, float("nan"), dtype=dtype, device="cuda")
    kerns.flash_attn_decode_paged(q.cuda(), kp.cuda(), vp.cuda(), table.cuda(), lens.cuda(), out_p)
    out_c = torch.full(q.shape, float("nan"), dtype=dtype, device="cuda")
    kerns.flash_attn_decode(q.cuda(), kc.cuda(), vc.cuda(), lens.cuda(), out_c)
    torch.cuda.synchronize()
    check_close(out_p, want, f"paged D={D} page={page}", bf16=dtype == torch.bfloat16)
    assert torch.equal(out_p, out_c)


def test_paged_q8_through_the_c_abi(kerns):
    """Q8_0 pools: strides in bytes, pages of 32 rows; equals the contiguous Q8_0 kernel on the gathered cache."""
    from minfer.kernels.torch_ext import _lib
    B, H, Hkv, D, page = 3, 8, 2, 128, 32
    lens = torch.tensor([40, 1000, 513], dtype=torch.int32)
    g = torch.Generator().manual_seed(123)
    max_pages = 33
    n_pages = B * max_pages
    kf = torch.randn(n_pages, Hkv, page, D, generator=g)
    vf = torch.randn(n_pages, Hkv, page, D, generator=g)
    kq = O.q8_0_quantize(kf)   # uint8 [n_pages, Hkv, page, D / 32 * 34]
    vq = O.q8_0_quantize(vf)
    perm = torch.randperm(n_pages, generator=g).reshape(B, max_pages).to(torch.int32)
    kc = kq[perm.long()].permute(0, 2, 1, 3, 4).reshape(B, Hkv, max_pages * page, -1).contiguous()
    vc = vq[perm.long()].permute(0, 2, 1, 3, 4).reshape(B, Hkv, max_pages * page, -1).contiguous()
    q = torch.randn(B, H, 1, D, generator=g).half()
    out_c = torch.full(q.shape, float("nan"), dtype=torch.float16, device="cuda")
    kerns.flash_attn_decode_q8(q.cuda(), kc.cuda(), vc.cuda(), lens.cuda(), out_c)

    qd, kd, vd, td, ld = q.cuda(), kq.cuda(), vq.cuda(), perm.cuda(), lens.cuda()
    out_p = torch.full(q.shape, float("nan"), dtype=torch.float16, device="cuda")
    p = _lib.DecodeParams()
    p.q, p.k_cache, p.v_cache, p.lens, p.out = qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), ld.data_ptr(), out_p.data_ptr()
    p.batch, p.n_heads, p.n_kv_heads, p.head_dim = B, H, Hkv, D
    p.page_size, p.table_stride, p.block_table = page, max_pages, td.data_ptr()
    p.n_pages = n_pages
    p.max_len = page * max_pages
    p.dtype, p.chunk, p.softmax_scale, p.kv_format = _lib.F16, 0, 0.0, _lib.KV_Q8_0
    for i in range(2):
        p.q_stride[i], p.out_stride[i] = qd.stride(i), out_p.stride(i)
    for i in range(3):
        p.kv_stride[i] = kd.stride(i)          # uint8 tensor: element strides are byte strides
    need = _lib.lib.minfer_attn_decode_workspace_bytes(B, H, p.max_len, D, 0)
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    p.workspace, p.workspace_bytes = ws.data_ptr(), need
    rc = _lib.lib.minfer_attn_decode(ctypes.byref(p), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, _lib.strerror(rc)
    torch.cuda.synchronize()
    assert torch.isfinite(out_p).all()
    assert torch.equal(out_p, out_c)


def test_paged_argument_errors():
    from minfer.kernels.torch_ext import _lib
    p = _lib.DecodeParams()
    buf = torch.zeros(1 << 16, dtype=torch.float16, device="cuda")
    tab = torch.zeros(64, dtype=torch.int32, device="cuda")
    p.q = p.k_cache = p.v_cache = p.out = buf.data_ptr()
    p.lens = tab.data_ptr()
    p.batch, p.n_heads, p.n_kv_heads, p.head_dim, p.max_len = 1, 4, 2, 128, 128
    p.q_stride[0], p.q_stride[1], p.out_stride[0], p.out_stride[1] = 512, 128, 512, 128
    p.kv_stride[0], p.kv_stride[1], p.kv_stride[2] = 4096, 2048, 128
    p.workspace, p.workspace_bytes = buf.data_ptr(), buf.numel() * 2
    p.block_table = tab.data_ptr()
    for page, stride, n_pages, want in ((24, 8, 4, 1), (0, 8, 4, 1), (16, 0, 4, 1), (16, 7, 4, 1), (16, 8, 0, 1)):
        p.page_size, p.table_stride, p.n_pages = page, stride, n_pages
        assert _lib.lib.minfer_attn_decode(ctypes.byref(p), None) == want, (page, stride, n_pages)   # MINFER_ATTN_EINVAL


def test_block_table_entry_outside_the_pool_is_reported_not_followed(kerns):
    """A live table entry that points outside [0, n_pages): the kernel must not dereference it (it reads
    page 0 instead, so nothing outside the pools is touched) and must say so through the status word; the
    sequences with sound tables still get their results.  Same for the appending kernel: the row is
    dropped, every page keeps its content."""
    from minfer.kernels.torch_ext.ops import check_status
    B, H, Hkv, D, page = 3, 8, 2, 128, 16
    lens = torch.tensor([100, 40, 64], dtype=torch.int32)
    kp, vp, table, kc, vc = make_paged(B, Hkv, D, page, lens, torch.float16, seed=77)
    g = torch.Generator().manual_seed(5)
    q = torch.randn(B, H, 1, D, generator=g).half()
    want = O.decode_paged_oracle(q, kp, vp, table, lens)
    bad = table.clone()
    bad[1, 1] = kp.size(0) + 1000          # sequence 1, keys 16..31
    out = torch.full(q.shape, float("nan"), dtype=torch.float16, device="cuda")
    check_status()
    kerns.flash_attn_decode_paged(q.cuda(), kp.cuda(), vp.cuda(), bad.cuda(), lens.cuda(), out)
    with pytest.raises(RuntimeError, match="block-table entry"):
        check_status()
    check_status()                          # the report is cleared once read
    assert torch.isfinite(out).all()
    check_close(out[[0, 2]], want[[0, 2]], "sequences with sound tables")
    # append through the same bad table: nothing is written for the bad row
    kpd, vpd = kp.cuda(), vp.cuda()
    before_k, before_v = kpd.clone(), vpd.clone()
    qa = torch.randn(B, 1, H, D, generator=g).half().cuda()
    ka = torch.randn(B, 1, Hkv, D, generator=g).half().cuda()
    va = torch.randn(B, 1, Hkv, D, generator=g).half().cuda()
    start = torch.tensor([0, 20, 0], dtype=torch.int32, device="cuda")   # sequence 1 -> table slot 1 (bad)
    kerns.rope_kv_append_paged(D, 10000.0, 0, qa, ka, va, kpd, vpd, bad.cuda(), start)
    with pytest.raises(RuntimeError, match="block-table entry"):
        check_status()
    changed = (kpd != before_k).flatten(1).any(1).nonzero().flatten().tolist()
    assert sorted(changed) == sorted({int(bad[0, 0]), int(bad[2, 0])})


def test_rope_append_into_pages_then_decode(kerns):
    """Prefill rows and one decode row written through rope_kv_append_paged land where the contiguous append puts
    them (bit for bit, compared page by page), and paged decode over the result matches the oracle."""
    B, H, Hkv, D, page, L = 3, 8, 2, 128, 32, 75
    g = torch.Generator().manual_seed(4242)
    max_pages = 4
    n_pages = B * max_pages + 3
    perm = torch.randperm(n_pages, generator=g)[: B * max_pages].reshape(B, max_pages).to(torch.int32)
    kp = torch.zeros(n_pages, Hkv, page, D, dtype=torch.float16, device="cuda")
    vp = torch.zeros_like(kp)
    kc = torch.zeros(B, Hkv, max_pages * page, D, dtype=torch.float16, device="cuda")
    vc = torch.zeros_like(kc)
    start = torch.tensor([0, 0, 0], dtype=torch.int32, device="cuda")
    table = perm.cuda()
    for (Lc, st) in ((L, [0, 0, 0]), (1, [L, L, L])):
        q = torch.randn(B, Lc, H, D, generator=g).half().cuda()
        k = torch.randn(B, Lc, Hkv, D, generator=g).half().cuda()
        v = torch.randn(B, Lc, Hkv, D, generator=g).half().cuda()
        start = torch.tensor(st, dtype=torch.int32, device="cuda")
        q2 = q.clone()
        kerns.rope_kv_append(D, 10000.0, 1, q, k, v, kc, vc, start)
        kerns.rope_kv_append_paged(D, 10000.0, 1, q2, k, v, kp, vp, table, start)
        assert torch.equal(q, q2)
    torch.cuda.synchronize()
    gathered_k = kp[perm.long().cuda()].permute(0, 2, 1, 3, 4).reshape(B, Hkv, max_pages * page, D)
    gathered_v = vp[perm.long().cuda()].permute(0, 2, 1, 3, 4).reshape(B, Hkv, max_pages * page, D)
    assert torch.equal(gathered_k, kc) and torch.equal(gathered_v, vc)
    lens = torch.full((B,), L + 1, dtype=torch.int32)
    qd = torch.randn(B, H, 1, D, generator=g).half()
    want = O.decode_oracle(qd, kc.cpu(), vc.cpu(), lens)
    out = torch.full(qd.shape, float("nan"), dtype=torch.float16, device="cuda")
    kerns.flash_attn_decode_paged(qd.cuda(), kp, vp, table, lens.cuda(), out)
    torch.cuda.synchronize()
    check_close(out, want, "append + paged decode")
