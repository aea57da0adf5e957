"""minfer_attn_decode_static: decode for callers that cannot allocate device memory.

A serving process that reserved all device memory for its own pool, or a decode loop that
must never reach the allocator, cannot hand minfer_attn_decode() a workspace.  The static
entry point keeps the split-KV partials in an array inside the library instead.  These tests
call it through the C ABI and compare it with minfer_attn_decode() on the same inputs.

Collected last on purpose: a run that stops at the first failure has then already run
every other test."""
import ctypes

import pytest
import torch

from _util import check_close
from oracle import oracle as O


def _params(_lib, q, kc, vc, lens, out, chunk=0):
    p = _lib.DecodeParams()
    p.q, p.k_cache, p.v_cache, p.lens, p.out = q.data_ptr(), kc.data_ptr(), vc.data_ptr(), lens.data_ptr(), out.data_ptr()
    p.batch, p.n_heads, p.n_kv_heads = q.size(0), q.size(1), kc.size(1)
    p.max_len, p.head_dim = kc.size(2), q.size(3)
    p.dtype, p.chunk, p.softmax_scale = _lib.F16, chunk, 0.0
    for i in range(2):
        p.q_stride[i], p.out_stride[i] = q.stride(i), out.stride(i)
    for i in range(3):
        p.kv_stride[i] = kc.stride(i)
    return p


def test_oversize_shape_is_refused_before_any_launch():
    """Partials beyond the built-in 32 MiB are refused with a clear error; no device is needed for that."""
    from minfer.kernels.torch_ext import _lib
    p = _lib.DecodeParams()
    p.batch, p.n_heads, p.n_kv_heads, p.max_len, p.head_dim, p.chunk = 64, 128, 8, 65536, 128, 64
    need = _lib.lib.minfer_attn_decode_workspace_bytes(64, 128, 65536, 128, 64)
    assert need > (32 << 20)
    rc = _lib.lib.minfer_attn_decode_static(ctypes.byref(p), None)
    assert rc == 6
    assert "static" in _lib.strerror(rc)
    assert _lib.lib.minfer_attn_decode_static(None, None) == 1


@pytest.mark.gpu
def test_static_scratch_decode_matches_workspace_decode_twice_in_a_row():
    from minfer.kernels.torch_ext import _lib
    L = _lib.lib
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    B, H, Hkv, Lmax, D = 6, 32, 8, 3000, 128
    for call, lens_list in enumerate(([3000, 1, 512, 513, 2048, 77], [64, 2999, 1500, 16, 1025, 300])):
        g = torch.Generator().manual_seed(500 + call)
        q = torch.randn(B, H, 1, D, generator=g).half()
        kc = torch.randn(B, Hkv, Lmax, D, generator=g).half()
        vc = torch.randn(B, Hkv, Lmax, D, generator=g).half()
        lens = torch.tensor(lens_list, dtype=torch.int32)
        qd, kd, vd, ld = q.cuda(), kc.cuda(), vc.cuda(), lens.cuda()

        out_ws = torch.full((B, H, 1, D), float("nan"), dtype=torch.float16, device="cuda")
        need = L.minfer_attn_decode_workspace_bytes(B, H, Lmax, D, 0)
        ws = torch.empty(need, dtype=torch.uint8, device="cuda")
        p = _params(_lib, qd, kd, vd, ld, out_ws)
        p.workspace, p.workspace_bytes = ws.data_ptr(), need
        assert L.minfer_attn_decode(ctypes.byref(p), stream) == 0

        out_st = torch.full((B, H, 1, D), float("nan"), dtype=torch.float16, device="cuda")
        p2 = _params(_lib, qd, kd, vd, ld, out_st)  # no workspace at all
        rc = L.minfer_attn_decode_static(ctypes.byref(p2), stream)
        assert rc == 0, _lib.strerror(rc)
        torch.cuda.synchronize()

        check_close(out_st, out_ws, f"static vs workspace, call {call}")
        assert torch.equal(out_st, out_ws), "same kernels, same inputs: results must be identical"
        check_close(out_st, O.decode_oracle(q, kc, vc, lens), f"static vs oracle, call {call}")
