"""Python op surface of the attention path.

`flash_attn` keeps the reference's wrapper signature and schema
(src/minfer/kernels/torch_ext/ops.py:234-266, csrc/reg.cpp:30 of
dsuarez01/minfer-python) and the argument checks of its launcher
(csrc/cuda/flash_attn/op.cuh:32-78), relaxed only to admit bfloat16 and
head_dim 64.  `flash_attn_causal` and `flash_attn_decode` are additions the
reference has no counterpart for.  Every op forwards raw pointers, strides
and the current CUDA stream to libminfer_attn.so; nothing here computes.

Two bindings reach the library.  When the torch extension `_C` has been built
(csrc/torch_binding: schemas and CUDA implementations registered through
LibTorch's stable ABI, the reference's own mechanism, csrc/reg.cpp:21-33 and
csrc/cuda/reg.cu:16-27) the attention ops dispatch into it and this module
only adds the fake implementations and the ops it does not cover.  Otherwise -
or with MINFER_ATTN_BINDING=ctypes - the schemas are defined here with
torch.library and every op is a Python function that fills the C-ABI structs
through ctypes.  Both paths end in the same extern "C" entry points.
"""
from __future__ import annotations

import contextlib
import ctypes
import os

import torch

from . import _lib

_DEBUG = os.environ.get("MINFER_ATTN_DEBUG", "0") not in ("", "0")
_max_ctas = 0  # upper bound on the prefill grid (0: one thread block per SM), see prefill_cta_limit()


@contextlib.contextmanager
def prefill_cta_limit(n: int):
    """Inside the block every prefill call launches at most `n` thread blocks (0 = one per SM).
    The prefill kernel is persistent and fills every SM it is given; a caller that wants a kernel
    of another stream to run beside it - the multi-GPU harness overlaps the output all-gather of
    one row block with the attention of the next - leaves a few SMs free this way."""
    global _max_ctas
    old, _max_ctas = _max_ctas, int(n)
    _push_cta_limit()
    try:
        yield
    finally:
        _max_ctas = old
        _push_cta_limit()


def _push_cta_limit() -> None:
    if _C is not None:
        torch.ops.minfer.attn_set_prefill_cta_limit.default(torch.empty(0, device="cuda"), _max_ctas)

_DEFS = {
    "flash_attn": "(int qtype_int, int qblock_size, int qtype_size, Tensor q, Tensor k, Tensor v, "
                  "Tensor(a!) mask, Tensor(a!) out) -> ()",
    "flash_attn_causal": "(Tensor q, Tensor k, Tensor v, Tensor(a!) out) -> ()",
    "flash_attn_decode": "(Tensor q, Tensor k_cache, Tensor v_cache, Tensor lens, Tensor(a!) out) -> ()",
    # the reference's schemas (csrc/reg.cpp:25-26)
    "il_rope": "(int rotary_dim, int start_pos, float freq_base, Tensor(a!) x) -> ()",
    "neox_rope": "(int rotary_dim, int start_pos, float freq_base, Tensor(a!) x) -> ()",
    "rope_kv_append": "(int rotary_dim, float freq_base, int style, Tensor(a!) q, Tensor k, Tensor v, "
                      "Tensor(a!) k_cache, Tensor(a!) v_cache, Tensor start) -> ()",
    # GGML Q8_0 KV cache: uint8 tensors [B, Hkv, Lmax, head_dim / 32 * 34]
    "flash_attn_decode_q8": "(Tensor q, Tensor k_cache, Tensor v_cache, Tensor lens, Tensor(a!) out) -> ()",
    # paged KV cache: pools [n_pages, Hkv, page_size, D] reached through block_table int32 [B, max_pages]
    "flash_attn_decode_paged": "(Tensor q, Tensor k_pages, Tensor v_pages, Tensor block_table, Tensor lens, "
                               "Tensor(a!) out) -> ()",
    "rope_kv_append_paged": "(int rotary_dim, float freq_base, int style, Tensor(a!) q, Tensor k, Tensor v, "
                            "Tensor(a!) k_pages, Tensor(a!) v_pages, Tensor block_table, Tensor start) -> ()",
    "rope_kv_append_q8": "(int rotary_dim, float freq_base, int style, Tensor(a!) q, Tensor k, Tensor v, "
                         "Tensor(a!) k_cache, Tensor(a!) v_cache, Tensor start) -> ()",
}
_binding_choice = os.environ.get("MINFER_ATTN_BINDING", "auto")
if _binding_choice not in ("auto", "ctypes", "stable"):
    raise ImportError(f"MINFER_ATTN_BINDING={_binding_choice!r}: expected auto, ctypes or stable")
_C = None
if _binding_choice != "ctypes":
    try:
        from . import _C  # noqa: F401  (loading it registers the schemas and the C++ CUDA implementations)
    except ImportError:
        if _binding_choice == "stable":
            raise
        _C = None
BINDING = "stable" if _C is not None else "ctypes"
# ops whose CUDA implementation lives in the extension
_IN_EXTENSION = tuple(_DEFS) if _C is not None else ()

if _C is None:
    _library = torch.library.Library("minfer", "FRAGMENT")
    for _name, _schema in _DEFS.items():
        _library.define(_name + _schema)
else:
    _library = None   # every op has its CUDA implementation in the extension

_status: dict[int, torch.Tensor] = {}
_workspace: dict[int, torch.Tensor] = {}        # decode split-KV partials, per device
_mask_workspace: dict[int, torch.Tensor] = {}   # prefill mask tile classes, per device


def _status_word(device: torch.device) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _status.get(idx)
    if t is None:
        if _C is not None:   # one word per device, shared with the extension's launches
            t = torch.ops.minfer.attn_status_word.default(torch.empty(0, device=torch.device("cuda", idx)))
        else:
            t = torch.zeros(4, dtype=torch.int32, device=device)
        _status[idx] = t
    return t


def check_status(device=None) -> None:
    """Synchronise and raise if a kernel on `device` left a report in the status word: a bounded wait
    that ran out (code 100), a block-table entry outside the page pool (101: sequence, table index,
    entry) or a cache position outside [0, max_len) (102: sequence, position, max_len)."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    t = _status_word(device)
    torch.cuda.synchronize(device)
    vals = t.tolist()
    if vals[0] != 0:
        t.zero_()
        what = {100: "a bounded wait ran out (code, block x, block y/z, wait site)",
                101: "block-table entry outside the page pool (code, sequence, table index, entry)",
                102: "cache position out of range (code, sequence, position, max_len)"}.get(vals[0], "unknown code")
        raise RuntimeError(f"minfer attention kernel reported status {vals}: {what}")


def _dtype_tag(t: torch.Tensor) -> int:
    if t.dtype == torch.float16:
        return _lib.F16
    if t.dtype == torch.bfloat16:
        return _lib.BF16
    raise RuntimeError(f"minfer attention: dtype {t.dtype} not supported (float16 or bfloat16)")


def _check_qkv(q, k, v, out):
    torch._check(q.is_cuda and k.is_cuda and v.is_cuda and out.is_cuda, lambda: "all tensors must be on CUDA")
    torch._check(q.device == k.device == v.device == out.device, lambda: "tensors on different devices")
    torch._check(q.dim() == 4 and k.dim() == 4 and v.dim() == 4 and out.dim() == 4, lambda: "tensors must be 4-D")
    torch._check(q.dtype == k.dtype == v.dtype == out.dtype, lambda: "q, k, v, out must share one dtype")
    torch._check(q.stride(-1) == 1 and k.stride(-1) == 1 and v.stride(-1) == 1 and out.stride(-1) == 1,
                 lambda: "innermost stride must be 1")
    torch._check(k.stride()[:3] == v.stride()[:3], lambda: "k and v must share strides")
    torch._check(q.shape == out.shape, lambda: "q and out shapes differ")
    torch._check(k.shape == v.shape, lambda: "k and v shapes differ")
    torch._check(q.size(0) == k.size(0) and q.size(3) == k.size(3), lambda: "batch or head_dim mismatch")
    torch._check(q.size(1) % k.size(1) == 0, lambda: "n_heads must be a multiple of n_kv_heads")


def _prefill(q, k, v, mask, out, causal: bool, peer_out=()) -> None:
    p = _lib.PrefillParams()
    p.n_peer_out = len(peer_out)
    for i, ptr in enumerate(peer_out):
        p.peer_out[i] = ptr
    p.q, p.k, p.v, p.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
    p.mask = mask.data_ptr() if mask is not None else None
    p.status = _status_word(q.device).data_ptr()
    for i in range(3):
        p.q_stride[i] = q.stride(i)
        p.kv_stride[i] = k.stride(i)
        p.out_stride[i] = out.stride(i)
    p.batch, p.n_heads, p.n_kv_heads = q.size(0), q.size(1), k.size(1)
    p.seq_q, p.seq_k, p.head_dim = q.size(2), k.size(2), q.size(3)
    p.dtype = _dtype_tag(q)
    p.causal = 1 if causal else 0
    p.softmax_scale = 0.0
    p.flags = 0
    p.max_ctas = _max_ctas
    # mask tile classes (dense mask) or the persistent kernel's work-item counter (causal)
    need = _lib.lib.minfer_attn_prefill_workspace_bytes(p.batch, p.seq_q, p.seq_k) if mask is not None else 16
    ws = _workspace_for(q.device, need, _mask_workspace, torch.cuda.current_stream(q.device).cuda_stream)
    p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel()
    with torch.cuda.device(q.device):
        stream = torch.cuda.current_stream().cuda_stream
        _lib.check(_lib.lib.minfer_attn_prefill(ctypes.byref(p), ctypes.c_void_p(stream)), "minfer_attn_prefill")
    if _DEBUG:
        check_status(q.device)


def _flash_attn_cuda(qtype_int, qblock_size, qtype_size, q, k, v, mask, out) -> None:
    _check_qkv(q, k, v, out)
    torch._check(mask.is_cuda and mask.device == q.device, lambda: "mask must be on the same CUDA device")
    torch._check(mask.dtype == torch.bool, lambda: "mask must be bool")
    torch._check(mask.dim() == 4 and mask.is_contiguous(), lambda: "mask must be a contiguous 4-D tensor")
    torch._check(q.size(2) == k.size(2), lambda: "flash_attn requires seq_q == seq_k")
    torch._check(tuple(mask.shape) == (q.size(0), 1, q.size(2), k.size(2)), lambda: "mask must be [B, 1, L, L]")
    _prefill(q, k, v, mask, out, causal=False)


def _flash_attn_causal_cuda(q, k, v, out) -> None:
    _check_qkv(q, k, v, out)
    torch._check(k.size(2) >= q.size(2), lambda: "causal attention requires seq_k >= seq_q")
    _prefill(q, k, v, None, out, causal=True)


def flash_attn_causal_multi_out(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor, peer_out) -> None:
    """flash_attn_causal whose kernel stores every output tile to `out` and to each address in `peer_out`: device
    pointers (ints), writable from this process, of the same [B, H, L, D] view in the memory of up to seven other
    GPUs.  The multi-GPU harness uses it to fuse the output exchange of head-parallel prefill into the attention
    kernel (minfer.dist.PeerOutputs builds the pointers).  The stores are complete when the kernel is; ordering the
    readers on the other GPUs after that is the caller's business.  Always goes through the ctypes binding."""
    _check_qkv(q, k, v, out)
    torch._check(k.size(2) >= q.size(2), lambda: "causal attention requires seq_k >= seq_q")
    torch._check(len(peer_out) <= 7, lambda: "at most 7 output replicas")
    _prefill(q, k, v, None, out, causal=True, peer_out=tuple(int(x) for x in peer_out))


def _workspace_for(device: torch.device, nbytes: int, cache: dict, stream: int = 0) -> torch.Tensor:
    """Scratch owned by this layer (the library itself never allocates), one buffer per device and
    stream so that calls on different streams never share one; grown on demand."""
    idx = (device.index if device.index is not None else torch.cuda.current_device(), stream)
    t = cache.get(idx)
    if t is None or t.numel() < nbytes:
        t = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        cache[idx] = t
    return t


def _check_q8_cache(cache: torch.Tensor, batch: int, head_dim: int, what: str) -> None:
    torch._check(cache.is_cuda and cache.dtype == torch.uint8 and cache.dim() == 4, lambda: f"{what} must be a CUDA uint8 [B, Hkv, Lmax, bytes] tensor")
    torch._check(cache.size(0) == batch and cache.size(3) == head_dim // 32 * 34, lambda: f"{what}: batch or row bytes do not match (row = head_dim/32 blocks of 34 bytes)")
    torch._check(cache.stride(3) == 1 and cache.stride(2) == cache.size(3), lambda: f"{what}: rows of one head must be contiguous")
    mult = 4 if head_dim == 64 else 2  # rows of one (batch, head) must end on a 16-byte boundary
    torch._check(cache.size(2) % mult == 0, lambda: f"{what}: the padded length must be a multiple of {mult}")


def _flash_attn_decode_q8_cuda(q, k_cache, v_cache, lens, out) -> None:
    torch._check(q.is_cuda and out.is_cuda and q.dim() == 4 and out.dim() == 4 and q.shape == out.shape, lambda: "q/out must be CUDA [B, H, 1, D] tensors")
    torch._check(q.dtype == out.dtype and q.stride(-1) == 1 and out.stride(-1) == 1, lambda: "q/out dtype or innermost stride")
    torch._check(q.size(2) == 1, lambda: "decode takes one query token per sequence")
    _check_q8_cache(k_cache, q.size(0), q.size(3), "k_cache")
    _check_q8_cache(v_cache, q.size(0), q.size(3), "v_cache")
    torch._check(k_cache.shape == v_cache.shape and k_cache.stride() == v_cache.stride(), lambda: "the caches must share shape and strides")
    torch._check(q.size(1) % k_cache.size(1) == 0, lambda: "n_heads must be a multiple of n_kv_heads")
    _decode_call(q, k_cache, v_cache, lens, out, _lib.KV_Q8_0)


def _flash_attn_decode_cuda(q, k_cache, v_cache, lens, out) -> None:
    _check_qkv(q, k_cache, v_cache, out)
    torch._check(q.size(2) == 1, lambda: "decode takes one query token per sequence")
    _decode_call(q, k_cache, v_cache, lens, out, _lib.KV_16BIT)


def _flash_attn_decode_paged_cuda(q, k_pages, v_pages, block_table, lens, out) -> None:
    torch._check(q.is_cuda and out.is_cuda and q.dim() == 4 and out.dim() == 4 and q.shape == out.shape,
                 lambda: "q/out must be CUDA [B, H, 1, D] tensors")
    torch._check(q.size(2) == 1, lambda: "decode takes one query token per sequence")
    torch._check(q.dtype in (torch.float16, torch.bfloat16) and out.dtype == q.dtype, lambda: "q/out must be float16 or bfloat16")
    torch._check(k_pages.is_cuda and v_pages.is_cuda and k_pages.dim() == 4 and v_pages.dim() == 4,
                 lambda: "the page pools must be CUDA [n_pages, n_kv_heads, page_size, D] tensors")
    torch._check(k_pages.dtype == q.dtype and v_pages.dtype == q.dtype, lambda: "the page pools must have q's dtype")
    torch._check(k_pages.shape == v_pages.shape and k_pages.stride() == v_pages.stride(),
                 lambda: "the page pools must share shape and strides")
    torch._check(k_pages.size(3) == q.size(3) and k_pages.stride(-1) == 1 and q.stride(-1) == 1 and out.stride(-1) == 1,
                 lambda: "head_dim mismatch or innermost stride not 1")
    torch._check(k_pages.size(2) % 16 == 0, lambda: "page_size must be a multiple of 16")
    torch._check(q.size(1) % k_pages.size(1) == 0, lambda: "n_heads must be a multiple of n_kv_heads")
    torch._check(block_table.is_cuda and block_table.dtype == torch.int32 and block_table.dim() == 2 and
                 block_table.is_contiguous() and block_table.size(0) == q.size(0),
                 lambda: "block_table must be a contiguous CUDA int32 [B, max_pages] tensor")
    _decode_call(q, k_pages, v_pages, lens, out, _lib.KV_16BIT, block_table)


def _decode_call(q, k_cache, v_cache, lens, out, kv_format, block_table=None) -> None:
    torch._check(lens.is_cuda and lens.device == q.device, lambda: "lens must be on the same CUDA device")
    torch._check(lens.dtype == torch.int32 and lens.dim() == 1 and lens.is_contiguous(),
                 lambda: "lens must be a contiguous int32 vector")
    torch._check(lens.numel() == q.size(0), lambda: "lens must have one entry per sequence")
    p = _lib.DecodeParams()
    p.q, p.k_cache, p.v_cache = q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr()
    p.lens, p.out = lens.data_ptr(), out.data_ptr()
    p.batch, p.n_heads, p.n_kv_heads = q.size(0), q.size(1), k_cache.size(1)
    p.max_len, p.head_dim = k_cache.size(2), q.size(3)
    if block_table is not None:
        p.block_table = block_table.data_ptr()
        p.page_size, p.table_stride = k_cache.size(2), block_table.size(1)
        p.max_len = p.page_size * p.table_stride
        p.n_pages = k_cache.size(0)
    p.status = _status_word(q.device).data_ptr()
    p.dtype = _dtype_tag(q)
    p.chunk = 0
    p.softmax_scale = 0.0
    p.kv_format = kv_format
    for i in range(2):
        p.q_stride[i] = q.stride(i)
        p.out_stride[i] = out.stride(i)
    for i in range(3):
        p.kv_stride[i] = k_cache.stride(i)
    need = _lib.lib.minfer_attn_decode_workspace_bytes(p.batch, p.n_heads, p.max_len, p.head_dim, 0)
    ws = _workspace_for(q.device, need, _workspace, torch.cuda.current_stream(q.device).cuda_stream)
    p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel()
    with torch.cuda.device(q.device):
        stream = torch.cuda.current_stream().cuda_stream
        _lib.check(_lib.lib.minfer_attn_decode(ctypes.byref(p), ctypes.c_void_p(stream)), "minfer_attn_decode")


def _rope_call(p: "_lib.RopeParams", device) -> None:
    with torch.cuda.device(device):
        stream = torch.cuda.current_stream().cuda_stream
        _lib.check(_lib.lib.minfer_attn_rope_append(ctypes.byref(p), ctypes.c_void_p(stream)), "minfer_attn_rope_append")


def _rope_inplace_cuda(style: int, rotary_dim, start_pos, freq_base, x) -> None:
    # the checks of the reference's launcher (csrc/cuda/il_rope/op.cuh:27-31), bfloat16 admitted
    torch._check(x.is_cuda, lambda: "x must be on CUDA")
    torch._check(x.is_contiguous(), lambda: "x must be contiguous")
    torch._check(x.dim() == 4, lambda: "x must be [B, L, n_heads, head_dim]")
    torch._check(rotary_dim <= x.size(3), lambda: "rotary_dim exceeds head_dim")
    p = _lib.RopeParams()
    p.q = x.data_ptr()
    for i in range(3):
        p.q_stride[i] = x.stride(i)
    p.batch, p.seq, p.n_heads, p.head_dim = x.size(0), x.size(1), x.size(2), x.size(3)
    p.rotary_dim, p.start_pos, p.freq_base = rotary_dim, start_pos, freq_base
    p.dtype, p.style = _dtype_tag(x), style
    _rope_call(p, x.device)


def _il_rope_cuda(rotary_dim, start_pos, freq_base, x) -> None:
    _rope_inplace_cuda(0, rotary_dim, start_pos, freq_base, x)


def _neox_rope_cuda(rotary_dim, start_pos, freq_base, x) -> None:
    _rope_inplace_cuda(1, rotary_dim, start_pos, freq_base, x)


def _rope_kv_append_q8_cuda(rotary_dim, freq_base, style, q, k, v, k_cache, v_cache, start) -> None:
    _rope_kv_append_cuda(rotary_dim, freq_base, style, q, k, v, k_cache, v_cache, start, q8=True)


def _rope_kv_append_paged_cuda(rotary_dim, freq_base, style, q, k, v, k_pages, v_pages, block_table, start) -> None:
    torch._check(block_table.is_cuda and block_table.dtype == torch.int32 and block_table.dim() == 2 and
                 block_table.is_contiguous() and block_table.size(0) == q.size(0),
                 lambda: "block_table must be a contiguous CUDA int32 [B, max_pages] tensor")
    _rope_kv_append_cuda(rotary_dim, freq_base, style, q, k, v, k_pages, v_pages, start, block_table=block_table)


def _rope_kv_append_cuda(rotary_dim, freq_base, style, q, k, v, k_cache, v_cache, start, q8=False, block_table=None) -> None:
    torch._check(q.is_cuda and k.is_cuda and v.is_cuda and k_cache.is_cuda and v_cache.is_cuda and start.is_cuda,
                 lambda: "all tensors must be on CUDA")
    torch._check(q.dim() == 4 and k.dim() == 4 and v.dim() == 4 and k_cache.dim() == 4 and v_cache.dim() == 4,
                 lambda: "q/k/v must be [B, L, H, D] and the caches [B, Hkv, Lmax, D]")
    if q8:
        torch._check(q.dtype == k.dtype == v.dtype, lambda: "dtypes differ")
        _check_q8_cache(k_cache, q.size(0), q.size(3), "k_cache")
        _check_q8_cache(v_cache, q.size(0), q.size(3), "v_cache")
    else:
        torch._check(q.dtype == k.dtype == v.dtype == k_cache.dtype == v_cache.dtype, lambda: "dtypes differ")
    torch._check(k.shape == v.shape and k.stride() == v.stride(), lambda: "k and v must share shape and strides")
    torch._check(k_cache.shape == v_cache.shape and k_cache.stride() == v_cache.stride(),
                 lambda: "the caches must share shape and strides")
    torch._check(q.size(0) == k.size(0) and (block_table is not None or k.size(0) == k_cache.size(0)) and
                 q.size(1) == k.size(1), lambda: "batch / seq mismatch")
    torch._check(k.size(2) == k_cache.size(1) and q.size(3) == k.size(3), lambda: "head count / head_dim mismatch")
    torch._check(q8 or k.size(3) == k_cache.size(3), lambda: "head_dim mismatch")
    torch._check(q.stride(-1) == 1 and k.stride(-1) == 1 and k_cache.stride(-1) == 1, lambda: "innermost stride must be 1")
    torch._check(start.dtype == torch.int32 and start.dim() == 1 and start.numel() == q.size(0) and start.is_contiguous(),
                 lambda: "start must be a contiguous int32 vector with one entry per sequence")
    p = _lib.RopeParams()
    p.q, p.k, p.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
    p.k_cache, p.v_cache, p.start = k_cache.data_ptr(), v_cache.data_ptr(), start.data_ptr()
    for i in range(3):
        p.q_stride[i], p.kv_stride[i], p.cache_stride[i] = q.stride(i), k.stride(i), k_cache.stride(i)
    p.batch, p.seq, p.n_heads, p.n_kv_heads, p.head_dim = q.size(0), q.size(1), q.size(2), k.size(2), q.size(3)
    p.rotary_dim, p.start_pos, p.max_len, p.freq_base = rotary_dim, 0, k_cache.size(2), freq_base
    if block_table is not None:
        p.block_table = block_table.data_ptr()
        p.page_size, p.table_stride = k_cache.size(2), block_table.size(1)
        p.max_len = p.page_size * p.table_stride
        p.n_pages = k_cache.size(0)
    p.status = _status_word(q.device).data_ptr()
    p.dtype, p.style = _dtype_tag(q), style
    p.cache_format = _lib.KV_Q8_0 if q8 else _lib.KV_16BIT
    _rope_call(p, q.device)


for _name, _fn in (("il_rope", _il_rope_cuda), ("neox_rope", _neox_rope_cuda), ("rope_kv_append", _rope_kv_append_cuda),
                   ("rope_kv_append_q8", _rope_kv_append_q8_cuda), ("rope_kv_append_paged", _rope_kv_append_paged_cuda),
                   ("flash_attn_decode_q8", _flash_attn_decode_q8_cuda), ("flash_attn", _flash_attn_cuda),
                   ("flash_attn_causal", _flash_attn_causal_cuda), ("flash_attn_decode", _flash_attn_decode_cuda),
                   ("flash_attn_decode_paged", _flash_attn_decode_paged_cuda)):
    if _name not in _IN_EXTENSION:
        _library.impl(_name, _fn, "CUDA")


def flash_attn(
    qtype_int: int,
    qblock_size: int,
    qtype_size: int,
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    mask: torch.Tensor,
    out: torch.Tensor,
):
    """
    attention with a dense bool mask [B, 1, L, L] (True = attend); result written to `out`.
    q/out: [B, n_heads, L, D], k/v: [B, n_kv_heads, L, D]; the three leading ints are unused
    by attention, as in the reference.
    """
    return torch.ops.minfer.flash_attn.default(qtype_int, qblock_size, qtype_size, q, k, v, mask, out)


def flash_attn_causal(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor):
    """causal attention (key j visible to query i iff j <= i + Lk - Lq) without a materialised mask."""
    return torch.ops.minfer.flash_attn_causal.default(q, k, v, out)


def flash_attn_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, lens: torch.Tensor,
                      out: torch.Tensor):
    """
    one-token decode over a padded KV cache: q/out [B, n_heads, 1, D], caches
    [B, n_kv_heads, max_len, D], lens int32 [B]; sequence b attends keys [0, lens[b]).
    """
    return torch.ops.minfer.flash_attn_decode.default(q, k_cache, v_cache, lens, out)


def flash_attn_decode_paged(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_table: torch.Tensor,
                            lens: torch.Tensor, out: torch.Tensor):
    """
    flash_attn_decode over a paged KV cache: pools [n_pages, n_kv_heads, page_size, D] (page_size a multiple
    of 16), block_table int32 [B, max_pages]; key j of sequence b is row j % page_size of page
    block_table[b, j // page_size].  Only the entries below ceil(lens[b] / page_size) are read.
    """
    return torch.ops.minfer.flash_attn_decode_paged.default(q, k_pages, v_pages, block_table, lens, out)


def il_rope(rotary_dim: int, start_pos: int, freq_base: float, x: torch.Tensor):
    """
    Applies il_rope in-place (per-head): interleaved pairs of x [B, L, n_heads, head_dim]
    """
    return torch.ops.minfer.il_rope.default(rotary_dim, start_pos, freq_base, x)


def neox_rope(rotary_dim: int, start_pos: int, freq_base: float, x: torch.Tensor):
    """
    Applies neox_rope in-place (per-head): halves of x [B, L, n_heads, head_dim]
    """
    return torch.ops.minfer.neox_rope.default(rotary_dim, start_pos, freq_base, x)


def rope_kv_append(rotary_dim: int, freq_base: float, style: int, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                   k_cache: torch.Tensor, v_cache: torch.Tensor, start: torch.Tensor):
    """
    one pass before attention: rotate q [B, L, Hq, D] in place, write rotated k and plain v
    [B, L, Hkv, D] into the caches [B, Hkv, Lmax, D] at rows start[b] + l (start: int32 [B]).
    style 0 = interleaved (il_rope), 1 = neox.
    """
    return torch.ops.minfer.rope_kv_append.default(rotary_dim, freq_base, style, q, k, v, k_cache, v_cache, start)


def flash_attn_decode_q8(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, lens: torch.Tensor,
                         out: torch.Tensor):
    """
    flash_attn_decode over a GGML Q8_0 KV cache: caches are uint8 [B, n_kv_heads, max_len, D/32*34]
    (32 int8 + one fp16 scale per block); equals flash_attn_decode on the dequantised cache.
    """
    return torch.ops.minfer.flash_attn_decode_q8.default(q, k_cache, v_cache, lens, out)


def rope_kv_append_paged(rotary_dim: int, freq_base: float, style: int, q: torch.Tensor, k: torch.Tensor,
                         v: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_table: torch.Tensor,
                         start: torch.Tensor):
    """rope_kv_append into a paged cache: pools [n_pages, Hkv, page_size, D], block_table int32 [B, max_pages];
    position p of sequence b goes to row p % page_size of page block_table[b, p // page_size]."""
    return torch.ops.minfer.rope_kv_append_paged.default(rotary_dim, freq_base, style, q, k, v, k_pages, v_pages,
                                                         block_table, start)


def rope_kv_append_q8(rotary_dim: int, freq_base: float, style: int, q: torch.Tensor, k: torch.Tensor,
                      v: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, start: torch.Tensor):
    """rope_kv_append into GGML Q8_0 caches: the rows the 16-bit cache would get, quantised block by block."""
    return torch.ops.minfer.rope_kv_append_q8.default(rotary_dim, freq_base, style, q, k, v, k_cache, v_cache, start)


@torch.library.register_fake("minfer::flash_attn_decode_q8")
def _(q, k_cache, v_cache, lens, out):
    torch._check(q.dtype in (torch.float16, torch.bfloat16) and out.dtype == q.dtype)
    torch._check(k_cache.dtype == torch.uint8 and v_cache.dtype == torch.uint8)
    torch._check(lens.dtype == torch.int32)
    torch._check(q.device.type == "cuda")


@torch.library.register_fake("minfer::rope_kv_append_paged")
def _(rotary_dim, freq_base, style, q, k, v, k_pages, v_pages, block_table, start):
    torch._check(q.dtype in (torch.float16, torch.bfloat16))
    torch._check(k.dtype == q.dtype and v.dtype == q.dtype and k_pages.dtype == q.dtype and v_pages.dtype == q.dtype)
    torch._check(start.dtype == torch.int32 and block_table.dtype == torch.int32)
    torch._check(q.device.type == "cuda")
    torch._check(q.dim() == 4 and k.dim() == 4 and v.dim() == 4 and k_pages.dim() == 4 and v_pages.dim() == 4)


@torch.library.register_fake("minfer::rope_kv_append_q8")
def _(rotary_dim, freq_base, style, q, k, v, k_cache, v_cache, start):
    torch._check(q.dtype in (torch.float16, torch.bfloat16))
    torch._check(k_cache.dtype == torch.uint8 and v_cache.dtype == torch.uint8)
    torch._check(start.dtype == torch.int32)
    torch._check(q.device.type == "cuda")


@torch.library.register_fake("minfer::il_rope")
def _(rotary_dim, start_pos, freq_base, x):
    torch._check(x.dtype in (torch.float16, torch.bfloat16))
    torch._check(x.dim() == 4)
    torch._check(x.device.type == "cuda")
    torch._check(rotary_dim <= x.size(3))


@torch.library.register_fake("minfer::neox_rope")
def _(rotary_dim, start_pos, freq_base, x):
    torch._check(x.dtype in (torch.float16, torch.bfloat16))
    torch._check(x.dim() == 4)
    torch._check(x.device.type == "cuda")
    torch._check(rotary_dim <= x.size(3))


@torch.library.register_fake("minfer::rope_kv_append")
def _(rotary_dim, freq_base, style, q, k, v, k_cache, v_cache, start):
    torch._check(q.dtype in (torch.float16, torch.bfloat16))
    torch._check(q.dim() == 4 and k.dim() == 4 and v.dim() == 4 and k_cache.dim() == 4 and v_cache.dim() == 4)
    torch._check(start.dtype == torch.int32)
    torch._check(q.device.type == "cuda")


@torch.library.register_fake("minfer::flash_attn")
def _(qtype_int, qblock_size, qtype_size, q, k, v, mask, out):
    torch._check(q.dtype in (torch.float16, torch.bfloat16))
    torch._check(k.dtype == q.dtype)
    torch._check(v.dtype == q.dtype)
    torch._check(mask.dtype == torch.bool)
    torch._check(out.dtype == q.dtype)
    torch._check(q.device == k.device == v.device == out.device)
    torch._check(q.device.type == "cuda")
    torch._check(q.dim() == 4)
    torch._check(k.dim() == 4)
    torch._check(v.dim() == 4)
    torch._check(mask.dim() == 4)
    torch._check(out.dim() == 4)


@torch.library.register_fake("minfer::flash_attn_causal")
def _(q, k, v, out):
    torch._check(q.dtype in (torch.float16, torch.bfloat16))
    torch._check(k.dtype == q.dtype and v.dtype == q.dtype and out.dtype == q.dtype)
    torch._check(q.device.type == "cuda")
    torch._check(q.dim() == 4 and k.dim() == 4 and v.dim() == 4 and out.dim() == 4)


@torch.library.register_fake("minfer::flash_attn_decode_paged")
def _(q, k_pages, v_pages, block_table, lens, out):
    torch._check(q.dtype in (torch.float16, torch.bfloat16))
    torch._check(k_pages.dtype == q.dtype and v_pages.dtype == q.dtype and out.dtype == q.dtype)
    torch._check(lens.dtype == torch.int32 and block_table.dtype == torch.int32)
    torch._check(q.device.type == "cuda")
    torch._check(q.dim() == 4 and k_pages.dim() == 4 and v_pages.dim() == 4 and out.dim() == 4)
    torch._check(lens.dim() == 1 and block_table.dim() == 2)


@torch.library.register_fake("minfer::flash_attn_decode")
def _(q, k_cache, v_cache, lens, out):
    torch._check(q.dtype in (torch.float16, torch.bfloat16))
    torch._check(k_cache.dtype == q.dtype and v_cache.dtype == q.dtype and out.dtype == q.dtype)
    torch._check(lens.dtype == torch.int32)
    torch._check(q.device.type == "cuda")
    torch._check(q.dim() == 4 and k_cache.dim() == 4 and v_cache.dim() == 4 and out.dim() == 4)
    torch._check(lens.dim() == 1)


@torch.library.register_fake("minfer::attn_status_word") if _C is not None else (lambda f: f)
def _(like):
    return torch.empty(4, dtype=torch.int32, device=like.device)


@torch.library.register_fake("minfer::attn_set_prefill_cta_limit") if _C is not None else (lambda f: f)
def _(like, max_ctas):
    return None
