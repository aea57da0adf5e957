"""CPU oracle for the attention path — TEST INFRASTRUCTURE ONLY.

Only tests/, the smoke check and the benchmark's CPU-baseline leg import this
module; the product library never does.

Two restatements of the reference's semantics live here:

* `sdpa_reference(Q, K, V, mask)` — the reference's own CPU path restated: its
  refs.flash_attn is one call to torch's scaled_dot_product_attention with
  attn_mask (src/minfer/kernels/refs.py:53-55 of dsuarez01/minfer-python), and
  its callers expand K/V for grouped-query heads with repeat_interleave
  (test/kernels.py:253-255, apps/benchmark.py:240-242).  The arithmetic is
  PyTorch ATen's (torch 2.10.0 pinned by the reference, uv.lock:601-602).
* `attention_f64(...)` — the definition out = softmax(q k^T * scale + mask) v
  written out in C with double accumulation (attn_oracle.c), independent of
  torch; used to cross-check the first and to check row blocks of problems too
  large for a dense SDPA call.

Pinned: tests/golden/ holds outputs of the reference's refs.flash_attn itself
(imported from the reference tree by tests/golden/make_golden.py); the CPU test
suite checks both restatements against those vectors.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np
import torch
import torch.nn.functional as F

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_HERE, "_build", "libattn_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile attn_oracle.c (gcc) if the shared object is missing or stale."""
    src = os.path.join(_HERE, "attn_oracle.c")
    if force or not os.path.exists(_LIB) or os.path.getmtime(_LIB) < os.path.getmtime(src):
        os.makedirs(os.path.dirname(_LIB), exist_ok=True)
        cc = "/usr/bin/gcc" if os.path.exists("/usr/bin/gcc") else "gcc"
        base = [cc, "-O2", "-fPIC", "-shared", "-o", _LIB, src, "-lm"]
        if subprocess.run(base[:3] + ["-fopenmp"] + base[3:], capture_output=True).returncode != 0:
            subprocess.run(base, check=True)
    return _LIB


def _load():
    global _lib
    if _lib is None:
        build()
        lib = ctypes.CDLL(_LIB)
        lib.attn_oracle_f32.restype = ctypes.c_int
        lib.attn_oracle_f32.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int] * 6 + [ctypes.c_float] + [ctypes.c_int] * 3
        _lib = lib
    return _lib


def attention_f64(q, k, v, mask=None, lens=None, causal=False, scale=0.0, rows=None) -> torch.Tensor:
    """softmax(q k^T * scale + mask) v with double accumulation, on CPU.

    q [B,H,Lq,D], k/v [B,Hkv,Lk,D] (any float dtype; upcast to fp32 exactly),
    mask bool [B,1,Lq,Lk] or None, lens int [B] or None, causal j <= i + Lk - Lq.
    rows=(r0, r1) restricts the computed query rows; the returned fp32 tensor has
    only those rows.
    """
    lib = _load()
    q32 = q.detach().to("cpu", torch.float32).contiguous()
    k32 = k.detach().to("cpu", torch.float32).contiguous()
    v32 = v.detach().to("cpu", torch.float32).contiguous()
    B, H, Lq, D = q32.shape
    Hkv, Lk = k32.shape[1], k32.shape[2]
    r0, r1 = (0, Lq) if rows is None else rows
    out = torch.zeros_like(q32)
    m8 = None
    if mask is not None:
        m8 = mask.detach().to("cpu").expand(B, 1, Lq, Lk).to(torch.uint8).contiguous()
    l32 = None
    if lens is not None:
        l32 = lens.detach().to("cpu", torch.int32).contiguous()
    rc = lib.attn_oracle_f32(
        q32.data_ptr(), k32.data_ptr(), v32.data_ptr(),
        m8.data_ptr() if m8 is not None else None,
        l32.data_ptr() if l32 is not None else None,
        out.data_ptr(), B, H, Hkv, Lq, Lk, D, float(scale), int(bool(causal)), int(r0), int(r1))
    if rc != 0:
        raise RuntimeError(f"attn_oracle_f32 failed with {rc}")
    return out[:, :, r0:r1, :]


def expand_kv(x: torch.Tensor, n_heads: int) -> torch.Tensor:
    """Grouped-query expansion exactly as the reference's callers do it."""
    n_rep = n_heads // x.shape[1]
    return x if n_rep == 1 else x.repeat_interleave(n_rep, dim=1)


def sdpa_reference(Q, K, V, mask) -> torch.Tensor:
    """The reference's refs.flash_attn restated; K/V must already be expanded."""
    return F.scaled_dot_product_attention(Q, K, V, attn_mask=mask)


def causal_mask(B: int, L: int) -> torch.Tensor:
    """The reference's causal mask construction (test/kernels.py:242)."""
    return (torch.arange(L).unsqueeze(0) <= torch.arange(L).unsqueeze(1)).unsqueeze(0).unsqueeze(0).expand(B, 1, L, L).to(torch.bool)


def window_mask(B: int, L: int, window: int) -> torch.Tensor:
    """The reference's symmetric sliding-window mask (test/kernels.py:276-278)."""
    dist = torch.arange(L).unsqueeze(0) - torch.arange(L).unsqueeze(1)
    return (dist.abs() < window).unsqueeze(0).unsqueeze(0).expand(B, 1, L, L).to(torch.bool)


def length_mask(lens: torch.Tensor, max_len: int) -> torch.Tensor:
    """Decode mask: sequence b sees keys [0, lens[b]).  Shape [B,1,1,max_len]."""
    return (torch.arange(max_len)[None, :] < lens.to(torch.int64)[:, None])[:, None, None, :]


def prefill_oracle(q, k, v, mask=None, causal=False) -> torch.Tensor:
    """fp32 oracle for prefill: inputs upcast to fp32, reference SDPA path."""
    B, H, L, _ = q.shape
    qf, kf, vf = q.float().cpu(), k.float().cpu(), v.float().cpu()
    if causal and mask is None:
        mask = causal_mask(B, L) if k.shape[2] == L else None
        if mask is None:
            return attention_f64(qf, kf, vf, causal=True)
    return sdpa_reference(qf, expand_kv(kf, H), expand_kv(vf, H), mask.cpu() if mask is not None else None)


def decode_oracle(q, k_cache, v_cache, lens) -> torch.Tensor:
    """fp32 oracle for decode: reference SDPA path with the length mask."""
    H = q.shape[1]
    qf, kf, vf = q.float().cpu(), k_cache.float().cpu(), v_cache.float().cpu()
    m = length_mask(lens.cpu(), k_cache.shape[2])
    return F.scaled_dot_product_attention(qf, kf, vf, attn_mask=m, enable_gqa=(kf.shape[1] != H))


def gather_pages(pages: torch.Tensor, block_table: torch.Tensor, lens) -> torch.Tensor:
    """Contiguous cache [B, Hkv, max_pages * page, D] of a paged one: pool [n_pages, Hkv, page, D], block_table
    [B, max_pages].  Only the table entries a sequence needs (below ceil(lens[b] / page)) are followed; the
    rows of the other pages are zeros.  The reference's cache (src/minfer/core.py:105-127) has no pages: this
    is the definition the paged kernels are held to."""
    pages = pages.cpu()
    n_pages, Hkv, page, D = pages.shape
    B, max_pages = block_table.shape
    out = torch.zeros(B, Hkv, max_pages * page, D, dtype=pages.dtype)
    for b in range(B):
        for j in range((int(lens[b]) + page - 1) // page):
            out[b, :, j * page:(j + 1) * page] = pages[int(block_table[b, j])]
    return out


def decode_paged_oracle(q, k_pages, v_pages, block_table, lens) -> torch.Tensor:
    """decode_oracle over the gathered cache."""
    return decode_oracle(q, gather_pages(k_pages, block_table, lens), gather_pages(v_pages, block_table, lens), lens)


def il_rope_reference(x: torch.Tensor, rotary_dim: int, start_pos: int, base_freq: float) -> torch.Tensor:
    """Interleaved RoPE restated from the reference (src/minfer/kernels/refs.py:12-28): fp32 angles
    (pos + start_pos) * base^(-2i/rot), complex rotation of pairs (2i, 2i+1); x is [B, L, H, D]."""
    rot = rotary_dim
    f = torch.arange(rot // 2, dtype=torch.float32)
    f = base_freq ** (-2.0 * f / rot)
    ang = (torch.arange(x.shape[1], dtype=torch.float32) + start_pos)[:, None] * f[None, :]
    c, s_ = torch.cos(ang)[None, :, None, :], torch.sin(ang)[None, :, None, :]
    xf = x.float().clone()
    a, b = xf[..., 0:rot:2].clone(), xf[..., 1:rot:2].clone()
    xf[..., 0:rot:2] = a * c - b * s_
    xf[..., 1:rot:2] = a * s_ + b * c
    return xf.to(x.dtype)


def neox_rope_reference(x: torch.Tensor, rotary_dim: int, start_pos: int, base_freq: float) -> torch.Tensor:
    """Two-halves RoPE restated from the reference (src/minfer/kernels/refs.py:30-47): pairs
    (i, i + rot/2)."""
    rot = rotary_dim
    f = torch.arange(rot // 2, dtype=torch.float32)
    f = base_freq ** (-2.0 * f / rot)
    ang = (torch.arange(x.shape[1], dtype=torch.float32) + start_pos)[:, None] * f[None, :]
    c, s_ = torch.cos(ang)[None, :, None, :], torch.sin(ang)[None, :, None, :]
    xf = x.float().clone()
    a, b = xf[..., : rot // 2].clone(), xf[..., rot // 2:rot].clone()
    xf[..., : rot // 2] = a * c - b * s_
    xf[..., rot // 2:rot] = a * s_ + b * c
    return xf.to(x.dtype)


# ---------------------------------------------------------------------------------------------
# GGML Q8_0 blocks (32 int8 + one fp16 scale = 34 bytes), restated from the reference's codec:
#   block layout   src/minfer/kernels/torch_ext/csrc/common/types.hpp:141-146
#   quant_row_q8_0 src/minfer/kernels/torch_ext/csrc/quants/impl.cpp:1169-1193
#   dequant_row_q8_0 src/minfer/kernels/torch_ext/csrc/quants/impl.cpp:1153-1166
# The reference's codec compiles from its own source (see Makefile, target _ref); when that build
# exists, q8_0_*_ref call it and the tests check the restatement against it byte for byte.
# ---------------------------------------------------------------------------------------------
def q8_0_quantize(x: torch.Tensor) -> torch.Tensor:
    """x [..., k] (k % 32 == 0, any float dtype, upcast exactly to fp32) -> uint8 [..., k/32*34]."""
    xf = x.detach().to("cpu", torch.float32).contiguous().numpy()
    lead, k = xf.shape[:-1], xf.shape[-1]
    assert k % 32 == 0
    blocks = xf.reshape(-1, k // 32, 32)
    amax = np.abs(blocks).max(axis=-1)
    d = (amax / np.float32(127.0)).astype(np.float32)
    with np.errstate(divide="ignore"):
        inv = np.where(d != 0, np.float32(1.0) / d, np.float32(0.0)).astype(np.float32)
    scaled = (blocks * inv[..., None]).astype(np.float32)
    # C roundf: half away from zero
    q = np.where(scaled >= 0, np.floor(scaled + np.float32(0.5)), np.ceil(scaled - np.float32(0.5))).astype(np.int8)
    out = np.empty(blocks.shape[:2] + (34,), dtype=np.uint8)
    out[..., :2] = d.astype(np.float16).view(np.uint8).reshape(d.shape + (2,))
    out[..., 2:] = q.view(np.uint8)
    return torch.from_numpy(out.reshape(lead + (k // 32 * 34,)))


def q8_0_dequantize(qb: torch.Tensor, dtype=torch.float16) -> torch.Tensor:
    """uint8 [..., nb*34] -> [..., nb*32] in `dtype`: each value is (dtype)(q * d) with d the block's fp16 scale."""
    raw = qb.detach().to("cpu").contiguous().numpy()
    lead = raw.shape[:-1]
    blocks = raw.reshape(-1, raw.shape[-1] // 34, 34)
    d = blocks[..., :2].copy().view(np.float16).astype(np.float32)[..., 0]
    q = blocks[..., 2:].copy().view(np.int8).astype(np.float32)
    with np.errstate(invalid="ignore", over="ignore"):  # garbage scales (inf/nan) in never-used rows are allowed
        vals = torch.from_numpy((q * d[..., None]).astype(np.float32)).to(dtype)
    return vals.reshape(lead + (blocks.shape[1] * 32,))


_REF_LIB = os.path.join(_HERE, "_ref", "libminfer_ref_quants.so")
_ref = None


def reference_build_available() -> bool:
    return os.path.exists(_REF_LIB)


def _load_ref():
    global _ref
    if _ref is None:
        lib = ctypes.CDLL(_REF_LIB)
        lib.ref_quant_row_q8_0.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64]
        lib.ref_dequant_row_q8_0_f32.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64]
        lib.ref_dequant_row_q8_0_f16.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64]
        _ref = lib
    return _ref


def q8_0_quantize_ref(x: torch.Tensor) -> torch.Tensor:
    """The reference's own quant_row_q8_0 (compiled from its source into oracle/_ref)."""
    lib = _load_ref()
    xf = x.detach().to("cpu", torch.float32).contiguous()
    k = xf.shape[-1]
    out = torch.empty(xf.shape[:-1] + (k // 32 * 34,), dtype=torch.uint8)
    lib.ref_quant_row_q8_0(xf.data_ptr(), out.data_ptr(), xf.numel())
    return out


def q8_0_dequantize_ref(qb: torch.Tensor, dtype=torch.float16) -> torch.Tensor:
    """The reference's own dequant_row_q8_0<float> / <half>."""
    lib = _load_ref()
    raw = qb.detach().to("cpu").contiguous()
    n = raw.numel() // 34 * 32
    out = torch.empty(raw.shape[:-1] + (raw.shape[-1] // 34 * 32,), dtype=dtype)
    if dtype == torch.float16:
        lib.ref_dequant_row_q8_0_f16(raw.data_ptr(), out.data_ptr(), n)
    else:
        assert dtype == torch.float32
        lib.ref_dequant_row_q8_0_f32(raw.data_ptr(), out.data_ptr(), n)
    return out


def find_reference_root(reference_root=None):
    """Where the reference's source tree is mounted, or None: the argument, else $MINFER_REFERENCE_ROOT, else
    a checkout named `reference` beside this repository."""
    candidates = [reference_root, os.environ.get("MINFER_REFERENCE_ROOT"),
                  os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")]
    for c in candidates:
        if c and os.path.exists(os.path.join(c, "src", "minfer", "kernels", "torch_ext", "csrc", "quants", "impl.cpp")):
            return c
    return None


def build_ref(reference_root=None) -> bool:
    """Compile the reference's quant codec from its own sources (only where the reference tree exists)."""
    reference_root = find_reference_root(reference_root)
    if reference_root is None:
        return reference_build_available()
    rc = subprocess.run(["make", "-C", _HERE, "_ref", f"REFERENCE={reference_root}",
                         f"TORCH_INCLUDE={os.path.join(os.path.dirname(torch.__file__), 'include')}"],
                        capture_output=True, text=True)
    if rc.returncode != 0:
        raise RuntimeError("building oracle/_ref failed:\n" + rc.stdout + rc.stderr)
    return True


def within_tolerance(actual: torch.Tensor, expected: torch.Tensor, atol: float = 2e-3, rtol: float = 2e-3):
    """allclose with the path's stated tolerance; returns (ok, max_abs_err, n_bad)."""
    a = actual.detach().float().cpu()
    e = expected.detach().float().cpu()
    err = (a - e).abs()
    bad = err > (atol + rtol * e.abs())
    bad |= ~torch.isfinite(a)
    return (not bool(bad.any())), float(err.max()), int(bad.sum())
