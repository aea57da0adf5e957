"""PyTorch statements of the attention path's ops, for the callers that compare against them.

Counterpart of the reference's src/minfer/kernels/refs.py (dsuarez01/minfer-python): its test file
and its two apps do `from minfer.kernels import refs` and call `refs.flash_attn` as the expected
value / the `--which ref` leg (test/kernels.py:9, apps/benchmark.py:11,248, apps/profile.py:118).
Only the functions that belong to the attention path exist here.  This module is a comparison aid:
nothing in minfer.kernels.torch_ext imports it and no op falls back to it.
"""
import torch
import torch.nn.functional as F


def flash_attn(Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    """torch SDPA with a bool mask (True = attend), as refs.py:53-55 of the reference states it.
    Q/K/V: [B, n_heads, L, head_dim]; K/V already expanded to n_heads for grouped-query attention."""
    return F.scaled_dot_product_attention(Q, K, V, attn_mask=mask)


def flash_attn_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, lens: torch.Tensor) -> torch.Tensor:
    """One query token per sequence over a padded cache: the same SDPA call with a length mask
    (key j of sequence b visible iff j < lens[b]).  q [B, n_heads, 1, D]; caches [B, n_kv_heads, Lmax, D]."""
    Lmax = k_cache.size(2)
    mask = (torch.arange(Lmax, device=q.device)[None, :] < lens.to(q.device).long()[:, None])[:, None, None, :]
    return F.scaled_dot_product_attention(q, k_cache, v_cache, attn_mask=mask, enable_gqa=True)


def _rope_angles(x: torch.Tensor, rotary_dim: int, start_pos: int, base_freq: float) -> torch.Tensor:
    # [L, 1, rotary_dim/2] complex rotations: freq_i = base^(-2i/rot), angle = (start_pos + l) * freq_i (fp32)
    i = torch.arange(rotary_dim // 2, dtype=torch.float32, device=x.device)
    pos = torch.arange(x.size(1), dtype=torch.float32, device=x.device) + start_pos
    ang = pos[:, None] * (base_freq ** (-2.0 * i / rotary_dim))[None, :]
    return torch.polar(torch.ones_like(ang), ang)[:, None, :]


def il_rope(x: torch.Tensor, rotary_dim: int, start_pos: int, base_freq: float) -> torch.Tensor:
    """Interleaved-pair RoPE of x [B, L, n_heads, head_dim] (semantics of refs.py:12-28 of the reference,
    with the angle table broadcast over the head axis so that any L works)."""
    xf = x.float()
    pairs = torch.view_as_complex(xf[..., :rotary_dim].reshape(*xf.shape[:-1], rotary_dim // 2, 2).contiguous())
    xf[..., :rotary_dim] = torch.view_as_real(pairs * _rope_angles(x, rotary_dim, start_pos, base_freq)).flatten(-2)
    return xf.to(x.dtype)


def neox_rope(x: torch.Tensor, rotary_dim: int, start_pos: int, base_freq: float) -> torch.Tensor:
    """Two-halves RoPE of x [B, L, n_heads, head_dim] (semantics of refs.py:30-47 of the reference)."""
    xf = x.float()
    half = rotary_dim // 2
    pairs = torch.complex(xf[..., :half].contiguous(), xf[..., half:rotary_dim].contiguous())
    rot = pairs * _rope_angles(x, rotary_dim, start_pos, base_freq)
    xf[..., :half] = rot.real
    xf[..., half:rotary_dim] = rot.imag
    return xf.to(x.dtype)
