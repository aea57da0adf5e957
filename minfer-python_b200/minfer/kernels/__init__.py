"""Dispatch facade with the reference's shape (src/minfer/kernels/__init__.py:2-18).

Only the attention path's attributes exist: `flash_attn`, `il_rope` and `neox_rope`
keep the reference's signatures; `flash_attn_causal`, `flash_attn_decode` (also over a
Q8_0 or a paged cache) and `rope_kv_append` are additions.
"""


class KernelBackend:
    def __init__(self, backend: str):
        if backend == "torch_ext":
            from .torch_ext import flash_attn, flash_attn_causal, flash_attn_decode
            from .torch_ext import il_rope, neox_rope, rope_kv_append
            from .torch_ext import flash_attn_decode_q8, rope_kv_append_q8
            from .torch_ext import flash_attn_decode_paged, rope_kv_append_paged
            self.flash_attn_decode_paged = flash_attn_decode_paged
            self.rope_kv_append_paged = rope_kv_append_paged
            self.flash_attn_decode_q8 = flash_attn_decode_q8
            self.rope_kv_append_q8 = rope_kv_append_q8
            self.il_rope = il_rope
            self.neox_rope = neox_rope
            self.rope_kv_append = rope_kv_append
            self.flash_attn = flash_attn
            self.flash_attn_causal = flash_attn_causal
            self.flash_attn_decode = flash_attn_decode
        else:
            raise ValueError(f"KernelBackend init: unsupported backend {backend}")
