"""Dispatch facade with the reference's shape (src/minfer/kernels/__init__.py:2-18).

Only the attention attributes exist: `flash_attn` keeps the reference's
signature; `flash_attn_causal` and `flash_attn_decode` are additions.
"""


class KernelBackend:
    def __init__(self, backend: str):
        if backend == "torch_ext":
            from .torch_ext import flash_attn, flash_attn_causal, flash_attn_decode
            self.flash_attn = flash_attn
            self.flash_attn_causal = flash_attn_causal
            self.flash_attn_decode = flash_attn_decode
        else:
            raise ValueError(f"KernelBackend init: unsupported backend {backend}")
