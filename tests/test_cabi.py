"""CPU: the C-ABI library loads, exports what include/minfer_attn.h declares, and
rejects bad arguments before touching a device."""
import ctypes
import os
import re

import pytest

from conftest import ROOT


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "minfer_attn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(minfer_attn_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_entry_points():
    syms = declared_symbols()
    for s in ("minfer_attn_prefill", "minfer_attn_decode", "minfer_attn_decode_workspace_bytes",
              "minfer_attn_strerror", "minfer_attn_abi_version"):
        assert s in syms


def test_library_exports_every_declared_symbol():
    from minfer.kernels.torch_ext import _lib
    for s in declared_symbols():
        assert hasattr(_lib.lib, s), f"{s} declared in the header but not exported"
    assert _lib.lib.minfer_attn_abi_version() == 5
    assert set(_lib.EXPORTS) <= set(declared_symbols())


def test_invalid_arguments_are_rejected_without_a_device():
    from minfer.kernels.torch_ext import _lib
    L = _lib.lib
    assert L.minfer_attn_prefill(None, None) == 1
    p = _lib.PrefillParams()
    assert L.minfer_attn_prefill(ctypes.byref(p), None) == 1          # null pointers
    p.q = p.k = p.v = p.out = 0x1000
    p.batch, p.n_heads, p.n_kv_heads, p.seq_q, p.seq_k, p.head_dim = 1, 6, 4, 128, 128, 128
    assert L.minfer_attn_prefill(ctypes.byref(p), None) == 1          # heads not a multiple of kv heads
    p.n_kv_heads = 2
    p.head_dim = 96
    assert L.minfer_attn_prefill(ctypes.byref(p), None) == 2          # unsupported head_dim
    p.head_dim = 128
    p.q = 0x1004
    assert L.minfer_attn_prefill(ctypes.byref(p), None) == 1          # misaligned base pointer
    p.q = 0x1000
    p.q_stride[2] = 132
    assert L.minfer_attn_prefill(ctypes.byref(p), None) == 1          # stride not a multiple of 8 elements
    p.q_stride[2] = 128
    p.causal, p.seq_k = 1, 64
    assert L.minfer_attn_prefill(ctypes.byref(p), None) == 1          # causal with fewer keys than queries
    p.causal, p.seq_k = 1, 128
    p.n_peer_out = 8
    assert L.minfer_attn_prefill(ctypes.byref(p), None) == 1          # more output replicas than the struct holds
    p.n_peer_out = 1
    assert L.minfer_attn_prefill(ctypes.byref(p), None) == 1          # a null replica pointer
    p.peer_out[0] = 0x2000
    p.causal, p.mask = 0, 0x3000
    assert L.minfer_attn_prefill(ctypes.byref(p), None) == 2          # replicas with a dense mask: unsupported
    p.n_peer_out, p.mask, p.flags = 0, None, 4
    assert L.minfer_attn_prefill(ctypes.byref(p), None) == 2          # reserved flags word
    d = _lib.DecodeParams()
    assert L.minfer_attn_decode(ctypes.byref(d), None) == 1
    d.q = d.k_cache = d.v_cache = d.lens = d.out = 0x1000
    d.batch, d.n_heads, d.n_kv_heads, d.max_len, d.head_dim = 2, 8, 2, 1024, 128
    d.chunk = 100
    assert L.minfer_attn_decode(ctypes.byref(d), None) == 1           # chunk not a multiple of 64
    d.chunk = 0
    assert L.minfer_attn_decode(ctypes.byref(d), None) == 5           # no workspace
    d.n_heads, d.n_kv_heads = 34, 2
    assert L.minfer_attn_decode(ctypes.byref(d), None) == 2           # group of 17 > 16
    r = _lib.RopeParams()
    assert L.minfer_attn_rope_append(ctypes.byref(r), None) == 1      # no tensors at all
    r.q = 0x1000
    r.batch, r.seq, r.n_heads, r.head_dim, r.rotary_dim, r.freq_base = 1 << 15, 1 << 13, 8, 128, 128, 10000.0
    assert L.minfer_attn_rope_append(ctypes.byref(r), None) == 1      # 2^32 (token, chunk) pairs: beyond the 32-bit index
    r.batch, r.seq, r.rotary_dim = 2, 16, 12
    assert L.minfer_attn_rope_append(ctypes.byref(r), None) == 1      # rotary_dim not a multiple of 8
    r.head_dim, r.rotary_dim = 256, 256
    assert L.minfer_attn_rope_append(ctypes.byref(r), None) == 2      # more than 64 frequencies: unsupported
    for code in range(0, 6):
        assert len(_lib.strerror(code)) > 0


def test_workspace_size_formula():
    from minfer.kernels.torch_ext import _lib
    L = _lib.lib
    assert L.minfer_attn_decode_default_chunk(64, 8, 8192) == 512
    assert L.minfer_attn_decode_workspace_bytes(64, 32, 8192, 128, 512) == 64 * 32 * 16 * 130 * 4
    assert L.minfer_attn_decode_workspace_bytes(64, 32, 8192, 128, 0) == 64 * 32 * 16 * 130 * 4
    assert L.minfer_attn_decode_workspace_bytes(64, 32, 8192, 96, 512) == 0
    assert L.minfer_attn_decode_workspace_bytes(1, 1, 1, 64, 64) == 66 * 4


def test_prefill_mask_workspace_size():
    from minfer.kernels.torch_ext import _lib
    L = _lib.lib
    assert L.minfer_attn_prefill_workspace_bytes(4, 4096, 4096) == 16 + 4 * 32 * 32   # work-item counter + tile classes
    assert L.minfer_attn_prefill_workspace_bytes(1, 129, 1) == 16 + 2
    assert L.minfer_attn_prefill_workspace_bytes(0, 128, 128) == 0
    p = _lib.PrefillParams()
    p.q = p.k = p.v = p.out = p.mask = 0x1000
    p.batch, p.n_heads, p.n_kv_heads, p.seq_q, p.seq_k, p.head_dim = 1, 2, 2, 128, 128 * 1024 + 1, 128
    assert L.minfer_attn_prefill(ctypes.byref(p), None) == 2           # masked call beyond 1024 key tiles


def test_ops_have_no_cpu_path():
    import torch
    from minfer.kernels import KernelBackend
    k = KernelBackend("torch_ext")
    q = torch.zeros(1, 2, 8, 64, dtype=torch.float16)
    m = torch.ones(1, 1, 8, 8, dtype=torch.bool)
    with pytest.raises(NotImplementedError):
        k.flash_attn(1, 1, 2, q, q, q, m, q.clone())
    with pytest.raises(NotImplementedError):
        k.flash_attn_causal(q, q, q, q.clone())
    with pytest.raises(ValueError):
        KernelBackend("triton")


def test_reference_callers_find_their_imports():
    """The reference's test file and apps begin with `from minfer.kernels import refs`, `from minfer.kernels
    import KernelBackend`, `from minfer.const import GGMLQuantizationType, GGML_QUANT_SIZES` and (conftest)
    `import minfer.kernels.torch_ext` (test/kernels.py:9-11, test/conftest.py:2, apps/benchmark.py:11-13):
    all of them resolve against this package, the qtype the attention callers pass is an int-valued enum
    member with the (1, 2) size pair, and refs.flash_attn is torch's SDPA on a bool mask."""
    import torch
    from minfer.kernels import refs
    from minfer.kernels import KernelBackend
    from minfer.const import GGMLQuantizationType, GGML_QUANT_SIZES
    import minfer.kernels.torch_ext  # noqa: F401

    kerns = KernelBackend("torch_ext")
    assert callable(kerns.flash_attn) and callable(kerns.il_rope) and callable(kerns.neox_rope)
    assert "flash_attn" in [k for k in vars(kerns) if not k.startswith("_")]   # the apps build --kernel choices this way
    qtype = GGMLQuantizationType.F16
    assert int(qtype) == 1 and GGML_QUANT_SIZES[qtype] == (1, 2)
    with pytest.raises(ValueError):
        KernelBackend("triton")
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(1, 2, 5, 8, generator=g) for _ in range(3))
    mask = torch.tril(torch.ones(5, 5, dtype=torch.bool))[None, None]
    want = torch.softmax((q @ k.transpose(-1, -2) / 8 ** 0.5).masked_fill(~mask, float("-inf")), -1) @ v
    assert torch.allclose(refs.flash_attn(q, k, v, mask), want, atol=1e-6)
    lens = torch.tensor([3])
    assert torch.allclose(refs.flash_attn_decode(q[:, :, :1], k, v, lens),
                          torch.softmax(q[:, :, :1] @ k[:, :, :3].transpose(-1, -2) / 8 ** 0.5, -1) @ v[:, :, :3], atol=1e-6)


def test_refs_rope_matches_the_oracle_restatement():
    import torch
    from minfer.kernels import refs
    from oracle import oracle as O
    x = torch.randn(2, 5, 3, 64, generator=torch.Generator().manual_seed(1)).half()
    for rot in (64, 32):
        assert torch.allclose(refs.il_rope(x, rot, 7, 10000.0).float(), O.il_rope_reference(x, rot, 7, 10000.0).float(), atol=2e-3)
        assert torch.allclose(refs.neox_rope(x, rot, 7, 10000.0).float(), O.neox_rope_reference(x, rot, 7, 10000.0).float(), atol=2e-3)
