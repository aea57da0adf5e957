"""Generate tests/golden/*.npz by running the REFERENCE's own CPU attention.

Run in a container where the reference tree is mounted:

    python tests/golden/make_golden.py [/path/to/reference]

It loads the reference's src/minfer/kernels/refs.py by file path (the module is
plain PyTorch) and records refs.flash_attn outputs for seeded inputs, with K/V
expanded by repeat_interleave and masks built the way the reference's tests do
(test/kernels.py:242,253-255,276-278).  16-bit cases store the rounded inputs
as raw uint16 and the output of the reference on their fp32 upcast; the decode
cases use the same function with a one-row query and a length mask.  The
vectors pin the oracle under oracle/ and are compared with the CUDA kernels in
the GPU tests.  Nothing reads the reference tree at test time.
"""
from __future__ import annotations

import hashlib
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def load_reference_refs(root: str):
    path = os.path.join(root, "src", "minfer", "kernels", "refs.py")
    spec = importlib.util.spec_from_file_location("reference_refs", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def bits16(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def causal_mask(B, L):
    return (torch.arange(L).unsqueeze(0) <= torch.arange(L).unsqueeze(1)).unsqueeze(0).unsqueeze(0).expand(B, 1, L, L).to(torch.bool)


def window_mask(B, L, w):
    dist = torch.arange(L).unsqueeze(0) - torch.arange(L).unsqueeze(1)
    return (dist.abs() < w).unsqueeze(0).unsqueeze(0).expand(B, 1, L, L).to(torch.bool)


PREFILL_CASES = [
    # name, seed, B, H, Hkv, L, D, dtype, mask kind
    ("prefill_causal_g4_d128", 11, 1, 8, 2, 160, 128, torch.float16, "causal"),
    ("prefill_window_g6_d128", 12, 1, 6, 1, 200, 128, torch.float16, "window48"),
    ("prefill_random_g1_d64", 13, 2, 2, 2, 130, 64, torch.float16, "random"),
    ("prefill_causal_bf16_g8_d128", 14, 1, 8, 1, 128, 128, torch.bfloat16, "causal"),
    ("prefill_causal_g4_d64", 15, 1, 4, 1, 257, 64, torch.float16, "causal"),
]

DECODE_CASES = [
    # name, seed, B, H, Hkv, Lmax, D, dtype, lens
    ("decode_g4_d128", 21, 3, 8, 2, 300, 128, torch.float16, [1, 17, 300]),
    ("decode_g1_d64_bf16", 22, 3, 4, 4, 100, 64, torch.bfloat16, [100, 64, 33]),
    ("decode_g6_d128", 23, 2, 6, 1, 1100, 128, torch.float16, [1100, 513]),
]


def main():
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("MINFER_REFERENCE_ROOT")
    if not root:
        raise SystemExit("usage: make_golden.py /path/to/minfer-python   (or set MINFER_REFERENCE_ROOT)")
    refs = load_reference_refs(root)
    torch.set_num_threads(1)  # one summation order, whatever the host

    # configuration 1 of the benchmark list: fp32, B=1, 8/8 heads, D=64, L=256,
    # seed 0 drawn in the order Q, K, V; causal
    g = torch.Generator().manual_seed(0)
    q = torch.randn(1, 8, 256, 64, generator=g)
    k = torch.randn(1, 8, 256, 64, generator=g)
    v = torch.randn(1, 8, 256, 64, generator=g)
    out = refs.flash_attn(q, k, v, causal_mask(1, 256))
    # inputs are regenerated from the seed at test time; their digest guards
    # against a generator that draws different numbers
    digest = hashlib.sha256(q.numpy().tobytes() + k.numpy().tobytes() + v.numpy().tobytes()).hexdigest()
    np.savez(os.path.join(HERE, "config1_fp32.npz"), out=out.numpy(), inputs_sha256=np.array(digest))

    for name, seed, B, H, Hkv, L, D, dtype, kind in PREFILL_CASES:
        g = torch.Generator().manual_seed(seed)
        q = torch.randn(B, H, L, D, generator=g).to(dtype)
        k = torch.randn(B, Hkv, L, D, generator=g).to(dtype)
        v = torch.randn(B, Hkv, L, D, generator=g).to(dtype)
        if kind == "causal":
            mask = causal_mask(B, L)
        elif kind.startswith("window"):
            mask = window_mask(B, L, int(kind[6:]))
        else:
            mask = (torch.rand(B, 1, L, L, generator=g) < 0.5)
            mask[:, :, 7, :] = False  # a row that sees nothing
            mask[:, :, 9, :] = False
            mask[:, :, 9, 100] = True  # a row that sees exactly one key
        n_rep = H // Hkv
        out = refs.flash_attn(q.float(), k.float().repeat_interleave(n_rep, dim=1),
                              v.float().repeat_interleave(n_rep, dim=1), mask)
        np.savez(os.path.join(HERE, name + ".npz"), q=bits16(q), k=bits16(k), v=bits16(v),
                 mask=np.packbits(mask.contiguous().numpy()), mask_shape=np.array(mask.shape),
                 out=out.numpy(), bf16=np.array(dtype == torch.bfloat16))

    for name, seed, B, H, Hkv, Lmax, D, dtype, lens in DECODE_CASES:
        g = torch.Generator().manual_seed(seed)
        q = torch.randn(B, H, 1, D, generator=g).to(dtype)
        kc = torch.randn(B, Hkv, Lmax, D, generator=g).to(dtype)
        vc = torch.randn(B, Hkv, Lmax, D, generator=g).to(dtype)
        lens_t = torch.tensor(lens, dtype=torch.int32)
        mask = (torch.arange(Lmax)[None, :] < lens_t[:, None].long())[:, None, None, :]
        n_rep = H // Hkv
        out = refs.flash_attn(q.float(), kc.float().repeat_interleave(n_rep, dim=1),
                              vc.float().repeat_interleave(n_rep, dim=1), mask)
        np.savez(os.path.join(HERE, name + ".npz"), q=bits16(q), k=bits16(kc), v=bits16(vc),
                 lens=lens_t.numpy(), out=out.numpy(), bf16=np.array(dtype == torch.bfloat16))
    # RoPE: the reference's il_rope / neox_rope oracles (refs.py:12-47) on fp16 inputs [B, L, H, D].
    # Those functions broadcast their [L, rot/2] angle table against the HEAD axis of x, so they
    # only run for L == 1; the vectors are therefore assembled one token at a time, token l being
    # rotated by a call with start_pos + l — the per-token position the reference's CUDA kernels use
    # (csrc/cuda/il_rope/kernel.cuh:17-23).
    def per_token(fn, x, rot, start, base):
        return torch.cat([fn(x[:, l:l + 1].clone(), rot, start + l, base) for l in range(x.shape[1])], dim=1)
    for name, seed, B, L, H, D, rot, base in [("rope_d128_rot64", 31, 2, 40, 3, 128, 64, 1e6),
                                              ("rope_d64_rot64", 32, 1, 24, 2, 64, 64, 500000.0)]:
        g = torch.Generator().manual_seed(seed)
        x = torch.randn(B, L, H, D, generator=g).half()
        out = {}
        for start in (0, 2048):
            out[f"il_{start}"] = bits16(per_token(refs.il_rope, x, rot, start, base))
            out[f"neox_{start}"] = bits16(per_token(refs.neox_rope, x, rot, start, base))
        np.savez(os.path.join(HERE, name + ".npz"), x=bits16(x), rot=np.array(rot), base=np.array(base), **out)
    # GGML Q8_0: bytes produced by the reference's own quant_row_q8_0 (compiled from its source into
    # oracle/_ref by `make -C oracle _ref`) and its fp16 dequantisation
    sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
    from oracle import oracle as O
    if O.build_ref(root):
        g = torch.Generator().manual_seed(41)
        x = (torch.randn(24, 128, generator=g) * torch.logspace(-3, 2, 24)[:, None]).half()
        x[3, :32] = 0
        x[5, 40] = 60000.0
        qb = O.q8_0_quantize_ref(x.float())
        np.savez(os.path.join(HERE, "q8_0_rows.npz"), x=bits16(x), q=qb.numpy(),
                 deq16=bits16(O.q8_0_dequantize_ref(qb, torch.float16)))
    print("wrote", sorted(f for f in os.listdir(HERE) if f.endswith(".npz")))


if __name__ == "__main__":
    main()
