"""Timing harness with the reference's CLI (apps/benchmark.py:210-289 of dsuarez01/minfer-python):

    python apps/benchmark.py --kernel flash_attn --which minfer
    python apps/benchmark.py --kernel flash_attn --which ref       # torch SDPA on the GPU, for comparison

Same set-up as the reference: B=4, 48 query / 8 kv heads, head_dim 128, L in {4096, 8192, 16384},
inputs as transposed views, a dense causal bool mask, medians from torch.utils.benchmark's
blocked_autorange.  `--which ref` times torch's own scaled_dot_product_attention on expanded K/V
exactly as the reference's harness does; it is a comparison leg only, nothing in the package's ops
calls it.  `flash_attn_causal` and `flash_attn_decode` are added kernels.
"""
import argparse
import gc
import os
import sys

import torch
from torch.utils.benchmark import Compare, Timer

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from minfer.const import GGML_QUANT_SIZES, GGMLQuantizationType  # noqa: E402
from minfer.kernels import KernelBackend  # noqa: E402
from minfer.kernels import refs  # noqa: E402


def _views(B, L, n_heads, n_kv_heads, head_dim):
    Q = (1 / head_dim ** 0.5) * torch.randn((B, L, n_heads * head_dim), dtype=torch.float16).cuda()
    Q = Q.view(B, L, n_heads, head_dim).transpose(1, 2)
    K = (1 / head_dim ** 0.5) * torch.randn((B, L, n_kv_heads * head_dim), dtype=torch.float16).cuda()
    K = K.view(B, L, n_kv_heads, head_dim).transpose(1, 2)
    V = (1 / head_dim ** 0.5) * torch.randn((B, L, n_kv_heads * head_dim), dtype=torch.float16).cuda()
    V = V.view(B, L, n_kv_heads, head_dim).transpose(1, 2)
    return Q, K, V


def flash_attn(backend: str, which: str, causal_entry: bool = False):
    """flash_attn against pytorch SDPA"""
    kerns = KernelBackend(backend)
    B, n_heads, n_kv_heads, head_dim = 4, 48, 8, 128
    qtype = GGMLQuantizationType.F16
    qblock_size, qtype_size = GGML_QUANT_SIZES[qtype]
    results = []
    for L in [4096, 8192, 16384]:
        Q, K, V = _views(B, L, n_heads, n_kv_heads, head_dim)
        mask = (torch.arange(L).unsqueeze(0) <= torch.arange(L).unsqueeze(1))
        mask = mask.unsqueeze(0).unsqueeze(0).expand(B, 1, L, L).to(torch.bool).cuda()
        out = torch.zeros((B, n_heads, L, head_dim), dtype=torch.float16).cuda()
        n_rep = n_heads // n_kv_heads
        if which == "ref":
            K_exp = K.repeat_interleave(n_rep, dim=1)
            V_exp = V.repeat_interleave(n_rep, dim=1)

        def my_flash_attn():
            if causal_entry:
                kerns.flash_attn_causal(Q, K, V, out)
            else:
                kerns.flash_attn(qtype, qblock_size, qtype_size, Q, K, V, mask, out)

        def ref_flash_attn():
            refs.flash_attn(Q, K_exp, V_exp, mask)

        fn = my_flash_attn if which == "minfer" else ref_flash_attn
        timer = Timer(stmt="fn(); torch.cuda.synchronize()", globals={"fn": fn, "torch": torch},
                      label="flash_attn_causal" if causal_entry else "flash_attn",
                      sub_label=f"B={B}, L={L}, n_heads={n_heads}, n_kv_heads={n_kv_heads}, head_dim={head_dim}",
                      description=f"{which}")
        m = timer.blocked_autorange(min_run_time=0.5)
        results.append(m)
        print(f"L={L}: {m.median * 1e3:.3f} ms  {4 * B * n_heads * L * L * head_dim / 2 / m.median / 1e12:.1f} TFLOP/s "
              f"(causal-half convention)", flush=True)
        del Q, K, V, mask, out
        gc.collect()
        torch.cuda.empty_cache()
    Compare(results).print()


def flash_attn_causal(backend: str, which: str):
    flash_attn(backend, which, causal_entry=True)


def flash_attn_decode(backend: str, which: str):
    """split-KV decode over a padded cache: B=64, 32/8 heads, D=128, lengths uniform in [512, 8192]"""
    kerns = KernelBackend(backend)
    B, H, Hkv, D, Lmax = 64, 32, 8, 128, 8192
    lens = torch.randint(512, Lmax + 1, (B,), generator=torch.Generator().manual_seed(2), dtype=torch.int32)
    q = torch.randn(B, H, 1, D, dtype=torch.float16, device="cuda")
    kc = torch.randn(B, Hkv, Lmax, D, dtype=torch.float16, device="cuda")
    vc = torch.randn(B, Hkv, Lmax, D, dtype=torch.float16, device="cuda")
    out = torch.zeros_like(q)
    ld = lens.cuda()

    def mine():
        kerns.flash_attn_decode(q, kc, vc, ld, out)

    def ref():
        refs.flash_attn_decode(q, kc, vc, ld)

    fn = mine if which == "minfer" else ref
    m = Timer(stmt="fn(); torch.cuda.synchronize()", globals={"fn": fn, "torch": torch}, label="flash_attn_decode",
              sub_label=f"B={B}, Lmax={Lmax}", description=which).blocked_autorange(min_run_time=0.5)
    live = 2.0 * 2 * Hkv * D * float(lens.sum())
    print(f"{m.median * 1e3:.4f} ms  {live / m.median / 1e9:.0f} GB/s of live KV bytes", flush=True)
    Compare([m]).print()


if __name__ == "__main__":
    KERNELS = {"flash_attn": flash_attn, "flash_attn_causal": flash_attn_causal, "flash_attn_decode": flash_attn_decode}
    # the reference's two-stage parse (apps/benchmark.py:282-289): --kernel offers the public attributes of the backend
    parser = argparse.ArgumentParser()
    parser.add_argument("--backend", choices=["torch_ext"], default="torch_ext")
    args, _ = parser.parse_known_args()
    parser.add_argument("--kernel", choices=[k for k in vars(KernelBackend(args.backend)) if not k.startswith("_") and k in KERNELS],
                        required=True)
    parser.add_argument("--which", choices=["minfer", "ref"], required=True)
    args = parser.parse_args()
    KERNELS[args.kernel](backend=args.backend, which=args.which)
