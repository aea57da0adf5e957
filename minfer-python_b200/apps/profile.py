"""Single-shot launches of the attention kernels, for `ncu`.

Same role and flags as the reference's apps/profile.py (apps/profile.py:96-143 of
dsuarez01/minfer-python: one un-timed call per kernel under torch.no_grad()), with
shape flags added so a capture can run on a small case.  `--which ref` launches
torch's SDPA through refs.flash_attn, as the reference's script does.

    python apps/profile.py --kernel flash_attn_causal --batch 2 --seq 4096 --calls 3
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from minfer.const import GGML_QUANT_SIZES, GGMLQuantizationType  # noqa: E402
from minfer.kernels import KernelBackend  # noqa: E402
from minfer.kernels import refs  # noqa: E402


def _qkv(args, dtype):
    B, L, H, Hkv, D = args.batch, args.seq, args.heads, args.kv_heads, args.head_dim
    g = torch.Generator(device="cuda").manual_seed(args.seed)
    if args.transposed:  # the layout the reference's callers pass: [B, L, H*D] viewed as [B, H, L, D]
        q = torch.randn((B, L, H * D), dtype=dtype, device="cuda", generator=g).view(B, L, H, D).transpose(1, 2)
        k = torch.randn((B, L, Hkv * D), dtype=dtype, device="cuda", generator=g).view(B, L, Hkv, D).transpose(1, 2)
        v = torch.randn((B, L, Hkv * D), dtype=dtype, device="cuda", generator=g).view(B, L, Hkv, D).transpose(1, 2)
    else:
        q = torch.randn((B, H, L, D), dtype=dtype, device="cuda", generator=g)
        k = torch.randn((B, Hkv, L, D), dtype=dtype, device="cuda", generator=g)
        v = torch.randn((B, Hkv, L, D), dtype=dtype, device="cuda", generator=g)
    return q, k, v


def flash_attn(kerns, args, dtype):
    qtype = GGMLQuantizationType.F16
    qblock_size, qtype_size = GGML_QUANT_SIZES[qtype]
    q, k, v = _qkv(args, dtype)
    L = args.seq
    mask = (torch.arange(L, device="cuda").unsqueeze(0) <= torch.arange(L, device="cuda").unsqueeze(1))
    mask = mask.unsqueeze(0).unsqueeze(0).expand(args.batch, 1, L, L).to(torch.bool).contiguous()
    out = torch.zeros((args.batch, args.heads, L, args.head_dim), dtype=dtype, device="cuda")
    if args.which == "ref":
        n_rep = args.heads // args.kv_heads
        k_exp, v_exp = k.repeat_interleave(n_rep, dim=1), v.repeat_interleave(n_rep, dim=1)
        return lambda: refs.flash_attn(q, k_exp, v_exp, mask)
    return lambda: kerns.flash_attn(qtype, qblock_size, qtype_size, q, k, v, mask, out)


def flash_attn_causal(kerns, args, dtype):
    q, k, v = _qkv(args, dtype)
    out = torch.zeros((args.batch, args.heads, args.seq, args.head_dim), dtype=dtype, device="cuda")
    return lambda: kerns.flash_attn_causal(q, k, v, out)


def flash_attn_decode(kerns, args, dtype):
    B, H, Hkv, D, Lmax = args.batch, args.heads, args.kv_heads, args.head_dim, args.seq
    g = torch.Generator().manual_seed(args.seed)
    lens = torch.randint(max(1, Lmax // 16), Lmax + 1, (B,), generator=g, dtype=torch.int32)
    print(f"decode: sum(lens) = {int(lens.sum())}, live KV bytes = {int(lens.sum()) * Hkv * D * 2 * 2}")
    lens = lens.cuda()
    q = torch.randn((B, H, 1, D), dtype=dtype, device="cuda")
    kc = torch.randn((B, Hkv, Lmax, D), dtype=dtype, device="cuda")
    vc = torch.randn((B, Hkv, Lmax, D), dtype=dtype, device="cuda")
    out = torch.zeros_like(q)
    return lambda: kerns.flash_attn_decode(q, kc, vc, lens, out)


def flash_attn_decode_q8(kerns, args, dtype):
    """the same decode over a GGML Q8_0 cache (random int8 values, every block scale 2^-7)"""
    B, H, Hkv, D, Lmax = args.batch, args.heads, args.kv_heads, args.head_dim, args.seq
    g = torch.Generator().manual_seed(args.seed)
    lens = torch.randint(max(1, Lmax // 16), Lmax + 1, (B,), generator=g, dtype=torch.int32)
    print(f"decode q8: sum(lens) = {int(lens.sum())}, live KV bytes = {int(lens.sum()) * Hkv * (D // 32) * 34 * 2}")
    lens = lens.cuda()
    q = torch.randn((B, H, 1, D), dtype=dtype, device="cuda")
    caches = []
    for _ in range(2):
        c = torch.randint(0, 256, (B, Hkv, Lmax, D // 32, 34), dtype=torch.uint8, device="cuda")
        c[..., 0] = 0x00
        c[..., 1] = 0x20   # fp16 0x2000 = 2^-7
        caches.append(c.view(B, Hkv, Lmax, D // 32 * 34))
    out = torch.zeros_like(q)
    return lambda: kerns.flash_attn_decode_q8(q, caches[0], caches[1], lens, out)


def rope_kv_append(kerns, args, dtype):
    """interleaved RoPE of q and k fused with the append of k and v to a [B, Hkv, 2*seq, D] cache"""
    B, H, Hkv, D, L = args.batch, args.heads, args.kv_heads, args.head_dim, args.seq
    q = torch.randn((B, L, H, D), dtype=dtype, device="cuda")
    k = torch.randn((B, L, Hkv, D), dtype=dtype, device="cuda")
    v = torch.randn((B, L, Hkv, D), dtype=dtype, device="cuda")
    kc = torch.zeros((B, Hkv, 2 * L, D), dtype=dtype, device="cuda")
    vc = torch.zeros_like(kc)
    start = torch.zeros(B, dtype=torch.int32, device="cuda")
    print(f"rope_kv_append: bytes = {2 * B * L * D * (2 * H + 4 * Hkv)}")
    return lambda: kerns.rope_kv_append(D, 500000.0, 0, q, k, v, kc, vc, start)


if __name__ == "__main__":
    KERNELS = {"flash_attn": flash_attn, "flash_attn_causal": flash_attn_causal, "flash_attn_decode": flash_attn_decode,
               "flash_attn_decode_q8": flash_attn_decode_q8, "rope_kv_append": rope_kv_append}
    parser = argparse.ArgumentParser()
    parser.add_argument("--backend", choices=["torch_ext"], default="torch_ext")
    parser.add_argument("--kernel", choices=sorted(KERNELS), required=True)
    parser.add_argument("--which", choices=["minfer", "ref"], default="minfer")
    parser.add_argument("--batch", type=int, default=4)
    parser.add_argument("--seq", type=int, default=4096, help="sequence length (prefill) or padded cache length (decode)")
    parser.add_argument("--heads", type=int, default=32)
    parser.add_argument("--kv-heads", type=int, default=8)
    parser.add_argument("--head-dim", type=int, default=128)
    parser.add_argument("--dtype", choices=["float16", "bfloat16"], default="float16")
    parser.add_argument("--transposed", action="store_true")
    parser.add_argument("--calls", type=int, default=1)
    parser.add_argument("--seed", type=int, default=0)
    args = parser.parse_args()
    fn = KERNELS[args.kernel](KernelBackend(args.backend), args, getattr(torch, args.dtype))
    with torch.no_grad():
        for _ in range(args.calls):
            fn()
    torch.cuda.synchronize()
