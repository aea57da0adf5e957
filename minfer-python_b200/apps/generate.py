"""Greedy generation with a Llama-shaped decoder on the B200 attention path.

The reference's apps/generate.py is a one-line stub ("# TODO: complete") and its model layer
does not import (src/minfer/utils.py:260); the call order implemented here is the one its
skeleton intends (src/minfer/core.py:65-75 and :219-241): embed -> per layer [rmsnorm -> qkv ->
RoPE -> attention -> o-proj -> rmsnorm -> SwiGLU] -> rmsnorm -> lm head, with per-layer KV caches
of shape [batch, n_kv_heads, max_seq_len, head_dim] (core.py:105-127).

Projections, norms and the FFN are library calls (torch / cuBLAS): they are outside this
package's scope.  Attention is this package: `rope_kv_append` rotates q/k and appends k/v to
the cache in one pass, `flash_attn_causal` does the prompt, `flash_attn_decode` every generated
token.  Weights are random N(0, 0.02) — there is no checkpoint to load here.

    python apps/generate.py                         # Llama-3.2-1B shape, 8 prompts x 512, 128 new tokens
    python apps/generate.py --layers 4 --hidden 512 --heads 8 --kv-heads 2 --ffn 1024 --vocab 1000 \
        --batch 2 --prompt-len 64 --new-tokens 8
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from dataclasses import dataclass

import torch
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from minfer.kernels import KernelBackend  # noqa: E402


@dataclass
class Shape:
    layers: int = 16
    hidden: int = 2048
    heads: int = 32
    kv_heads: int = 8
    head_dim: int = 64
    ffn: int = 8192
    vocab: int = 128256
    rope_theta: float = 500000.0
    rope_style: int = 0          # 0 interleaved pairs (the reference's il_rope), 1 neox halves
    eps: float = 1e-5


class Decoder:
    """Decoder-only transformer with random weights; attention through KernelBackend."""

    def __init__(self, shape: Shape, batch: int, max_len: int, device="cuda", dtype=torch.float16, seed: int = 4,
                 init_on_device: bool = False):
        self.s, self.batch, self.max_len, self.dev, self.dtype = shape, batch, max_len, torch.device(device), dtype
        self.kerns = KernelBackend("torch_ext")
        # weights drawn on the CPU are the same bits everywhere (the tests' CPU twin needs that); drawing the
        # 1.2 G values of the full shape on the device saves ten seconds where only timing matters
        g = torch.Generator(device=self.dev if init_on_device else "cpu").manual_seed(seed)
        s = shape
        qkv_out = (s.heads + 2 * s.kv_heads) * s.head_dim

        def w(*dims):
            if init_on_device:
                return (0.02 * torch.randn(*dims, generator=g, device=self.dev)).to(dtype)
            return (0.02 * torch.randn(*dims, generator=g)).to(dtype).to(self.dev)

        self.embed = w(s.vocab, s.hidden)
        self.lm_head = w(s.vocab, s.hidden)
        self.final_norm = torch.ones(s.hidden, dtype=dtype, device=self.dev)
        self.layers = []
        for _ in range(s.layers):
            self.layers.append(dict(
                attn_norm=torch.ones(s.hidden, dtype=dtype, device=self.dev),
                wqkv=w(qkv_out, s.hidden),
                wo=w(s.hidden, s.heads * s.head_dim),
                ffn_norm=torch.ones(s.hidden, dtype=dtype, device=self.dev),
                w_gate_up=w(2 * s.ffn, s.hidden),
                w_down=w(s.hidden, s.ffn),
                k_cache=torch.zeros(batch, s.kv_heads, max_len, s.head_dim, dtype=dtype, device=self.dev),
                v_cache=torch.zeros(batch, s.kv_heads, max_len, s.head_dim, dtype=dtype, device=self.dev),
            ))
        self.lens = torch.zeros(batch, dtype=torch.int32, device=self.dev)  # tokens in the cache per sequence
        self.attn_ms = 0.0
        self._ev = []

    # -- attention through the package's ops --------------------------------------------------
    def _attention(self, lay, qkv: torch.Tensor, L: int, time_it: bool) -> torch.Tensor:
        s, B = self.s, qkv.shape[0]
        nq, nkv = s.heads * s.head_dim, s.kv_heads * s.head_dim
        q = qkv[..., :nq].view(B, L, s.heads, s.head_dim)
        k = qkv[..., nq:nq + nkv].view(B, L, s.kv_heads, s.head_dim)
        v = qkv[..., nq + nkv:].view(B, L, s.kv_heads, s.head_dim)
        out = torch.empty(B, L, s.heads, s.head_dim, dtype=self.dtype, device=self.dev)
        if time_it:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        self.kerns.rope_kv_append(s.head_dim, s.rope_theta, s.rope_style, q, k, v, lay["k_cache"], lay["v_cache"],
                                  self.lens)
        if L > 1:   # prompt: causal attention over the rows just written (the cache starts empty)
            self.kerns.flash_attn_causal(q.transpose(1, 2), lay["k_cache"][:, :, :L], lay["v_cache"][:, :, :L],
                                         out.transpose(1, 2))
        else:       # one new token per sequence over lens + 1 cached keys
            self.kerns.flash_attn_decode(q.transpose(1, 2), lay["k_cache"], lay["v_cache"], self._lens_plus,
                                         out.transpose(1, 2))
        if time_it:
            e1.record()
            self._ev.append((e0, e1))
        return out.view(B, L, nq)

    def forward(self, tokens: torch.Tensor, time_attention: bool = False) -> torch.Tensor:
        """tokens [B, L] (L = prompt length, or 1 for a decode step) -> logits of the last position [B, vocab]."""
        s = self.s
        B, L = tokens.shape
        x = self.embed[tokens]
        if L == 1:
            self._lens_plus = self.lens + 1
        for lay in self.layers:
            h = F.rms_norm(x, (s.hidden,), lay["attn_norm"], s.eps)
            a = self._attention(lay, F.linear(h, lay["wqkv"]), L, time_attention)
            x = x + F.linear(a, lay["wo"])
            h = F.rms_norm(x, (s.hidden,), lay["ffn_norm"], s.eps)
            gu = F.linear(h, lay["w_gate_up"])
            x = x + F.linear(F.silu(gu[..., :s.ffn]) * gu[..., s.ffn:], lay["w_down"])
        self.lens += L
        x = F.rms_norm(x[:, -1], (s.hidden,), self.final_norm, s.eps)
        return F.linear(x, self.lm_head)

    def attention_ms(self) -> float:
        torch.cuda.synchronize()
        ms = sum(a.elapsed_time(b) for a, b in self._ev)
        self._ev = []
        return ms


def generate(model: Decoder, prompts: torch.Tensor, new_tokens: int, time_attention: bool = True,
             use_graph: bool = False):
    """Greedy decoding; returns (generated ids [B, new_tokens], timing dict).

    use_graph captures one decode step (all layers) in a CUDA graph and replays it per token: the
    step is ~200 small launches and launch-bound otherwise.  Attention is not timed separately then.
    """
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    torch.cuda.synchronize()
    ev[0].record()
    logits = model.forward(prompts, time_attention)
    nxt = logits.argmax(dim=-1)
    ev[1].record()
    prefill_attn = model.attention_ms() if time_attention else None
    out = [nxt]
    if use_graph and new_tokens > 1:
        time_attention = False
        tok = nxt[:, None].clone()
        lens0 = model.lens.clone()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):          # one eager step on the side stream, as capture requires
            model.forward(tok)
        torch.cuda.current_stream().wait_stream(side)
        model.lens.copy_(lens0)                # undo the warm-up step's cache advance
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            static_logits = model.forward(tok)
        model.lens.copy_(lens0)
        torch.cuda.synchronize()
        ev[3].record()                         # decode timing starts after the capture
        for _ in range(new_tokens - 1):
            graph.replay()
            nxt = static_logits.argmax(dim=-1)
            tok.copy_(nxt[:, None])
            out.append(nxt)
    else:
        for _ in range(new_tokens - 1):
            logits = model.forward(nxt[:, None], time_attention)
            nxt = logits.argmax(dim=-1)
            out.append(nxt)
    ev[2].record()
    torch.cuda.synchronize()
    decode_attn = model.attention_ms() if time_attention else None
    B, L = prompts.shape
    t_prefill = ev[0].elapsed_time(ev[1])
    t_decode = ev[3].elapsed_time(ev[2]) if (use_graph and new_tokens > 1) else ev[1].elapsed_time(ev[2])
    stats = {
        "prefill_ms": t_prefill, "prefill_tokens_per_s": B * L / t_prefill * 1e3,
        "decode_ms_per_step": t_decode / max(1, new_tokens - 1),
        "decode_tokens_per_s": B * (new_tokens - 1) / t_decode * 1e3 if new_tokens > 1 else None,
        "prefill_attention_share": prefill_attn / t_prefill if time_attention else None,
        "decode_attention_share": decode_attn / t_decode if time_attention and new_tokens > 1 else None,
    }
    return torch.stack(out, dim=1), stats


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--backend", choices=["torch_ext"], default="torch_ext")
    ap.add_argument("--layers", type=int, default=16)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=64)
    ap.add_argument("--ffn", type=int, default=8192)
    ap.add_argument("--vocab", type=int, default=128256)
    ap.add_argument("--rope-theta", type=float, default=500000.0)
    ap.add_argument("--rope-style", type=int, choices=[0, 1], default=0)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--new-tokens", type=int, default=128)
    ap.add_argument("--seed", type=int, default=5)
    ap.add_argument("--no-attention-timing", action="store_true")
    ap.add_argument("--cuda-graph", action="store_true", help="replay the decode step from a CUDA graph")
    args = ap.parse_args()
    shape = Shape(args.layers, args.hidden, args.heads, args.kv_heads, args.head_dim, args.ffn, args.vocab,
                  args.rope_theta, args.rope_style)
    model = Decoder(shape, args.batch, args.prompt_len + args.new_tokens)
    g = torch.Generator().manual_seed(args.seed)
    prompts = torch.randint(0, args.vocab, (args.batch, args.prompt_len), generator=g).cuda()
    with torch.no_grad():
        # untimed warm-up at the full shape (module loads, cuBLAS handles and algorithm choices, the allocator's
        # blocks, first-launch set-up), then reset the caches
        generate(model, prompts, 2, False)
        model.lens.zero_()
        ids, stats = generate(model, prompts, args.new_tokens, not args.no_attention_timing, args.cuda_graph)
    stats["first_ids"] = ids[0, :8].tolist()
    print(json.dumps(stats))
