"""GPU: the generate app's decoder (prefill -> cache -> decode steps on the package's ops) against an
fp32 CPU twin that recomputes full causal attention with the oracle at every step (teacher-forced)."""
import importlib.util
import os
import sys

import pytest
import torch
import torch.nn.functional as F

from conftest import PKG_ROOT
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def load_generate_app():
    """Import apps/generate.py by path (putting apps/ on sys.path would shadow the stdlib `profile`)."""
    spec = importlib.util.spec_from_file_location("minfer_generate_app", os.path.join(PKG_ROOT, "apps", "generate.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod  # dataclasses look their module up there
    spec.loader.exec_module(mod)
    return mod


def twin_logits(model, tokens):
    """fp32 CPU forward over the whole sequence, no cache; logits of the last position."""
    s = model.s
    x = model.embed.float().cpu()[tokens.cpu()]
    B, T, _ = x.shape
    rope = O.il_rope_reference if s.rope_style == 0 else O.neox_rope_reference
    nq, nkv = s.heads * s.head_dim, s.kv_heads * s.head_dim
    for lay in model.layers:
        h = F.rms_norm(x, (s.hidden,), lay["attn_norm"].float().cpu(), s.eps)
        qkv = F.linear(h, lay["wqkv"].float().cpu())
        q = rope(qkv[..., :nq].reshape(B, T, s.heads, s.head_dim), s.head_dim, 0, s.rope_theta)
        k = rope(qkv[..., nq:nq + nkv].reshape(B, T, s.kv_heads, s.head_dim), s.head_dim, 0, s.rope_theta)
        v = qkv[..., nq + nkv:].reshape(B, T, s.kv_heads, s.head_dim)
        a = O.attention_f64(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), causal=True)
        x = x + F.linear(a.transpose(1, 2).reshape(B, T, nq), lay["wo"].float().cpu())
        h = F.rms_norm(x, (s.hidden,), lay["ffn_norm"].float().cpu(), s.eps)
        gu = F.linear(h, lay["w_gate_up"].float().cpu())
        x = x + F.linear(F.silu(gu[..., :s.ffn]) * gu[..., s.ffn:], lay["w_down"].float().cpu())
    x = F.rms_norm(x[:, -1], (s.hidden,), model.final_norm.float().cpu(), s.eps)
    return F.linear(x, model.lm_head.float().cpu())


@pytest.mark.parametrize("rope_style,head_dim", [(0, 64), (1, 128)])
def test_prefill_then_decode_matches_twin(rope_style, head_dim):
    G = load_generate_app()
    shape = G.Shape(layers=2, hidden=256, heads=4, kv_heads=2, head_dim=head_dim, ffn=512, vocab=500,
                    rope_theta=500000.0, rope_style=rope_style)
    B, L, steps = 2, 150, 4
    model = G.Decoder(shape, B, L + steps)
    g = torch.Generator().manual_seed(5)
    tokens = torch.randint(0, shape.vocab, (B, L), generator=g)
    with torch.no_grad():
        got = model.forward(tokens.cuda())
        want = twin_logits(model, tokens)
        assert torch.allclose(got.float().cpu(), want, atol=2e-2, rtol=2e-2), (got.float().cpu() - want).abs().max()
        for _ in range(steps):
            nxt = want.argmax(dim=-1)                      # teacher forcing with the twin's choice
            tokens = torch.cat([tokens, nxt[:, None]], dim=1)
            got = model.forward(nxt[:, None].cuda())
            want = twin_logits(model, tokens)
            assert torch.allclose(got.float().cpu(), want, atol=2e-2, rtol=2e-2), (got.float().cpu() - want).abs().max()
    assert model.lens.tolist() == [L + steps] * B


def test_generate_runs_and_reports():
    G = load_generate_app()
    shape = G.Shape(layers=2, hidden=256, heads=8, kv_heads=2, head_dim=64, ffn=512, vocab=300)
    model = G.Decoder(shape, 3, 64 + 6)
    prompts = torch.randint(0, 300, (3, 64), generator=torch.Generator().manual_seed(1)).cuda()
    with torch.no_grad():
        ids, stats = G.generate(model, prompts, 6)
    assert ids.shape == (3, 6)
    assert 0.0 < stats["prefill_attention_share"] < 1.0 and stats["decode_tokens_per_s"] > 0
    # the CUDA-graph decode loop produces the same tokens
    model.lens.zero_()
    with torch.no_grad():
        ids_g, _ = G.generate(model, prompts, 6, False, use_graph=True)
    assert torch.equal(ids, ids_g)
