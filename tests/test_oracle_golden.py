"""CPU: the oracle against vectors produced by the reference's own refs.flash_attn."""
import hashlib

import numpy as np
import pytest
import torch

from _util import GOLDEN, load_decode, load_prefill
from oracle import oracle as O

PREFILL = ["prefill_causal_g4_d128", "prefill_window_g6_d128", "prefill_random_g1_d64",
           "prefill_causal_bf16_g8_d128", "prefill_causal_g4_d64"]
DECODE = ["decode_g4_d128", "decode_g1_d64_bf16", "decode_g6_d128"]


def test_config1_fp32_matches_reference_output():
    z = np.load(f"{GOLDEN}/config1_fp32.npz")
    g = torch.Generator().manual_seed(0)
    q = torch.randn(1, 8, 256, 64, generator=g)
    k = torch.randn(1, 8, 256, 64, generator=g)
    v = torch.randn(1, 8, 256, 64, generator=g)
    digest = hashlib.sha256(q.numpy().tobytes() + k.numpy().tobytes() + v.numpy().tobytes()).hexdigest()
    assert digest == str(z["inputs_sha256"]), "seeded generator draws different inputs than when the vector was made"
    want = torch.from_numpy(z["out"])
    mask = O.causal_mask(1, 256)
    got_sdpa = O.sdpa_reference(q, k, v, mask)
    got_c = O.attention_f64(q, k, v, mask=mask)
    got_causal = O.attention_f64(q, k, v, causal=True)
    assert torch.allclose(got_sdpa, want, atol=2e-6, rtol=1e-5)
    assert torch.allclose(got_c, want, atol=5e-6, rtol=1e-5)
    assert torch.equal(got_c, got_causal)


@pytest.mark.parametrize("name", PREFILL)
def test_prefill_oracles_match_reference_vectors(name):
    q, k, v, mask, want = load_prefill(name)
    got = O.prefill_oracle(q, k, v, mask=mask)
    got_c = O.attention_f64(q, k, v, mask=mask)
    assert torch.allclose(got, want, atol=2e-6, rtol=1e-5)
    assert torch.allclose(got_c, want, atol=5e-6, rtol=1e-5)


@pytest.mark.parametrize("name", DECODE)
def test_decode_oracles_match_reference_vectors(name):
    q, k, v, lens, want = load_decode(name)
    got = O.decode_oracle(q, k, v, lens)
    got_c = O.attention_f64(q, k, v, lens=lens)
    assert torch.allclose(got, want, atol=2e-6, rtol=1e-5)
    assert torch.allclose(got_c, want, atol=5e-6, rtol=1e-5)


def test_fully_masked_rows_are_zero():
    q, k, v, mask, want = load_prefill("prefill_random_g1_d64")
    assert not mask[0, 0, 7].any()
    assert torch.count_nonzero(want[:, :, 7]) == 0
    assert torch.count_nonzero(O.attention_f64(q, k, v, mask=mask)[:, :, 7]) == 0


def test_row_block_oracle_equals_full():
    q, k, v, mask, _ = load_prefill("prefill_causal_g4_d128")
    full = O.attention_f64(q, k, v, causal=True)
    part = O.attention_f64(q, k, v, causal=True, rows=(100, 140))
    assert torch.equal(full[:, :, 100:140], part)


def test_split_kv_merge_identity():
    """The (max, sum, unnormalised output) merge the decode kernel performs is exact algebra."""
    q, k, v, lens, want = load_decode("decode_g6_d128")
    b, chunk = 0, 512
    L = int(lens[b])
    qf, kf, vf = q[b].float(), k[b].float(), v[b].float()
    group = qf.shape[0] // kf.shape[0]
    scale = qf.shape[-1] ** -0.5
    for h in range(qf.shape[0]):
        kv = h // group
        s = (kf[kv, :L] @ qf[h, 0]) * scale
        parts = []
        for c0 in range(0, L, chunk):
            sc = s[c0:c0 + chunk]
            m = sc.max()
            p = torch.exp(sc - m)
            parts.append((m, p.sum(), p @ vf[kv, c0:c0 + chunk]))
        M = max(p[0] for p in parts)
        l = sum(torch.exp(m - M) * ls for m, ls, _ in parts)
        o = sum(torch.exp(m - M) * ov for m, _, ov in parts) / l
        assert torch.allclose(o, want[b, h, 0], atol=1e-5, rtol=1e-4)
