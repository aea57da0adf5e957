"""CPU: the Q8_0 restatement against the reference's own codec — golden bytes always, and the compiled
reference (oracle/_ref) wherever that build is present."""
import numpy as np
import pytest
import torch

from _util import GOLDEN, from_bits16
from oracle import oracle as O


def test_restatement_matches_reference_bytes():
    z = np.load(f"{GOLDEN}/q8_0_rows.npz")
    x = from_bits16(z["x"], False)
    want_q = torch.from_numpy(z["q"])
    got_q = O.q8_0_quantize(x)
    assert torch.equal(got_q, want_q)
    assert torch.equal(O.q8_0_dequantize(want_q, torch.float16), from_bits16(z["deq16"], False))
    # a zero block quantises to d = 0, q = 0 and dequantises to zeros
    assert int(got_q[3, :34].sum()) == 0
    # quantisation error: half a step, plus up to 127 steps times the fp16 rounding of the stored scale
    deq = O.q8_0_dequantize(got_q, torch.float32).reshape(24, 4, 32)
    d = x.float().reshape(24, 4, 32).abs().amax(-1, keepdim=True) / 127
    finite = torch.isfinite(deq)  # the 60000 outlier's block keeps a finite scale; guard anyway
    assert ((deq - x.float().reshape(24, 4, 32)).abs()[finite] <= (0.57 * d.expand_as(deq))[finite] + 1e-30).all()


@pytest.mark.skipif(not O.reference_build_available(), reason="oracle/_ref not built (needs the reference tree)")
def test_restatement_matches_compiled_reference():
    g = torch.Generator().manual_seed(99)
    x = torch.randn(64, 256, generator=g) * torch.logspace(-4, 3, 64)[:, None]
    q = O.q8_0_quantize(x)
    assert torch.equal(q, O.q8_0_quantize_ref(x))
    assert torch.equal(O.q8_0_dequantize(q, torch.float16), O.q8_0_dequantize_ref(q, torch.float16))
    assert torch.equal(O.q8_0_dequantize(q, torch.float32), O.q8_0_dequantize_ref(q, torch.float32))
