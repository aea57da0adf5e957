"""CPU: the RoPE restatement against vectors produced by the reference's own refs.il_rope / refs.neox_rope."""
import numpy as np
import pytest
import torch

from _util import GOLDEN, from_bits16
from oracle import oracle as O


@pytest.mark.parametrize("name", ["rope_d128_rot64", "rope_d64_rot64"])
@pytest.mark.parametrize("start", [0, 2048])
def test_rope_restatement_matches_reference_vectors(name, start):
    z = np.load(f"{GOLDEN}/{name}.npz")
    x = from_bits16(z["x"], False)
    rot, base = int(z["rot"]), float(z["base"])
    want_il = from_bits16(z[f"il_{start}"], False)
    want_neox = from_bits16(z[f"neox_{start}"], False)
    # the restatement evaluates cos/sin separately instead of through complex polar form:
    # identical up to the last fp16 bit
    assert torch.allclose(O.il_rope_reference(x, rot, start, base).float(), want_il.float(), atol=2e-3, rtol=0)
    assert torch.allclose(O.neox_rope_reference(x, rot, start, base).float(), want_neox.float(), atol=2e-3, rtol=0)
    # elements beyond rotary_dim are untouched
    assert torch.equal(want_il[..., rot:], x[..., rot:])
