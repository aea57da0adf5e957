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


def test_conversion_free_dequantisation_is_exact():
    """The decode kernel turns an int8 q and its block scale d into (16-bit type)(q * d) without a conversion
    instruction.  float16: the byte q ^ 0x80 becomes the mantissa of the half 1024.0 (bits 0x6400 | byte = 1152 + q),
    1152 is subtracted and one half multiply by d rounds once.  bfloat16: the same in fp32 (0x4B000000 | byte =
    2^23 + 128 + q), the product q * d is exact there, one rounding to bfloat16.  Restated with numpy / torch for
    all 256 bytes against every finite fp16 scale of either sign: identical to the reference's dequantisation
    (csrc/quants/impl.cpp:1153-1166: (half)(q * d) with the product in fp32)."""
    q = np.arange(-128, 128, dtype=np.int32)
    byte = (q & 0xFF) ^ 0x80
    scales = np.arange(0x0000, 0x7C00, dtype=np.uint16)                      # every finite non-negative fp16
    scales = np.concatenate([scales, scales | 0x8000]).view(np.float16)
    # float16 route
    x = (0x6400 | byte).astype(np.uint16).view(np.float16)                     # 1152 + q, exactly
    qi = x - np.float16(1152.0)
    assert np.array_equal(qi.astype(np.int32), q)
    with np.errstate(over="ignore"):
        got16 = qi[None, :] * scales[:, None]                                  # one fp16 multiply (rounds once)
        want16 = (q[None, :].astype(np.float32) * scales[:, None].astype(np.float32)).astype(np.float16)
    assert np.array_equal(got16.view(np.uint16), want16.view(np.uint16))
    # bfloat16 route
    xf = (0x4B000000 | byte).astype(np.uint32).view(np.float32)               # 2^23 + 128 + q, exactly
    qf = xf - np.float32(8388736.0)
    assert np.array_equal(qf.astype(np.int32), q)
    some = scales[::37].astype(np.float32)
    prod = torch.from_numpy(qf[None, :] * some[:, None])                       # exact: 8 bits x 11 bits
    want = torch.from_numpy(q[None, :].astype(np.float32) * some[:, None])
    assert torch.equal(prod.bfloat16().view(torch.int16), want.bfloat16().view(torch.int16))
