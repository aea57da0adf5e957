"""Element-type tags the attention callers pass.

Subset of the reference's enum (src/minfer/const.py:4-36 and :39-70 of
dsuarez01/minfer-python): attention takes plain 16-bit tensors, so only the
unquantised tags exist here.  The (qblock size, qtype size) pairs are the
reference's, including its (256, 512) entry for BF16.
"""
from enum import IntEnum


class GGMLQuantizationType(IntEnum):
    F32 = 0
    F16 = 1
    BF16 = 30


GGML_QUANT_SIZES: dict[GGMLQuantizationType, tuple[int, int]] = {
    GGMLQuantizationType.F32: (1, 4),
    GGMLQuantizationType.F16: (1, 2),
    GGMLQuantizationType.BF16: (256, 512),
}
