"""GPU parity tests of RoPE and the fused RoPE + KV-cache append.

Tolerance: atol 5e-3, the reference's own for this op (test/kernels.py:76-96, "adjusted for large
angle vals"): positions reach several thousand radians in fp32, where one ulp of the angle is
already ~5e-4."""
import numpy as np
import pytest
import torch

from _util import GOLDEN, from_bits16
from oracle import oracle as O

pytestmark = pytest.mark.gpu
ROPE_ATOL = 5e-3


@pytest.mark.parametrize("name", ["rope_d128_rot64", "rope_d64_rot64"])
@pytest.mark.parametrize("start", [0, 2048])
def test_golden_vectors_in_place(kerns, name, start):
    z = np.load(f"{GOLDEN}/{name}.npz")
    x = from_bits16(z["x"], False)
    rot, base = int(z["rot"]), float(z["base"])
    for style, fn in (("il", kerns.il_rope), ("neox", kerns.neox_rope)):
        want = from_bits16(z[f"{style}_{start}"], False)
        got = x.clone().cuda()
        fn(rot, start, base, got)
        torch.cuda.synchronize()
        assert torch.allclose(got.cpu().float(), want.float(), atol=ROPE_ATOL, rtol=0), style
        assert torch.equal(got.cpu()[..., rot:], x[..., rot:])


@pytest.mark.parametrize("rope_type", ["il", "neox"])
@pytest.mark.parametrize("start_pos", [0, 2048])
def test_reference_test_rope_shapes(kerns, rope_type, start_pos):
    """The reference's test_rope (test/kernels.py:76-96): B=8 L=4096 48 heads D=128 rot=64 base 1e6."""
    B, L, H, D, rot, base = 8, 4096, 48, 128, 64, 1e6
    g = torch.Generator().manual_seed(3)
    x = torch.randn(B, L, H, D, generator=g).half()
    actual = x.clone().cuda()
    (kerns.il_rope if rope_type == "il" else kerns.neox_rope)(rot, start_pos, base, actual)
    torch.cuda.synchronize()
    for b in (0, 7):  # the oracle on two batch elements keeps the CPU side short
        ref = (O.il_rope_reference if rope_type == "il" else O.neox_rope_reference)(x[b:b + 1], rot, start_pos, base)
        assert torch.allclose(ref.float(), actual[b:b + 1].cpu().float(), atol=ROPE_ATOL, rtol=0)


@pytest.mark.parametrize("style", [0, 1])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_fused_append_equals_rotate_then_write(kerns, style, dtype):
    """rope_kv_append == (rotate q, rotate k, scatter k and v into the cache rows start[b] + l)."""
    B, L, Hq, Hkv, D, Lmax, rot, base = 3, 37, 8, 2, 128, 200, 128, 500000.0
    g = torch.Generator().manual_seed(11)
    q = torch.randn(B, L, Hq, D, generator=g).to(dtype)
    k = torch.randn(B, L, Hkv, D, generator=g).to(dtype)
    v = torch.randn(B, L, Hkv, D, generator=g).to(dtype)
    start = torch.tensor([0, 100, 163], dtype=torch.int32)
    kc = torch.full((B, Hkv, Lmax, D), 7.0, dtype=dtype)
    vc = torch.full((B, Hkv, Lmax, D), 7.0, dtype=dtype)
    rope = O.il_rope_reference if style == 0 else O.neox_rope_reference
    want_q = torch.stack([rope(q[b:b + 1], rot, int(start[b]), base)[0] for b in range(B)])
    want_kc, want_vc = kc.clone(), vc.clone()
    for b in range(B):
        kr = rope(k[b:b + 1], rot, int(start[b]), base)[0]            # [L, Hkv, D]
        want_kc[b, :, int(start[b]):int(start[b]) + L] = kr.transpose(0, 1)
        want_vc[b, :, int(start[b]):int(start[b]) + L] = v[b].transpose(0, 1)
    qd, kcd, vcd = q.cuda(), kc.cuda(), vc.cuda()
    kerns.rope_kv_append(rot, base, style, qd, k.cuda(), v.cuda(), kcd, vcd, start.cuda())
    torch.cuda.synchronize()
    tol = ROPE_ATOL if dtype == torch.float16 else 4e-2  # bfloat16 output: half an ulp at |x| ~ 4 is 1.6e-2
    assert torch.allclose(qd.cpu().float(), want_q.float(), atol=tol, rtol=0)
    assert torch.allclose(kcd.cpu().float(), want_kc.float(), atol=tol, rtol=0)
    assert torch.equal(vcd.cpu(), want_vc)                           # v is a plain copy; untouched rows keep their fill


def test_decode_step_append_then_attend(kerns):
    """One decode step end to end on the ops: append the new token's k/v at row lens[b], then attend over
    lens[b] + 1 keys; compared with the oracle on the same cache."""
    B, Hq, Hkv, D, Lmax, base = 4, 8, 2, 128, 300, 500000.0
    g = torch.Generator().manual_seed(12)
    kc = torch.randn(B, Hkv, Lmax, D, generator=g).half()
    vc = torch.randn(B, Hkv, Lmax, D, generator=g).half()
    lens = torch.tensor([0, 5, 128, 299], dtype=torch.int32)
    q = torch.randn(B, 1, Hq, D, generator=g).half()
    k = torch.randn(B, 1, Hkv, D, generator=g).half()
    v = torch.randn(B, 1, Hkv, D, generator=g).half()
    qd, kcd, vcd = q.cuda(), kc.cuda(), vc.cuda()
    kerns.rope_kv_append(D, base, 1, qd, k.cuda(), v.cuda(), kcd, vcd, lens.cuda())
    out = torch.zeros(B, Hq, 1, D, dtype=torch.float16, device="cuda")
    new_lens = (lens + 1).cuda()
    kerns.flash_attn_decode(qd.transpose(1, 2), kcd, vcd, new_lens, out)
    torch.cuda.synchronize()
    want = O.decode_oracle(qd.transpose(1, 2).cpu(), kcd.cpu(), vcd.cpu(), new_lens.cpu())
    ok, err, bad = O.within_tolerance(out, want)
    assert ok, (err, bad)


def test_rope_argument_errors(kerns):
    x = torch.zeros(1, 4, 2, 128, dtype=torch.float16, device="cuda")
    with pytest.raises(RuntimeError):
        kerns.il_rope(256, 0, 1e4, x)                                  # rotary_dim > head_dim
    with pytest.raises(RuntimeError):
        kerns.il_rope(64, 0, 1e4, x.transpose(1, 2))                   # not contiguous
    with pytest.raises(RuntimeError):
        kerns.neox_rope(24, 0, 1e4, x)                                 # neox needs a multiple of 16
    with pytest.raises(RuntimeError):
        kerns.il_rope(64, 0, 1e4, x.float())                           # dtype


def test_out_of_range_start_is_dropped_and_reported(kerns):
    """start[b] + l outside [0, max_len): the row is not written anywhere (the neighbouring cache rows and
    the other sequences keep their content), q is still rotated, and the status word names the sequence."""
    from minfer.kernels.torch_ext.ops import check_status
    B, L, H, Hkv, D, Lmax = 3, 2, 4, 2, 64, 32
    g = torch.Generator().manual_seed(8)
    q = torch.randn(B, L, H, D, generator=g).half().cuda()
    k = torch.randn(B, L, Hkv, D, generator=g).half().cuda()
    v = torch.randn(B, L, Hkv, D, generator=g).half().cuda()
    kc = torch.full((B, Hkv, Lmax, D), 7.0, dtype=torch.float16, device="cuda")
    vc = torch.full((B, Hkv, Lmax, D), 7.0, dtype=torch.float16, device="cuda")
    start = torch.tensor([3, Lmax - 1, -1], dtype=torch.int32, device="cuda")   # seq 1: second token overflows; seq 2: first is negative
    check_status()
    kerns.rope_kv_append(D, 10000.0, 0, q, k, v, kc, vc, start)
    with pytest.raises(RuntimeError, match="cache position out of range"):
        check_status()
    untouched = torch.ones(B, Lmax, dtype=torch.bool)
    untouched[0, 3:5] = False
    untouched[1, Lmax - 1] = False
    untouched[2, 0] = False
    wrote = (kc != 7.0).any(-1).any(1).cpu()           # [B, Lmax]
    assert torch.equal(wrote, ~untouched)
    assert torch.equal((vc != 7.0).any(-1).any(1).cpu(), ~untouched)
