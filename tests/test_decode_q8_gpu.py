"""GPU parity tests of the Q8_0 KV-cache path: decode over quantised caches and the quantising append.

Definition under test: the Q8_0 decode equals the 16-bit decode run on the reference's fp16
dequantisation of the cache; the quantising append writes the reference's quantisation of the rows
the 16-bit cache would receive."""
import pytest
import torch

from _util import check_close
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def make_q8_cache(B, Hkv, Lmax, D, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    x = (scale * torch.randn(B, Hkv, Lmax, D, generator=g)).half()
    return O.q8_0_quantize(x)          # uint8 [B, Hkv, Lmax, D/32*34]


@pytest.mark.parametrize("D,H,Hkv,dtype", [(128, 32, 8, torch.float16), (64, 8, 2, torch.float16),
                                            (128, 12, 2, torch.bfloat16)])
def test_decode_q8_equals_decode_on_dequantised_cache(kerns, D, H, Hkv, dtype):
    B, Lmax = 7, 2100
    g = torch.Generator().manual_seed(5 + D + H)
    q = torch.randn(B, H, 1, D, generator=g).to(dtype)
    kq, vq = make_q8_cache(B, Hkv, Lmax, D, 1), make_q8_cache(B, Hkv, Lmax, D, 2)
    lens = torch.tensor([1, 15, 16, 17, 513, 1025, 2100], dtype=torch.int32)
    # poison everything beyond lens: must never be read or used
    for b in range(B):
        kq[b, :, int(lens[b]):] = 0xFF
        vq[b, :, int(lens[b]):] = 0x7C   # fp16 scale bytes 0x7C7C = +inf-ish garbage
    out = torch.full((B, H, 1, D), float("nan"), dtype=dtype, device="cuda")
    kerns.flash_attn_decode_q8(q.cuda(), kq.cuda(), vq.cuda(), lens.cuda(), out)
    torch.cuda.synchronize()
    kd, vd = O.q8_0_dequantize(kq, dtype), O.q8_0_dequantize(vq, dtype)
    for b in range(B):                   # keep the poison out of the comparison inputs
        kd[b, :, int(lens[b]):] = 0
        vd[b, :, int(lens[b]):] = 0
    ref16 = torch.full((B, H, 1, D), float("nan"), dtype=dtype, device="cuda")
    kerns.flash_attn_decode(q.cuda(), kd.cuda(), vd.cuda(), lens.cuda(), ref16)
    torch.cuda.synchronize()
    assert torch.equal(out, ref16), "Q8_0 decode must equal the 16-bit decode on the dequantised cache"
    check_close(out, O.decode_oracle(q, kd, vd, lens), "q8 decode vs oracle", bf16=dtype == torch.bfloat16)


def test_decode_q8_config3_shape(kerns):
    """Batch 64, 32/8 heads, D=128, lengths uniform in [512, 8192], cache padded to 8192."""
    B, H, Hkv, Lmax, D = 64, 32, 8, 8192, 128
    g = torch.Generator().manual_seed(2)
    lens = torch.randint(512, 8193, (B,), generator=g, dtype=torch.int32)
    q = torch.randn(B, H, 1, D, generator=g).half()
    kq = torch.randint(0, 256, (B, Hkv, Lmax, 136), dtype=torch.uint8, device="cuda")
    vq = torch.randint(0, 256, (B, Hkv, Lmax, 136), dtype=torch.uint8, device="cuda")
    # random bytes are fine for q; make the scales sane fp16 values (0.01 .. 0.02)
    for c in (kq, vq):
        blocks = c.view(B, Hkv, Lmax, 4, 34)
        blocks[..., 0] = torch.randint(0, 256, blocks[..., 0].shape, dtype=torch.uint8, device="cuda")
        blocks[..., 1] = 0x21
    out = torch.full((B, H, 1, D), float("nan"), dtype=torch.float16, device="cuda")
    kerns.flash_attn_decode_q8(q.cuda(), kq, vq, lens.cuda(), out)
    torch.cuda.synchronize()
    for b0 in (0, 48):
        kd = O.q8_0_dequantize(kq[b0:b0 + 16].cpu(), torch.float16)
        vd = O.q8_0_dequantize(vq[b0:b0 + 16].cpu(), torch.float16)
        check_close(out[b0:b0 + 16], O.decode_oracle(q[b0:b0 + 16], kd, vd, lens[b0:b0 + 16]), f"q8 config3 b={b0}")


@pytest.mark.parametrize("style", [0, 1])
def test_quantising_append(kerns, style):
    B, L, Hq, Hkv, D, Lmax, rot, base = 3, 21, 8, 2, 128, 64, 128, 500000.0
    g = torch.Generator().manual_seed(13)
    q = torch.randn(B, L, Hq, D, generator=g).half()
    k = torch.randn(B, L, Hkv, D, generator=g).half()
    v = torch.randn(B, L, Hkv, D, generator=g).half()
    start = torch.tensor([0, 30, 43], dtype=torch.int32)
    kc = torch.full((B, Hkv, Lmax, 136), 0xAB, dtype=torch.uint8)
    vc = torch.full((B, Hkv, Lmax, 136), 0xAB, dtype=torch.uint8)
    rope = O.il_rope_reference if style == 0 else O.neox_rope_reference
    qd, kcd, vcd = q.cuda(), kc.cuda(), vc.cuda()
    kerns.rope_kv_append_q8(rot, base, style, qd, k.cuda(), v.cuda(), kcd, vcd, start.cuda())
    torch.cuda.synchronize()
    want_q = torch.stack([rope(q[b:b + 1], rot, int(start[b]), base)[0] for b in range(B)])
    assert torch.allclose(qd.cpu().float(), want_q.float(), atol=5e-3, rtol=0)
    for b in range(B):
        s0 = int(start[b])
        # v: exactly the reference quantisation of the rows
        want_v = O.q8_0_quantize(v[b].transpose(0, 1))                 # [Hkv, L, 136]
        assert torch.equal(vcd[b, :, s0:s0 + L].cpu(), want_v)
        # k: rotation first (last-ulp differences of sin/cos may move a rounded int8 by one step)
        kr = rope(k[b:b + 1], rot, s0, base)[0].transpose(0, 1)         # [Hkv, L, D] fp16
        got = O.q8_0_dequantize(kcd[b, :, s0:s0 + L].cpu(), torch.float32)
        step = kr.float().reshape(Hkv, L, 4, 32).abs().amax(-1, keepdim=True) / 127
        err = (got.reshape(Hkv, L, 4, 32) - kr.float().reshape(Hkv, L, 4, 32)).abs()
        assert (err <= 1.6 * step + 5e-3).all()
        # rows outside [start, start + L) keep their fill
        untouched = torch.ones(Lmax, dtype=torch.bool)
        untouched[s0:s0 + L] = False
        assert (kcd[b, :, untouched].cpu() == 0xAB).all() and (vcd[b, :, untouched].cpu() == 0xAB).all()


def test_append_then_decode_q8(kerns):
    """A decode step on the Q8_0 cache: append the new token, attend over lens + 1 keys."""
    B, Hq, Hkv, D, Lmax, base = 4, 8, 2, 128, 300, 500000.0
    kq, vq = make_q8_cache(B, Hkv, Lmax, D, 21), make_q8_cache(B, Hkv, Lmax, D, 22)
    g = torch.Generator().manual_seed(14)
    lens = torch.tensor([0, 5, 128, 299], dtype=torch.int32)
    q = torch.randn(B, 1, Hq, D, generator=g).half()
    k = torch.randn(B, 1, Hkv, D, generator=g).half()
    v = torch.randn(B, 1, Hkv, D, generator=g).half()
    qd, kqd, vqd = q.cuda(), kq.cuda(), vq.cuda()
    kerns.rope_kv_append_q8(D, base, 0, qd, k.cuda(), v.cuda(), kqd, vqd, lens.cuda())
    out = torch.zeros(B, Hq, 1, D, dtype=torch.float16, device="cuda")
    new_lens = (lens + 1).cuda()
    kerns.flash_attn_decode_q8(qd.transpose(1, 2), kqd, vqd, new_lens, out)
    torch.cuda.synchronize()
    kd, vd = O.q8_0_dequantize(kqd.cpu(), torch.float16), O.q8_0_dequantize(vqd.cpu(), torch.float16)
    check_close(out, O.decode_oracle(qd.transpose(1, 2).cpu(), kd, vd, new_lens.cpu()), "append + decode q8")


def test_q8_argument_errors(kerns):
    q = torch.zeros(2, 8, 1, 128, dtype=torch.float16, device="cuda")
    lens = torch.tensor([5, 6], dtype=torch.int32, device="cuda")
    ok = torch.zeros(2, 2, 64, 136, dtype=torch.uint8, device="cuda")
    with pytest.raises(RuntimeError):
        kerns.flash_attn_decode_q8(q, ok[..., :128], ok[..., :128], lens, torch.zeros_like(q))   # wrong row bytes
    with pytest.raises(RuntimeError):
        kerns.flash_attn_decode_q8(q, ok[:, :, :63], ok[:, :, :63], lens, torch.zeros_like(q))   # odd padded length
    with pytest.raises(RuntimeError):
        kerns.flash_attn_decode_q8(q, ok.half(), ok.half(), lens, torch.zeros_like(q))           # not uint8
    # head_dim 64: rows are 68 bytes, so the padded length must be a multiple of 4 (62 is even but is refused)
    q64 = torch.zeros(2, 8, 1, 64, dtype=torch.float16, device="cuda")
    c64 = torch.zeros(2, 2, 64, 68, dtype=torch.uint8, device="cuda")
    kerns.flash_attn_decode_q8(q64, c64, c64, lens, torch.zeros_like(q64))
    with pytest.raises(RuntimeError):
        kerns.flash_attn_decode_q8(q64, c64[:, :, :62].contiguous(), c64[:, :, :62].contiguous(), lens, torch.zeros_like(q64))


@pytest.mark.parametrize("D,Lmax", [(64, 60), (64, 36), (128, 34)])
def test_q8_full_length_sequences_at_the_end_of_the_allocation(kerns, D, Lmax):
    """lens == max_len for every sequence, caches sized exactly: the last 16-byte copy of the last tile ends
    where the allocation ends (the copies move whole 16-byte chunks of 68- or 136-byte rows)."""
    B, H, Hkv = 2, 4, 2
    g = torch.Generator().manual_seed(D + Lmax)
    q = torch.randn(B, H, 1, D, generator=g).half()
    kq, vq = make_q8_cache(B, Hkv, Lmax, D, 31), make_q8_cache(B, Hkv, Lmax, D, 32)
    lens = torch.full((B,), Lmax, dtype=torch.int32)
    out = torch.full((B, H, 1, D), float("nan"), dtype=torch.float16, device="cuda")
    kerns.flash_attn_decode_q8(q.cuda(), kq.cuda(), vq.cuda(), lens.cuda(), out)
    torch.cuda.synchronize()
    kd, vd = O.q8_0_dequantize(kq, torch.float16), O.q8_0_dequantize(vq, torch.float16)
    check_close(out, O.decode_oracle(q, kd, vd, lens), f"q8 full length D={D}")


@pytest.mark.parametrize("seed", range(8))
def test_decode_q8_random_shapes_equal_the_16bit_decode(kerns, seed):
    """Random GQA groups (1, 2, 3, 4, 6, 8), both head sizes and dtypes, ragged lengths from 1 key up, scales
    spread over orders of magnitude: the Q8_0 decode must produce the bits of the 16-bit decode on the
    dequantised cache (the fragments are built from the raw blocks, K in the order of the 16-bit path)."""
    g = torch.Generator().manual_seed(100 + seed)
    D = (64, 128)[seed % 2]
    dtype = (torch.float16, torch.bfloat16)[(seed // 2) % 2]
    group = (1, 2, 3, 4, 6, 8, 4, 2)[seed]
    Hkv = int(torch.randint(1, 4, (1,), generator=g))
    H = Hkv * group
    B = int(torch.randint(1, 6, (1,), generator=g))
    Lmax = 4 * int(torch.randint(8, 700, (1,), generator=g))
    lens = torch.randint(1, Lmax + 1, (B,), generator=g, dtype=torch.int32)
    lens[0] = 1
    q = torch.randn(B, H, 1, D, generator=g).to(dtype)
    # per-row magnitudes from 1e-3 to 1e+2: block scales then cover five orders of magnitude
    mag = 10.0 ** (5 * torch.rand(B, Hkv, Lmax, 1, generator=g) - 3)
    kq = O.q8_0_quantize((mag * torch.randn(B, Hkv, Lmax, D, generator=g)).half())
    vq = O.q8_0_quantize((mag * torch.randn(B, Hkv, Lmax, D, generator=g)).half())
    out = torch.full((B, H, 1, D), float("nan"), dtype=dtype, device="cuda")
    kerns.flash_attn_decode_q8(q.cuda(), kq.cuda(), vq.cuda(), lens.cuda(), out)
    kd, vd = O.q8_0_dequantize(kq, dtype), O.q8_0_dequantize(vq, dtype)
    ref16 = torch.full((B, H, 1, D), float("nan"), dtype=dtype, device="cuda")
    kerns.flash_attn_decode(q.cuda(), kd.cuda(), vd.cuda(), lens.cuda(), ref16)
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all()
    assert torch.equal(out, ref16), f"seed {seed}: D={D} {dtype} group={group} B={B} Lmax={Lmax}"
