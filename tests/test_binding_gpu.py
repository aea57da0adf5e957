"""GPU: the two bindings of the op surface - the torch extension `_C` (LibTorch stable ABI, the reference's
mechanism: csrc/reg.cpp:21-33, csrc/cuda/reg.cu:16-27) and the ctypes one - reach the same C ABI and give
the same bits; the extension's ops pass torch.library.opcheck."""
import os
import subprocess
import sys

import pytest
import torch

from conftest import PKG_ROOT, ROOT
from _util import check_close
from oracle import oracle as O

pytestmark = pytest.mark.gpu

_SCRIPT = r"""
import sys, torch
sys.path.insert(0, {pkg!r}); sys.path.insert(0, {root!r})
from minfer.kernels import KernelBackend
from minfer.kernels.torch_ext import ops
assert ops.BINDING == {binding!r}, ops.BINDING
kerns = KernelBackend("torch_ext")
g = torch.Generator().manual_seed(11)
q = torch.randn(2, 6, 300, 128, generator=g).half().cuda()
k = torch.randn(2, 2, 300, 128, generator=g).half().cuda()
v = torch.randn(2, 2, 300, 128, generator=g).half().cuda()
mask = (torch.rand(2, 1, 300, 300, generator=g) < 0.5).cuda()
lens = torch.tensor([300, 17], dtype=torch.int32).cuda()
o1, o2, o3 = torch.zeros_like(q), torch.zeros_like(q), torch.zeros(2, 6, 1, 128, dtype=torch.float16, device="cuda")
kerns.flash_attn_causal(q, k, v, o1)
kerns.flash_attn(1, 1, 2, q, k, v, mask, o2)
kerns.flash_attn_decode(q[:, :, :1].contiguous(), k, v, lens, o3)
with ops.prefill_cta_limit(7):
    o4 = torch.zeros_like(q)
    kerns.flash_attn_causal(q, k, v, o4)
ops.check_status()
torch.save([o1.cpu(), o2.cpu(), o3.cpu(), o4.cpu()], {out!r})
"""


def _run(binding, out):
    env = dict(os.environ, MINFER_ATTN_BINDING=binding)
    script = _SCRIPT.format(pkg=PKG_ROOT, root=ROOT, binding=binding, out=out)
    r = subprocess.run([sys.executable, "-c", script], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    return torch.load(out)


def test_stable_abi_extension_and_ctypes_binding_agree(tmp_path):
    from minfer.kernels.torch_ext import ops
    assert os.path.exists(os.path.join(PKG_ROOT, "minfer", "kernels", "torch_ext", "_C.abi3.so")), "the torch extension was not built"
    assert ops.BINDING == "stable", "the extension is present but the ops did not bind to it"
    a = _run("stable", str(tmp_path / "stable.pt"))
    b = _run("ctypes", str(tmp_path / "ctypes.pt"))
    for x, y in zip(a, b):
        assert torch.equal(x, y)
    assert torch.equal(a[0], a[3])
    g = torch.Generator().manual_seed(11)
    q = torch.randn(2, 6, 300, 128, generator=g).half()
    k = torch.randn(2, 2, 300, 128, generator=g).half()
    v = torch.randn(2, 2, 300, 128, generator=g).half()
    check_close(a[0], O.prefill_oracle(q, k, v, causal=True), "extension, causal")


def test_opcheck_on_the_extension_ops(kerns):
    g = torch.Generator().manual_seed(3)
    q = torch.randn(1, 4, 128, 64, generator=g).half().cuda()
    k = torch.randn(1, 2, 128, 64, generator=g).half().cuda()
    v = torch.randn(1, 2, 128, 64, generator=g).half().cuda()
    out = torch.zeros_like(q)
    lens = torch.tensor([100], dtype=torch.int32, device="cuda")
    torch.library.opcheck(torch.ops.minfer.flash_attn_decode.default, (q[:, :, :1].contiguous(), k, v, lens, out[:, :, :1].contiguous()),
                          test_utils=("test_schema", "test_faketensor"))
    pages = torch.randn(8, 2, 16, 64, generator=g).half().cuda()
    table = torch.arange(8, dtype=torch.int32, device="cuda").view(1, 8)
    torch.library.opcheck(torch.ops.minfer.flash_attn_decode_paged.default,
                          (q[:, :, :1].contiguous(), pages, pages.clone(), table, lens, out[:, :, :1].contiguous()),
                          test_utils=("test_schema", "test_faketensor"))


def test_extension_argument_errors_are_runtime_errors(kerns):
    q = torch.zeros(1, 4, 128, 128, dtype=torch.float16, device="cuda")
    k = torch.zeros(1, 2, 128, 128, dtype=torch.float16, device="cuda")
    with pytest.raises(RuntimeError):
        kerns.flash_attn_causal(q, k, k[:, :, :64], torch.zeros_like(q))          # k/v shapes differ
    with pytest.raises(RuntimeError):
        kerns.flash_attn_causal(q, k, k, torch.zeros(1, 4, 128, 64, dtype=torch.float16, device="cuda"))
    with pytest.raises(RuntimeError):
        kerns.flash_attn_decode(q[:, :, :1], k, k, torch.zeros(1, dtype=torch.int64, device="cuda"), torch.zeros_like(q[:, :, :1]))
