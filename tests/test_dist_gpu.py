"""GPU (needs >= 2 devices, skipped otherwise): the head-parallel prefill and batch-parallel decode
harness over NCCL against the single-GPU result."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import PKG_ROOT, ROOT

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, result_dir):
    import sys
    for p in (ROOT, PKG_ROOT):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from minfer.dist import DecodeShards, decode_batch_parallel, head_shard, prefill_head_parallel
        from minfer.kernels.torch_ext.ops import prefill_cta_limit
        from minfer.kernels import KernelBackend
        kerns = KernelBackend("torch_ext")
        g = torch.Generator().manual_seed(9)
        B, H, Hkv, L, D = 2, 16, 4, 512, 128
        q = torch.randn(B, H, L, D, generator=g).half().cuda()
        k = torch.randn(B, Hkv, L, D, generator=g).half().cuda()
        v = torch.randn(B, Hkv, L, D, generator=g).half().cuda()
        single = torch.empty_like(q)
        kerns.flash_attn_causal(q, k, v, single)
        for blocks in (1, 2):
            full = prefill_head_parallel(kerns.flash_attn_causal, q, k, v, blocks=blocks)
            torch.cuda.synchronize()
            assert torch.equal(full, single), f"head-parallel prefill differs from the single-GPU result (blocks={blocks})"
        # B = 1, this rank's slices only, a caller-owned output buffer, the exchange overlapped with the
        # attention of the next block while the attention leaves 8 SMs to the exchange
        qs, kvs = head_shard(H, Hkv, world, rank)
        buf = torch.full((1, H, L, D), float("nan"), dtype=torch.float16, device="cuda")
        with prefill_cta_limit(140):
            prefill_head_parallel(kerns.flash_attn_causal, q[:1, qs].contiguous(), k[:1, kvs].contiguous(),
                                  v[:1, kvs].contiguous(), out=buf, blocks=2, inputs_are_shards=True)
        torch.cuda.synchronize()
        assert torch.equal(buf, single[:1]), "B=1 shard inputs"
        buf.fill_(float("nan"))
        prefill_head_parallel(kerns.flash_attn_causal, q[:1], k[:1], v[:1], out=buf)
        torch.cuda.synchronize()
        assert torch.equal(buf, single[:1]), "B=1 in-place all-gather"

        # the exchange fused into the kernel: every rank's output tensor is shared through CUDA IPC and the
        # attention kernel stores its tiles into all of them; twice in a row on the same buffers
        from minfer.dist import PeerOutputs, prefill_head_parallel_fused
        for Bf in (1, 2):
            outs = PeerOutputs((Bf, H, L, D), torch.float16, torch.device("cuda", rank))
            for _ in range(2):
                outs.local.fill_(float("nan"))
                torch.cuda.synchronize()
                dist.barrier()
                res = prefill_head_parallel_fused(q[:Bf], k[:Bf], v[:Bf], outs)
                torch.cuda.synchronize()
                assert torch.equal(res, single[:Bf]), f"fused head-parallel prefill differs (B={Bf})"
            outs.close()
            del outs

        Bd, Lmax = 8, 1500
        qd = torch.randn(Bd, H, 1, D, generator=g).half().cuda()
        kc = torch.randn(Bd, Hkv, Lmax, D, generator=g).half().cuda()
        vc = torch.randn(Bd, Hkv, Lmax, D, generator=g).half().cuda()
        lens = torch.tensor([1500, 3, 700, 1025, 64, 512, 513, 999], dtype=torch.int32).cuda()
        shards = DecodeShards(lens.tolist(), world)
        mine = torch.tensor(shards.mine(rank), device="cuda")
        outd = decode_batch_parallel(kerns.flash_attn_decode, qd[mine], kc[mine], vc[mine], lens[mine].contiguous(), shards)
        single_d = torch.empty_like(qd)
        kerns.flash_attn_decode(qd, kc, vc, lens, single_d)
        torch.cuda.synchronize()
        assert torch.equal(outd, single_d), "batch-parallel decode differs from the single-GPU result"
        open(os.path.join(result_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_rank_nccl_harness(tmp_path):
    world = 2
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert sorted(os.listdir(tmp_path)) == ["ok0", "ok1"]
