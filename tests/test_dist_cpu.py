"""CPU: the multi-GPU harness (partition maps, gather layout) on two gloo ranks, with the oracle
standing in for the CUDA ops."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import PKG_ROOT, ROOT


def test_head_shard_map():
    from minfer.dist import head_shard
    assert head_shard(64, 8, 8, 3) == (slice(24, 32), slice(3, 4))
    assert head_shard(32, 8, 2, 1) == (slice(16, 32), slice(4, 8))
    assert head_shard(48, 8, 1, 0) == (slice(0, 48), slice(0, 8))
    with pytest.raises(ValueError):
        head_shard(32, 8, 3, 0)


def test_balanced_batch_shards():
    from minfer.dist import balanced_batch_shards
    g = torch.Generator().manual_seed(2)
    lens = torch.randint(512, 8193, (64,), generator=g).tolist()
    for world in (1, 2, 4, 8):
        shards = balanced_batch_shards(lens, world)
        assert sorted(i for s in shards for i in s) == list(range(64))
        assert all(len(s) == 64 // world for s in shards)
        loads = [sum(lens[i] for i in s) for s in shards]
        assert max(loads) - min(loads) <= max(lens)            # snake dealing keeps the loads within one sequence
    with pytest.raises(ValueError):
        balanced_batch_shards([1, 2, 3], 2)


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
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from minfer.dist import balanced_batch_shards, decode_batch_parallel, prefill_head_parallel
        from oracle import oracle as O
        torch.set_num_threads(2)

        def prefill_fn(q, k, v, out):
            out.copy_(O.attention_f64(q, k, v, causal=True))

        def decode_fn(q, kc, vc, lens, out):
            out.copy_(O.attention_f64(q, kc, vc, lens=lens))

        g = torch.Generator().manual_seed(5)
        B, H, Hkv, L, D = 2, 8, 4, 48, 16
        q = torch.randn(B, H, L, D, generator=g)
        k = torch.randn(B, Hkv, L, D, generator=g)
        v = torch.randn(B, Hkv, L, D, generator=g)
        full = prefill_head_parallel(prefill_fn, q, k, v)
        want = O.attention_f64(q, k, v, causal=True)
        assert torch.equal(full, want), "prefill gather layout"

        Bd, Lmax = 6, 40
        qd = torch.randn(Bd, H, 1, D, generator=g)
        kc = torch.randn(Bd, Hkv, Lmax, D, generator=g)
        vc = torch.randn(Bd, Hkv, Lmax, D, generator=g)
        lens = torch.tensor([40, 3, 17, 25, 1, 33], dtype=torch.int32)
        shards = balanced_batch_shards(lens.tolist(), world)
        outd = decode_batch_parallel(decode_fn, qd, kc, vc, lens, shards)
        assert torch.equal(outd, O.attention_f64(qd, kc, vc, lens=lens)), "decode gather order"
        open(os.path.join(result_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_harness(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert sorted(os.listdir(tmp_path)) == ["ok0", "ok1"]
