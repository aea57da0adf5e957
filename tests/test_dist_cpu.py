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


def test_head_blocks():
    from minfer.dist import head_blocks
    # several kv heads per rank: blocks of whole kv-head groups
    assert head_blocks(4, 8, 2) == [(slice(0, 16), slice(0, 2)), (slice(16, 32), slice(2, 4))]
    assert head_blocks(4, 4, 8) == [(slice(4 * i, 4 * i + 4), slice(i, i + 1)) for i in range(4)]
    # one kv head per rank: its query heads in pairs
    assert head_blocks(1, 8, 4) == [(slice(2 * i, 2 * i + 2), slice(0, 1)) for i in range(4)]
    assert head_blocks(1, 8, 3) == [(slice(0, 2), slice(0, 1)), (slice(2, 6), slice(0, 1)), (slice(6, 8), slice(0, 1))]
    assert head_blocks(1, 3, 2) == [(slice(0, 2), slice(0, 1)), (slice(2, 3), slice(0, 1))]
    assert head_blocks(1, 4, 1) == [(slice(0, 4), slice(0, 1))]
    for n_kv, grp, blocks in ((4, 8, 3), (1, 6, 2), (2, 4, 5), (1, 1, 4)):
        parts = head_blocks(n_kv, grp, blocks)
        assert parts[0][0].start == 0 and parts[-1][0].stop == n_kv * grp
        assert all(a[0].stop == b[0].start for a, b in zip(parts[:-1], parts[1:]))


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
        from minfer.dist import DecodeShards, decode_batch_parallel, prefill_head_parallel
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
        want = O.attention_f64(q, k, v, causal=True)
        for blocks in (1, 2):
            full = prefill_head_parallel(prefill_fn, q, k, v, blocks=blocks)
            assert torch.equal(full, want), f"prefill gather layout, blocks={blocks}"
        # B = 1 (every shard one contiguous block of the output), shard inputs, caller's output buffer
        from minfer.dist import head_shard
        qs, kvs = head_shard(H, Hkv, world, rank)
        buf = torch.full((1, H, L, D), float("nan"))
        got = prefill_head_parallel(prefill_fn, q[:1, qs].contiguous(), k[:1, kvs].contiguous(), v[:1, kvs].contiguous(),
                                    out=buf, inputs_are_shards=True)
        assert got is buf and torch.equal(buf, want[:1]), "B=1 in-place gather"
        # one kv head per rank: the exchange is cut into pairs of query heads
        k1, v1 = k[:, :world], v[:, :world]
        want1 = O.attention_f64(q, k1, v1, causal=True)
        assert torch.equal(prefill_head_parallel(prefill_fn, q, k1, v1, blocks=2), want1), "query-head blocks"

        Bd, Lmax = 8, 40
        qd = torch.randn(Bd, H, 1, D, generator=g)
        kc = torch.randn(Bd, Hkv, Lmax, D, generator=g)
        vc = torch.randn(Bd, Hkv, Lmax, D, generator=g)
        lens = torch.tensor([40, 3, 17, 25, 1, 33, 40, 9], dtype=torch.int32)
        shards = DecodeShards(lens.tolist(), world)
        mine = torch.tensor(shards.mine(rank))
        outd = decode_batch_parallel(decode_fn, qd[mine], kc[mine], vc[mine], lens[mine], shards)
        assert torch.equal(outd, O.attention_f64(qd, kc, vc, lens=lens)), "decode gather order"
        open(os.path.join(result_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_gloo_harness(tmp_path, world):
    """Two ranks (two kv heads each) and four ranks (one kv head each: the exchange then has three peers and the
    head blocks are cut inside the one kv head's query heads)."""
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert sorted(os.listdir(tmp_path)) == [f"ok{r}" for r in range(world)]
