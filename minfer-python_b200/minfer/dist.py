"""Multi-GPU harness of the attention path: partition maps and the one collective.

Attention shards into independent units — a kv-head group for prefill, a sequence for
decode — so no reduction ever crosses ranks; the only exchange is an all-gather of the
outputs.  The reference has no distributed code at all (its Params merely store
world_size / rank / dp_size, src/minfer/utils.py:198-214 of dsuarez01/minfer-python);
this module is the design for the path the benchmark configuration asks for: prefill
partitioned by kv-head group, decode by batch, NCCL only for the final output gather.

One process per GPU (torchrun); the process group is the caller's.  Everything here is
plain index arithmetic plus torch.distributed calls, so it runs unchanged on CPU ranks
with the gloo backend, where the tests drive it with a stand-in attention function.
"""
from __future__ import annotations

from typing import Callable, List, Sequence, Tuple

import torch
import torch.distributed as dist


def head_shard(n_heads: int, n_kv_heads: int, world: int, rank: int) -> Tuple[slice, slice]:
    """Query-head and kv-head slices owned by `rank` when kv-head groups are dealt out in order."""
    if n_kv_heads % world != 0:
        raise ValueError(f"n_kv_heads={n_kv_heads} is not divisible by world size {world}")
    if n_heads % n_kv_heads != 0:
        raise ValueError("n_heads must be a multiple of n_kv_heads")
    group = n_heads // n_kv_heads
    per = n_kv_heads // world
    kv = slice(rank * per, (rank + 1) * per)
    return slice(kv.start * group, kv.stop * group), kv


def balanced_batch_shards(lens: Sequence[int], world: int) -> List[List[int]]:
    """Deal sequences to ranks, equal counts per rank, total cache length balanced: sort by
    length (descending) and deal in a snake (0..w-1, w-1..0, ...).  Returns the sequence indices
    of every rank."""
    n = len(lens)
    if n % world != 0:
        raise ValueError(f"batch {n} is not divisible by world size {world}")
    order = sorted(range(n), key=lambda i: (-int(lens[i]), i))
    shards: List[List[int]] = [[] for _ in range(world)]
    for pos, idx in enumerate(order):
        rnd, k = divmod(pos, world)
        shards[k if rnd % 2 == 0 else world - 1 - k].append(idx)
    return shards


def prefill_head_parallel(attn_fn: Callable, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                          group=None) -> torch.Tensor:
    """Causal prefill with the heads partitioned by kv-head group.

    q [B,H,L,D], k/v [B,Hkv,L,D] are the FULL tensors (replicated or not — only this rank's
    head slices are read).  attn_fn(q_shard, k_shard, v_shard, out_shard) computes attention in
    place (the CUDA op, or a stand-in).  Returns the full [B,H,L,D] output on every rank.
    """
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    B, H, L, D = q.shape
    qs, kvs = head_shard(H, k.shape[1], world, rank)
    hp = H // world
    # gather buffer [world, B, H/world, L, D]: each rank's shard is one contiguous block
    gathered = torch.empty((world, B, hp, L, D), dtype=q.dtype, device=q.device)
    attn_fn(q[:, qs], k[:, kvs], v[:, kvs], gathered[rank])
    if world > 1:
        dist.all_gather_into_tensor(gathered.view(-1), gathered[rank].reshape(-1).clone(), group=group)
    # [world, B, hp, L, D] -> [B, world*hp, L, D]
    return gathered.permute(1, 0, 2, 3, 4).reshape(B, H, L, D)


def decode_batch_parallel(attn_fn: Callable, q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                          lens: torch.Tensor, shards: List[List[int]], group=None) -> torch.Tensor:
    """Decode with the batch partitioned over ranks (`shards` from balanced_batch_shards).

    q [B,H,1,D], caches [B,Hkv,Lmax,D], lens [B]: the full batch; this rank touches only its own
    sequences.  attn_fn(q_s, k_s, v_s, lens_s, out_s) is the decode op or a stand-in.  Returns the
    full [B,H,1,D] output, in the original batch order, on every rank.
    """
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    B, H, _, D = q.shape
    per = B // world
    mine = torch.tensor(shards[rank], dtype=torch.long, device=q.device)
    out_local = torch.empty((per, H, 1, D), dtype=q.dtype, device=q.device)
    attn_fn(q.index_select(0, mine), k_cache.index_select(0, mine), v_cache.index_select(0, mine),
            lens.index_select(0, mine).contiguous(), out_local)
    gathered = torch.empty((world, per, H, 1, D), dtype=q.dtype, device=q.device)
    if world > 1:
        dist.all_gather_into_tensor(gathered.view(-1), out_local.view(-1), group=group)
    else:
        gathered[0] = out_local
    order = torch.tensor([i for s in shards for i in s], dtype=torch.long, device=q.device)
    out = torch.empty((B, H, 1, D), dtype=q.dtype, device=q.device)
    out.index_copy_(0, order, gathered.view(B, H, 1, D))
    return out
