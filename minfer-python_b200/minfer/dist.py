"""Multi-GPU harness of the attention path: partition maps and the one exchange.

Attention shards into independent units - a kv-head group for prefill, a sequence for
decode - so no reduction ever crosses ranks; the only exchange is a gather of the outputs.
The reference has no distributed code at all (its Params merely store world_size / rank /
dp_size, src/minfer/utils.py:198-214 of dsuarez01/minfer-python); this module is the design
for the partition the benchmark configuration asks for: prefill by kv-head group, decode by
batch, NCCL only for the final output gather.

One process per GPU (torchrun); the process group is the caller's.  Everything here is index
arithmetic plus torch.distributed calls, so it runs unchanged on CPU ranks with the gloo
backend, where the tests drive it with a stand-in attention function.

Prefill output exchange.  Every rank ends with the full [B, H, L, D] output, and every byte is
written exactly once, straight into its final place: a rank's attention call writes its heads
into a strided view of the full tensor, and the exchange delivers each peer's heads into theirs.
(A second form, prefill_head_parallel_fused, needs no exchange step at all: the attention kernel itself stores
every output tile into the other ranks' output tensors.)  The exchange is cut into head blocks: a block of a rank's heads is, per batch element, one
contiguous [heads, L, D] region of the output, so a block travels as plain point-to-point
transfers (grouped into one NCCL launch) with no staging copy on either side.  The attention of
block i+1 runs while block i travels; the two compute streams alternate, so the thread blocks
of one attention call fill the SMs as those of the previous call drain.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

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


def head_blocks(n_kv_local: int, group: int, blocks: int) -> List[Tuple[slice, slice]]:
    """Cut a rank's kv heads (and their query heads) into `blocks` consecutive blocks, as even as
    the kv-head count allows; a rank with a single kv head splits that head's query heads instead
    (in pairs, the unit the prefill kernel works in).  Returns (local q-head slice, local kv-head
    slice) per block."""
    blocks = max(1, int(blocks))
    if n_kv_local > 1:
        blocks = min(blocks, n_kv_local)
        cuts = [round(i * n_kv_local / blocks) for i in range(blocks + 1)]
        return [(slice(a * group, b * group), slice(a, b)) for a, b in zip(cuts[:-1], cuts[1:]) if b > a]
    unit = 2 if group % 2 == 0 else 1
    n_units = group // unit
    blocks = min(blocks, n_units)
    cuts = [round(i * n_units / blocks) * unit for i in range(blocks + 1)]
    return [(slice(a, b), slice(0, 1)) for a, b in zip(cuts[:-1], cuts[1:]) if b > a]


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


class _Streams:
    """Per-device side streams of the prefill pipeline (a second compute stream and a
    high-priority stream from which the exchange is enqueued), created once."""
    _cache: dict = {}

    @classmethod
    def get(cls, device: torch.device):
        key = device.index if device.index is not None else torch.cuda.current_device()
        if key not in cls._cache:
            cls._cache[key] = (torch.cuda.Stream(device), torch.cuda.Stream(device, priority=-1))
        return cls._cache[key]


def _exchange_block(out: torch.Tensor, hp: int, qsl: slice, world: int, rank: int, group, in_place_ok: bool) -> None:
    """Every rank delivers out[:, rank*hp + qsl] to all peers and receives theirs into out[:, p*hp + qsl]."""
    B = out.size(0)
    whole_shard = qsl.start == 0 and qsl.stop == hp
    if B == 1 and whole_shard:
        # the shards of all ranks tile the output in rank order: one all-gather, in place on NCCL
        flat = out.view(-1)
        n = flat.numel() // world
        mine = flat[rank * n:(rank + 1) * n]
        dist.all_gather_into_tensor(flat, mine if in_place_ok else mine.clone(), group=group)
        return
    ops = []
    for p in range(world):
        if p == rank:
            continue
        peer = dist.get_global_rank(group, p) if group is not None else p
        for b in range(B):
            ops.append(dist.P2POp(dist.isend, out[b, rank * hp + qsl.start: rank * hp + qsl.stop], peer, group))
            ops.append(dist.P2POp(dist.irecv, out[b, p * hp + qsl.start: p * hp + qsl.stop], peer, group))
    for w in dist.batch_isend_irecv(ops):
        w.wait()


class PeerOutputs:
    """A [B, H, L, D] output tensor per rank that every other rank of the node can write: the buffers are shared
    through CUDA IPC (one process per GPU), so a kernel on rank r can store its heads straight into the memory of
    all the others.  `local` is this rank's tensor; `peer_ptr(view)` gives, for a view of `local`, the addresses
    of the same view inside every other rank's tensor, in rank order."""

    def __init__(self, shape, dtype, device, group=None):
        from torch.multiprocessing.reductions import reduce_tensor
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.local = torch.zeros(shape, dtype=dtype, device=device)
        # one handle per consumer: torch's IPC bookkeeping counts one consumer per exported handle
        mine = [reduce_tensor(self.local) if r != self.rank else None for r in range(self.world)]
        handles = [None] * self.world
        dist.all_gather_object(handles, mine, group=group)
        self._peers = []          # keeps the mappings alive
        self._bases = []
        my_index = self.local.device.index
        for r in range(self.world):
            if r == self.rank:
                continue
            rebuild, args = handles[r][self.rank]
            # Open the peer's IPC handle with THIS rank's device current (argument 6 of torch's rebuild function is
            # the device the storage is opened on): the mapping then belongs to this device's context, peer access
            # to the owner is enabled by the open itself, and no context is created on any other GPU.
            args = list(args)
            args[6] = my_index
            t = rebuild(*args)
            self._peers.append(t)
            self._bases.append(t.data_ptr())
        dist.barrier(group=group)

    def close(self) -> None:
        """Drop this rank's mappings of the other ranks' tensors (every rank, before any of them frees its own)."""
        self._peers.clear()
        self._bases.clear()
        torch.cuda.synchronize(self.local.device)
        torch.cuda.ipc_collect()          # consumer side: unmap what was opened from the other ranks
        dist.barrier(group=self.group)
        torch.cuda.ipc_collect()          # producer side: every consumer has let go of this rank's tensor

    def peer_ptrs(self, view: torch.Tensor):
        off = view.data_ptr() - self.local.data_ptr()
        assert 0 <= off < self.local.numel() * self.local.element_size(), "not a view of the shared output"
        return [b + off for b in self._bases]


def prefill_head_parallel_fused(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, outputs: PeerOutputs,
                                inputs_are_shards: bool = False) -> torch.Tensor:
    """Head-parallel causal prefill with the output exchange inside the attention kernel: this rank's kv-head
    group is computed once and every output tile is stored into the local output and, over NVLink, into the
    output tensors of all other ranks (`outputs`, shared through CUDA IPC), so the transfer overlaps the math tile
    by tile and no SM is set aside for a collective.  A barrier across the ranks (the one NCCL call) ends the step:
    after it every rank holds the full [B, H, L, D] result in outputs.local.  CUDA only."""
    from .kernels.torch_ext.ops import flash_attn_causal_multi_out
    group = outputs.group
    world, rank = outputs.world, outputs.rank
    out = outputs.local
    B, H, L, D = out.shape
    Hkv = k.shape[1] * world if inputs_are_shards else k.shape[1]
    qs, kvs = head_shard(H, Hkv, world, rank)
    q_loc = q if inputs_are_shards else q[:, qs]
    k_loc = k if inputs_are_shards else k[:, kvs]
    v_loc = v if inputs_are_shards else v[:, kvs]
    mine = out[:, qs]
    flash_attn_causal_multi_out(q_loc, k_loc, v_loc, mine, outputs.peer_ptrs(mine))
    if world > 1:
        dist.barrier(group=group)
    return out


def prefill_head_parallel(attn_fn: Callable, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                          out: Optional[torch.Tensor] = None, group=None, blocks: int = 1,
                          inputs_are_shards: bool = False) -> torch.Tensor:
    """Causal prefill with the heads partitioned by kv-head group; the full output on every rank.

    q [B,H,L,D], k/v [B,Hkv,L,D]: the full tensors, of which only this rank's head slices are read,
    or (inputs_are_shards) this rank's slices [B,H/W,L,D], [B,Hkv/W,L,D] themselves.
    attn_fn(q_part, k_part, v_part, out_part) computes attention in place (the CUDA op, or a stand-in);
    out_part is a strided view of the full output.  `out`: optional contiguous [B,H,L,D] result buffer.
    blocks > 1 cuts the rank's heads into that many blocks and overlaps the exchange of one block with
    the attention of the next (CUDA tensors only; on CPU the blocks simply run in turn).
    """
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    B, Hq_in, L, D = q.shape
    H = Hq_in * world if inputs_are_shards else Hq_in
    Hkv = k.shape[1] * world if inputs_are_shards else k.shape[1]
    qs, kvs = head_shard(H, Hkv, world, rank)
    hp = H // world
    grp = H // Hkv
    if out is None:
        out = torch.empty((B, H, L, D), dtype=q.dtype, device=q.device)
    elif tuple(out.shape) != (B, H, L, D) or not out.is_contiguous():
        raise ValueError("out must be a contiguous [B, H, L, D] tensor")
    q_loc = q if inputs_are_shards else q[:, qs]
    k_loc = k if inputs_are_shards else k[:, kvs]
    v_loc = v if inputs_are_shards else v[:, kvs]
    out_loc = out[:, qs]
    parts = head_blocks(Hkv // world, grp, blocks if world > 1 else 1)
    nccl = q.is_cuda and dist.get_backend(group) == "nccl"

    if not q.is_cuda or len(parts) == 1:
        for qsl, ksl in parts:
            attn_fn(q_loc[:, qsl], k_loc[:, ksl], v_loc[:, ksl], out_loc[:, qsl])
        if world > 1:
            for qsl, _ in parts:
                _exchange_block(out, hp, qsl, world, rank, group, nccl)
        return out

    cur = torch.cuda.current_stream(q.device)
    aux, comm = _Streams.get(q.device)
    aux.wait_stream(cur)
    comm.wait_stream(cur)
    for i, (qsl, ksl) in enumerate(parts):
        s = cur if i % 2 == 0 else aux
        with torch.cuda.stream(s):
            attn_fn(q_loc[:, qsl], k_loc[:, ksl], v_loc[:, ksl], out_loc[:, qsl])
            done = torch.cuda.Event()
            done.record(s)
        with torch.cuda.stream(comm):
            comm.wait_event(done)
            _exchange_block(out, hp, qsl, world, rank, group, nccl)
    cur.wait_stream(aux)
    cur.wait_stream(comm)
    return out


class DecodeShards:
    """The batch partition of a decode step: which sequences each rank owns (balanced by cache
    length) and the index that puts the gathered outputs back into the original batch order."""

    def __init__(self, lens: Sequence[int], world: int):
        self.world = world
        self.shards = balanced_batch_shards([int(x) for x in lens], world)
        self._order: dict = {}

    def mine(self, rank: int) -> List[int]:
        return self.shards[rank]

    def order(self, device) -> torch.Tensor:
        key = str(device)
        if key not in self._order:
            self._order[key] = torch.tensor([i for s in self.shards for i in s], dtype=torch.long, device=device)
        return self._order[key]


def decode_batch_parallel(attn_fn: Callable, q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                          lens: torch.Tensor, shards: DecodeShards, out: Optional[torch.Tensor] = None,
                          group=None) -> torch.Tensor:
    """Decode with the batch partitioned over ranks.

    q [B/W,H,1,D], caches [B/W,Hkv,Lmax,D], lens [B/W]: THIS RANK'S sequences, in the order of
    shards.mine(rank) - a rank holds only its own share of the cache and nothing is copied or
    re-indexed per step.  attn_fn(q, k_cache, v_cache, lens, out_local) is the decode op or a
    stand-in.  Returns the full [B,H,1,D] output in the original batch order on every rank (one
    all-gather of 2*H*D bytes per sequence, then a scatter by a cached index).
    """
    world = dist.get_world_size(group)
    per, H, _, D = q.shape
    gathered = torch.empty((world, per, H, 1, D), dtype=q.dtype, device=q.device)
    rank = dist.get_rank(group)
    attn_fn(q, k_cache, v_cache, lens, gathered[rank])
    if world > 1:
        nccl = q.is_cuda and dist.get_backend(group) == "nccl"
        mine = gathered[rank].view(-1)
        dist.all_gather_into_tensor(gathered.view(-1), mine if nccl else mine.clone(), group=group)
    if out is None:
        out = torch.empty((world * per, H, 1, D), dtype=q.dtype, device=q.device)
    out.index_copy_(0, shards.order(q.device), gathered.view(world * per, H, 1, D))
    return out
