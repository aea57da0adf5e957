#!/usr/bin/env python
"""Benchmark of the attention path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--legs all|core]

A step is one pass of the hot path over one batch of synthetic input.  The JSON line holds:
  * headline (`value`): causal GQA prefill, Llama-3-8B shape (batch 4 per GPU, 32 query / 8 kv
    heads, head_dim 128, seq_len 4096, fp16), inputs resident in HBM, CUDA-event timing, TFLOP/s
    in the causal-half convention (4*B*H*L^2*D / 2 floating-point operations per step); with N > 1
    every rank runs that workload on its own batch shard (weak scaling, no collective in `value`;
    `value_with_gather` adds the NCCL all-gather of the outputs to the timed region);
  * `sustained`: the same step looped for at least a second, whatever --steps is, with its own clock
    samples, against the sustained matmul peak (the GPU then sits at its power cap);
  * `e2e`: the same call through KernelBackend("torch_ext") with pinned HOST buffers, host->device and
    device->host copies inside the timed region, consecutive steps overlapped (three streams, two
    device buffer sets); the one-stream figure and each direction's copy bandwidth beside it;
  * `config4`: the long-context configuration (batch 1, 64/8 heads, head_dim 128, seq_len 32768,
    bf16) with a FIXED total problem partitioned by kv-head group over the N ranks through
    minfer.dist.prefill_head_parallel, the output exchange over NCCL inside the timed region
    (strong scaling: kernel-only ms, total ms, the exposed exchange, and the single-GPU time of the
    whole problem measured in the same run);
  * `decode`: the split-KV decode kernel over a padded KV cache (batch 64, 32/8 heads, head_dim 128,
    lengths uniform in [512, 8192]), GB/s of live KV-cache bytes; `decode_dist` (N > 1): the same
    global batch partitioned by sequence over the ranks, output all-gather included;
  * `legs` (N = 1): the reference's own op signature flash_attn(qtype, .., mask, out) with dense causal
    and sliding-window masks at the reference benchmark's shapes, head_dim 64 prefill, Q8_0 and paged
    decode, RoPE + KV append - each with its roofline - and `config5`, the Llama-3.2-1B-shaped
    generation run of apps/generate.py;
  * `cpu_baseline` / `--impl reference`: the reference's CPU path (torch SDPA with
    repeat_interleave-expanded K/V and a dense causal mask, restated in oracle/oracle.py) on the
    box's host cores, timed on the full step.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "minfer-python_b200"))

import torch  # noqa: E402

PREFILL = dict(batch=4, n_heads=32, n_kv_heads=8, head_dim=128, seq_len=4096)
DECODE = dict(batch=64, n_heads=32, n_kv_heads=8, head_dim=128, max_len=8192, min_len=512)
CONFIG4 = dict(batch=1, n_heads=64, n_kv_heads=8, head_dim=128, seq_len=32768)
WORKLOAD = "config2: causal GQA prefill B=4/GPU Hq=32 Hkv=8 D=128 L=4096 fp16, contiguous [B,H,S,D]"
METRIC = "prefill attn TFLOP/s per B200 (causal-half FLOP convention); decode KV-cache GB/s in `decode`"
# exchange pipeline of the config-4 record: head blocks per rank and SMs left to NCCL while attention runs
C4_BLOCKS = int(os.environ.get("MINFER_BENCH_C4_BLOCKS", "4"))
C4_SM_MARGIN = int(os.environ.get("MINFER_BENCH_C4_SM_MARGIN", "8"))


def prefill_flops(c) -> float:
    return 4.0 * c["batch"] * c["n_heads"] * c["seq_len"] ** 2 * c["head_dim"] / 2.0


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(tflops=float(p["bf16_tflops"]), tflops_sustained=float(p["bf16_tflops_sustained"]),
                    hbm_gbs=float(p["hbm_gbs"]), source="measured (MEASURED_PEAKS.json)")
    return dict(tflops=1590.0, tflops_sustained=1400.0, hbm_gbs=6650.0, source="fallback (file absent)")


def load_traffic():
    """DRAM bytes per launch taken from the committed ncu summaries (profiles/traffic.json), if present."""
    path = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f)
    return {}


class ClockSampler:
    """nvidia-smi samples during a timed region (read-only queries)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int, period_ms: int = 50):
        self.proc = None
        self.gpu_index = gpu_index
        self.period_ms = period_ms

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", str(self.period_ms),
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
        return self

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.12)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out = ""
        sm, smax, power, reasons = [], [], [], set()
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
                power.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        # samples taken while the GPU was busy: the upper half by power draw
        busy = sm
        if len(power) >= 4:
            cut = statistics.median(power)
            busy = [c for c, p in zip(sm, power) if p >= cut] or sm
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(smax) if smax else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def dist_env():
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")),
            int(os.environ.get("LOCAL_RANK", "0")))


def reduce_ranks(x: float, world: int, device, op="max") -> float:
    if world == 1:
        return x
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX if op == "max" else dist.ReduceOp.MIN)
    return float(t.item())


def barrier(world: int):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()


def time_gpu(fn, steps: int, warmup: int, world: int, dev, stream=None) -> float:
    """ms per call: `warmup` untimed calls, then `steps` calls between two CUDA events on the launching stream,
    a barrier and a device synchronisation on both sides, the maximum over ranks."""
    for _ in range(warmup):
        fn()
    barrier(world)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        fn()
    e1.record(stream)
    torch.cuda.synchronize()
    barrier(world)
    return reduce_ranks(e0.elapsed_time(e1), world, dev) / steps


# --------------------------------------------------------------------------
# CPU arm: the reference's torch path on host cores
# --------------------------------------------------------------------------
def cpu_reference_inputs(seed: int = 1):
    """The full prefill step of the headline workload, as the reference's callers would hand it to refs.flash_attn."""
    from oracle import oracle as O
    c = PREFILL
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(c["batch"], c["n_heads"], c["seq_len"], c["head_dim"], generator=g).half()
    k = torch.randn(c["batch"], c["n_kv_heads"], c["seq_len"], c["head_dim"], generator=g).half()
    v = torch.randn(c["batch"], c["n_kv_heads"], c["seq_len"], c["head_dim"], generator=g).half()
    mask = O.causal_mask(c["batch"], c["seq_len"])
    return q, O.expand_kv(k, c["n_heads"]), O.expand_kv(v, c["n_heads"]), mask


def time_cpu_reference(steps: int, warmup: int):
    from oracle import oracle as O
    # all host cores this process may use (torchrun pins OMP_NUM_THREADS=1 otherwise)
    try:
        torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    except (AttributeError, OSError):
        torch.set_num_threads(max(1, os.cpu_count() or 1))
    q, k, v, mask = cpu_reference_inputs()
    for _ in range(warmup):
        O.sdpa_reference(q, k, v, mask)
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        O.sdpa_reference(q, k, v, mask)
        times.append(time.perf_counter() - t0)
    sec = statistics.median(times)
    return prefill_flops(PREFILL) / sec / 1e12, sec, torch.get_num_threads()


CPU_SAMPLE = ("the full step (B=4, 32 heads, L=4096, fp16) through torch CPU SDPA with expanded K/V and a dense "
              "causal mask, all host threads")


def run_reference_arm(args):
    rank, _, _ = dist_env()
    if rank != 0:
        return
    # every step is the full B=4 step (about half a second on a few dozen cores); the count is bounded so that
    # the run ends within a few minutes whatever --steps says, and the counts printed are the ones run
    steps, warmup = max(1, min(args.steps, 40)), max(1, min(args.warmup, 3))
    tflops, sec, cores = time_cpu_reference(steps, warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": tflops, "unit": "TFLOP/s", "n_gpus": 1,
        "steps": steps, "warmup": warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "l2": "n/a (CPU)", "flop_convention": "causal half: 4*B*H*L^2*D/2",
                   "ranks": "rank 0 alone runs the CPU arm, on one GPU's share of the workload"},
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                         "sample": CPU_SAMPLE + f"; median of {steps}"},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------
# GPU arm: pieces
# --------------------------------------------------------------------------
def headline_and_e2e(kerns, args, rank, world, local, dev, peaks):
    from minfer.kernels.torch_ext.ops import check_status
    c = PREFILL
    B, H, Hkv, L, D = c["batch"], c["n_heads"], c["n_kv_heads"], c["seq_len"], c["head_dim"]
    flops = prefill_flops(c)
    warm = max(args.warmup, 3)

    # inputs: seeded on the host (pinned), so the end-to-end leg can copy them every step
    g = torch.Generator().manual_seed(1 + rank)
    hq = torch.randn(B, H, L, D, generator=g).half().pin_memory()
    hk = torch.randn(B, Hkv, L, D, generator=g).half().pin_memory()
    hv = torch.randn(B, Hkv, L, D, generator=g).half().pin_memory()
    hout = torch.empty(B, H, L, D, dtype=torch.float16).pin_memory()
    q, k, v = hq.to(dev), hk.to(dev), hv.to(dev)
    out = torch.zeros(B, H, L, D, dtype=torch.float16, device=dev)
    in_bytes = (hq.numel() + hk.numel() + hv.numel()) * 2
    out_bytes = hout.numel() * 2

    def step():
        kerns.flash_attn_causal(q, k, v, out)

    # ---- device-resident headline ----
    for _ in range(warm):
        step()
    check_status(dev)
    sampler = ClockSampler(local).start() if rank == 0 else None
    ms = time_gpu(step, args.steps, 0, world, dev)
    clocks = sampler.stop() if sampler else None
    check_status(dev)

    # ---- the same step for at least a second: clocks and power settle at the power cap ----
    n_sus = max(args.steps, int(math.ceil(1100.0 / ms)))
    sampler = ClockSampler(local).start() if rank == 0 else None
    ms_sus = time_gpu(step, n_sus, 0, world, dev)
    clocks_sus = sampler.stop() if sampler else None
    sustained = {"steps": n_sus, "ms_per_step": ms_sus, "timed_s": ms_sus * n_sus / 1e3,
                 "value": flops * world / (ms_sus * 1e-3) / 1e12, "unit": "TFLOP/s",
                 "per_gpu": flops / (ms_sus * 1e-3) / 1e12,
                 "frac_of_sustained_peak": flops / (ms_sus * 1e-3) / 1e12 / peaks["tflops_sustained"],
                 "frac_of_nominal_2250": flops / (ms_sus * 1e-3) / 1e12 / 2250.0, "clocks": clocks_sus}

    # ---- weak-scaling step with the output all-gather inside the timed region ----
    with_gather = None
    if world > 1:
        import torch.distributed as dist
        gathered = torch.empty(world * B, H, L, D, dtype=torch.float16, device=dev)
        mine = gathered[rank * B:(rank + 1) * B]

        def step_gather():
            kerns.flash_attn_causal(q, k, v, mine)
            dist.all_gather_into_tensor(gathered, mine)

        ms_g = time_gpu(step_gather, min(args.steps, 50), 2, world, dev)
        with_gather = {"value": flops * world / (ms_g * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_g,
                       "gather_bytes_per_rank": out_bytes * (world - 1),
                       "note": "attention, then one NCCL all-gather of every rank's [B,H,L,D] output, not overlapped"}
        del gathered, mine

    # ---- end to end: every step copies its inputs from pinned host memory, runs the call and reads the result
    # back.  Copies and kernels of consecutive steps overlap the way a serving loop would overlap them: an
    # upload stream, the stream the library launches on, and a download stream, over two sets of device buffers.
    s_in, s_run, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    bufs = [(q, k, v, out), (torch.empty_like(q), torch.empty_like(k), torch.empty_like(v), torch.empty_like(out))]
    ev_in = [torch.cuda.Event(), torch.cuda.Event()]    # inputs of the set have arrived
    ev_run = [torch.cuda.Event(), torch.cuda.Event()]   # the call on the set has finished
    ev_out = [torch.cuda.Event(), torch.cuda.Event()]   # the set's result has reached the host

    def step_e2e(i):
        bq, bk, bv, bo = bufs[i & 1]
        with torch.cuda.stream(s_in):
            if i >= 2:
                s_in.wait_event(ev_run[i & 1])          # the call two steps ago has read these inputs
            bq.copy_(hq, non_blocking=True)
            bk.copy_(hk, non_blocking=True)
            bv.copy_(hv, non_blocking=True)
            ev_in[i & 1].record(s_in)
        with torch.cuda.stream(s_run):
            s_run.wait_event(ev_in[i & 1])
            if i >= 2:
                s_run.wait_event(ev_out[i & 1])         # the result two steps ago has left this buffer
            kerns.flash_attn_causal(bq, bk, bv, bo)
            ev_run[i & 1].record(s_run)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_run[i & 1])
            hout.copy_(bo, non_blocking=True)
            ev_out[i & 1].record(s_out)

    def step_e2e_serial():
        q.copy_(hq, non_blocking=True)
        k.copy_(hk, non_blocking=True)
        v.copy_(hv, non_blocking=True)
        kerns.flash_attn_causal(q, k, v, out)
        hout.copy_(out, non_blocking=True)

    e2e_steps = min(args.steps, 100)  # each step moves 336 MB over PCIe; 100 steps are ~0.4 s
    for i in range(4):
        step_e2e(i)
    torch.cuda.synchronize()
    barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(s_run)
    for i in range(e2e_steps):
        step_e2e(i)
    s_run.wait_stream(s_out)
    s_run.wait_stream(s_in)
    e1.record(s_run)
    torch.cuda.synchronize()
    barrier(world)
    ms_e2e = reduce_ranks(e0.elapsed_time(e1), world, dev) / e2e_steps
    check_status(dev)
    ms_e2e_serial = time_gpu(step_e2e_serial, min(e2e_steps, 30), 2, world, dev)

    # each direction alone, all ranks copying at the same time: what the host side gives one rank
    def up():
        q.copy_(hq, non_blocking=True)

    def down():
        hout.copy_(out, non_blocking=True)

    n_copy = 20
    for fn in (up, down):
        fn()
    barrier(world)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(n_copy):
        up()
    e1.record()
    torch.cuda.synchronize()
    t_up = e0.elapsed_time(e1) / n_copy
    barrier(world)
    e0.record()
    for _ in range(n_copy):
        down()
    e1.record()
    torch.cuda.synchronize()
    t_down = e0.elapsed_time(e1) / n_copy
    h2d = hq.numel() * 2 / (t_up * 1e-3) / 1e9
    d2h = out_bytes / (t_down * 1e-3) / 1e9
    copies = {"h2d_gbs_per_rank_min": -reduce_ranks(-h2d, world, dev), "h2d_gbs_per_rank_max": reduce_ranks(h2d, world, dev),
              "d2h_gbs_per_rank_min": -reduce_ranks(-d2h, world, dev), "d2h_gbs_per_rank_max": reduce_ranks(d2h, world, dev),
              "note": "134 MB pinned copies, one direction at a time, every rank copying at once"}

    # the reference-facing signature flash_attn(qtype, qblock, qsize, q, k, v, mask, out) on the same inputs, the
    # dense causal mask resident on the device (a constant of the call site, built once as the reference's own
    # benchmark does): device-resident and end to end
    mask = (torch.arange(L, device=dev)[None, :] <= torch.arange(L, device=dev)[:, None])[None, None].expand(B, 1, L, L).contiguous()

    def step_mask():
        kerns.flash_attn(1, 1, 2, q, k, v, mask, out)

    ms_mask = time_gpu(step_mask, min(args.steps, 100), 3, world, dev)

    def step_mask_serial():
        q.copy_(hq, non_blocking=True)
        k.copy_(hk, non_blocking=True)
        v.copy_(hv, non_blocking=True)
        kerns.flash_attn(1, 1, 2, q, k, v, mask, out)
        hout.copy_(out, non_blocking=True)

    ms_mask_e2e = time_gpu(step_mask_serial, min(e2e_steps, 30), 2, world, dev)
    check_status(dev)
    del mask

    per_gpu = flops / (ms * 1e-3) / 1e12
    res = dict(ms=ms, per_gpu_tflops=per_gpu, clocks=clocks, sustained=sustained, with_gather=with_gather,
               e2e={"value": flops * world / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": in_bytes, "d2h_bytes_per_step": out_bytes, "ms_per_step": ms_e2e,
                    "steps": e2e_steps, "overlap": "uploads, launches and downloads of consecutive steps overlap "
                    "(three streams, two device buffer sets)", "ms_per_step_one_stream": ms_e2e_serial,
                    "copies": copies,
                    "via_flash_attn_dense_mask": {
                        "device_resident_tflops": flops * world / (ms_mask * 1e-3) / 1e12, "ms_per_step": ms_mask,
                        "e2e_one_stream_tflops": flops * world / (ms_mask_e2e * 1e-3) / 1e12,
                        "e2e_one_stream_ms": ms_mask_e2e,
                        "note": "the reference's op signature with a dense causal bool mask [B,1,L,L] kept on the device"}})
    return res


def decode_leg(kerns, args, rank, world, dev, peaks, traffic):
    d = DECODE
    gd = torch.Generator().manual_seed(2)
    lens = torch.randint(d["min_len"], d["max_len"] + 1, (d["batch"],), generator=gd, dtype=torch.int32)
    dq = torch.randn(d["batch"], d["n_heads"], 1, d["head_dim"], device=dev, dtype=torch.float16)
    kc = torch.randn(d["batch"], d["n_kv_heads"], d["max_len"], d["head_dim"], device=dev, dtype=torch.float16)
    vc = torch.randn(d["batch"], d["n_kv_heads"], d["max_len"], d["head_dim"], device=dev, dtype=torch.float16)
    dout = torch.zeros_like(dq)
    dlens = lens.to(dev)
    ms_dec = time_gpu(lambda: kerns.flash_attn_decode(dq, kc, vc, dlens, dout), args.steps, 5, world, dev)
    dec_bytes = 2.0 * 2 * d["n_kv_heads"] * d["head_dim"] * float(lens.sum())  # K and V, 16-bit, live rows only
    dec_gbs = dec_bytes / (ms_dec * 1e-3) / 1e9
    rec = {"value": dec_gbs * world, "unit": "GB/s", "ms_per_step": ms_dec,
           "workload": "config3: B=64/GPU Hq=32 Hkv=8 D=128, lens U[512,8192] seed 2, cache padded to 8192",
           "bytes_per_step": dec_bytes, "gpu_launches_per_step": DECODE_LAUNCHES,
           "roofline": {"bound": "hbm", "achieved": dec_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                        "frac": dec_gbs / peaks["hbm_gbs"], "traffic": traffic.get("decode"),
                        "frac_of_nominal_8000": dec_gbs / 8000.0, "kernel": DECODE_KERNELS}}
    extra = None
    if world > 1:
        # strong scaling: the SAME global batch of 64 partitioned by sequence (sorted by length, dealt in a
        # snake), every rank holding only its own share of the cache; one all-gather of the outputs per step
        from minfer.dist import DecodeShards, decode_batch_parallel
        shards = DecodeShards(lens.tolist(), world)
        mine = torch.tensor(shards.mine(rank), device=dev)
        q_s, k_s, v_s, l_s = dq[mine].contiguous(), kc[mine].contiguous(), vc[mine].contiguous(), dlens[mine].contiguous()
        del kc, vc
        full = torch.empty_like(dq)
        o_s = torch.empty_like(q_s)
        ms_k = time_gpu(lambda: kerns.flash_attn_decode(q_s, k_s, v_s, l_s, o_s), min(args.steps, 200), 5, world, dev)
        ms_t = time_gpu(lambda: decode_batch_parallel(kerns.flash_attn_decode, q_s, k_s, v_s, l_s, shards, out=full),
                        min(args.steps, 200), 5, world, dev)
        extra = {"workload": "config3, global batch 64 partitioned by sequence over the ranks (strong scaling)",
                 "ms_kernel_only": ms_k, "ms_total": ms_t, "value": dec_bytes / (ms_t * 1e-3) / 1e9, "unit": "GB/s",
                 "value_kernel_only": dec_bytes / (ms_k * 1e-3) / 1e9,
                 "note": "total = decode of this rank's sequences + NCCL all-gather of [B/N,H,1,D] + reorder"}
    return rec, extra


DECODE_LAUNCHES = 2
DECODE_KERNELS = "decode_split_kernel<128,f16> + decode_combine_kernel"


def config4_record(kerns, args, rank, world, dev, peaks):
    """Strong scaling of the long-context prefill: fixed total problem, kv-head-group partition, output exchange
    (NCCL) inside the timed region."""
    from minfer.dist import PeerOutputs, head_shard, prefill_head_parallel, prefill_head_parallel_fused
    from minfer.kernels.torch_ext.ops import check_status, prefill_cta_limit
    c = CONFIG4
    B, H, Hkv, L, D = c["batch"], c["n_heads"], c["n_kv_heads"], c["seq_len"], c["head_dim"]
    flops = prefill_flops(c)
    qs, kvs = head_shard(H, Hkv, world, rank)
    g = torch.Generator(device=dev).manual_seed(3)
    q = torch.randn(B, H, L, D, generator=g, device=dev, dtype=torch.float32).bfloat16()
    k = torch.randn(B, Hkv, L, D, generator=g, device=dev, dtype=torch.float32).bfloat16()
    v = torch.randn(B, Hkv, L, D, generator=g, device=dev, dtype=torch.float32).bfloat16()
    out = torch.zeros(B, H, L, D, dtype=torch.bfloat16, device=dev)
    n = max(3, min(args.steps, 10))

    # the whole problem on one GPU (every rank times it on its own device at the same moment)
    ms_1 = time_gpu(lambda: kerns.flash_attn_causal(q, k, v, out), max(3, min(args.steps, 5)), 2, world, dev)
    check_status(dev)
    rec = {"workload": "config4: B=1 Hq=64 Hkv=8 D=128 L=32768 bf16 causal, fixed total problem",
           "flops": flops, "t1_ms_whole_problem_one_gpu": ms_1, "t1_tflops": flops / (ms_1 * 1e-3) / 1e12}
    if world == 1:
        rec.update({"ms_total": ms_1, "ms_kernel_only": ms_1, "value": rec["t1_tflops"], "unit": "TFLOP/s",
                    "strong_efficiency": 1.0, "frac_of_nominal_2250": rec["t1_tflops"] / 2250.0,
                    "frac_of_burst_peak": rec["t1_tflops"] / peaks["tflops"]})
        return rec
    reference = out[:, qs].clone()       # this rank's heads from the single-GPU run: the exchange must deliver the same
    q_s, k_s, v_s = q[:, qs].contiguous(), k[:, kvs].contiguous(), v[:, kvs].contiguous()
    del q, k, v
    out.zero_()
    ms_k = time_gpu(lambda: kerns.flash_attn_causal(q_s, k_s, v_s, out[:, qs]), n, 2, world, dev)

    def step(blocks, margin):
        with prefill_cta_limit(0 if margin == 0 else max(1, torch.cuda.get_device_properties(dev).multi_processor_count - margin)):
            prefill_head_parallel(kerns.flash_attn_causal, q_s, k_s, v_s, out=out, blocks=blocks, inputs_are_shards=True)

    ms_plain = time_gpu(lambda: step(1, 0), n, 2, world, dev)           # attention, then one in-place all-gather
    ms_pipe = time_gpu(lambda: step(C4_BLOCKS, C4_SM_MARGIN), n, 2, world, dev)
    check_status(dev)
    # the exchange fused into the attention kernel: every output tile is stored into all ranks' output tensors
    # (shared through CUDA IPC) as it is produced; one barrier across the ranks ends the step
    ms_fused, fused_ok, fused_err = None, None, None
    try:
        if os.environ.get("MINFER_BENCH_FUSED", "1") in ("", "0"):
            raise RuntimeError("fused form switched off (MINFER_BENCH_FUSED=0)")
        shared = PeerOutputs((B, H, L, D), torch.bfloat16, dev)
        ms_fused = time_gpu(lambda: prefill_head_parallel_fused(q_s, k_s, v_s, shared, inputs_are_shards=True), n, 2, world, dev)
        check_status(dev)
        fsums = shared.local.view(world, -1).float().abs().sum(dim=1).double()
        fhi, flo = fsums.clone(), fsums.clone()
        import torch.distributed as dist
        dist.all_reduce(fhi, op=dist.ReduceOp.MAX)
        dist.all_reduce(flo, op=dist.ReduceOp.MIN)
        fused_ok = bool(torch.equal(fhi, flo)) and bool(torch.equal(shared.local[:, qs], reference)) and bool(torch.isfinite(fsums).all())
        fused_ok = reduce_ranks(0.0 if fused_ok else 1.0, world, dev) == 0.0
        shared.close()
        del shared
    except Exception as e:  # noqa: BLE001  (peer mapping unavailable: the NCCL forms stand)
        fused_err = repr(e)[:200]
    # every rank must now hold every shard: compare per-shard checksums across ranks, and this rank's shard
    # with what the single-GPU run produced
    import torch.distributed as dist
    sums = out.view(world, -1).float().abs().sum(dim=1).double()
    hi, lo = sums.clone(), sums.clone()
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    ok = bool(torch.equal(hi, lo)) and bool(torch.equal(out[:, qs], reference)) and bool(torch.isfinite(sums).all())
    ok = reduce_ranks(0.0 if ok else 1.0, world, dev) == 0.0
    best = min(x for x in (ms_plain, ms_pipe, ms_fused if fused_ok else None) if x is not None)
    rec.update({
        "ms_kernel_only": ms_k, "ms_total": best, "ms_total_unpipelined": ms_plain, "ms_total_pipelined": ms_pipe,
        "ms_total_fused": ms_fused, "fused_verified": fused_ok, "fused_error": fused_err,
        "forms": "unpipelined: attention, then one in-place NCCL all-gather; pipelined: head blocks exchanged by NCCL "
                 "point-to-point while the next block is computed; fused: the attention kernel stores every output tile "
                 "into all ranks' outputs (CUDA IPC, plain TMA stores over NVLink), one NCCL barrier ends the step",
        "exchange_exposed_ms": best - ms_k, "pipeline": {"head_blocks": C4_BLOCKS, "sm_margin": C4_SM_MARGIN},
        "value": flops / (best * 1e-3) / 1e12, "unit": "TFLOP/s", "value_kernel_only": flops / (ms_k * 1e-3) / 1e12,
        "strong_efficiency": ms_1 / (world * best), "strong_efficiency_kernel_only": ms_1 / (world * ms_k),
        "exchange_bytes_received_per_rank": out.numel() * 2 * (world - 1) // world, "exchange_verified": ok,
        "partition": f"rank g owns kv heads [{Hkv // world}g, {Hkv // world}(g+1)) and their query heads"})
    return rec


def extra_legs(kerns, args, dev, peaks):
    """Device-resident legs beyond the headline (one GPU): each returns ms and a roofline."""
    from minfer.kernels.torch_ext.ops import check_status
    legs = {}
    hbm, tpeak = peaks["hbm_gbs"], peaks["tflops"]

    def tensor_roof(tflops, kernel):
        return {"bound": "tensor", "achieved": tflops, "peak": tpeak, "unit": "TFLOP/s", "frac": tflops / tpeak,
                "frac_of_nominal_2250": tflops / 2250.0, "kernel": kernel}

    def hbm_roof(gbs, kernel):
        return {"bound": "hbm", "achieved": gbs, "peak": hbm, "unit": "GB/s", "frac": gbs / hbm,
                "frac_of_nominal_8000": gbs / 8000.0, "kernel": kernel}

    # --- the reference's op signature at the reference benchmark's shapes: B=4, 48/8 heads, D=128, inputs as
    # transposed views of [B, L, H*D] storage, dense bool masks [B,1,L,L] (causal; sliding window 256)
    B, H, Hkv, D = 4, 48, 8, 128
    for L in (4096, 8192, 16384):
        q = torch.randn(B, L, H * D, device=dev, dtype=torch.float16).view(B, L, H, D).transpose(1, 2)
        k = torch.randn(B, L, Hkv * D, device=dev, dtype=torch.float16).view(B, L, Hkv, D).transpose(1, 2)
        v = torch.randn(B, L, Hkv * D, device=dev, dtype=torch.float16).view(B, L, Hkv, D).transpose(1, 2)
        out = torch.zeros(B, H, L, D, dtype=torch.float16, device=dev)
        i = torch.arange(L, device=dev)
        for kind in ("causal", "window256"):
            m2 = (i[None, :] <= i[:, None]) if kind == "causal" else ((i[None, :] - i[:, None]).abs() < 256)
            visible = float(m2.sum())
            mask = m2[None, None].expand(B, 1, L, L).contiguous()
            del m2
            ms = time_gpu(lambda: kerns.flash_attn(1, 1, 2, q, k, v, mask, out), 10 if L > 4096 else 20, 3, 1, dev)
            fl = 4.0 * B * H * D * visible          # QK^T and PV over the visible (query, key) pairs only
            legs[f"flash_attn_mask_{kind}_L{L}"] = {
                "ms": ms, "flops_visible_pairs": fl, "mask_bytes": B * L * L,
                "roofline": tensor_roof(fl / (ms * 1e-3) / 1e12, "mask_classify_kernel + prefill_persist_kernel<128,f16,masked>")}
            del mask
        if L == 8192:
            ms = time_gpu(lambda: kerns.flash_attn_causal(q, k, v, out), 10, 3, 1, dev)
            legs["flash_attn_causal_entry_L8192_48h"] = {
                "ms": ms, "roofline": tensor_roof(4.0 * B * H * L * L * D / 2 / (ms * 1e-3) / 1e12, "prefill_persist_kernel<128,f16>")}
        del q, k, v, out
        torch.cuda.empty_cache()

    # --- head_dim 64 prefill (the end-to-end model's head size), causal entry
    for (B, H, Hkv, L, dt) in ((4, 32, 8, 8192, torch.float16), (8, 32, 8, 512, torch.float16)):
        q = torch.randn(B, H, L, 64, device=dev, dtype=dt)
        k = torch.randn(B, Hkv, L, 64, device=dev, dtype=dt)
        v = torch.randn(B, Hkv, L, 64, device=dev, dtype=dt)
        out = torch.zeros_like(q)
        ms = time_gpu(lambda: kerns.flash_attn_causal(q, k, v, out), 20, 3, 1, dev)
        legs[f"prefill_d64_B{B}_L{L}"] = {"ms": ms, "roofline": tensor_roof(4.0 * B * H * L * L * 64 / 2 / (ms * 1e-3) / 1e12,
                                                                              "prefill_persist_kernel<64,f16>")}
        del q, k, v, out

    # --- decode variants at config 3: Q8_0 cache, paged cache
    d = DECODE
    Bd, Hd, Hk, Dd, Lm = d["batch"], d["n_heads"], d["n_kv_heads"], d["head_dim"], d["max_len"]
    lens = torch.randint(d["min_len"], Lm + 1, (Bd,), generator=torch.Generator().manual_seed(2), dtype=torch.int32)
    dl = lens.to(dev)
    dq = torch.randn(Bd, Hd, 1, Dd, device=dev, dtype=torch.float16)
    dout = torch.zeros_like(dq)
    row = Dd // 32 * 34
    kq = torch.randint(0, 256, (Bd, Hk, Lm, row), dtype=torch.uint8, device=dev)
    vq = torch.randint(0, 256, (Bd, Hk, Lm, row), dtype=torch.uint8, device=dev)
    for cq in (kq, vq):                                  # sane fp16 scales (about 0.01), random int8 values
        blocks = cq.view(Bd, Hk, Lm, Dd // 32, 34)
        blocks[..., 1] = 0x21
    ms = time_gpu(lambda: kerns.flash_attn_decode_q8(dq, kq, vq, dl, dout), 200, 5, 1, dev)
    q8_bytes = 2.0 * Hk * row * float(lens.sum())
    legs["decode_q8_0"] = {"ms": ms, "bytes_per_step": q8_bytes, "tokens_per_s_equivalent_16bit_gbs": 2.0 * 2 * Hk * Dd * float(lens.sum()) / (ms * 1e-3) / 1e9,
                           "roofline": hbm_roof(q8_bytes / (ms * 1e-3) / 1e9, "decode_split_kernel<128,f16,q8> + decode_combine_kernel")}
    del kq, vq
    page = 64
    pages_per_seq = Lm // page
    n_pages = Bd * pages_per_seq
    kp = torch.randn(n_pages, Hk, page, Dd, device=dev, dtype=torch.float16)
    vp = torch.randn(n_pages, Hk, page, Dd, device=dev, dtype=torch.float16)
    table = torch.randperm(n_pages, generator=torch.Generator().manual_seed(3)).reshape(Bd, pages_per_seq).to(torch.int32).to(dev)
    ms = time_gpu(lambda: kerns.flash_attn_decode_paged(dq, kp, vp, table, dl, dout), 200, 5, 1, dev)
    fp_bytes = 2.0 * 2 * Hk * Dd * float(lens.sum())
    legs["decode_paged_64"] = {"ms": ms, "bytes_per_step": fp_bytes, "page_size": page, "page_order": "shuffled",
                               "roofline": hbm_roof(fp_bytes / (ms * 1e-3) / 1e9, "decode_split_kernel<128,f16,paged> + decode_combine_kernel")}
    del kp, vp, table
    torch.cuda.empty_cache()

    # --- RoPE + KV append: a prefill-sized call (B=4, L=4096, 32/8 heads, D=128) and a decode-sized one
    for (B, L, tag) in ((4, 4096, "prefill"), (64, 1, "decode")):
        Hq, Hk2, D2, Lmax = 32, 8, 128, 8192
        q = torch.randn(B, L, Hq, D2, device=dev, dtype=torch.float16)
        k = torch.randn(B, L, Hk2, D2, device=dev, dtype=torch.float16)
        v = torch.randn(B, L, Hk2, D2, device=dev, dtype=torch.float16)
        kcache = torch.zeros(B, Hk2, Lmax, D2, device=dev, dtype=torch.float16)
        vcache = torch.zeros_like(kcache)
        start = torch.zeros(B, dtype=torch.int32, device=dev)
        ms = time_gpu(lambda: kerns.rope_kv_append(D2, 500000.0, 0, q, k, v, kcache, vcache, start), 50, 5, 1, dev)
        nbytes = 2.0 * B * L * D2 * (2 * Hq + 4 * Hk2)     # q read + written, k and v read, two cache rows written
        legs[f"rope_kv_append_{tag}"] = {"ms": ms, "bytes_per_step": nbytes,
                                         "roofline": hbm_roof(nbytes / (ms * 1e-3) / 1e9, "rope_append_kernel<f16,il>")}
        del q, k, v, kcache, vcache
    check_status(dev)
    torch.cuda.empty_cache()
    return legs


HOST_OVERHEAD_SCRIPT = r"""
import sys, time, json, torch
sys.path.insert(0, {pkg!r})
from minfer.kernels import KernelBackend
from minfer.kernels.torch_ext import ops
kerns = KernelBackend("torch_ext")
dev = torch.device("cuda", 0)
q = torch.randn(1, 4, 128, 128, device=dev, dtype=torch.float16); k = torch.randn(1, 2, 128, 128, device=dev, dtype=torch.float16)
v = torch.randn_like(k); out = torch.zeros_like(q)
mask = torch.ones(1, 1, 128, 128, dtype=torch.bool, device=dev)
dq = torch.randn(4, 8, 1, 128, device=dev, dtype=torch.float16); kc = torch.randn(4, 2, 256, 128, device=dev, dtype=torch.float16)
vc = torch.randn_like(kc); lens = torch.full((4,), 200, dtype=torch.int32, device=dev); dout = torch.zeros_like(dq)
calls = {{"flash_attn_causal": lambda: kerns.flash_attn_causal(q, k, v, out),
          "flash_attn": lambda: kerns.flash_attn(1, 1, 2, q, k, v, mask, out),
          "flash_attn_decode": lambda: kerns.flash_attn_decode(dq, kc, vc, lens, dout)}}
res = {{"binding": ops.BINDING}}
for name, fn in calls.items():
    for _ in range(200): fn()
    torch.cuda.synchronize()
    total, n = 0.0, 0
    for _ in range(20):                      # 20 x 500 = 10 k calls; the device is drained between batches, untimed
        t0 = time.perf_counter()
        for _ in range(500): fn()
        total += time.perf_counter() - t0; n += 500
        torch.cuda.synchronize()
    res[name] = total / n * 1e6
print(json.dumps(res))
"""


def host_overhead_record():
    """CPU-side cost of one op call (microseconds, 10 k calls on tiny shapes so that the device never back-pressures
    the host), for the torch-extension binding and for the ctypes binding, each in a process of its own."""
    out = {}
    for binding in ("stable", "ctypes"):
        env = dict(os.environ, MINFER_ATTN_BINDING=binding)
        script = HOST_OVERHEAD_SCRIPT.format(pkg=os.path.join(ROOT, "minfer-python_b200"))
        try:
            r = subprocess.run([sys.executable, "-c", script], env=env, capture_output=True, text=True, timeout=300)
            out[binding] = json.loads(r.stdout.strip().splitlines()[-1]) if r.returncode == 0 else {"error": (r.stderr or "")[-200:]}
        except Exception as e:  # noqa: BLE001  (a missing extension must not take the benchmark down)
            out[binding] = {"error": repr(e)[:200]}
    out["unit"] = "microseconds of host time per call"
    return out


def config5_record(dev):
    """apps/generate.py at the Llama-3.2-1B shape: 8 prompts x 512 tokens, 128 greedy steps."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("minfer_b200_generate", os.path.join(ROOT, "minfer-python_b200", "apps", "generate.py"))
    gen = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = gen
    spec.loader.exec_module(gen)
    B, Lp, new = 8, 512, 128
    with torch.no_grad():
        model = gen.Decoder(gen.Shape(), B, Lp + new, device=dev, init_on_device=True)
        prompts = torch.randint(0, gen.Shape().vocab, (B, Lp), generator=torch.Generator().manual_seed(5)).to(dev)
        gen.generate(model, prompts, 2, False)      # warm-up at the full shape (allocator blocks, cuBLAS algorithms)
        model.lens.zero_()
        _, eager = gen.generate(model, prompts, new, True, False)
        model.lens.zero_()
        _, graph = gen.generate(model, prompts, new, False, True)
    del model
    torch.cuda.empty_cache()
    return {"workload": "config5: Llama-3.2-1B shape (16 layers, hidden 2048, 32/8 heads, D=64, FFN 8192, vocab 128256), "
                        "fp16, random N(0,0.02) weights, 8 prompts x 512 tokens, 128 greedy steps",
            "prefill_ms": eager["prefill_ms"], "prefill_tokens_per_s": eager["prefill_tokens_per_s"],
            "prefill_attention_share": eager["prefill_attention_share"],
            "decode_ms_per_step_eager": eager["decode_ms_per_step"], "decode_attention_share_eager": eager["decode_attention_share"],
            "decode_ms_per_step_cuda_graph": graph["decode_ms_per_step"], "decode_tokens_per_s_cuda_graph": graph["decode_tokens_per_s"]}


def run_gpu_arm(args):
    rank, world, local = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the attention path has no CPU fallback "
                         "(use --impl reference for the CPU arm)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    from minfer.kernels import KernelBackend
    kerns = KernelBackend("torch_ext")
    peaks = load_peaks()
    traffic = load_traffic()
    c = PREFILL

    head = headline_and_e2e(kerns, args, rank, world, local, dev, peaks)
    torch.cuda.empty_cache()
    decode, decode_dist = decode_leg(kerns, args, rank, world, dev, peaks, traffic)
    torch.cuda.empty_cache()
    c4 = config4_record(kerns, args, rank, world, dev, peaks)
    torch.cuda.empty_cache()
    legs = c5 = None
    if world == 1 and args.legs == "all":
        legs = extra_legs(kerns, args, dev, peaks)
        legs["host_overhead"] = host_overhead_record()
        c5 = config5_record(dev)

    if rank == 0:
        ms, per_gpu = head["ms"], head["per_gpu_tflops"]
        # a timed region of a few hundred ms runs under the 1 kW power cap (clocks settle well below
        # the maximum), so it is compared with the sustained matmul peak; a short burst with the burst peak
        long_run = ms * args.steps > 300.0
        tensor_peak = peaks["tflops_sustained"] if long_run else peaks["tflops"]
        line = {
            "metric": METRIC, "value": per_gpu * world, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "global_batch": c["batch"] * world,
                       "parallelism": f"dp{world} over batch for `value` (no data-path collective; `value_with_gather` "
                                      "adds the output all-gather); `config4` is the kv-head-group partition",
                       "l2": "inputs+outputs 336 MB per step exceed the 126 MB L2; no explicit flush",
                       "flop_convention": "causal half: 4*B*H*L^2*D/2"},
            "clocks": head["clocks"],
            "e2e": head["e2e"],
            "gpu_launches": args.steps,
            "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": tensor_peak, "unit": "TFLOP/s",
                         "frac": per_gpu / tensor_peak, "traffic": traffic.get("prefill"),
                         "peak_source": f"{peaks['source']}, {'sustained' if long_run else 'burst'} bf16 matmul figure",
                         "frac_of_nominal_2250": per_gpu / 2250.0,
                         "kernel": "prefill_persist_kernel<128,f16>"},
            "sustained": head["sustained"],
            "decode": decode,
            "config4": c4,
        }
        if head["with_gather"] is not None:
            line["value_with_gather"] = head["with_gather"]
        if decode_dist is not None:
            line["decode_dist"] = decode_dist
        if legs is not None:
            line["legs"] = legs
            line["config5"] = c5
        if world == 1:
            cpu_tflops, cpu_sec, cores = time_cpu_reference(3, 1)
            line["cpu_baseline"] = {"value": cpu_tflops, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                                    "sample": CPU_SAMPLE + f"; {cpu_sec * 1e3:.0f} ms median of 3"}
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--legs", choices=["all", "core"], default="all",
                    help="core: skip the extra single-GPU legs and the config-5 generation run")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
