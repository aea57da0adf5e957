#!/usr/bin/env python
"""Benchmark of the attention path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A step is one pass of the hot path over one batch of synthetic input:
  * headline (`value`): causal GQA prefill, Llama-3-8B shape (batch 4 per GPU,
    32 query / 8 kv heads, head_dim 128, seq_len 4096, fp16), inputs resident
    in HBM, CUDA-event timing, TFLOP/s in the causal-half convention
    (4*B*H*L^2*D / 2 floating-point operations per step);
  * `e2e`: the same call through KernelBackend("torch_ext").flash_attn_causal
    with pinned HOST buffers, host->device and device->host copies inside the
    timed region; consecutive steps overlap their uploads, launches and
    downloads (three streams, two sets of device buffers), and the figure
    without any overlap is reported beside it (`ms_per_step_one_stream`);
  * `decode`: the split-KV decode kernel over a padded KV cache (batch 64,
    32/8 heads, head_dim 128, lengths uniform in [512, 8192]), GB/s of live
    KV-cache bytes;
  * `cpu_baseline` / `--impl reference`: the reference's CPU path (torch SDPA
    with repeat_interleave-expanded K/V and a dense causal mask, restated in
    oracle/oracle.py) on the box's host cores, on a bounded sample.

With N > 1 (launched under torchrun) every rank runs the same per-GPU workload
on its own batch shard (attention is independent per sequence and per kv-head
group, so there is no collective inside the data path); `value` is the sum over
ranks divided by the slowest rank's time.  The output all-gather the multi-GPU
harness offers is timed separately and reported as `allgather_ms`.
"""
from __future__ import annotations

import argparse
import json
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
WORKLOAD = "config2: causal GQA prefill B=4/GPU Hq=32 Hkv=8 D=128 L=4096 fp16, contiguous [B,H,S,D]"
METRIC = "prefill attn TFLOP/s per B200 (causal-half FLOP convention); decode KV-cache GB/s in `decode`"


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


class ClockSampler:
    """nvidia-smi samples during the timed region (read-only queries)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.proc = None
        self.gpu_index = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out = ""
        sm, smax, reasons = [], [], set()
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        busy = [x for x in sm if x > 0.5 * max(smax or [1])] or sm
        return {"sm_mhz": statistics.median(busy) if busy else None,
                "sm_max_mhz": max(smax) if smax else None, "samples": len(sm), "reasons": sorted(reasons)}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def max_over_ranks(x: float, world: int, device) -> float:
    if world == 1:
        return x
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier(world: int):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()


# --------------------------------------------------------------------------
# CPU arm: the reference's torch path on host cores
# --------------------------------------------------------------------------
def cpu_reference_step_inputs(seed: int = 1):
    """One batch element of the prefill workload (a bounded sample: 1/4 of a step)."""
    from oracle import oracle as O
    c = PREFILL
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(1, c["n_heads"], c["seq_len"], c["head_dim"], generator=g).half()
    k = torch.randn(1, c["n_kv_heads"], c["seq_len"], c["head_dim"], generator=g).half()
    v = torch.randn(1, c["n_kv_heads"], c["seq_len"], c["head_dim"], generator=g).half()
    mask = O.causal_mask(1, c["seq_len"])
    return q, O.expand_kv(k, c["n_heads"]), O.expand_kv(v, c["n_heads"]), mask


def time_cpu_reference(steps: int, warmup: int):
    from oracle import oracle as O
    # all host cores this process may use (torchrun pins OMP_NUM_THREADS=1 otherwise)
    try:
        torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    except (AttributeError, OSError):
        torch.set_num_threads(max(1, os.cpu_count() or 1))
    q, k, v, mask = cpu_reference_step_inputs()
    for _ in range(warmup):
        O.sdpa_reference(q, k, v, mask)
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        O.sdpa_reference(q, k, v, mask)
        times.append(time.perf_counter() - t0)
    sample_flops = prefill_flops(PREFILL) / PREFILL["batch"]
    sec = statistics.median(times)
    return sample_flops / sec / 1e12, sec, torch.get_num_threads()


def run_reference_arm(args):
    rank, world, _ = dist_env()
    if rank != 0:
        return
    tflops, sec, cores = time_cpu_reference(min(args.steps, 20), min(max(args.warmup, 1), 3))
    sample = ("one batch element of the step (B=1 of 4, all 32 heads, L=4096) in fp16 through torch CPU SDPA "
              "with expanded K/V and a dense causal mask")
    line = {
        "impl": "reference", "metric": METRIC, "value": tflops, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": min(args.steps, 20), "warmup": min(max(args.warmup, 1), 3), "ms_per_step": sec * 1e3 * PREFILL["batch"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "l2": "n/a (CPU)"},
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------
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
    from minfer.kernels.torch_ext.ops import check_status
    kerns = KernelBackend("torch_ext")
    peaks = load_peaks()
    c = PREFILL
    B, H, Hkv, L, D = c["batch"], c["n_heads"], c["n_kv_heads"], c["seq_len"], c["head_dim"]

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

    # End-to-end leg: every step copies its inputs from pinned host memory, runs the call and reads the result
    # back.  Copies and kernels of consecutive steps overlap the way a serving loop would overlap them: an
    # upload stream, the stream the library launches on, and a download stream, over two sets of device buffers.
    # Every step's three uploads, its launch and its download are inside the timed region.
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

    # ---- device-resident timing ----
    for _ in range(max(args.warmup, 3)):
        step()
    check_status(dev)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    barrier(world)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    barrier(world)
    ms = max_over_ranks(e0.elapsed_time(e1), world, dev) / args.steps
    clocks = sampler.stop() if rank == 0 else None
    check_status(dev)

    # ---- end-to-end timing (host buffers) ----
    e2e_steps = min(args.steps, 100)  # each step moves 336 MB over PCIe; 100 steps are ~0.4 s
    for i in range(4):
        step_e2e(i)
    torch.cuda.synchronize()
    barrier(world)
    e0.record(s_run)
    for i in range(e2e_steps):
        step_e2e(i)
    s_run.wait_stream(s_out)
    s_run.wait_stream(s_in)
    e1.record(s_run)
    torch.cuda.synchronize()
    barrier(world)
    ms_e2e = max_over_ranks(e0.elapsed_time(e1), world, dev) / e2e_steps
    check_status(dev)
    # the same without overlap between steps (one stream), for reference
    for _ in range(2):
        step_e2e_serial()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(min(e2e_steps, 30)):
        step_e2e_serial()
    e1.record()
    torch.cuda.synchronize()
    ms_e2e_serial = max_over_ranks(e0.elapsed_time(e1), world, dev) / min(e2e_steps, 30)

    # ---- decode leg (per GPU; the same shard on every rank) ----
    d = DECODE
    gd = torch.Generator().manual_seed(2)
    lens = torch.randint(d["min_len"], d["max_len"] + 1, (d["batch"],), generator=gd, dtype=torch.int32)
    dq = torch.randn(d["batch"], d["n_heads"], 1, d["head_dim"], device=dev, dtype=torch.float16)
    kc = torch.randn(d["batch"], d["n_kv_heads"], d["max_len"], d["head_dim"], device=dev, dtype=torch.float16)
    vc = torch.randn(d["batch"], d["n_kv_heads"], d["max_len"], d["head_dim"], device=dev, dtype=torch.float16)
    dout = torch.zeros_like(dq)
    dlens = lens.to(dev)
    for _ in range(5):
        kerns.flash_attn_decode(dq, kc, vc, dlens, dout)
    barrier(world)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(args.steps):
        kerns.flash_attn_decode(dq, kc, vc, dlens, dout)
    e1.record()
    torch.cuda.synchronize()
    ms_dec = max_over_ranks(e0.elapsed_time(e1), world, dev) / args.steps
    dec_bytes = 2.0 * 2 * d["n_kv_heads"] * d["head_dim"] * float(lens.sum())  # K and V, 16-bit, live rows only
    dec_gbs = dec_bytes / (ms_dec * 1e-3) / 1e9

    # ---- optional: the output all-gather of the multi-GPU harness ----
    allgather_ms = None
    if world > 1:
        import torch.distributed as dist
        gathered = torch.empty(world * B, H, L, D, dtype=torch.float16, device=dev)
        for _ in range(2):
            dist.all_gather_into_tensor(gathered, out)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(5):
            dist.all_gather_into_tensor(gathered, out)
        e1.record()
        torch.cuda.synchronize()
        allgather_ms = max_over_ranks(e0.elapsed_time(e1), world, dev) / 5
        del gathered

    if rank == 0:
        flops = prefill_flops(c)
        per_gpu_tflops = flops / (ms * 1e-3) / 1e12
        # a timed region of a few hundred ms runs under the 1 kW power cap (clocks settle well below
        # the maximum), so it is compared with the sustained matmul peak; a short burst with the burst peak
        sustained = ms * args.steps > 300.0
        tensor_peak = peaks["tflops_sustained"] if sustained else peaks["tflops"]
        peak_kind = "sustained" if sustained else "burst"
        cpu_tflops, cpu_sec, cores = time_cpu_reference(3, 1)
        traffic = load_traffic()
        line = {
            "metric": METRIC, "value": per_gpu_tflops * world, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "global_batch": B * world,
                       "parallelism": f"dp{world} over batch, no data-path collective",
                       "l2": "inputs+outputs 336 MB per step exceed the 126 MB L2; no explicit flush",
                       "flop_convention": "causal half: 4*B*H*L^2*D/2"},
            "clocks": clocks,
            "e2e": {"value": flops * world / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": in_bytes, "d2h_bytes_per_step": out_bytes, "ms_per_step": ms_e2e,
                    "steps": e2e_steps, "overlap": "uploads, launches and downloads of consecutive steps overlap "
                    "(three streams, two device buffer sets)", "ms_per_step_one_stream": ms_e2e_serial},
            "gpu_launches": args.steps,
            "roofline": {"bound": "tensor", "achieved": per_gpu_tflops, "peak": tensor_peak, "unit": "TFLOP/s",
                         "frac": per_gpu_tflops / tensor_peak, "traffic": traffic.get("prefill"),
                         "peak_source": f"{peaks['source']}, {peak_kind} bf16 matmul figure",
                         "frac_of_nominal_2250": per_gpu_tflops / 2250.0,
                         "kernel": "prefill_persist_kernel<128,f16>"},
            "decode": {"value": dec_gbs * world, "unit": "GB/s", "ms_per_step": ms_dec,
                       "workload": "config3: B=64/GPU Hq=32 Hkv=8 D=128, lens U[512,8192] seed 2, cache padded to 8192",
                       "bytes_per_step": dec_bytes, "gpu_launches_per_step": 2,
                       "roofline": {"bound": "hbm", "achieved": dec_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                    "frac": dec_gbs / peaks["hbm_gbs"], "traffic": traffic.get("decode"),
                                    "frac_of_nominal_8000": dec_gbs / 8000.0,
                                    "kernel": "decode_split_kernel<128,f16> + decode_combine_kernel"}},
            "cpu_baseline": {"value": cpu_tflops, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                             "sample": "B=1 of the step's 4 batch elements, fp16, torch CPU SDPA with expanded K/V "
                                       f"and dense causal mask; {cpu_sec * 1e3:.0f} ms median of 3"},
        }
        if allgather_ms is not None:
            line["allgather_ms"] = allgather_ms
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


def load_traffic():
    """DRAM bytes per launch taken from the committed ncu summaries (profiles/traffic.json), if present."""
    path = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f)
    return {}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
