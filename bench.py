#!/usr/bin/env python
"""Benchmark of the fused FP8 MoE layer (one JSON line on stdout).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--no-sweep]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload (every N): the full 256-expert DeepSeek-V3-shape layer, expert-parallel over N
GPUs (256/N experts per GPU), 4096 tokens per rank per step, seeded synthetic data.  A
step is one layer call on every rank.  `value` = tokens of all ranks per second, device
timed (CUDA events, barrier + synchronize on both sides, max over ranks) with the step's
inputs already in HBM.  `e2e` = the same through the host entry point with the step's
tokens in pinned host memory and the bf16 result copied back, inside the timed region
(expert weights are model state and stay resident); uploads and downloads of neighbouring
steps overlap the kernels of the current one (two slots, two copy streams).

Extra objects on the line: `roofline` (GEMM1, the dominant kernel, timed in place with
CUDA events through b200moe_profile_next_gemm1), `cpu_baseline` (the reference's torch function
on the host cores over a bounded sample), `clocks` (nvidia-smi samples during the timed region)
and, at N=1, `sweep`: the 32-local-expert slice at T = 1..16384 with per-T microseconds
and roofline fractions (L2 flushed between iterations).

--impl reference times the reference project's own torch function on the host cores alone
(rank 0 only under torchrun), one 32-expert slice of the layer per step.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch  # noqa: E402

TOKENS_PER_RANK = 4096
HIDDEN, INTER = 7168, 2048
RSF = 2.5
METRIC = "moe_layer_tokens_per_s"
UNIT = "tokens/s"

# DRAM traffic of one GEMM1 launch per packed row and per active expert, from the ncu
# capture summarised under profiles/ (None until a capture exists).
NCU_TRAFFIC = {"per_row": 14812.0, "per_expert": 31.02e6}   # profiles/grouped_gemm_slice8192_zipf2048.md


def bind_to_gpu_numa_node(local_rank: int):
    """Runs this process on the CPUs of the NUMA node its GPU hangs off, BEFORE any pinned buffer is
    allocated (pages are placed on the node of the thread that first touches them): with eight ranks
    copying ~90 MB per step each, buffers that all sit on node 0 send half of the traffic across the
    socket link.  Returns the node, or None where the topology cannot be read."""
    try:
        bus = torch.cuda.get_device_properties(local_rank).pci_bus_id
        dom = torch.cuda.get_device_properties(local_rank).pci_domain_id
        dev_id = torch.cuda.get_device_properties(local_rank).pci_device_id
        path = f"/sys/bus/pci/devices/{dom:04x}:{bus:02x}:{dev_id:02x}.0/numa_node"
        with open(path) as fh:
            node = int(fh.read().strip())
        if node < 0:
            return None
        with open(f"/sys/devices/system/node/node{node}/cpulist") as fh:
            cpus = set()
            for part in fh.read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = os.sched_getaffinity(0)
        use = cpus & allowed
        if use:
            os.sched_setaffinity(0, use)
            return node
    except (OSError, ValueError, AttributeError):
        pass
    return None


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as fh:
            p = json.load(fh)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clock/throttle samples while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.lines = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0: float, t1: float):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for ts, line in self.lines:
            if ts < t0 - 0.05 or ts > t1 + 0.15:
                continue
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                 f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ----------------------------------------------------------------------------------------
# CPU arm: the reference's own torch function on the host cores, one 32-expert slice per step
# ----------------------------------------------------------------------------------------
SLICE_EXPERTS = 32
N_SLICES = 256 // SLICE_EXPERTS


def host_threads() -> int:
    """All host cores for torch's intra-op pool, whatever OMP_NUM_THREADS the launcher exported
    (torch.distributed.run sets it to 1); returns the thread count actually in use."""
    torch.set_num_threads(os.cpu_count() or 1)
    return torch.get_num_threads()


def load_cpu_function():
    """(callable with the ten reference arguments -> bf16 [T, hidden], kind).  kind "reference":
    the reference project's own `_reference_impl` (from its checkout, or the copy that
    oracle/make_ref.py extracted into oracle/_ref/); kind "port": the numpy/torch restatement."""
    from oracle import ref_loader
    if ref_loader.available():
        return ref_loader.load_reference_impl(), "reference", ref_loader.source()
    from oracle import moe_oracle

    def port(*args):
        return moe_oracle.moe_layer_torch(*args)["out"]
    return port, "port", "oracle/moe_oracle.py"


def cpu_slice_seconds(fn, tokens, bias, weights, slice_idx):
    """One call of the CPU function: all tokens of one rank, experts [32 s, 32 s + 32)."""
    logits, hq, hsc = tokens
    t0 = time.perf_counter()
    fn(logits, bias, hq, hsc, *weights, SLICE_EXPERTS * slice_idx, RSF)
    return time.perf_counter() - t0


def cpu_sample_text(kind, src, n_calls, secs, same_weights):
    return (f"each step = the {'reference project' if kind == 'reference' else 'port'}'s torch function "
            f"({src}) on all {TOKENS_PER_RANK} tokens of rank 0 for one 32-expert slice "
            f"(local_expert_offset = 32 * (step mod 8)); 8 consecutive steps cover every (token, expert) pair of "
            f"the 256-expert layer once, so tokens/s = {TOKENS_PER_RANK} / (8 * mean step time); {n_calls} slice "
            f"calls timed, {secs:.1f} s of CPU work"
            + ("; the slices reuse one set of 32 experts' weight bytes (routing, rows and shapes are each "
               "slice's own)" if same_weights else ""))


def run_reference_arm(args):
    from fused_moe_b200 import synth
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = host_threads()
    fn, kind, src = load_cpu_function()
    tokens = synth.make_tokens(TOKENS_PER_RANK, 0, 0)
    bias = synth.make_bias(0)
    weights = synth.make_weights(SLICE_EXPERTS, 0, 0)   # ~20 s; reused by every slice (timing only)
    times = []
    for i in range(args.warmup + args.steps):
        t = cpu_slice_seconds(fn, tokens, bias, weights, i % N_SLICES)
        if i >= args.warmup:
            times.append(t)
    mean_s = statistics.mean(times)
    value = TOKENS_PER_RANK / (N_SLICES * mean_s)
    whole = sum(times[:N_SLICES]) if len(times) >= N_SLICES else None
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1000.0 * mean_s,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic (seeded generators, contest shapes)",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind,
                         "sample": cpu_sample_text(kind, src, len(times), sum(times), True),
                         "whole_pass_s_measured": whole, "whole_pass_s_from_mean": N_SLICES * mean_s},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(n_gpus):
    return {"workload": f"DeepSeek-V3-shape FP8 block-scale MoE layer, 256 experts expert-parallel over {n_gpus} "
                        f"GPU(s) ({256 // n_gpus} experts/GPU), {TOKENS_PER_RANK} tokens per rank per step",
            "tokens_per_rank": TOKENS_PER_RANK, "experts_per_gpu": 256 // n_gpus, "hidden": HIDDEN,
            "intermediate": INTER, "top_k": 8, "routed_scaling_factor": RSF,
            "l2_policy": "inputs larger than L2 (>= 1.4 GB of expert weights read per step); "
                         "sweep rows flush L2 between iterations",
            "parallelism": f"ep{n_gpus}"}


# ----------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------

def run_b200_arm(args):
    import torch.distributed as dist
    from fused_moe_b200 import _capi, kernel, synth
    from fused_moe_b200.ep import ExpertParallelMoE

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run for --gpus > 1")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    numa_node = bind_to_gpu_numa_node(local_rank) if world > 1 else None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    peaks = load_peaks()
    lib = _capi.lib()

    e_local = 256 // world
    local_off = rank * e_local
    w1, s1, w2, s2 = synth.make_weights(e_local, local_off, 0, HIDDEN, INTER, device=dev, fast_device_rng=True)
    logits_c, hq_c, hsc_c = synth.make_tokens(TOKENS_PER_RANK, rank, 0)
    bias = synth.make_bias(0).to(dev)
    host = [t.pin_memory() for t in (logits_c, hq_c.view(torch.uint8), hsc_c)]
    logits, hq, hsc = (t.to(dev) for t in (logits_c, hq_c, hsc_c))
    ep = ExpertParallelMoE() if world > 1 else None

    def step(lg, h, sc):
        if ep is not None:
            return ep.forward(lg, bias, h, sc, w1, s1, w2, s2, RSF)
        return kernel.custom_kernel(lg, bias, h, sc, w1, s1, w2, s2, 0, RSF)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        out = step(logits, hq, hsc)
    barrier()
    ws = kernel.get_workspace(dev, ep.last_ws_rows if ep else TOKENS_PER_RANK, e_local, HIDDEN, INTER)
    code, detail = ws.read_status(torch.cuda.current_stream().cuda_stream)
    if code != 0:
        raise SystemExit(f"device status {code} {detail} after warm-up")
    meta = ws.view("meta", torch.int32, (8,)).cpu().numpy()
    counts = ws.view("expert_count", torch.int32, (e_local,)).cpu().numpy()
    m_local, n_active = int(meta[2]), int((counts > 0).sum())

    # ---- timed region: K steps, device timed, GEMM1 timed in place
    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(0.3)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t_wall0 = time.time()
    ev0.record()
    for i in range(args.steps):
        out = step(logits, hq, hsc)
    ev1.record()
    barrier()
    t_wall1 = time.time()
    ms_total = ev0.elapsed_time(ev1)

    phases = None
    if ep is not None:   # phase breakdown of one extra step (CUDA events at the phase boundaries), every rank
        ep._trace = True
        out = step(logits, hq, hsc)
        phases = {k: round(v, 3) for k, v in ep.phase_ms().items()}
        ep._trace = False
        ep._marks = []
        barrier()

    # GEMM1 in place (separate short loop so that event creation stays out of the headline region)
    g1_ms = []
    for i in range(min(args.steps, 10)):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()   # materialises the underlying cudaEvent_t
        b.record()
        lib.b200moe_profile_next_gemm1(a.cuda_event, b.cuda_event)
        out = step(logits, hq, hsc)
        torch.cuda.synchronize()
        g1_ms.append(a.elapsed_time(b))
    g1_avg_ms = statistics.mean(g1_ms)

    # ---- end to end: pinned host inputs in, bf16 result out, every step
    # Two slots of device inputs / outputs and two copy streams: step i+1's upload and step
    # i-1's download run under step i's kernels, as a serving loop would pipeline them.  Every
    # step still uploads its own inputs from pinned memory and downloads its own result.
    out_host = [torch.empty((TOKENS_PER_RANK, HIDDEN), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    d_in = [[torch.empty_like(t, device=dev) for t in host] for _ in range(2)]
    d_out = [torch.empty((TOKENS_PER_RANK, HIDDEN), dtype=torch.bfloat16, device=dev) for _ in range(2)]
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    cur = torch.cuda.current_stream(dev)
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_done = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]
    for e in ev_done + ev_out:
        e.record(cur)

    def upload(i):
        k = i & 1
        s_in.wait_event(ev_done[k])                 # the kernels that read this input slot are done
        with torch.cuda.stream(s_in):
            for d, h in zip(d_in[k], host):
                d.copy_(h, non_blocking=True)
            ev_in[k].record(s_in)

    def compute_and_download(i):
        k = i & 1
        cur.wait_event(ev_in[k])
        cur.wait_event(ev_out[k])                   # the download that read this output slot is done
        if ep is not None:
            o = step(d_in[k][0], d_in[k][1].view(torch.float8_e4m3fn), d_in[k][2])
            o.record_stream(s_out)
        else:
            o = kernel.custom_kernel(d_in[k][0], bias, d_in[k][1].view(torch.float8_e4m3fn), d_in[k][2],
                                     w1, s1, w2, s2, 0, RSF, out=d_out[k])
        ev_done[k].record(cur)
        s_out.wait_event(ev_done[k])
        with torch.cuda.stream(s_out):
            out_host[k].copy_(o, non_blocking=True)
            ev_out[k].record(s_out)

    # Step i+1's upload is enqueued BEFORE step i's layer call: the expert-parallel call reads the row counts
    # on the host in its middle, and an upload enqueued behind it would start that much later.
    upload(0)
    for i in range(4):
        upload(i + 1)
        compute_and_download(i)
    barrier()
    t0 = time.perf_counter()
    for i in range(4, 4 + args.steps):
        upload(i + 1)
        compute_and_download(i)
    barrier()
    e2e_s = time.perf_counter() - t0
    # clock samples from the start of the device-timed region to the end of the end-to-end loop
    # (all of it is the same step under load; the timed region alone can be shorter than one sample)
    clocks = sampler.stop(t_wall0, time.time())
    clocks["window"] = "timed steps + GEMM1 timing + end-to-end steps"

    times = torch.tensor([ms_total, e2e_s * 1000.0, g1_avg_ms, float(m_local), float(n_active)],
                         dtype=torch.float64, device=dev)
    all_phases = None
    if world > 1:
        gathered = [torch.zeros_like(times) for _ in range(world)]
        dist.all_gather(gathered, times)
        allt = torch.stack(gathered).cpu().numpy()
        all_phases = [None] * world
        dist.all_gather_object(all_phases, {"rank": rank, "numa_node": numa_node, "phases_ms": phases})
    else:
        allt = times.cpu().numpy()[None]
    ms_total_max = float(allt[:, 0].max())
    e2e_ms_max = float(allt[:, 1].max())
    slow = int(allt[:, 2].argmax())            # roofline of the rank whose GEMM1 is slowest
    g1_ms_r, m_r, act_r = float(allt[slow, 2]), int(allt[slow, 3]), int(allt[slow, 4])

    total_tokens = TOKENS_PER_RANK * world
    ms_per_step = ms_total_max / args.steps
    value = total_tokens / (ms_per_step / 1000.0)
    e2e_value = total_tokens * args.steps / (e2e_ms_max / 1000.0)

    g1_bytes = synth.gemm1_bytes(m_r, act_r)
    g1_flops = synth.gemm1_flops(m_r)
    fp8_peak_tf = 2.0 * peaks["bf16_tflops_sustained"]
    t_hbm = g1_bytes / (peaks["hbm_gbs"] * 1e9)
    t_tc = g1_flops / (fp8_peak_tf * 1e12)
    if t_hbm >= t_tc:
        roof = {"bound": "hbm", "achieved": g1_bytes / (g1_ms_r * 1e-3) / 1e9, "peak": peaks["hbm_gbs"],
                "unit": "GB/s"}
    else:
        roof = {"bound": "tensor", "achieved": g1_flops / (g1_ms_r * 1e-3) / 1e12, "peak": fp8_peak_tf,
                "unit": "TFLOP/s"}
    roof["frac"] = roof["achieved"] / roof["peak"]
    roof.update({"kernel": "grouped_gemm_kernel<1,*> (GEMM1 + SwiGLU)", "launch_ms": g1_ms_r,
                 "rows": m_r, "active_experts": act_r, "algorithmic_bytes": g1_bytes,
                 "algorithmic_flops": g1_flops, "peak_source": peaks["source"] +
                 (" HBM copy" if roof["bound"] == "hbm" else " cuBLAS bf16 (sustained) x2 for dense e4m3"),
                 "traffic": (NCU_TRAFFIC["per_row"] * m_r + NCU_TRAFFIC["per_expert"] * act_r)
                 if NCU_TRAFFIC else None})

    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    h2d = sum(t.numel() * t.element_size() for t in host)
    d2h = out_host[0].numel() * out_host[0].element_size()
    # N > 1: route, plan + copy (pack), count, the 7 kernels of the local expert pipeline, combine;
    # with the exchanges read from mapped peer memory one more (the ids pull)
    launches_per_step = kernel.launches_per_run(TOKENS_PER_RANK, e_local) if world == 1 else \
        (13 if ep.last_mode == "peer" else 12)
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp8_e4m3 (fp32 block scales, fp32 accumulate, bf16 out)",
        "data": "synthetic (seeded generators, contest shapes)",
        "config": workload_config(world),
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d * world,
                "d2h_bytes_per_step": d2h * world},
        "gpu_launches": launches_per_step * args.steps,
        "roofline": roof, "clocks": clocks,
        "rows_per_rank": [int(x) for x in allt[:, 3]],
        "ep_phases": all_phases,
        "ep_exchange": (ep.last_mode if ep is not None else None),
    }

    if world == 1 and not args.no_sweep:
        cpu_fn = None
        if not args.no_cpu:
            host_threads()
            cpu_fn = load_cpu_function()[0]
        line["sweep"] = sweep(kernel, synth, dev, bias, (w1, s1, w2, s2), peaks, cpu_fn)
    if world == 1 and not args.no_yardstick:
        del out
        torch.cuda.empty_cache()
        line["yardstick"] = run_yardstick()
    if world == 1 and not args.no_cpu:
        cores = host_threads()
        fn, kind, src = load_cpu_function()
        times, sl = [], 0
        while sl < N_SLICES and (sum(times) < args.cpu_budget or not times):
            wsl = tuple(t[sl * SLICE_EXPERTS:(sl + 1) * SLICE_EXPERTS].cpu() for t in (w1, s1, w2, s2))
            times.append(cpu_slice_seconds(fn, (logits_c, hq_c, hsc_c), bias.cpu(), wsl, sl))
            sl += 1
        v = TOKENS_PER_RANK / (N_SLICES * statistics.mean(times))
        line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": cores, "kind": kind,
                                "sample": cpu_sample_text(kind, src, len(times), sum(times), False)}
    elif not args.no_cpu:
        line["cpu_baseline"] = None
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# (tokens, token seed, Zipf bias): BASELINE configs 1 (T = 8), 2 (decode, two token seeds per T that give
# at least one local row where such a seed exists), 3 (prefill) and 5 (Zipf load imbalance, T = 2048)
SWEEP_CASES = ((1, 2, False), (1, 1, False), (4, 1, False), (4, 2, False), (8, 0, False), (16, 0, False),
               (16, 1, False), (64, 0, False), (64, 1, False), (1024, 0, False), (4096, 0, False),
               (16384, 0, False), (2048, 0, True))


def sweep(kernel, synth, dev, bias, weights, peaks, cpu_fn=None):
    """32-local-expert slice (experts 0..31) at the decode, prefill and Zipf token counts; with `cpu_fn`
    (the reference's torch function) each row also carries its CPU time on the host cores."""
    w1, s1, w2, s2 = (t[:32] for t in weights)
    w_cpu = tuple(t.cpu() for t in (w1, s1, w2, s2)) if cpu_fn is not None else None
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    fp8_peak = 2.0 * peaks["bf16_tflops"]
    rows = []
    for T, tseed, zipf in SWEEP_CASES:
        lg_c, hq_c, hsc_c = synth.make_tokens(T, 0, tseed)
        lg, hq, hsc = (t.to(dev) for t in (lg_c, hq_c, hsc_c))
        b = synth.make_bias(0, zipf=True).to(dev) if zipf else bias
        for _ in range(3):
            kernel.custom_kernel(lg, b, hq, hsc, w1, s1, w2, s2, 0, RSF)
        torch.cuda.synchronize()
        ws = kernel.get_workspace(dev, T, 32, HIDDEN, INTER)
        meta = ws.view("meta", torch.int32, (8,)).cpu().numpy()
        counts = ws.view("expert_count", torch.int32, (32,)).cpu().numpy()
        m_local, n_active = int(meta[2]), int((counts > 0).sum())
        ts = []
        for _ in range(10):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            kernel.custom_kernel(lg, b, hq, hsc, w1, s1, w2, s2, 0, RSF)
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        us = statistics.median(ts) * 1000.0
        nbytes = synth.algorithmic_bytes(T, n_active)
        flops = synth.algorithmic_flops(m_local)
        row = {"T": T, "token_seed": tseed, "zipf": zipf, "us": us, "tokens_per_s": T / (us * 1e-6),
               "rows": m_local, "active_experts": n_active,
               "hbm_gbs": nbytes / (us * 1e-6) / 1e9, "hbm_frac": nbytes / (us * 1e-6) / 1e9 / peaks["hbm_gbs"],
               "fp8_tflops": flops / (us * 1e-6) / 1e12, "fp8_frac": flops / (us * 1e-6) / 1e12 / fp8_peak,
               "bound": "hbm" if nbytes / (peaks["hbm_gbs"] * 1e9) >= flops / (fp8_peak * 1e12) else "tensor"}
        if cpu_fn is not None:
            t0 = time.perf_counter()
            cpu_fn(lg_c, b.cpu(), hq_c, hsc_c, *w_cpu, 0, RSF)
            row["cpu_s"] = time.perf_counter() - t0
        rows.append(row)
    return rows


def run_yardstick():
    """The reference's own CUDA solution on the same GPU and inputs (baseline/run_ref.py, in a child
    process so that a failure there cannot take this process down).  Single-GPU runs only."""
    script = os.path.join(ROOT, "baseline", "run_ref.py")
    if not os.path.isfile(script) or not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "build")):
        return {"unavailable": "baseline/_ref (the reference's built CUDA solution) is not present"}
    try:
        r = subprocess.run([sys.executable, script], capture_output=True, text=True, timeout=420, cwd=ROOT)
    except subprocess.TimeoutExpired:
        return {"unavailable": "baseline/run_ref.py did not finish within 420 s"}
    lines = [l for l in r.stdout.strip().splitlines() if l.startswith("{")]
    if r.returncode != 0 or not lines:
        return {"unavailable": f"baseline/run_ref.py exited {r.returncode}: {(r.stderr or r.stdout)[-300:]}"}
    return json.loads(lines[-1])


def run_profile_case(args):
    """A small single-GPU case for profilers: the 32-local-expert slice at --tokens tokens,
    W warm-up calls and K timed calls, nothing else (no sweep, no CPU arm, no end-to-end leg).
    Prints a JSON line that is NOT a benchmark value (it is meant to run under ncu)."""
    from fused_moe_b200 import kernel, synth
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    E = args.experts
    w = synth.make_weights(E, 0, 0, HIDDEN, INTER, device=dev, fast_device_rng=True)
    lg, hq, hsc = (t.to(dev) for t in synth.make_tokens(args.tokens, 0, 0))
    bias = synth.make_bias(0, zipf=args.zipf).to(dev)
    for _ in range(args.warmup):
        kernel.custom_kernel(lg, bias, hq, hsc, *w, 0, RSF)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(args.steps):
        kernel.custom_kernel(lg, bias, hq, hsc, *w, 0, RSF, check_status=False)
    b.record()
    torch.cuda.synchronize()
    ws = kernel.get_workspace(dev, args.tokens, E, HIDDEN, INTER)
    code, detail = ws.read_status(0)
    meta = ws.view("meta", torch.int32, (8,)).cpu().numpy()
    counts = ws.view("expert_count", torch.int32, (E,)).cpu().numpy()
    prof = None
    if os.environ.get("B200MOE_PROF"):
        raw = ws.view("meta", torch.int64, (32,)).cpu().numpy()      # meta + its padding, as u64 words
        names = ("wait_acc", "promote", "mma_issue", "kblocks", "epi_role_total", "tile_epilogues", "unused2",
                 "mma_wait_epilogue", "mma_wait_tma")
        if args.tokens <= 16 and os.environ.get("B200MOE_DECODE", "") != "0":   # the decode kernels' counters
            names = ("prod_wait_stage", "prod_issue", "prod_total", "kblocks", "mma_wait_acc", "mma_wait_tma",
                     "mma_issue", "promo_wait_acc", "promo_total")
        prof = {"gemm1": dict(zip(names, (int(x) for x in raw[4:13]))),
                "gemm2": dict(zip(names, (int(x) for x in raw[17:26])))}
        # eight cycle stamps per K block of CTA 0: issuer wait start, operands landed, accumulator free,
        # MMAs issued; promotion warp 0: accumulator ready, first chunks read, accumulator released, done
        tr = ws.view("trace", torch.int64, (2, 64, 8)).cpu().numpy()
        for name, t in (("gemm1", tr[0]), ("gemm2", tr[1])) if args.tokens > 16 else ():
            base = int(t[8, 0])
            prof[name]["trace_kb8_31"] = [[int(x) - base for x in t[i]] for i in range(8, 32)]
    print(json.dumps({"profile_case": f"slice{E}", "tokens": args.tokens, "zipf": args.zipf, "status": code,
                      "cycle_counters_cta0": prof,
                      "ms_per_call": a.elapsed_time(b) / max(args.steps, 1), "rows": int(meta[2]),
                      "padded_rows": int(meta[1]), "active_experts": int((counts > 0).sum())}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-sweep", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-yardstick", action="store_true",
                    help="skip timing the reference's own CUDA solution (baseline/_ref) beside this library")
    ap.add_argument("--cpu-budget", type=float, default=15.0, help="seconds of oracle work for cpu_baseline")
    ap.add_argument("--profile-case", action="store_true",
                    help="small single-GPU slice case for ncu (see run_profile_case); not a benchmark")
    ap.add_argument("--tokens", type=int, default=8192, help="tokens of --profile-case")
    ap.add_argument("--zipf", action="store_true", help="Zipf routing bias for --profile-case")
    ap.add_argument("--experts", type=int, default=32, choices=[32, 64, 128, 256],
                    help="local experts of --profile-case (experts [0, E) of the 256)")
    args = ap.parse_args()
    if args.profile_case:
        run_profile_case(args)
    elif args.impl == "reference":
        run_reference_arm(args)
    else:
        run_b200_arm(args)


if __name__ == "__main__":
    main()
