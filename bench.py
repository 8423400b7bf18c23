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
CUDA events through b200moe_profile_next_gemm1), `cpu_baseline` (the numpy oracle on the
host cores over a bounded sample), `clocks` (nvidia-smi samples during the timed region)
and, at N=1, `sweep`: the 32-local-expert slice at T = 1..16384 with per-T microseconds
and roofline fractions (L2 flushed between iterations).

--impl reference times the CPU oracle port alone (rank 0 only under torchrun).
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
NCU_TRAFFIC = {"per_row": 14858.0, "per_expert": 31.04e6}   # profiles/grouped_gemm_slice8192_zipf2048.md


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
# CPU arm: the oracle port on the host cores, bounded sample
# ----------------------------------------------------------------------------------------

def cpu_sample(tokens, bias, expert_loader, n_experts_total, budget_s, max_experts=None):
    """Runs the oracle port on all tokens of one rank through a sample of the experts and
    extrapolates to the whole layer.  Experts are visited in a fixed scattered order
    (e = 37*i mod 256); dequantisation (a per-expert cost) and the row work (GEMM1, SwiGLU,
    requant, GEMM2, combine: a per-row cost) are timed apart, and the whole-layer time is
    front + per-expert cost * active experts + per-row cost * rows of the full routing.
    Returns (tokens/s, description, experts visited)."""
    from oracle import moe_oracle as O
    logits, hq, hsc = tokens
    T = logits.shape[0]
    t0 = time.perf_counter()
    ids, w, _, _ = O.route(logits.numpy(), bias.float().numpy(), RSF)
    x = O.dequant_rows(hq.view(torch.uint8).numpy(), O.hidden_scale_rows(hsc.numpy(), T, HIDDEN // 128))
    t_front = time.perf_counter() - t0
    counts = O.local_counts(ids, 0, n_experts_total)
    done, rows, t_deq, t_rows = 0, 0, 0.0, 0.0
    out = np.zeros((T, HIDDEN), dtype=np.float32)
    while done < n_experts_total and (t_deq + t_rows < budget_s or done == 0):
        if max_experts is not None and done >= max_experts:
            break
        e = (37 * done) % n_experts_total
        w1q, s1, w2q, s2 = expert_loader(e)
        t1 = time.perf_counter()
        w1 = O.dequant_blocks(w1q, s1)
        w2 = O.dequant_blocks(w2q, s2)
        t2 = time.perf_counter()
        hit = ids == e
        sel = np.nonzero(hit.any(axis=1))[0]
        if sel.size:
            act = O.swiglu(x[sel] @ w1.T)
            q, scale = O.requant_rows(act)
            g2 = (O.e4m3_decode(q) * scale[:, None]).astype(np.float32) @ w2.T
            wk = w[sel, hit[sel].argmax(axis=1)]
            out[sel] = O.round_bf16(out[sel] + O.round_bf16(g2 * wk[:, None]))
            rows += sel.size
        t3 = time.perf_counter()
        t_deq += t2 - t1
        t_rows += t3 - t2
        done += 1
    n_active = int((counts > 0).sum())
    est = t_front + t_deq / max(done, 1) * n_active + t_rows / max(rows, 1) * int(counts.sum())
    desc = (f"all {T} tokens of one rank through {done} of {n_experts_total} experts (scattered ids, {rows} of "
            f"{int(counts.sum())} expert rows, {t_front + t_deq + t_rows:.1f} s of CPU work); whole layer = front "
            f"{t_front:.2f} s + {t_deq / max(done, 1):.3f} s/expert x {n_active} + "
            f"{1e3 * t_rows / max(rows, 1):.3f} ms/row x {int(counts.sum())}")
    return T / est, desc, done


def make_expert_loader_cpu():
    from fused_moe_b200 import synth

    def load(e):
        q1, s1, q2, s2 = synth.make_expert(e, 0)
        return (q1.view(torch.uint8).numpy(), s1.numpy(), q2.view(torch.uint8).numpy(), s2.numpy())
    return load


def run_reference_arm(args):
    from fused_moe_b200 import synth
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    tokens = synth.make_tokens(TOKENS_PER_RANK, 0, 0)
    bias = synth.make_bias(0)
    loader = make_expert_loader_cpu()
    cache = {}

    def cached(e):
        if e not in cache:
            cache[e] = loader(e)
        return cache[e]
    # calibrate on one expert, then size a step so that the whole run stays within a few minutes
    t0 = time.perf_counter()
    cpu_sample(tokens, bias, cached, 256, 0.0, max_experts=1)
    one = time.perf_counter() - t0
    per_step_budget = max(2.0, min(20.0, 150.0 / max(args.steps + args.warmup, 1)))
    n_exp = int(max(1, min(256, per_step_budget / max(one, 1e-3))))
    for i in range(n_exp):
        cached((37 * i) % 256)
    vals, desc = [], ""
    for i in range(args.warmup + args.steps):
        v, desc, _ = cpu_sample(tokens, bias, cached, 256, 1e9, max_experts=n_exp)
        if i >= args.warmup:
            vals.append(v)
    value = statistics.median(vals)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1000.0 * TOKENS_PER_RANK / value,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic (seeded generators, contest shapes)",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": desc},
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
    ws = kernel.get_workspace(dev, ep.last_recv_rows if ep else TOKENS_PER_RANK, e_local, HIDDEN, INTER)
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

    if ep is not None and os.environ.get("B200MOE_EP_TRACE"):   # phase breakdown of one step, every rank, to stderr
        out = step(logits, hq, hsc)
        print(f"[rank {rank}] ep phases ms: " + json.dumps({k: round(v, 3) for k, v in ep.phase_ms().items()}) +
              f" recv_rows {ep.last_recv_rows}", file=sys.stderr, flush=True)
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

    def e2e_step(i):
        k = i & 1
        s_in.wait_event(ev_done[k])                 # the kernels that read this input slot are done
        with torch.cuda.stream(s_in):
            for d, h in zip(d_in[k], host):
                d.copy_(h, non_blocking=True)
            ev_in[k].record(s_in)
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

    for i in range(4):
        e2e_step(i)
    barrier()
    t0 = time.perf_counter()
    for i in range(args.steps):
        e2e_step(i)
    barrier()
    e2e_s = time.perf_counter() - t0
    # clock samples from the start of the device-timed region to the end of the end-to-end loop
    # (all of it is the same step under load; the timed region alone can be shorter than one sample)
    clocks = sampler.stop(t_wall0, time.time())
    clocks["window"] = "timed steps + GEMM1 timing + end-to-end steps"

    times = torch.tensor([ms_total, e2e_s * 1000.0, g1_avg_ms, float(m_local), float(n_active)],
                         dtype=torch.float64, device=dev)
    if world > 1:
        gathered = [torch.zeros_like(times) for _ in range(world)]
        dist.all_gather(gathered, times)
        allt = torch.stack(gathered).cpu().numpy()
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
        "ep_exchange": (ep.last_mode if ep is not None else None),
    }

    if world == 1 and not args.no_sweep:
        line["sweep"] = sweep(kernel, synth, dev, bias, (w1, s1, w2, s2), peaks)
    if world == 1 and not args.no_cpu:
        cores = os.cpu_count() or 1
        torch.set_num_threads(cores)

        def gpu_loader(e):
            u8 = lambda t: t.view(torch.uint8).cpu().numpy()
            return u8(w1[e]), s1[e].cpu().numpy(), u8(w2[e]), s2[e].cpu().numpy()
        v, desc, _ = cpu_sample((logits_c, hq_c, hsc_c), bias.cpu(), gpu_loader, 256, args.cpu_budget)
        line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": cores, "kind": "port", "sample": desc}
    elif not args.no_cpu:
        line["cpu_baseline"] = None
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def sweep(kernel, synth, dev, bias, weights, peaks):
    """32-local-expert slice (experts 0..31) at the decode and prefill token counts."""
    w1, s1, w2, s2 = (t[:32] for t in weights)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    fp8_peak = 2.0 * peaks["bf16_tflops"]
    rows = []
    for T, tseed in ((1, 2), (4, 1), (16, 0), (64, 0), (1024, 0), (4096, 0), (16384, 0)):
        lg, hq, hsc = (t.to(dev) for t in synth.make_tokens(T, 0, tseed))
        for _ in range(3):
            kernel.custom_kernel(lg, bias, hq, hsc, w1, s1, w2, s2, 0, RSF)
        torch.cuda.synchronize()
        ws = kernel.get_workspace(dev, T, 32, HIDDEN, INTER)
        meta = ws.view("meta", torch.int32, (8,)).cpu().numpy()
        counts = ws.view("expert_count", torch.int32, (32,)).cpu().numpy()
        m_local, n_active = int(meta[2]), int((counts > 0).sum())
        ts = []
        for _ in range(10):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            kernel.custom_kernel(lg, bias, hq, hsc, w1, s1, w2, s2, 0, RSF)
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        us = statistics.median(ts) * 1000.0
        nbytes = synth.algorithmic_bytes(T, n_active)
        flops = synth.algorithmic_flops(m_local)
        rows.append({"T": T, "token_seed": tseed, "us": us, "tokens_per_s": T / (us * 1e-6), "rows": m_local,
                     "active_experts": n_active,
                     "hbm_gbs": nbytes / (us * 1e-6) / 1e9, "hbm_frac": nbytes / (us * 1e-6) / 1e9 / peaks["hbm_gbs"],
                     "fp8_tflops": flops / (us * 1e-6) / 1e12, "fp8_frac": flops / (us * 1e-6) / 1e12 / fp8_peak,
                     "bound": "hbm" if nbytes / (peaks["hbm_gbs"] * 1e9) >= flops / (fp8_peak * 1e12) else "tensor"})
    return rows


def run_profile_case(args):
    """A small single-GPU case for profilers: the 32-local-expert slice at --tokens tokens,
    W warm-up calls and K timed calls, nothing else (no sweep, no CPU arm, no end-to-end leg).
    Prints a JSON line that is NOT a benchmark value (it is meant to run under ncu)."""
    from fused_moe_b200 import kernel, synth
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    w = synth.make_weights(32, 0, 0, HIDDEN, INTER, device=dev, fast_device_rng=True)
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
    ws = kernel.get_workspace(dev, args.tokens, 32, HIDDEN, INTER)
    code, detail = ws.read_status(0)
    meta = ws.view("meta", torch.int32, (8,)).cpu().numpy()
    counts = ws.view("expert_count", torch.int32, (32,)).cpu().numpy()
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
    print(json.dumps({"profile_case": "slice32", "tokens": args.tokens, "zipf": args.zipf, "status": code,
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
    ap.add_argument("--cpu-budget", type=float, default=15.0, help="seconds of oracle work for cpu_baseline")
    ap.add_argument("--profile-case", action="store_true",
                    help="small single-GPU slice case for ncu (see run_profile_case); not a benchmark")
    ap.add_argument("--tokens", type=int, default=8192, help="tokens of --profile-case")
    ap.add_argument("--zipf", action="store_true", help="Zipf routing bias for --profile-case")
    args = ap.parse_args()
    if args.profile_case:
        run_profile_case(args)
    elif args.impl == "reference":
        run_reference_arm(args)
    else:
        run_b200_arm(args)


if __name__ == "__main__":
    main()
