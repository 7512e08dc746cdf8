#!/usr/bin/env python
"""Benchmark of the chunked gated-delta-rule (GDN) hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload c2|c3|c5|decode|c2s|c3s] [--lean]

One "step" = one pass of the hot path over one synthetic batch.  The default workload (``c2``) is the
configuration the headline metric is quoted on: single-GPU forward prefill, B=1, T=32768, H_q=H_v=64, K=V=128,
bf16 q/k/v, fp32 gates.  The metric names the forward AND forward+backward, so the same JSON line carries
``fwd_bwd``: the training configuration ``c3`` (B=4, T=8192, H_q=16, H_v=32) through the differentiable operator.

Prints ONE JSON line (rank 0).
* ``value`` - forward tokens/s, device-timed (CUDA events around the K steps, max over ranks), through the public
  operator as a prefill caller uses it (``chunk_gated_delta_rule`` without gradients; the inverse A, which only the
  backward reads, is then not stored).  ``fwd_stage_api`` is the same through ``chunk_gated_delta_rule_fwd`` (the
  function the reference's benchmark times; its return tuple contains A, so A is stored).
* ``roofline`` - the dominant kernel (``gdr_fwd_kernel``), plus ``step_frac`` for the whole step and one block per
  further kernel under ``kernels``.  Kernel times are CUDA-event pairs around every C-ABI launch, recorded inside the
  timed region.
* ``e2e`` - the same metric through the public operator with HOST (pinned) buffers, host<->device copies inside the
  timed region.
* ``cpu_baseline`` - the reference's CPU path (the PyTorch oracle port under oracle/) on the box's host cores.
* under torchrun (N > 1) every rank runs the same workload on its own GPU for ``value`` (the path shards by
  batch x head with no collective: weak scaling), and ``multi_gpu`` adds the two configurations that divide ONE
  problem over the N GPUs (strong scaling): ``c5`` (one 1M-token sequence, sequence parallel with an all_gather of
  per-rank state summaries) and ``c3_sharded`` (config 3's 64 (batch, QK-head group) units split over the ranks).

``--impl reference`` times the reference's CPU implementation of the path (oracle port, all host threads) on a
bounded sample of the same workload, full head count.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    "c2": dict(B=1, T=32768, Hq=64, Hv=64, bwd=False,
               desc="fwd prefill B=1 T=32768 Hq=Hv=64 K=V=128 bf16, g=logsigmoid(randn) fp32, h0=zeros"),
    "c2s": dict(B=1, T=16384, Hq=32, Hv=32, bwd=False, lean=True,
                desc="(profiling case) fwd B=1 T=16384 Hq=Hv=32 K=V=128 bf16"),
    "c5": dict(B=1, T=1048576, Hq=8, Hv=8, bwd=True, seq_parallel=True,
               desc="fwd+bwd B=1 T=1048576 Hq=Hv=8 K=V=128 bf16, ONE sequence split contiguously over the GPUs"),
    "c3": dict(B=4, T=8192, Hq=16, Hv=32, bwd=True,
               desc="fwd+bwd B=4 T=8192 Hq=16 Hv=32 K=V=128 bf16, h0=0.1 randn, dht=0.01 randn"),
    "c3s": dict(B=2, T=8192, Hq=8, Hv=16, bwd=True, lean=True,
                desc="(profiling case) fwd+bwd B=2 T=8192 Hq=8 Hv=16 K=V=128 bf16"),
    # decode side of the path: one new token for each of N sequences, state resident on the device
    "decode": dict(B=256, T=1, Hq=64, Hv=64, bwd=False, decode=True, tokens_per_step=64,
                   desc="decode: 64 consecutive tokens for each of 256 sequences (one kernel call per token), Hq=Hv=64 "
                        "K=V=128, fp32 state 1 GiB resident in HBM"),
}
# Algorithmic work per unit = one (chunk, V-head), at Hq == Hv (q, k bytes divide by Hv/Hq otherwise):
#   forward: q, k, v read + o write (4 x 16 KiB) + g, beta (2 x 256 B); 10.49 MFLOP in the 7 products
#   backward: q, k, v, do read + dq, dk, dv write (7 x 16 KiB) + g, beta, dg, dbeta (4 x 256 B); 31.46 MFLOP, of which
#             26.21 MFLOP are the chunk-parallel kernel's
FWD_BYTES_PER_UNIT = 4 * 16384 + 512
BWD_BYTES_PER_UNIT = 7 * 16384 + 1024
FWD_MFLOP, BWD_MFLOP, BWD_CHUNK_MFLOP = 10.49, 31.46, 26.21
# DRAM traffic per unit from ncu captures of the profiling cases (dram__bytes_read.sum + dram__bytes_write.sum over the
# units of the captured launch; traffic grows in proportion to the units, so a full launch is units x this figure)
NCU_TRAFFIC_PER_UNIT = {"gdr_fwd_kernel": 604.4e6 / 8192, "kkt_solve_tc_kernel": 178.7e6 / 8192,
                        "gdr_bwd_chunk_kernel": 183.0e3}


def l2norm(x):
    return x * torch.rsqrt((x * x).sum(-1, keepdim=True) + 1e-6)


def make_inputs(w, device, seed=0, pin=False):
    gen = torch.Generator(device="cpu").manual_seed(seed)
    B, T, Hq, Hv = w["B"], w["T"], w["Hq"], w["Hv"]

    def rn(*shape):
        return torch.randn(*shape, generator=gen)

    host = dict(
        q=l2norm(rn(B, T, Hq, 128)).bfloat16(), k=l2norm(rn(B, T, Hq, 128)).bfloat16(), v=rn(B, T, Hv, 128).bfloat16(),
        g=torch.nn.functional.logsigmoid(rn(B, T, Hv)), beta=rn(B, T, Hv).sigmoid(),
        h0=(0.1 * rn(B, Hv, 128, 128)) if (w["bwd"] or w.get("decode")) else torch.zeros(B, Hv, 128, 128))
    if w["bwd"]:
        host["do"] = rn(B, T, Hv, 128).bfloat16()
        host["dht"] = 0.01 * rn(B, Hv, 128, 128)
    if pin:
        host = {k_: v_.pin_memory() for k_, v_ in host.items()}
    if device is None:
        return host, None
    return host, {k_: v_.to(device, non_blocking=True) for k_, v_ in host.items()}


def device_inputs(B, T, Hq, Hv, dev, seed, bwd=True):
    """Inputs of the benchmark distribution drawn on the device (fast for the 1M-token configuration)."""
    gen = torch.Generator(device=dev).manual_seed(seed)
    rn = lambda *s: torch.randn(*s, device=dev, generator=gen)
    d = dict(q=l2norm(rn(B, T, Hq, 128)).bfloat16(), k=l2norm(rn(B, T, Hq, 128)).bfloat16(), v=rn(B, T, Hv, 128).bfloat16(),
             g=torch.nn.functional.logsigmoid(rn(B, T, Hv)), beta=rn(B, T, Hv).sigmoid())
    if bwd:
        d["do"] = rn(B, T, Hv, 128).bfloat16()
    return d


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed regions run."""

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap,utilization.gpu")
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={q}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is None:
            return None
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        rows = [r for r in self.rows if r and r[0].isdigit()]
        if not rows:
            return None
        # median over the samples taken under load (GPU utilisation reported > 0), else over all samples
        busy = [r for r in rows if len(r) > 6 and r[6].isdigit() and int(r[6]) > 0] or rows
        sm = sorted(int(r[0]) for r in busy)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i].lower() == "active" for r in rows)]
        smax = max(int(r[1]) for r in rows if len(r) > 1 and r[1].isdigit())
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": smax, "reasons": reasons, "samples": len(rows),
                "samples_under_load": len(busy)}


def bind_to_gpu_numa(index):
    """Run this rank's host threads on the CPUs next to its GPU (NVML's affinity mask for the device, intersected with
    the CPUs this process may use), so that its pinned buffers are allocated on the NUMA node whose PCIe root the GPU
    hangs on.  With several ranks per host this keeps the ranks' host<->device copies from sharing one memory
    controller.  Reads NVML only; returns a short description for the bench line."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(index)
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (os.cpu_count() + 63) // 64 + 16)
        cpus = {64 * i + b for i, wd in enumerate(words) for b in range(64) if (wd >> b) & 1}
        allowed = os.sched_getaffinity(0)
        use = cpus & allowed
        if use and use != allowed:
            os.sched_setaffinity(0, use)
            return f"{len(use)} of {len(allowed)} CPUs (NVML affinity of GPU {index})"
        return f"unchanged ({len(allowed)} CPUs)"
    except Exception as e:  # no NVML, no permission: carry on unbound
        return f"unchanged ({type(e).__name__})"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured (MEASURED_PEAKS.json)"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


# --------------------------------------------------------------------------------------------------------------------
# CPU arm: the oracle port on the host cores
_CPU_RATE = {}


def cpu_oracle_sample(w, threads, budget_s):
    """Time the CPU oracle port on a bounded sample of workload `w`: the full head count and distribution, the token
    axis cut to what fits `budget_s` (the cost is linear in T).  Returns (tokens/s, seconds, description)."""
    from oracle import gdr_oracle as orc
    torch.set_num_threads(threads)
    key = (w["Hq"], w["Hv"], w["bwd"])
    if key not in _CPU_RATE:   # calibrate on a short sample (also warms the thread pool up)
        cal = dict(B=1, T=1024, Hq=w["Hq"], Hv=w["Hv"], bwd=w["bwd"])
        _CPU_RATE[key] = 1024 / _run_oracle(orc, cal, seed=7)
    total = w["B"] * w["T"]
    Ts = int(min(total, max(512, _CPU_RATE[key] * budget_s)))
    Ts = max(64, Ts // 64 * 64)
    sw = dict(B=1, T=Ts, Hq=w["Hq"], Hv=w["Hv"], bwd=w["bwd"])
    dt = _run_oracle(orc, sw, seed=1)
    what = "the whole workload" if Ts == total else f"{Ts} of the {total} tokens (cost is linear in T)"
    return Ts / dt, dt, f"oracle port (PyTorch fp32, {threads} threads), full head count Hq={w['Hq']} Hv={w['Hv']}, {what}"


def _run_oracle(orc, sw, seed):
    host, _ = make_inputs(sw, None, seed=seed)
    f = {k_: v_.float() for k_, v_ in host.items()}
    t0 = time.perf_counter()
    gc, A, o, h, fs = orc.gdr_fwd(f["q"], f["k"], f["v"], f["g"], f["beta"], None, f["h0"], None)
    if sw["bwd"]:
        orc.gdr_bwd(f["q"], f["k"], f["v"], gc, f["beta"], f["do"], f["dht"], None, f["h0"], None)
    return time.perf_counter() - t0


def run_reference(args, w, rank, world):
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    # the whole run (warm-up + steps) is sized to about two and a half minutes of host time
    budget = 150.0 / max(1, args.steps + args.warmup)
    vals = []
    for i in range(args.warmup + args.steps):
        tps, dt, sample = cpu_oracle_sample(w, threads, budget)
        if i >= args.warmup:
            vals.append((tps, dt))
    tps = sum(v[0] for v in vals) / len(vals)
    ms = 1e3 * sum(v[1] for v in vals) / len(vals)
    line = {"impl": "reference", "metric": metric_name(w), "value": tps, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
            "config": {"workload": w["desc"], "timing": "CPU wall clock per bounded sample"},
            "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def metric_name(w):
    return "GDN fwd+bwd tokens/s per B200" if w["bwd"] else "GDN fwd tokens/s per B200"


# --------------------------------------------------------------------------------------------------------------------
# timing helpers
class Bench:
    def __init__(self, rank, world, local):
        import torch.distributed as dist
        self.rank, self.world, self.local, self.dist = rank, world, local, dist
        self.dev = torch.device("cuda", local)

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, values):
        t = torch.tensor(list(values), device=self.dev, dtype=torch.float64)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(x) for x in t.tolist()]

    def timed(self, step, steps, warmup, record=True):
        """W warm-up steps, then exactly K steps between a barrier + synchronise on both sides, timed with CUDA events
        on the launching stream.  Returns (ms per step on this rank, {launch name: ms per step}, launches per step)."""
        from flashqla_b200 import _lib
        for _ in range(max(3, warmup)):
            step()
        self.barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        kernel_ms, launches = {}, 0
        if record:
            with _lib.record_launches() as rec:
                self.barrier()
                t0.record()
                for _ in range(steps):
                    rec.new_step()
                    step()
                t1.record()
                self.barrier()
                summ = rec.summary()
            kernel_ms = {n: ms / steps for n, (cnt, ms) in summ.items()}
            launches = sum(cnt for cnt, _ in summ.values()) / steps
        else:
            self.barrier()
            t0.record()
            for _ in range(steps):
                step()
            t1.record()
            self.barrier()
        return t0.elapsed_time(t1) / steps, kernel_ms, launches


def pick(kernel_ms, *prefixes):
    """Time of the LAST launch per step whose entry-point name starts with one of the prefixes (the final pass of an
    entry point that is launched twice), or None."""
    hits = sorted((n for n in kernel_ms if any(n == p or n.startswith(p + "#") for p in prefixes)),
                  key=lambda n: (int(n.split("#")[1]) if "#" in n else 0))
    return kernel_ms[hits[-1]] if hits else None


def hbm_block(kernel, ms, alg_bytes, peaks, how, traffic=None, extra=None):
    achieved = alg_bytes / (ms * 1e-3) / 1e9
    b = {"kernel": kernel, "bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
         "frac": achieved / peaks["hbm_gbs"], "peak_source": how, "kernel_ms": ms, "algorithmic_bytes": alg_bytes,
         "traffic": traffic}
    b.update(extra or {})
    return b


def tensor_block(kernel, ms, flop, peaks, how, traffic=None, extra=None):
    achieved = flop / (ms * 1e-3) / 1e12
    b = {"kernel": kernel, "bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
         "frac": achieved / peaks["bf16_tflops"], "peak_source": how + ", burst figure (a 1-3 ms step)", "kernel_ms": ms,
         "algorithmic_flop": flop, "traffic": traffic}
    b.update(extra or {})
    return b


def unit_bytes(base, Hq, Hv):
    return base - 2 * 16384 + 2 * 16384 * Hq // Hv   # q, k are shared by the Hv/Hq V-heads of a group


# --------------------------------------------------------------------------------------------------------------------
def measure_forward(bn, w, d, steps, warmup):
    """Forward through the public operator without gradients (prefill), and through the stage function."""
    import flashqla_b200 as fq
    scale = 128 ** -0.5

    def step():
        with torch.no_grad():
            return fq.chunk_gated_delta_rule(d["q"], d["k"], d["v"], d["g"], d["beta"], scale=scale, initial_state=d["h0"],
                                             output_final_state=True)

    def step_stage():
        return fq.chunk_gated_delta_rule_fwd(d["q"], d["k"], d["v"], d["g"], d["beta"], scale, d["h0"], None, True, False, True)

    ms, kernel_ms, launches = bn.timed(step, steps, warmup)
    ms_stage, _, _ = bn.timed(step_stage, max(20, steps // 4), 3, record=False)
    return ms, kernel_ms, launches, ms_stage


def graph_replay_ms(bn, step, steps, warmup):
    """ms per step of `step` captured once in a CUDA graph and replayed, or None when the capture failed on any rank
    (the replay is timed between barriers: every rank takes part, or none does)."""
    cg = None
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                step()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        cg = torch.cuda.CUDAGraph()
        with torch.cuda.graph(cg):
            step()
    except Exception as exc:  # the eager figure stands
        cg = None
        print(f"[bench] CUDA graph capture of the step failed: {exc}", file=sys.stderr, flush=True)
    if bn.max_over_ranks([0.0 if cg is not None else 1.0])[0] != 0.0:
        return None
    return bn.timed(cg.replay, steps, warmup, record=False)[0]


def measure_fwd_bwd(bn, w, d, steps, warmup, graph=False):
    """Forward + backward through the differentiable operator and torch.autograd.  ``graph``: additionally capture the
    step in a CUDA graph and time its replay (a step of a few hundred microseconds is bound by the host's launch rate
    otherwise); returns a fourth value then, the replay's ms per step or None when the capture failed."""
    import flashqla_b200 as fq
    scale = 128 ** -0.5
    leaves = [d[k_].detach().requires_grad_() for k_ in ("q", "k", "v", "g", "beta", "h0")]

    def step():
        for x in leaves:
            x.grad = None
        o, fs = fq.chunk_gated_delta_rule(leaves[0], leaves[1], leaves[2], leaves[3], leaves[4], scale=scale,
                                          initial_state=leaves[5], output_final_state=True)
        torch.autograd.backward([o, fs], [d["do"], d["dht"]])

    if not graph:
        return bn.timed(step, steps, warmup)
    eager = bn.timed(step, steps, warmup, record=False)
    replay_ms = graph_replay_ms(bn, step, steps, warmup)
    return eager + (replay_ms,)


def fwd_blocks(w, ms_step, kernel_ms, peaks, how):
    B, T, Hq, Hv = w["B"], w["T"], w["Hq"], w["Hv"]
    units = B * ((T + 63) // 64) * Hv
    ub = unit_bytes(FWD_BYTES_PER_UNIT, Hq, Hv)
    alg = units * ub + 2 * B * Hv * 128 * 128 * 4     # + h0 read, final state write
    fwd_ms = pick(kernel_ms, "fq_gdr_fwd_cp_ex", "fq_gdr_fwd")
    kkt_ms = pick(kernel_ms, "fq_kkt_solve_fused")
    same = Hq == Hv
    roof = hbm_block("gdr_fwd_kernel", fwd_ms, alg, peaks, how,
                     traffic=units * NCU_TRAFFIC_PER_UNIT["gdr_fwd_kernel"] if same else None)
    roof["step_ms"] = ms_step
    roof["step_achieved"] = alg / (ms_step * 1e-3) / 1e9
    roof["step_frac"] = roof["step_achieved"] / peaks["hbm_gbs"]
    roof["step_tensor_frac"] = units * FWD_MFLOP * 1e6 / (ms_step * 1e-3) / 1e12 / peaks["bf16_tflops"]
    # the tile kernel's own input / output: k per QK head; g, beta in; g_cumsum, A_g out per V-head
    kkt_own = units * (16384 * Hq // Hv + 8192 + 3 * 256)
    kkt = hbm_block("kkt_solve_tc_kernel", kkt_ms, kkt_own, peaks, how,
                    traffic=units * NCU_TRAFFIC_PER_UNIT["kkt_solve_tc_kernel"] if same else None,
                    extra={"bytes_are": "the kernel's own inputs and outputs (k, g, beta; g_cumsum, A_g); its "
                                        "outputs are intermediates of the forward, so they do not count in step_frac"})
    return roof, {"kkt_solve_tc_kernel": kkt}


def bwd_blocks(w, ms_step, kernel_ms, peaks, how):
    B, T, Hq, Hv = w["B"], w["T"], w["Hq"], w["Hv"]
    units = B * ((T + 63) // 64) * Hv
    chunk_ms = pick(kernel_ms, "fq_gdr_bwd_chunk_grouped", "fq_gdr_bwd_chunk")
    blk = tensor_block("gdr_bwd_chunk_kernel", chunk_ms, units * BWD_CHUNK_MFLOP * 1e6, peaks, how,
                       traffic=units * NCU_TRAFFIC_PER_UNIT["gdr_bwd_chunk_kernel"])
    alg = units * (unit_bytes(FWD_BYTES_PER_UNIT, Hq, Hv) + unit_bytes(BWD_BYTES_PER_UNIT, Hq, Hv))
    blk["step_ms"] = ms_step
    blk["step_tensor_frac"] = units * (FWD_MFLOP + BWD_MFLOP) * 1e6 / (ms_step * 1e-3) / 1e12 / peaks["bf16_tflops"]
    blk["step_hbm_frac"] = alg / (ms_step * 1e-3) / 1e9 / peaks["hbm_gbs"]
    blk["hbm_frac_of_kernel"] = units * unit_bytes(BWD_BYTES_PER_UNIT, Hq, Hv) / (chunk_ms * 1e-3) / 1e9 / peaks["hbm_gbs"]
    return blk


def measure_e2e(bn, w, host, n_steps):
    """The public operator with pinned host buffers; every step's uploads and downloads inside the timed region.
    Steady-state pipeline, as a serving / training loop would run it: the inputs of a step go host -> device on one copy
    stream into one of two device buffer sets, the operator runs on the compute stream, and the results go device ->
    pinned host memory on a second copy stream, so the upload of step i+1 overlaps the download of step i."""
    import flashqla_b200 as fq
    dev = bn.dev
    scale = 128 ** -0.5
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    main = torch.cuda.current_stream(dev)
    dev_in = [{k_: torch.empty(host[k_].shape, dtype=host[k_].dtype, device=dev) for k_ in host} for _ in range(2)]
    in_free, out_done, host_out = [None, None], [None, None], [None, None]
    d2h = [0]

    def e2e_step(i):
        slot = i & 1
        buf = dev_in[slot]
        with torch.cuda.stream(s_in):
            if in_free[slot] is not None:
                s_in.wait_event(in_free[slot])  # the step that last used this buffer set has finished computing
            for k_ in host:
                buf[k_].copy_(host[k_], non_blocking=True)
            ev_in = s_in.record_event()
        main.wait_event(ev_in)
        if not w["bwd"]:
            with torch.no_grad():
                o, fs = fq.chunk_gated_delta_rule(buf["q"], buf["k"], buf["v"], buf["g"], buf["beta"], scale=scale,
                                                  initial_state=buf["h0"], output_final_state=True)
            outs = [o, fs]
        else:
            leaves = [buf[k_].detach().requires_grad_() for k_ in ("q", "k", "v", "g", "beta", "h0")]
            o, fs = fq.chunk_gated_delta_rule(leaves[0], leaves[1], leaves[2], leaves[3], leaves[4], scale=scale,
                                              initial_state=leaves[5], output_final_state=True)
            torch.autograd.backward([o, fs], [buf["do"], buf["dht"]])
            outs = [x.grad for x in leaves] + [o.detach()]
        in_free[slot] = main.record_event()
        if host_out[slot] is None:
            host_out[slot] = [torch.empty(x.shape, dtype=x.dtype, pin_memory=True) for x in outs]
        d2h[0] = sum(x.numel() * x.element_size() for x in outs)
        with torch.cuda.stream(s_out):
            s_out.wait_event(in_free[slot])
            if out_done[slot] is not None:
                out_done[slot].synchronize()  # the pinned result buffers of this slot were consumed two steps ago
            for dst, src in zip(host_out[slot], outs):
                dst.copy_(src, non_blocking=True)
                src.record_stream(s_out)
            out_done[slot] = s_out.record_event()

    for i in range(3):
        e2e_step(i)
    bn.barrier()
    w0 = time.perf_counter()
    for i in range(n_steps):
        e2e_step(i)
    bn.barrier()
    ms = 1e3 * (time.perf_counter() - w0) / n_steps
    h2d = sum(host[k_].numel() * host[k_].element_size() for k_ in host)
    return ms, h2d, d2h[0]


# --------------------------------------------------------------------------------------------------------------------
# strong-scaling blocks (N > 1)
def sequence_parallel_run(bn, w, steps, warmup, check=True):
    """One long sequence, rank r owns tokens [r*T/N, (r+1)*T/N): forward + backward with the exchange of per-rank
    summaries.  Returns a dict (ms per step = max over ranks)."""
    from flashqla_b200 import dist as fqd
    from flashqla_b200 import ops
    T, H = w["T"], w["Hv"]
    rank, world, dev = bn.rank, bn.world, bn.dev
    b = fqd.shard_sequence(T, world)
    Tl = b[rank + 1] - b[rank]
    d = device_inputs(1, Tl, H, H, dev, seed=100 + rank)
    scale = 128 ** -0.5
    impl = fqd.CudaImpl()
    out = {}
    if check and world > 1:
        # first step: this rank's slice against the single-GPU operator on the whole sequence (every rank rebuilds the
        # other ranks' tokens from their seeds)
        full = [device_inputs(1, b[r + 1] - b[r], H, H, dev, seed=100 + r) for r in range(world)]
        cat = {k_: torch.cat([f[k_] for f in full], 1) for k_ in full[0]}
        del full
        gc, A, o_ref, _, fs_ref = ops.chunk_gated_delta_rule_fwd(cat["q"], cat["k"], cat["v"], cat["g"], cat["beta"], scale,
                                                                 None, None, True, False, True)
        ref = ops.chunk_gated_delta_rule_bwd(cat["q"], cat["k"], cat["v"], gc, cat["beta"], A, cat["do"], None, scale, None, None)
        o, fs, saved = fqd.cp_forward(d["q"], d["k"], d["v"], d["g"], d["beta"], scale, None, None, impl=impl)
        grads = fqd.cp_backward(saved, d["do"], None, None, impl=impl)
        sl = slice(b[rank], b[rank + 1])
        rel = lambda x, r: ((x.float() - r.float()).abs().max() / r.float().abs().max().clamp_min(1e-30)).item()
        errs = [rel(o, o_ref[:, sl]), rel(fs, fs_ref)] + [rel(x, r[:, sl]) for x, r in zip(grads[:5], ref[:5])]
        worst = bn.max_over_ranks([max(errs)])[0]
        out["parity_vs_single_gpu"] = {"max_rel_to_max_err": worst, "tolerance": 1e-2, "ok": worst < 1e-2,
                                       "compared": "o, final_state, dq, dk, dv, dbeta, dg of every rank's slice"}
        del cat, gc, A, o_ref, fs_ref, ref, o, fs, saved, grads
        torch.cuda.empty_cache()

    def step():
        if world == 1:   # the whole sequence on one GPU: the plain operator (tiles and states kept for the backward, as autograd does)
            gc, A, o, _, fs, tiles, _ = ops.chunk_gated_delta_rule_fwd(d["q"], d["k"], d["v"], d["g"], d["beta"], scale, None, None,
                                                                    True, False, True, _return_tiles=True, _keep_h=True)
            ops.chunk_gated_delta_rule_bwd(d["q"], d["k"], d["v"], gc, d["beta"], A, d["do"], None, scale, None, None,
                                           _gated_tiles=tiles[:2], _h_saved=tiles[2])
            return
        o, fs, saved = fqd.cp_forward(d["q"], d["k"], d["v"], d["g"], d["beta"], scale, None, None, impl=impl)
        fqd.cp_backward(saved, d["do"], None, None, impl=impl)

    ms, _, _ = bn.timed(step, steps, warmup, record=False)
    ms = bn.max_over_ranks([ms])[0]
    out["ms_per_step_eager"] = ms
    if world > 1 and os.environ.get("FQ_BENCH_SP_GRAPH", "0") == "1":
        # the step (kernels and NCCL collectives) captured once and replayed: shows what the host's launch rate costs
        ms_g = graph_replay_ms(bn, step, steps, warmup)
        if ms_g is not None:
            ms_g = bn.max_over_ranks([ms_g])[0]
            out["ms_per_step_graph"] = ms_g
            ms = min(ms, ms_g)
    out.update({"ms_per_step": ms, "tokens_per_s": T / (ms * 1e-3), "steps": steps,
                "exchange": "all_gather of per-rank (end state from zero, transition matrix) in the forward and of the "
                            "left-edge state gradient in the backward; no halo, no serial hand-over",
                "nccl_bytes_per_step_per_rank": (2 + 1 + 1) * H * 128 * 128 * 4 if world > 1 else 0,
                "tokens_per_rank": Tl})
    return out


def multi_gpu_blocks(bn, t1_c3_ms):
    """The two configurations that divide one problem over the ranks (strong scaling)."""
    import flashqla_b200 as fq
    from flashqla_b200 import dist as fqd
    world, rank, dev = bn.world, bn.rank, bn.dev
    res = {}
    # ---- config 5: the single-GPU time first (rank 0 alone; the others wait), then the N-rank run
    w5 = WORKLOADS["c5"]
    t1 = [0.0]
    if rank == 0:
        solo = Bench(0, 1, bn.local)
        t1[0] = sequence_parallel_run(solo, w5, 5, 3, check=False)["ms_per_step"]
        torch.cuda.empty_cache()
    t1 = bn.max_over_ranks(t1)[0]
    c5 = sequence_parallel_run(bn, w5, 10, 3)
    c5.update({"scaling": "strong", "workload": w5["desc"], "ms_per_step_1gpu": t1,
               "efficiency_vs_1gpu": t1 / (world * c5["ms_per_step"])})
    res["c5"] = c5
    torch.cuda.empty_cache()
    # ---- config 3 sharded: the 64 (batch, QK-head group) units split over the ranks
    w3 = WORKLOADS["c3"]
    bs, qs, vs = fqd.shard_units(w3["B"], w3["Hq"], w3["Hv"], world, rank)
    Bl, Hql, Hvl = bs.stop - bs.start, qs.stop - qs.start, vs.stop - vs.start
    d = device_inputs(Bl, w3["T"], Hql, Hvl, dev, seed=300 + rank)
    gen = torch.Generator(device=dev).manual_seed(400 + rank)
    d["h0"] = 0.1 * torch.randn(Bl, Hvl, 128, 128, device=dev, generator=gen)
    d["dht"] = 0.01 * torch.randn(Bl, Hvl, 128, 128, device=dev, generator=gen)
    ms_eager, _, _, ms_graph = measure_fwd_bwd(bn, w3, d, 50, 3, graph=True)
    ms_eager, ms_graph = bn.max_over_ranks([ms_eager, ms_graph if ms_graph is not None else float("inf")])
    ms = min(ms_eager, ms_graph)
    res["c3_sharded"] = {"scaling": "strong", "workload": w3["desc"], "ms_per_step": ms,
                         "launch": "CUDA graph replay of the captured fwd+bwd step" if ms == ms_graph else "eager",
                         "ms_per_step_eager": ms_eager, "ms_per_step_graph": ms_graph if ms_graph != float("inf") else None,
                         "tokens_per_s": w3["B"] * w3["T"] / (ms * 1e-3), "ms_per_step_1gpu": t1_c3_ms,
                         "efficiency_vs_1gpu": t1_c3_ms / (world * ms), "collective": "none (units are independent)",
                         "units_per_rank": Bl * Hql, "shard": f"B={Bl} Hq={Hql} Hv={Hvl} per rank"}
    return res


# --------------------------------------------------------------------------------------------------------------------
def run_sequence_parallel(args, w, bn):
    """--workload c5: the 1M-token sequence over the N GPUs as the whole bench line."""
    sampler = ClockSampler(bn.local) if bn.rank == 0 else None
    if sampler:
        sampler.start()
    r = sequence_parallel_run(bn, w, args.steps, args.warmup)
    clocks = sampler.stop() if sampler else None
    if bn.rank == 0:
        peaks, how = measured_peaks()
        units = (w["T"] // 64) * w["Hv"]
        ms = r["ms_per_step"]
        print(json.dumps({
            "metric": "GDN fwd+bwd tokens/s, one 1M-token sequence split over the GPUs", "value": r["tokens_per_s"],
            "unit": "tokens/s", "n_gpus": bn.world, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": w["desc"], "l2": "inputs exceed the 126 MB L2; no flush needed", **r},
            "roofline": {"bound": "tensor", "unit": "TFLOP/s", "peak": bn.world * peaks["bf16_tflops"], "peak_source": how,
                         "achieved": units * (FWD_MFLOP + BWD_MFLOP) * 1e6 / (ms * 1e-3) / 1e12,
                         "frac": units * (FWD_MFLOP + BWD_MFLOP) * 1e6 / (ms * 1e-3) / 1e12 / (bn.world * peaks["bf16_tflops"]),
                         "traffic": None},
            "clocks": clocks}), flush=True)


def run_decode(args, w, bn):
    """One recurrent step for N sequences per GPU (weak scaling: every rank has its own N sequences)."""
    import flashqla_b200 as fq
    rank, world, dev, dist = bn.rank, bn.world, bn.dev, bn.dist
    host, d = make_inputs(w, dev, seed=rank, pin=True)
    N, Hq, Hv = w["B"], w["Hq"], w["Hv"]
    scale = 128 ** -0.5
    state = d["h0"].clone()
    n_tok = w["tokens_per_step"]

    def step():
        for _ in range(n_tok):
            fq.fused_recurrent_gated_delta_rule(d["q"], d["k"], d["v"], d["g"], d["beta"], scale=scale,
                                                initial_state=state, inplace_state=True)

    sampler = ClockSampler(bn.local) if rank == 0 else None
    if sampler:
        sampler.start()
    ms_step, _, _ = bn.timed(step, args.steps, args.warmup, record=False)

    # end to end: the new token's q, k, v, g, beta come from pinned host memory, o goes back; the state stays on the GPU
    small = {k_: host[k_] for k_ in ("q", "k", "v", "g", "beta")}
    o_host = torch.empty(N, 1, Hv, 128, dtype=torch.bfloat16, pin_memory=True)

    def e2e_step():
        for _ in range(n_tok):
            dd = {k_: small[k_].to(dev, non_blocking=True) for k_ in small}
            o, _ = fq.fused_recurrent_gated_delta_rule(dd["q"], dd["k"], dd["v"], dd["g"], dd["beta"], scale=scale,
                                                       initial_state=state, inplace_state=True)
            o_host.copy_(o, non_blocking=True)
            torch.cuda.synchronize()  # a decode loop needs the token's output before it can form the next input

    for _ in range(3):
        e2e_step()
    bn.barrier()
    n_e2e = max(3, min(args.steps, 10))
    w0 = time.perf_counter()
    for _ in range(n_e2e):
        e2e_step()
    bn.barrier()
    e2e_ms = 1e3 * (time.perf_counter() - w0) / n_e2e
    clocks = sampler.stop() if sampler else None
    ms_step, e2e_ms = bn.max_over_ranks([ms_step, e2e_ms])
    if rank == 0:
        peaks, how = measured_peaks()
        # state read + write (2 x 64 KiB per head) + q, k, v, o, g, beta of the token
        alg_bytes = N * Hv * (2 * 128 * 128 * 4 + 2 * 256 + 8) + N * Hq * 2 * 256  # per kernel launch (one token)
        kernel_ms = ms_step / n_tok
        h2d = sum(small[k_].numel() * small[k_].element_size() for k_ in small)
        line = {
            "metric": "GDN decode tokens/s per B200", "value": world * N * n_tok / (ms_step * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": w["desc"], "l2": "the 1 GiB state exceeds the 126 MB L2; no flush needed"},
            "gpu_launches": n_tok * args.steps,
            "roofline": hbm_block("gdr_recurrent_kernel", kernel_ms, alg_bytes, peaks, how),
            "clocks": clocks,
            "e2e": {"value": world * N * n_tok / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": h2d * n_tok, "d2h_bytes_per_step": o_host.numel() * 2 * n_tok},
        }
        if not args.no_cpu_baseline:
            from oracle import gdr_oracle as orc
            threads = os.cpu_count() or 1
            torch.set_num_threads(threads)
            ns = 16
            t_0 = time.perf_counter()
            orc.gdr_recurrent(host["q"][:ns].float(), host["k"][:ns].float(), host["v"][:ns].float(), host["g"][:ns],
                              host["beta"][:ns], scale, host["h0"][:ns], dtype=torch.float32)
            dt = time.perf_counter() - t_0
            line["cpu_baseline"] = {"value": ns / dt, "unit": "tokens/s", "cores": threads, "kind": "port",
                                    "sample": f"token-level oracle, {ns} of the {N} sequences, fp32", "seconds": dt}
        print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--lean", action="store_true", help="main timed loop only (no e2e, no extra blocks): for profiling")
    args = ap.parse_args()
    w = WORKLOADS[args.workload]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, w, rank, world)
        return

    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    affinity = bind_to_gpu_numa(local) if world > 1 else "unchanged (one rank)"
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    bn = Bench(rank, world, local)
    bn.affinity = affinity
    try:
        if w.get("seq_parallel"):
            run_sequence_parallel(args, w, bn)
        elif w.get("decode"):
            run_decode(args, w, bn)
        else:
            run_main(args, w, bn)
    finally:
        if world > 1:
            dist.destroy_process_group()


def run_main(args, w, bn):
    rank, world, dev = bn.rank, bn.world, bn.dev
    lean = args.lean or w.get("lean", False)
    host, d = make_inputs(w, dev, seed=rank, pin=True)
    torch.cuda.synchronize()
    B, T, Hq, Hv = w["B"], w["T"], w["Hq"], w["Hv"]
    tokens = B * T
    peaks, how = measured_peaks()
    sampler = ClockSampler(bn.local) if rank == 0 else None
    if sampler:
        sampler.start()

    line = {"metric": metric_name(w), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic"}
    config = {"workload": w["desc"], "l2": "inputs exceed the 126 MB L2; no flush needed"}
    from flashqla_b200 import kernels
    from flashqla_b200.planner import plan_cp, plan_dense
    cp = plan_cp(plan_dense(B, T), B, T, Hv, kernels.sm_count(dev), dev)
    config["context_parallel_piece_chunks"] = None if cp is None else cp.piece_chunks
    config["host_cpu_affinity"] = getattr(bn, "affinity", None)

    fwd_bwd = None
    if not w["bwd"]:
        ms, kernel_ms, launches, ms_stage = measure_forward(bn, w, d, args.steps, args.warmup)
        ms, ms_stage = bn.max_over_ranks([ms, ms_stage])
        roof, kernels_blk = fwd_blocks(w, ms, kernel_ms, peaks, how)
        config["entry"] = "chunk_gated_delta_rule without gradients (prefill: the inverse A is not stored)"
        line["fwd_stage_api"] = {"entry": "chunk_gated_delta_rule_fwd (returns A: A is stored)", "ms_per_step": ms_stage,
                                 "tokens_per_s": world * tokens / (ms_stage * 1e-3)}
    else:
        ms, kernel_ms, launches = measure_fwd_bwd(bn, w, d, args.steps, args.warmup)
        ms = bn.max_over_ranks([ms])[0]
        roof = bwd_blocks(w, ms, kernel_ms, peaks, how)
        kernels_blk = {}
        config["entry"] = "chunk_gated_delta_rule + torch.autograd.backward"
    config["kernel_ms"] = {k_: round(v_, 4) for k_, v_ in kernel_ms.items()}
    line.update({"value": world * tokens / (ms * 1e-3), "ms_per_step": ms, "config": config,
                 "gpu_launches": int(round(launches * args.steps)), "roofline": roof})
    if kernels_blk:
        line["roofline"]["kernels"] = kernels_blk

    if not lean:
        # ---- the other half of the metric: forward + backward on the training configuration
        if not w["bwd"]:
            w3 = WORKLOADS["c3"]
            _, d3 = make_inputs(w3, dev, seed=50 + rank)
            ms3, k3, l3 = measure_fwd_bwd(bn, w3, d3, args.steps, args.warmup)
            ms3 = bn.max_over_ranks([ms3])[0]
            fwd_bwd = {"workload": w3["desc"], "entry": "chunk_gated_delta_rule + torch.autograd.backward",
                       "ms_per_step": ms3, "tokens_per_s": world * w3["B"] * w3["T"] / (ms3 * 1e-3), "steps": args.steps,
                       "kernel_ms": {k_: round(v_, 4) for k_, v_ in k3.items()},
                       "gpu_launches": int(round(l3 * args.steps)), "roofline": bwd_blocks(w3, ms3, k3, peaks, how)}
            line["fwd_bwd"] = fwd_bwd
            del d3
            torch.cuda.empty_cache()
        # ---- end to end with host buffers
        e2e_ms, h2d, d2h = measure_e2e(bn, w, host, max(4, min(args.steps, 10)))
        e2e_ms = bn.max_over_ranks([e2e_ms])[0]
        line["e2e"] = {"value": world * tokens / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                       "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h}
        if world > 1 and fwd_bwd is not None:
            del d
            torch.cuda.empty_cache()
            line["multi_gpu"] = multi_gpu_blocks(bn, fwd_bwd["ms_per_step"])
    line["clocks"] = sampler.stop() if sampler else None

    if rank == 0:
        if not args.no_cpu_baseline and not lean:
            threads = os.cpu_count() or 1
            tps, dt, sample = cpu_oracle_sample(w, threads, 20.0)
            line["cpu_baseline"] = {"value": tps, "unit": "tokens/s", "cores": threads, "kind": "port",
                                    "sample": sample, "seconds": dt}
        print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
