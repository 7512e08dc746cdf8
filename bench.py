#!/usr/bin/env python
"""Benchmark of the chunked gated-delta-rule (GDN) hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c3|c5|decode|c2s|c3s]

One "step" = one pass of the hot path over one synthetic batch.  The default workload is the
configuration the headline metric is quoted on: single-GPU forward prefill,
B=1, T=32768, H_q=H_v=64, K=V=128, bf16 q/k/v, fp32 gates (``c2``).  ``c3`` adds the training
forward+backward on B=4, T=8192, H_q=16, H_v=32.

Prints ONE JSON line (rank 0).  ``value`` is device-timed throughput with the inputs resident in
HBM; ``e2e`` is the same metric through the public operator with HOST (pinned) buffers, the
host<->device copies inside the timed region.  Under torchrun every rank runs the same workload
on its own GPU (the path shards by batch x head with no collective): weak scaling.

``--impl reference`` times the reference's CPU implementation of the path (the PyTorch oracle
port under oracle/, all host threads) on a bounded sample of the same workload.
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
    # name: (B, T, Hq, Hv, backward)
    "c2": dict(B=1, T=32768, Hq=64, Hv=64, bwd=False,
               desc="fwd prefill B=1 T=32768 Hq=Hv=64 K=V=128 bf16, g=logsigmoid(randn) fp32, h0=zeros"),
    "c2s": dict(B=1, T=16384, Hq=32, Hv=32, bwd=False,
                desc="(profiling case) fwd B=1 T=16384 Hq=Hv=32 K=V=128 bf16"),
    "c5": dict(B=1, T=1048576, Hq=8, Hv=8, bwd=True, seq_parallel=True,
               desc="fwd+bwd B=1 T=1048576 Hq=Hv=8 K=V=128 bf16, ONE sequence split contiguously over the GPUs"),
    "c3": dict(B=4, T=8192, Hq=16, Hv=32, bwd=True,
               desc="fwd+bwd B=4 T=8192 Hq=16 Hv=32 K=V=128 bf16, h0=0.1 randn, dht=0.01 randn"),
    "c3s": dict(B=2, T=8192, Hq=8, Hv=16, bwd=True,
                desc="(profiling case) fwd+bwd B=2 T=8192 Hq=8 Hv=16 K=V=128 bf16"),
    # decode side of the path: one new token for each of N sequences, state resident on the device
    "decode": dict(B=256, T=1, Hq=64, Hv=64, bwd=False, decode=True, tokens_per_step=64,
                   desc="decode: 64 consecutive tokens for each of 256 sequences (one kernel call per token), Hq=Hv=64 "
                        "K=V=128, fp32 state 1 GiB resident in HBM"),
}
# algorithmic HBM bytes per (chunk, V-head) of the fused forward kernel at Hq == Hv:
# q, k, v read + o write (4 x 16 KiB) + g, beta (2 x 256 B)
FWD_BYTES_PER_UNIT = 4 * 16384 + 512
# DRAM traffic of gdr_fwd_kernel per (chunk, V-head) from one ncu capture of the smaller case c2s (Hq == Hv):
# dram__bytes_read.sum + dram__bytes_write.sum = 665,837,312 B over 8192 units (profiles/forward_kernels_*.md);
# traffic grows in proportion to the units, so a full launch is reported as units x this figure
FWD_TRAFFIC_PER_UNIT_NCU = 674940416 / 8192


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


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
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
        sm = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        if not sm:
            return None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i].lower() == "active" for r in self.rows)]
        smax = max(int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit())
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": smax, "reasons": reasons, "samples": len(sm)}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return d, "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


def cpu_oracle_sample(w, threads):
    """Time the CPU oracle port on a bounded sample: same distribution, T and H cut down.
    Cost is linear in T*H, so tokens/s at the full head count = T_s * (H_s / Hv) / time."""
    from oracle import gdr_oracle as orc
    torch.set_num_threads(threads)
    Ts, Hs = 32768, 32
    Hqs = max(1, Hs * w["Hq"] // w["Hv"])
    sw = dict(B=1, T=Ts, Hq=Hqs, Hv=Hs, bwd=w["bwd"])
    host, _ = make_inputs(sw, None, seed=1)
    f = {k_: v_.float() for k_, v_ in host.items()}
    t0 = time.perf_counter()
    gc, A, o, h, fs = orc.gdr_fwd(f["q"], f["k"], f["v"], f["g"], f["beta"], None, f["h0"], None)
    if w["bwd"]:
        orc.gdr_bwd(f["q"], f["k"], f["v"], gc, f["beta"], f["do"], f["dht"], None, f["h0"], None)
    dt = time.perf_counter() - t0
    tokens_equiv = Ts * Hs / w["Hv"]
    return tokens_equiv / dt, dt, f"oracle port, B=1 T={Ts} Hq={Hqs} Hv={Hs} fp32, scaled by heads to Hv={w['Hv']}"


def run_reference(args, w, rank, world):
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    vals = []
    for i in range(args.warmup + args.steps):
        tps, dt, sample = cpu_oracle_sample(w, threads)
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


def run_sequence_parallel(args, w, rank, world, local):
    """Config 5: one long sequence, rank r owns tokens [r*T/N, (r+1)*T/N); halo exchange over NCCL."""
    import torch.distributed as dist
    from flashqla_b200 import dist as fqd
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if not dist.is_initialized():
        dist.init_process_group("nccl" if world > 1 else "gloo", device_id=dev if world > 1 else None,
                                rank=rank, world_size=world,
                                init_method=None if "MASTER_ADDR" in os.environ else "tcp://127.0.0.1:29533")
    T, H = w["T"], w["Hv"]
    b = fqd.shard_sequence(T, world)
    Tl = b[rank + 1] - b[rank]
    gen = torch.Generator(device="cpu").manual_seed(100 + rank)
    rn = lambda *shape: torch.randn(*shape, generator=gen)
    q = l2norm(rn(1, Tl, H, 128)).bfloat16().to(dev); k = l2norm(rn(1, Tl, H, 128)).bfloat16().to(dev)
    v = rn(1, Tl, H, 128).bfloat16().to(dev); g = torch.nn.functional.logsigmoid(rn(1, Tl, H)).to(dev)
    beta = rn(1, Tl, H).sigmoid().to(dev); do = rn(1, Tl, H, 128).bfloat16().to(dev)
    scale = 128 ** -0.5

    def step():
        o, fs, info = fqd.cp_forward(q, k, v, g, beta, scale, None, None)
        fqd.cp_backward(q, k, v, g, beta, do, None, scale, info["h_in"], None, mode=info["mode"])
        return info

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(3, args.warmup)):
        info = step()
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t0.record()
    for _ in range(args.steps):
        step()
    t1.record()
    barrier()
    ms = torch.tensor([t0.elapsed_time(t1) / args.steps], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    clocks = sampler.stop() if sampler else None
    if rank == 0:
        ms_step = float(ms.item())
        print(json.dumps({
            "metric": "GDN fwd+bwd tokens/s, one 1M-token sequence split over the GPUs", "value": T / (ms_step * 1e-3),
            "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": w["desc"], "exchange": info["mode"], "halo_chunks": info["halo_chunks"],
                       "replayed_chunks": info["replayed"]},
            "clocks": clocks}), flush=True)
    if world > 1:
        dist.destroy_process_group()


def metric_name(w):
    return "GDN fwd+bwd tokens/s per B200" if w["bwd"] else "GDN fwd tokens/s per B200"


def run_decode(args, w, rank, world, local):
    """One recurrent step for N sequences per GPU (weak scaling: every rank has its own N sequences)."""
    import torch.distributed as dist
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    import flashqla_b200 as fq
    host, d = make_inputs(w, dev, seed=rank, pin=True)
    N, Hq, Hv = w["B"], w["Hq"], w["Hv"]
    scale = 128 ** -0.5
    state = d["h0"].clone()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    n_tok = w["tokens_per_step"]

    def step():
        for _ in range(n_tok):
            fq.fused_recurrent_gated_delta_rule(d["q"], d["k"], d["v"], d["g"], d["beta"], scale=scale,
                                                initial_state=state, inplace_state=True)

    for _ in range(max(3, args.warmup)):
        step()
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t0.record()
    for _ in range(args.steps):
        step()
    t1.record()
    barrier()
    ms_step = t0.elapsed_time(t1) / args.steps

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
    barrier()
    n_e2e = max(3, min(args.steps, 10))
    w0 = time.perf_counter()
    for _ in range(n_e2e):
        e2e_step()
    barrier()
    e2e_ms = 1e3 * (time.perf_counter() - w0) / n_e2e
    clocks = sampler.stop() if sampler else None
    ms = torch.tensor([ms_step, e2e_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_step, e2e_ms = (float(x) for x in ms.tolist())
    if rank == 0:
        peaks, how = measured_peaks()
        # state read + write (2 x 64 KiB per head) + q, k, v, o, g, beta of the token
        alg_bytes = N * Hv * (2 * 128 * 128 * 4 + 2 * 256 + 8) + N * Hq * 2 * 256  # per kernel launch (one token)
        kernel_ms = ms_step / n_tok
        achieved = alg_bytes / (kernel_ms * 1e-3) / 1e9
        h2d = sum(small[k_].numel() * small[k_].element_size() for k_ in small)
        line = {
            "metric": "GDN decode tokens/s per B200", "value": world * N * n_tok / (ms_step * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": w["desc"], "l2": "the 1 GiB state exceeds the 126 MB L2; no flush needed"},
            "gpu_launches": n_tok,
            "roofline": {"kernel": "gdr_recurrent_kernel", "bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"],
                         "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                         "peak_source": "measured copy bandwidth (MEASURED_PEAKS.json)" if how == "measured" else "fallback",
                         "kernel_ms": kernel_ms, "algorithmic_bytes": alg_bytes, "traffic": None},
            "clocks": clocks,
            "e2e": {"value": world * N * n_tok / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": h2d * n_tok, "d2h_bytes_per_step": o_host.numel() * 2 * n_tok},
        }
        if not args.no_cpu_baseline:
            sys.path.insert(0, ROOT)
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
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    w = WORKLOADS[args.workload]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        if args.impl == "reference" and args.steps > 3:
            args.steps, args.warmup = min(args.steps, 3), min(args.warmup, 1)
        run_reference(args, w, rank, world)
        return

    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    if w.get("seq_parallel"):
        run_sequence_parallel(args, w, rank, world, local)
        return
    if w.get("decode"):
        run_decode(args, w, rank, world, local)
        return
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    import flashqla_b200 as fq
    from flashqla_b200 import kernels
    from flashqla_b200.planner import plan_cp, plan_dense

    host, d = make_inputs(w, dev, seed=rank, pin=True)
    torch.cuda.synchronize()
    B, T, Hq, Hv = w["B"], w["T"], w["Hq"], w["Hv"]
    tokens = B * T
    scale = 128 ** -0.5
    plan = plan_dense(B, T)
    cp = plan_cp(plan, B, T, Hv, kernels.sm_count(dev), dev)
    stamps = []          # per step: list of (name, start_event, end_event) for the forward kernels
    launches = [0]

    def timed(name, fn, rec):
        if rec is None:
            return fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out = fn()
        e1.record()
        rec.append((name, e0, e1))
        return out

    def step(record=False):
        rec = [] if record else None
        # chunk-local cumsum of g, A and the gated tiles in one launch
        # (A, which only the backward reads, is stored in the fwd+bwd workloads only)
        g_cum, A, Ag, Pg = timed("kkt_solve", lambda: kernels.kkt_solve_fused(d["k"], d["q"], d["beta"], d["g"], scale, plan,
                                                                              want_A=w["bwd"]), rec)
        warm = timed("cp_warmup", lambda: kernels.cp_warmup(g_cum, cp, Hv), rec) if cp is not None else None
        # transition-matrix fallback for slowly decaying heads: state pass + chain (near-empty launches when no head needs it)
        h0p = timed("cp_correct", lambda: kernels.cp_correct_states(d["q"], d["k"], d["v"], Ag, g_cum, d["beta"], scale,
                                                                    d["h0"], cp, warm), rec) if cp is not None else None
        o, _, fs = timed("gdr_fwd", lambda: kernels.fused_gdr_fwd(d["q"], d["k"], d["v"], Ag, Pg, g_cum, d["beta"], scale,
                                                                 initial_state=d["h0"], plan=plan, cp=cp, warmup=warm,
                                                                 h0_piece=h0p), rec)
        n = 2 + (3 if cp is not None else 0)  # kkt_solve, gdr_fwd (+ plan kernel, state pass, chain)
        if w["bwd"]:
            # as in the autograd function, which keeps the forward's gated tiles for its backward
            timed("backward", lambda: fq.chunk_gated_delta_rule_bwd(d["q"], d["k"], d["v"], g_cum, d["beta"], A, d["do"],
                                                                     d["dht"], scale, d["h0"], None,
                                                                     _gated_tiles=(Ag, Pg)), rec)
            # fwd(h) + bwd_dh + bwd_chunk + reverse cumsum (+ plan kernel, state pass, chain, gradient pass, reverse chain;
            # + 2 head sums)
            n += 4 + (5 if cp is not None else 0) + (2 if Hq < Hv else 0)
        if record:
            stamps.append(rec)
        launches[0] = n
        return o, fs

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(3, args.warmup)):
        step()
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t0.record()
    for _ in range(args.steps):
        step(record=True)
    t1.record()
    barrier()
    ms_total = t0.elapsed_time(t1)
    kernel_ms = {}
    for rec in stamps:
        for name, e0, e1 in rec:
            kernel_ms[name] = kernel_ms.get(name, 0.0) + e0.elapsed_time(e1) / len(stamps)
    fwd_ms = kernel_ms["gdr_fwd"]

    # ---- end to end through the public operator with host buffers (pinned), copies inside the timed region.
    # Steady-state pipeline, as a serving / training loop would run it: the inputs of a step go host -> device on
    # one copy stream into one of two device buffer sets, the operator runs on the compute stream, and the results
    # go device -> pinned host memory on a second copy stream, so the upload of step i+1 overlaps the download of
    # step i (PCIe is full duplex).  Every step's copies are inside the timed region; one synchronise at the end.
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    main = torch.cuda.current_stream(dev)
    dev_in = [{k_: torch.empty(host[k_].shape, dtype=host[k_].dtype, device=dev) for k_ in host} for _ in range(2)]
    in_free = [None, None]
    out_done = [None, None]
    host_out = [None, None]

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
            _, _, o, _, fs = fq.chunk_gated_delta_rule_fwd(buf["q"], buf["k"], buf["v"], buf["g"], buf["beta"], scale,
                                                           buf["h0"], None, True, False, True)
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
        with torch.cuda.stream(s_out):
            s_out.wait_event(in_free[slot])
            if out_done[slot] is not None:
                out_done[slot].synchronize()  # the pinned result buffers of this slot were consumed two steps ago
            for dst, src in zip(host_out[slot], outs):
                dst.copy_(src, non_blocking=True)
                src.record_stream(s_out)
            out_done[slot] = s_out.record_event()

    for i in range(2):
        e2e_step(i)
    torch.cuda.synchronize()
    barrier()
    n_e2e = max(4, min(args.steps, 10))
    w0 = time.perf_counter()
    for i in range(n_e2e):
        e2e_step(i)
    torch.cuda.synchronize()
    barrier()
    e2e_ms = 1e3 * (time.perf_counter() - w0) / n_e2e
    h2d = sum(host[k_].numel() * host[k_].element_size() for k_ in host)
    d2h = tokens * Hv * 128 * 2 + B * Hv * 128 * 128 * 4
    if w["bwd"]:
        d2h = sum(host[k_].numel() * host[k_].element_size() for k_ in ("q", "k", "v", "g", "beta", "h0")) + tokens * Hv * 256
    clocks = sampler.stop() if sampler else None

    ms = torch.tensor([ms_total / args.steps, fwd_ms, e2e_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_step, fwd_ms, e2e_ms = (float(x) for x in ms.tolist())

    if rank == 0:
        peaks, how = measured_peaks()
        units = plan.total_chunks * Hv
        unit_bytes = FWD_BYTES_PER_UNIT - 2 * 16384 + 2 * 16384 * Hq // Hv  # q,k are shared by Hv/Hq V-heads
        alg_bytes = units * unit_bytes + 2 * B * Hv * 128 * 128 * 4          # + h0 read, final state write
        achieved = alg_bytes / (fwd_ms * 1e-3) / 1e9
        line = {
            "metric": metric_name(w), "value": world * tokens / (ms_step * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": w["desc"], "l2": "inputs exceed the 126 MB L2; no flush needed",
                       "context_parallel_piece_chunks": None if cp is None else cp.piece_chunks,
                       "kernel_ms": {k_: round(v_, 4) for k_, v_ in kernel_ms.items()}},
            "gpu_launches": launches[0] * args.steps,
            "roofline": {"kernel": "gdr_fwd_kernel", "bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"],
                         "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                         "peak_source": "measured copy bandwidth (MEASURED_PEAKS.json)" if how == "measured" else "fallback",
                         "kernel_ms": fwd_ms, "algorithmic_bytes": alg_bytes,
                         "traffic": (units * FWD_TRAFFIC_PER_UNIT_NCU if Hq == Hv else None)},
            "clocks": clocks,
            "e2e": {"value": world * tokens / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        }
        if not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            tps, dt, sample = cpu_oracle_sample(w, threads)
            line["cpu_baseline"] = {"value": tps, "unit": "tokens/s", "cores": threads, "kind": "port",
                                    "sample": sample, "seconds": dt}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
