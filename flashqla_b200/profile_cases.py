"""Small, self-contained launches of the kernels that the two benchmark workloads do not exercise alone, sized for an
ncu capture (inputs larger than the 126 MB L2, a few hundred MB on the device) and timed with CUDA events:

    python -m flashqla_b200.profile_cases [--case all|cumsum|group_reduce|recurrent|l2norm|cp_chain|dg_fix|gate_act] [--once]

Prints one line per kernel: time per launch, the bytes it must move (inputs read once + outputs written once) and the
achieved GB/s.  The same command under ``ncu -k regex:<kernel>`` gives the DRAM traffic of a launch.
"""
from __future__ import annotations

import argparse

import torch

from . import _lib, kernels
from .planner import plan_dense


_ONCE = False


def _time(fn, n=20):
    if _ONCE:  # one warm-up launch and one timed launch: the form for an ncu capture
        n = 1
    for _ in range(1 if _ONCE else 3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / n


def _report(name, ms, nbytes):
    print(f"{name:28s} {ms * 1e3:9.1f} us   {nbytes / 1e6:9.1f} MB   {nbytes / (ms * 1e-3) / 1e9:8.1f} GB/s", flush=True)


def case_cumsum():
    # the long-sequence shape: B=1, T=1M, H=8 fp32 (32 MiB in, 32 MiB out) - and a 64-head shape
    for T, H in ((1 << 20, 8), (1 << 18, 64)):
        g = torch.randn(1, T, H, device="cuda")
        plan = plan_dense(1, T)
        ms = _time(lambda: kernels.chunk_local_cumsum(g, reverse=True, plan=plan))
        _report(f"chunk_cumsum T={T} H={H}", ms, 2 * g.numel() * 4)


def case_group_reduce():
    lib = _lib.load()
    rows, H, Hg = 32768, 32, 16
    a = torch.randn(rows, H, 128, device="cuda").bfloat16()
    b = torch.randn(rows, H, 128, device="cuda").bfloat16()
    oa = torch.empty(rows, Hg, 128, device="cuda", dtype=torch.bfloat16)
    ob = torch.empty_like(oa)
    ms = _time(lambda: _lib.check(lib.fq_group_reduce_pair(a.data_ptr(), oa.data_ptr(), b.data_ptr(), ob.data_ptr(), rows, H, Hg,
                                                            kernels._stream()), "fq_group_reduce_pair"))
    _report("group_reduce (dq and dk)", ms, 2 * (a.numel() + oa.numel()) * 2)


def case_recurrent():
    from .decode import fused_recurrent_gated_delta_rule
    N, H = 128, 64
    q = torch.randn(N, 1, H, 128, device="cuda").bfloat16()
    k = torch.nn.functional.normalize(torch.randn(N, 1, H, 128, device="cuda"), dim=-1).bfloat16()
    v = torch.randn(N, 1, H, 128, device="cuda").bfloat16()
    g = torch.nn.functional.logsigmoid(torch.randn(N, 1, H, device="cuda"))
    beta = torch.rand(N, 1, H, device="cuda")
    state = 0.1 * torch.randn(N, H, 128, 128, device="cuda")
    ms = _time(lambda: fused_recurrent_gated_delta_rule(q, k, v, g, beta, initial_state=state, inplace_state=True))
    _report("gdr_recurrent (one token)", ms, 2 * state.numel() * 4 + 4 * q.numel() * 2)


def case_l2norm():
    from .ops import l2norm
    x = torch.randn(1, 1 << 18, 16, 128, device="cuda").bfloat16().requires_grad_()
    dy = torch.randn_like(x)
    ms = _time(lambda: l2norm(x))
    _report("l2norm forward", ms, 2 * x.numel() * 2)
    y = l2norm(x)
    ms = _time(lambda: torch.autograd.grad(y, x, dy, retain_graph=True))
    _report("l2norm backward", ms, 3 * x.numel() * 2)


def case_cp_chain():
    lib = _lib.load()
    P, H = 64, 32
    add = torch.randn(P, H, 128, 128, device="cuda")
    tm = torch.randn(P, H, 128, 128, device="cuda") / 12
    out = torch.empty(P + 1, H, 128, 128, device="cuda")
    flags = torch.ones(1, H, dtype=torch.int32, device="cuda")
    off = torch.tensor([0, P + 1], dtype=torch.int32, device="cuda")
    ms = _time(lambda: _lib.check(lib.fq_cp_chain_ex(add.data_ptr(), tm.data_ptr(), out.data_ptr(), flags.data_ptr(),
                                                      off.data_ptr(), None, 1, H, 0, 0, kernels._stream()), "fq_cp_chain_ex"))
    _report(f"cp_chain {P} pieces x {H} heads", ms, (add.numel() + tm.numel() + out.numel()) * 4)


def case_dg_fix():
    lib = _lib.load()
    B, T, H = 64, 256, 32    # many short sequences: the case the correction is made for
    nc = T // 64
    h0 = torch.randn(B, H, 128, 128, device="cuda")
    dht = torch.randn(B, H, 128, 128, device="cuda")
    h = torch.randn(B * nc, H, 128, 128, device="cuda").bfloat16()
    dh = torch.randn(B * nc, H, 128, 128, device="cuda").bfloat16()
    g = -torch.rand(B, T, H, device="cuda")
    dg = torch.zeros(B, T, H, device="cuda")
    ms = _time(lambda: _lib.check(lib.fq_dg_boundary_fix(h0.data_ptr(), dht.data_ptr(), h.data_ptr(), dh.data_ptr(), g.data_ptr(),
                                                          dg.data_ptr(), B, T, H, None, None, B, B * nc, kernels._stream()),
                                  "fq_dg_boundary_fix"))
    _report("dg_boundary_fix", ms, (h0.numel() + dht.numel()) * 4 + 2 * B * H * 128 * 128 * 2)


def case_gate_act():
    T, H = 1 << 20, 8
    dg = torch.randn(1, T, H, device="cuda")
    db = torch.randn(1, T, H, device="cuda")
    g_raw = torch.randn(1, T, H, device="cuda")
    b_raw = torch.randn(1, T, H, device="cuda")
    A_log = torch.zeros(H, device="cuda")
    dt_bias = torch.zeros(H, device="cuda")
    ms = _time(lambda: kernels.gate_act_bwd(dg, db, g_raw, b_raw, 2, 1, A_log, dt_bias))
    _report("gate_act_bwd", ms, 6 * dg.numel() * 4)


CASES = {"cumsum": case_cumsum, "group_reduce": case_group_reduce, "recurrent": case_recurrent, "l2norm": case_l2norm,
         "cp_chain": case_cp_chain, "dg_fix": case_dg_fix, "gate_act": case_gate_act}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default="all", choices=["all"] + sorted(CASES))
    ap.add_argument("--once", action="store_true", help="one warm-up and one timed launch per kernel (for ncu)")
    a = ap.parse_args()
    global _ONCE
    _ONCE = a.once
    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device")
    for name, fn in CASES.items():
        if a.case in ("all", name):
            fn()


if __name__ == "__main__":
    main()
