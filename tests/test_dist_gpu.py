"""GPU parity of the sequence-parallel path (flashqla_b200/dist.py with its CUDA implementation).

(1) On ONE GPU the ranks are emulated one after the other: every rank's CUDA steps (local tile kernel, summary state
    pass / replay, chains, local forward and backward with the boundary state / gradient) run exactly as under
    torch.distributed, and the all_gather is a torch.stack.  Compared with the single-GPU operator on the whole
    sequence and with the fp32 oracle.
(2) With two or more GPUs, two NCCL ranks run cp_forward / cp_backward for real (child processes, NVLS off) and are
    compared with the single-GPU operator.  Skipped on a one-GPU box.
(3) The chain kernel's modes (plain, from a given start, reverse, product of the transition matrices) against torch.

Tolerance (stated): 1e-2 rel-to-max for o and the bf16 / fp32 gradients, 5e-3 for the final state.
"""
import os
import socket
import subprocess
import sys

import pytest
import torch

from conftest import ROOT, check_close
from oracle import gdr_oracle as orc

pytestmark = pytest.mark.gpu
os.environ.setdefault("FLASHQLA_CHECK_STATUS", "1")
NAMES = ["dq", "dk", "dv", "db", "dg", "dh0"]


def _inputs(gates, T, H, seed=3):
    torch.manual_seed(seed)
    q = orc.l2norm(torch.randn(1, T, H, 128)).bfloat16()
    k = orc.l2norm(torch.randn(1, T, H, 128)).bfloat16()
    v = torch.randn(1, T, H, 128).bfloat16()
    g = torch.nn.functional.logsigmoid(torch.randn(1, T, H))
    beta = torch.randn(1, T, H).sigmoid()
    h0, dht = 0.1 * torch.randn(1, H, 128, 128), 0.01 * torch.randn(1, H, 128, 128)
    if gates == "reftest":   # the reference tests' distribution: slow decay, one head that never decays
        g = g / 16
        g[:, :, -1] = 0.0
        h0, dht = torch.randn(1, H, 128, 128), torch.randn(1, H, 128, 128) / 8
    do = torch.randn(1, T, H, 128).bfloat16()
    return [x.cuda() for x in (q, k, v, g, beta, h0, do, dht)]


@pytest.mark.parametrize("gates,T,H,world,pc", [("baseline", 4096, 2, 2, 8), ("reftest", 4096, 2, 2, 8), ("reftest", 6144 + 100, 3, 3, 16),
                                               ("reftest", 2048, 2, 4, 64), ("baseline", 16384, 2, 2, None)])
def test_emulated_ranks_match_single_gpu(gates, T, H, world, pc):
    from flashqla_b200 import dist as fqd
    from flashqla_b200 import ops
    q, k, v, g, beta, h0, do, dht = _inputs(gates, T, H)
    scale = 128 ** -0.5
    gc, A, o_ref, _, fs_ref = ops.chunk_gated_delta_rule_fwd(q, k, v, g, beta, scale, h0, None, True, False, True)
    ref = ops.chunk_gated_delta_rule_bwd(q, k, v, gc, beta, A, do, dht, scale, h0, None)
    impl = fqd.CudaImpl(piece_chunks=pc)
    b = fqd.shard_sequence(T, world)
    sl = [slice(b[r], b[r + 1]) for r in range(world)]
    part = lambda x, r: x[:, sl[r]].contiguous()
    ctx = [impl.prepare(part(q, r), part(k, r), part(v, r), part(g, r), part(beta, r), scale) for r in range(world)]
    summ = [impl.summary_fwd(ctx[r], h0 if r == 0 else None, r, world) for r in range(world)]
    b_all, t_all = torch.stack([s[0] for s in summ]), torch.stack([s[1] for s in summ])
    h_all = impl.chain(b_all, t_all, reverse=False)
    h_in = [h0] + [h_all[r:r + 1] for r in range(1, world)]
    outs = [impl.forward(ctx[r], h_in[r], want_final=(r == world - 1)) for r in range(world)]
    o = torch.cat([x[0] for x in outs], 1)
    check_close([o, outs[-1][1]], [o_ref, fs_ref], {"o": 1e-2, "final_state": 5e-3}, ["o", "final_state"], "vs single GPU: ")
    zero = torch.zeros(H, 128, 128, device="cuda")
    cs = [zero] + [impl.summary_bwd(ctx[r], part(do, r), dht if r == world - 1 else None, r, world) for r in range(1, world)]
    e_all = impl.chain(torch.stack(cs), t_all, reverse=True)
    e_in = [e_all[r:r + 1] for r in range(world - 1)] + [dht]
    grads = [impl.backward(ctx[r], part(do, r), e_in[r], h_in[r]) for r in range(world)]
    got = [torch.cat([gr[i] for gr in grads], 1) for i in range(5)] + [grads[0][5]]
    check_close(got, ref, 1e-2, NAMES, "vs single GPU: ")
    torch.cuda.synchronize()
    # and against the oracle
    cpu = lambda x: x.float().cpu()
    gcr, _, o_or, _, fs_or = orc.gdr_fwd(cpu(q), cpu(k), cpu(v), g.cpu(), beta.cpu(), scale, h0.cpu(), None)
    check_close([o, outs[-1][1]], [o_or, fs_or], {"o": 1e-2, "final_state": 5e-3}, ["o", "final_state"], "vs oracle: ")
    ref_or = orc.gdr_bwd(cpu(q), cpu(k), cpu(v), gcr, beta.cpu(), cpu(do), dht.cpu(), scale, h0.cpu(), None)
    check_close(got, ref_or, 1e-2, NAMES, "vs oracle: ")


def test_chain_kernel_modes():
    from flashqla_b200 import _lib, kernels
    lib, st = _lib.load(), kernels._stream()
    torch.manual_seed(0)
    P, H = 5, 3
    add = torch.randn(P, H, 128, 128, device="cuda")
    tm = torch.randn(P, H, 128, 128, device="cuda") / 12
    init = torch.randn(H, 128, 128, device="cuda")
    flags = torch.tensor([[1, 0, 1]], dtype=torch.int32, device="cuda")
    off = torch.tensor([0, P + 1], dtype=torch.int32, device="cuda")
    off_r = torch.tensor([0, P], dtype=torch.int32, device="cuda")

    def run(add_t, init_t, offsets, reverse, compose):
        out = torch.full((P + 1, H, 128, 128), float("nan"), device="cuda")
        rc = lib.fq_cp_chain_ex(None if add_t is None else add_t.data_ptr(), tm.data_ptr(), out.data_ptr(), flags.data_ptr(),
                                offsets.data_ptr(), None if init_t is None else init_t.data_ptr(), 1, H, reverse, compose, st)
        _lib.check(rc, "fq_cp_chain_ex")
        torch.cuda.synchronize()
        return out

    a, t = add.double(), tm.double()
    for h in (0, 2):
        # plain: out[1] = add[0]; out[r+1] = T_r out[r] + add[r]
        out = run(add, None, off, 0, 0)
        x = a[0, h]
        for r in range(P):
            if r > 0:
                x = t[r, h] @ x + a[r, h]
            assert (out[r + 1, h].double() - x).abs().max() < 1e-4 * x.abs().max(), ("plain", r)
        # from a given start: every step applies T
        out = run(add, init, off, 0, 0)
        x = init[h].double()
        for r in range(P):
            x = t[r, h] @ x + a[r, h]
            assert (out[r + 1, h].double() - x).abs().max() < 1e-4 * x.abs().max(), ("init", r)
        # product of the transition matrices
        out = run(None, None, off, 0, 1)
        x = t[0, h]
        for r in range(P):
            if r > 0:
                x = t[r, h] @ x
            assert (out[r + 1, h].double() - x).abs().max() < 1e-4 * x.abs().max(), ("compose", r)
        # reverse: out[P-2] = add[P-1]; out[r-1] = T_r^T out[r] + add[r]
        out = run(add, None, off_r, 1, 0)
        x = a[P - 1, h]
        for r in range(P - 1, 0, -1):
            if r < P - 1:
                x = t[r, h].T @ x + a[r, h]
            assert (out[r - 1, h].double() - x).abs().max() < 1e-4 * x.abs().max(), ("reverse", r)
    assert torch.isnan(run(add, None, off, 0, 0)[1:, 1]).all()   # the unflagged head is left alone


_CHILD = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, os.path.join(sys.argv[1], "tests"))
rank, world, gates = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), sys.argv[2]
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
from test_dist_gpu import _inputs
from conftest import check_close
from flashqla_b200 import dist as fqd, ops
T, H = 16384, 2
q, k, v, g, beta, h0, do, dht = _inputs(gates, T, H)
scale = 128 ** -0.5
gc, A, o_ref, _, fs_ref = ops.chunk_gated_delta_rule_fwd(q, k, v, g, beta, scale, h0, None, True, False, True)
ref = ops.chunk_gated_delta_rule_bwd(q, k, v, gc, beta, A, do, dht, scale, h0, None)
b = fqd.shard_sequence(T, world)
sl = slice(b[rank], b[rank + 1])
part = lambda x: x[:, sl].contiguous()
impl = fqd.CudaImpl(piece_chunks=16)
o, fs, saved = fqd.cp_forward(part(q), part(k), part(v), part(g), part(beta), scale, h0 if rank == 0 else None, None, impl=impl)
grads = fqd.cp_backward(saved, part(do), dht if rank == world - 1 else None, None, impl=impl)
torch.cuda.synchronize()
check_close([o, fs], [o_ref[:, sl], fs_ref], {"o": 1e-2, "final_state": 5e-3}, ["o", "final_state"], f"rank {rank}: ")
check_close(list(grads[:5]), [x[:, sl] for x in ref[:5]], 1e-2, ["dq", "dk", "dv", "db", "dg"], f"rank {rank}: ")
if rank == 0:
    check_close([grads[5]], [ref[5]], 1e-2, ["dh0"], "rank 0: ")
dist.barrier()
dist.destroy_process_group()
print(f"rank {rank} ok")
'''


@pytest.mark.parametrize("gates", ["baseline", "reftest"])
def test_two_nccl_ranks_match_single_gpu(gates, tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "child.py"
    script.write_text(_CHILD)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        procs.append(subprocess.Popen([sys.executable, str(script), ROOT, gates], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=300)
        except subprocess.TimeoutExpired:
            for p2 in procs:
                p2.kill()
            raise
        outs.append(out)
    for rank, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and f"rank {rank} ok" in out, out[-3000:]
