"""world_size-2 and -3 gloo tests of the multi-GPU orchestration: the sequence-parallel exchange of per-rank
summaries (end state from zero, transition matrix; left-edge gradient) and the head / unit sharding helpers.  The
local compute is injected: on these CPU ranks an fp64 stand-in built on the oracle follows the same protocol as the
CUDA implementation, so the test checks the exchange logic (what is gathered, how it is chained, which state and
gradient enter which rank), not the kernels."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import gdr_oracle as orc

F64 = torch.float64


class OracleImpl:
    def prepare(self, q, k, v, g, beta, scale, want_grad=True):
        return dict(q=q, k=k, v=v, g=g, beta=beta, scale=scale)

    def summary_fwd(self, c, h0, rank, world):
        H, K = c["v"].shape[2], c["k"].shape[-1]
        _, _, _, _, B = orc.gdr_fwd(c["q"], c["k"], c["v"], c["g"], c["beta"], c["scale"], h0, None, dtype=F64)
        eye = torch.eye(K, dtype=F64).expand(1, H, K, K).contiguous()
        _, _, _, _, Tm = orc.gdr_fwd(c["q"], c["k"], torch.zeros_like(c["v"]), c["g"], c["beta"], c["scale"], eye, None, dtype=F64)
        return B[0].float(), Tm[0].float()

    def summary_bwd(self, c, do, dht, rank, world):
        gc = orc.chunk_local_cumsum(c["g"], None, dtype=F64)
        return orc.gdr_bwd(c["q"], c["k"], c["v"], gc, c["beta"], do, dht, c["scale"], None, None, dtype=F64)[5][0].float()

    def chain(self, add, tmat, reverse):
        W = add.shape[0]
        out = torch.zeros((W + 1,) + tuple(add.shape[1:]), dtype=F64)
        a, t = add.double(), tmat.double()
        if not reverse:
            out[1] = a[0]
            for r in range(1, W):
                out[r + 1] = t[r] @ out[r] + a[r]
        else:
            out[W - 2] = a[W - 1]
            for r in range(W - 2, 0, -1):
                out[r - 1] = t[r].transpose(-1, -2) @ out[r] + a[r]
        return out.float()

    def forward(self, c, h_in, want_final):
        _, _, o, _, fs = orc.gdr_fwd(c["q"], c["k"], c["v"], c["g"], c["beta"], c["scale"], h_in, None, dtype=F64)
        return o.float(), fs.float()

    def backward(self, c, do, e_in, h_in):
        gc = orc.chunk_local_cumsum(c["g"], None, dtype=F64)
        outs = orc.gdr_bwd(c["q"], c["k"], c["v"], gc, c["beta"], do, e_in, c["scale"], h_in, None, dtype=F64)
        return tuple(x.float() for x in outs)


def _inputs(dist_name, T=1536, H=2):
    torch.manual_seed(5)
    q = orc.l2norm(torch.randn(1, T, H, 128)); k = orc.l2norm(torch.randn(1, T, H, 128)); v = torch.randn(1, T, H, 128)
    g = torch.nn.functional.logsigmoid(torch.randn(1, T, H)); beta = torch.randn(1, T, H).sigmoid()
    if dist_name == "zero_gate_head":
        g = g / 16
        g[:, :, -1] = 0.0
    h0 = 0.1 * torch.randn(1, H, 128, 128); do = torch.randn(1, T, H, 128); dht = 0.01 * torch.randn(1, H, 128, 128)
    return q, k, v, g, beta, h0, do, dht


def _worker(rank, world, port, dist_name, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from flashqla_b200 import dist as fqd
        torch.set_num_threads(2)
        q, k, v, g, beta, h0, do, dht = _inputs(dist_name)
        T = q.shape[1]
        b = fqd.shard_sequence(T, world)
        sl = slice(b[rank], b[rank + 1])
        impl = OracleImpl()
        o, fs, saved = fqd.cp_forward(q[:, sl], k[:, sl], v[:, sl], g[:, sl], beta[:, sl], None,
                                      h0 if rank == 0 else None, None, impl=impl)
        outs = fqd.cp_backward(saved, do[:, sl], dht if rank == world - 1 else None, None, impl=impl)
        out[rank] = dict(o=o, fs=fs, grads=[x for x in outs], sl=(b[rank], b[rank + 1]))
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("dist_name,world", [("strong_gates", 2), ("zero_gate_head", 2), ("zero_gate_head", 3)])
def test_sequence_parallel_ranks(dist_name, world):
    """Every rank's slice of o, the final state and all gradients equal the single-process run - also with a head
    whose gate never decays: its exact (end state, transition matrix) pair travels instead of a replayed halo, and no
    rank waits for another rank's forward."""
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), dist_name, out), nprocs=world, join=True)
    q, k, v, g, beta, h0, do, dht = _inputs(dist_name)
    _, _, o_ref, _, fs_ref = orc.gdr_fwd(q, k, v, g, beta, None, h0, None, dtype=F64)
    gc = orc.chunk_local_cumsum(g, None, dtype=F64)
    ref = orc.gdr_bwd(q, k, v, gc, beta, do, dht, None, h0, None, dtype=F64)
    tol = 1e-5
    for r in range(world):
        res = out[r]
        s, e = res["sl"]
        assert orc.rel_to_max(res["o"], o_ref[:, s:e]) < tol
        assert orc.rel_to_max(res["fs"], fs_ref) < tol
        for name, got, full in zip(["dq", "dk", "dv", "db", "dg"], res["grads"][:5], ref[:5]):
            assert orc.rel_to_max(got, full[:, s:e]) < tol, (name, r)
    assert orc.rel_to_max(out[0]["grads"][5], ref[5]) < tol


def test_sharding_helpers():
    from flashqla_b200 import dist as fqd
    assert fqd.shard_sequence(1000, 4) == [0, 256, 512, 768, 1000]
    assert fqd.shard_sequence(1 << 20, 8)[3] == 3 * (1 << 17)
    qs, vs = fqd.shard_heads(16, 32, 8, 3)
    assert (qs.start, qs.stop, vs.start, vs.stop) == (6, 8, 12, 16)
    # B x Hq units over the ranks: whole batch rows first, then head groups inside a row
    bs, qs, vs = fqd.shard_units(4, 16, 32, 2, 1)
    assert (bs.start, bs.stop, qs.start, qs.stop, vs.start, vs.stop) == (2, 4, 0, 16, 0, 32)
    bs, qs, vs = fqd.shard_units(4, 16, 32, 8, 5)
    assert (bs.start, bs.stop, qs.start, qs.stop, vs.start, vs.stop) == (2, 3, 8, 16, 16, 32)
    seen = set()
    for r in range(8):
        bs, qs, _ = fqd.shard_units(4, 16, 32, 8, r)
        seen |= {(b, h) for b in range(bs.start, bs.stop) for h in range(qs.start, qs.stop)}
    assert len(seen) == 64
