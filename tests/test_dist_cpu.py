"""world_size-2 gloo tests of the multi-GPU orchestration (sequence-parallel halo exchange and its exact
serial fallback, head sharding).  The local compute is injected: on these CPU ranks the oracle stands in for
the CUDA operator, so the test checks the exchange logic, not the kernels."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import gdr_oracle as orc


class OracleImpl:
    def fwd(self, q, k, v, g, beta, scale, h0):
        _, _, o, _, fs = orc.gdr_fwd(q, k, v, g, beta, scale, h0, None, dtype=torch.float64)
        return o.float(), fs.float()

    def bwd(self, q, k, v, g, beta, do, dht, scale, h0):
        gc = orc.chunk_local_cumsum(g, None, dtype=torch.float64)
        outs = orc.gdr_bwd(q, k, v, gc, beta, do, dht, scale, h0, None, dtype=torch.float64)
        return tuple(x.float() for x in outs)


def _inputs(dist_name, T=1024, H=2):
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
        o, fs, info = fqd.cp_forward(q[:, sl], k[:, sl], v[:, sl], g[:, sl], beta[:, sl], None,
                                     h0 if rank == 0 else None, None, halo_chunks=4, impl=impl)
        outs = fqd.cp_backward(q[:, sl], k[:, sl], v[:, sl], g[:, sl], beta[:, sl], do[:, sl],
                               dht if rank == world - 1 else None, None, info["h_in"], None, halo_chunks=4, impl=impl,
                               mode=info["mode"])
        out[rank] = dict(mode=info["mode"], o=o, fs=fs, grads=[x for x in outs], sl=(b[rank], b[rank + 1]))
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("dist_name,expect_mode", [("strong_gates", "halo"), ("zero_gate_head", "serial")])
def test_sequence_parallel_two_ranks(dist_name, expect_mode):
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), dist_name, out), nprocs=world, join=True)
    q, k, v, g, beta, h0, do, dht = _inputs(dist_name)
    _, _, o_ref, _, fs_ref = orc.gdr_fwd(q, k, v, g, beta, None, h0, None, dtype=torch.float64)
    gc = orc.chunk_local_cumsum(g, None, dtype=torch.float64)
    ref = orc.gdr_bwd(q, k, v, gc, beta, do, dht, None, h0, None, dtype=torch.float64)
    tol = 1e-5 if expect_mode == "halo" else 1e-5
    for r in range(world):
        res = out[r]
        assert res["mode"] == expect_mode
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
