"""Multi-GPU use of the operator (one process per GPU, torch.distributed).

Two patterns; the reference has no multi-GPU code at all:

* batch x head sharding - sequences and heads are independent, so every rank simply calls the
  operator on its own shard; no collective is involved (``shard_heads`` gives the slices that keep
  the V-heads of a QK group together, so the grouped-head dq / dk sum stays local).

* sequence (context) parallel for ONE very long sequence - rank r owns a contiguous range of
  tokens (a multiple of 64).  The state that enters a rank's range is rebuilt from a short HALO of
  the previous rank's last chunks: the gates make older history negligible once the accumulated
  log-decay over the halo is below ``threshold`` (the same argument as the in-GPU split).  One
  neighbour exchange of the halo tokens (k, v, g, beta: a few MB over NVLink) replaces the serial
  hand-over of boundary states.  When some head does not decay within the halo (e.g. g == 0), the
  ranks fall back to the exact serial chain: rank r waits for rank r-1's final state.  The
  backward mirrors this with the state gradient flowing right to left.

The compute is injected (``impl``) so that the orchestration can be exercised on CPU ranks
(gloo) with a stand-in; by default it is the CUDA operator of this package.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

CHUNK = 64


def shard_heads(Hq: int, Hv: int, world: int, rank: int):
    """(qk-head slice, v-head slice) of `rank` when the QK heads are split evenly over `world` ranks."""
    assert Hq % world == 0, "number of QK heads must be divisible by the number of ranks"
    per = Hq // world
    G = Hv // Hq
    return slice(rank * per, (rank + 1) * per), slice(rank * per * G, (rank + 1) * per * G)


def shard_sequence(T: int, world: int):
    """Token boundaries [world+1] of a contiguous split into multiples of 64 tokens (last rank takes the rest)."""
    n_chunks = (T + CHUNK - 1) // CHUNK
    base, rem = divmod(n_chunks, world)
    bounds = [0]
    for r in range(world):
        bounds.append(min(T, bounds[-1] + (base + (1 if r < rem else 0)) * CHUNK))
    bounds[-1] = T
    return bounds


class CudaImpl:
    """The operator of this package as the local compute."""

    def fwd(self, q, k, v, g, beta, scale, h0):
        from . import ops
        _, _, o, _, fs = ops.chunk_gated_delta_rule_fwd(q, k, v, g, beta, scale, h0, None, True, False, True)
        return o, fs

    def bwd(self, q, k, v, g, beta, do, dht, scale, h0):
        from . import ops
        g_cum, A, _, _, _ = ops.chunk_gated_delta_rule_fwd(q, k, v, g, beta, scale, h0, None, False, False, True)
        return ops.chunk_gated_delta_rule_bwd(q, k, v, g_cum, beta, A, do, dht, scale, h0, None)


def _chunk_decay(g):
    """Total log-decay of every whole 64-token chunk of g [1, T, H] -> [n, H]."""
    T = g.shape[1]
    n = T // CHUNK
    return g[0, :n * CHUNK].float().reshape(n, CHUNK, -1).sum(1)


def _exchange(send_list, recv_list, dst, src, group):
    """Post the sends to `dst` and the receives from `src` (either may be None) and wait for them."""
    ops_ = []
    if dst is not None:
        ops_ += [dist.P2POp(dist.isend, t.contiguous(), dst, group) for t in send_list]
    if src is not None:
        ops_ += [dist.P2POp(dist.irecv, t, src, group) for t in recv_list]
    if ops_:
        for w in dist.batch_isend_irecv(ops_):
            w.wait()


def _all_decayed(decay_rows, threshold):
    """True when, summed over the given chunks, every head's log-decay is below the threshold."""
    return bool((decay_rows.sum(0) < threshold).all().item()) if decay_rows.numel() else False


def cp_forward(q, k, v, g, beta, scale=None, initial_state=None, group=None, halo_chunks=8, threshold=-16.0,
               impl=None):
    """Forward of ONE sequence whose tokens are split contiguously over the ranks of `group`.

    Every rank passes its own token range ([1, T_local, ...], T_local a multiple of 64 except on the
    last rank) and gets its slice of `o`; `final_state` is returned on every rank (broadcast from the
    last one).  `initial_state` is used by rank 0.
    Returns (o_local, final_state, info) with info["mode"] in {"halo", "serial"}.
    """
    impl = impl or CudaImpl()
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    K = k.shape[-1]
    scale = K ** -0.5 if scale is None else scale
    H = v.shape[2]
    T_local = k.shape[1]
    n_local = T_local // CHUNK
    hc = min(halo_chunks, n_local)
    nxt = rank + 1 if rank + 1 < world else None
    prv = rank - 1 if rank > 0 else None
    ranks = dist.get_process_group_ranks(group) if group is not None else list(range(world))
    gr = lambda r: None if r is None else ranks[r]

    # ---- neighbour exchange of the last `hc` chunks (k, v, g, beta); all ranks use the same hc
    hc_t = torch.tensor([hc], device=k.device, dtype=torch.int32)
    dist.all_reduce(hc_t, op=dist.ReduceOp.MIN, group=group)
    hc = int(hc_t.item())
    ht = hc * CHUNK
    tail = lambda x: x[:, T_local - (T_local % CHUNK) - ht: T_local - (T_local % CHUNK)] if rank != world - 1 else x[:, :0]
    send = [tail(k), tail(v), tail(g), tail(beta)] if nxt is not None else []
    halo = [torch.empty((1, ht) + tuple(x.shape[2:]), dtype=x.dtype, device=x.device) for x in (k, v, g, beta)] \
        if prv is not None else []
    _exchange(send, halo, gr(nxt), gr(prv), group)

    # ---- can the halo stand in for the whole prefix?  (one tiny all-reduce decides for everybody)
    need_serial = torch.zeros(1, device=k.device, dtype=torch.int32)
    w = 0
    if prv is not None:
        dec = _chunk_decay(halo[2])                         # [hc, H]
        csum = torch.flip(torch.cumsum(torch.flip(dec, (0,)), 0), (0,))  # decay from chunk i to the halo end
        ok = (csum < threshold).all(1)                      # chunks from which every head has decayed
        idx = torch.nonzero(ok)
        if idx.numel() == 0:
            need_serial[0] = 1
        else:
            w = hc - int(idx.max().item())                  # replay the last w halo chunks
    dist.all_reduce(need_serial, op=dist.ReduceOp.MAX, group=group)

    if int(need_serial.item()) == 0:
        h_in = initial_state
        if prv is not None:
            hk, hv_, hg, hb = (x[:, ht - w * CHUNK:] for x in halo)
            _, h_in = impl.fwd(torch.zeros_like(hk), hk, hv_, hg, hb, scale, None)   # state only: q is irrelevant
        o, fs = impl.fwd(q, k, v, g, beta, scale, h_in)
        mode = "halo"
    else:
        # exact serial chain: wait for the previous rank's final state
        h_in = initial_state
        if prv is not None:
            h_in = torch.empty(1, H, K, v.shape[-1], dtype=torch.float32, device=k.device)
            dist.recv(h_in, gr(prv), group=group)
        o, fs = impl.fwd(q, k, v, g, beta, scale, h_in)
        if nxt is not None:
            dist.send(fs.contiguous(), gr(nxt), group=group)
        mode = "serial"
    fs = fs.contiguous()
    dist.broadcast(fs, gr(world - 1), group=group)
    return o, fs, {"mode": mode, "halo_chunks": hc, "replayed": w, "h_in": h_in}


def cp_backward(q, k, v, g, beta, do, dht=None, scale=None, h_in=None, group=None, halo_chunks=8, threshold=-16.0,
                impl=None, mode="halo"):
    """Backward of the sequence-parallel forward.  `h_in` is the state that entered this rank's range
    (info["h_in"] of cp_forward), `dht` the gradient of the final state (used by the last rank).
    Returns (dq, dk, dv, dbeta, dg) of the local tokens and dh0 (meaningful on rank 0)."""
    impl = impl or CudaImpl()
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    K = k.shape[-1]
    scale = K ** -0.5 if scale is None else scale
    H = v.shape[2]
    T_local = k.shape[1]
    nxt = rank + 1 if rank + 1 < world else None
    prv = rank - 1 if rank > 0 else None
    ranks = dist.get_process_group_ranks(group) if group is not None else list(range(world))
    gr = lambda r: None if r is None else ranks[r]
    hc_t = torch.tensor([min(halo_chunks, T_local // CHUNK)], device=k.device, dtype=torch.int32)
    dist.all_reduce(hc_t, op=dist.ReduceOp.MIN, group=group)
    hc = int(hc_t.item())
    ht = hc * CHUNK
    # the state gradient flows right to left: the halo is the NEXT rank's first chunks
    head = lambda x: x[:, :ht]
    send = [head(q), head(k), head(v), head(g), head(beta), head(do)] if prv is not None else []
    halo = [torch.empty((1, ht) + tuple(x.shape[2:]), dtype=x.dtype, device=x.device) for x in (q, k, v, g, beta, do)] \
        if nxt is not None else []
    _exchange(send, halo, gr(prv), gr(nxt), group)
    need_serial = torch.zeros(1, device=k.device, dtype=torch.int32)
    if mode == "serial":
        need_serial[0] = 1
    w = 0
    if nxt is not None:
        dec = _chunk_decay(halo[3])
        csum = torch.cumsum(dec, 0)                          # decay from the halo start through chunk i
        ok = (csum < threshold).all(1)
        idx = torch.nonzero(ok)
        if idx.numel() == 0:
            need_serial[0] = 1
        else:
            w = int(idx.min().item()) + 1
    dist.all_reduce(need_serial, op=dist.ReduceOp.MAX, group=group)
    if int(need_serial.item()) == 0:
        d_in = dht
        if nxt is not None:
            hq, hk, hv_, hg, hb, hdo = (x[:, :w * CHUNK] for x in halo)
            d_in = impl.bwd(hq, hk, hv_, hg, hb, hdo, None, scale, torch.zeros(1, H, K, v.shape[-1], device=k.device))[5]
        outs = impl.bwd(q, k, v, g, beta, do, d_in, scale, h_in if h_in is not None else torch.zeros(1, H, K, v.shape[-1], device=k.device))
    else:
        d_in = dht
        if nxt is not None:
            d_in = torch.empty(1, H, K, v.shape[-1], dtype=torch.float32, device=k.device)
            dist.recv(d_in, gr(nxt), group=group)
        outs = impl.bwd(q, k, v, g, beta, do, d_in, scale, h_in if h_in is not None else torch.zeros(1, H, K, v.shape[-1], device=k.device))
        if prv is not None:
            dist.send(outs[5].contiguous(), gr(prv), group=group)
    return outs
