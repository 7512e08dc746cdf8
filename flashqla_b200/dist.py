"""Multi-GPU use of the operator (one process per GPU, torch.distributed).  The reference has no multi-GPU code;
its context parallelism lives inside one card (flash_qla/ops/gated_delta_rule/chunk/cp_context.py:106-163).

Two patterns:

* batch x head sharding - sequences and heads are independent, so every rank simply calls the operator on its own
  shard; no collective is involved (``shard_heads`` gives the slices that keep the V-heads of a QK group together, so
  the grouped-head dq / dk sum stays local).

* sequence (context) parallel for ONE very long sequence - rank r owns a contiguous range of tokens (a multiple of
  64).  The state recurrence is affine in the state, so a rank's whole range acts on the state that enters it as

      S_out = T_r S_in + B_r            (T_r: K x K transition matrix, B_r: end state from a zero start)

  and the state gradient leaves it as  e_out = T_r^T e_in + C_r.  This is the pair ``(ht, mt)`` that the reference
  chains between the pieces of one card (hopper/prepare_h.py:245-277, hopper/cp_fwd.py:144-165), taken across GPUs:

    1. every rank forms its own summary ``(B_r, T_r)`` - PER HEAD: a head whose gate has decayed below
       ``threshold`` within a short stretch at the end of the range has T_r = 0 and gets B_r from a replay of that
       stretch alone; a head that does not decay (g = 0 heads) gets the exact pair from a state pass over the pieces of
       the range and two short chains;
    2. ONE all_gather of the summaries (2 x H x 64 KiB per rank), after which every rank chains the summaries of the
       ranks before it locally and owns the state that enters its range - no rank waits for another rank's forward;
    3. the ordinary forward on the local range with that state as ``initial_state``.

  The backward mirrors it with one all_gather of ``C_r`` (the transition matrices are kept from the forward).
  Nothing is read back to the host, so the exchange is stream-ordered like the rest of the operator.  The gathered
  tensors land in this GPU's memory through NCCL; the kernels only ever read local memory.

The local compute is injected (``impl``), so the exchange logic can run on CPU ranks (gloo) with a stand-in that follows
the same protocol; by default it is the CUDA implementation of this package.
"""
from __future__ import annotations

from collections import OrderedDict
from dataclasses import dataclass

import torch
import torch.distributed as dist

CHUNK = 64
_SKIP, _TRANSITION, _PIECE_START, _SEQ_START = 1 << 27, 1 << 28, 1 << 29, 1 << 30


def shard_heads(Hq: int, Hv: int, world: int, rank: int):
    """(qk-head slice, v-head slice) of `rank` when the QK heads are split evenly over `world` ranks."""
    assert Hq % world == 0, "number of QK heads must be divisible by the number of ranks"
    per = Hq // world
    G = Hv // Hq
    return slice(rank * per, (rank + 1) * per), slice(rank * per * G, (rank + 1) * per * G)


def shard_units(B: int, Hq: int, Hv: int, world: int, rank: int):
    """(batch slice, qk-head slice, v-head slice) of `rank` when the B x Hq (batch, QK-head group) units of a batch
    are split evenly over `world` ranks: whole batch rows first, then head groups inside a row."""
    assert (B * Hq) % world == 0, "B * Hq must be divisible by the number of ranks"
    G = Hv // Hq
    if world <= B:
        assert B % world == 0
        per = B // world
        return slice(rank * per, (rank + 1) * per), slice(0, Hq), slice(0, Hv)
    assert world % B == 0
    per_row = world // B                       # ranks that share one batch row
    b, part = divmod(rank, per_row)
    assert Hq % per_row == 0
    per = Hq // per_row
    return slice(b, b + 1), slice(part * per, (part + 1) * per), slice(part * per * G, (part + 1) * per * G)


def shard_sequence(T: int, world: int):
    """Token boundaries [world+1] of a contiguous split into multiples of 64 tokens (last rank takes the rest)."""
    n_chunks = (T + CHUNK - 1) // CHUNK
    base, rem = divmod(n_chunks, world)
    bounds = [0]
    for r in range(world):
        bounds.append(min(T, bounds[-1] + (base + (1 if r < rem else 0)) * CHUNK))
    bounds[-1] = T
    return bounds


# --------------------------------------------------------------------------------------------------------------------
# the CUDA implementation of the per-rank steps
@dataclass
class _SummaryPlan:
    """Pieces of a rank's local range for the state pass of the heads that need an exact summary (int32 device tensors)."""
    n_pieces: int
    n_chunks: int
    piece_cu: torch.Tensor       # [P+1] token boundaries of the pieces
    piece_off: torch.Tensor      # [P+1] prefix sums of chunks per piece
    zeros_p: torch.Tensor        # [P] zeros: every piece belongs to sequence 0 (slot of h0 / dht)
    entry_piece: torch.Tensor    # [2P] piece of every entry of the state pass (0..P-1 twice)
    entry_slot: torch.Tensor     # [2P] 0..2P-1
    slot_plus1: torch.Tensor     # [P] 1..P: where the gradient pass puts the left-edge gradient of piece p
    seq_end: torch.Tensor        # [P] first token after the range
    is_first: torch.Tensor       # [P] bool
    is_last: torch.Tensor        # [P] bool
    chain_off: torch.Tensor      # [2] = [0, P+1]: one virtual piece beyond the real ones
    v_end_cu: torch.Tensor       # [2] = [Tl, Tl]: the empty piece at the right end (forward summary)
    v_end_off: torch.Tensor      # [2] = [n_chunks, n_chunks]
    v_start: torch.Tensor        # [2] = [0, 0]: the empty piece at the left end (backward summary)
    scan_f: tuple                # (edge [1] = Tl, aux [1] = n_chunks)
    scan_r: tuple                # (edge [1] = 0, aux [1] = tokens of the last chunk, chunks_after [1] = n_chunks)
    zero1: torch.Tensor          # [1] zeros


_SP_CACHE: "OrderedDict[tuple, _SummaryPlan]" = OrderedDict()


def _summary_plan(Tl: int, L: int, device) -> _SummaryPlan:
    key = (Tl, L, str(device))
    hit = _SP_CACHE.get(key)
    if hit is not None:
        return hit
    from .planner import _to_device_i32 as t
    nl = (Tl + CHUNK - 1) // CHUNK
    starts = list(range(0, nl, L))
    P = len(starts)
    cu = [min(Tl, c * CHUNK) for c in starts] + [Tl]
    off = starts + [nl]
    d = lambda x: t(x, device)
    sp = _SummaryPlan(P, nl, d(cu), d(off), d([0] * P), d(list(range(P)) * 2), d(list(range(2 * P))),
                      d(list(range(1, P + 1))), d([Tl] * P),
                      torch.tensor([p == 0 for p in range(P)], device=device),
                      torch.tensor([p == P - 1 for p in range(P)], device=device),
                      d([0, P + 1]), d([Tl, Tl]), d([nl, nl]), d([0, 0]),
                      (d([Tl]), d([nl])), (d([0]), d([Tl - (nl - 1) * CHUNK]), d([nl])), d([0]))
    _SP_CACHE[key] = sp
    if len(_SP_CACHE) > 64:
        _SP_CACHE.popitem(last=False)
    return sp


class CudaImpl:
    """The kernels of this package as the local compute of the sequence-parallel protocol."""

    def __init__(self, threshold: float = -16.0, piece_chunks: int | None = None):
        self.threshold = float(threshold)
        self.piece_chunks = piece_chunks   # pieces of the summary state pass (None: the in-GPU planner's choice)

    # ---- local, chunk-parallel work: gate cumsum, A, gated tiles
    def prepare(self, q, k, v, g, beta, scale, want_grad=True):
        from . import kernels
        plan = kernels.make_plan(1, k.shape[1], None, q.device)
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        g_cum, A, Ag, _ = kernels.kkt_solve_fused(k, q, beta, g, scale, plan, want_A=want_grad)
        # the forward recurrence fills P_g (an input of the backward kernels)
        Pg = torch.empty_like(Ag) if want_grad else None
        bf = beta.contiguous() if beta.dtype == torch.float32 else beta.float().contiguous()
        return dict(q=q, k=k, v=v, beta=bf, g_cum=g_cum, A=A, Ag=Ag, Pg=Pg, scale=float(scale), plan=plan,
                    H=v.shape[2], Hg=k.shape[2], Tl=k.shape[1], want_grad=want_grad)

    def _pieces(self, c):
        from . import kernels
        from .planner import plan_cp
        if "sp" not in c:
            L = self.piece_chunks
            nl = (c["Tl"] + CHUNK - 1) // CHUNK
            if L is None:
                cp = plan_cp(c["plan"], 1, c["Tl"], c["H"], kernels.sm_count(c["q"].device), c["q"].device)
                L = cp.piece_chunks if cp is not None else nl
            c["sp"] = _summary_plan(c["Tl"], max(1, min(L, nl)), c["q"].device)
            c["cap"] = max(1, min(L, nl))
        return c["sp"]

    def _scan(self, c, rank, world):
        """Replay codes of the two virtual pieces and the per-head decision `exact` (bool [H]): the head's summary
        comes from the state pass instead of a replay."""
        if "exact" in c:
            return
        from . import _lib, kernels
        lib, st = _lib.load(), kernels._stream()
        sp, H, dev = self._pieces(c), c["H"], c["q"].device
        flags = torch.zeros(1, H, dtype=torch.int32, device=dev)
        raw_f = torch.zeros(1, H, dtype=torch.int32, device=dev)
        raw_r = torch.zeros(1, H, dtype=torch.int32, device=dev)
        g = c["g_cum"]
        if rank < world - 1:   # forward summary: walk back from the end of the range
            rc = lib.fq_cp_warmup(g.data_ptr(), sp.scan_f[0].data_ptr(), sp.scan_f[1].data_ptr(), None, raw_f.data_ptr(), 1, H,
                                  self.threshold, 0, c["cap"], sp.zero1.data_ptr(), flags.data_ptr(), st)
            _lib.check(rc, "fq_cp_warmup")
        if rank > 0:           # backward summary: walk forward from the start of the range
            rc = lib.fq_cp_warmup(g.data_ptr(), sp.scan_r[0].data_ptr(), sp.scan_r[1].data_ptr(), sp.scan_r[2].data_ptr(),
                                  raw_r.data_ptr(), 1, H, self.threshold, 1, c["cap"], sp.zero1.data_ptr(), flags.data_ptr(), st)
            _lib.check(rc, "fq_cp_warmup")
        exact = flags[0] != 0
        # a walk that reached the far end of the range without enough decay is only exact where that end is the end of
        # the whole sequence (rank 0 forward, last rank backward); elsewhere the head needs the exact pair too
        if rank > 0:
            exact = exact | ((raw_f[0] >> 30) & 1).bool()
        if rank < world - 1:
            exact = exact | ((raw_r[0] >> 30) & 1).bool()
        c.update(exact=exact, exact_i32=exact.to(torch.int32).reshape(1, H).contiguous(), raw_f=raw_f, raw_r=raw_r)

    # ---- forward summary (B_r, T_r) of the local range
    def summary_fwd(self, c, h0, rank, world):
        from . import _lib, kernels
        lib, st = _lib.load(), kernels._stream()
        sp, H, Hg, dev = self._pieces(c), c["H"], c["Hg"], c["q"].device
        self._scan(c, rank, world)
        P, K = sp.n_pieces, 128
        exact = c["exact"]
        need_b, need_t = rank < world - 1, rank > 0      # rank 0's T and the last rank's B have no reader
        p = lambda t: None if t is None else t.data_ptr()
        # state pass over 2P entries for the exact heads: B_p (end state from zero; rank 0's first piece from h0), T_p
        ex = exact[None, :]
        skip = torch.full((P, H), _SKIP, dtype=torch.int32, device=dev)
        code_b = torch.where(ex, torch.where(sp.is_first[:, None] & (rank == 0), _SEQ_START, 0).to(torch.int32), skip) \
            if need_b else skip
        # the transition matrices serve the chain of the piece states (every piece but the range's first), the
        # product T_r and the backward's reverse chain (every piece)
        code_t = torch.where(ex & ~(sp.is_first[:, None] & (not need_t)), torch.full_like(skip, _TRANSITION), skip)
        codes = torch.cat([code_b, code_t], 0).contiguous()
        bt = torch.empty(2 * P, H, K, K, dtype=torch.float32, device=dev)
        rc = lib.fq_gdr_fwd_cp_ex(c["q"].data_ptr(), c["k"].data_ptr(), c["v"].data_ptr(), c["Ag"].data_ptr(), None,
                                  c["g_cum"].data_ptr(), c["beta"].data_ptr(), p(h0), bt.data_ptr(), sp.entry_slot.data_ptr(),
                                  sp.zeros_p.data_ptr(), codes.data_ptr(), sp.entry_piece.data_ptr(), 2 * P, None, None, None,
                                  1, c["Tl"], H, Hg, sp.piece_cu.data_ptr(), sp.piece_off.data_ptr(), P, sp.n_chunks,
                                  c["scale"], None, st)
        _lib.check(rc, "fq_gdr_fwd_cp_ex (summary state pass)")
        c["bt"] = bt
        zero = torch.zeros(H, K, K, dtype=torch.float32, device=dev)
        Bout, Tout = zero, zero
        if need_b:
            # exact heads: chain of the piece states from zero; slot P = the state at the end of the range
            s_piece = torch.empty(P + 1, H, K, K, dtype=torch.float32, device=dev)
            rc = lib.fq_cp_chain_ex(bt.data_ptr(), bt[P:].data_ptr(), s_piece.data_ptr(), c["exact_i32"].data_ptr(),
                                    sp.chain_off.data_ptr(), None, 1, H, 0, 0, st)
            _lib.check(rc, "fq_cp_chain_ex")
            # all heads: the empty piece at the end of the range.  Exact heads start from the chained state (nothing to
            # run), the others replay the last chunks from zero (rank 0: from h0 when the walk reached the start)
            vcode = torch.where(ex, torch.full_like(c["raw_f"], _PIECE_START), c["raw_f"]).contiguous()
            Bout = torch.empty(1, H, K, K, dtype=torch.float32, device=dev)
            rc = lib.fq_gdr_fwd_cp_ex(c["q"].data_ptr(), c["k"].data_ptr(), c["v"].data_ptr(), c["Ag"].data_ptr(), None,
                                      c["g_cum"].data_ptr(), c["beta"].data_ptr(), p(h0), Bout.data_ptr(), sp.zero1.data_ptr(),
                                      sp.zero1.data_ptr(), vcode.data_ptr(), None, 1, s_piece[P:].data_ptr(), None, None, 1,
                                      c["Tl"], H, Hg, sp.v_end_cu.data_ptr(), sp.v_end_off.data_ptr(), 1, sp.n_chunks,
                                      c["scale"], None, st)
            _lib.check(rc, "fq_gdr_fwd_cp_ex (summary replay)")
            Bout = Bout[0]
        if need_t:
            x_piece = torch.empty(P + 1, H, K, K, dtype=torch.float32, device=dev)
            rc = lib.fq_cp_chain_ex(None, bt[P:].data_ptr(), x_piece.data_ptr(), c["exact_i32"].data_ptr(),
                                    sp.chain_off.data_ptr(), None, 1, H, 0, 1, st)
            _lib.check(rc, "fq_cp_chain_ex (compose)")
            Tout = torch.where(exact[:, None, None], x_piece[P], zero)
        return Bout, Tout

    # ---- backward summary C_r: the state gradient that leaves the range at its left edge when none enters at the right
    def summary_bwd(self, c, do, dht, rank, world):
        from . import _lib, kernels
        lib, st = _lib.load(), kernels._stream()
        sp, H, Hg, dev = self._pieces(c), c["H"], c["Hg"], c["q"].device
        self._scan(c, rank, world)
        P, K = sp.n_pieces, 128
        exact, ex = c["exact"], c["exact"][None, :]
        p = lambda t: None if t is None else t.data_ptr()
        do = do.contiguous()
        last_rank = rank == world - 1
        dh_scratch = torch.empty(sp.n_chunks, H, K, K, dtype=torch.bfloat16, device=dev)
        args = (c["q"].data_ptr(), c["k"].data_ptr(), c["Ag"].data_ptr(), c["Pg"].data_ptr(), do.data_ptr(),
                c["g_cum"].data_ptr(), c["beta"].data_ptr(), p(dht))
        # gradient pass of the exact heads: left-edge gradient C_p of every piece from zero (the last piece of the last
        # rank from dht), into slots 1..P
        skip = torch.full((P, H), _SKIP, dtype=torch.int32, device=dev)
        code_c = torch.where(ex, torch.where(sp.is_last[:, None] & last_rank, _SEQ_START, 0).to(torch.int32), skip).contiguous()
        c_ext = torch.empty(P + 1, H, K, K, dtype=torch.float32, device=dev)
        rc = lib.fq_gdr_bwd_dh_cp_ex(*args, c_ext.data_ptr(), dh_scratch.data_ptr(), sp.zeros_p.data_ptr(),
                                     sp.slot_plus1.data_ptr(), sp.seq_end.data_ptr(), code_c.data_ptr(), None, 1, c["Tl"], H, Hg,
                                     sp.piece_cu.data_ptr(), sp.piece_off.data_ptr(), P, sp.n_chunks, c["scale"], None, st)
        _lib.check(rc, "fq_gdr_bwd_dh_cp_ex (summary gradient pass)")
        # e_{p-1} = T_p^T e_p + C_p down the pieces (pieces sit at index p + 1, so that slot 0 receives the gradient
        # that leaves the range); the transition matrices are those of the forward's state pass
        bt = c["bt"]
        e_ext = torch.empty(P + 1, H, K, K, dtype=torch.float32, device=dev)
        rc = lib.fq_cp_chain_ex(c_ext.data_ptr(), bt[P - 1:].data_ptr(), e_ext.data_ptr(), c["exact_i32"].data_ptr(),
                                sp.chain_off.data_ptr(), None, 1, H, 1, 0, st)
        _lib.check(rc, "fq_cp_chain_ex (reverse)")
        # all heads: the empty piece at the start of the range
        vcode = torch.where(ex, torch.full_like(c["raw_r"], _PIECE_START), c["raw_r"]).contiguous()
        Cout = torch.empty(1, H, K, K, dtype=torch.float32, device=dev)
        rc = lib.fq_gdr_bwd_dh_cp_ex(*args, Cout.data_ptr(), dh_scratch.data_ptr(), sp.zero1.data_ptr(), sp.zero1.data_ptr(),
                                     sp.seq_end.data_ptr(), vcode.data_ptr(), e_ext.data_ptr(), 1, c["Tl"], H, Hg,
                                     sp.v_start.data_ptr(), sp.v_start.data_ptr(), 1, sp.n_chunks, c["scale"], None, st)
        _lib.check(rc, "fq_gdr_bwd_dh_cp_ex (summary replay)")
        return Cout[0]

    # ---- chains of the rank summaries (gathered): states entering every rank / gradients entering every rank
    def chain(self, add, tmat, reverse):
        from . import _lib, kernels
        from .planner import _to_device_i32
        W, H = add.shape[0], add.shape[1]
        dev = add.device
        out = torch.zeros(W + 1, H, 128, 128, dtype=torch.float32, device=dev)
        ones = torch.ones(1, H, dtype=torch.int32, device=dev)
        add, tmat = add.contiguous(), tmat.contiguous()
        if not reverse:
            # out[r+1] = T_r out[r] + B_r, out[1] = B_0 (rank 0's summary already contains the initial state)
            off = _to_device_i32([0, W + 1], dev)
            rc = _lib.load().fq_cp_chain_ex(add.data_ptr(), tmat.data_ptr(), out.data_ptr(), ones.data_ptr(), off.data_ptr(),
                                            None, 1, H, 0, 0, kernels._stream())
        else:
            # out[r-1] = T_r^T out[r] + C_r, out[W-2] = C_{W-1} (the last rank's summary already contains dht)
            off = _to_device_i32([0, W], dev)
            rc = _lib.load().fq_cp_chain_ex(add.data_ptr(), tmat.data_ptr(), out.data_ptr(), ones.data_ptr(), off.data_ptr(),
                                            None, 1, H, 1, 0, kernels._stream())
        _lib.check(rc, "fq_cp_chain_ex (ranks)")
        return out

    # ---- the ordinary local passes with the boundary state / gradient
    def forward(self, c, h_in, want_final):
        from . import kernels
        from .planner import plan_cp
        dev = c["q"].device
        cp = plan_cp(c["plan"], 1, c["Tl"], c["H"], kernels.sm_count(dev), dev)
        warm = kernels.cp_warmup(c["g_cum"], cp, c["H"]) if cp is not None else None
        # a forward whose backward follows keeps the bf16 state before every chunk when it fits the budget of the
        # single-GPU operator (FLASHQLA_KEEP_STATES_MB): the backward then skips its state pass
        from .ops import _KEEP_STATES_BYTES
        keep_h = c["want_grad"] and c["plan"].total_chunks * c["H"] * 128 * 128 * 2 <= _KEEP_STATES_BYTES
        o, h, fs = kernels.fused_gdr_fwd(c["q"], c["k"], c["v"], c["Ag"], c["Pg"], c["g_cum"], c["beta"], c["scale"],
                                         initial_state=h_in, output_final_state=want_final, output_h=keep_h, plan=c["plan"],
                                         cp=cp, warmup=warm)
        c["h"] = h
        return o, fs

    def backward(self, c, do, e_in, h_in):
        from . import bwd
        return bwd.chunk_gated_delta_rule_bwd(c["q"], c["k"], c["v"], c["g_cum"], c["beta"], c["A"], do, e_in, c["scale"], h_in,
                                              None, gated_tiles=(c["Ag"], c["Pg"]), plan=c["plan"], want_dh0=True,
                                              h_saved=c.get("h"))


# --------------------------------------------------------------------------------------------------------------------
# the protocol
def _gather(x, group):
    world = dist.get_world_size(group)
    flat = x.contiguous().reshape(-1)
    out = torch.empty(world * flat.numel(), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, flat, group=group)
    return out.reshape((world,) + tuple(x.shape))


def cp_forward(q, k, v, g, beta, scale=None, initial_state=None, group=None, impl=None, want_grad=True):
    """Forward of ONE sequence whose tokens are split contiguously over the ranks of `group`.

    Every rank passes its own token range ([1, T_local, ...], T_local a multiple of 64 except on the last rank) and
    gets its slice of `o`; `final_state` is returned on every rank (broadcast from the last one).  `initial_state`
    ([1, H, 128, 128]) is used by rank 0.  Returns (o_local, final_state, saved) where `saved` goes to cp_backward.
    """
    impl = impl or CudaImpl()
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    scale = k.shape[-1] ** -0.5 if scale is None else scale
    c = impl.prepare(q, k, v, g, beta, scale, want_grad)
    h_in = initial_state
    t_all = None
    if world > 1:
        B_r, T_r = impl.summary_fwd(c, initial_state if rank == 0 else None, rank, world)
        both = _gather(torch.stack([B_r, T_r]), group)                    # [W, 2, H, 128, 128]
        t_all = both[:, 1]
        h_all = impl.chain(both[:, 0], t_all, reverse=False)              # h_all[r]: the state that enters rank r (r >= 1)
        if rank > 0:
            h_in = h_all[rank:rank + 1]
    o, fs = impl.forward(c, h_in, want_final=(rank == world - 1))
    if world > 1:
        if fs is None:
            fs = torch.empty(1, v.shape[2], k.shape[-1], v.shape[-1], dtype=torch.float32, device=k.device)
        fs = fs.contiguous()
        ranks = dist.get_process_group_ranks(group) if group is not None else list(range(world))
        dist.broadcast(fs, ranks[world - 1], group=group)
    saved = dict(ctx=c, h_in=h_in, t_all=t_all)
    return o, fs, saved


def cp_backward(saved, do, dht=None, group=None, impl=None):
    """Backward of cp_forward.  `dht` is the gradient of the final state (used by the last rank).  Returns
    (dq, dk, dv, dbeta, dg) of the local tokens and dh0 (the gradient of `initial_state`; meaningful on rank 0)."""
    impl = impl or CudaImpl()
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    c, h_in = saved["ctx"], saved["h_in"]
    e_in = dht
    if world > 1:
        H = do.shape[2]
        if rank > 0:
            C_r = impl.summary_bwd(c, do, dht if rank == world - 1 else None, rank, world)
        else:
            C_r = torch.zeros(H, 128, 128, dtype=torch.float32, device=do.device)
        c_all = _gather(C_r, group)                                        # [W, H, 128, 128]
        e_all = impl.chain(c_all, saved["t_all"], reverse=True)            # e_all[r]: the gradient that enters rank r
        if rank < world - 1:
            e_in = e_all[rank:rank + 1]
    return impl.backward(c, do, e_in, h_in)
