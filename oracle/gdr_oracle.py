"""CPU oracle for the chunked gated-delta-rule (GDN) forward and backward.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package may import this file:
it is the checker used by the tests, by the smoke entry and by the CPU-baseline
leg of the benchmark.  It is never the thing that is shipped or measured as the
product.

What it restates (paths are relative to the FlashQLA project root):

* ``tests/ref_gdr.py:560-615``  chunk_gated_delta_rule_fwd  (the reference's own
  PyTorch implementation: cumsum -> KK^T -> solve -> w/u -> state recurrence -> o)
* ``tests/ref_gdr.py:618-700``  chunk_gated_delta_rule_bwd
* the kernel algebra of ``flash_qla/ops/gated_delta_rule/chunk/hopper/kkt_solve.py:101-165``
  (gate-free inverse ``A = (I + tril(diag(beta) K K^T, -1))^-1``),
  ``hopper/fused_fwd.py:225-360`` (U, W, A_g, V_d, V', P_g, O, state update) and
  ``hopper/fused_bwd.py:303-759`` (the fused backward formulas),
* tail-chunk conventions of ``flash_qla/utils/pack.py:52-83`` (padded g = last
  valid cumsum, padded beta/q/k/v = 0).

Parity pin: the functions here are checked against outputs of the UNMODIFIED
``tests/ref_gdr.py`` (imported by file path through a small shim) that are stored
under ``tests/golden/`` together with the script that produced them
(``tests/golden/make_golden.py``).

Everything is plain torch on the CPU, in the dtype given by ``dtype`` (fp32 by
default, fp64 for tight algebra checks).  Work is vectorised over heads and over
the chunks of one sequence; only the inter-chunk recurrences are Python loops.
"""

from __future__ import annotations

import math

import torch

CHUNK = 64


# --------------------------------------------------------------------------- helpers
def l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """x * rsqrt(sum(x^2) + eps) over the last dim  (flash_qla/utils/math.py:7-21)."""
    xf = x.float()
    return (xf * torch.rsqrt((xf * xf).sum(-1, keepdim=True) + eps)).to(x.dtype)


def _seq_bounds(B: int, T: int, cu_seqlens):
    """List of (batch_index, start, end) for every sequence."""
    if cu_seqlens is None:
        return [(b, 0, T) for b in range(B)]
    cu = [int(x) for x in cu_seqlens.tolist()]
    return [(0, cu[i], cu[i + 1]) for i in range(len(cu) - 1)]


def _pad_chunks(x: torch.Tensor, n_chunks: int) -> torch.Tensor:
    """[T, ...] -> [N, C, ...] zero padded (flash_qla/utils/pack.py:38-49)."""
    T = x.shape[0]
    pad = n_chunks * CHUNK - T
    if pad:
        x = torch.cat([x, x.new_zeros((pad,) + tuple(x.shape[1:]))], 0)
    return x.reshape((n_chunks, CHUNK) + tuple(x.shape[1:]))


def chunk_local_cumsum(g: torch.Tensor, cu_seqlens=None, reverse: bool = False,
                       dtype=torch.float32) -> torch.Tensor:
    """Inclusive prefix sum (or suffix sum) of g inside every 64-token chunk.

    Chunks restart at every sequence start.  tests/ref_gdr.py:15-39;
    flash_qla/ops/utils/cumsum.py:131-165.
    """
    B, T, H = g.shape
    out = torch.empty_like(g, dtype=dtype)
    for b, s, e in _seq_bounds(B, T, cu_seqlens):
        L = e - s
        if L == 0:
            continue
        n = (L + CHUNK - 1) // CHUNK
        x = _pad_chunks(g[b, s:e].to(dtype), n)  # [N, C, H]
        if reverse:
            x = torch.flip(torch.flip(x, (1,)).cumsum(1), (1,))
        else:
            x = x.cumsum(1)
        out[b, s:e] = x.reshape(n * CHUNK, H)[:L]
    return out


def _prep_seq(q, k, v, gc, beta, dtype):
    """Chunk one sequence.  q,k [L,Hg,K]; v [L,H,V]; gc,beta [L,H]  ->  head-major chunk tensors."""
    L, Hg, _ = k.shape
    H = v.shape[1]
    n = (L + CHUNK - 1) // CHUNK
    rep = H // Hg
    kk = k.to(dtype).repeat_interleave(rep, dim=1) if rep > 1 else k.to(dtype)
    Kc = _pad_chunks(kk, n).permute(2, 0, 1, 3)  # [H,N,C,K]
    Vc = _pad_chunks(v.to(dtype), n).permute(2, 0, 1, 3)
    Bc = _pad_chunks(beta.to(dtype), n).permute(2, 0, 1)  # [H,N,C]  (padded beta = 0)
    Gc = _pad_chunks(gc.to(dtype), n).permute(2, 0, 1).clone()
    tail = L - (n - 1) * CHUNK
    if tail < CHUNK:  # padded rows take the last valid cumsum (pack.py:52-83)
        Gc[:, -1, tail:] = Gc[:, -1, tail - 1:tail]
    Qc = None
    if q is not None:
        qq = q.to(dtype).repeat_interleave(rep, dim=1) if rep > 1 else q.to(dtype)
        Qc = _pad_chunks(qq, n).permute(2, 0, 1, 3)
    return Qc, Kc, Vc, Gc, Bc, n, tail


def _decay_mask(Gc: torch.Tensor) -> torch.Tensor:
    """G[i,j] = exp(g_i - g_j) for i >= j else 0 (never exponentiates a positive number)."""
    d = Gc[..., :, None] - Gc[..., None, :]
    keep = torch.ones(CHUNK, CHUNK, dtype=torch.bool).tril()
    return torch.where(keep, d, d.new_full((), -math.inf)).exp()


def kkt_inverse(Kc: torch.Tensor, Bc: torch.Tensor) -> torch.Tensor:
    """Gate-free A = (I + tril(diag(beta) K K^T, -1))^-1 per chunk and head.

    hopper/kkt_solve.py:101-165.  The reference's torch version
    (tests/ref_gdr.py:42-104) folds the gate in: A_ref = A o G.
    """
    Lm = torch.tril(Bc[..., :, None] * (Kc @ Kc.transpose(-1, -2)), -1)
    eye = torch.eye(CHUNK, dtype=Kc.dtype).expand_as(Lm)
    return torch.linalg.solve_triangular(eye + Lm, eye.clone(), upper=False)


# --------------------------------------------------------------------------- forward
def gdr_fwd(q, k, v, g, beta, scale=None, initial_state=None, cu_seqlens=None,
            output_h: bool = False, dtype=torch.float32):
    """Chunked GDN forward.

    Shapes: q,k [B,T,Hg,K]; v [B,T,H,V]; g,beta [B,T,H] (g = raw log-gate);
    initial_state [N,H,K,V] or None; cu_seqlens int [N+1] or None (then B must be 1).

    Returns (g_cumsum [B,T,H], A [B,T,H,64] gate-free, o [B,T,H,V],
             h [B,Nc_total,H,K,V] or None (state BEFORE each chunk), final_state [N,H,K,V]).
    Follows tests/ref_gdr.py:560-615 in the algebra of hopper/fused_fwd.py:225-360.
    """
    B, T, Hg, K = k.shape
    H, V = v.shape[2], v.shape[3]
    scale = K ** -0.5 if scale is None else scale
    gc_all = chunk_local_cumsum(g, cu_seqlens, dtype=dtype)
    seqs = _seq_bounds(B, T, cu_seqlens)
    o = torch.zeros(B, T, H, V, dtype=dtype)
    A_out = torch.zeros(B, T, H, CHUNK, dtype=dtype)
    final = torch.zeros(len(seqs), H, K, V, dtype=dtype)
    hs = []
    for si, (b, s, e) in enumerate(seqs):
        L = e - s
        S = (torch.zeros(H, K, V, dtype=dtype) if initial_state is None
             else initial_state[si].to(dtype).clone())
        if L == 0:
            final[si] = S
            continue
        Qc, Kc, Vc, Gc, Bc, n, tail = _prep_seq(q[b, s:e], k[b, s:e], v[b, s:e],
                                                 gc_all[b, s:e], beta[b, s:e], dtype)
        A = kkt_inverse(Kc, Bc)
        Gm = _decay_mask(Gc)
        Ag = A * Gm * Bc[..., None, :]
        Pg = scale * Gm * (Qc @ Kc.transpose(-1, -2))
        gam = Gc.exp()  # e^{g_i}
        rho = (Gc[..., -1:] - Gc).exp()  # e^{g_last - g_i}
        if tail < CHUNK:
            rho[:, -1, tail:] = 0.0  # padded rows never reach the state
        gL = gam[..., -1]
        oc = torch.empty(H, n, CHUNK, V, dtype=dtype)
        for c in range(n):
            if output_h:
                hs.append(S.clone())
            U = Kc[:, c] @ S
            W = Vc[:, c] - gam[:, c, :, None] * U
            Vd = Ag[:, c] @ W
            oc[:, c] = scale * gam[:, c, :, None] * (Qc[:, c] @ S) + Pg[:, c] @ Vd
            S = gL[:, c, None, None] * S + Kc[:, c].transpose(-1, -2) @ (rho[:, c, :, None] * Vd)
        final[si] = S
        o[b, s:e] = oc.permute(1, 2, 0, 3).reshape(n * CHUNK, H, V)[:L]
        A_out[b, s:e] = A.permute(1, 2, 0, 3).reshape(n * CHUNK, H, CHUNK)[:L]
    h = None
    if output_h:
        h = torch.stack(hs, 0)  # [Nc_total(seq-major), H, K, V]
        if cu_seqlens is None:
            h = h.reshape(B, -1, H, K, V)
        else:
            h = h[None]
    return gc_all, A_out, o, h, final


# --------------------------------------------------------------------------- backward
def gdr_bwd(q, k, v, g_cumsum, beta, do, dht=None, scale=None, initial_state=None,
            cu_seqlens=None, dtype=torch.float32):
    """Chunked GDN backward in the fused-kernel algebra (hopper/fused_bwd.py:303-759).

    ``g_cumsum`` is the chunk-local cumsum returned by the forward.  Returns
    (dq [B,T,Hg,K], dk, dv [B,T,H,V], dbeta [B,T,H], dg [B,T,H] w.r.t. the RAW gate,
    dh0 [N,H,K,V]).  dq/dk are summed over the V-heads of each QK head
    (tests/ref_gdr.py:694-698); dg is turned from d/d(cumsum) into d/d(raw) by a
    reverse chunk-local cumsum (tests/ref_gdr.py:699).
    """
    B, T, Hg, K = k.shape
    H, V = v.shape[2], v.shape[3]
    scale = K ** -0.5 if scale is None else scale
    seqs = _seq_bounds(B, T, cu_seqlens)
    dq = torch.zeros(B, T, H, K, dtype=dtype)
    dk = torch.zeros(B, T, H, K, dtype=dtype)
    dv = torch.zeros(B, T, H, V, dtype=dtype)
    db = torch.zeros(B, T, H, dtype=dtype)
    dgc = torch.zeros(B, T, H, dtype=dtype)
    dh0 = torch.zeros(len(seqs), H, K, V, dtype=dtype)
    keepl = torch.ones(CHUNK, CHUNK, dtype=torch.bool).tril(-1)
    for si, (b, s, e) in enumerate(seqs):
        L = e - s
        dS = (torch.zeros(H, K, V, dtype=dtype) if dht is None else dht[si].to(dtype).clone())
        if L == 0:
            dh0[si] = dS
            continue
        Qc, Kc, Vc, Gc, Bc, n, tail = _prep_seq(q[b, s:e], k[b, s:e], v[b, s:e],
                                                 g_cumsum[b, s:e], beta[b, s:e], dtype)
        dOc = _pad_chunks(do[b, s:e].to(dtype), n).permute(2, 0, 1, 3)
        A = kkt_inverse(Kc, Bc)
        Gm = _decay_mask(Gc)
        Ab = A * Bc[..., None, :]
        Ag = Ab * Gm
        KKt = Kc @ Kc.transpose(-1, -2)
        Pg = scale * Gm * (Qc @ Kc.transpose(-1, -2))
        gam = Gc.exp()
        rho = (Gc[..., -1:] - Gc).exp()
        if tail < CHUNK:
            rho[:, -1, tail:] = 0.0
        gL = gam[..., -1]
        # forward sweep: state before every chunk
        S = (torch.zeros(H, K, V, dtype=dtype) if initial_state is None
             else initial_state[si].to(dtype).clone())
        S0s = []
        for c in range(n):
            S0s.append(S)
            U = Kc[:, c] @ S
            Vd = Ag[:, c] @ (Vc[:, c] - gam[:, c, :, None] * U)
            S = gL[:, c, None, None] * S + Kc[:, c].transpose(-1, -2) @ (rho[:, c, :, None] * Vd)
        dQ = torch.empty(H, n, CHUNK, K, dtype=dtype)
        dK = torch.empty(H, n, CHUNK, K, dtype=dtype)
        dV = torch.empty(H, n, CHUNK, V, dtype=dtype)
        dG = torch.empty(H, n, CHUNK, dtype=dtype)
        dB = torch.empty(H, n, CHUNK, dtype=dtype)
        for c in reversed(range(n)):
            S0 = S0s[c]
            Kn, Qn, Vn, dOn = Kc[:, c], Qc[:, c], Vc[:, c], dOc[:, c]
            ga, rh, gl = gam[:, c, :, None], rho[:, c, :, None], gL[:, c, None, None]
            U = Kn @ S0
            W = Vn - ga * U
            Vp = Ag[:, c] @ W
            dVp = rh * (Kn @ dS) + Pg[:, c].transpose(-1, -2) @ dOn
            dW = Ag[:, c].transpose(-1, -2) @ dVp
            dVg = -ga * dW
            dg_ = (dVg * U).sum(-1)
            dK1 = rh * (Vp @ dS.transpose(-1, -2))
            kk = (Kn * dK1).sum(-1)
            dg_ = dg_ - kk
            dgl = kk.sum(-1)
            dKn = dK1 + dVg @ S0.transpose(-1, -2)
            dS0 = gl * dS
            dgl = dgl + (dS0 * S0).sum((-1, -2))
            dS0 = dS0 + Kn.transpose(-1, -2) @ dVg + Qn.transpose(-1, -2) @ (scale * ga * dOn)
            dPg = dOn @ Vp.transpose(-1, -2)
            T1 = dPg * Pg[:, c]
            dg_ = dg_ + T1.sum(-1) - T1.sum(-2)
            dP = scale * Gm[:, c] * dPg
            dQn = scale * ga * (dOn @ S0.transpose(-1, -2))
            dg_ = dg_ + (Qn * dQn).sum(-1)
            dQn = dQn + dP @ Kn
            dKn = dKn + dP.transpose(-1, -2) @ Qn
            dAg = dVp @ W.transpose(-1, -2)
            dAb = Gm[:, c] * dAg
            T2 = dAb * Ab[:, c]
            dg_ = dg_ + T2.sum(-1) - T2.sum(-2)
            db_ = (dAb * A[:, c]).sum(-2)
            dA = dAb * Bc[:, c, None, :]
            At = A[:, c].transpose(-1, -2)
            dLm = torch.where(keepl, -(At @ dA @ At), dA.new_zeros(()))
            db_ = db_ + (dLm * KKt[:, c]).sum(-1)
            dAt = Bc[:, c, :, None] * dLm
            dKn = dKn + (dAt + dAt.transpose(-1, -2)) @ Kn
            dg_[:, -1] = dg_[:, -1] + dgl
            if c == n - 1 and tail < CHUNK:  # padded g aliases the last valid token
                dg_[:, tail - 1] = dg_[:, tail - 1] + dg_[:, tail:].sum(-1)
            dQ[:, c], dK[:, c], dV[:, c], dG[:, c], dB[:, c] = dQn, dKn, dW, dg_, db_
            dS = dS0
        dh0[si] = dS
        dq[b, s:e] = dQ.permute(1, 2, 0, 3).reshape(n * CHUNK, H, K)[:L]
        dk[b, s:e] = dK.permute(1, 2, 0, 3).reshape(n * CHUNK, H, K)[:L]
        dv[b, s:e] = dV.permute(1, 2, 0, 3).reshape(n * CHUNK, H, V)[:L]
        dgc[b, s:e] = dG.permute(1, 2, 0).reshape(n * CHUNK, H)[:L]
        db[b, s:e] = dB.permute(1, 2, 0).reshape(n * CHUNK, H)[:L]
    if Hg < H:
        dq = dq.reshape(B, T, Hg, H // Hg, K).sum(3)
        dk = dk.reshape(B, T, Hg, H // Hg, K).sum(3)
    dg = chunk_local_cumsum(dgc, cu_seqlens, reverse=True, dtype=dtype)
    return dq, dk, dv, db, dg, dh0


# --------------------------------------------------------------------------- naive recurrence
def gdr_recurrent(q, k, v, g, beta, scale=None, initial_state=None, cu_seqlens=None,
                  dtype=torch.float64):
    """Token-by-token recurrence, independent of chunking (tiny shapes only).

    S_t = e^{g_t} S_{t-1} + k_t (x) beta_t (v_t - k_t^T e^{g_t} S_{t-1});  o_t = scale q_t^T S_t.
    Differentiable with torch.autograd (used to check the hand-derived backward).
    """
    B, T, Hg, K = k.shape
    H, V = v.shape[2], v.shape[3]
    rep = H // Hg
    scale = K ** -0.5 if scale is None else scale
    seqs = _seq_bounds(B, T, cu_seqlens)
    o = [[None] * T for _ in range(B)]
    finals = []
    for si, (b, s, e) in enumerate(seqs):
        S = (torch.zeros(H, K, V, dtype=dtype) if initial_state is None
             else initial_state[si].to(dtype))
        for t in range(s, e):
            kt = k[b, t].to(dtype).repeat_interleave(rep, 0)
            qt = q[b, t].to(dtype).repeat_interleave(rep, 0)
            S = S * g[b, t].to(dtype).exp()[:, None, None]
            pred = torch.einsum("hk,hkv->hv", kt, S)
            S = S + torch.einsum("hk,hv->hkv", kt, (v[b, t].to(dtype) - pred) * beta[b, t].to(dtype)[:, None])
            o[b][t] = torch.einsum("hk,hkv->hv", qt * scale, S)
        finals.append(S)
    o = torch.stack([torch.stack(row, 0) for row in o], 0)
    return o, torch.stack(finals, 0)


# --------------------------------------------------------------------------- metrics
def rel_to_max(x: torch.Tensor, ref: torch.Tensor) -> float:
    """max|x-ref| / max|ref| — the acceptance metric of tests/test_gdr.py:203-235."""
    den = ref.double().abs().max().item()
    num = (x.double() - ref.double()).abs().max().item()
    return num / den if den > 0 else num
