"""Generate the golden fixtures in this folder from the UNMODIFIED reference oracle.

Run where the FlashQLA sources are mounted:

    python tests/golden/make_golden.py [--ref /path/to/FlashQLA]

The reference's ``tests/ref_gdr.py`` imports five helpers from ``flash_qla.utils``,
and importing that package needs an sm_90 GPU plus TileLang.  The helpers it needs
are pure torch, so this script loads ``flash_qla/utils/pack.py`` by file path, adds a
torch ``prepare_chunk_offsets`` (the reference's is a GPU kernel,
``flash_qla/utils/index.py:126-138``; ``ref_gdr.py`` needs the bare offsets tensor),
registers both under a temporary fake ``flash_qla`` module and then executes
``tests/ref_gdr.py`` itself, by path, without touching it.

Every fixture stores the inputs and the reference's outputs, so the tests never
need the reference at run time.  bf16-exact tensors are stored as their bf16 bit
patterns (uint16) to keep the files small.
"""

from __future__ import annotations

import argparse
import importlib.util
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def load_reference(ref_root: str):
    spec = importlib.util.spec_from_file_location("_ref_pack", os.path.join(ref_root, "flash_qla/utils/pack.py"))
    pack_mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(pack_mod)
    fq, fu = types.ModuleType("flash_qla"), types.ModuleType("flash_qla.utils")
    for n in ("pad_and_reshape", "pack", "unpack", "fill_last_chunk_of_g"):
        setattr(fu, n, getattr(pack_mod, n))

    def prepare_chunk_offsets(cu, cs):
        nc = (cu[1:] - cu[:-1] + cs - 1) // cs
        return torch.nn.functional.pad(torch.cumsum(nc, 0), (1, 0)).to(cu.dtype)

    fu.prepare_chunk_offsets = prepare_chunk_offsets
    fq.utils = fu
    saved = {n: sys.modules.get(n) for n in ("flash_qla", "flash_qla.utils")}
    sys.modules["flash_qla"], sys.modules["flash_qla.utils"] = fq, fu
    try:
        spec = importlib.util.spec_from_file_location("_ref_gdr", os.path.join(ref_root, "tests/ref_gdr.py"))
        ref = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(ref)
    finally:
        for n, m in saved.items():
            if m is None:
                sys.modules.pop(n, None)
            else:
                sys.modules[n] = m
    return ref


def l2(x):
    return x * torch.rsqrt((x * x).sum(-1, keepdim=True) + 1e-6)


def bf16_bits(x: torch.Tensor) -> np.ndarray:
    return x.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)


def make_inputs(seed, B, T, Hq, Hv, dist, round_bf16, n_seq=None, K=128):
    """dist 'baseline': g = logsigmoid(randn), h0 = 0.1 randn, dht = 0.01 randn (BASELINE configs).
    dist 'reftest' : g = logsigmoid(randn)/16 with the last head's gate = 0, h0 = randn,
                     dht = randn/8 (tests/test_gdr.py:49-111 of the reference)."""
    torch.manual_seed(seed)
    N = B if n_seq is None else n_seq
    q, k, v = l2(torch.randn(B, T, Hq, K)), l2(torch.randn(B, T, Hq, K)), torch.randn(B, T, Hv, K)
    g = torch.nn.functional.logsigmoid(torch.randn(B, T, Hv))
    beta = torch.randn(B, T, Hv).sigmoid()
    do = torch.randn(B, T, Hv, K)
    if dist == "baseline":
        h0, dht = 0.1 * torch.randn(N, Hv, K, K), 0.01 * torch.randn(N, Hv, K, K)
    else:
        g = g / 16
        g[:, :, -1] = 0.0
        h0, dht = torch.randn(N, Hv, K, K), torch.randn(N, Hv, K, K) / 8
    if round_bf16:
        q, k, v, do = (x.bfloat16().float() for x in (q, k, v, do))
    return q, k, v, g, beta, h0, do, dht


def run_case(ref, name, seed, B, T, Hq, Hv, dist, round_bf16, cu=None, bwd=True, keep_h=False):
    K = 128
    scale = K ** -0.5
    cu_t = None if cu is None else torch.tensor(cu, dtype=torch.int32)
    q, k, v, g, beta, h0, do, dht = make_inputs(seed, B, T, Hq, Hv, dist, round_bf16,
                                                n_seq=None if cu is None else len(cu) - 1)
    gc, o, A_gated, h, fs = ref.chunk_gated_delta_rule_fwd(
        q, k, v, g, beta, cu_seqlens=cu_t, initial_state=h0, scale=scale)
    out = dict(scale=np.float32(scale), g=g.numpy(), beta=beta.numpy(), h0=h0.numpy(),
               g_cumsum=gc.numpy(), o=o.numpy(), final_state=fs.numpy(), A_gated=A_gated.numpy())
    if cu is not None:
        out["cu_seqlens"] = np.asarray(cu, dtype=np.int32)
    if round_bf16:
        out.update(q_bf16=bf16_bits(q), k_bf16=bf16_bits(k), v_bf16=bf16_bits(v))
    else:
        out.update(q=q.numpy(), k=k.numpy(), v=v.numpy())
    if keep_h:
        out["h"] = h.numpy()
    if bwd:
        dq, dk, dv, db, dg, dh0 = ref.chunk_gated_delta_rule_bwd(
            q, k, v, gc, beta, A_gated, scale, h0, do, dht, cu_t)
        out.update(dht=dht.numpy(), dq=dq.numpy(), dk=dk.numpy(), dv=dv.numpy(), db=db.numpy(),
                   dg=dg.numpy(), dh0=dh0.numpy())
        if round_bf16:
            out["do_bf16"] = bf16_bits(do)
        else:
            out["do"] = do.numpy()
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **out)
    print(f"{name}: wrote {os.path.getsize(path) / 1e6:.2f} MB  |o|max={o.abs().max():.4f}")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default="/root/reference")
    args = ap.parse_args()
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    ref = load_reference(args.ref)
    # BASELINE config 1: fp32, seed 0, B=1 T=512 Hq=Hv=4, compare o and final_state.
    run_case(ref, "c1_fwd_fp32", 0, 1, 512, 4, 4, "baseline", False, bwd=False)
    # dense batch with a tail chunk (T % 64 != 0), bf16-exact inputs, fwd + bwd, keeps h.
    run_case(ref, "dense_tail_bf16", 1, 2, 136, 2, 2, "baseline", True, keep_h=True)
    # packed varlen + GVA (Hq=1, Hv=2) on the reference's own test distribution (weak gates, one g=0 head).
    run_case(ref, "varlen_gva_reftest_bf16", 42, 1, 261, 1, 2, "reftest", True, cu=[0, 70, 198, 261])


if __name__ == "__main__":
    main()
