"""Forward + backward parity on the reference's own test presets (tests/settings/varlen.csv and product.csv of
FlashQLA, reproduced in tests/golden/reference_presets.csv by tests/golden/make_presets.py) with the reference's input
distribution (tests/test_gdr.py:49-111 of FlashQLA): seed 42, q/k l2-normalised randn, g = logsigmoid(randn)/16 with
a quarter of the heads at g = 0 (picked by a random permutation), beta = sigmoid(randn), h0 = randn, dht = randn/8,
do = randn; rows with varlen and no cu_seqlens draw one length per batch row in [1, num_tokens) and pack the rows.

Tolerance (stated): max|x - ref| <= 1e-2 * max|ref| for o, dq, dk, dv, dbeta, dg, dh0 and 5e-3 for final_state,
against the fp32 oracle on the same bf16 inputs (the reference accepts 2e-2, tests/test_gdr.py:203-235,362-420).
"""
import csv
import math
import os

import pytest
import torch

from conftest import GOLDEN, check_close
from oracle import gdr_oracle as orc

pytestmark = pytest.mark.gpu
os.environ.setdefault("FLASHQLA_CHECK_STATUS", "1")

HK = HV = 4


def _rows():
    with open(os.path.join(GOLDEN, "reference_presets.csv")) as f:
        return [r for r in csv.DictReader(f)]


def _preset_inputs(row):
    B, T = int(row["batch_size"]), int(row["num_tokens"])
    varlen = row["varlen"] == "True"
    torch.manual_seed(42)
    q = orc.l2norm(torch.randn(B, T, HK, 128)).bfloat16()
    k = orc.l2norm(torch.randn(B, T, HK, 128)).bfloat16()
    v = torch.randn(B, T, HV, 128).bfloat16()
    g = torch.nn.functional.logsigmoid(torch.randn(B, T, HV)) / 16
    beta = torch.randn(B, T, HV).sigmoid()
    h0 = torch.randn(B, HV, 128, 128)
    do = torch.randn(B, T, HV, 128).bfloat16()
    dht = torch.randn(B, HV, 128, 128) / 8
    mask = torch.zeros(HV, dtype=torch.bool)
    mask[: math.ceil(0.75 * HV)] = True
    mask = mask[torch.randperm(HV)]
    g[:, :, ~mask] = 0.0
    cu = None
    if varlen:
        if row["cu_seqlens"]:
            cu = torch.tensor([int(x) for x in row["cu_seqlens"].split("-")], dtype=torch.int32)
            n = cu.numel() - 1
            # one initial state / final-state gradient per packed sequence
            h0 = torch.randn(n, HV, 128, 128)
            dht = torch.randn(n, HV, 128, 128) / 8
        else:
            lens = torch.randint(1, T, (B,), dtype=torch.int32)
            cu = torch.nn.functional.pad(torch.cumsum(lens, 0), (1, 0)).to(torch.int32)
            pack = lambda x: torch.cat([x[b, : int(lens[b])] for b in range(B)], 0).unsqueeze(0).contiguous()
            q, k, v, g, beta, do = (pack(x) for x in (q, k, v, g, beta, do))
    return q, k, v, g, beta, h0, do, dht, cu


@pytest.mark.parametrize("idx", range(14))
def test_reference_preset(idx):
    from flashqla_b200 import ops
    rows = _rows()
    assert len(rows) == 14
    row = rows[idx]
    q, k, v, g, beta, h0, do, dht, cu = _preset_inputs(row)
    dev = "cuda"
    c = lambda x: None if x is None else x.to(dev)
    gc, A, o, _, fs = ops.chunk_gated_delta_rule_fwd(c(q), c(k), c(v), c(g), c(beta), None, c(h0), c(cu), True, False, True)
    got = ops.chunk_gated_delta_rule_bwd(c(q), c(k), c(v), gc, c(beta), A, c(do), c(dht), None, c(h0), c(cu))
    torch.cuda.synchronize()
    gcr, _, o_ref, _, fs_ref = orc.gdr_fwd(q.float(), k.float(), v.float(), g, beta, None, h0, cu)
    ref = orc.gdr_bwd(q.float(), k.float(), v.float(), gcr, beta, do.float(), dht, None, h0, cu)
    what = f"preset {row['source']} B={row['batch_size']} T={row['num_tokens']} varlen={row['varlen']}: "
    check_close([o, fs], [o_ref, fs_ref], {"o": 1e-2, "final_state": 5e-3}, ["o", "final_state"], what)
    check_close(got, ref, 1e-2, ["dq", "dk", "dv", "db", "dg", "dh0"], what)
