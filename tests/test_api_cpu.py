"""CPU-side checks: the C-ABI library loads and exports every declared symbol, the host planner,
argument validation of the public operator, and the autograd arity."""
import ast
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "flashqla.h")).read()
    return sorted(set(re.findall(r"FQ_API\s+[\w\s\*]+?\b(fq_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from flashqla_b200 import _lib
    if not os.path.exists(_lib.LIB_PATH):
        from flashqla_b200 import build
        build.build()
    lib = ctypes.CDLL(_lib.LIB_PATH)
    names = _declared_symbols()
    assert len(names) >= 8
    for n in names:
        assert hasattr(lib, n), n
    assert set(names) == set(_lib.SIGNATURES), "ctypes table and header disagree"
    assert _lib.load().fq_version() >= 100


def test_argument_errors_are_reported_without_a_gpu():
    from flashqla_b200 import _lib
    lib = _lib.load()
    rc = lib.fq_chunk_cumsum(None, None, 1, 64, 1, None, None, 1, 1, 0, None)
    assert rc == -1 and b"null tensor" in lib.fq_last_error()


def test_planner_chunk_tables():
    from flashqla_b200 import planner
    cu = torch.tensor([0, 1, 64, 65, 300, 300, 777, 1000], dtype=torch.int32)
    plan = planner.plan_packed(cu, "cpu")
    assert plan.offsets_host == [0, 1, 2, 3, 7, 7, 15, 19] and plan.total_chunks == 19 and plan.n_seq == 7
    assert planner.plan_packed(cu, "cpu") is plan  # cached by tensor identity
    idx = planner.prepare_chunk_indices(cu)
    assert idx.shape == (19, 2) and idx[3].tolist() == [3, 0] and idx[6].tolist() == [3, 3] and idx[7].tolist() == [5, 0]
    off, total = planner.prepare_chunk_offsets(cu)
    assert off.tolist() == plan.offsets_host and total == 19
    with pytest.raises(ValueError):
        planner.plan_packed(torch.tensor([0, 5, 3], dtype=torch.int32), "cpu")
    d = planner.plan_dense(3, 200)
    assert (d.n_seq, d.total_chunks, d.max_chunks) == (3, 12, 4)


def test_planner_takes_a_host_copy_of_cu_seqlens():
    """A plan made from the host copy equals the plan made by reading the tensor itself."""
    from flashqla_b200 import planner
    cu = torch.tensor([0, 3, 64, 64, 200, 1000], dtype=torch.int32)
    a = planner.plan_packed(cu.clone(), "cpu")
    b = planner.plan_packed(cu.clone(), "cpu", host=cu.clone())
    assert (a.n_seq, a.total_chunks, a.total_tokens, a.max_chunks) == (b.n_seq, b.total_chunks, b.total_tokens, b.max_chunks)
    assert a.offsets_host == b.offsets_host and torch.equal(a.chunk_offsets, b.chunk_offsets)
    with pytest.raises(ValueError):
        planner.plan_packed(cu.clone(), "cpu", host=torch.tensor([0, 3], dtype=torch.int32))


def test_plan_checks_the_sequence_end_against_the_tensors():
    """cu_seqlens[-1] beyond the packed tensors is refused (the kernels' tail stores are plain pointer writes);
    shorter is allowed, and the tile tensors of such a batch start from zeros."""
    from flashqla_b200 import kernels
    cu = torch.tensor([0, 100, 300], dtype=torch.int32)
    with pytest.raises(ValueError, match="exceeds"):
        kernels.make_plan(1, 256, cu, "cpu")
    assert kernels._tile_alloc(kernels.make_plan(1, 300, cu, "cpu"), 1, 300) is torch.empty
    assert kernels._tile_alloc(kernels.make_plan(1, 320, cu, "cpu"), 1, 320) is torch.zeros
    with pytest.raises(ValueError, match="batch size"):
        kernels.make_plan(2, 300, cu, "cpu")


def test_public_operator_validation():
    import flash_qla
    q = torch.zeros(2, 64, 2, 128, dtype=torch.bfloat16)
    g = torch.zeros(2, 64, 2)
    with pytest.raises(AssertionError):
        flash_qla.chunk_gated_delta_rule(q.float(), q.float(), q.float(), g, g)
    with pytest.raises(AssertionError):
        flash_qla.chunk_gated_delta_rule(q, q, q, g, g, head_first=True)
    with pytest.raises(AssertionError):
        flash_qla.chunk_gated_delta_rule(q, q, q[:, :, :1].repeat(1, 1, 3, 1), g, g)
    with pytest.raises(ValueError):
        flash_qla.chunk_gated_delta_rule(q, q, q, g, g, cu_seqlens=torch.tensor([0, 64], dtype=torch.int32))
    with pytest.raises(ValueError):
        flash_qla.chunk_gated_delta_rule(q[:1], q[:1], q[:1], g[:1], g[:1], initial_state=torch.zeros(3, 2, 128, 128),
                                         cu_seqlens=torch.tensor([0, 32, 64], dtype=torch.int32))
    # no CPU path: CPU tensors are refused by the kernels
    from flashqla_b200._lib import FlashQLAError
    with pytest.raises(FlashQLAError):
        flash_qla.chunk_gated_delta_rule(q, q, q, g, g)


def test_autograd_backward_arity():
    """backward returns one gradient per forward input (tests/test_function_signature.py of the reference)."""
    src = open(os.path.join(ROOT, "flashqla_b200", "ops.py")).read()
    cls = next(n for n in ast.parse(src).body if isinstance(n, ast.ClassDef) and n.name == "ChunkGatedDeltaRuleFunction")
    fwd = next(n for n in cls.body if isinstance(n, ast.FunctionDef) and n.name == "forward")
    bwd = next(n for n in cls.body if isinstance(n, ast.FunctionDef) and n.name == "backward")
    ret = [n for n in ast.walk(bwd) if isinstance(n, ast.Return)][-1]
    assert len(ret.value.elts) == len(fwd.args.args) - 1


def test_context_parallel_planner():
    from flashqla_b200 import planner
    # pieces tile every sequence, keep 64-token chunk boundaries and mark first / last pieces
    cu = torch.tensor([0, 100, 100, 5000, 9000], dtype=torch.int32)
    plan = planner.plan_packed(cu, "cpu")
    cp = planner.plan_cp(plan, 1, 9000, 4, 148, "cpu", piece_chunks=16)
    b = cp.cu_seqlens.tolist()
    assert b[0] == 0 and b[-1] == 9000 and cp.n_pieces == len(b) - 1 == 11
    assert all((s - cu_s) % 64 == 0 for s, cu_s in zip(cp.piece_start.tolist(), [0, 100, 100, 100, 100, 100, 100, 5000, 5000, 5000, 5000]))
    assert cp.out_index_fwd.tolist() == [0, 1, -1, -1, -1, -1, 2, -1, -1, -1, 3]
    assert cp.out_index_bwd.tolist() == [0, 1, 2, -1, -1, -1, -1, 3, -1, -1, -1]
    assert cp.chunks_before.tolist() == [0, 0, 0, 16, 32, 48, 64, 0, 16, 32, 48]
    assert cp.chunk_offsets.tolist()[-1] == plan.total_chunks == cp.total_chunks
    assert cp.seq_end.tolist() == [100, 100, 5000, 5000, 5000, 5000, 5000, 9000, 9000, 9000, 9000]
    # the split is chosen from a makespan model of one CTA per SM
    assert planner.choose_piece_chunks([128] * 4, 32, 148) is None          # 128 CTAs already fill the GPU
    L = planner.choose_piece_chunks([512], 64, 148)
    assert L is not None and 8 <= L < 512
    assert planner.choose_piece_chunks([4, 4, 4], 2, 148) is None           # too short to split
    assert planner.plan_cp(planner.plan_dense(4, 8192), 4, 8192, 32, 148, "cpu") is None
    # dense batches are split over the flattened token axis
    cp2 = planner.plan_cp(planner.plan_dense(2, 1024), 2, 1024, 1, 148, "cpu", piece_chunks=4)
    assert cp2.cu_seqlens.tolist() == [0, 256, 512, 768, 1024, 1280, 1536, 1792, 2048]
    assert cp2.seq_index.tolist() == [0, 0, 0, 0, 1, 1, 1, 1]


def test_recurrent_operator_refuses_cpu_tensors():
    """The decode-step operator has no CPU path either."""
    import flashqla_b200 as fq
    from flashqla_b200 import _lib
    q = torch.zeros(1, 1, 1, 128, dtype=torch.bfloat16)
    g = torch.zeros(1, 1, 1)
    with pytest.raises(_lib.FlashQLAError):
        fq.fused_recurrent_gated_delta_rule(q, q, q, g, g)

