"""Pins top-2 gating and gating under a non-zero used capacity to vectors computed by the reference's own code
(tests/golden/make_golden.py): `top2gating` of docker/resources/sharded_moe.py:253-324 with its noise off, and
FakeMoeEncodeOp (models/benchmark/pytorch/utils.py:313-379) called on chained chunks.  The CPU tests check the
NumPy oracle, the GPU tests the CUDA kernels through the C ABI, both against the same files."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import moe_oracle as O

HERE = os.path.dirname(__file__)
TOP2 = sorted(glob.glob(os.path.join(HERE, "golden", "top2_ref_*.npz")))
CHAIN = sorted(glob.glob(os.path.join(HERE, "golden", "chain_ref_*.npz")))
TOP2CHAIN = sorted(glob.glob(os.path.join(HERE, "golden", "top2chain_ref_*.npz")))
ids = lambda p: os.path.basename(p)[:-4]


def check_top2(rec, gs, il, cap):
    """gs [2,S] float32, il [4,S] int32, cap [E] int32 of a top-2 gate against the reference's vectors."""
    S, E, C = int(rec["S"]), int(rec["E"]), int(rec["C"])
    kept1, kept2 = rec["kept1"] == 1, rec["kept2"] == 1
    # expert choice: reference indices where kept, -1 where the reference's capacity mask removed the choice
    np.testing.assert_array_equal(il[0], np.where(kept1, rec["idx1"], -1))
    np.testing.assert_array_equal(il[2], np.where(kept2, rec["idx2"], -1))
    # locations before the mask (the second choice is offset by the count of first choices, sharded_moe.py:282-285)
    np.testing.assert_array_equal(il[1], rec["loc1_all"])
    np.testing.assert_array_equal(il[3], rec["loc2_all"])
    # ... and after it, as the reference stores them (zero for a dropped choice)
    np.testing.assert_array_equal(np.where(il[0] >= 0, il[1], 0), rec["loc1_s"])
    np.testing.assert_array_equal(np.where(il[2] >= 0, il[3], 0), rec["loc2_s"])
    # normalised gates: g_j / clamp(g_1 + g_2, eps) in float32 (:306-312): one division, bit-exact
    np.testing.assert_array_equal(gs[0], rec["gates1_s"])
    np.testing.assert_array_equal(gs[1], rec["gates2_s"])
    # rows used per expert = kept first + kept second choices
    used = np.bincount(rec["idx1"][kept1], minlength=E) + np.bincount(rec["idx2"][kept2], minlength=E)
    np.testing.assert_array_equal(cap, np.minimum(used, C))
    np.testing.assert_array_equal(np.bincount(rec["idx1"], minlength=E), rec["exp_counts"])


@pytest.mark.parametrize("path", TOP2, ids=ids)
def test_oracle_top2_matches_reference_gate(path):
    rec = np.load(path)
    S, E, M, C = (int(rec[k]) for k in ("S", "E", "M", "C"))
    assert O.capacity(S, E, float(rec["cf"]), 2) == C, "shape chosen so that both capacity roundings agree"
    gs, il, cap, elems = O.moe_gate(rec["gate"], np.zeros(E, np.int32), C, M, 2)
    check_top2(rec, gs, il, cap)
    if "x" in rec.files:
        disp = O.moe_encode_fwd(il, rec["x"], E, C)
        np.testing.assert_array_equal(disp, rec["disp"])          # 0/1 mask times x summed with zeros: exact
        out = O.moe_decode_fwd(rec["eo"], gs, il)
        np.testing.assert_allclose(out, rec["out"], rtol=1e-5, atol=1e-6)
    # gradient of the normalised gates w.r.t. the gate probabilities: autograd through the reference's own code
    dg = O.moe_encode_dg_top2(rec["d_gates_s"], il, rec["gate"], E)
    np.testing.assert_allclose(dg, rec["d_gate"], rtol=1e-5, atol=1e-6 * float(np.abs(rec["d_gate"]).max()))


@pytest.mark.parametrize("path", CHAIN, ids=ids)
def test_oracle_chained_used_capacity_matches_reference_operator(path):
    rec = np.load(path)
    S, E, M, n, C = (int(rec[k]) for k in ("S", "E", "M", "n", "C"))
    Sp = S // n
    assert O.capacity(Sp, E, 1.0) == C
    used = rec["used_in"][0].copy()
    for c in range(n):
        np.testing.assert_array_equal(used, rec["used_in"][c])
        gs, il, cap, elems = O.moe_gate(rec["gate"][c * Sp:(c + 1) * Sp], used, C, M)
        np.testing.assert_array_equal(il, rec["idx_loc"][c])
        np.testing.assert_array_equal(gs[0], rec["gates_s"][c])
        used = cap


def expected_top2_chain(rec, cf):
    """What n chained top-2 encodes must give, assembled from the reference gate's per-chunk vectors (choices, locations
    before the capacity mask, probabilities: docker/resources/sharded_moe.py:253-324) and the CUDA operator's chaining
    rules: a choice is dropped when loc >= C - used[e] (tutel_moe_dispatch.cu:199-201), used[e] grows by the tokens routed
    to e and saturates at C (:207-209), gates are g_j / clamp(sum of kept g, eps) (sharded_moe.py:306-312)."""
    S, E, n = int(rec["S"]), int(rec["E"]), int(rec["n"])
    Sp = S // n
    C = O.capacity(Sp, E, cf * n, 2)
    used = np.zeros(E, np.int64)
    il = np.zeros((n, 4, Sp), np.int32)
    gs = np.zeros((n, 2, Sp), np.float32)
    chain = [used.copy()]
    rows = np.arange(Sp)
    for c in range(n):
        gate = rec["gate"][c * Sp:(c + 1) * Sp]
        raw, keep = [], []
        for j, (idx, loc) in enumerate(((rec["idx1"][c], rec["loc1_all"][c]), (rec["idx2"][c], rec["loc2_all"][c]))):
            k = loc < C - used[idx]
            il[c, 2 * j] = np.where(k, idx, -1)
            il[c, 2 * j + 1] = loc                       # per-call location; the shared-buffer row adds used[idx]
            raw.append(np.where(k, gate[rows, idx], np.float32(0)).astype(np.float32))
            keep.append(k)
        denom = np.maximum(raw[0] + raw[1], np.float32(np.finfo(np.float32).eps)).astype(np.float32)
        gs[c, 0], gs[c, 1] = raw[0] / denom, raw[1] / denom
        cnt = np.bincount(rec["idx1"][c], minlength=E) + np.bincount(rec["idx2"][c], minlength=E)
        base = used.copy()
        used = np.minimum(used + cnt, C)
        chain.append(used.copy())
        il[c, 1] += base[rec["idx1"][c]].astype(np.int32)
        il[c, 3] += base[rec["idx2"][c]].astype(np.int32)
    return C, il, gs, np.stack(chain).astype(np.int32)


@pytest.mark.parametrize("path", TOP2CHAIN, ids=ids)
def test_oracle_chained_top2_matches_reference_gate_per_chunk(path):
    rec = np.load(path)
    S, E, n = int(rec["S"]), int(rec["E"]), int(rec["n"])
    Sp = S // n
    C, il, gs, chain = expected_top2_chain(rec, 0.5)       # a tight capacity: later chunks lose choices
    assert (il[:, 0] < 0).any() and (il[:, 2] < 0).any() and (il[0, 0] >= 0).all()
    used = np.zeros(E, np.int32)
    for c in range(n):
        g, l, cap, _ = O.moe_gate(rec["gate"][c * Sp:(c + 1) * Sp], used, C, 8, 2)
        np.testing.assert_array_equal(l[0::2], il[c, 0::2])
        np.testing.assert_array_equal(l[1::2] + np.where(True, used[np.stack([rec["idx1"][c], rec["idx2"][c]])], 0), il[c, 1::2])
        np.testing.assert_array_equal(g, gs[c])
        used = cap
        np.testing.assert_array_equal(used, chain[c + 1])


# ---- the same vectors against the CUDA kernels -----------------------------------------------------------------
DEV = "cuda:0"


def cu(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


@pytest.mark.gpu
@pytest.mark.parametrize("path", TOP2, ids=ids)
def test_gpu_top2_matches_reference_gate(path):
    import lancet_b200 as LB
    rec = np.load(path)
    S, E, M, C = (int(rec[k]) for k in ("S", "E", "M", "C"))
    cap0 = torch.zeros(E, dtype=torch.int32, device=DEV)
    gs, il, cap, elems = LB.moe_gate(cu(rec["gate"]), cap0, C, M, k=2)
    check_top2(rec, gs.cpu().numpy().reshape(2, S), il.cpu().numpy(), cap.cpu().numpy())
    dg = LB.moe_encode_dg(cu(rec["d_gates_s"]), il, E, gate=cu(rec["gate"]))
    np.testing.assert_allclose(dg.cpu().numpy(), rec["d_gate"], rtol=1e-5, atol=1e-6 * float(np.abs(rec["d_gate"]).max()))
    if "x" in rec.files:
        g1, il1, cap1, el1, disp = LB.moe_encode(cu(rec["x"]), cu(rec["gate"]), cap0, float(rec["cf"]), k=2)
        assert tuple(disp.shape) == (E, C, M)
        np.testing.assert_array_equal(disp.cpu().numpy(), rec["disp"])
        out = LB.moe_decode(cu(rec["eo"]), g1, il1)
        np.testing.assert_allclose(out.cpu().numpy(), rec["out"], rtol=1e-5, atol=1e-6)


@pytest.mark.gpu
@pytest.mark.parametrize("path", CHAIN, ids=ids)
def test_gpu_chained_used_capacity_matches_reference_operator(path):
    import lancet_b200 as LB
    rec = np.load(path)
    S, E, M, n, C = (int(rec[k]) for k in ("S", "E", "M", "n", "C"))
    Sp = S // n
    used = cu(rec["used_in"][0])
    for c in range(n):
        gs, il, cap, elems = LB.moe_gate(cu(rec["gate"][c * Sp:(c + 1) * Sp]), used, C, M)
        np.testing.assert_array_equal(il.cpu().numpy(), rec["idx_loc"][c])
        np.testing.assert_array_equal(gs.cpu().numpy().reshape(-1), rec["gates_s"][c])
        used = cap
    # the single-call chained gate (all chunks in one launch, capacity factor cf*n with cf = 1/n) gives the same table
    if bool((rec["used_in"][0] == 0).all()):
        plan = LB.ChunkedMoE(S, M, E, 1, 1.0 / n, n, torch.float32, device=DEV)
        assert plan.C == C
        plan.dispatch(torch.zeros((S, M), device=DEV), cu(rec["gate"]))
        il = plan.idx_loc.cpu().numpy()
        np.testing.assert_array_equal(il[:, 0], rec["idx_loc"][:, 0])
        # the plan's locations are rows of the one shared buffer: the used capacity of the expert before the chunk
        # plus the reference's per-call location
        first = np.argmax(rec["gate"], axis=1).reshape(n, Sp)
        base = np.take_along_axis(rec["used_in"], first, axis=1)
        np.testing.assert_array_equal(il[:, 1] - base, rec["idx_loc"][:, 1])
        np.testing.assert_array_equal(plan.gates_s.cpu().numpy().reshape(n, -1), rec["gates_s"])


@pytest.mark.gpu
@pytest.mark.parametrize("path", TOP2CHAIN, ids=ids)
@pytest.mark.parametrize("cf", [0.5, 1.25])
def test_gpu_chained_top2_matches_reference_gate_per_chunk(path, cf):
    """The configuration the headline benchmark runs (top-2, chained chunks, one launch for all chunks) against vectors
    assembled from the reference gate's own per-chunk outputs."""
    import lancet_b200 as LB
    rec = np.load(path)
    S, E, n = int(rec["S"]), int(rec["E"]), int(rec["n"])
    C, il, gs, chain = expected_top2_chain(rec, cf)
    plan = LB.ChunkedMoE(S, 8, E, 2, cf, n, torch.float16, device=DEV)
    assert plan.C == C
    plan.dispatch(torch.zeros((S, 8), dtype=torch.float16, device=DEV), cu(rec["gate"]))
    np.testing.assert_array_equal(plan.idx_loc.cpu().numpy(), il)
    np.testing.assert_array_equal(plan.gates_s.cpu().numpy(), gs)
    np.testing.assert_array_equal(plan.capused.cpu().numpy(), chain)
