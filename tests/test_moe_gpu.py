"""Parity of the CUDA MoE path (through the C ABI) with the CPU oracle and the golden vectors
made by the reference's own operators.  Integer outputs and fp32 data moves must be bit-exact."""
import glob
import os

import numpy as np
import pytest
import torch

import lancet_b200 as LB
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "moe_ref_*.npz")))
TDT = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


def cu(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
    return t.to(dtype) if dtype is not None else t


def host(t):
    if t.dtype == torch.bfloat16:
        return t.float().cpu().numpy()
    if t.dtype == torch.uint64:
        return t.cpu().view(torch.int64).numpy().astype(np.uint64)
    return t.cpu().numpy()


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[8:-4] for p in GOLDEN])
def test_golden_reference_vectors(path):
    rec = np.load(path)
    S, E, M, C = (int(rec[k]) for k in ("S", "E", "M", "C"))
    gate = cu(rec["gate"])
    cap0 = torch.zeros(E, dtype=torch.int32, device=DEV)
    gs, il, cap, elems = LB.moe_gate(gate, cap0, C, M)
    np.testing.assert_array_equal(host(il), rec["idx_loc"])
    np.testing.assert_array_equal(host(cap), rec["capused"])
    np.testing.assert_array_equal(host(elems).astype(np.int64), rec["elems"])
    np.testing.assert_array_equal(host(gs)[0], rec["gates_s"])
    if "x" not in rec.files:
        return
    x = cu(rec["x"])
    g1, il1, cap1, el1, disp = LB.moe_encode(x, gate, cap0, 1.0)
    np.testing.assert_array_equal(host(il1), rec["idx_loc"])
    np.testing.assert_array_equal(host(disp), rec["disp"])
    out = LB.moe_decode(cu(rec["eo"]), g1, il1)
    np.testing.assert_array_equal(host(out), rec["out"])
    np.testing.assert_array_equal(host(LB.moe_encode_dx(cu(rec["d_disp"]), il1)), rec["enc_dx"])
    dg = host(LB.moe_encode_dg(cu(rec["d_gates"]), il1, E))
    ref_dg = np.zeros((S, E), np.float32)
    ref_dg[tuple(rec["enc_dg_nnz"])] = rec["enc_dg_val"]
    np.testing.assert_array_equal(dg, ref_dg)
    np.testing.assert_array_equal(host(LB.moe_decode_dx(cu(rec["d_out"]), g1, il1, E, C)), rec["dec_dx"])
    rows_used = cap1
    np.testing.assert_array_equal(host(LB.moe_decode_dx(cu(rec["d_out"]), g1, il1, E, C, rows_used=rows_used)),
                                  rec["dec_dx"])
    np.testing.assert_allclose(host(LB.moe_decode_dg(cu(rec["d_out"]), cu(rec["eo"]), il1)), rec["dec_dg"],
                               rtol=1e-5, atol=1e-5)


def test_config1_from_seed():
    """S=2048, E=8, M=512 fp32, softmax gate, seed 0 (the reference's CPU-runnable configuration)."""
    g = torch.Generator().manual_seed(0)
    gate = torch.softmax(torch.randn(2048, 8, generator=g), dim=1)
    x = torch.randn(2048, 512, generator=g)
    want = O.moe_encode(x.numpy(), gate.numpy(), np.zeros(8, np.int32), 1.0)
    got = LB.moe_encode(x.to(DEV), gate.to(DEV), torch.zeros(8, dtype=torch.int32, device=DEV), 1.0)
    np.testing.assert_array_equal(host(got[0]), want[0][0])
    for a, b in zip(got[1:], want[1:]):
        np.testing.assert_array_equal(host(a), b)
    out = LB.moe_decode(got[4], got[0], got[1])
    np.testing.assert_array_equal(host(out), O.moe_decode_fwd(want[4], want[0], want[1]))


CASES = [
    # S, E, M, k, dtype, gate dtype, capacity factor
    (1024, 32, 128, 1, "f32", "f32", 1.0),
    (2048, 64, 128, 1, "f32", "f32", 1.0),
    (1000, 7, 36, 1, "f32", "f32", 1.0),      # ragged: S % E != 0, 16-byte rows
    (513, 3, 5, 1, "f32", "f32", 2.0),        # rows not a multiple of 16 bytes
    (300, 5, 7, 2, "f16", "f32", 1.25),       # 2-byte access path
    (300, 5, 6, 2, "bf16", "f32", 1.25),      # 4-byte access path
    (4096, 16, 256, 2, "f16", "f32", 1.25),
    (4096, 2, 64, 2, "f16", "f16", 1.25),     # E = 2: heavy contention; fp16 gate
    (4096, 16, 256, 2, "bf16", "bf16", 1.0),
    (1, 4, 8, 1, "f32", "f32", 1.0),
    (31, 2, 8, 2, "f32", "f32", 1.0),
    (70000, 8, 8, 1, "f32", "f32", 1.0),      # more than 256 tiles: tile-scan pass
    (70000, 6, 8, 2, "f16", "f32", 0.5),
]


@pytest.mark.parametrize("S,E,M,k,dt,gdt,cf", CASES)
def test_encode_decode_and_grads_match_oracle(S, E, M, k, dt, gdt, cf):
    rng = np.random.default_rng(S * 131 + E * 7 + k)
    tdt, tgdt = TDT[dt], TDT[gdt]
    gate_t = torch.softmax(torch.from_numpy(rng.standard_normal((S, E)).astype(np.float32)), dim=1).to(tgdt)
    x_t = torch.from_numpy(rng.standard_normal((S, M)).astype(np.float32)).to(tdt)
    cap0 = rng.integers(0, 4, E).astype(np.int32)
    gate_np = gate_t.float().numpy()           # exact widening of the 16-bit gate
    x_np = x_t.float().numpy() if dt == "bf16" else x_t.numpy()
    C = O.capacity(S, E, cf, k)
    w_gs, w_il, w_cap, w_el = O.moe_gate(gate_np, cap0, C, M, k)
    w_disp = O.moe_encode_fwd(w_il, x_np, E, C, cap0)
    gs, il, cap, el, disp = LB.moe_encode(x_t.to(DEV), gate_t.to(DEV), cu(cap0), cf, k=k)
    assert disp.shape == (E, C, M)
    np.testing.assert_array_equal(host(il), w_il)
    np.testing.assert_array_equal(host(cap), w_cap)
    np.testing.assert_array_equal(host(el), w_el)
    np.testing.assert_array_equal(host(gs).reshape(k, S), w_gs)      # fp32 gates: bit-exact, k=2 included
    np.testing.assert_array_equal(host(disp), w_disp)                # data move: bit-exact, padding rows zero
    # Oracle results are float32 values computed from the widened inputs; rounding them once to the
    # data dtype (round-to-nearest-even, as the kernels do) must reproduce the device bit for bit.
    def rnd(a):
        return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(tdt).float().numpy()

    def f32(t):
        return host(t).astype(np.float32)

    # combine on a random expert output
    eo_t = torch.from_numpy(rng.standard_normal((E, C, M)).astype(np.float32)).to(tdt)
    eo_np = eo_t.float().numpy()
    out = LB.moe_decode(eo_t.to(DEV), gs, il)
    np.testing.assert_array_equal(f32(out), rnd(O.moe_decode_fwd(eo_np, w_gs, w_il)))
    # gradients
    dy_t = torch.from_numpy(rng.standard_normal((E, C, M)).astype(np.float32)).to(tdt)
    dx = LB.moe_encode_dx(dy_t.to(DEV), il)
    np.testing.assert_array_equal(f32(dx), rnd(O.moe_encode_dx(w_il, dy_t.float().numpy(), S)))
    do_t = torch.from_numpy(rng.standard_normal((S, M)).astype(np.float32)).to(tdt)
    do_np = do_t.float().numpy()
    ddx = LB.moe_decode_dx(do_t.to(DEV), gs, il, E, C)
    np.testing.assert_array_equal(f32(ddx), rnd(O.moe_decode_dx(w_gs, w_il, do_np, E, C)))
    rows_used = cu((w_cap - cap0).astype(np.int32))
    ddx2 = LB.moe_decode_dx(do_t.to(DEV), gs, il, E, C, rows_used=rows_used)
    np.testing.assert_array_equal(f32(ddx2), f32(ddx))
    ddg = LB.moe_decode_dg(do_t.to(DEV), eo_t.to(DEV), il)
    w_ddg = O.moe_decode_dg(w_il, do_np, eo_np)
    # fp32 accumulation of M products: rel 1e-5 of the sum of magnitudes
    np.testing.assert_allclose(host(ddg).reshape(k, S), w_ddg, rtol=1e-5, atol=1e-5 * M)
    dgs = rng.standard_normal((k, S)).astype(np.float32)
    if k == 1:
        edg = LB.moe_encode_dg(cu(dgs[0]), il, E)
        np.testing.assert_array_equal(host(edg), O.moe_encode_dg(dgs, w_il, E))
    else:
        edg = LB.moe_encode_dg(cu(dgs), il, E, gate=gate_t.to(DEV))
        w_edg = O.moe_encode_dg_top2(dgs, w_il, gate_np, E)
        np.testing.assert_allclose(host(edg).astype(np.float32), w_edg.astype(np.float32),
                                   rtol=1e-5 if gdt == "f32" else 1e-2, atol=1e-6 if gdt == "f32" else 1e-2)


def test_empty_inputs():
    E, M = 4, 8
    x = torch.zeros((0, M), device=DEV)
    gate = torch.zeros((0, E), device=DEV)
    cap0 = torch.tensor([1, 0, 2, 0], dtype=torch.int32, device=DEV)
    gs, il, cap, el, disp = LB.moe_encode(x, gate, cap0, 1.0)
    assert disp.shape == (E, 0, M) and il.shape == (2, 0)
    np.testing.assert_array_equal(host(cap), [0, 0, 0, 0])   # min(in + 0, C = 0)
    out = LB.moe_decode(torch.zeros((E, 0, M), device=DEV), gs, il)
    assert out.shape == (0, M)


def test_all_tokens_to_one_expert_and_drops():
    S, E, M = 512, 4, 16
    gate = torch.zeros((S, E)); gate[:, 2] = 1.0
    x = torch.randn(S, M)
    gs, il, cap, el, disp = LB.moe_encode(x.to(DEV), gate.to(DEV), torch.zeros(E, dtype=torch.int32, device=DEV), 1.0)
    C = S // E
    ilh = host(il)
    assert (ilh[0][:C] == 2).all() and (ilh[0][C:] == -1).all()
    np.testing.assert_array_equal(ilh[1], np.arange(S))
    np.testing.assert_array_equal(host(cap), [0, 0, C, 0])
    np.testing.assert_array_equal(host(disp)[2], x[:C].numpy())
    assert host(disp)[[0, 1, 3]].sum() == 0


def test_ties_pick_first_maximum():
    gate = torch.tensor([[0.5, 0.5, 0.0], [0.1, 0.4, 0.4], [0.3, 0.3, 0.3]], dtype=torch.float32)
    for k in (1, 2):
        C = 4
        want = O.moe_gate(gate.numpy(), np.zeros(3, np.int32), C, 1, k)
        got = LB.moe_gate(gate.to(DEV), torch.zeros(3, dtype=torch.int32, device=DEV), C, 1, k=k)
        np.testing.assert_array_equal(host(got[1]), want[1])
    assert host(got[1])[0].tolist() == [0, 1, 0] and host(got[1])[2].tolist() == [1, 2, 1]


@pytest.mark.parametrize("n,k", [(2, 1), (4, 1), (4, 2)])
def test_chained_partitions_share_one_buffer(n, k):
    """n chained moe_encode calls with capacity factor cf*n (reference PartitionMoEEncode,
    src/pass/dist_optimization/partition_exprs.cc:1709-1795): per-call outputs match the oracle, and
    the shared-buffer mode (row = used_capacity + location) reproduces merge+redispatch."""
    rng = np.random.default_rng(n * 10 + k)
    S, M, E, cf = 2048, 32, 4, 1.0
    x = rng.standard_normal((S, M)).astype(np.float32)
    gate = rng.random((S, E), dtype=np.float32)
    Sp = S // n
    C = O.capacity(Sp, E, cf * n, k)
    shared = torch.full((E, C, M), 7.0, device=DEV)
    cap = np.zeros(E, np.int32)
    cap_t = torch.zeros(E, dtype=torch.int32, device=DEV)
    ils, disps = [], []
    for i in range(n):
        sl = slice(i * Sp, (i + 1) * Sp)
        w = O.moe_encode(x[sl], gate[sl], cap, cf * n, k)
        got = LB.moe_encode(cu(x[sl]), cu(gate[sl]), cap_t, cf * n, k=k)
        np.testing.assert_array_equal(host(got[1]), w[1])
        np.testing.assert_array_equal(host(got[2]), w[2])
        np.testing.assert_array_equal(host(got[3]), w[3])
        np.testing.assert_array_equal(host(got[4]), w[4])
        LB.moe_encode_fwd(got[1], cu(x[sl]), E, C, used_capacity=cap_t, out=shared,
                          flags=LB._capi.ENCODE_GLOBAL_LOC | LB._capi.ENCODE_NO_ZERO)
        ils.append(w[1]); disps.append(w[4])
        cap, cap_t = w[2], got[2]
    LB.moe_zero_tail(shared, cap_t)
    if k == 1:
        np.testing.assert_array_equal(host(shared), O.moe_redispatch(disps, ils))
    want = np.zeros((E, C, M), np.float32)
    base = np.zeros(E, np.int64)
    for d, il in zip(disps, ils):
        for e in range(E):
            cnt = sum(int(((il[2 * j] == e)).sum()) for j in range(k))
            want[e, base[e]:base[e] + cnt] = d[e, :cnt]
            base[e] += cnt
    np.testing.assert_array_equal(host(shared), want)


def test_errors_are_reported_not_launched():
    x = torch.zeros((8, 4), device=DEV)
    gate = torch.zeros((8, 1), device=DEV)
    with pytest.raises(LB.LancetError) as ei:
        LB.moe_encode(x, gate, torch.zeros(1, dtype=torch.int32, device=DEV), 1.0, k=2)   # E < k
    assert ei.value.code == 1
    torch.cuda.synchronize()


@pytest.mark.parametrize("S,E,M,k,n,cf", [(4096, 2, 64, 2, 4, 1.25), (2048, 16, 128, 2, 4, 1.25), (1024, 8, 32, 1, 2, 1.0)])
def test_chunked_plan_matches_chained_oracle(S, E, M, k, n, cf):
    rng = np.random.default_rng(S + E + n)
    x = torch.from_numpy(rng.standard_normal((S, M)).astype(np.float32)).half()
    gate = torch.softmax(torch.from_numpy(rng.standard_normal((S, E)).astype(np.float32)), dim=1)
    plan = LB.ChunkedMoE(S, M, E, k, cf, n, torch.float16, device=DEV)
    for _ in range(2):   # second pass checks that buffers are reusable without re-initialisation
        plan.dispatched.fill_(3.0)
        disp = plan.dispatch(x.to(DEV), gate.to(DEV))
        Sp = S // n
        C = O.capacity(Sp, E, cf * n, k)
        assert plan.C == C
        want = np.zeros((E, C, M), np.float16)
        cap = np.zeros(E, np.int32)
        outs = []
        for i in range(n):
            sl = slice(i * Sp, (i + 1) * Sp)
            gs, il, cap2, el = O.moe_gate(gate[sl].numpy(), cap, C, M, k)
            gl = il.copy()
            # the device adds in_cap[e] of the pre-drop expert choice to every location
            raw = O.moe_gate(gate[sl].numpy(), np.zeros(E, np.int32), 1 << 30, M, k)[1]
            for j in range(k):
                gl[2 * j + 1] = il[2 * j + 1] + cap[raw[2 * j]]
            np.testing.assert_array_equal(host(plan.idx_loc[i]), gl)
            np.testing.assert_array_equal(host(plan.gates_s[i]), gs)
            np.testing.assert_array_equal(host(plan.capused[i + 1]), cap2)
            np.testing.assert_array_equal(host(plan.elems[i]), el)
            want += O.moe_encode_fwd(il, x[sl].numpy(), E, C, cap, global_loc=True)
            outs.append((gs, gl))
            cap = cap2
        np.testing.assert_array_equal(host(disp), want)
        out = plan.combine()
        ref = np.concatenate([O.moe_decode_fwd(want.astype(np.float32), gs, gl) for gs, gl in outs])
        np.testing.assert_array_equal(host(out).astype(np.float32),
                                      torch.from_numpy(ref).half().float().numpy())


@pytest.mark.parametrize("n,dt", [(2, "f32"), (4, "f32"), (3, "f16")])
def test_merge_masks_and_redispatch_equal_unpartitioned(n, dt):
    """tests/python/op/cuda/test_cuda_moe.py:387-471 of the reference: n chained moe_encode(cf*n) +
    moe_merge_masks + moe_redispatch == one moe_encode(cf) after masking."""
    rng = np.random.default_rng(n)
    S, M, E = 1536, 24, 2 if n != 3 else 4   # capacities of the partitioned and the single call must agree
    tdt = TDT[dt]
    x = torch.from_numpy(rng.standard_normal((S, M)).astype(np.float32)).to(tdt)
    gate = torch.from_numpy(rng.random((S, E), dtype=np.float32))
    ref = LB.moe_encode(x.to(DEV), gate.to(DEV), torch.zeros(E, dtype=torch.int32, device=DEV), 1.0)
    cap = torch.zeros(E, dtype=torch.int32, device=DEV)
    ils, ds = [], []
    for i in range(n):
        sl = slice(i * S // n, (i + 1) * S // n)
        out = LB.moe_encode(x[sl].to(DEV), gate[sl].to(DEV), cap, float(n))
        ils.append(out[1]); ds.append(out[4]); cap = out[2]
    mil = LB.moe_merge_masks(ils, E)
    md = LB.moe_redispatch(ds, ils)
    w_mil = O.moe_merge_masks([host(t) for t in ils], E)
    w_md = O.moe_redispatch([host(t).astype(np.float32) for t in ds], [host(t) for t in ils])
    np.testing.assert_array_equal(host(mil), w_mil)
    np.testing.assert_array_equal(host(md).astype(np.float32), w_md)
    ril = host(ref[1]).copy()
    ril[1][ril[0] < 0] = -1
    np.testing.assert_array_equal(host(mil), ril)
    for e in range(E):
        kept = int((ril[0] == e).sum())
        np.testing.assert_array_equal(host(md)[e, :kept], host(ref[4])[e, :kept])


def test_redispatch_expert_input():
    """tests/python/distributed/test_partitioned_moe.py:99-196 pattern: [C,G,M] partitions compacted by counts."""
    rng = np.random.default_rng(12)
    n, C, G, M, LE, le = 3, 40, 4, 16, 2, 1
    datas = [rng.standard_normal((C, G, M)).astype(np.float32) for _ in range(n)]
    rcs = [(rng.integers(0, 15, G * LE) * M).astype(np.uint64) for _ in range(n)]
    rcs[1][0 * LE + le] = 30 * M                                   # overflow past C is clipped
    got = LB.moe_redispatch_expert_input([cu(d) for d in datas], [cu(r.astype(np.int64)) for r in rcs], le, LE)
    want = O.moe_redispatch_expert_input(datas, rcs, le, LE, M)
    np.testing.assert_array_equal(host(got), want)


@pytest.mark.parametrize("S,E,M,n,cf,dt", [(1024, 32, 128, 1, 1.0, "f32"), (2048, 64, 128, 1, 1.0, "f32"),
                                           (2048, 32, 16, 2, 2.0, "f32"), (2048, 64, 8, 4, 4.0, "f16"),
                                           (999, 3, 8, 1, 1.0, "f32"), (1200, 8, 8, 3, 1.5, "f32"),
                                           (65536, 2, 8, 4, 0.5, "f32"),     # two large buckets, half of the tokens dropped
                                           (40000, 5, 8, 1, 0.25, "f16")])
def test_batch_prioritized_routing(S, E, M, n, cf, dt):
    """Shapes of tests/python/op/cuda/test_cuda_moe.py:160-327 of the reference (gate ~ U[0,1), seed 0),
    plus ragged ones and a case with many ties."""
    rng = np.random.default_rng(0)
    x = torch.from_numpy(rng.standard_normal((S, M)).astype(np.float32)).to(TDT[dt])
    gate = rng.random((S, E), dtype=np.float32)
    if S in (999, 40000):
        gate = np.round(gate * 4) / 4                # heavy ties: resolved towards the lower token index
    x_np = x.float().numpy() if dt != "f32" else x.numpy()
    for pid in range(n):
        want = O.moe_encode_bpr(x_np, gate, n, pid, cf)
        got = LB.moe_encode_batch_prioritized(x.to(DEV), cu(gate), n, pid, cf)
        np.testing.assert_array_equal(host(got[0]), want[0])
        np.testing.assert_array_equal(host(got[1]), want[1])
        np.testing.assert_array_equal(host(got[2]), want[2])
        np.testing.assert_array_equal(host(got[3]), want[3])
        np.testing.assert_array_equal(host(got[4]).astype(np.float32), want[4].astype(np.float32))


def test_scatter_with_an_existing_routing_table():
    """lancet_moe_scatter_chunked moves another tensor with the routing of the last chained dispatch."""
    S, M, E, k, n = 4096, 64, 8, 2, 4
    g = torch.Generator(device=DEV).manual_seed(3)
    gate = torch.softmax(torch.randn((S, E), device=DEV, generator=g), dim=1)
    x = torch.randn((S, M), device=DEV, generator=g).half()
    y = torch.randn((S, M), device=DEV, generator=g).half()
    plan = LB.ChunkedMoE(S, M, E, k, 1.0, n, torch.float16, device=DEV)
    first = plan.dispatch(x, gate).clone()
    other = torch.full_like(first, 7.0)
    plan.scatter(y, out=other)
    again = torch.full_like(first, 7.0)
    plan.scatter(x, out=again)
    assert torch.equal(again, first)                       # same rows, same zero padding
    il = plan.idx_loc.cpu().numpy()
    yh, oh = y.cpu().numpy(), other.cpu().numpy()
    Sp = S // n
    for c in range(n):
        for j in range(k):
            idx, loc = il[c, 2 * j], il[c, 2 * j + 1]
            kept = idx >= 0
            np.testing.assert_array_equal(oh[idx[kept], loc[kept]], yh[c * Sp:(c + 1) * Sp][kept])
    used = plan.capused.cpu().numpy()[-1]
    for e in range(E):
        assert (oh[e, used[e]:] == 0).all()


def test_chained_and_plain_launches_give_the_same_bits():
    """lancet_set_chained_launch: programmatic stream serialization only overlaps launch latency and drain."""
    from lancet_b200 import _capi
    rng = np.random.default_rng(5)
    S, E, M = 4096, 8, 256
    x = torch.from_numpy(rng.standard_normal((S, M)).astype(np.float32)).half().to(DEV)
    gate = torch.softmax(torch.from_numpy(rng.standard_normal((S, E)).astype(np.float32)), dim=1).to(DEV)
    used = torch.zeros(E, dtype=torch.int32, device=DEV)
    outs = []
    try:
        for on in (1, 0, 1):
            _capi.check(_capi.lib().lancet_set_chained_launch(on))
            for _ in range(3):          # back-to-back steps: the next gate starts while the previous combine drains
                enc = LB.moe_encode(x, gate, used, 1.25, k=2)
                dec = LB.moe_decode(enc[4], enc[0], enc[1])
            torch.cuda.synchronize()
            outs.append([t.clone() for t in enc] + [dec.clone()])
    finally:
        _capi.check(_capi.lib().lancet_set_chained_launch(1))
    for other in outs[1:]:
        for a, b in zip(outs[0], other):
            assert torch.equal(a, b)

