"""The product's kernels against the reference project's OWN CUDA kernels, run on the same GPU.

oracle/_ref/libraf_ref_kernels.so holds src/op/dialect/cuda/kernels/{tutel_moe_dispatch,multi_tensor_lans}.cu of the
reference, compiled unmodified for sm_100a (oracle/ref_build/build_ref.py).  What the reference's operator classes
compute with TVM-compiled functions around those kernels (argmax, masked gate, argsort: src/op/dialect/cuda/moe.cc:133-150)
is prepared on the host here.  Inputs are restricted to what the reference kernels handle without reading or writing out
of bounds: merge_masks only with S a multiple of 1024 (tutel_moe_dispatch.cu:232 has no bound on S + thid),
redispatch_expert_input only with counts that fit the capacity (:440-452 has no bound on the target row), LANS without
empty tensors (multi_tensor_apply.cuh:67-70 never flushes after one).

Bars: bit-exact for indices, locations, counts and row movement; fp32 dot products rtol 1e-5; fp16 dot products (the
reference accumulates in half) atol 2e-2 of the row scale; LANS rel 1e-5 on parameters and moments and rel 1e-4 on the
step p_new - p_old.
"""
import numpy as np
import pytest
import torch

import lancet_b200 as LB
from oracle import lans_oracle
from tests import ref_kernels as R

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not R.available(), reason="oracle/_ref/libraf_ref_kernels.so not built")]
DEV = "cuda:0"
TDT = {"f32": torch.float32, "f16": torch.float16}


def rand_gate(rng, S, E, tilt=0.0):
    logits = rng.standard_normal((S, E)).astype(np.float32) + tilt * np.linspace(-1, 1, E, dtype=np.float32)
    return torch.softmax(torch.from_numpy(logits), dim=1).to(DEV)


@pytest.mark.parametrize("S,E,M,cf,dt,used", [
    (2048, 8, 512, 1.0, "f32", "zero"),        # the reference's CPU-runnable case
    (2048, 8, 512, 1.0, "f16", "random"),
    (3001, 5, 64, 0.5, "f32", "random"),       # ragged, many drops
    (1024, 32, 128, 1.25, "f16", "full"),      # some experts already full
    (16384, 16, 2048, 1.25, "f16", "random"),  # rows and experts of the benchmark configuration, one choice
])
def test_gate_locations_and_encode(S, E, M, cf, dt, used):
    rng = np.random.default_rng(S + E)
    x = torch.from_numpy(rng.standard_normal((S, M)).astype(np.float32)).to(TDT[dt]).to(DEV)
    gate = rand_gate(rng, S, E, tilt=1.0)
    C = LB.moe_capacity(S, E, cf, 1)
    if used == "zero":
        u = np.zeros(E, np.int32)
    elif used == "random":
        u = rng.integers(0, C + 1, E).astype(np.int32)
    else:
        u = np.where(np.arange(E) % 3 == 0, C, rng.integers(0, C, E)).astype(np.int32)
    used_t = torch.from_numpy(u).to(DEV)
    r_gs, r_idx, r_loc, r_cap, r_el, r_disp = R.encode(x, gate, used_t.clone(), C)
    gs, il, cap, el, disp = LB.moe_encode(x, gate, used_t.clone(), cf, k=1)
    assert torch.equal(il[0], r_idx), "indices (with -1 for dropped tokens)"
    kept = r_idx >= 0
    assert torch.equal(il[1][kept], r_loc[kept]), "locations of the kept tokens"
    assert torch.equal(cap, r_cap) and torch.equal(el.view(torch.int64), r_el)
    assert torch.equal(gs.view(-1), r_gs.to(gs.dtype))
    assert torch.equal(disp, r_disp), "dispatched rows and zero padding"
    assert int(kept.sum()) < S or used == "zero", "the case is meant to drop tokens"

    # decode and the four gradients on the same plan
    L = R.lib()
    tdt = TDT[dt]
    eo = torch.from_numpy(rng.standard_normal((E, C, M)).astype(np.float32)).to(tdt).to(DEV)
    dy = torch.from_numpy(rng.standard_normal((S, M)).astype(np.float32)).to(tdt).to(DEV)
    g_t = r_gs.to(tdt)
    h = R.is_half(x)
    out_r = torch.empty((S, M), dtype=tdt, device=DEV)
    R.ok(L.raf_ref_decode_forward(h, R.ptr(g_t), R.ptr(r_idx), R.ptr(r_loc), R.ptr(out_r), R.ptr(eo), S, M, C, E, R.stream()))
    assert torch.equal(LB.moe_decode(eo, g_t, il), out_r), "decode forward"
    dx_r = torch.empty((S, M), dtype=tdt, device=DEV)
    R.ok(L.raf_ref_encode_backward_data(h, R.ptr(r_idx), R.ptr(r_loc), R.ptr(dx_r), R.ptr(eo), S, M, C, E, R.stream()))
    assert torch.equal(LB.moe_encode_dx(eo, il), dx_r), "encode data gradient"
    dgs = torch.from_numpy(rng.standard_normal(S).astype(np.float32)).to(tdt).to(DEV)
    dg_r = torch.empty((S, E), dtype=tdt, device=DEV)
    R.ok(L.raf_ref_encode_backward_gate(h, R.ptr(dgs), R.ptr(r_idx), R.ptr(dg_r), S, E, R.stream()))
    assert torch.equal(LB.moe_encode_dg(dgs, il, E), dg_r), "encode gate gradient"
    de_r = torch.empty((E, C, M), dtype=tdt, device=DEV)
    R.ok(L.raf_ref_decode_backward_data(h, R.ptr(g_t), R.ptr(r_idx), R.ptr(r_loc), R.ptr(dy), R.ptr(de_r), S, M, C, E, R.stream()))
    assert torch.equal(LB.moe_decode_dx(dy, g_t, il, E, C), de_r), "decode data gradient"
    dgate_r = torch.empty(S, dtype=tdt, device=DEV)
    R.ok(L.raf_ref_decode_backward_gate(h, R.ptr(dgate_r), R.ptr(r_idx), R.ptr(r_loc), R.ptr(dy), R.ptr(eo), S, M, C, R.stream()))
    got = LB.moe_decode_dg(dy, eo, il, gates_dtype=tdt).view(-1).float()
    if dt == "f32":
        torch.testing.assert_close(got, dgate_r, rtol=1e-5, atol=1e-5 * float(np.sqrt(M)))
    else:   # the reference sums M half products in half precision
        torch.testing.assert_close(got, dgate_r.float(), rtol=2e-2, atol=2e-2 * float(np.sqrt(M)))


@pytest.mark.parametrize("n,dt", [(2, "f32"), (4, "f16")])
def test_chain_merge_masks_and_redispatch(n, dt):
    """n chained encodes (used capacity of one call feeds the next, capacity factor cf*n), then merge_masks and redispatch,
    every step with the reference kernels and with the product's (tests/python/op/cuda/test_cuda_moe.py:387-471)."""
    rng = np.random.default_rng(n)
    S, M, E, cf = 4096, 64, 4, 1.0
    Sp = S // n
    assert Sp % 1024 == 0
    tdt = TDT[dt]
    x = torch.from_numpy(rng.standard_normal((S, M)).astype(np.float32)).to(tdt).to(DEV)
    gate = rand_gate(rng, S, E, tilt=0.7)
    C = LB.moe_capacity(Sp, E, cf * n, 1)
    cap_r = torch.zeros(E, dtype=torch.int32, device=DEV)
    cap = cap_r.clone()
    r_il, r_d, ils, ds = [], [], [], []
    for i in range(n):
        sl = slice(i * Sp, (i + 1) * Sp)
        _, idx, loc, cap_r, _, disp = R.encode(x[sl].contiguous(), gate[sl].contiguous(), cap_r, C)
        r_il.append(torch.stack([idx, loc])); r_d.append(disp)
        out = LB.moe_encode(x[sl].contiguous(), gate[sl].contiguous(), cap, cf * n, k=1)
        ils.append(out[1]); ds.append(out[4]); cap = out[2]
        assert torch.equal(out[1][0], idx) and torch.equal(cap, cap_r) and torch.equal(out[4], disp)
    L = R.lib()
    tab = torch.zeros(2 * n, dtype=torch.int64, device=DEV)
    merged_r = torch.full((2, S), -7, dtype=torch.int32, device=DEV)
    R.ok(L.raf_ref_merge_masks(R.table([t[0] for t in r_il]), R.table([t[1] for t in r_il]), R.ptr(tab), R.ptr(merged_r[0]),
                               R.ptr(merged_r[1]), Sp, E, n, R.stream()))
    merged = LB.moe_merge_masks(ils, E)
    assert torch.equal(merged, merged_r), "merged masks"
    red_r = torch.zeros((E, C, M), dtype=tdt, device=DEV)   # the reference leaves rows past the merged count unwritten
    R.ok(L.raf_ref_redispatch(R.is_half(x), R.table(r_d), R.table([t[0] for t in r_il]), R.ptr(tab), R.ptr(red_r), Sp, M, C, E, n,
                              R.stream()))
    assert torch.equal(LB.moe_redispatch(ds, ils), red_r), "redispatched rows"


def test_redispatch_expert_input():
    rng = np.random.default_rng(12)
    n, C, G, M, LE, le = 3, 48, 4, 16, 2, 1
    datas = [torch.from_numpy(rng.standard_normal((C, G, M)).astype(np.float32)).to(DEV) for _ in range(n)]
    rcs = [torch.from_numpy((rng.integers(0, 16, G * LE) * M).astype(np.int64)).to(DEV) for _ in range(n)]   # sums stay below C*M
    tab = torch.zeros(2 * n, dtype=torch.int64, device=DEV)
    want = torch.zeros((C, G, M), dtype=torch.float32, device=DEV)
    R.ok(R.lib().raf_ref_redispatch_expert_input(0, R.table(datas), R.table(rcs), R.ptr(tab), R.ptr(want), le, LE, C, M, G, n, 1,
                                                 R.stream()))
    got = LB.moe_redispatch_expert_input(datas, rcs, le, LE)
    live = torch.zeros((C, G), dtype=torch.bool, device=DEV)
    for g in range(G):
        live[: int(sum(int(r[g * LE + le]) for r in rcs)) // M, g] = True
    assert torch.equal(got[live], want[live]), "compacted rows"


@pytest.mark.parametrize("S,E,M,n,cf", [(1024, 32, 128, 1, 1.0), (2048, 64, 128, 1, 1.0), (2048, 32, 16, 2, 2.0),
                                        (4096, 8, 32, 4, 2.0), (999, 3, 8, 1, 1.0), (65536, 2, 8, 4, 0.5)])
def test_batch_prioritized_locations(S, E, M, n, cf):
    """gen_location_bpr_kernel with the order a stable descending sort of the masked gate gives (equal gate values keep
    their token order: the product's documented tie rule; the operator's own argsort is TVM's), against
    moe_encode_batch_prioritized; shapes of tests/python/op/cuda/test_cuda_moe.py:160-327."""
    rng = np.random.default_rng(0)
    gate_np = rng.random((S, E), dtype=np.float32)
    x = torch.from_numpy(rng.standard_normal((S, M)).astype(np.float32)).to(DEV)
    gate = torch.from_numpy(gate_np).to(DEV)
    idx_full = torch.argmax(gate, dim=1).to(torch.int32)
    gs_full = gate.gather(1, idx_full.long()[:, None])[:, 0].contiguous()
    order = torch.sort(gs_full, descending=True, stable=True)[1].to(torch.int32)
    Sp = S // n
    L = R.lib()
    for pid in range(n):
        got = LB.moe_encode_batch_prioritized(x, gate, n, pid, cf)
        C = got[4].shape[1]
        idx = idx_full.clone()            # the operator recomputes the argmax on every call (moe.cc:638-645)
        loc = torch.zeros(Sp, dtype=torch.int32, device=DEV)
        mask = torch.zeros(S, dtype=torch.bool, device=DEV)
        cap = torch.zeros(E, dtype=torch.int32, device=DEV)
        el = torch.zeros(E, dtype=torch.int64, device=DEV)
        R.ok(L.raf_ref_gen_location_bpr(R.ptr(idx), R.ptr(order), R.ptr(loc), R.ptr(mask), R.ptr(cap), R.ptr(el), C, S, E, M, n, pid,
                                        R.stream()))
        p_idx = idx[pid * Sp:(pid + 1) * Sp].contiguous()
        disp = torch.empty((E, C, M), dtype=torch.float32, device=DEV)
        R.ok(L.raf_ref_encode_forward(0, R.ptr(p_idx), R.ptr(loc), None, R.ptr(x[pid * Sp:(pid + 1) * Sp].contiguous()), R.ptr(disp),
                                      Sp, M, C, E, R.stream()))
        assert torch.equal(got[1][0], p_idx), "indices"
        assert torch.equal(got[1][1], loc), "locations (-1 for dropped)"
        assert torch.equal(got[2], cap) and torch.equal(got[3].view(torch.int64), el)
        assert torch.equal(got[0].view(-1), gs_full[pid * Sp:(pid + 1) * Sp])
        assert torch.equal(got[4], disp), "dispatched rows"


LANS_SHAPES = [(64, 64), (1000,), (8191,), (8192,), (8193,), (3,), (1,), (300, 129), (70001,), (65536,), (200000,)]


def lans_inputs(shapes, seed, zero_grad=(), zero_param=()):
    rng = np.random.default_rng(seed)
    p = [rng.normal(0, 0.02, s).astype(np.float32) for s in shapes]
    g = [rng.normal(0, 1e-3, s).astype(np.float32) for s in shapes]
    m = [rng.normal(0, 1e-4, s).astype(np.float32) for s in shapes]
    v = [rng.uniform(0, 1e-6, s).astype(np.float32) for s in shapes]
    for i in zero_grad:
        g[i][...] = 0
    for i in zero_param:
        p[i][...] = 0
    return g, p, m, v


def lans_close(a, b, what, rtol=1e-5):
    scale = max(float(b.abs().max()), 1e-30)
    torch.testing.assert_close(a, b, rtol=rtol, atol=1e-6 * scale, msg=lambda s: what + ": " + s)


def step_close(p_new, p_ref, p_old, what):
    """The step p_new - p_old carries the rounding of p itself (two units in the last place of the largest parameter);
    elements whose step nearly cancels are held to 1e-6 of the largest step."""
    atol = max(2.0 ** -22 * float(p_old.abs().max()), 1e-6 * float((p_ref - p_old).abs().max()), 1e-30)
    torch.testing.assert_close(p_new - p_old, p_ref - p_old, rtol=1e-4, atol=atol, msg=lambda s: what + ": " + s)


@pytest.mark.parametrize("kw", [
    dict(), dict(mode=0), dict(normalize_grad=False), dict(bias_correction=0), dict(grad_averaging=0),
    dict(weight_decay=0.0), dict(mode=0, weight_decay=0.0, normalize_grad=False),
])
def test_lans_steps_match_the_reference_kernels(kw):
    """Three consecutive steps of multi_tensor_lans_cuda<float> (chunks of 65536, several chunks per tensor, aligned and
    unaligned sizes, a zero gradient and a zero parameter tensor) against lancet_lans, and both against the NumPy oracle."""
    g, p, m, v = lans_inputs(LANS_SHAPES, 1, zero_grad=(1,), zero_param=(2,))
    n = len(LANS_SHAPES)
    mine = [torch.from_numpy(a.copy()).to(DEV) for a in g + p + m + v]
    for step in (1, 2, 10):
        rng = np.random.default_rng(100 + step)
        g = [rng.normal(0, 1e-3, s).astype(np.float32) for s in LANS_SHAPES]
        g[1][...] = 0
        ref = [torch.from_numpy(a.copy()).to(DEV) for a in g] + [t.clone() for t in mine[n:]]
        for i in range(n):
            mine[i].copy_(ref[i])
        p_old = [t.clone() for t in mine[n:2 * n]]
        want = lans_oracle.lans_step(g, [t.cpu().numpy() for t in mine[n:2 * n]], [t.cpu().numpy() for t in mine[2 * n:3 * n]],
                                     [t.cpu().numpy() for t in mine[3 * n:]], step=step, **kw)
        R.lans(ref[:n], ref[n:2 * n], ref[2 * n:3 * n], ref[3 * n:], step, **kw)
        LB.lans(mine, step, **kw)
        for i in range(n):
            tag = "step %d tensor %d " % (step, i)
            lans_close(mine[n + i], ref[n + i], tag + "p")
            lans_close(mine[2 * n + i], ref[2 * n + i], tag + "m")
            lans_close(mine[3 * n + i], ref[3 * n + i], tag + "v")
            step_close(mine[n + i], ref[n + i], p_old[i], tag + "p_new - p_old")
            lans_close(torch.from_numpy(want[0][i]).to(DEV), ref[n + i], tag + "oracle p")
            lans_close(torch.from_numpy(want[1][i]).to(DEV), ref[2 * n + i], tag + "oracle m")
            lans_close(torch.from_numpy(want[2][i]).to(DEV), ref[3 * n + i], tag + "oracle v")
            step_close(torch.from_numpy(want[0][i]).to(DEV), ref[n + i], p_old[i], tag + "oracle step")


def test_lans_many_tensors_match_the_reference_kernels():
    """More tensors than one launch of the reference's multi-tensor harness holds (30 for five lists)."""
    shapes = [(int(s),) for s in np.random.default_rng(3).integers(1, 30000, 100)]
    g, p, m, v = lans_inputs(shapes, 4)
    n = len(shapes)
    mine = [torch.from_numpy(a.copy()).to(DEV) for a in g + p + m + v]
    ref = [t.clone() for t in mine]
    R.lans(ref[:n], ref[n:2 * n], ref[2 * n:3 * n], ref[3 * n:], 7)
    LB.lans(mine, 7)
    for i in range(n):
        lans_close(mine[n + i], ref[n + i], "p[%d]" % i)
        lans_close(mine[2 * n + i], ref[2 * n + i], "m[%d]" % i)
        lans_close(mine[3 * n + i], ref[3 * n + i], "v[%d]" % i)
        step_close(mine[n + i], ref[n + i], torch.from_numpy(p[i]).to(DEV), "step[%d]" % i)


def test_reference_kernel_times(capsys):
    """Same-GPU timing of the reference's kernels beside the product's, printed for the record (no bar): one-choice
    dispatch + combine at the benchmark's row count and width, and one LANS step over 77 M elements."""
    S, E, M, cf = 16384, 16, 2048, 1.25
    rng = np.random.default_rng(0)
    x = torch.from_numpy(rng.standard_normal((S, M)).astype(np.float32)).half().to(DEV)
    gate = rand_gate(rng, S, E)
    C = LB.moe_capacity(S, E, cf, 1)
    used = torch.zeros(E, dtype=torch.int32, device=DEV)
    out_r = torch.empty((S, M), dtype=torch.float16, device=DEV)
    L = R.lib()

    def ref_step():
        gs, idx, loc, _, _, disp = R.encode(x, gate, used, C)
        g_t = gs.half()
        R.ok(L.raf_ref_decode_forward(1, R.ptr(g_t), R.ptr(idx), R.ptr(loc), R.ptr(out_r), R.ptr(disp), S, M, C, E, R.stream()))

    def my_step():
        gs, il, _, _, disp = LB.moe_encode(x, gate, used, cf, k=1, gates_dtype=torch.float16)
        LB.moe_decode(disp, gs, il)

    def time_ms(fn, reps=10):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps

    t_ref, t_my = time_ms(ref_step), time_ms(my_step)
    shapes = [(4096, 4096)] * 4 + [(4096, 1024)] * 8 + [(1024,)] * 32 + [(50304, 256)]
    tl = [torch.randn(s, device=DEV) * 1e-2 for _ in range(4) for s in shapes]
    for i in range(3 * len(shapes), 4 * len(shapes)):
        tl[i].abs_()
    n = len(shapes)
    tr = [t.clone() for t in tl]
    t_lref = time_ms(lambda: R.lans(tr[:n], tr[n:2 * n], tr[2 * n:3 * n], tr[3 * n:], 5), reps=5)
    t_lmy = time_ms(lambda: LB.lans(tl, 5), reps=5)
    with capsys.disabled():
        print("\nreference kernels on this GPU (host-synchronised calls, eager): encode+decode S=%d M=%d E=%d fp16 top-1: "
              "reference %.3f ms, product %.3f ms; LANS %.1f M elements: reference %.3f ms, product %.3f ms"
              % (S, M, E, t_ref, t_my, sum(int(np.prod(s)) for s in shapes) / 1e6, t_lref, t_lmy))
