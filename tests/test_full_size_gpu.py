"""Full benchmark sizes, checked through size-independent properties (the CPU oracle would take too long):
dispatch followed by combine with identity experts returns sum_j gate_j * x for kept choices and 0 for dropped
ones; kept (expert, location) pairs are unique, dense per expert and in token order; capacity accounting adds
up; the LANS step at the 354.6 M-element tensor list equals a float32 torch restatement of the same update."""
import numpy as np
import pytest
import torch

import lancet_b200 as LB

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("E", [2, 16])
def test_moe_config3_properties(E):
    S, M, k, cf, n = 16384, 2048, 2, 1.25, 4
    g = torch.Generator(device=DEV).manual_seed(1000)
    x = torch.randn((S, M), device=DEV, generator=g).half()
    bias = torch.linspace(1.5, -1.5, E, device=DEV)                                      # popular and unpopular experts: forces drops
    gate = torch.softmax(torch.randn((S, E), device=DEV, generator=g) + bias, dim=1)
    plan = LB.ChunkedMoE(S, M, E, k, cf, n, torch.float16, device=DEV)
    disp = plan.dispatch(x, gate)
    out = plan.combine()
    torch.cuda.synchronize()
    Sp, C = S // n, plan.C
    il = plan.idx_loc.permute(1, 0, 2).reshape(2 * k, S)           # [2k, S] in token order
    gs = plan.gates_s.permute(1, 0, 2).reshape(k, S)
    idx = torch.stack([il[0], il[2]])
    loc = torch.stack([il[1], il[3]])
    kept = idx >= 0
    assert E == 2 or int((~kept).sum()) > 0      # with E == k every expert receives exactly S rows: nothing can drop
    # round trip with identity experts
    want = torch.zeros((S, M), device=DEV, dtype=torch.float32)
    for j in range(k):
        want += torch.where(kept[j], gs[j], torch.zeros_like(gs[j])).unsqueeze(1) * x.float()
    assert torch.allclose(out.float(), want, rtol=2e-3, atol=2e-3)
    # kept rows hold exactly their token; all other rows are zero
    rows = (idx.long() * C + loc.long())[kept]
    assert rows.unique().numel() == rows.numel()
    flat = disp.view(E * C, M)
    tok = torch.arange(S, device=DEV).repeat(k, 1)[kept]
    assert torch.equal(flat[rows], x[tok])
    mask = torch.ones(E * C, dtype=torch.bool, device=DEV)
    mask[rows] = False
    assert int(flat[mask].abs().sum()) == 0
    # dense per expert, in token order (first choices of a chunk before its second choices), capacity chain adds up
    cap = plan.capused[-1]
    for e in range(E):
        le = loc[kept & (idx == e)]
        assert le.numel() == int(cap[e]) and le.numel() <= C
        assert torch.equal(le.sort().values, torch.arange(le.numel(), device=DEV, dtype=le.dtype))
    chain = plan.capused.cpu().numpy()
    el = plan.elems.cpu().view(torch.int64).numpy()
    assert (chain[0] == 0).all() and (np.diff(chain, axis=0) >= 0).all()
    np.testing.assert_array_equal(el, np.diff(chain, axis=0).astype(np.int64) * M)
    # chained single-chunk calls give the same masks as the one-pass chain
    cap_t = torch.zeros(E, dtype=torch.int32, device=DEV)
    for c in range(n):
        gsc, ilc, cap_t, _ = LB.moe_gate(gate[c * Sp:(c + 1) * Sp].contiguous(), cap_t, C, M, k=k,
                                         flags=LB._capi.GATE_GLOBAL_LOC)
        assert torch.equal(ilc, plan.idx_loc[c]) and torch.equal(gsc, plan.gates_s[c])


def test_lans_config2_against_torch():
    import sys, os
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from bench import lans_shapes
    shapes = lans_shapes()
    g = torch.Generator(device=DEV).manual_seed(0)
    P = [torch.randn(s, device=DEV, generator=g) * 0.02 for s in shapes]
    G = [torch.randn(s, device=DEV, generator=g) * 1e-3 for s in shapes]
    Mo = [torch.randn(s, device=DEV, generator=g) * 1e-4 for s in shapes]
    V = [torch.rand(s, device=DEV, generator=g) * 1e-6 for s in shapes]
    assert len(shapes) == 196 and abs(sum(p.numel() for p in P) - 350e6) < 10e6
    lr, b1, b2, eps, wd, step = 1e-3, 0.9, 0.999, 1e-6, 0.01, 10
    # the op takes float32 hyper-parameters and forms 1 - beta in float32 (as the reference kernels do,
    # multi_tensor_lans.cu:283-307): 1 - 0.999f differs from 0.001 by 1.3e-5 relative, so use the same constants
    f32 = np.float32
    b1, b2, eps, wd, lr = (float(f32(v)) for v in (b1, b2, eps, wd, lr))
    omb1, omb2 = float(f32(1) - f32(b1)), float(f32(1) - f32(b2))
    bc1, bc2 = float(f32(1 - b1 ** step)), float(f32(1 - b2 ** step))
    # spot-check tensors of every shape class against a float64 torch restatement (lans_oracle semantics)
    picks = [0, 1, 2, 6, 7, 8, 195]
    want = {}
    for i in picks:
        gi, pi, mi, vi = (t[i].double() for t in (G, P, Mo, V))
        sg = gi / (gi.norm() + eps)
        m2 = mi * b1 + omb1 * sg
        v2 = vi * b2 + omb2 * sg * sg
        den = (v2 / bc2).sqrt() + eps
        um = (m2 / bc1) / den + wd * pi
        ug = sg / den + wd * pi
        rm = lr * pi.norm() / um.norm() * b1
        rg = lr * pi.norm() / ug.norm() * omb1
        want[i] = (pi - rm * um - rg * ug, m2, v2)
    LB.lans(G + P + Mo + V, step)
    torch.cuda.synchronize()
    for i in picks:
        for got, w in zip((P[i], Mo[i], V[i]), want[i]):
            scale = float(w.abs().max())
            assert float((got.double() - w).abs().max()) <= 1e-5 * scale + 1e-12
