"""LANS step through the C ABI against the NumPy oracle (float32 arithmetic order of the reference
kernels, and its float64 variant).  Tolerance: rel 1e-5 on parameters and moments."""
import numpy as np
import pytest
import torch

import lancet_b200 as LB
from oracle import lans_oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def make(shapes, seed, zero_grad=(), zero_param=()):
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


def close(a, b, what):
    scale = max(float(np.abs(b).max()), 1e-30) if b.size else 1.0
    np.testing.assert_allclose(a, b, rtol=1e-5, atol=1e-6 * scale, err_msg=what)


SHAPES = [(64, 64), (1000,), (8191,), (8192,), (8193,), (3,), (1,), (0,), (300, 129), (20000,)]


@pytest.mark.parametrize("kw", [
    dict(), dict(mode=0), dict(normalize_grad=False), dict(bias_correction=0), dict(grad_averaging=0),
    dict(weight_decay=0.0), dict(mode=0, weight_decay=0.0, normalize_grad=False),
])
def test_one_step_matches_oracle(kw):
    g, p, m, v = make(SHAPES, 1, zero_grad=(1,), zero_param=(2,))
    wp, wm, wv = lans_oracle.lans_step(g, p, m, v, step=10, **kw)
    wp64, wm64, wv64 = lans_oracle.lans_step(g, p, m, v, step=10, dtype=np.float64, **kw)
    tl = [torch.from_numpy(a.copy()).to(DEV) for a in g + p + m + v]
    g_before = [t.clone() for t in tl[:len(SHAPES)]]
    LB.lans(tl, 10, **kw)
    n = len(SHAPES)
    for i in range(n):
        close(tl[n + i].cpu().numpy(), wp[i], "p[%d]" % i)
        close(tl[2 * n + i].cpu().numpy(), wm[i], "m[%d]" % i)
        close(tl[3 * n + i].cpu().numpy(), wv[i], "v[%d]" % i)
        close(tl[n + i].cpu().numpy(), wp64[i].astype(np.float32), "p64[%d]" % i)
        assert torch.equal(tl[i], g_before[i]), "gradients must stay untouched"


def test_steps_reuse_tables_and_unaligned_views():
    shapes = [(4097,), (33, 7), (12345,)]
    g, p, m, v = make(shapes, 2)
    # views that start one element into a buffer: not 16-byte aligned -> scalar path
    def off1(a):
        buf = torch.zeros(a.size + 1, dtype=torch.float32, device=DEV)
        view = buf[1:].view(*a.shape)
        view.copy_(torch.from_numpy(a))
        return view
    tl = [off1(a) for a in g + p + m + v]
    assert tl[0].data_ptr() % 16 != 0
    state = LB.LansState(tl[0:3], tl[3:6], tl[6:9], tl[9:12])
    for step in range(1, 5):
        p, m, v = lans_oracle.lans_step(g, p, m, v, step=step, lr=2e-3)
        LB.lans(tl, step, learning_rate=2e-3, state=state)
        assert state.ready
    for i in range(3):
        close(tl[3 + i].cpu().numpy(), p[i], "p[%d]" % i)
        close(tl[6 + i].cpu().numpy(), m[i], "m[%d]" % i)
        close(tl[9 + i].cpu().numpy(), v[i], "v[%d]" % i)


def test_many_tensors_deterministic():
    shapes = [(int(s),) for s in np.random.default_rng(3).integers(1, 30000, 300)]
    g, p, m, v = make(shapes, 4)
    outs = []
    for _ in range(2):
        tl = [torch.from_numpy(a.copy()).to(DEV) for a in g + p + m + v]
        LB.lans(tl, 3)
        outs.append(torch.cat([t.flatten() for t in tl[300:600]]).cpu())
    assert torch.equal(outs[0], outs[1])        # fixed-order reductions: run-to-run identical
    wp, _, _ = lans_oracle.lans_step(g, p, m, v, step=3)
    close(outs[0].numpy(), np.concatenate([a.ravel() for a in wp]), "p")


def test_step_counter_on_the_device_gives_the_same_bits():
    """`lancet_lans_dev_step`: the step stays a float32 scalar on the device, as raf.op.lans receives it
    (src/op/dialect/cuda/lans.cc:102-107 of the reference reads it back; here no host round trip)."""
    shapes = [(4096,), (8193,), (5, 7)]
    g, p, m, v = make(shapes, 9)
    a = [torch.from_numpy(x.copy()).to(DEV) for x in g + p + m + v]
    b = [torch.from_numpy(x.copy()).to(DEV) for x in g + p + m + v]
    step = torch.zeros((), dtype=torch.float32, device=DEV)
    for it in (1, 2, 37):
        step.fill_(float(it))
        LB.lans(a, step)
        LB.lans(b, it)
        for x, y in zip(a, b):
            assert torch.equal(x, y)
    with pytest.raises(TypeError):
        LB.lans(a, torch.zeros((), dtype=torch.int32, device=DEV))
