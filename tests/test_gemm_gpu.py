"""Grouped expert GEMM (tcgen05) against a float32 torch reference of the same contraction.
Tolerance for 16-bit operands with fp32 accumulation: rel 1e-2 of the row scale."""
import ctypes

import numpy as np
import pytest
import torch

import lancet_b200 as LB
from lancet_b200 import _capi

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def reference(a, b, bias, act):
    groups, C, K = a.shape
    LE = b.shape[0]
    out = torch.empty((groups, C, b.shape[1]), dtype=torch.float32, device=a.device)
    for g in range(groups):
        y = a[g].float() @ b[g % LE].float().t()
        if bias is not None:
            y = y + bias[g % LE].float()
        if act == "relu":
            y = torch.relu(y)
        elif act == "gelu":
            y = torch.nn.functional.gelu(y)
        elif act == "gelu_tanh":
            y = torch.nn.functional.gelu(y, approximate="tanh")
        out[g] = y
    return out


def check_status():
    st = LB.gemm_status(torch.device(DEV))
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    _capi.check(_capi.lib().lancet_p2p_status(ctypes.c_void_p(st.data_ptr()), stream))


@pytest.mark.parametrize("groups,LE,C,N,K,dt,act,use_bias,ragged", [
    (2, 2, 128, 256, 64, torch.bfloat16, None, False, False),       # one tile, one k block
    (2, 1, 128, 256, 256, torch.bfloat16, None, False, False),      # pipeline wraps the 4 stages once
    (4, 2, 256, 512, 1024, torch.bfloat16, "gelu", True, False),
    (4, 2, 200, 256, 136, torch.float16, "relu", True, True),       # C and K not multiples of the tile
    (16, 2, 640, 1024, 512, torch.bfloat16, "gelu_tanh", True, True),
    (6, 2, 2560, 2048, 2048, torch.bfloat16, "gelu", True, True),   # many tiles per CTA, both accumulators
])
def test_grouped_gemm_matches_fp32_reference(groups, LE, C, N, K, dt, act, use_bias, ragged):
    g = torch.Generator(device=DEV).manual_seed(groups * 1000 + C + N + K)
    a = torch.randn((groups, C, K), device=DEV, generator=g).to(dt)
    b = (torch.randn((LE, N, K), device=DEV, generator=g) * 0.02).to(dt)
    bias = (torch.randn((LE, N), device=DEV, generator=g) * 0.1).to(dt) if use_bias else None
    counts = None
    if ragged:
        counts = torch.randint(0, C + 1, (groups,), device=DEV, generator=g, dtype=torch.int32)
        counts[0] = C
        counts[-1] = 0
    out = torch.full((groups, C, N), 7.0, dtype=dt, device=DEV)
    pre = torch.full((groups, C, N), 7.0, dtype=dt, device=DEV)
    LB.grouped_gemm_nt(a, b, bias=bias, counts=counts, act=act, out=out, preact=pre)
    torch.cuda.synchronize()
    check_status()
    want = reference(a, b, bias, act)
    want_pre = reference(a, b, bias, None)
    scale = float(want_pre.abs().max()) + 1e-6
    for gi in range(groups):
        n = C if counts is None else int(counts[gi])
        got = out[gi, :n].float()
        assert torch.allclose(got, want[gi, :n], rtol=1e-2, atol=1e-2 * scale), (gi, (got - want[gi, :n]).abs().max())
        assert torch.allclose(pre[gi, :n].float(), want_pre[gi, :n], rtol=1e-2, atol=1e-2 * scale)
        pad_end = min(C, (n + 127) // 128 * 128)
        assert (out[gi, n:pad_end].float() == 0.0).all(), "dead rows of a live tile are zero"
        assert (out[gi, pad_end:].float() == 7.0).all(), "rows of dead tiles must not be written"


def test_gemm_rejects_bad_arguments():
    a = torch.zeros((2, 128, 64), dtype=torch.bfloat16, device=DEV)
    b = torch.zeros((2, 100, 64), dtype=torch.bfloat16, device=DEV)    # N not a multiple of 256
    with pytest.raises(LB.LancetError) as ei:
        LB.grouped_gemm_nt(a, b)
    assert ei.value.code == 1
    with pytest.raises(TypeError):
        LB.grouped_gemm_nt(a.float(), b.float())


def dact_ref(x, act):
    x = x.detach().clone().requires_grad_(True)
    if act == "relu":
        y = torch.relu(x)
    elif act == "gelu":
        y = torch.nn.functional.gelu(x)
    elif act == "gelu_tanh":
        y = torch.nn.functional.gelu(x, approximate="tanh")
    else:
        return torch.ones_like(x)
    y.sum().backward()
    return x.grad


@pytest.mark.parametrize("groups,LE,C,N,K,dt,act,ragged", [
    (2, 2, 128, 256, 64, torch.bfloat16, None, False),
    (4, 2, 256, 512, 1024, torch.bfloat16, "gelu", False),
    (4, 2, 200, 256, 192, torch.float16, "relu", True),
    (6, 2, 1280, 2048, 512, torch.bfloat16, "gelu_tanh", True),
])
def test_data_gradient_gemm(groups, LE, C, N, K, dt, act, ragged):
    g = torch.Generator(device=DEV).manual_seed(groups * 77 + C + N + K)
    a = torch.randn((groups, C, K), device=DEV, generator=g).to(dt)
    b = (torch.randn((LE, K, N), device=DEV, generator=g) * 0.05).to(dt)
    pre = torch.randn((groups, C, N), device=DEV, generator=g).to(dt)
    counts = None
    if ragged:
        counts = torch.randint(0, C + 1, (groups,), device=DEV, generator=g, dtype=torch.int32)
        counts[0] = C
    out = torch.full((groups, C, N), 7.0, dtype=dt, device=DEV)
    LB.grouped_gemm_nn(a, b, counts=counts, act=act, preact=pre if act else None, out=out)
    torch.cuda.synchronize()
    check_status()
    for gi in range(groups):
        n = C if counts is None else int(counts[gi])
        want = (a[gi, :n].float() @ b[gi % LE].float()) * dact_ref(pre[gi, :n].float(), act)
        scale = float(want.abs().max()) + 1e-6 if n else 1.0
        assert torch.allclose(out[gi, :n].float(), want, rtol=1e-2, atol=1e-2 * scale), (gi, (out[gi, :n].float() - want).abs().max())


@pytest.mark.parametrize("groups,LE,C,Mout,N,dt,ragged", [
    (2, 2, 64, 128, 256, torch.bfloat16, False),
    (4, 2, 256, 256, 512, torch.bfloat16, False),
    (8, 2, 200, 128, 256, torch.float16, True),
    (6, 2, 1280, 1024, 512, torch.bfloat16, True),
    (4, 2, 160, 128, 256, torch.bfloat16, False),      # C not a multiple of the 64-row reduction block
    (4, 2, 100, 128, 256, torch.bfloat16, True),
])
def test_weight_gradient_gemm(groups, LE, C, Mout, N, dt, ragged):
    g = torch.Generator(device=DEV).manual_seed(groups * 55 + C + Mout + N)
    a = torch.randn((groups, C, Mout), device=DEV, generator=g).to(dt)
    b = torch.randn((groups, C, N), device=DEV, generator=g).to(dt)
    counts = None
    if ragged:
        counts = torch.randint(0, C + 1, (groups,), device=DEV, generator=g, dtype=torch.int32)
        counts[1] = 0
        for gi in range(groups):                       # contract: dead rows of a partial 64-row block are zero in one operand
            n = int(counts[gi])
            b[gi, n:] = 0
            a[gi, n:] = 3.0                            # finite garbage in the other
    out = LB.grouped_gemm_tn(a, b, LE, counts=counts)
    torch.cuda.synchronize()
    check_status()
    for e in range(LE):
        want = torch.zeros((Mout, N), dtype=torch.float32, device=DEV)
        for gi in range(e, groups, LE):
            n = C if counts is None else int(counts[gi])
            want += a[gi, :n].float().t() @ b[gi, :n].float()
        scale = float(want.abs().max()) + 1e-6
        assert torch.allclose(out[e].float(), want, rtol=1e-2, atol=1e-2 * scale), (e, (out[e].float() - want).abs().max())


def test_weight_gradient_all_groups_empty():
    a = torch.randn((2, 64, 128), device=DEV).bfloat16()
    b = torch.randn((2, 64, 256), device=DEV).bfloat16()
    counts = torch.zeros(2, dtype=torch.int32, device=DEV)
    out = LB.grouped_gemm_tn(a, b, 2, counts=counts)
    torch.cuda.synchronize()
    check_status()
    assert (out == 0).all()


def test_gemm_empty_groups_and_zero_capacity():
    a = torch.randn((4, 256, 64), device=DEV).bfloat16()
    b = torch.randn((2, 256, 64), device=DEV).bfloat16()
    out = torch.full((4, 256, 256), 7.0, dtype=torch.bfloat16, device=DEV)
    counts = torch.zeros(4, dtype=torch.int32, device=DEV)
    LB.grouped_gemm_nt(a, b, counts=counts, out=out)          # nothing is live: nothing may be written
    torch.cuda.synchronize()
    check_status()
    assert (out.float() == 7.0).all()
    empty = LB.grouped_gemm_nt(a[:, :0].contiguous(), b)      # C == 0
    assert empty.shape == (4, 0, 256)
    dw = LB.grouped_gemm_tn(torch.zeros((4, 0, 128), dtype=torch.bfloat16, device=DEV),
                            torch.zeros((4, 0, 256), dtype=torch.bfloat16, device=DEV), 2)
    torch.cuda.synchronize()
    assert dw.shape == (2, 128, 256) and (dw == 0).all()     # an empty reduction is zero


@pytest.mark.parametrize("groups,LE,C,N,K,stages", [(8, 2, 1000, 512, 256, 4), (3, 1, 300, 256, 64, 3), (40, 2, 130, 256, 128, 2)])
def test_row_windows_tile_the_full_product(groups, LE, C, N, K, stages):
    """Stages over disjoint row windows reproduce the one-call result bit for bit and touch nothing outside
    their window (plus the zeroed rest of the last tile)."""
    g = torch.Generator(device=DEV).manual_seed(groups * 7 + stages)
    a = torch.randn((groups, C, K), device=DEV, generator=g).bfloat16()
    b = (torch.randn((LE, N, K), device=DEV, generator=g) * 0.1).bfloat16()
    bias = torch.randn((LE, N), device=DEV, generator=g).bfloat16()
    counts = torch.randint(0, C + 1, (groups,), device=DEV, generator=g, dtype=torch.int32)
    counts[0] = C
    if groups > 2:
        counts[2] = 0
    full = torch.full((groups, C, N), 3.0, device=DEV, dtype=torch.bfloat16)
    pre_full = torch.full_like(full, 3.0)
    LB.grouped_gemm_nt(a, b, bias=bias, counts=counts, act="gelu", out=full, preact=pre_full)
    # stage s ends at a random point of the live rows rounded down to a tile; the last one at the count
    cuts = torch.sort(torch.rand((stages - 1, groups), device=DEV, generator=g), dim=0).values
    ends = [(cuts[s] * counts).to(torch.int32) // 128 * 128 for s in range(stages - 1)] + [counts]
    begins = [torch.zeros_like(counts)] + ends[:-1]
    out = torch.full_like(full, 3.0)
    pre = torch.full_like(full, 3.0)
    for s in range(stages):
        before = out.clone()
        LB.grouped_gemm_nt(a, b, bias=bias, counts=ends[s].contiguous(), row_begin=begins[s].contiguous(), act="gelu", out=out,
                           preact=pre)
        lo, hi = begins[s].cpu().numpy(), ends[s].cpu().numpy()
        changed = (out != before).any(dim=2).cpu().numpy()
        for gi in range(groups):
            rows = np.nonzero(changed[gi])[0]
            if rows.size:
                assert rows.min() >= lo[gi] and rows.max() < (hi[gi] + 127) // 128 * 128, (s, gi, rows.min(), rows.max())
    assert torch.equal(out, full) and torch.equal(pre, pre_full)
    # data-gradient form
    w = (torch.randn((LE, K, N), device=DEV, generator=g) * 0.1).bfloat16()
    dfull = torch.full((groups, C, N), 5.0, device=DEV, dtype=torch.bfloat16)
    LB.grouped_gemm_nn(a, w, counts=counts, act="gelu", preact=pre_full, out=dfull) if K % 64 == 0 else None
    if K % 64 == 0:
        dout = torch.full_like(dfull, 5.0)
        for s in range(stages):
            LB.grouped_gemm_nn(a, w, counts=ends[s].contiguous(), row_begin=begins[s].contiguous(), act="gelu", preact=pre_full,
                               out=dout)
        assert torch.equal(dout, dfull)
    check_status()


@pytest.mark.parametrize("C,G,M,N,elements,stride,offset,scale,dt", [
    (256, 5, 768, 3072, [128, 32, 256, 32, 64], 2, 1, 1, torch.float16),   # the reference's own test configuration
    (300, 3, 264, 256, [300, 0, 17], 1, 0, 1, torch.bfloat16),             # full, empty and ragged blocks; C, M off the tile
    (128, 16, 128, 512, list(range(0, 128, 8)), 3, 2, 4, torch.bfloat16),  # counts given in units of 4 elements
])
def test_sparse_expert_matmul_nt(C, G, M, N, elements, stride, offset, scale, dt):
    """tests/python/op/cublas/test_sparse_expert_matmul_nt.py of the reference: [C, G, M] x [N, M]^T with per-source
    element counts; here the rows past the counts must come out zero."""
    from oracle import moe_oracle as O
    rng = np.random.default_rng(C + G)
    x = rng.standard_normal((C, G, M)).astype(np.float32)
    w = (rng.standard_normal((N, M)) * 0.1).astype(np.float32)
    nelem = rng.integers(0, 256, size=stride * G).astype(np.int64)
    for i, e in enumerate(elements):
        nelem[i * stride + offset] = e * M // scale
    xd = torch.from_numpy(x).to(DEV).to(dt)
    wd = torch.from_numpy(w).to(DEV).to(dt)
    out = torch.full((C, G, N), 9.0, device=DEV, dtype=dt)
    LB.sparse_expert_matmul_nt(xd, wd, torch.from_numpy(nelem).to(DEV), offset, stride, scale, out=out)
    ref = O.sparse_expert_matmul_nt(xd.float().cpu().numpy(), wd.float().cpu().numpy(), nelem, offset, stride, scale)
    got = out.float().cpu().numpy()
    for gi, e in enumerate(elements):
        assert (got[e:, gi] == 0).all(), "rows past the count of block %d must be zero" % gi
    scale_ = np.abs(ref).max() + 1e-6
    assert np.abs(got - ref).max() <= 1e-2 * scale_          # 16-bit operands, fp32 accumulation
    check_status()


@pytest.mark.parametrize("C,counts_kind", [(2560, "full"), (640, "ragged"), (384, "odd")])
def test_paired_and_single_cta_forms_agree_bit_for_bit(C, counts_kind):
    """The two-CTA form (tcgen05 cta_group::2, 256 x 256 tile per CTA pair) and the single-CTA form run the same
    contraction in the same order per output element: forward, data-gradient and weight-gradient forms must agree exactly."""
    L = _capi.lib()
    groups, LE, M, H = 8, 2, 512, 1024
    g = torch.Generator(device=DEV).manual_seed(C)
    x = torch.randn((groups, C, M), device=DEV, generator=g).bfloat16()
    w1 = (torch.randn((LE, H, M), device=DEV, generator=g) * 0.05).bfloat16()
    b1 = (torch.randn((LE, H), device=DEV, generator=g) * 0.1).bfloat16()
    dy = torch.randn((groups, C, H), device=DEV, generator=g).bfloat16()
    counts = None
    if counts_kind == "ragged":
        counts = torch.randint(0, C + 1, (groups,), device=DEV, generator=g, dtype=torch.int32)
        counts[1] = C
        counts[2] = 0
    elif counts_kind == "odd":
        counts = torch.tensor([384, 129, 128, 1, 0, 257, 300, 383], device=DEV, dtype=torch.int32)   # odd tile counts: dead second halves
    res = []
    try:
        for paired in (1, 0):
            _capi.check(L.lancet_set_gemm_paired(paired))
            h = torch.zeros((groups, C, H), dtype=torch.bfloat16, device=DEV)
            pre = torch.zeros_like(h)
            LB.grouped_gemm_nt(x, w1, bias=b1, counts=counts, act="gelu", out=h, preact=pre)
            dx = torch.zeros_like(x)
            LB.grouped_gemm_nn(dy, w1, counts=counts, out=dx)
            dh = torch.zeros_like(h)
            LB.grouped_gemm_nn(x, w1.transpose(1, 2).contiguous(), counts=counts, act="gelu", preact=pre, out=dh)
            dw = torch.zeros_like(w1)
            LB.grouped_gemm_tn(dy, x, LE, counts=counts, out=dw)
            torch.cuda.synchronize()
            check_status()
            res.append((h, pre, dx, dh, dw))
    finally:
        _capi.check(L.lancet_set_gemm_paired(1))
    for a, b in zip(*res):
        assert torch.equal(a, b)
    # and the paired results are right: spot check the forward against float32
    want = reference(x, w1, b1, "gelu")
    n0 = C if counts is None else int(counts[0])
    assert torch.allclose(res[0][0][0, :n0].float(), want[0, :n0], rtol=1e-2, atol=1e-2 * float(want.abs().max()))
