"""Forward and backward of the fused expert-parallel MoE layer (W virtual ranks on one GPU) against a
float32 torch autograd reference of the same routing.  bf16 operands: tolerance rel 1e-2 of the scale."""
import numpy as np
import pytest
import torch

import lancet_b200 as LB

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def close(a, b, what, tol=2e-2):
    scale = float(b.abs().max()) + 1e-6
    err = float((a.float() - b).abs().max())
    assert err <= tol * scale, "%s: max err %g vs scale %g" % (what, err, scale)


@pytest.mark.parametrize("W,k,n,act", [(1, 2, 4, "gelu"), (2, 2, 2, "gelu"), (2, 1, 1, "gelu"), (2, 2, 2, "relu")])
def test_layer_forward_backward(W, k, n, act):
    S, M, H, LE, cf = 512, 256, 512, 2, 1.25
    E = LE * W
    shared = {}
    layers = [LB.MoELayer(S, M, H, k, cf, n, torch.bfloat16, DEV, LE, fabric=LB.LocalFabric(W, r, shared), seed=5, act=act)
              for r in range(W)]
    assert (layers[0].hpre is None) == (act == "relu")        # ReLU keeps no pre-activation copy
    fact = torch.relu if act == "relu" else torch.nn.functional.gelu
    g = torch.Generator(device=DEV).manual_seed(W * 10 + k)
    xs = [torch.randn((S, M), device=DEV, generator=g).bfloat16() for _ in range(W)]
    gates = [torch.softmax(torch.randn((S, E), device=DEV, generator=g), dim=1) for _ in range(W)]
    douts = [torch.randn((S, M), device=DEV, generator=g).bfloat16() for _ in range(W)]
    for step in range(2):
        for r, l in enumerate(layers):
            l.fwd_dispatch(xs[r], gates[r])
        for l in layers:
            l.fwd_experts()
        outs = [l.fwd_combine().clone() for l in layers]
        for r, l in enumerate(layers):
            l.bwd_combine(douts[r])
        for l in layers:
            l.bwd_experts()
        res = [l.bwd_dispatch() for l in layers]
        torch.cuda.synchronize()
    # ---- float32 reference with the routing the device chose ----
    xr = [x.float().requires_grad_(True) for x in xs]
    w1 = [l.w1.float().requires_grad_(True) for l in layers]
    w2 = [l.w2.float().requires_grad_(True) for l in layers]
    b1 = [l.b1.float().requires_grad_(True) for l in layers]
    b2 = [l.b2.float().requires_grad_(True) for l in layers]
    gs = [l.moe.gates_s.clone().requires_grad_(True) for l in layers]        # [n, k, Sp]
    loss = 0
    ref_out = []
    Sp = S // n
    for r, l in enumerate(layers):
        il = l.moe.idx_loc                                                   # [n, 2k, Sp]
        out = torch.zeros((S, M), device=DEV)
        for c in range(n):
            for j in range(k):
                idx = il[c, 2 * j]
                for e in range(E):
                    sel = (idx == e).nonzero().flatten()
                    if sel.numel() == 0:
                        continue
                    own, le = e // LE, e % LE
                    tok = c * Sp + sel
                    hpre = xr[r][tok] @ w1[own][le].t() + b1[own][le]
                    y = fact(hpre) @ w2[own][le].t() + b2[own][le]
                    out = out.index_add(0, tok, gs[r][c, j, sel].unsqueeze(1) * y)
        ref_out.append(out)
        loss = loss + (out * douts[r].float()).sum()
    loss.backward()
    # ReLU's derivative jumps at 0: a pre-activation within rounding of 0 can take the other branch in the float32
    # reference (another summation order), which moves one row of dx by one |dh * w1| term; the tolerance allows for it
    gtol = 5e-2 if act == "relu" else 2e-2
    for r, l in enumerate(layers):
        close(outs[r], ref_out[r].detach(), "out[%d]" % r)
        dx, dgates = res[r]
        close(dx, xr[r].grad, "dx[%d]" % r, gtol)
        close(dgates, gs[r].grad, "dgates[%d]" % r)
        close(l.dw1, w1[r].grad, "dw1[%d]" % r, gtol)
        close(l.dw2, w2[r].grad, "dw2[%d]" % r)
        close(l.db1, b1[r].grad, "db1[%d]" % r, gtol)
        close(l.db2, b2[r].grad, "db2[%d]" % r)
    st = LB.gemm_status(torch.device(DEV))
    assert int(st.item()) == 0


def test_combine_backward_halves_equal_the_joint_pass():
    """lancet_moe_combine_bwd_part_p2p: rows only (part 1), then gate gradients only (part 2) == both in one pass."""
    W, k, n, S, M, H, LE = 2, 2, 4, 1024, 256, 512, 2
    shared = {}
    layers = [LB.MoELayer(S, M, H, k, 1.25, n, torch.bfloat16, DEV, LE, fabric=LB.LocalFabric(W, r, shared), seed=3) for r in range(W)]
    g = torch.Generator(device=DEV).manual_seed(77)
    xs = [torch.randn((S, M), device=DEV, generator=g).bfloat16() for _ in range(W)]
    gates = [torch.softmax(torch.randn((S, LE * W), device=DEV, generator=g), dim=1) for _ in range(W)]
    douts = [torch.randn((S, M), device=DEV, generator=g).bfloat16() for _ in range(W)]
    for r, l in enumerate(layers):
        l.fwd_dispatch(xs[r], gates[r])
    for l in layers:
        l.fwd_experts()
    for l in layers:
        l.fwd_combine()

    def poison():
        for l in layers:
            l.moe.d_expert_out.fill_(3.0)
            l.moe.dgates.fill_(-7.0)

    poison()
    for r, l in enumerate(layers):
        l.moe.combine_backward_send(douts[r])
    want = [(l.moe.d_expert_out.clone(), l.moe.dgates.clone()) for l in layers]
    poison()
    for r, l in enumerate(layers):
        l.moe.combine_backward_send(douts[r], part=1)
    for l, (deo, _) in zip(layers, want):
        assert torch.equal(l.moe.d_expert_out, deo) and bool((l.moe.dgates == -7.0).all())
    for l in layers:
        l.moe.d_expert_out.fill_(3.0)
    for r, l in enumerate(layers):
        l.moe.combine_backward_send(douts[r], part=2)
    for l, (_, dg) in zip(layers, want):
        assert torch.equal(l.moe.dgates, dg) and bool((l.moe.d_expert_out == 3.0).all())
    with pytest.raises(LB.LancetError):
        layers[0].moe.combine_backward_send(douts[0], part=3)


def _run_plain(layers, xs, gates, douts):
    for r, l in enumerate(layers):
        l.fwd_dispatch(xs[r], gates[r])
    for l in layers:
        l.fwd_experts()
    outs = [l.fwd_combine().clone() for l in layers]
    for r, l in enumerate(layers):
        l.bwd_combine(douts[r])
    for l in layers:
        l.bwd_experts()
    res = [tuple(t.clone() for t in l.bwd_dispatch()) for l in layers]
    grads = [[t.clone() for t in (l.dw1, l.dw2, l.db1, l.db2)] for l in layers]
    return outs, res, grads


def _run_staged(layers, xs, gates, douts, n):
    """The pipeline's units in an order a two-stream schedule can produce: exchange stage c+1 before expert stage c,
    chunk c combined after expert stage c+1."""
    for r, l in enumerate(layers):
        l.fwd_gate(xs[r], gates[r])
    for l in layers:
        l.fwd_stage_dispatch(0)
    for l in layers:
        l.fwd_prepare()
    for c in range(n):
        if c + 1 < n:
            for l in layers:
                l.fwd_stage_dispatch(c + 1)
        for l in layers:
            l.fwd_stage_experts(c)
        if c >= 1:
            for l in layers:
                l.fwd_stage_combine(c - 1)
    for l in layers:
        l.fwd_stage_combine(n - 1)
    outs = [l.moe.out.clone() for l in layers]
    for r, l in enumerate(layers):
        l.bwd_stage_combine(douts[r], 0)
    for l in layers:
        l.bwd_prepare()
    for c in range(n):
        if c + 1 < n:
            for r, l in enumerate(layers):
                l.bwd_stage_combine(douts[r], c + 1)
        for l in layers:
            l.bwd_stage_experts(c)
        if c >= 1:
            for l in layers:
                l.bwd_stage_dispatch(c - 1)
    for l in layers:
        l.bwd_stage_dispatch(n - 1)
        l.bwd_weights()
    res = [(l.moe.dx.clone(), l.moe.dgates.clone()) for l in layers]
    grads = [[t.clone() for t in (l.dw1, l.dw2, l.db1, l.db2)] for l in layers]
    return outs, res, grads


@pytest.mark.parametrize("W,k,n,S,stages", [(2, 2, 4, 2048, None), (1, 2, 4, 4096, 2), (2, 1, 2, 1024, None),
                                             (4, 2, 1, 512, None), (2, 2, 4, 1024, 1),
                                             (2, 2, 8, 512, None),       # 64 tokens per chunk: blocks grow by less than a tile per chunk
                                             (4, 1, 4, 256, 2)])
def test_staged_pipeline_is_bit_identical(W, k, n, S, stages):
    """The staged exchange + row-window GEMMs give exactly the results of the unpipelined layer."""
    M, H, LE, cf = 256, 512, 2, 1.25
    E = LE * W
    shared = {}
    layers = [LB.MoELayer(S, M, H, k, cf, n, torch.bfloat16, DEV, LE, fabric=LB.LocalFabric(W, r, shared), seed=9,
                          stages=stages) for r in range(W)]
    g = torch.Generator(device=DEV).manual_seed(W * 100 + k * 10 + n)
    xs = [torch.randn((S, M), device=DEV, generator=g).bfloat16() for _ in range(W)]
    gates = [torch.softmax(torch.randn((S, E), device=DEV, generator=g), dim=1) for _ in range(W)]
    douts = [torch.randn((S, M), device=DEV, generator=g).bfloat16() for _ in range(W)]
    ref = _run_plain(layers, xs, gates, douts)
    for l in layers:                      # stale results must not pass for fresh ones
        for t in (l.h, l.hpre if l.hpre is not None else l.h, l.dh, l.moe.out, l.moe.dx, l.moe.expert_out, l.moe.d_expert_in, l.dw1, l.dw2):
            t.fill_(float("nan"))
    got = _run_staged(layers, xs, gates, douts, len(layers[0].stage_chunks))
    torch.cuda.synchronize()
    for r in range(W):
        assert torch.equal(got[0][r], ref[0][r]), "out[%d]" % r
        assert torch.equal(got[1][r][0], ref[1][r][0]), "dx[%d]" % r
        assert torch.equal(got[1][r][1], ref[1][r][1]), "dgates[%d]" % r
        for a, b, name in zip(got[2][r], ref[2][r], ("dw1", "dw2", "db1", "db2")):
            assert torch.equal(a, b), "%s[%d]" % (name, r)
    # the windows equal the CPU restatement and cover the live rows of every block without gaps
    from oracle import moe_oracle as O
    for l in layers:
        ob, oe, oc = O.stage_windows(l.moe.chain[l.moe.parity].cpu().numpy(), l.moe.ROW_ALIGN)
        assert (l.win_begin.cpu().numpy() == ob).all() and (l.win_end.cpu().numpy() == oe).all()
        assert (l.cnt.cpu().numpy() == oc).all()
        lo, hi, cnt = l.win_begin.cpu().numpy(), l.win_end.cpu().numpy(), l.cnt.cpu().numpy()
        assert (lo[0] == 0).all() and (hi[-1] == cnt).all()
        A = l.moe.ROW_ALIGN
        assert (lo[1:] == hi[:-1] // A * A).all() and (lo % A == 0).all()
    assert int(LB.gemm_status(torch.device(DEV)).item()) == 0


def test_pipelined_two_stream_schedule_single_rank():
    """forward_pipelined / backward_pipelined (two streams, events) on one rank equal the plain path."""
    S, M, H, LE, k, n = 4096, 256, 512, 4, 2, 4
    layer = LB.MoELayer(S, M, H, k, 1.25, n, torch.bfloat16, DEV, LE, fabric=LB.LocalFabric(1, 0, {}), seed=3)
    g = torch.Generator(device=DEV).manual_seed(77)
    x = torch.randn((S, M), device=DEV, generator=g).bfloat16()
    gate = torch.softmax(torch.randn((S, LE), device=DEV, generator=g), dim=1)
    dout = torch.randn((S, M), device=DEV, generator=g).bfloat16()
    out0 = layer.forward(x, gate).clone()
    dx0, dg0 = [t.clone() for t in layer.backward(dout)]
    w0 = [t.clone() for t in (layer.dw1, layer.dw2, layer.db1, layer.db2)]
    for step in range(2):
        out1 = layer.forward_pipelined(x, gate).clone()
        dx1, dg1 = [t.clone() for t in layer.backward_pipelined(dout)]
    torch.cuda.synchronize()
    assert torch.equal(out0, out1) and torch.equal(dx0, dx1) and torch.equal(dg0, dg1)
    for a, b in zip(w0, (layer.dw1, layer.dw2, layer.db1, layer.db2)):
        assert torch.equal(a, b)
