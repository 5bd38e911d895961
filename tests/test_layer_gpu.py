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


@pytest.mark.parametrize("W,k,n", [(1, 2, 4), (2, 2, 2), (2, 1, 1)])
def test_layer_forward_backward(W, k, n):
    S, M, H, LE, cf = 512, 256, 512, 2, 1.25
    E = LE * W
    shared = {}
    layers = [LB.MoELayer(S, M, H, k, cf, n, torch.bfloat16, DEV, LE, fabric=LB.LocalFabric(W, r, shared), seed=5)
              for r in range(W)]
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
                    y = torch.nn.functional.gelu(hpre) @ w2[own][le].t() + b2[own][le]
                    out = out.index_add(0, tok, gs[r][c, j, sel].unsqueeze(1) * y)
        ref_out.append(out)
        loss = loss + (out * douts[r].float()).sum()
    loss.backward()
    for r, l in enumerate(layers):
        close(outs[r], ref_out[r].detach(), "out[%d]" % r)
        dx, dgates = res[r]
        close(dx, xr[r].grad, "dx[%d]" % r)
        close(dgates, gs[r].grad, "dgates[%d]" % r)
        close(l.dw1, w1[r].grad, "dw1[%d]" % r)
        close(l.dw2, w2[r].grad, "dw2[%d]" % r)
        close(l.db1, b1[r].grad, "db1[%d]" % r)
        close(l.db2, b2[r].grad, "db2[%d]" % r)
    st = LB.gemm_status(torch.device(DEV))
    assert int(st.item()) == 0
