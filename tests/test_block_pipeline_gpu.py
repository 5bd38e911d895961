"""The MoE block with its neighbouring operators inside the layer's chunk pipeline (layer norm and gate projection of
chunk c+1 under the exchange of chunk c, residual add under the remaining combines; the reference's forward partition
of non-MoE operators, src/pass/dist_optimization/partition_exprs.cc:1709-1795), and the deferred weight gradients of
dense layers (its dW scheduling, scheduler_utils.cc:517-640) against the unpipelined forms."""
import pytest
import torch
import torch.nn.functional as F

import lancet_b200 as LB
from lancet_b200.autograd import DeferredGrads, DeferredLinear

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("S,M,E,dt", [(1000, 256, 16, torch.bfloat16), (64, 72, 3, torch.float32), (513, 1024, 64, torch.float16)])
def test_gate_projection_matches_torch_and_ignores_chunking(S, M, E, dt):
    g = torch.Generator(device=DEV).manual_seed(S + E)
    h = torch.randn((S, M), device=DEV, generator=g).to(dt)
    wg = torch.randn((E, M), device=DEV, generator=g) * 0.1
    p = LB.gate_softmax(h, wg)
    ref = torch.softmax(h.double() @ wg.double().t(), dim=1)
    torch.testing.assert_close(p.double(), ref, rtol=1e-5, atol=1e-7)          # fp32 arithmetic: rel 1e-5
    # any split into calls gives the same bits (one warp per token, fixed order)
    cut = S // 3 + 1
    parts = torch.cat([LB.gate_softmax(h[:cut].contiguous(), wg), LB.gate_softmax(h[cut:].contiguous(), wg)])
    assert torch.equal(parts, p)
    # backward against autograd in float64
    dp = torch.randn((S, E), device=DEV, generator=g)
    dlogits, dh = LB.gate_softmax_bwd(p, dp, wg, dt)
    hd = h.double().requires_grad_(True)
    wd = wg.double()
    pr = torch.softmax(hd @ wd.t(), dim=1)
    (gh,) = torch.autograd.grad(pr, hd, dp.double())
    tol = 1e-5 if dt == torch.float32 else 1e-2
    torch.testing.assert_close(dh.double(), gh, rtol=tol, atol=tol * float(gh.abs().max()))
    logits = (h.double() @ wd.t()).requires_grad_(True)
    (gl,) = torch.autograd.grad(torch.softmax(logits, dim=1), logits, dp.double())
    torch.testing.assert_close(dlogits.double(), gl, rtol=1e-4, atol=1e-6)


def make_block(pipeline, stages=None, k=2, n_chunks=4, S=2048, M=256, H=512, seed=5):
    moe = LB.MoE(S, M, H, 2, k=k, capacity_factor=1.25, n_chunks=n_chunks, dtype=torch.bfloat16, device=DEV, local_experts=2,
                 fabric=LB.LocalFabric(1, 0, {}), seed=seed, pipeline=pipeline, stages=stages)
    torch.manual_seed(seed)
    ln = torch.nn.LayerNorm(M).to(DEV)
    with torch.no_grad():
        ln.weight.add_(0.1 * torch.randn_like(ln.weight))
        ln.bias.add_(0.1 * torch.randn_like(ln.bias))
        moe.wg.weight.copy_(torch.randn_like(moe.wg.weight) * 0.2)
    return moe, ln


@pytest.mark.parametrize("k,stages", [(2, 4), (2, 2), (1, 4)])
def test_chunked_block_equals_unchunked_block(k, stages):
    S, M = 2048, 256
    g = torch.Generator(device=DEV).manual_seed(11)
    x0 = torch.randn((4, S // 4, M), device=DEV, generator=g)
    dy = torch.randn((4, S // 4, M), device=DEV, generator=g)
    res = []
    for pipeline in (False, True):
        moe, ln = make_block(pipeline, stages=stages if pipeline else None, k=k)
        x = x0.clone().requires_grad_(True)
        for step in range(2):                     # twice: the receive buffers alternate
            for p in list(moe.parameters()) + list(ln.parameters()) + [x]:
                p.grad = None
            y = moe.block_forward(x, ln)
            y.backward(dy)
        torch.cuda.synchronize()
        moe.layer.moe.check()
        res.append((y.detach().clone(), x.grad.clone(), {n: p.grad.clone() for n, p in moe.named_parameters()},
                    {n: p.grad.clone() for n, p in ln.named_parameters()}, moe.layer.moe.idx_loc.clone()))
    (y0, dx0, gm0, gl0, il0), (y1, dx1, gm1, gl1, il1) = res
    assert torch.equal(il0, il1)                  # same routing
    assert torch.equal(y0, y1)                    # same bits in the block output ...
    assert torch.equal(dx0, dx1)                  # ... and in the input gradient (row-wise arithmetic in both)
    for n in ("w1", "b1", "w2", "b2"):
        assert torch.equal(gm0[n], gm1[n]), n     # expert gradients: the same kernels on the same tiles
    # sums over tokens are taken chunk by chunk in the pipeline: same value up to float32 summation order
    torch.testing.assert_close(gm0["wg.weight"], gm1["wg.weight"], rtol=1e-4, atol=1e-5 * float(gm0["wg.weight"].abs().max()))
    for n in gl0:
        torch.testing.assert_close(gl0[n], gl1[n], rtol=1e-4, atol=1e-5 * float(gl0[n].abs().max()))


def test_block_gradients_against_float32_torch():
    """The fused block against plain torch autograd on the same routing (float32 experts, same gate probabilities)."""
    S, M, H, E, k = 1024, 256, 512, 2, 2
    moe, ln = make_block(True, S=S, M=M, H=H, k=k)
    l = moe.layer.moe
    g = torch.Generator(device=DEV).manual_seed(2)
    x = torch.randn((S, M), device=DEV, generator=g).requires_grad_(True)
    dy = torch.randn((S, M), device=DEV, generator=g)
    y = moe.block_forward(x, ln)
    y.backward(dy)
    got = {"x": x.grad.clone(), "wg": moe.wg.weight.grad.clone(), "lnw": ln.weight.grad.clone(), "lnb": ln.bias.grad.clone(),
           "w1": moe.w1.grad.clone(), "w2": moe.w2.grad.clone()}
    for p in list(moe.parameters()) + list(ln.parameters()) + [x]:
        p.grad = None
    # reference: float32 torch with the library's routing decisions
    h = F.layer_norm(x, (M,), ln.weight, ln.bias, ln.eps)
    gate = torch.softmax(h @ moe.wg.weight.t(), dim=1)
    il = l.idx_loc.permute(1, 0, 2).reshape(2 * k, S)
    rows = torch.arange(S, device=DEV)
    kept = [il[2 * j] >= 0 for j in range(k)]
    raw = [torch.where(kept[j], gate[rows, il[2 * j].clamp(min=0).long()], torch.zeros((), device=DEV)) for j in range(k)]
    denom = sum(raw).clamp(min=torch.finfo(torch.float32).eps)
    out = torch.zeros_like(h)
    for j in range(k):
        for e in range(E):
            sel = ((il[2 * j] == e) & kept[j]).nonzero().flatten()
            if sel.numel():
                z = F.gelu(h[sel] @ moe.w1[e].t() + moe.b1[e])
                out = out.index_add(0, sel, (raw[j] / denom)[sel].unsqueeze(1) * (z @ moe.w2[e].t() + moe.b2[e]))
    yr = x + out
    torch.testing.assert_close(y.detach(), yr.detach(), rtol=3e-2, atol=3e-2)
    yr.backward(dy)
    ref = {"x": x.grad, "wg": moe.wg.weight.grad, "lnw": ln.weight.grad, "lnb": ln.bias.grad, "w1": moe.w1.grad, "w2": moe.w2.grad}
    for n in got:
        scale = float(ref[n].abs().max()) + 1e-8
        assert float((got[n] - ref[n]).abs().max()) <= 5e-2 * scale, n      # bf16 experts against float32 torch


def test_backward_needs_the_matching_forward():
    layer = LB.MoELayer(512, 256, 256, 2, 1.25, 2, torch.bfloat16, DEV, 2, fabric=LB.LocalFabric(1, 0, {}))
    x = torch.randn((512, 256), device=DEV).bfloat16()
    gate = torch.softmax(torch.randn((512, 2), device=DEV), dim=1)
    layer.forward(x, gate)
    with pytest.raises(RuntimeError):
        layer.backward_pipelined(x)          # row windows exist only after forward_pipelined
    layer.backward(x)
    with pytest.raises(RuntimeError):
        layer.backward(x)                    # the activations of that forward are consumed


def test_deferred_linear_matches_linear_under_autocast():
    torch.manual_seed(0)
    a = DeferredLinear(64, 48).to(DEV)
    b = torch.nn.Linear(64, 48).to(DEV)
    b.load_state_dict(a.state_dict())
    x = torch.randn((4, 32, 64), device=DEV)
    xa, xb = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        ya, yb = a(xa), b(xb)
    assert torch.equal(ya, yb)
    dy = torch.randn_like(ya)
    ya.backward(dy)
    yb.backward(dy)
    assert a.weight.grad is None                  # queued, not computed yet
    DeferredGrads.join(torch.device(DEV))
    torch.cuda.synchronize()
    torch.testing.assert_close(xa.grad, xb.grad, rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(a.weight.grad, b.weight.grad, rtol=2e-2, atol=2e-2 * float(b.weight.grad.abs().max()))
    torch.testing.assert_close(a.bias.grad, b.bias.grad, rtol=2e-2, atol=2e-2 * float(b.bias.grad.abs().max()))


def test_gpt_step_with_pipelined_blocks_matches_plain_blocks():
    """Two LANS steps of a small GPT-MoE with the chunk pipeline and deferred weight gradients against the same model
    without them: same routing, losses equal to bf16 accuracy."""
    from lancet_b200.gpt_moe import GPTMoE, LansTrainer
    vocab, m, nh, nl, seq, batch, ffn = 512, 256, 4, 2, 64, 8, 512
    losses = []
    for pipeline in (False, True):
        model = GPTMoE(vocab, m, nh, nl, seq, batch, ffn, 2, 2, 1.25, 4, DEV, fabric=LB.LocalFabric(1, 0, {}), seed=0,
                       act="relu", pipeline=pipeline)
        tr = LansTrainer(model, lr=1e-3)
        ids = torch.randint(0, vocab, (batch, seq), device=DEV, generator=torch.Generator(device=DEV).manual_seed(1))
        losses.append([float(tr.step(ids)) for _ in range(3)])
    for a, b in zip(*losses):
        assert abs(a - b) <= 2e-2 * abs(a), losses
    assert losses[1][-1] < losses[1][0]
