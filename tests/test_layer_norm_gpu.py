"""lancet_layer_norm_fwd / _bwd against torch's float32 layer_norm on the same rows: output, input gradient and the weight /
bias gradients rel 1e-5 of the row scale (16-bit outputs: the float32 result rounded once); chunked calls give the bits of
the whole call."""
import pytest
import torch
import torch.nn.functional as F

import lancet_b200 as LB

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("R,M,out_dt,dy_dt", [
    (8192, 1024, torch.bfloat16, torch.bfloat16), (65536, 1024, torch.bfloat16, torch.bfloat16),   # 268 MB of rows: larger than L2
    (1000, 1024, torch.float32, torch.float32), (37, 128, torch.float32, torch.float32),
    (513, 768, torch.float16, torch.float16), (2048, 2048, torch.bfloat16, torch.float32), (5, 256, torch.float32, torch.bfloat16),
    (300, 1536, torch.bfloat16, torch.bfloat16), (64, 512, torch.float32, torch.float32),
])
def test_forward_and_backward_match_torch(R, M, out_dt, dy_dt):
    g = torch.Generator(device=DEV).manual_seed(R + M)
    x = torch.randn((R, M), device=DEV, generator=g) * 2 + 0.5
    w = torch.randn(M, device=DEV, generator=g) * 0.5 + 1
    b = torch.randn(M, device=DEV, generator=g) * 0.1
    dy = torch.randn((R, M), device=DEV, generator=g).to(dy_dt)
    y, mean, rstd = LB.layer_norm_fwd(x, w, b, 1e-5, out_dt)
    xr, wr, br = x.clone().requires_grad_(True), w.clone().requires_grad_(True), b.clone().requires_grad_(True)
    yr = F.layer_norm(xr, (M,), wr, br, 1e-5)
    if out_dt == torch.float32:
        torch.testing.assert_close(y, yr.detach(), rtol=1e-5, atol=1e-5)
    else:
        eps = 2.0 ** -8 if out_dt == torch.bfloat16 else 2.0 ** -11
        assert bool(((y.float() - yr.detach()).abs() <= yr.detach().abs() * eps + 1e-5).all())
    yr.backward(dy.float())
    dx, dw, db = LB.layer_norm_bwd(x, dy, w, mean, rstd)
    torch.testing.assert_close(dx, xr.grad, rtol=1e-4, atol=1e-5 * float(xr.grad.abs().max()))
    torch.testing.assert_close(dw, wr.grad, rtol=1e-4, atol=1e-5 * float(wr.grad.abs().max()))
    torch.testing.assert_close(db, br.grad, rtol=1e-4, atol=1e-5 * float(br.grad.abs().max()))


def test_chunked_rows_give_the_same_bits_and_results_are_reproducible():
    R, M = 4096, 1024
    g = torch.Generator(device=DEV).manual_seed(3)
    x = torch.randn((R, M), device=DEV, generator=g)
    w = torch.randn(M, device=DEV, generator=g)
    b = torch.randn(M, device=DEV, generator=g)
    dy = torch.randn((R, M), device=DEV, generator=g).bfloat16()
    y, mean, rstd = LB.layer_norm_fwd(x, w, b, 1e-5, torch.bfloat16)
    parts = [LB.layer_norm_fwd(x[i:i + 1024], w, b, 1e-5, torch.bfloat16) for i in range(0, R, 1024)]
    assert torch.equal(torch.cat([p[0] for p in parts]), y) and torch.equal(torch.cat([p[1] for p in parts]), mean)
    a = LB.layer_norm_bwd(x, dy, w, mean, rstd)
    c = LB.layer_norm_bwd(x, dy, w, mean, rstd)
    assert all(torch.equal(p, q) for p, q in zip(a, c))
    dx_parts = torch.cat([LB.layer_norm_bwd(x[i:i + 1024], dy[i:i + 1024], w, mean[i:i + 1024], rstd[i:i + 1024])[0]
                          for i in range(0, R, 1024)])
    assert torch.equal(dx_parts, a[0])


def test_module_under_autocast_and_bad_shapes():
    M = 256
    ln = LB.LayerNorm(M).to(DEV)
    ref = torch.nn.LayerNorm(M).to(DEV)
    with torch.no_grad():
        ln.weight.copy_(torch.randn(M, device=DEV) * 0.3 + 1)
        ln.bias.copy_(torch.randn(M, device=DEV) * 0.1)
        ref.weight.copy_(ln.weight)
        ref.bias.copy_(ln.bias)
    x = torch.randn((4, 33, M), device=DEV, requires_grad=True)
    xr = x.detach().clone().requires_grad_(True)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y = ln(x)
        lin = torch.nn.Linear(M, 8).to(DEV)
        out = lin(y)
        outr = lin(ref(xr))
    assert y.dtype == torch.bfloat16, "under autocast the normalised rows come out in the type the next GEMM reads"
    out.float().sum().backward()
    outr.float().sum().backward()
    torch.testing.assert_close(x.grad, xr.grad, rtol=2e-2, atol=2e-2 * float(xr.grad.abs().max()))
    torch.testing.assert_close(ln.weight.grad, ref.weight.grad, rtol=2e-2, atol=2e-2 * float(ref.weight.grad.abs().max()))
    y32 = ln(x.detach())
    assert y32.dtype == torch.float32
    torch.testing.assert_close(y32, ref(x.detach()), rtol=1e-5, atol=1e-5)
    with pytest.raises(LB.LancetError):
        LB.layer_norm_fwd(torch.randn((4, 100), device=DEV), torch.ones(100, device=DEV), torch.zeros(100, device=DEV), 1e-5,
                          torch.float32)
