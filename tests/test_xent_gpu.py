"""Softmax cross-entropy over a padded vocabulary (lancet_softmax_xent_fwd / _bwd) against torch's float32
log_softmax + nll_loss on the same logits: loss rel 1e-5; gradients rel 1e-5 for float32 logits, and for 16-bit logits
within half a unit in the last place of the 16-bit result plus rel 1e-3 (the gradient is rounded once to the logits' type)."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

import lancet_b200 as LB

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("rows,vocab,cols,dt", [
    (64, 1000, 1024, torch.bfloat16), (33, 50257, 50304, torch.bfloat16),
    (2048, 50257, 50304, torch.bfloat16),                  # 206 MB of logits: larger than L2 (the case the profile captures) (17, 777, 777, torch.float32),
    (40, 4099, 4104, torch.float16), (8, 5, 8, torch.float32), (12, 1001, 1001, torch.bfloat16),   # odd stride: scalar path
])
def test_loss_and_gradient_match_torch(rows, vocab, cols, dt):
    g = torch.Generator(device=DEV).manual_seed(rows + vocab)
    logits = (torch.randn((rows, cols), device=DEV, generator=g) * 3).to(dt).requires_grad_(True)
    target = torch.randint(0, vocab, (rows,), device=DEV, generator=g)
    target[::5] = -1                                     # ignored rows
    up = torch.tensor(0.37, device=DEV)                   # an upstream factor, as a loss scaler would apply
    loss = LB.softmax_cross_entropy(logits, target, vocab)
    (loss * up).backward()
    ref_in = logits.detach().float()[:, :vocab].requires_grad_(True)
    ref = F.nll_loss(F.log_softmax(ref_in, dim=1), target, ignore_index=-1)
    (ref * up).backward()
    torch.testing.assert_close(loss, ref, rtol=1e-5, atol=1e-6)
    got = logits.grad.float()
    assert bool((got[:, vocab:] == 0).all()), "padded columns carry no gradient"
    assert bool((got[target < 0] == 0).all()), "ignored rows carry no gradient"
    want = ref_in.grad
    if dt == torch.float32:
        torch.testing.assert_close(got[:, :vocab], want, rtol=1e-5, atol=1e-9)
    else:
        eps = 2.0 ** -8 if dt == torch.bfloat16 else 2.0 ** -11
        floor = 1e-12 if dt == torch.bfloat16 else 2.0 ** -24      # float16 gradients this small are subnormal: fixed spacing
        err = (got[:, :vocab] - want).abs()
        assert bool((err <= want.abs() * (eps + 1e-3) + floor).all())


def test_all_rows_ignored_and_bad_arguments():
    logits = torch.randn((4, 16), device=DEV).bfloat16().requires_grad_(True)
    target = torch.full((4,), -1, device=DEV, dtype=torch.int64)
    loss = LB.softmax_cross_entropy(logits, target, 10)
    loss.backward()
    assert float(loss.detach()) == 0.0 and bool((logits.grad == 0).all())
    with pytest.raises(LB.LancetError):
        LB.softmax_xent_fwd(torch.randn((4, 16), device=DEV), target, 17)     # vocabulary wider than the rows
    with pytest.raises(TypeError):
        LB.softmax_xent_fwd(torch.randn((4, 16), device=DEV), target.int(), 10)


def test_gpt_loss_equals_the_unfused_form():
    """The model's loss line: next-token targets with the last position ignored, on padded 16-bit logits."""
    B, T, V, Vp = 3, 9, 50, 128
    g = torch.Generator(device=DEV).manual_seed(1)
    logits = torch.randn((B, T, Vp), device=DEV, generator=g).bfloat16()
    ids = torch.randint(0, V, (B, T), device=DEV, generator=g)
    target = torch.full_like(ids, -1)
    target[:, :-1] = ids[:, 1:]
    got = LB.softmax_cross_entropy(logits.view(-1, Vp), target.view(-1), V)
    want = F.cross_entropy(logits[:, :-1, :V].float().reshape(-1, V), ids[:, 1:].reshape(-1))
    torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-6)
