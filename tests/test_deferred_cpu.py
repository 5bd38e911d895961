"""Deferred weight gradients of dense layers (the static form of the reference's dW scheduling,
src/pass/dist_optimization/scheduler_utils.cc:517-640: weight-gradient operators have no consumer before the
optimizer and are moved under communication windows): host logic on CPU."""
import torch

import lancet_b200  # noqa: F401
from lancet_b200.autograd import DeferredGrads, DeferredLinear


def test_deferred_linear_queues_weight_gradients_until_the_queue_runs():
    torch.manual_seed(0)
    a, b = DeferredLinear(8, 5), torch.nn.Linear(8, 5)
    b.load_state_dict(a.state_dict())
    x = torch.randn(3, 4, 8, requires_grad=True)
    x2 = x.detach().clone().requires_grad_()
    DeferredGrads.queue.clear()
    a(x).square().sum().backward()
    b(x2).square().sum().backward()
    assert a.weight.grad is None and a.bias.grad is None and len(DeferredGrads.queue) == 1
    torch.testing.assert_close(x.grad, x2.grad)                 # the input gradient is returned at once
    DeferredGrads.join(None)
    assert not DeferredGrads.queue
    torch.testing.assert_close(a.weight.grad, b.weight.grad)
    torch.testing.assert_close(a.bias.grad, b.bias.grad)


def test_deferred_gradients_accumulate_into_existing_buffers_in_order():
    torch.manual_seed(1)
    lin = DeferredLinear(6, 6, bias=False)
    ref = torch.nn.Linear(6, 6, bias=False)
    ref.load_state_dict(lin.state_dict())
    lin.weight.grad = torch.zeros_like(lin.weight)
    buf = lin.weight.grad
    DeferredGrads.queue.clear()
    for _ in range(3):                                           # e.g. three micro-batches before one optimizer step
        x = torch.randn(5, 6)
        lin(lin(x)).sum().backward()                            # the layer used twice in one graph: two queued entries
        ref(ref(x)).sum().backward()
    assert len(DeferredGrads.queue) == 6
    DeferredGrads.run(None)
    assert lin.weight.grad is buf                                # accumulated in place (a trainer may pre-allocate it)
    torch.testing.assert_close(lin.weight.grad, ref.weight.grad)


def test_no_grad_path_is_a_plain_linear():
    lin = DeferredLinear(4, 3)
    with torch.no_grad():
        y = lin(torch.ones(2, 4))
    assert y.shape == (2, 3) and not DeferredGrads.queue
