"""torch.autograd glue for the fused MoE layer: lets a torch model (the reference's GPT-2 / BERT MoE
builders wrap MOELayerImpl the same way, models/benchmark/pytorch/utils.py:576-634) train through the
library's forward and backward.  torch is the host framework here; every MoE kernel is the library's."""
import torch

from . import ops
from .layer import MoELayer


class _MoEFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gate, w1, b1, w2, b2, layer):
        # the working (16-bit) copies of the expert weights follow the master parameters
        layer.w1.copy_(w1)
        layer.b1.copy_(b1)
        layer.w2.copy_(w2)
        layer.b2.copy_(b2)
        ctx.layer = layer
        ctx.gate = gate
        ctx.in_dtype = x.dtype
        out = layer.forward(x.to(layer.moe.dtype).contiguous(), gate.float().contiguous())
        return out.to(x.dtype)

    @staticmethod
    def backward(ctx, dout):
        layer = ctx.layer
        moe = layer.moe
        dx, dgates_s = layer.backward(dout.to(moe.dtype).contiguous())
        gate = ctx.gate.float().contiguous()
        # gradient of the gate matrix from the gradient of the (k=2: normalised) gate values, chunk by chunk
        dgate = torch.empty_like(gate)
        Sp = moe.Sp
        for c in range(moe.n):
            sl = slice(c * Sp, (c + 1) * Sp)
            il = moe.idx_loc[c]
            dg = dgates_s[c] if moe.k == 2 else dgates_s[c, 0]
            dgate[sl] = ops.moe_encode_dg(dg.contiguous(), il, moe.E, gate=gate[sl] if moe.k == 2 else None)
        torch.cuda.current_stream().wait_stream(layer.side) if layer.side is not None else None
        return (dx.to(ctx.in_dtype), dgate.to(ctx.gate.dtype), layer.dw1.float(), layer.db1.float(), layer.dw2.float(),
                layer.db2.float(), None)


class MoE(torch.nn.Module):
    """Expert-parallel MoE block: gate (Linear + softmax, as the reference's Gate module,
    models/benchmark/pytorch/utils.py:565-573) + the fused layer.  Expert parameters are float32 masters of
    this rank's local experts; the layer computes in `dtype`."""

    def __init__(self, tokens, model_dim, hidden_dim, world_experts, k=2, capacity_factor=1.25, n_chunks=1,
                 dtype=torch.bfloat16, device="cuda", local_experts=2, fabric=None, group=None, seed=0, act="gelu"):
        super().__init__()
        self.layer = MoELayer(tokens, model_dim, hidden_dim, k, capacity_factor, n_chunks, dtype, device, local_experts,
                              fabric=fabric, group=group, seed=seed, act=act)
        assert self.layer.moe.E == world_experts
        self.wg = torch.nn.Linear(model_dim, world_experts, bias=False, device=device)
        self.w1 = torch.nn.Parameter(self.layer.w1.float().clone())
        self.b1 = torch.nn.Parameter(self.layer.b1.float().clone())
        self.w2 = torch.nn.Parameter(self.layer.w2.float().clone())
        self.b2 = torch.nn.Parameter(self.layer.b2.float().clone())

    def forward(self, x):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        gate = torch.softmax(self.wg(x2.float()), dim=1)
        out = _MoEFunction.apply(x2, gate, self.w1, self.b1, self.w2, self.b2, self.layer)
        return out.reshape(shape)
