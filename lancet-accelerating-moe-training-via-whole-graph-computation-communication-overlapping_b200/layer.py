"""A trainable expert-parallel MoE layer on the fused kernels: gate -> dispatch (+exchange) -> expert FFN
(grouped tcgen05 GEMMs) -> combine (+exchange), and its backward with the weight-gradient GEMMs issued on
a side stream so that they run under the returning exchange (the reference's dW scheduling,
src/pass/dist_optimization/lancet_optimization.cc:1980-1998, as a fixed schedule).

Mirrors MOELayerImpl + Experts of the reference (models/benchmark/pytorch/utils.py:546-634) with the
gate probabilities as an input; the two nn.Linear layers of an expert keep their [out, in] layout."""
import torch

from . import ops
from .dist import DistChunkedMoE


class MoELayer:
    def __init__(self, S, M, H, k=2, capacity_factor=1.25, n_chunks=4, dtype=torch.bfloat16, device="cuda",
                 local_experts=2, fabric=None, group=None, act="gelu", seed=0, overlap_dw=True):
        self.moe = DistChunkedMoE(S, M, k, capacity_factor, n_chunks, dtype, device, local_experts, fabric=fabric,
                                  group=group, train=True)
        self.S, self.M, self.H, self.LE, self.act = S, M, H, local_experts, act
        self.device = self.moe.device
        d, W, C = self.device, self.moe.W, self.moe.C
        g = torch.Generator(device=d).manual_seed(seed + 17 * self.moe.rank)
        self.w1 = (torch.randn((local_experts, H, M), device=d, generator=g) * 0.02).to(dtype)
        self.b1 = (torch.randn((local_experts, H), device=d, generator=g) * 0.02).to(dtype)
        self.w2 = (torch.randn((local_experts, M, H), device=d, generator=g) * 0.02).to(dtype)
        self.b2 = (torch.randn((local_experts, M), device=d, generator=g) * 0.02).to(dtype)
        G = W * local_experts
        self.h = torch.empty((G, C, H), dtype=dtype, device=d)
        self.hpre = torch.empty((G, C, H), dtype=dtype, device=d)
        self.dh = torch.empty((G, C, H), dtype=dtype, device=d)
        self.dw1 = torch.empty_like(self.w1)
        self.dw2 = torch.empty_like(self.w2)
        self.db1 = torch.empty_like(self.b1)
        self.db2 = torch.empty_like(self.b2)
        self.side = torch.cuda.Stream(device=d) if overlap_dw else None
        self.G, self.C = G, C

    # ---- forward, in the three phases between which the ranks meet ----
    def fwd_dispatch(self, x, gate):
        self.moe.dispatch_send(x, gate)

    def fwd_experts(self):
        recv = self.moe.dispatch_finish()
        self.x_e = recv.view(self.G, self.C, self.M)
        self.cnt = self.moe.counts[self.moe.parity]
        ops.grouped_gemm_nt(self.x_e, self.w1, bias=self.b1, counts=self.cnt, act=self.act, out=self.h, preact=self.hpre)
        ops.grouped_gemm_nt(self.h, self.w2, bias=self.b2, counts=self.cnt,
                            out=self.moe.expert_out.view(self.G, self.C, self.M))

    def fwd_combine(self):
        return self.moe.combine(from_expert_out=True)

    def forward(self, x, gate):
        self.fwd_dispatch(x, gate)
        self.fwd_experts()
        return self.fwd_combine()

    # ---- backward ----
    def bwd_combine(self, dout):
        self.moe.combine_backward_send(dout)

    def bwd_experts(self):
        d_eo, _ = self.moe.combine_backward_finish()
        dy = d_eo.view(self.G, self.C, self.M)
        main = torch.cuda.current_stream(self.device)
        # dH first: both the data path (dX) and dW1 need it
        ops.grouped_gemm_nn(dy, self.w2, counts=self.cnt, act=self.act, preact=self.hpre, out=self.dh)
        if self.side is not None:
            self.side.wait_stream(main)
        ops.grouped_gemm_nn(self.dh, self.w1, counts=self.cnt, out=self.moe.d_expert_in.view(self.G, self.C, self.M))
        # weight gradients have no consumer before the optimizer: they go to the side stream and run while the
        # main stream gathers dX over NVLink
        with torch.cuda.stream(self.side if self.side is not None else main):
            ops.grouped_gemm_tn(dy, self.h, self.LE, counts=self.cnt, out=self.dw2)
            ops.grouped_gemm_tn(self.dh, self.x_e, self.LE, counts=self.cnt, out=self.dw1)
            ops.grouped_bias_grad(dy, self.LE, counts=self.cnt, out=self.db2)
            ops.grouped_bias_grad(self.dh, self.LE, counts=self.cnt, out=self.db1)

    def bwd_dispatch(self):
        dx = self.moe.dispatch_backward()
        if self.side is not None:
            torch.cuda.current_stream(self.device).wait_stream(self.side)
        return dx, self.moe.dgates

    def backward(self, dout):
        self.bwd_combine(dout)
        self.bwd_experts()
        return self.bwd_dispatch()
