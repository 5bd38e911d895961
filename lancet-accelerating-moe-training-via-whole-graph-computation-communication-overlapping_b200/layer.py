"""A trainable expert-parallel MoE layer on the fused kernels: gate -> dispatch (+exchange) -> expert FFN
(grouped tcgen05 GEMMs) -> combine (+exchange), and its backward with the weight-gradient GEMMs issued on
a side stream so that they run under the returning exchange (the reference's dW scheduling,
src/pass/dist_optimization/lancet_optimization.cc:1980-1998, as a fixed schedule).

Mirrors MOELayerImpl + Experts of the reference (models/benchmark/pytorch/utils.py:546-634) with the
gate probabilities as an input; the two nn.Linear layers of an expert keep their [out, in] layout."""
import torch

from . import _capi, ops
from .dist import DistChunkedMoE


class MoELayer:
    def __init__(self, S, M, H, k=2, capacity_factor=1.25, n_chunks=4, dtype=torch.bfloat16, device="cuda",
                 local_experts=2, fabric=None, group=None, act="gelu", seed=0, overlap_dw=True, stages=None,
                 exchange_ctas=0, gemm_ctas=0):
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
        # ReLU's derivative can be read off the activated output (h > 0 iff pre > 0): no pre-activation copy, which
        # saves a second [G, C, H] output of the first GEMM and its buffer
        self.hpre = None if act == "relu" else torch.empty((G, C, H), dtype=dtype, device=d)
        self.dh = torch.empty((G, C, H), dtype=dtype, device=d)
        self.dw1 = torch.empty_like(self.w1)
        self.dw2 = torch.empty_like(self.w2)
        self.db1 = torch.empty_like(self.b1)
        self.db2 = torch.empty_like(self.b2)
        self.side = torch.cuda.Stream(device=d) if overlap_dw else None
        self.G, self.C = G, C
        # pipeline stages of the staged schedule: consecutive chunks grouped into `stages` exchange steps
        P = n_chunks if stages is None else stages
        if P < 1 or n_chunks % P:
            raise ValueError("stages must divide n_chunks")
        self.stage_chunks = [(s * n_chunks // P, (s + 1) * n_chunks // P) for s in range(P)]
        # staged schedule only: grid caps of the exchange kernels and of the expert GEMMs while both are in flight
        # (0 = each asks for the whole GPU); see lancet_set_cta_limits
        self.exchange_ctas, self.gemm_ctas = int(exchange_ctas), int(gemm_ctas)
        # which schedule produced the activations a backward pass is about to read
        self._fwd_schedule = None

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
        self._fwd_schedule = "plain"
        return self.fwd_combine()

    def _limits(self, on):
        if self.exchange_ctas or self.gemm_ctas:
            _capi.check(_capi.lib().lancet_set_cta_limits(self.exchange_ctas if on else 0, self.gemm_ctas if on else 0))

    # ---- pipelined forward: the rows of chunk c+1 cross NVLink while the experts work on chunk c --------
    # Stage c of the expert GEMMs covers the whole 128-row tiles of every (source, expert) block that have arrived
    # with chunks 0..c, so no tile is computed twice and none is padded; the rows of chunk c are therefore complete
    # after stage c+1 (or the last stage), which is when its tokens are combined.  The stage methods below are the
    # units; `forward_pipelined` issues them on two streams.  Results are bit-identical to `forward`.
    def fwd_gate(self, x, gate):
        self._x = x
        self.moe.stage_gate(gate)

    def _window(self, c):
        return self._win[c]

    def fwd_stage_dispatch(self, c):
        self.moe.stage_dispatch(self._x, *self.stage_chunks[c])

    def _zero_tail_aside(self, buf=None):
        """The rows past each block's total are read by nothing in the layer (every GEMM is count-aware); they are zeroed
        for the buffer's contract, on a side stream, so that the first expert GEMM need not wait for it."""
        main = torch.cuda.current_stream(self.device)
        ev = main.record_event()
        with torch.cuda.stream(self.post_stream):
            self.post_stream.wait_event(ev)
            self.moe.zero_tail(buf)

    def fwd_prepare(self, zero=True):
        self.win_begin, self.win_end, self.cnt = self.moe.stage_prepare(zero=zero)
        self._win = [(self.win_begin[c0], self.win_end[c1 - 1]) for c0, c1 in self.stage_chunks]
        # (per-chunk windows: a stage of several chunks begins where its first chunk's window begins, which is at or
        # before the tile holding the previous stage's end, and ends where its last chunk's window ends)
        self.x_e = self.moe.recv[self.moe.parity].view(self.G, self.C, self.M)

    def fwd_stage_experts_1(self, c):
        lo, hi = self._window(c)
        ops.grouped_gemm_nt(self.x_e, self.w1, bias=self.b1, counts=hi, row_begin=lo, act=self.act, out=self.h,
                            preact=self.hpre)

    def fwd_stage_experts_2(self, c):
        lo, hi = self._window(c)
        ops.grouped_gemm_nt(self.h, self.w2, bias=self.b2, counts=hi, row_begin=lo,
                            out=self.moe.expert_out.view(self.G, self.C, self.M))

    def fwd_stage_experts(self, c):
        self.fwd_stage_experts_1(c)
        self.fwd_stage_experts_2(c)

    def fwd_stage_combine(self, c):
        return self.moe.stage_combine(*self.stage_chunks[c])

    def _streams(self):
        if getattr(self, "comm", None) is None:
            self.comm = torch.cuda.Stream(device=self.device)
            self.post_stream = torch.cuda.Stream(device=self.device)
        return torch.cuda.current_stream(self.device), self.comm

    def forward_pipelined(self, x, gate):
        """Two streams: `comm` carries the exchange stages and the flag barriers, the current stream the expert GEMMs,
        both in one fixed order on every rank.  (With the two GEMMs of a stage on two compute streams the persistent
        kernels race for the SMs, the ranks end up in different orders and every flag barrier then waits for the
        slowest: measured at 2 GPUs, up to 0.9 ms of barrier wait per step against 0.1 ms of idle last waves saved.)"""
        n = len(self.stage_chunks)
        main, comm = self._streams()
        self._limits(True)
        self.fwd_gate(x, gate)
        comm.wait_stream(main)
        arrived = []
        with torch.cuda.stream(comm):
            for c in range(n):
                self.fwd_stage_dispatch(c)
                self.moe.barrier()
                arrived.append(comm.record_event())
        main.wait_event(arrived[0])
        self.fwd_prepare(zero=False)
        self._zero_tail_aside()
        for c in range(n):
            main.wait_event(arrived[c])
            self.fwd_stage_experts_1(c)
            self.fwd_stage_experts_2(c)
            done = main.record_event()
            if c >= 1 or n == 1:
                with torch.cuda.stream(comm):
                    comm.wait_event(done)
                    self.moe.barrier()
                    if n > 1:
                        self.fwd_stage_combine(c - 1)
                    if c == n - 1:
                        self.fwd_stage_combine(c)
        main.wait_stream(comm)
        main.wait_stream(self.post_stream)
        self._limits(False)
        self._fwd_schedule = "staged"
        return self.moe.out

    # ---- pipelined forward with the neighbouring operators in the same chunk pipeline --------------------------
    def forward_chunked(self, pre, post=None):
        """The staged forward for callers that also split the operators in front of and behind the layer into the
        same token chunks (the reference's forward partition of non-MoE operators,
        src/pass/dist_optimization/partition_exprs.cc:1709-1795): the gate probabilities of stage s+1 need not exist
        when the rows of stage s start to travel.

        pre(c0, c1), called on the current stream stage by stage, returns (rows [tokens, M], gate [tokens, E] float32)
        of the tokens of chunks [c0, c1): whatever produces the layer's input (layer norm, gate projection) runs for
        stage s+1 while the rows of stage s cross NVLink.  post(c0, c1, out_rows), if given, is called on a side
        stream as soon as the combined output of those tokens is complete (residual add under the remaining
        exchange stages).  Gating is chained chunk by chunk and the owners learn each stage's row layout just before
        its rows arrive; results are bit-identical to `forward` on the concatenated inputs."""
        n = len(self.stage_chunks)
        main, comm = self._streams()
        moe, Sp = self.moe, self.moe.Sp
        if getattr(self, "x_in", None) is None:
            self.x_in = torch.empty((self.S, self.M), dtype=moe.dtype, device=self.device)
        self._limits(True)
        moe.begin_step()
        arrived = []
        for c0, c1 in self.stage_chunks:
            rows, gate = pre(c0, c1)
            dst = self.x_in[c0 * Sp:c1 * Sp]
            if rows.data_ptr() != dst.data_ptr():
                dst.copy_(rows)
            moe.stage_gate_chunks(gate, c0, c1)
            ready = main.record_event()
            with torch.cuda.stream(comm):
                comm.wait_event(ready)
                moe.stage_dispatch(self.x_in, c0, c1)
                moe.barrier()
                arrived.append(comm.record_event())
        self._x = self.x_in
        self.x_e = moe.recv[moe.parity].view(self.G, self.C, self.M)
        self.cnt = moe.counts[moe.parity]
        self._win = [None] * n
        for s in range(n):
            main.wait_event(arrived[s])
            self._win[s] = moe.stage_window(s, *self.stage_chunks[s], prev_c0=self.stage_chunks[s - 1][0] if s else -1)
            if s == n - 1:
                moe.zero_tail()          # the row totals are known with the last stage
            self.fwd_stage_experts_1(s)
            self.fwd_stage_experts_2(s)
            done = main.record_event()
            if s >= 1 or n == 1:
                with torch.cuda.stream(comm):
                    comm.wait_event(done)
                    moe.barrier()
                    for t in ([s - 1] if n > 1 else []) + ([s] if s == n - 1 else []):
                        rows = self.fwd_stage_combine(t)
                        if post is not None:
                            ev = comm.record_event()
                            with torch.cuda.stream(self.post_stream):
                                self.post_stream.wait_event(ev)
                                post(*self.stage_chunks[t], rows)
        main.wait_stream(comm)
        main.wait_stream(self.post_stream)
        self._limits(False)
        self._fwd_schedule = "staged"
        return moe.out

    # ---- pipelined backward ----
    def bwd_stage_combine(self, dout, c):
        self.moe.stage_combine_backward(dout, *self.stage_chunks[c])

    def bwd_prepare(self, zero=True):
        if zero:
            self.moe.stage_prepare(self.moe.d_expert_out)
        self.dy = self.moe.d_expert_out.view(self.G, self.C, self.M)

    def bwd_stage_experts_1(self, c):
        lo, hi = self._window(c)
        ops.grouped_gemm_nn(self.dy, self.w2, counts=hi, row_begin=lo, act=self.act, preact=self.h if self.hpre is None else self.hpre, out=self.dh)

    def bwd_stage_experts_2(self, c):
        lo, hi = self._window(c)
        ops.grouped_gemm_nn(self.dh, self.w1, counts=hi, row_begin=lo, out=self.moe.d_expert_in.view(self.G, self.C, self.M))

    def bwd_stage_experts(self, c):
        self.bwd_stage_experts_1(c)
        self.bwd_stage_experts_2(c)

    def bwd_weights(self):
        ops.grouped_gemm_tn(self.dy, self.h, self.LE, counts=self.cnt, out=self.dw2)
        ops.grouped_gemm_tn(self.dh, self.x_e, self.LE, counts=self.cnt, out=self.dw1)
        ops.grouped_bias_grad(self.dy, self.LE, counts=self.cnt, out=self.db2)
        ops.grouped_bias_grad(self.dh, self.LE, counts=self.cnt, out=self.db1)

    def bwd_stage_dispatch(self, c):
        return self.moe.stage_dispatch_backward(*self.stage_chunks[c])

    def backward_pipelined(self, dout, post=None):
        """post(c0, c1, dx_rows, dgates), if given, is called on a side stream as soon as the input gradient and the gate
        gradients of the tokens of chunks [c0, c1) are complete (backward of the operators in front of the layer, chunk
        by chunk, under the remaining exchange stages)."""
        if self._fwd_schedule != "staged":
            raise RuntimeError("backward_pipelined needs the row windows of forward_pipelined of the same step "
                               "(the last forward ran the %s schedule)" % self._fwd_schedule)
        n = len(self.stage_chunks)
        main, comm = self._streams()
        self._limits(True)
        comm.wait_stream(main)
        arrived = []
        with torch.cuda.stream(comm):
            for c in range(n):
                self.bwd_stage_combine(dout, c)
                self.moe.barrier()
                arrived.append(comm.record_event())
        main.wait_event(arrived[0])
        self.bwd_prepare(zero=False)
        self._zero_tail_aside(self.moe.d_expert_out)
        for c in range(n):
            main.wait_event(arrived[c])
            self.bwd_stage_experts_1(c)
            self.bwd_stage_experts_2(c)
            done = main.record_event()
            if c >= 1 or n == 1:
                with torch.cuda.stream(comm):
                    comm.wait_event(done)
                    self.moe.barrier()
                    for t in ([c - 1] if n > 1 else []) + ([c] if c == n - 1 else []):
                        rows = self.bwd_stage_dispatch(t)
                        if post is not None:
                            ev = comm.record_event()
                            c0, c1 = self.stage_chunks[t]
                            with torch.cuda.stream(self.post_stream):
                                self.post_stream.wait_event(ev)
                                post(c0, c1, rows, self.moe.dgates[c0:c1])
        # the weight gradients have no consumer before the optimizer: they run under the last gathers
        self.bwd_weights()
        main.wait_stream(comm)
        main.wait_stream(self.post_stream)
        self._limits(False)
        self._fwd_schedule = None
        return self.moe.dx, self.moe.dgates

    # ---- backward ----
    def bwd_combine(self, dout):
        # Both halves of the backward combine in one pass.  Sending the rows first and gathering the gate gradients on a
        # side stream beside the data-gradient GEMMs (lancet_moe_combine_bwd_part_p2p) shortens this step from 221 to
        # 114 us at 2 GPUs but slows the GEMMs it runs beside by more: 6.0 against 5.7 ms per forward+backward.
        self.moe.combine_backward_send(dout)

    def bwd_experts(self):
        d_eo, _ = self.moe.combine_backward_finish()
        dy = d_eo.view(self.G, self.C, self.M)
        main = torch.cuda.current_stream(self.device)
        # dH first: both the data path (dX) and dW1 need it
        ops.grouped_gemm_nn(dy, self.w2, counts=self.cnt, act=self.act, preact=self.h if self.hpre is None else self.hpre, out=self.dh)
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
        if self._fwd_schedule is None:
            raise RuntimeError("backward without a forward of the same step: the saved activations were consumed")
        self._fwd_schedule = None
        self.bwd_combine(dout)
        self.bwd_experts()
        return self.bwd_dispatch()
