"""torch.autograd glue for the fused MoE layer: lets a torch model (the reference's GPT-2 / BERT MoE
builders wrap MOELayerImpl the same way, models/benchmark/pytorch/utils.py:576-634) train through the
library's forward and backward.  torch is the host framework here; every MoE kernel is the library's."""
import torch
import torch.nn.functional as F

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


class DeferredGrads:
    """Weight-gradient work that has no consumer before the optimizer, collected during backward and run later on a side
    stream: the static counterpart of the reference's dW scheduling, which labels every backward operator without a
    path to an all-to-all as a candidate and packs the candidates under the all-to-all windows
    (src/pass/dist_optimization/scheduler_utils.cc:382-480, :517-640; lancet_optimization.cc:1980-1998).  Dense layers
    queue their dW here; the MoE block's backward runs the queue when its returning exchange starts."""
    queue = []
    stream = None

    @classmethod
    def push(cls, fn, *tensors):
        cls.queue.append((fn, tensors))

    @classmethod
    def run(cls, device=None):
        """Enqueue everything collected so far on the side stream (after the work already issued on the current one)."""
        if not cls.queue:
            return
        if device is None or not torch.cuda.is_available():
            for fn, _ in cls.queue:
                fn()
            cls.queue = []
            return
        if cls.stream is None:
            cls.stream = torch.cuda.Stream(device=device)
        cls.stream.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(cls.stream):
            for fn, tensors in cls.queue:
                for t in tensors:
                    t.record_stream(cls.stream)
                fn()
        cls.queue = []

    @classmethod
    def join(cls, device=None):
        """Run what is still queued and make the current stream wait for all of it (call before the optimizer)."""
        cls.run(device)
        if cls.stream is not None and device is not None:
            torch.cuda.current_stream(device).wait_stream(cls.stream)


class _DeferredLinearFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, owner):
        cdt = torch.get_autocast_dtype("cuda") if (x.is_cuda and torch.is_autocast_enabled()) else x.dtype
        xc, wc = x.to(cdt), weight.to(cdt)
        ctx.save_for_backward(xc, wc)
        ctx.owner = owner
        # every operand already has the compute type, so an enclosing autocast region changes nothing here
        return F.linear(xc, wc, None if bias is None else bias.to(cdt))

    @staticmethod
    def backward(ctx, dy):
        xc, wc = ctx.saved_tensors
        owner = ctx.owner
        dy = dy.contiguous()
        dx = dy.to(wc.dtype) @ wc          # (backward passes run outside autocast regions)
        x2, dy2 = xc.reshape(-1, xc.shape[-1]), dy.reshape(-1, dy.shape[-1]).to(xc.dtype)

        def weight_grads():
            with torch.no_grad():
                dw = dy2.t() @ x2
                owner.weight.grad = dw.to(owner.weight.dtype) if owner.weight.grad is None else owner.weight.grad.add_(dw)
                if owner.bias is not None:
                    db = dy2.sum(dim=0, dtype=torch.float32)
                    owner.bias.grad = db.to(owner.bias.dtype) if owner.bias.grad is None else owner.bias.grad.add_(db)

        DeferredGrads.push(weight_grads, x2, dy2)
        return dx.to(dy.dtype), None, None, None


class DeferredLinear(torch.nn.Linear):
    """nn.Linear whose backward returns the input gradient at once and queues the weight and bias gradients on
    DeferredGrads (they are accumulated into `.grad` when the queue runs)."""

    def forward(self, x):
        if not torch.is_grad_enabled():
            return F.linear(x, self.weight, self.bias)
        return _DeferredLinearFunction.apply(x, self.weight, self.bias, self)


class _MoEBlockFunction(torch.autograd.Function):
    """y = x + MoE(LayerNorm(x)) with the layer norm, the gate projection and the residual add inside the layer's
    chunk pipeline: the rows of token chunk c cross NVLink while chunk c+1 is normalised and gated, and the residual of
    chunk c is added under the remaining combines (backward: gate and layer-norm gradients of chunk c under the remaining
    gathers).  With pipeline off the same arithmetic runs unchunked; both give the same bits in y and dx."""

    @staticmethod
    def forward(ctx, x, ln_w, ln_b, wg, w1, b1, w2, b2, blk):
        layer, eps = blk.layer, blk.ln_eps
        moe = layer.moe
        Sp, M, dt = moe.Sp, moe.M, moe.dtype
        layer.w1.copy_(w1)
        layer.b1.copy_(b1)
        layer.w2.copy_(w2)
        layer.b2.copy_(b2)
        x = x.contiguous()
        y = torch.empty_like(x)
        probs = torch.empty((moe.S, moe.E), dtype=torch.float32, device=x.device)
        if getattr(layer, "x_in", None) is None:
            layer.x_in = torch.empty((moe.S, M), dtype=dt, device=x.device)
        lw, lb, wgf = ln_w.detach().float(), ln_b.detach().float(), wg.detach().float().contiguous()
        # float32 rows of a width the library's layer norm takes: its kernels write the normalised rows straight into the
        # layer's input buffer and keep mean and 1/std per row for the backward pass; otherwise torch's layer norm
        native_ln = x.dtype == torch.float32 and M in ops.LAYER_NORM_WIDTHS
        mean = torch.empty((moe.S,), dtype=torch.float32, device=x.device) if native_ln else None
        rstd = torch.empty((moe.S,), dtype=torch.float32, device=x.device) if native_ln else None

        def pre(c0, c1):
            sl = slice(c0 * Sp, c1 * Sp)
            if native_ln:
                ops.layer_norm_fwd(x[sl], lw, lb, eps, out=layer.x_in[sl], mean=mean[sl], rstd=rstd[sl])
            else:
                layer.x_in[sl] = F.layer_norm(x[sl].float(), (M,), lw, lb, eps)     # float32 under autocast as well
            ops.gate_softmax(layer.x_in[sl], wgf, out=probs[sl])
            return layer.x_in[sl], probs[sl]

        def post(c0, c1, rows):
            sl = slice(c0 * Sp, c1 * Sp)
            torch.add(x[sl], rows, out=y[sl])

        if blk.pipeline:
            layer.forward_chunked(pre, post)
        else:
            h, g = pre(0, moe.n)
            post(0, moe.n, layer.forward(h, g))
        ctx.save_for_backward(x, ln_w, ln_b, wg, probs)
        ctx.blk, ctx.ln_stats = blk, (mean, rstd)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, ln_w, ln_b, wg, probs = ctx.saved_tensors
        blk = ctx.blk
        layer, eps = blk.layer, blk.ln_eps
        moe = layer.moe
        Sp, M, dt, E, k = moe.Sp, moe.M, moe.dtype, moe.E, moe.k
        # weight gradients of the dense blocks whose backward has already run have no consumer before the optimizer:
        # they go to the side stream now and run under this layer's returning exchange
        DeferredGrads.run(x.device)
        dy = dy.contiguous()
        dx = torch.empty_like(x)
        wgf = wg.detach().float().contiguous()
        lwf = ln_w.detach().float().contiguous()
        mean, rstd = ctx.ln_stats
        acc = {"lw": torch.zeros_like(ln_w, dtype=torch.float32), "lb": torch.zeros_like(ln_b, dtype=torch.float32),
               "wg": torch.zeros_like(wgf)}

        def post(c0, c1, dx_rows, dgates):
            sl = slice(c0 * Sp, c1 * Sp)
            p = probs[sl]
            dprobs = torch.empty_like(p)
            for c in range(c0, c1):
                cs = slice((c - c0) * Sp, (c - c0 + 1) * Sp)
                dg = dgates[c - c0] if k == 2 else dgates[c - c0, 0]
                dprobs[cs] = ops.moe_encode_dg(dg.contiguous(), moe.idx_loc[c], E, gate=p[cs].contiguous() if k == 2 else None)
            dlogits, dh_gate = ops.gate_softmax_bwd(p.contiguous(), dprobs, wgf, dt)
            # float32 arithmetic: backward passes run outside autocast regions
            acc["wg"].addmm_(dlogits.t(), layer.x_in[sl].float())
            dh = dx_rows.float() + dh_gate.float()
            if mean is not None:
                gx, gw, gb = ops.layer_norm_bwd(x[sl], dh, lwf, mean[sl], rstd[sl])
            else:
                xs = x[sl].detach().float().requires_grad_(True)
                lw = ln_w.detach().float().requires_grad_(True)
                lb = ln_b.detach().float().requires_grad_(True)
                with torch.enable_grad():
                    hh = F.layer_norm(xs, (M,), lw, lb, eps)
                gx, gw, gb = torch.autograd.grad(hh, [xs, lw, lb], dh)
            dx[sl] = dy[sl].float() + gx
            acc["lw"] += gw
            acc["lb"] += gb

        dyl = dy.to(dt).contiguous()
        if blk.pipeline:
            layer.backward_pipelined(dyl, post=post)
        else:
            dxh, dg = layer.backward(dyl)
            post(0, moe.n, dxh, dg)
            if layer.side is not None:
                torch.cuda.current_stream().wait_stream(layer.side)
        return (dx, acc["lw"].to(ln_w.dtype), acc["lb"].to(ln_b.dtype), acc["wg"].to(wg.dtype), layer.dw1.float(),
                layer.db1.float(), layer.dw2.float(), layer.db2.float(), None)


class MoE(torch.nn.Module):
    """Expert-parallel MoE block: gate (Linear + softmax, as the reference's Gate module,
    models/benchmark/pytorch/utils.py:565-573) + the fused layer.  Expert parameters are float32 masters of
    this rank's local experts; the layer computes in `dtype`."""

    def __init__(self, tokens, model_dim, hidden_dim, world_experts, k=2, capacity_factor=1.25, n_chunks=1,
                 dtype=torch.bfloat16, device="cuda", local_experts=2, fabric=None, group=None, seed=0, act="gelu",
                 pipeline=False, stages=None):
        """pipeline: `block_forward` runs the layer norm, the gate projection and the residual add inside the layer's
        chunk pipeline (see _MoEBlockFunction); `forward` is unaffected."""
        super().__init__()
        self.layer = MoELayer(tokens, model_dim, hidden_dim, k, capacity_factor, n_chunks, dtype, device, local_experts,
                              fabric=fabric, group=group, seed=seed, act=act, stages=stages)
        self.pipeline = bool(pipeline)
        self.ln_eps = 1e-5
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

    def block_forward(self, x, ln):
        """x + MoE(ln(x)) for a transformer block's second half; `ln` is the block's LayerNorm module.  The gate
        projection runs through `gate_softmax` (float32 accumulation, per-token order) in both modes."""
        shape = x.shape
        self.ln_eps = ln.eps
        y = _MoEBlockFunction.apply(x.reshape(-1, shape[-1]), ln.weight, ln.bias, self.wg.weight, self.w1, self.b1, self.w2,
                                    self.b2, self)
        return y.reshape(shape)


class _SoftmaxCrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, target, vocab):
        loss_rows, lse = ops.softmax_xent_fwd(logits, target, vocab)
        live = (target >= 0).sum()
        ctx.save_for_backward(logits, target, lse, live)
        ctx.vocab = vocab
        return loss_rows.sum() / live.clamp(min=1)

    @staticmethod
    def backward(ctx, gout):
        logits, target, lse, live = ctx.saved_tensors
        # the mean's 1/live factor stays on the device with the upstream gradient: no host round trip
        g = (gout.float() / live.clamp(min=1)).reshape(1).contiguous()
        return ops.softmax_xent_bwd(logits, target, ctx.vocab, lse, g, 1.0), None, None


def softmax_cross_entropy(logits, target, vocab=None):
    """Mean cross-entropy of `logits` [rows, cols] (float32, float16 or bfloat16; columns from `vocab` on are padding) against
    `target` [rows] int64 (negative = ignored), computed by the library's two kernels on the 16-bit logits themselves: the
    language-model head of the reference's benchmark models (log_softmax + nll_loss, models/benchmark/raf/raf_bencher.py:84)
    without float32 copies of the [tokens, vocabulary] matrix."""
    return _SoftmaxCrossEntropy.apply(logits, target, logits.shape[1] if vocab is None else vocab)


class _LayerNormFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps, out_dtype):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1]).float()
        y, mean, rstd = ops.layer_norm_fwd(x2, weight.float(), bias.float(), eps, out_dtype)
        ctx.save_for_backward(x2, weight, mean, rstd)
        ctx.shape, ctx.in_dtype = shape, x.dtype
        return y.view(shape)

    @staticmethod
    def backward(ctx, dy):
        x2, weight, mean, rstd = ctx.saved_tensors
        dx, dw, db = ops.layer_norm_bwd(x2, dy.reshape(x2.shape), weight.float(), mean, rstd)
        return dx.view(ctx.shape).to(ctx.in_dtype), dw.to(weight.dtype), db.to(weight.dtype), None, None


class LayerNorm(torch.nn.Module):
    """Layer normalisation over the last axis on the library's kernels (parameters named as torch.nn.LayerNorm's).  Under
    CUDA autocast the normalised rows come out in the autocast type, which is what the following GEMM reads: the separate
    float32 -> 16-bit pass disappears, and the backward pass takes the 16-bit gradient as it is."""

    def __init__(self, normalized_shape, eps=1e-5):
        super().__init__()
        self.weight = torch.nn.Parameter(torch.ones(normalized_shape))
        self.bias = torch.nn.Parameter(torch.zeros(normalized_shape))
        self.eps = eps

    def forward(self, x):
        out = torch.get_autocast_dtype("cuda") if torch.is_autocast_enabled("cuda") else torch.float32
        return _LayerNormFunction.apply(x, self.weight, self.bias, self.eps, out)

