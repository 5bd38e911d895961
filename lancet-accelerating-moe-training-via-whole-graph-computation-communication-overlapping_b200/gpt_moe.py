"""GPT-2-style decoder with an expert-parallel MoE block in every other layer: the model family of the
reference's benchmark (gpt2_moe_nl12_m1024_nh16_sl512, models/benchmark/pytorch/nlp.py:303-316,
`moe_expert_interval=2`, `num_experts = 2 * world_size`, models/benchmark_raf.py:53).  Attention and the
embeddings are plain torch modules (outside the hot path this library implements); the MoE blocks run on the
library's fused layer, layer norm and the loss on its kernels, the optimizer step on its LANS op."""
import torch
import torch.nn.functional as F

from . import _capi
from .autograd import DeferredGrads, DeferredLinear, LayerNorm, MoE, softmax_cross_entropy
from .ops import LansState, gemm_status, lans


def _norm(m):
    """The library's layer norm where its kernels take the width (a multiple of 128 up to 2048), torch's otherwise."""
    return LayerNorm(m) if m in (128, 256, 512, 768, 1024, 1536, 2048) else torch.nn.LayerNorm(m)


class Attention(torch.nn.Module):
    def __init__(self, m, nh, linear=torch.nn.Linear):
        super().__init__()
        self.nh = nh
        self.qkv = linear(m, 3 * m)
        self.proj = linear(m, m)

    def forward(self, x):
        B, T, M = x.shape
        # split along the last axis (the same columns as a [3, heads, head_dim] view): the backward pass then writes the three
        # gradients straight into one [B, T, 3M] buffer instead of stacking them on a new leading axis and permuting a copy
        q, k, v = (t.view(B, T, self.nh, M // self.nh).transpose(1, 2) for t in self.qkv(x).split(M, dim=2))
        y = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        return self.proj(y.transpose(1, 2).reshape(B, T, M))


class Block(torch.nn.Module):
    def __init__(self, m, nh, ffn, linear=torch.nn.Linear, fused_moe=False):
        super().__init__()
        self.ln1, self.ln2 = _norm(m), _norm(m)
        self.attn = Attention(m, nh, linear)
        self.ffn = ffn
        self.fused_moe = fused_moe and isinstance(ffn, MoE)

    def forward(self, x):
        x = x + self.attn(self.ln1(x))
        if self.fused_moe:
            return self.ffn.block_forward(x, self.ln2)       # layer norm, gate and residual inside the chunk pipeline
        return x + self.ffn(self.ln2(x))


class GPTMoE(torch.nn.Module):
    def __init__(self, vocab, m, nh, nl, seq, batch, ffn_dim, world_experts, k=2, capacity_factor=1.25, n_chunks=4,
                 device="cuda", fabric=None, group=None, seed=0, act="gelu", pipeline=False):
        """act: activation of every FFN; the reference's GPT-2 uses ReLU (models/benchmark/pytorch/nlp.py:161-165),
        its BERT / ViT GELU (:137-141).  pipeline: the MoE blocks run layer norm, gate projection and residual add
        inside the layer's chunk pipeline, and the dense layers queue their weight gradients (DeferredLinear) so that
        they run under the next MoE layer's returning exchange; the trainer joins the queue before the optimizer."""
        super().__init__()
        linear = DeferredLinear if pipeline else torch.nn.Linear
        self.pipeline = bool(pipeline)
        torch.manual_seed(seed)
        # the tied output projection is a GEMM with the vocabulary as one extent: an odd size (50257) forces the library
        # onto an unaligned legacy kernel that costs a third of the step, so the table is padded to a multiple of 128
        # rows; the extra rows are never indexed and their logits are dropped before the loss
        self.vocab = vocab
        self.emb = torch.nn.Embedding((vocab + 127) // 128 * 128, m)
        self.pos = torch.nn.Embedding(seq, m)
        blocks = []
        for i in range(nl):
            if i % 2 == 1:
                ffn = MoE(seq * batch, m, ffn_dim, world_experts, k, capacity_factor, n_chunks, torch.bfloat16, device, 2,
                          fabric=fabric, group=group, seed=seed + i, act=act, pipeline=pipeline)
            else:
                ffn = torch.nn.Sequential(linear(m, ffn_dim), torch.nn.ReLU() if act == "relu" else torch.nn.GELU(),
                                          linear(ffn_dim, m))
            blocks.append(Block(m, nh, ffn, linear, fused_moe=pipeline))
        self.blocks = torch.nn.ModuleList(blocks)
        self.ln = _norm(m)
        torch.nn.init.normal_(self.emb.weight, std=0.02)
        torch.nn.init.normal_(self.pos.weight, std=0.01)
        self.to(device)

    def expert_parameters(self):
        out = []
        for b in self.blocks:
            if isinstance(b.ffn, MoE):
                out += [b.ffn.w1, b.ffn.b1, b.ffn.w2, b.ffn.b2]
        return out

    def forward(self, ids):
        x = self.emb(ids) + self.pos(torch.arange(ids.shape[1], device=ids.device))[None]
        with torch.autocast("cuda", dtype=torch.bfloat16):
            for b in self.blocks:
                x = b(x)
            logits = F.linear(self.ln(x), self.emb.weight)         # tied output embedding
        # next-token loss on the padded 16-bit logits themselves: position t is scored against token t+1, the last
        # position of every sequence is ignored, the padded vocabulary columns are never read
        target = torch.full_like(ids, -1)
        target[:, :-1] = ids[:, 1:]
        return softmax_cross_entropy(logits.view(-1, logits.shape[-1]), target.view(-1), self.vocab)

    def close(self):
        for b in self.blocks:
            if isinstance(b.ffn, MoE):
                b.ffn.layer.moe.close()


class LansTrainer:
    """One training step: forward, backward, gradient average of the replicated parameters across ranks
    (torch.distributed, outside this library's scope), LANS update through the library."""

    def __init__(self, model, lr=1e-3, group=None, overlap_dw=True):
        self.model = model
        self.overlap_dw = overlap_dw
        self.device = next(model.parameters()).device
        self.params = [p for p in model.parameters()]
        expert_ids = {id(p) for p in model.expert_parameters()}
        self.shared = [p for p in self.params if id(p) not in expert_ids]
        self.m = [torch.zeros_like(p) for p in self.params]
        self.v = [torch.zeros_like(p) for p in self.params]
        # Gradients are taken from autograd as it produces them (`.grad` is cleared before every backward pass, so nothing is
        # added into a preset buffer and no buffer has to be zeroed).  With several ranks the gradients of the replicated
        # parameters are gathered into one flat buffer by a multi-tensor copy, averaged with one all-reduce, and the optimizer
        # reads them from there; the experts' gradients are rank-local and are used where they are.
        self.lr = lr
        self.step_no = 0
        self.group = group
        self.world = torch.distributed.get_world_size(group) if torch.distributed.is_initialized() else 1
        self.flat_shared, self.shared_views = None, None
        if self.world > 1 and self.shared:
            sizes = [(p.numel() + 3) // 4 * 4 for p in self.shared]                 # keep every view 16-byte aligned
            self.flat_shared = torch.zeros(sum(sizes), dtype=torch.float32, device=self.device)
            self.shared_views, off = [], 0
            for p, n in zip(self.shared, sizes):
                self.shared_views.append(self.flat_shared[off:off + p.numel()].view_as(p))
                off += n
        self._shared_ids = {id(p): i for i, p in enumerate(self.shared)}

    def step(self, ids):
        self.step_no += 1
        for p in self.params:
            p.grad = None
        loss = self.model(ids)
        loss.backward()
        # weight gradients still queued (dense blocks after the last MoE layer of the backward pass) and those running on
        # the side stream must be complete before they are averaged and applied
        DeferredGrads.join(self.device if self.device.type == "cuda" else None)
        self.check_status()
        grads = [p.grad for p in self.params]
        if self.flat_shared is not None:
            torch._foreach_copy_(self.shared_views, [p.grad for p in self.shared])
            torch.distributed.all_reduce(self.flat_shared, op=torch.distributed.ReduceOp.AVG, group=self.group)
            grads = [self.shared_views[self._shared_ids[id(p)]] if id(p) in self._shared_ids else p.grad for p in self.params]
        with torch.no_grad():
            # the pointer table is rebuilt when the gradient tensors moved (a few kilobytes and one small launch)
            lans([g.contiguous() for g in grads] + [p.data for p in self.params] + self.m + self.v, self.step_no,
                 learning_rate=self.lr)
        return loss.detach()

    def check_status(self):
        """Bounded device-side waits (flag barriers between ranks, pipeline barriers of the expert GEMM) only record
        that they ran out and let the kernels go on: read the status words once per step, before the update, and raise
        LancetError(LANCET_ERR_TIMEOUT) instead of applying gradients computed from incomplete rows."""
        words = [b.ffn.layer.moe.status for b in self.model.blocks if isinstance(b.ffn, MoE)]
        if self.device.type == "cuda":
            words.append(gemm_status(self.device))
        if not words:
            return
        bad = torch.stack([w.reshape(-1)[0] for w in words]).cpu()      # one small copy; the step synchronises here anyway
        for i, v in enumerate(bad.tolist()):
            if v != 0:
                raise _capi.LancetError(_capi.ERR_TIMEOUT, "a bounded wait ran out during this step (status word %d = %d): "
                                        "a peer did not arrive; the optimizer step was skipped" % (i, v))
