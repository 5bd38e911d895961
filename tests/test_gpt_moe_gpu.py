"""A small GPT-style MoE training step (the shape of the reference's gpt2_moe benchmark model: every other
block MoE, top-2, capacity factor 1.25, LANS) through the library's layer and optimizer, against the same
model with a plain torch MoE block.  Reduced size; seeded uniform random token ids stand in for text."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

import lancet_b200 as LB
from oracle import lans_oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


class Block(torch.nn.Module):
    def __init__(self, m, nh, ffn):
        super().__init__()
        self.ln1, self.ln2 = torch.nn.LayerNorm(m), torch.nn.LayerNorm(m)
        self.attn = torch.nn.MultiheadAttention(m, nh, batch_first=True)
        self.ffn = ffn

    def forward(self, x):
        h = self.ln1(x)
        mask = torch.triu(torch.ones(x.shape[1], x.shape[1], dtype=torch.bool, device=x.device), 1)
        x = x + self.attn(h, h, h, attn_mask=mask, need_weights=False)[0]
        return x + self.ffn(self.ln2(x))


class TorchMoE(torch.nn.Module):
    """Reference MoE block in float32 torch that reuses the routing decided by the library layer."""

    def __init__(self, moe):
        super().__init__()
        self.moe = moe

    def forward(self, x):
        m = self.moe
        l = m.layer.moe
        shape = x.shape
        x2 = x.reshape(-1, shape[-1]).float()
        gate = torch.softmax(m.wg(x2), dim=1)
        out = torch.zeros_like(x2)
        S = x2.shape[0]
        rows = torch.arange(S, device=x.device)
        il = l.idx_loc.permute(1, 0, 2).reshape(2 * l.k, S)              # [2k, S] over all chunks
        kept = [il[2 * j] >= 0 for j in range(l.k)]
        raw = [torch.where(kept[j], gate[rows, il[2 * j].clamp(min=0).long()], torch.zeros((), device=x.device)) for j in range(l.k)]
        denom = sum(raw).clamp(min=torch.finfo(torch.float32).eps) if l.k == 2 else None
        for j in range(l.k):
            g = raw[j] / denom if l.k == 2 else raw[j]
            for e in range(l.E):
                sel = ((il[2 * j] == e) & kept[j]).nonzero().flatten()
                if sel.numel() == 0:
                    continue
                h = F.gelu(x2[sel] @ m.w1[e].t() + m.b1[e])
                out = out.index_add(0, sel, g[sel].unsqueeze(1) * (h @ m.w2[e].t() + m.b2[e]))
        return out.reshape(shape)


def build(vocab, m, nh, nl, moe_block, seq, batch):
    torch.manual_seed(0)
    emb = torch.nn.Embedding(vocab, m)
    pos = torch.nn.Embedding(seq, m)
    blocks = []
    for i in range(nl):
        if i % 2 == 1:
            blocks.append(Block(m, nh, moe_block))
        else:
            blocks.append(Block(m, nh, torch.nn.Sequential(torch.nn.Linear(m, 4 * m), torch.nn.GELU(), torch.nn.Linear(4 * m, m))))
    return torch.nn.ModuleDict(dict(emb=emb, pos=pos, blocks=torch.nn.ModuleList(blocks), ln=torch.nn.LayerNorm(m),
                                    head=torch.nn.Linear(m, vocab, bias=False))).to(DEV)


def run(model, ids):
    x = model["emb"](ids) + model["pos"](torch.arange(ids.shape[1], device=DEV))[None]
    for b in model["blocks"]:
        x = b(x)
    logits = model["head"](model["ln"](x))
    return F.cross_entropy(logits[:, :-1].reshape(-1, logits.shape[-1]), ids[:, 1:].reshape(-1))


def test_training_steps_match_torch_reference_and_loss_falls():
    vocab, m, nh, nl, seq, batch, H, E = 512, 256, 4, 2, 64, 8, 512, 2
    S = seq * batch
    moe = LB.MoE(S, m, H, E, k=2, capacity_factor=1.25, n_chunks=2, dtype=torch.bfloat16, device=DEV, local_experts=2,
                 fabric=LB.LocalFabric(1, 0, {}), seed=3)
    model = build(vocab, m, nh, nl, moe, seq, batch)
    ids = torch.randint(0, vocab, (batch, seq), device=DEV, generator=torch.Generator(device=DEV).manual_seed(1))
    # ---- one step: loss and gradients against the float32 torch MoE block with the same routing ----
    loss = run(model, ids)
    loss.backward()
    got = {n: p.grad.clone() for n, p in model.named_parameters()}
    model.zero_grad()
    ref_block = TorchMoE(moe)
    model["blocks"][1].ffn = ref_block
    loss_ref = run(model, ids)
    loss_ref.backward()
    assert abs(float(loss.detach()) - float(loss_ref.detach())) < 2e-2 * abs(float(loss_ref.detach()))
    for n, p in model.named_parameters():
        n_lib = n.replace("ffn.moe.", "ffn.")
        g, r = got[n_lib], p.grad
        scale = float(r.abs().max()) + 1e-8
        assert float((g - r).abs().max()) <= 5e-2 * scale + 1e-6, "%s: %g vs scale %g" % (n, float((g - r).abs().max()), scale)
    model["blocks"][1].ffn = moe
    model.zero_grad()
    # ---- a few LANS steps through the library optimizer: the loss must fall ----
    params = [p for p in model.parameters()]
    ms = [torch.zeros_like(p) for p in params]
    vs = [torch.zeros_like(p) for p in params]
    losses = []
    for step in range(1, 9):
        loss = run(model, ids)
        loss.backward()
        grads = [p.grad.contiguous() for p in params]
        if step == 1:
            # first step also checked against the NumPy oracle
            w = lans_oracle.lans_step([g.cpu().numpy() for g in grads], [p.detach().cpu().numpy() for p in params],
                                      [t.cpu().numpy() for t in ms], [t.cpu().numpy() for t in vs], step=1, lr=2e-3)
        with torch.no_grad():
            LB.lans(grads + [p.data for p in params] + ms + vs, step, learning_rate=2e-3)
        if step == 1:
            for p, wp in zip(params, w[0]):
                np.testing.assert_allclose(p.detach().cpu().numpy(), wp, rtol=1e-4, atol=1e-6)
        model.zero_grad()
        losses.append(float(loss.detach()))
    assert losses[-1] < losses[0] - 0.05, losses
