"""A small Llama-style decoder (RMSNorm, causal SDPA attention with rotary embedding, SwiGLU) whose
block linears are `QuantizedLinear`s taken from a quantization package passed in -- the shape of the
reference's model (src/models/llama.py: c_attn / c_proj / w12 / c_proj per block, un-quantized
lm_head), written independently as a test harness."""
import math

import torch
import torch.nn as nn
import torch.nn.functional as F


class RMSNorm(nn.Module):
    def __init__(self, dim, eps=1e-6):
        super().__init__()
        self.eps, self.weight = eps, nn.Parameter(torch.ones(dim))

    def forward(self, x):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)).type_as(x) * self.weight


def rotary(q, k):
    b, h, t, d = q.shape
    pos = torch.arange(t, device=q.device, dtype=torch.float32)
    inv = 1.0 / (10000 ** (torch.arange(0, d, 2, device=q.device, dtype=torch.float32) / d))
    ang = torch.outer(pos, inv)
    cos, sin = ang.cos()[None, None], ang.sin()[None, None]

    def rot(x):
        x1, x2 = x.float()[..., 0::2], x.float()[..., 1::2]
        return torch.stack([x1 * cos - x2 * sin, x1 * sin + x2 * cos], -1).flatten(-2).type_as(x)

    return rot(q), rot(k)


class Block(nn.Module):
    def __init__(self, Q, d, n_head, hidden, gkw, n_kv_head=None, eps=1e-6, fuse_producers=False):
        super().__init__()
        # fuse_producers: the two norms and the SwiGLU product are computed inside the forward quantizer of the layer
        # they feed (Q.rmsnorm_linear / Q.swiglu_linear) instead of as torch operations in front of it
        self.fuse = fuse_producers
        self.rmsnorm_linear, self.swiglu_linear = getattr(Q, "rmsnorm_linear", None), getattr(Q, "swiglu_linear", None)

        def lin(i, o):
            return Q.QuantizedLinear(
                i, o, bias=False,
                weight_quantizer=Q.QUANTIZER_CLASSES["QuestMXFP4Quantizer"](),
                activation_quantizer=Q.QUANTIZER_CLASSES["QuestMXFP4Quantizer"](),
                gradient_quantizer=Q.QUANTIZER_CLASSES["AlbertTsengQuantizer"](**gkw),
                backward_scheme=Q.BACKWARD_SCHEMES["Q(E)Q(Wt)t_Q(Et)Q(Xt)t"](),
            )

        self.n_head, self.hidden = n_head, hidden
        # grouped-query attention when n_kv_head < n_head (the Llama-3 shape: qkv is d + 2 d n_kv/n_head wide)
        self.n_kv_head = n_kv_head or n_head
        self.kv_dim = d // n_head * self.n_kv_head
        self.ln1, self.ln2 = RMSNorm(d, eps), RMSNorm(d, eps)
        self.c_attn, self.attn_proj = lin(d, d + 2 * self.kv_dim), lin(d, d)
        self.w12, self.c_proj = lin(d, 2 * hidden), lin(hidden, d)

    def forward(self, x):
        b, t, d = x.shape
        hd = d // self.n_head
        if self.fuse:
            qkv = self.rmsnorm_linear(x, self.ln1.weight, self.ln1.eps, self.c_attn)
        else:
            qkv = self.c_attn(self.ln1(x))
        q, k, v = qkv.split([d, self.kv_dim, self.kv_dim], dim=2)
        q = q.view(b, t, self.n_head, hd).transpose(1, 2)
        k, v = (z.view(b, t, self.n_kv_head, hd).transpose(1, 2) for z in (k, v))
        q, k = rotary(q, k)
        y = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=self.n_kv_head != self.n_head)
        y = y.transpose(1, 2).reshape(b, t, d)
        x = x + self.attn_proj(y)
        if self.fuse:
            return x + self.swiglu_linear(self.rmsnorm_linear(x, self.ln2.weight, self.ln2.eps, self.w12), self.c_proj)
        up, gate = self.w12(self.ln2(x)).split(self.hidden, dim=-1)
        return x + self.c_proj(F.silu(up) * gate)


class TinyLlama(nn.Module):
    def __init__(self, Q, vocab=512, d=256, n_layer=2, n_head=2, multiple_of=128, gkw=None, n_kv_head=None, eps=1e-6, fuse_producers=False):
        super().__init__()
        hidden = int(2 * 4 * d / 3)
        hidden = multiple_of * ((hidden + multiple_of - 1) // multiple_of)
        self.wte = nn.Embedding(vocab, d)
        self.blocks = nn.ModuleList(Block(Q, d, n_head, hidden, gkw or {"stochastic": True, "rerotate": "signs"}, n_kv_head, eps, fuse_producers)
                                    for _ in range(n_layer))
        self.ln_f, self.lm_head = RMSNorm(d, eps), nn.Linear(d, vocab, bias=False)
        for n_, p in self.named_parameters():
            if p.dim() == 2:
                nn.init.normal_(p, 0.0, 0.02 / math.sqrt(2 * n_layer) if n_.endswith("c_proj.weight") else 0.02)

    def forward(self, idx, targets, return_logits=False):
        x = self.wte(idx)
        for blk in self.blocks:
            x = blk(x)
        logits = self.lm_head(self.ln_f(x))
        loss = F.cross_entropy(logits.float().view(-1, logits.size(-1)), targets.view(-1))
        return (loss, logits) if return_logits else loss
