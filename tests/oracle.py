"""Unsharded single-process restatement of the model, loss and optimizer in plain PyTorch
(fp32, eager attention, full-vocabulary cross entropy, torch AdamW). It uses the same
state_dict keys as the TP=1 model so weights can be exchanged through
``utils.reshard``. This is the oracle for the distributed CPU tests."""
import math

import torch
import torch.nn as nn
import torch.nn.functional as F


def rope_interleaved(x, cos, sin):
    # x: [S, B, nh, D]; cos/sin: [S, D/2]
    xe, xo = x[..., 0::2], x[..., 1::2]
    c, s = cos[:, None, None, :], sin[:, None, None, :]
    return torch.stack((xe * c - xo * s, xe * s + xo * c), dim=-1).flatten(-2)


class NaiveRMSNorm(nn.Module):
    def __init__(self, H, eps):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(H))
        self.eps = eps

    def forward(self, x):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.eps) * self.weight


class NaiveAttention(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        H = cfg.hidden_size
        self.nh = cfg.num_attention_heads
        self.D = H // self.nh
        bias = getattr(cfg, "bias", False)
        self.qkv_proj = nn.Linear(H, 3 * H, bias=bias)
        self.out_proj = nn.Linear(H, H, bias=bias)
        freqs = 1.0 / (10000.0 ** (torch.arange(0, self.D, 2, dtype=torch.float32) / self.D))
        self.rotary_emb = nn.Module()
        self.rotary_emb.register_buffer("freqs", freqs)

    def forward(self, x):
        S, B, H = x.shape
        q, k, v = self.qkv_proj(x).view(S, B, 3, self.nh, self.D).unbind(2)
        ang = torch.outer(torch.arange(S, dtype=torch.float32), self.rotary_emb.freqs)
        q, k = rope_interleaved(q, ang.cos(), ang.sin()), rope_interleaved(k, ang.cos(), ang.sin())
        q, k, v = (t.permute(1, 2, 0, 3) for t in (q, k, v))
        s = q @ k.transpose(-1, -2) / math.sqrt(self.D)
        s = s.masked_fill(~torch.ones(S, S, dtype=torch.bool).tril(), float("-inf"))
        o = torch.softmax(s, -1) @ v
        return self.out_proj(o.permute(2, 0, 1, 3).reshape(S, B, H))


class NaiveMLP(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        bias = getattr(cfg, "bias", False)
        self.gate_up_proj = nn.Linear(cfg.hidden_size, 2 * cfg.intermediate_size, bias=bias)
        self.down_proj = nn.Linear(cfg.intermediate_size, cfg.hidden_size, bias=bias)

    def forward(self, x):
        g, u = self.gate_up_proj(x).chunk(2, dim=-1)
        return self.down_proj(F.silu(g) * u)


class NaiveLayer(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.input_norm = NaiveRMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.attention = NaiveAttention(cfg)
        self.post_attention_norm = NaiveRMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.mlp = NaiveMLP(cfg)

    def forward(self, x):
        x = x + self.attention(self.input_norm(x))
        return x + self.mlp(self.post_attention_norm(x))


class NaiveGPT(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.embedding = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
        self.layers = nn.ModuleList([NaiveLayer(cfg) for _ in range(cfg.num_layers)])
        self.final_norm = NaiveRMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.output = nn.Linear(cfg.hidden_size, cfg.vocab_size, bias=False)

    def forward(self, ids):  # [B, S] -> [S, B, V]
        x = self.embedding(ids).transpose(0, 1)
        for layer in self.layers:
            x = layer(x)
        return self.output(self.final_norm(x))

    def loss(self, ids, labels):
        logits = self.forward(ids)
        return F.cross_entropy(logits.reshape(-1, logits.shape[-1]), labels.t().reshape(-1))


def naive_step(model, opt, ids, labels, clip):
    opt.zero_grad()
    loss = model.loss(ids, labels)
    loss.backward()
    if clip and clip > 0:
        grads = [p.grad for p in model.parameters()]
        norm = torch.sqrt(sum(g.float().pow(2).sum() for g in grads))
        if norm > clip:
            for g in grads:
                g.mul_(clip / (norm + 1e-6))
    opt.step()
    return loss.detach()
