"""Llama-style decoder used as the payload of the data-parallel training benchmark.

The transport does not care what the gradients belong to; this model only has to
produce the traffic pattern of a real step: 16 layers, d_model 2048, 32 query heads
over 8 KV heads, SwiGLU FFN of 8192, vocabulary 128256, rotary embeddings, bf16,
random initialisation.  Plain PyTorch on purpose (fused attention from
torch.nn.functional); the code under test is the gradient all_reduce below it.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class LlamaConfig:
    vocab_size: int = 128256
    d_model: int = 2048
    n_layers: int = 16
    n_heads: int = 32
    n_kv_heads: int = 8
    ffn_dim: int = 8192
    rope_theta: float = 500000.0
    norm_eps: float = 1e-5
    tie_embeddings: bool = True

    @staticmethod
    def tiny() -> "LlamaConfig":
        return LlamaConfig(vocab_size=512, d_model=64, n_layers=2, n_heads=4, n_kv_heads=2, ffn_dim=128)


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x):
        h = x.float()
        h = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + self.eps)
        return (h * self.weight.float()).to(x.dtype)


def rope_tables(seq_len: int, head_dim: int, theta: float, device, dtype):
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim))
    t = torch.arange(seq_len, device=device, dtype=torch.float32)
    ang = torch.outer(t, inv)
    return ang.cos().to(dtype), ang.sin().to(dtype)


def apply_rope(x, cos, sin):
    # x: [B, H, S, D]; rotate pairs (even, odd)
    x1, x2 = x[..., 0::2], x[..., 1::2]
    c, s = cos[None, None], sin[None, None]
    out = torch.stack((x1 * c - x2 * s, x1 * s + x2 * c), dim=-1)
    return out.flatten(-2)


class Attention(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.h, self.kv, self.d = cfg.n_heads, cfg.n_kv_heads, cfg.d_model // cfg.n_heads
        self.wq = nn.Linear(cfg.d_model, self.h * self.d, bias=False)
        self.wk = nn.Linear(cfg.d_model, self.kv * self.d, bias=False)
        self.wv = nn.Linear(cfg.d_model, self.kv * self.d, bias=False)
        self.wo = nn.Linear(self.h * self.d, cfg.d_model, bias=False)

    def forward(self, x, cos, sin):
        B, S, _ = x.shape
        q = self.wq(x).view(B, S, self.h, self.d).transpose(1, 2)
        k = self.wk(x).view(B, S, self.kv, self.d).transpose(1, 2)
        v = self.wv(x).view(B, S, self.kv, self.d).transpose(1, 2)
        q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
        rep = self.h // self.kv
        k = k.repeat_interleave(rep, dim=1)
        v = v.repeat_interleave(rep, dim=1)
        o = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        return self.wo(o.transpose(1, 2).reshape(B, S, self.h * self.d))


class Block(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.attn_norm = RMSNorm(cfg.d_model, cfg.norm_eps)
        self.attn = Attention(cfg)
        self.ffn_norm = RMSNorm(cfg.d_model, cfg.norm_eps)
        self.w_gate = nn.Linear(cfg.d_model, cfg.ffn_dim, bias=False)
        self.w_up = nn.Linear(cfg.d_model, cfg.ffn_dim, bias=False)
        self.w_down = nn.Linear(cfg.ffn_dim, cfg.d_model, bias=False)

    def forward(self, x, cos, sin):
        x = x + self.attn(self.attn_norm(x), cos, sin)
        h = self.ffn_norm(x)
        return x + self.w_down(F.silu(self.w_gate(h)) * self.w_up(h))


class LlamaDecoder(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.cfg = cfg
        self.embed = nn.Embedding(cfg.vocab_size, cfg.d_model)
        self.layers = nn.ModuleList([Block(cfg) for _ in range(cfg.n_layers)])
        self.norm = RMSNorm(cfg.d_model, cfg.norm_eps)
        self.lm_head = nn.Linear(cfg.d_model, cfg.vocab_size, bias=False)
        if cfg.tie_embeddings:
            self.lm_head.weight = self.embed.weight
        self.apply(self._init)

    @staticmethod
    def _init(m):
        if isinstance(m, (nn.Linear, nn.Embedding)):
            nn.init.normal_(m.weight, std=0.02)

    def forward(self, tokens, targets=None):
        B, S = tokens.shape
        x = self.embed(tokens)
        cos, sin = rope_tables(S, self.cfg.d_model // self.cfg.n_heads, self.cfg.rope_theta, x.device, x.dtype)
        for layer in self.layers:
            x = layer(x, cos, sin)
        logits = self.lm_head(self.norm(x))
        if targets is None:
            return logits
        return F.cross_entropy(logits.float().reshape(-1, logits.size(-1)), targets.reshape(-1))

    def num_parameters(self) -> int:
        return sum(p.numel() for p in self.parameters())
