"""A Llama-3-shaped decoder written with stock PyTorch modules only (``nn.Linear``, ``nn.RMSNorm``,
``F.scaled_dot_product_attention``, ``nn.Embedding``). The reference project has no model of its
own (its examples stack ``nn.TransformerEncoderLayer``), so this is the model its Trainer is given
for the 8B-shape configuration. Sub-module names contain ``attention`` and ``mlp`` so that the
reference's ``ActivationManager`` name matching (zenyx/memory/activation_manager.py:28-40) selects them."""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F


def rope_tables(seq_len: int, head_dim: int, theta: float, device, dtype):
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim))
    ang = torch.arange(seq_len, device=device, dtype=torch.float32)[:, None] * inv[None, :]
    return ang.cos().to(dtype), ang.sin().to(dtype)


def apply_rope(x, cos, sin):  # x [B,H,S,D]
    d = x.shape[-1] // 2
    x1, x2 = x[..., :d], x[..., d:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)


class Attention(nn.Module):
    def __init__(self, d_model, n_heads, n_kv_heads, head_dim, theta):
        super().__init__()
        self.n_heads, self.n_kv_heads, self.head_dim, self.theta = n_heads, n_kv_heads, head_dim, theta
        self.wqkv = nn.Linear(d_model, (n_heads + 2 * n_kv_heads) * head_dim, bias=False)
        self.wo = nn.Linear(n_heads * head_dim, d_model, bias=False)

    def forward(self, x):
        B, S, _ = x.shape
        H, Hk, D = self.n_heads, self.n_kv_heads, self.head_dim
        qkv = self.wqkv(x)
        q = qkv[..., : H * D].view(B, S, H, D).transpose(1, 2)
        k = qkv[..., H * D: (H + Hk) * D].view(B, S, Hk, D).transpose(1, 2)
        v = qkv[..., (H + Hk) * D:].view(B, S, Hk, D).transpose(1, 2)
        cos, sin = rope_tables(S, D, self.theta, x.device, x.dtype)
        q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
        o = F.scaled_dot_product_attention(q, k, v, is_causal=True, scale=1.0 / math.sqrt(D), enable_gqa=True)
        return self.wo(o.transpose(1, 2).reshape(B, S, H * D))


class MLP(nn.Module):
    def __init__(self, d_model, ffn_dim):
        super().__init__()
        self.gate = nn.Linear(d_model, ffn_dim, bias=False)
        self.up = nn.Linear(d_model, ffn_dim, bias=False)
        self.down = nn.Linear(ffn_dim, d_model, bias=False)

    def forward(self, x):
        return self.down(F.silu(self.gate(x)) * self.up(x))


class Block(nn.Module):
    def __init__(self, d_model, n_heads, n_kv_heads, head_dim, ffn_dim, eps, theta):
        super().__init__()
        self.norm1 = nn.RMSNorm(d_model, eps=eps)
        self.attention = Attention(d_model, n_heads, n_kv_heads, head_dim, theta)
        self.norm2 = nn.RMSNorm(d_model, eps=eps)
        self.mlp = MLP(d_model, ffn_dim)

    def forward(self, x):
        x = x + self.attention(self.norm1(x))
        return x + self.mlp(self.norm2(x))


class TorchLlama(nn.Module):
    def __init__(self, vocab_size=128256, d_model=4096, n_layers=32, n_heads=32, n_kv_heads=8, head_dim=128,
                 ffn_dim=14336, eps=1e-5, theta=500000.0):
        super().__init__()
        self.embed = nn.Embedding(vocab_size, d_model)
        self.blocks = nn.ModuleList([Block(d_model, n_heads, n_kv_heads, head_dim, ffn_dim, eps, theta)
                                     for _ in range(n_layers)])
        self.final_norm = nn.RMSNorm(d_model, eps=eps)
        self.lm_head = nn.Linear(d_model, vocab_size, bias=False)

    def forward(self, tokens):
        h = self.embed(tokens)
        for b in self.blocks:
            h = b(h)
        return self.lm_head(self.final_norm(h))


class TokenCrossEntropy(nn.Module):
    """CrossEntropyLoss over [B,S,V] logits and [B,S] targets."""

    def forward(self, logits, targets):
        return F.cross_entropy(logits.reshape(-1, logits.shape[-1]), targets.reshape(-1))
