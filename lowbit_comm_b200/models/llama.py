"""Llama-style decoder (RMSNorm, RoPE, grouped-query attention, SwiGLU) with
optional activation checkpointing; the 3B preset is the large DDP benchmark
configuration (28 layers, d_model 3072, 24 query / 8 KV heads, FFN 8192,
vocab 128256, sequence 2048).  The reference ships no model.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn
from torch.utils.checkpoint import checkpoint


@dataclass(frozen=True)
class LlamaConfig:
    n_layer: int = 28
    d_model: int = 3072
    n_head: int = 24
    n_kv_head: int = 8
    d_ff: int = 8192
    vocab_size: int = 128256
    seq_len: int = 2048
    rope_theta: float = 500000.0
    checkpoint_activations: bool = True
    name: str = "llama-3b"

    @classmethod
    def tiny(cls) -> "LlamaConfig":
        return cls(n_layer=2, d_model=64, n_head=4, n_kv_head=2, d_ff=128, vocab_size=257, seq_len=32,
                   checkpoint_activations=True, name="llama-tiny")


class RMSNorm(nn.Module):
    def __init__(self, d: int, eps: float = 1e-5) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.ones(d))
        self.eps = eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return F.rms_norm(x, (x.size(-1),), self.weight, self.eps)


def rope_tables(seq_len: int, head_dim: int, theta: float, device, dtype):
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim))
    ang = torch.outer(torch.arange(seq_len, device=device, dtype=torch.float32), inv)
    return ang.cos().to(dtype), ang.sin().to(dtype)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    # x: [b, h, t, d]; rotate pairs (even, odd halves)
    x1, x2 = x[..., : x.size(-1) // 2], x[..., x.size(-1) // 2:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)


class LlamaBlock(nn.Module):
    def __init__(self, cfg: LlamaConfig) -> None:
        super().__init__()
        self.cfg = cfg
        hd = cfg.d_model // cfg.n_head
        self.hd = hd
        self.norm1 = RMSNorm(cfg.d_model)
        self.wq = nn.Linear(cfg.d_model, cfg.n_head * hd, bias=False)
        self.wkv = nn.Linear(cfg.d_model, 2 * cfg.n_kv_head * hd, bias=False)
        self.wo = nn.Linear(cfg.n_head * hd, cfg.d_model, bias=False)
        self.norm2 = RMSNorm(cfg.d_model)
        self.w13 = nn.Linear(cfg.d_model, 2 * cfg.d_ff, bias=False)
        self.w2 = nn.Linear(cfg.d_ff, cfg.d_model, bias=False)

    def forward(self, x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        b, t, _ = x.shape
        h = self.norm1(x)
        q = self.wq(h).view(b, t, cfg.n_head, self.hd).transpose(1, 2)
        k, v = self.wkv(h).view(b, t, 2, cfg.n_kv_head, self.hd).permute(2, 0, 3, 1, 4)
        q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
        att = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
        x = x + self.wo(att.transpose(1, 2).reshape(b, t, -1))
        gate, up = self.w13(self.norm2(x)).chunk(2, dim=-1)
        return x + self.w2(F.silu(gate) * up)


class Llama(nn.Module):
    def __init__(self, cfg: LlamaConfig = LlamaConfig()) -> None:
        super().__init__()
        self.cfg = cfg
        self.embed = nn.Embedding(cfg.vocab_size, cfg.d_model)
        self.blocks = nn.ModuleList(LlamaBlock(cfg) for _ in range(cfg.n_layer))
        self.norm = RMSNorm(cfg.d_model)
        self.head = nn.Linear(cfg.d_model, cfg.vocab_size, bias=False)
        for p in self.parameters():
            if p.dim() >= 2:
                nn.init.normal_(p, mean=0.0, std=0.02)

    def forward(self, tokens: torch.Tensor, targets: torch.Tensor | None = None) -> torch.Tensor:
        cfg = self.cfg
        x = self.embed(tokens)
        cos, sin = rope_tables(tokens.size(1), cfg.d_model // cfg.n_head, cfg.rope_theta, x.device, x.dtype)
        for block in self.blocks:
            if cfg.checkpoint_activations and self.training:
                x = checkpoint(block, x, cos, sin, use_reentrant=False)
            else:
                x = block(x, cos, sin)
        logits = self.head(self.norm(x))
        if targets is None:
            return logits
        return F.cross_entropy(logits.float().view(-1, logits.size(-1)), targets.reshape(-1))

    def num_parameters(self) -> int:
        return sum(p.numel() for p in self.parameters())
