"""Plain PyTorch models for the reference arm of the benchmark.

The reference library ships no model, so its arm needs one from outside both
libraries: these are ordinary `torch.nn` modules (stock Linear / LayerNorm /
Embedding / scaled_dot_product_attention) with the architecture and
initialisation the benchmark configuration names.  Nothing here imports
`lowbit_comm_b200`.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import nn


class PlainGPT2Block(nn.Module):
    def __init__(self, d_model: int, n_head: int) -> None:
        super().__init__()
        self.n_head = n_head
        self.ln_1 = nn.LayerNorm(d_model)
        self.c_attn = nn.Linear(d_model, 3 * d_model)
        self.c_proj = nn.Linear(d_model, d_model)
        self.ln_2 = nn.LayerNorm(d_model)
        self.c_fc = nn.Linear(d_model, 4 * d_model)
        self.c_out = nn.Linear(4 * d_model, d_model)

    def forward(self, x):
        B, T, C = x.size()
        qkv = self.c_attn(self.ln_1(x))
        q, k, v = qkv.split(C, dim=2)
        q = q.view(B, T, self.n_head, C // self.n_head).transpose(1, 2)
        k = k.view(B, T, self.n_head, C // self.n_head).transpose(1, 2)
        v = v.view(B, T, self.n_head, C // self.n_head).transpose(1, 2)
        y = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        x = x + self.c_proj(y.transpose(1, 2).contiguous().view(B, T, C))
        return x + self.c_out(F.gelu(self.c_fc(self.ln_2(x)), approximate="tanh"))


class PlainGPT2(nn.Module):
    def __init__(self, n_layer=12, n_head=12, d_model=768, vocab_size=50257, seq_len=1024) -> None:
        super().__init__()
        self.tok = nn.Embedding(vocab_size, d_model)
        self.pos = nn.Embedding(seq_len, d_model)
        self.h = nn.ModuleList(PlainGPT2Block(d_model, n_head) for _ in range(n_layer))
        self.ln_f = nn.LayerNorm(d_model)
        for m in self.modules():
            if isinstance(m, (nn.Linear, nn.Embedding)):
                nn.init.normal_(m.weight, mean=0.0, std=0.02)
                if isinstance(m, nn.Linear) and m.bias is not None:
                    nn.init.zeros_(m.bias)
        for name, p in self.named_parameters():
            if name.endswith("c_proj.weight") or name.endswith("c_out.weight"):
                nn.init.normal_(p, mean=0.0, std=0.02 / math.sqrt(2 * n_layer))

    def forward(self, idx, targets):
        T = idx.size(1)
        x = self.tok(idx) + self.pos(torch.arange(T, device=idx.device))
        for block in self.h:
            x = block(x)
        logits = F.linear(self.ln_f(x), self.tok.weight)
        return F.cross_entropy(logits.float().view(-1, logits.size(-1)), targets.reshape(-1))


class PlainLlamaBlock(nn.Module):
    def __init__(self, d_model: int, n_head: int, n_kv_head: int, d_ff: int) -> None:
        super().__init__()
        self.n_head, self.n_kv_head, self.hd = n_head, n_kv_head, d_model // n_head
        self.norm1 = nn.RMSNorm(d_model, eps=1e-5)
        self.wq = nn.Linear(d_model, n_head * self.hd, bias=False)
        self.wkv = nn.Linear(d_model, 2 * n_kv_head * self.hd, bias=False)
        self.wo = nn.Linear(n_head * self.hd, d_model, bias=False)
        self.norm2 = nn.RMSNorm(d_model, eps=1e-5)
        self.w13 = nn.Linear(d_model, 2 * d_ff, bias=False)
        self.w2 = nn.Linear(d_ff, d_model, bias=False)

    @staticmethod
    def rope(x, cos, sin):
        a, b = x[..., : x.size(-1) // 2], x[..., x.size(-1) // 2:]
        return torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1)

    def forward(self, x, cos, sin):
        B, T, _ = x.shape
        h = self.norm1(x)
        q = self.wq(h).view(B, T, self.n_head, self.hd).transpose(1, 2)
        k, v = self.wkv(h).view(B, T, 2, self.n_kv_head, self.hd).permute(2, 0, 3, 1, 4)
        y = F.scaled_dot_product_attention(self.rope(q, cos, sin), self.rope(k, cos, sin), v, is_causal=True,
                                           enable_gqa=True)
        x = x + self.wo(y.transpose(1, 2).reshape(B, T, -1))
        gate, up = self.w13(self.norm2(x)).chunk(2, dim=-1)
        return x + self.w2(F.silu(gate) * up)


class PlainLlama(nn.Module):
    """Llama-style decoder: RMSNorm, rotary embeddings, grouped-query attention, SwiGLU, untied head,
    activation checkpointing per block while training."""

    def __init__(self, n_layer=28, d_model=3072, n_head=24, n_kv_head=8, d_ff=8192, vocab_size=128256, seq_len=2048,
                 rope_theta=500000.0) -> None:
        super().__init__()
        self.hd, self.rope_theta = d_model // n_head, rope_theta
        self.embed = nn.Embedding(vocab_size, d_model)
        self.blocks = nn.ModuleList(PlainLlamaBlock(d_model, n_head, n_kv_head, d_ff) for _ in range(n_layer))
        self.norm = nn.RMSNorm(d_model, eps=1e-5)
        self.head = nn.Linear(d_model, vocab_size, bias=False)
        for p in self.parameters():
            if p.dim() >= 2:
                nn.init.normal_(p, mean=0.0, std=0.02)

    def forward(self, idx, targets):
        from torch.utils.checkpoint import checkpoint

        x = self.embed(idx)
        T = idx.size(1)
        inv = 1.0 / (self.rope_theta ** (torch.arange(0, self.hd, 2, device=x.device, dtype=torch.float32) / self.hd))
        ang = torch.outer(torch.arange(T, device=x.device, dtype=torch.float32), inv)
        cos, sin = ang.cos().to(x.dtype), ang.sin().to(x.dtype)
        for block in self.blocks:
            x = checkpoint(block, x, cos, sin, use_reentrant=False) if self.training else block(x, cos, sin)
        logits = self.head(self.norm(x))
        return F.cross_entropy(logits.float().view(-1, logits.size(-1)), targets.reshape(-1))
