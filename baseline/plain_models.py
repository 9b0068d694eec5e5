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
