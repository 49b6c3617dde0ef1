"""PyTorch-autograd statement of the architecture: the specification every native path is
tested against (same model as the reference's tests/gen_reference.py:59-118: nn.LayerNorm
eps 1e-5, fused qkv Linear, mask-then-softmax attention, tanh GELU, tied head, mean CE)."""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from .layout import Config, LAYER_FIELDS


class Block(nn.Module):
    def __init__(self, d, H):
        super().__init__()
        self.H = H
        self.ln1 = nn.LayerNorm(d)
        self.qkv = nn.Linear(d, 3 * d)
        self.proj = nn.Linear(d, d)
        self.ln2 = nn.LayerNorm(d)
        self.fc = nn.Linear(d, 4 * d)
        self.fcproj = nn.Linear(4 * d, d)

    def forward(self, x):
        B, T, d = x.shape
        q, k, v = self.qkv(self.ln1(x)).split(d, dim=-1)
        sh = lambda t: t.view(B, T, self.H, d // self.H).transpose(1, 2)
        q, k, v = sh(q), sh(k), sh(v)
        att = (q @ k.transpose(-1, -2)) / math.sqrt(d // self.H)
        mask = torch.ones(T, T, dtype=torch.bool, device=x.device).tril()
        att = att.masked_fill(~mask, float("-inf")).softmax(-1)
        y = (att @ v).transpose(1, 2).reshape(B, T, d)
        x = x + self.proj(y)
        return x + self.fcproj(F.gelu(self.fc(self.ln2(x)), approximate="tanh"))


class OracleGPT(nn.Module):
    def __init__(self, cfg: Config, untied_head=False):
        super().__init__()
        self.cfg = cfg
        self.wte = nn.Embedding(cfg.vocab, cfg.d_model)
        self.wpe = nn.Embedding(cfg.seq, cfg.d_model)
        self.blocks = nn.ModuleList([Block(cfg.d_model, cfg.n_head) for _ in range(cfg.n_layer)])
        self.lnf = nn.LayerNorm(cfg.d_model)
        self.head = nn.Linear(cfg.d_model, cfg.vocab, bias=False) if untied_head else None
        for m in self.modules():
            if isinstance(m, (nn.Linear, nn.Embedding)):
                nn.init.normal_(m.weight, 0.0, 0.02)
            if isinstance(m, nn.Linear) and m.bias is not None:
                nn.init.zeros_(m.bias)

    def forward(self, idx, tgt=None):
        B, T = idx.shape
        x = self.wte(idx) + self.wpe(torch.arange(T, device=idx.device))
        for b in self.blocks:
            x = b(x)
        x = self.lnf(x)
        logits = x @ (self.head.weight if self.head is not None else self.wte.weight).t()
        loss = None
        if tgt is not None:
            loss = F.cross_entropy(logits.view(B * T, -1), tgt.reshape(-1))
        return logits, loss

    def named_tensors(self):
        """{framework parameter name: nn.Parameter} in arena order."""
        out = {"wte": self.wte.weight, "wpe": self.wpe.weight}
        for i, b in enumerate(self.blocks):
            mods = {"ln1": b.ln1, "qkv": b.qkv, "proj": b.proj, "ln2": b.ln2, "fc": b.fc, "fcproj": b.fcproj}
            for f in LAYER_FIELDS:
                mod, kind = f.rsplit("_", 1)
                out["l%d.%s" % (i, f)] = mods[mod].weight if kind == "w" else mods[mod].bias
        out["lnf_w"] = self.lnf.weight
        out["lnf_b"] = self.lnf.bias
        if self.head is not None:
            out["head_w"] = self.head.weight
        return out

    def load_from(self, model):
        """Copy the fp32 master weights of a framework GPT (single stage, tp = 1)."""
        with torch.no_grad():
            for n, p in self.named_tensors().items():
                p.copy_(model.params.p[n].cpu())
