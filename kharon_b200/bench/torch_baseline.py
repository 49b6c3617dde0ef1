"""PyTorch eager baseline on the same shapes as ``kharon_b200.train`` (bf16 autocast, SDPA attention,
``torch.optim.AdamW``): ``python -m kharon_b200.bench.torch_baseline --layers 8 --d 512 --heads 8 --vocab 50257
--seq 256 --batch 32 --steps 50``.  Counterpart of the reference's bench/torch_baseline.py; it is a
comparison point only -- nothing in the framework runs through it (and torch.compile is not used)."""
import argparse
import json
import time

import torch
import torch.nn.functional as F

from ..models import Config
from ..models.oracle import OracleGPT


def main(argv=None):
    p = argparse.ArgumentParser()
    for name, default in (("layers", 8), ("d", 512), ("heads", 8), ("vocab", 256), ("seq", 256), ("batch", 32), ("steps", 50)):
        p.add_argument("--" + name, type=int, default=default)
    a = p.parse_args(argv)
    dev = "cuda"
    cfg = Config(a.layers, a.d, a.heads, a.vocab, a.seq, a.batch)
    m = OracleGPT(cfg).to(dev)
    for b in m.blocks:                       # fused attention instead of the oracle's mask-then-softmax
        def fwd(x, b=b):
            B, T, d = x.shape
            q, k, v = b.qkv(b.ln1(x)).split(d, dim=-1)
            sh = lambda t: t.view(B, T, b.H, d // b.H).transpose(1, 2)
            y = F.scaled_dot_product_attention(sh(q), sh(k), sh(v), is_causal=True)
            x = x + b.proj(y.transpose(1, 2).reshape(B, T, d))
            return x + b.fcproj(F.gelu(b.fc(b.ln2(x)), approximate="tanh"))
        b.forward = fwd
    opt = torch.optim.AdamW(m.parameters(), lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1)
    idx = torch.randint(0, a.vocab, (a.batch, a.seq), device=dev)
    tgt = torch.randint(0, a.vocab, (a.batch, a.seq), device=dev)

    def step():
        opt.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            _, loss = m(idx, tgt)
        loss.backward()
        opt.step()

    for _ in range(10):
        step()
    torch.cuda.synchronize()
    t0 = time.time()
    for _ in range(a.steps):
        step()
    torch.cuda.synchronize()
    dt = (time.time() - t0) / a.steps
    res = dict(impl="torch eager " + torch.__version__, ms_per_step=dt * 1e3, tok_s=a.batch * a.seq / dt, **vars(a))
    print(json.dumps(res))
    return res


if __name__ == "__main__":
    main()
