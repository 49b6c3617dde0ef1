"""Generates the three CHRN fixtures of the reference's test suite from the PyTorch oracle, with the
reference's tensor names, so either project's tests can read the other's files:

``m1``    ``m1_ref.bin``: inputs, weights, logits, loss, every parameter gradient and the parameters
          after one ``torch.optim.AdamW`` step (tests/gen_reference.py:121-176; seed 1337, L2 d128 h4
          V256 seq64 batch8, lr 3e-4 betas (0.9, 0.95) eps 1e-8 wd 0.1);
``attn``  ``attn_ref.bin``: q, k, v, causal attention output, an upstream gradient and dq, dk, dv for
          B2 H4 T256 hd64, layout [B, H, T, hd] (tests/gen_attn_ref.py:9-10, seed 2024);
``gen``   ``gen_ref.bin``: weights of the same tiny model, four prompts of staggered length (the second
          shares a 6-token prefix with the first) and their greedy continuations
          (tests/gen_gen_ref.py:110-124).

``python -m kharon_b200.utils.gen_fixtures [m1|attn|gen] [path]`` (CPU, fp32, deterministic; a lone
path argument means ``m1``)."""
import sys

import torch

from ..models import Config
from ..models.oracle import OracleGPT
from . import chrn

CFG = Config(2, 128, 4, 256, 64, 8)
OPT = dict(lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1)
_REN = {"ln1_w": "ln1.w", "ln1_b": "ln1.b", "qkv_w": "qkv.w", "qkv_b": "qkv.b", "proj_w": "proj.w", "proj_b": "proj.b",
        "ln2_w": "ln2.w", "ln2_b": "ln2.b", "fc_w": "fc.w", "fc_b": "fc.b", "fcproj_w": "fcproj.w", "fcproj_b": "fcproj.b"}


def fixture_name(name: str) -> str:
    if name.startswith("l") and "." in name:
        l, f = name.split(".")
        return "blk%s.%s" % (l[1:], _REN[f])
    return {"lnf_w": "lnf.w", "lnf_b": "lnf.b"}.get(name, name)


def attn_fixture(path="tests/attn_ref.bin", B=2, H=4, T=256, hd=64, seed=2024):
    """Causal attention forward and backward in fp32 (explicit mask-then-softmax, the oracle's formula)."""
    import math
    torch.manual_seed(seed)
    q, k, v = (torch.randn(B, H, T, hd, requires_grad=True) for _ in range(3))
    att = (q @ k.transpose(-1, -2)) / math.sqrt(hd)
    mask = torch.ones(T, T, dtype=torch.bool).tril()
    o = att.masked_fill(~mask, float("-inf")).softmax(-1) @ v
    do = torch.randn_like(o)
    o.backward(do)
    w = chrn.Writer(path, [0, H * hd, H, 0, T, B], [0, 0, 0, 0, 0])
    for name, t in (("q", q), ("k", k), ("v", v), ("o", o), ("do", do), ("dq", q.grad), ("dk", k.grad), ("dv", v.grad)):
        w.put(name, t)
    w.close()
    print("wrote %s  B=%d H=%d T=%d hd=%d" % (path, B, H, T, hd))
    return path


@torch.no_grad()
def greedy(m, prompt, n_new):
    ids = list(prompt)
    for _ in range(n_new):
        logits, _ = m(torch.tensor([ids], dtype=torch.long))
        ids.append(int(logits[0, -1].argmax()))
    return ids


def gen_fixture(path="tests/gen_ref.bin", cfg=CFG, seed=1337):
    torch.manual_seed(seed)
    torch.use_deterministic_algorithms(True)
    m = OracleGPT(cfg)
    w = chrn.Writer(path, cfg.as_list(), [OPT["lr"], OPT["beta1"], OPT["beta2"], OPT["eps"], OPT["wd"]])
    for n, p in m.named_tensors().items():
        w.put(fixture_name(n), p)
    g = torch.Generator().manual_seed(7)
    draw = lambda k: torch.randint(0, cfg.vocab, (k,), generator=g).tolist()
    base = draw(12)
    prompts = [base[:6], base[:6] + draw(4), draw(10), draw(3)]
    n_new = [20, 16, 24, 28]
    w.put("n_seq", torch.tensor([len(prompts)], dtype=torch.int32))
    for i, (pr, k) in enumerate(zip(prompts, n_new)):
        w.put("prompt%d" % i, torch.tensor(pr, dtype=torch.int32))
        w.put("gen%d" % i, torch.tensor(greedy(m, pr, k), dtype=torch.int32))     # prompt + continuation
    w.close()
    torch.use_deterministic_algorithms(False)
    print("wrote %s  prompts=%d" % (path, len(prompts)))
    return path


def main(argv=None, cfg=CFG, seed=1337):
    args = list(sys.argv[1:] if argv is None else argv)
    if args and args[0] in ("m1", "attn", "gen"):
        kind, args = args[0], args[1:]
        if kind == "attn":
            return attn_fixture(*args[:1])
        if kind == "gen":
            return gen_fixture(*args[:1])
    path = (args or ["tests/m1_ref.bin"])[0]
    torch.manual_seed(seed)
    torch.use_deterministic_algorithms(True)
    m = OracleGPT(cfg)
    idx = torch.randint(0, cfg.vocab, (cfg.batch, cfg.seq))
    tgt = torch.randint(0, cfg.vocab, (cfg.batch, cfg.seq))
    w = chrn.Writer(path, cfg.as_list(), [OPT["lr"], OPT["beta1"], OPT["beta2"], OPT["eps"], OPT["wd"]])
    w.put("input_ids", idx)
    w.put("targets", tgt)
    named = m.named_tensors()
    for n, p in named.items():
        w.put(fixture_name(n), p)
    logits, loss = m(idx, tgt)
    loss.backward()
    w.put("logits", logits)
    w.put("loss", loss.item())
    for n, p in named.items():
        w.put(fixture_name(n) + ".grad", p.grad)
    opt = torch.optim.AdamW(m.parameters(), lr=OPT["lr"], betas=(OPT["beta1"], OPT["beta2"]), eps=OPT["eps"],
                            weight_decay=OPT["wd"])
    opt.step()
    for n, p in named.items():
        w.put(fixture_name(n) + ".step", p.detach())
    w.close()
    torch.use_deterministic_algorithms(False)
    print("wrote %s  loss=%.6f  params=%d" % (path, loss.item(), sum(p.numel() for p in m.parameters())))
    return path


if __name__ == "__main__":
    main()
