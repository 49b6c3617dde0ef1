"""Generates the CHRN fixture ``m1_ref.bin`` from the PyTorch oracle: inputs, weights, logits, loss,
every parameter gradient and the parameters after one ``torch.optim.AdamW`` step, with the tensor
names of the reference's tests/gen_reference.py:121-176, so either project's tests can read it.
``python -m kharon_b200.utils.gen_fixtures [tests/m1_ref.bin]`` (CPU, fp32, deterministic, seed 1337,
L2 d128 h4 V256 seq64 batch8, lr 3e-4 betas (0.9, 0.95) eps 1e-8 wd 0.1)."""
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


def main(argv=None, cfg=CFG, seed=1337):
    path = ((sys.argv[1:] if argv is None else argv) or ["tests/m1_ref.bin"])[0]
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
