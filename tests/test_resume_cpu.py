"""Checkpoint / resume is bit-exact: 16 uninterrupted steps versus 8 steps, a checkpoint, a fresh
process-like model and 8 more steps -- the loss bits and every parameter must be equal
(reference tests/test_resume.c:37-64).  Runs the public trainer entry point."""
import torch

from kharon_b200 import train
from kharon_b200.utils import ckpt


def _run(tmp, name, steps, resume=False, dtype_flag="--fp32"):
    argv = ["--layers", "2", "--d", "64", "--heads", "4", "--seq", "32", "--batch", "4", "--steps", str(steps),
            "--log", "1000", "--ckptevery", "0", "--ckpt", str(tmp / name), "--synthetic", "--vocab", "256",
            "--device", "cpu", dtype_flag]
    if resume:
        argv.append("--resume")
    return train.main(argv)


def test_resume_is_bit_exact_fp32(tmp_path):
    full = _run(tmp_path, "full.ckpt", 16)
    _run(tmp_path, "half.ckpt", 8)
    resumed = _run(tmp_path, "half.ckpt", 16, resume=True)
    assert resumed.model.step == 16
    assert resumed.loss() == full.loss()                       # equality of the float bits
    assert torch.equal(resumed.model.params.w, full.model.params.w)
    assert torch.equal(resumed.model.params.m, full.model.params.m)
    a, b = ckpt.peek(str(tmp_path / "full.ckpt")), ckpt.peek(str(tmp_path / "half.ckpt"))
    assert a == b                                              # same step, RNG state and sizes


def test_resume_is_bit_exact_bf16_emulated(tmp_path):
    full = _run(tmp_path, "f.ckpt", 6, dtype_flag="--bf16")
    _run(tmp_path, "h.ckpt", 3, dtype_flag="--bf16")
    resumed = _run(tmp_path, "h.ckpt", 6, resume=True, dtype_flag="--bf16")
    assert resumed.loss() == full.loss()
    assert torch.equal(resumed.model.params.w, full.model.params.w)
