"""Tracing / metrics plumbing: per-phase timers, roofline fractions, JSONL metrics."""
import json
import os

import torch

from kharon_b200 import train
from kharon_b200.engine import TrainEngine
from kharon_b200.utils import trace
from kharon_b200.utils.rng import Rng


def test_engine_phase_trace_and_roofline():
    eng = TrainEngine(2, 64, 4, 256, 16, 2, 2, device="cpu", dtype=torch.float32, trace=True)
    idx, tgt = Rng(1).batch(eng.tokens_per_step, 256)
    for _ in range(2):
        eng.train_step(idx, tgt)
    rep = eng.tracer.report()
    assert rep["forward"][0] == 4 and rep["backward"][0] == 4 and rep["optimizer"][0] == 2
    assert all(ms >= 0 for _, ms in rep.values())
    r = trace.roofline(flops=2 * 8192 ** 3, bytes_=3 * 8192 * 8192 * 2, ms=1.0)
    assert 0 < r["tensor_frac"] < 1 and r["of"] in ("measured", "fallback")


def test_jsonl_metrics(tmp_path):
    out = tmp_path / "m.jsonl"
    train.main(["--layers", "2", "--d", "64", "--heads", "4", "--seq", "16", "--batch", "2", "--steps", "4", "--log", "2",
                "--ckptevery", "0", "--ckpt", str(tmp_path / "c.ckpt"), "--synthetic", "--device", "cpu", "--fp32",
                "--jsonl", str(out)])
    rows = [json.loads(l) for l in open(out)]
    assert [r["step"] for r in rows] == [2, 4] and all("loss" in r and "tok_s" in r for r in rows)


def test_plot_writes_charts_without_a_display(tmp_path):
    """bench/plot.py renders the committed results file headlessly (SVG writer when matplotlib is absent)."""
    from kharon_b200.bench import plot
    made = plot.main([os.path.join(os.path.dirname(plot.__file__), "results.json"), str(tmp_path)])
    assert len(made) == 3
    for m in made:
        assert os.path.getsize(m) > 500
