"""GRPO pieces on CPU (reference tests/test_grpo.c:19-72): the coefficient form of the backward
pass reproduces cross-entropy exactly when coef = 1/R and scales linearly; a short SFT + GRPO run
of the addition task improves accuracy and keeps rewards finite."""
import torch

from kharon_b200.models import GPT, Config
from kharon_b200.rl import AddTask, GRPOTrainer, ReverseTask
from kharon_b200.utils.rng import Rng


def test_grpo_backward_equals_ce_when_coef_is_uniform():
    cfg = Config(2, 64, 4, 256, 8, 6)
    R = cfg.batch * cfg.seq
    idx, tgt = Rng(3).batch(R, cfg.vocab)
    grads = []
    for coef in (None, torch.full((R,), 1.0 / R), torch.full((R,), 2.0 / R)):
        m = GPT(cfg, "cpu", torch.float32)
        m.init_weights(1337)
        m.set_input(idx, tgt)
        m.forward(compute_loss=False)
        m.backward(coef=coef)
        grads.append(m.params.g.clone())
    assert torch.equal(grads[0], grads[1])                     # bit-identical to the CE backward
    assert torch.allclose(grads[2], 2 * grads[0], rtol=1e-3, atol=1e-7)


def test_tasks():
    r = Rng(1)
    p, a = ReverseTask().sample(r)
    assert len(p) == 9 and len(a) == 9 and a[:8] == p[:8][::-1] and ReverseTask().reward(a, a) == 1.0
    assert ReverseTask().reward(a[:-1] + [0], a) == 0.0
    p, a = AddTask().sample(r)
    assert chr(a[0]) == str(int(chr(p[0])) + int(chr(p[2])))
    assert AddTask().reward([ord("x")], a) == 0.0 and abs(AddTask().reward(a, a) - 1.1) < 1e-6


def test_short_sft_then_grpo_improves_addition():
    torch.manual_seed(0)
    tr = GRPOTrainer(AddTask(), layers=2, d_model=64, heads=4, G=4, prompts=8, lr=3e-3, rllr=3e-4, device="cpu",
                     dtype=torch.float32)
    acc0 = tr.eval_accuracy()
    for _ in range(60):
        tr.sft_step()
    acc1 = tr.eval_accuracy()
    assert acc1 > acc0 + 0.2, (acc0, acc1)
    tr.snapshot_reference()
    for s in range(1, 6):
        st = tr.grpo_step(s)
        assert 0.0 <= st["mean_reward"] <= 1.1 and st["prefix_saved_per_prompt"] == 3 * (4 // 2)
    assert tr.eval_accuracy() >= acc1 - 0.15
