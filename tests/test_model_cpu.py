"""CPU oracle tier: the explicit forward/backward/AdamW of the framework model in fp32 against
PyTorch autograd (reference tests test_forward / test_backward / test_step / test_bf16fwd /
test_bf16step, tests/*.c), on BASELINE config 1 (L2 d64 h4 V256 seq32 batch4)."""
import torch

from kharon_b200.models import GPT, Config
from kharon_b200.models.oracle import OracleGPT
from kharon_b200.utils.rng import Rng

CFG = Config(2, 64, 4, 256, 32, 4)


def _pair(cfg=CFG, dtype=torch.float32, seed=1337):
    m = GPT(cfg, "cpu", dtype)
    m.init_weights(seed)
    o = OracleGPT(cfg)
    o.load_from(m)
    idx, tgt = Rng(7).batch(cfg.batch * cfg.seq, cfg.vocab)
    return m, o, idx, tgt


def test_forward_logits_and_loss_match_autograd():
    m, o, idx, tgt = _pair()
    m.set_input(idx, tgt)
    m.forward()
    logits, loss = o(idx.long().view(CFG.batch, CFG.seq), tgt.long().view(CFG.batch, CFG.seq))
    got = m.slots[0].logits[:, :CFG.vocab]
    assert torch.allclose(got, logits.view(-1, CFG.vocab), rtol=1e-4, atol=1e-5)
    assert abs(m.loss() - loss.item()) < 1e-5


def test_backward_every_parameter_matches_autograd():
    m, o, idx, tgt = _pair()
    m.set_input(idx, tgt)
    m.forward()
    m.backward()
    _, loss = o(idx.long().view(CFG.batch, CFG.seq), tgt.long().view(CFG.batch, CFG.seq))
    loss.backward()
    for n, p in o.named_tensors().items():
        assert torch.allclose(m.params.grad[n], p.grad, rtol=1e-4, atol=1e-5), n


def test_adamw_step_matches_torch_optim():
    m, o, idx, tgt = _pair()
    opt = torch.optim.AdamW(o.parameters(), lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for _ in range(3):
        m.set_input(idx, tgt)
        m.forward()
        m.backward()
        m.adamw_step(3e-4, 0.9, 0.95, 1e-8, 0.1)
        opt.zero_grad()
        _, loss = o(idx.long().view(CFG.batch, CFG.seq), tgt.long().view(CFG.batch, CFG.seq))
        loss.backward()
        opt.step()
    for n, p in o.named_tensors().items():
        assert torch.allclose(m.params.p[n], p.data, rtol=1e-4, atol=3e-5), n
    assert m.params.g.abs().max().item() == 0


def test_bf16_forward_close_to_fp32_and_overfits():
    m32, o, idx, tgt = _pair()
    mb = GPT(CFG, "cpu", torch.bfloat16)
    mb.init_weights(1337)
    for mm in (m32, mb):
        mm.set_input(idx, tgt)
        mm.forward()
    assert abs(mb.loss() - m32.loss()) < 2e-2
    a = mb.slots[0].logits[:, :CFG.vocab].float()
    b = m32.slots[0].logits[:, :CFG.vocab]
    assert torch.allclose(a, b, rtol=2e-2, atol=2e-2)
    # gradients: relative Frobenius error of bf16 vs fp32, then overfit one batch
    m32.backward()
    mb.backward()
    num = (mb.params.g - m32.params.g).norm()
    assert (num / m32.params.g.norm()).item() < 3e-2
    first = mb.loss()
    for _ in range(30):
        mb.set_input(idx, tgt)
        mb.forward(compute_loss=False)
        mb.backward(loss_scale=1.0)
        mb.adamw_step(1e-2, 0.9, 0.95, 1e-8, 0.0)
    assert mb.loss() < 0.5 * first


def test_microbatch_accumulation_equals_one_big_batch():
    """Two half batches with inv_mb = 1/2 accumulate to the gradient of the full batch
    (reference tests/test_pp1.c:16-49)."""
    cfg2 = Config(2, 64, 4, 256, 32, 2)
    full, _, idx, tgt = _pair()
    full.set_input(idx, tgt)
    full.forward()
    full.backward()
    half = GPT(cfg2, "cpu", torch.float32)
    half.init_weights(1337)
    n = cfg2.batch * cfg2.seq
    for k in range(2):
        half.set_input(idx[k * n:(k + 1) * n], tgt[k * n:(k + 1) * n])
        half.forward(compute_loss=False)
        half.backward(inv_mb=0.5, loss_scale=0.5, accumulate_loss=k > 0)
    assert torch.allclose(half.params.g, full.params.g, rtol=1e-4, atol=1e-6)
    assert abs(half.loss() - full.loss()) < 1e-5
