"""GPU integration: the bf16 model on the native kernels against the fp32 CPU evaluation of the
same weights (reference tests/test_bf16fwd.c, test_bf16step.c) and the training engine."""
import pytest
import torch

from kharon_b200 import ops
from kharon_b200.models import GPT, Config
from kharon_b200.utils.rng import Rng

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("cfg", [Config(2, 128, 2, 256, 64, 4), Config(2, 256, 2, 1000, 128, 2)])
def test_bf16_gpu_forward_backward_vs_fp32_cpu(cfg):
    ref = GPT(cfg, "cpu", torch.float32)
    ref.init_weights(1337)
    gpu = GPT(cfg, "cuda", torch.bfloat16)
    gpu.init_weights(1337)
    idx, tgt = Rng(5).batch(cfg.batch * cfg.seq, cfg.vocab)
    for m in (ref, gpu):
        m.set_input(idx.to(m.device), tgt.to(m.device))
        m.forward()
    assert abs(gpu.loss() - ref.loss()) < 2e-2
    a = gpu.slots[0].logits[:, :cfg.vocab].float().cpu()
    b = ref.slots[0].logits[:, :cfg.vocab]
    assert torch.allclose(a, b, rtol=2e-2, atol=2e-2)
    ref.backward()
    gpu.backward()
    torch.cuda.synchronize()
    assert ops.error_word() == 0
    g, r = gpu.params.g.cpu(), ref.params.g
    assert ((g - r).norm() / r.norm()).item() < 3e-2
    for n in ("wte", "wpe", "l0.qkv_w", "l0.qkv_b", "l1.fcproj_w", "l1.ln2_w", "lnf_b", "l0.proj_b", "l0.fc_b"):
        gg, rr = gpu.params.grad[n].cpu(), ref.params.grad[n]
        assert ((gg - rr).norm() / (rr.norm() + 1e-12)).item() < 5e-2, n


def test_engine_overfits_and_microbatch_fusion_agrees():
    from kharon_b200.engine import TrainEngine
    kw = dict(layers=2, d_model=128, heads=2, vocab=512, seq=64, mbatch=2, n_micro=4, device="cuda", lr=3e-3, wd=0.0)
    a = TrainEngine(**kw)
    b = TrainEngine(fuse_microbatches=True, **kw)
    idx, tgt = Rng(9).batch(a.tokens_per_step, 512)
    la, lb = [], []
    for _ in range(20):
        a.train_step(idx, tgt); la.append(a.loss())
        b.train_step(idx, tgt); lb.append(b.loss())
    assert la[-1] < 0.6 * la[0]
    assert abs(la[0] - lb[0]) < 1e-2 and abs(la[-1] - lb[-1]) < 0.15
    assert ops.error_word() == 0


def test_gpu_run_is_bitwise_reproducible():
    """Two identical runs produce identical loss bits and parameters (no atomics anywhere)."""
    from kharon_b200.engine import TrainEngine
    outs = []
    for _ in range(2):
        e = TrainEngine(layers=2, d_model=128, heads=2, vocab=300, seq=64, mbatch=2, n_micro=2, device="cuda")
        idx, tgt = Rng(11).batch(e.tokens_per_step, 300)
        for _ in range(4):
            e.train_step(idx, tgt)
        outs.append((e.loss(), e.model.params.w.clone()))
    assert outs[0][0] == outs[1][0]
    assert torch.equal(outs[0][1], outs[1][1])


def test_gpu_checkpoint_resume_is_bit_exact(tmp_path):
    """bf16 training on the GPU: 12 uninterrupted steps == 6 steps + CKP1 file + fresh engine + 6
    steps, to the bit (loss and every parameter), through the public trainer entry point."""
    from kharon_b200 import train

    def run(name, steps, resume=False):
        argv = ["--layers", "2", "--d", "128", "--heads", "2", "--seq", "64", "--batch", "4", "--steps", str(steps),
                "--log", "1000", "--ckptevery", "0", "--ckpt", str(tmp_path / name), "--synthetic", "--vocab", "1000",
                "--device", "cuda"]
        return train.main(argv + (["--resume"] if resume else []))

    full = run("full.ckpt", 12)
    run("half.ckpt", 6)
    res = run("half.ckpt", 12, resume=True)
    assert res.model.step == 12 and res.loss() == full.loss()
    assert torch.equal(res.model.params.w, full.model.params.w)
    assert torch.equal(res.model.params.wb, full.model.params.wb)
    assert torch.equal(res.model.params.v, full.model.params.v)


def test_fp32_gpu_step_matches_fp32_cpu():
    """fp32 model on the GPU (the oracle configuration: PyTorch fp32 operators + the native fp32
    product) against the same model on the CPU: loss, gradients and one AdamW step."""
    cfg = Config(2, 128, 4, 256, 64, 4)
    ms = []
    for dev in ("cpu", "cuda"):
        m = GPT(cfg, dev, torch.float32)
        m.init_weights(1337)
        idx, tgt = Rng(5).batch(cfg.batch * cfg.seq, cfg.vocab)
        m.set_input(idx.to(m.device), tgt.to(m.device))
        m.forward()
        m.backward()
        ms.append(m)
    cpu, gpu = ms
    assert abs(cpu.loss() - gpu.loss()) < 1e-5
    assert torch.allclose(gpu.params.g.cpu(), cpu.params.g, rtol=1e-4, atol=1e-6)
    for m in ms:
        m.adamw_step(3e-4)
    assert torch.allclose(gpu.params.w.cpu(), cpu.params.w, rtol=1e-4, atol=3e-5)


def test_two_stream_step_is_independent_of_stream_priorities():
    """Race smoke test of the multi-stream step (optimizer buckets on a side stream under the backward pass,
    input staging on a copy stream): the same run with the side streams at the opposite priority, and with
    the optimizer kept on the compute stream, must give identical bits."""
    from kharon_b200.engine import TrainEngine
    outs = []
    for variant in ("default", "high_priority_side_streams", "single_stream"):
        e = TrainEngine(layers=3, d_model=128, heads=2, vocab=300, seq=64, mbatch=2, n_micro=2, device="cuda",
                        bucket_optimizer=variant != "single_stream")
        assert e.bucketed == (variant != "single_stream")
        if variant == "high_priority_side_streams":
            e.opt_stream = torch.cuda.Stream(e.device, priority=-1)
            e.copy_stream = torch.cuda.Stream(e.device, priority=-1)
        idx, tgt = Rng(11).batch(e.tokens_per_step, 300)
        hi, ht = idx.pin_memory(), tgt.pin_memory()
        for _ in range(5):
            e.train_step(hi, ht)
        outs.append((e.loss(), e.model.params.w.clone(), e.model.params.wb.clone()))
    for o in outs[1:]:
        assert o[0] == outs[0][0]
        assert torch.equal(o[1], outs[0][1]) and torch.equal(o[2], outs[0][2])
