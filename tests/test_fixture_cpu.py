"""The CHRN fixture path end to end (reference tests test_loadref / test_forward / test_backward /
test_step): generate m1_ref.bin from the PyTorch oracle, load it through the native reader into the
framework model, and reproduce logits, loss, every gradient and the post-AdamW parameters.  Plus the
sharding identities of test_tp1 / test_zero."""
import torch

from kharon_b200 import ops
from kharon_b200.models import GPT, Config
from kharon_b200.utils import chrn, gen_fixtures


def test_fixture_forward_backward_step(tmp_path):
    path = gen_fixtures.main([str(tmp_path / "m1_ref.bin")])
    cfg_l, opt, t = chrn.load(path)
    cfg = Config(*cfg_l)
    assert cfg == gen_fixtures.CFG and abs(opt[4] - 0.1) < 1e-7
    m = GPT(cfg, "cpu", torch.float32)
    m.load_ref(t)
    m.set_input(t["input_ids"].reshape(-1), t["targets"].reshape(-1))
    m.forward()
    assert torch.allclose(m.slots[0].logits[:, :cfg.vocab], t["logits"].view(-1, cfg.vocab), rtol=1e-4, atol=1e-5)
    assert abs(m.loss() - t["loss"].item()) < 1e-5
    m.backward()
    for n in m.params.names:
        assert torch.allclose(m.params.grad[n], t[gen_fixtures.fixture_name(n) + ".grad"].view_as(m.params.grad[n]),
                              rtol=1e-4, atol=1e-5), n
    m.adamw_step(opt[0], opt[1], opt[2], opt[3], opt[4])
    for n in m.params.names:
        assert torch.allclose(m.params.p[n], t[gen_fixtures.fixture_name(n) + ".step"].view_as(m.params.p[n]),
                              rtol=1e-4, atol=3e-5), n


def test_sharded_adamw_is_bit_identical_to_unsharded():
    """ZeRO-1 slices of the flat arena, padding included (reference tests/test_zero.c:17-61)."""
    torch.manual_seed(0)
    n = 10007
    p0, g0 = torch.randn(n), torch.randn(n)
    kw = dict(lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1)
    ref_p, ref_m, ref_v = p0.clone(), torch.zeros(n), torch.zeros(n)
    for step in (1, 2, 3):
        ops.adamw(ref_p, g0.clone(), ref_m, ref_v, None, step=step, **kw)
    for dp in (2, 4, 8):
        npad = (n + dp - 1) // dp * dp
        p = torch.zeros(npad); p[:n] = p0
        g = torch.zeros(npad); g[:n] = g0
        m, v = torch.zeros(npad), torch.zeros(npad)
        sh = npad // dp
        for step in (1, 2, 3):
            for r in range(dp):
                sl = slice(r * sh, (r + 1) * sh)
                ops.adamw(p[sl], g[sl].clone(), m[sl], v[sl], None, step=step, **kw)
        assert torch.equal(p[:n], ref_p) and torch.equal(m[:n], ref_m) and torch.equal(v[:n], ref_v)
        assert p[n:].abs().sum().item() == 0


def test_tp_seam_with_one_rank_is_bit_identical():
    """The TP code path with tp = 1 and an identity all-reduce equals the plain path to the bit
    (reference tests/test_tp1.c:15-33)."""
    from kharon_b200.utils.rng import Rng
    cfg = Config(2, 64, 4, 256, 16, 4)
    idx, tgt = Rng(2).batch(cfg.batch * cfg.seq, cfg.vocab)
    out = []
    for seam in (False, True):
        m = GPT(cfg, "cpu", torch.bfloat16, tp=1, tp_rank=0)
        m.init_weights(1337)
        if seam:
            m.tp_allreduce = lambda t: t
        m.set_input(idx, tgt)
        m.forward()
        m.backward()
        out.append((m.loss(), m.params.g.clone()))
    assert out[0][0] == out[1][0] and torch.equal(out[0][1], out[1][1])
