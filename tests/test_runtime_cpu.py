"""Host runtime: RNG stream, layout, data loader, CKP1/CHRN IO, GRPO math, 1F1B schedule."""
import os
import struct

import pytest
import torch

from kharon_b200 import _native
from kharon_b200.engine import pp_schedule, pp_num_slots
from kharon_b200.models import Config, GPT
from kharon_b200.models.layout import layout, n_params
from kharon_b200.utils import chrn, ckpt
from kharon_b200.utils.rng import Rng, ByteData


def test_xorshift_matches_python_statement():
    def u32(s):
        s ^= s >> 12
        s ^= (s << 25) & 0xFFFFFFFFFFFFFFFF
        s ^= s >> 27
        return s, ((s * 0x2545F4914F6CDD1D) & 0xFFFFFFFFFFFFFFFF) >> 32
    r = Rng(1337)
    s = 1337
    for _ in range(100):
        s, want = u32(s)
        assert r.u32() == want
    assert r.state == s
    assert Rng(0).state == 0x9E3779B97F4A7C15


def test_batch_and_normal_stream():
    a, b = Rng(5), Rng(5)
    idx, tgt = a.batch(64, 50257)
    assert idx.max() < 50257 and idx.min() >= 0
    i2, t2 = b.batch(64, 50257)
    assert torch.equal(idx, i2) and torch.equal(tgt, t2)
    x = Rng(9).normal(200000, 0.02)
    assert abs(x.mean().item()) < 2e-4 and abs(x.std().item() - 0.02) < 2e-4
    # block slicing consumes the same stream as the full draw
    full = Rng(3).normal(6 * 8, 1.0).view(6, 8)
    r = Rng(3)
    blk = r.normal_block(6, 8, 2, 5, 1, 4, 1.0)
    assert torch.equal(blk, full[2:5, 1:4])
    r2 = Rng(3); r2.normal(48, 1.0)
    assert r.state == r2.state


def test_layout_is_256_byte_aligned_and_counts_params():
    cfg = Config(2, 64, 4, 256, 32, 4)
    names, offs, nums, total = layout(cfg, 1, False, 4)
    assert all(o % 256 == 0 for o in offs)
    assert sum(nums) == n_params(cfg) == 118528
    assert offs[1] == 256 * 64 * 4 and names[2] == "l0.ln1_w"
    cfg = Config(2, 128, 4, 256, 64, 8)
    assert sum(layout(cfg, 1, False, 4)[2]) == 437760
    # TP shards: qkv rows / proj cols / fc rows / fcproj cols
    _, _, nums2, _ = layout(cfg, 2, False, 4)
    assert nums2[names.index("l0.qkv_w")] == 3 * 128 * 128 // 2
    with pytest.raises(_native.NativeError):
        layout(Config(2, 130, 4, 256, 64, 8), 4, False, 4)


def test_byte_loader_windows(tmp_path):
    p = tmp_path / "c.bin"
    p.write_bytes(bytes(range(256)) * 8)
    d = ByteData(str(p), 3, 16, 42)
    idx = torch.empty(48, dtype=torch.int32); tgt = torch.empty(48, dtype=torch.int32)
    d.next_into(idx, tgt)
    assert torch.equal(idx.view(3, 16)[:, 1:], tgt.view(3, 16)[:, :-1])
    r = Rng(42)
    o = r.u32() % (2048 - 16 - 1)
    assert idx[0].item() == o % 256


def test_ckpt_layout_and_errors(tmp_path):
    cfg = Config(2, 64, 4, 256, 32, 4)
    m = GPT(cfg, "cpu", torch.float32)
    m.init_weights(1337)
    m.params.m.normal_(); m.params.v.uniform_()
    m.step = 17
    path = str(tmp_path / "a.ckpt")
    m.save(path, rng_state=0xDEADBEEF12345678)
    raw = open(path, "rb").read()
    assert raw[:4] == b"CKP1"
    assert struct.unpack("<6i", raw[4:28]) == tuple(cfg.as_list())
    step, rng, pb, ob = struct.unpack("<iQQQ", raw[28:56])
    assert (step, rng, pb, ob) == (17, 0xDEADBEEF12345678, m.params.param_bytes, m.params.param_bytes)
    assert len(raw) == 56 + 3 * pb
    # the param block is the arena itself: wte first, wpe at the next 256-byte boundary
    wte = torch.frombuffer(bytearray(raw[56:56 + 256 * 64 * 4]), dtype=torch.float32)
    assert torch.equal(wte, m.params.p["wte"].flatten())
    m2 = GPT(cfg, "cpu", torch.float32)
    assert m2.load(path) == 0xDEADBEEF12345678 and m2.step == 17
    assert torch.equal(m2.params.w, m.params.w) and torch.equal(m2.params.v, m.params.v)
    # failure detection on the host: wrong config, truncated file, bad magic -> clean errors
    with pytest.raises(_native.NativeError, match="config mismatch"):
        GPT(Config(2, 64, 4, 256, 32, 8), "cpu", torch.float32).load(path)
    open(str(tmp_path / "t.ckpt"), "wb").write(raw[:1000])
    before = m2.params.w.clone()
    with pytest.raises(_native.NativeError, match="truncated"):
        m2.load(str(tmp_path / "t.ckpt"))
    assert torch.equal(before, m2.params.w)          # live buffers untouched by a failed load
    open(str(tmp_path / "b.ckpt"), "wb").write(b"NOPE" + raw[4:])
    with pytest.raises(_native.NativeError, match="bad magic"):
        m2.load(str(tmp_path / "b.ckpt"))
    with pytest.raises(_native.NativeError, match="cannot open"):
        m2.load(str(tmp_path / "missing.ckpt"))


def test_chrn_roundtrip(tmp_path):
    p = str(tmp_path / "f.bin")
    w = chrn.Writer(p, [2, 128, 4, 256, 64, 8], [3e-4, 0.9, 0.95, 1e-8, 0.1])
    a = torch.randn(3, 5); b = torch.arange(12).view(3, 4)
    w.put("a", a); w.put("ids", b); w.put("loss", 1.25)
    w.close()
    cfg, opt, t = chrn.load(p)
    assert cfg == [2, 128, 4, 256, 64, 8] and abs(opt[0] - 3e-4) < 1e-9
    assert torch.equal(t["a"], a) and torch.equal(t["ids"], b.int()) and t["loss"].item() == 1.25
    with pytest.raises(_native.NativeError):
        chrn.load(str(tmp_path / "nope.bin"))


def test_grpo_advantages_and_coef():
    import ctypes as C
    lib = _native.rt()
    r = torch.tensor([1.0, 0.0, 0.0, 1.0, 1.0, 1.0, 1.0, 1.0])
    adv = torch.empty(8)
    lib.kh_grpo_advantages(r.data_ptr(), 2, 4, 1e-4, adv.data_ptr())
    g0 = r[:4]
    want = (g0 - g0.mean()) / (g0.std(unbiased=False) + 1e-4)
    assert torch.allclose(adv[:4], want, atol=1e-6)
    assert adv[4:].abs().max().item() == 0
    rows, T = 2, 6
    pc = torch.rand(rows, T) * 0.5 + 0.1; pr = torch.rand(rows, T) * 0.5 + 0.1
    a = torch.tensor([0.5, -1.0]); coef = torch.empty(rows, T)
    lib.kh_grpo_coef(a.data_ptr(), pc.data_ptr(), pr.data_ptr(), rows, T, 2, 4, 0.04, coef.data_ptr())
    want = torch.zeros(rows, T)
    want[:, 2:5] = (a[:, None] - 0.04 * (1 - pr[:, 2:5] / pc[:, 2:5])) / 6
    assert torch.allclose(coef, want, atol=1e-6)


@pytest.mark.parametrize("P,M", [(1, 4), (2, 8), (4, 8), (4, 4), (3, 5)])
def test_1f1b_schedule_is_consistent(P, M):
    from kharon_b200.engine import (PP_FWD, PP_BWD, PP_SEND_ACT, PP_RECV_ACT, PP_SEND_GRAD, PP_RECV_GRAD,
                                    PP_SEND_ACT_RECV_GRAD, PP_SEND_GRAD_RECV_ACT)
    scheds = [pp_schedule(s, P, M) for s in range(P)]
    for s, ops_ in enumerate(scheds):
        f = [a0 for op, a0, _ in ops_ if op == PP_FWD]
        b = [a0 for op, a0, _ in ops_ if op == PP_BWD]
        assert f == list(range(M)) and b == list(range(M))
        nslots = pp_num_slots(s, P, M)
        assert nslots == min(P - 1 - s, M) + 1
        live = set()
        for op, a0, a1 in ops_:
            if op == PP_FWD:
                assert a1 == a0 % nslots and a1 not in live
                live.add(a1)
            elif op == PP_BWD:
                live.discard(a1)
    # message matching: simulate with blocking semantics (a fused exchange posts both sides at once)
    pc = [0] * P
    chan = {}
    def sends(op):
        return {PP_SEND_ACT: [("a", +1)], PP_SEND_GRAD: [("g", -1)], PP_SEND_ACT_RECV_GRAD: [("a", +1)],
                PP_SEND_GRAD_RECV_ACT: [("g", -1)]}.get(op, [])
    def recvs(op):
        return {PP_RECV_ACT: [("a", -1)], PP_RECV_GRAD: [("g", +1)], PP_SEND_ACT_RECV_GRAD: [("g", +1)],
                PP_SEND_GRAD_RECV_ACT: [("a", -1)]}.get(op, [])
    posted = [False] * P
    for _ in range(100000):
        progressed = False
        for s in range(P):
            if pc[s] >= len(scheds[s]):
                continue
            op = scheds[s][pc[s]][0]
            if not posted[s]:
                for kind, dirn in sends(op):
                    chan.setdefault((kind, s, s + dirn), []).append(1)
                posted[s] = True
            ok = all(chan.get((kind, s + dirn, s), []) for kind, dirn in recvs(op))
            if ok:
                for kind, dirn in recvs(op):
                    chan[(kind, s + dirn, s)].pop()
                pc[s] += 1
                posted[s] = False
                progressed = True
        if all(pc[s] >= len(scheds[s]) for s in range(P)):
            break
        assert progressed, "pipeline schedule deadlocks"
    assert all(not v for v in chan.values())


def test_deferred_pipeline_schedule_is_consistent():
    """Every micro-batch: receive -> forward -> send, receive grad -> backward -> send grad, each
    once and in that order; the weight-gradient passes cover [0, M) once, only over finished
    micro-batches; stages agree on the order of the messages they exchange."""
    from kharon_b200.engine import (pp_schedule_deferred, PP_FWD, PP_BWD, PP_FLUSH_DW, PP_RECV_ACT, PP_SEND_ACT,
                                    PP_RECV_GRAD, PP_SEND_GRAD)
    for P, M in [(1, 4), (2, 8), (4, 8), (3, 5), (2, 2), (4, 2)]:
        scheds = [pp_schedule_deferred(s, P, M) for s in range(P)]
        for s, sc in enumerate(scheds):
            f = [a for op, a, _ in sc if op == PP_FWD]
            b = [a for op, a, _ in sc if op == PP_BWD]
            assert f == list(range(M)) and b == list(range(M))
            done_b, covered = set(), []
            pos = {}
            for k, (op, a0, a1) in enumerate(sc):
                pos[(op, a0)] = k
                if op == PP_BWD:
                    assert (PP_FWD, a0) in pos
                    done_b.add(a0)
                if op == PP_FLUSH_DW:
                    assert all(i in done_b for i in range(a0, a1))
                    covered += list(range(a0, a1))
            assert covered == list(range(M))
            for i in range(M):
                if s > 0:
                    assert pos[(PP_RECV_ACT, i)] < pos[(PP_FWD, i)] and pos[(PP_BWD, i)] < pos[(PP_SEND_GRAD, i)]
                if s < P - 1:
                    assert pos[(PP_FWD, i)] < pos[(PP_SEND_ACT, i)] and pos[(PP_RECV_GRAD, i)] < pos[(PP_BWD, i)]
            # in-flight forwards never exceed the micro-batch slots
            assert len(sc) < 8 * (M + P) + 16


def test_cli_flags_accept_the_torchrun_safe_spelling():
    from kharon_b200.utils.cli import Flags
    f = Flags(["--layers", "3", "--kh-d", "96", "--kh-log", "7", "--synthetic", "--lr", "1e-3"])
    assert f.int("layers", 8) == 3 and f.int("d", 512) == 96 and f.int("log", 50) == 7
    assert f.has("synthetic") and not f.has("resume") and f.float("lr", 3e-4) == 1e-3
    assert f.int("heads", 8) == 8


def test_milestone_script_parses():
    import os
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sh = os.path.join(root, "kharon_b200", "bench", "milestones.sh")
    assert subprocess.run(["bash", "-n", sh]).returncode == 0
    out = subprocess.run(["bash", sh, "nosuchjob"], capture_output=True, text=True)
    assert out.returncode == 2 and "usage" in out.stdout
