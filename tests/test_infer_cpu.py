"""Paged-KV engine on CPU (fp32): token-for-token equality with plain greedy decoding of the
PyTorch oracle under several block sizes / concurrency limits, group generation with prefix
sharing, and the block pool's reference counting (reference tests/test_infer.c:67-95)."""
import ctypes as C

import pytest
import torch

from kharon_b200 import _native
from kharon_b200.infer import InferEngine
from kharon_b200.models import GPT, Config
from kharon_b200.models.oracle import OracleGPT

CFG = Config(2, 64, 4, 97, 48, 1)


@pytest.fixture(scope="module")
def pair():
    m = GPT(CFG, "cpu", torch.float32)
    m.init_weights(1234)
    # make the logits less flat so that greedy choices are stable
    m.params.w.mul_(8.0)
    m.params.p["lnf_w"].fill_(1.0)
    for l in range(CFG.n_layer):
        m.params.p["l%d.ln1_w" % l].fill_(1.0)
        m.params.p["l%d.ln2_w" % l].fill_(1.0)
    o = OracleGPT(CFG)
    o.load_from(m)
    return m, o


def greedy(o, prompt, n_new):
    toks = list(prompt)
    with torch.no_grad():
        for _ in range(n_new):
            logits, _ = o(torch.tensor([toks]))
            toks.append(int(logits[0, -1].argmax()))
    return toks


PROMPTS = [[5, 17, 3], [9, 1, 44, 23, 8, 61, 2], [70], [11, 12, 13, 14, 15, 16, 17, 18, 19, 20, 21]]
NEW = [12, 7, 20, 9]


@pytest.mark.parametrize("bs,active", [(4, 2), (64, 4), (8, 4), (3, 1)])
def test_continuous_batching_is_token_exact(pair, bs, active):
    m, o = pair
    eng = InferEngine(m, block_size=bs, max_seqs=4)
    outs, st, ms = eng.generate(PROMPTS, NEW, max_active=active)
    for p, n, got in zip(PROMPTS, NEW, outs):
        assert got == greedy(o, p, n)
    assert st["tokens_decoded"] == sum(NEW)
    assert _native.rt().kh_eng_blocks_in_use(eng._h) == 0      # everything returned to the pool


def test_group_generate_shares_prefix_and_matches_greedy(pair):
    m, o = pair
    bs, G, plen, n_new = 4, 8, 10, 9
    prompt = PROMPTS[3][:plen]
    eng = InferEngine(m, block_size=bs, max_seqs=G + 1)
    outs, st, ms = eng.generate_group(prompt, G, n_new)
    want = greedy(o, prompt, n_new)
    assert all(x == want for x in outs)
    assert st["prefix_blocks_saved"] == (G - 1) * (plen // bs)
    # peak = shared full blocks + one private tail chain per sample, far below G full copies
    full = plen // bs
    per_seq_total = (plen + n_new + bs - 1) // bs
    assert st["blocks_peak"] <= full + G * (per_seq_total - full) + 1
    assert st["blocks_peak"] < G * per_seq_total


def test_copy_on_write_refcounts():
    lib = _native.rt()
    h = lib.kh_eng_create(4, 32, 8, 8)
    p = torch.arange(6, dtype=torch.int32)
    parent = lib.kh_eng_add(h, p.data_ptr(), 6, 0)
    I = lambda n: torch.zeros(n, dtype=torch.int32)
    tok, pos, slot, rows, ids, btab, pairs = I(64), I(64), I(64), I(8), I(8), I(64), I(64)
    nt, ns, npair = C.c_int32(), C.c_int32(), C.c_int32()
    plan = lambda: lib.kh_eng_plan(h, 8, 64, tok.data_ptr(), pos.data_ptr(), slot.data_ptr(), rows.data_ptr(),
                                   ids.data_ptr(), btab.data_ptr(), C.byref(nt), C.byref(ns), pairs.data_ptr(), 32,
                                   C.byref(npair))
    assert plan() == 0 and nt.value == 6 and ns.value == 1
    lib.kh_eng_commit(h, I(1).data_ptr(), 1)
    kids = I(3)
    assert lib.kh_eng_fork(h, parent, 3, 4, kids.data_ptr()) == 0
    b0, b1 = int(btab[0]), int(btab[1])
    assert lib.kh_eng_block_ref(h, b0) == 4 and lib.kh_eng_block_ref(h, b1) == 4
    lib.kh_eng_release(h, parent)
    assert lib.kh_eng_block_ref(h, b1) == 3
    for k in kids:
        lib.kh_eng_push(h, int(k), 7)
    assert plan() == 0 and ns.value == 3 and nt.value == 3
    # the partial block b1 is written by all three: two get private copies, the last keeps it
    assert npair.value == 2 and pairs[0] == b1 and pairs[2] == b1
    assert lib.kh_eng_block_ref(h, b1) == 1 and lib.kh_eng_block_ref(h, b0) == 3
    # pool exhaustion is an error, not a crash
    big = lib.kh_eng_create(4, 2, 4, 8)
    q = torch.arange(20, dtype=torch.int32)
    lib.kh_eng_add(big, q.data_ptr(), 20, 4)
    rc = lib.kh_eng_plan(big, 4, 64, tok.data_ptr(), pos.data_ptr(), slot.data_ptr(), rows.data_ptr(),
                         ids.data_ptr(), btab.data_ptr(), C.byref(nt), C.byref(ns), pairs.data_ptr(), 32,
                         C.byref(npair))
    assert rc == -5 and b"cannot be admitted" in lib.kh_last_error()
    lib.kh_eng_free(h); lib.kh_eng_free(big)


def test_temperature_sampling_is_seeded(pair):
    m, _ = pair
    eng = InferEngine(m, block_size=4, max_seqs=5)
    eng.set_sampling(1.0, 77)
    a, _, _ = eng.generate_group(PROMPTS[1], 4, 6)
    eng.set_sampling(1.0, 77)
    eng.step_no = 0
    b, _, _ = eng.generate_group(PROMPTS[1], 4, 6)
    assert a == b
    assert len({tuple(x) for x in a}) > 1        # samples differ from one another


def test_fresh_prompt_detection_reads_the_step_metadata():
    """The tensor-core prefill is taken only when every token of a step belongs to a prompt that is listed whole,
    contiguously and from position 0 (and is long enough to be worth a launch)."""
    import torch
    from kharon_b200.infer import InferEngine
    from kharon_b200.models import GPT, Config
    m = GPT(Config(1, 32, 2, 64, 256, 1), "cpu", torch.float32)
    m.init_weights(1)
    e = InferEngine(m, block_size=8, max_seqs=4, max_tokens=400)
    e.flash_prefill = True                     # (off on CPU; only the host-side test of the metadata is exercised)

    def fill(segments):
        pos, slot = [], []
        for s_, (p0, n) in enumerate(segments):
            pos += list(range(p0, p0 + n)); slot += [s_] * n
        e.h_meta[e._o_pos:e._o_pos + len(pos)] = torch.tensor(pos, dtype=torch.int32)
        e.h_meta[e._o_slot:e._o_slot + len(slot)] = torch.tensor(slot, dtype=torch.int32)
        return len(pos), len(segments)

    assert e._fresh_prompts(*fill([(0, 64), (0, 100), (0, 70)])) == [(0, 64), (64, 100), (164, 70)]
    assert e._fresh_prompts(*fill([(0, 64), (5, 100)])) is None          # a chunk that continues a prompt
    assert e._fresh_prompts(*fill([(0, 64), (0, 10)])) is None           # a short prompt
    assert e._fresh_prompts(*fill([(7, 1), (9, 1)])) is None             # decode step
