"""``python -m kharon_b200.bench.bench_fused ROWS N`` (default 8192 2048, reference bench/bench_fused.c:30-31):
memory-bound kernels as achieved HBM bandwidth: LayerNorm fwd/bwd, column sum, cross-entropy
(fwd+bwd in place; and the vocabulary-sliced statistics / gradient pair of the TP head), the embedding
gather and its deterministic backward, the pipeline mailbox put (looped back to local memory), AdamW."""
import json
import sys

import torch

from .. import ops
from . import l2_flush_buffer, time_ms


def main(argv=None):
    a = [int(x) for x in (sys.argv[1:] if argv is None else argv) if x.isdigit()]
    R, N = (a + [8192, 2048][len(a):])[:2]
    dev = "cuda"
    fl = l2_flush_buffer()
    x = torch.randn(R, N, device=dev).bfloat16(); y = torch.empty_like(x); dy = torch.randn_like(x); dres = torch.randn_like(x)
    w = torch.ones(N, device=dev).bfloat16(); b = torch.zeros(N, device=dev).bfloat16()
    mean = torch.empty(R, device=dev); rstd = torch.empty(R, device=dev)
    dw = torch.zeros(N, device=dev); db = torch.zeros(N, device=dev)
    part = torch.zeros(ops.layernorm_bwd_scratch_elems(R, N), device=dev)
    cs = torch.zeros(ops.colsum_scratch_elems(R, N), device=dev)
    res = {}
    t = time_ms(lambda: ops.layernorm_fwd(x, w, b, y, mean, rstd), flush=fl)
    res["layernorm_fwd_GBs"] = 2 * R * N * 2 / t / 1e6
    t = time_ms(lambda: ops.layernorm_bwd(dy, x, w, mean, rstd, dres, y, dw, db, part), flush=fl)
    res["layernorm_bwd_GBs"] = 6 * R * N * 2 / t / 1e6          # dx pass reads 3, writes 1; dw/db pass re-reads 2
    t = time_ms(lambda: ops.colsum(x, dw, True, cs), flush=fl)
    res["colsum_GBs"] = R * N * 2 / t / 1e6
    V, ld, Rv = 50257, 50304, 2048
    lg = torch.randn(Rv, ld, device=dev).bfloat16(); tgt = torch.randint(0, V, (Rv,), device=dev, dtype=torch.int32)
    rl = torch.empty(Rv, device=dev)
    t = time_ms(lambda: ops.xent(lg, V, tgt, uniform=1.0 / Rv, rowloss=rl), flush=fl)
    res["xent_fwd_bwd_GBs"] = 3 * Rv * ld * 2 / t / 1e6
    st = torch.empty(Rv, 3, device=dev); gm = torch.zeros(Rv, device=dev); gs = torch.ones(Rv, device=dev)
    Vs = (V + 1) // 2
    t = time_ms(lambda: ops.xent_stats(lg, Vs, tgt, 0, st), flush=fl)
    res["xent_stats_GBs"] = Rv * Vs * 2 / t / 1e6
    t = time_ms(lambda: ops.xent_grad(lg, Vs, tgt, 0, gm, gs, uniform=1.0 / Rv), flush=fl)
    res["xent_grad_GBs"] = 2 * Rv * Vs * 2 / t / 1e6
    # embedding: R rows of width N gathered from a [V, N] table (+ positions), and the backward into fp32
    T = 512
    tok = torch.randint(0, V, (R,), device=dev, dtype=torch.int32)
    wte = torch.randn(V, N, device=dev).bfloat16(); wpe = torch.randn(T, N, device=dev).bfloat16()
    pos = (torch.arange(R, device=dev, dtype=torch.int32) % T)
    t = time_ms(lambda: ops.embed_fwd(tok, pos, wte, wpe, y, T), flush=fl)
    res["embed_fwd_GBs"] = 3 * R * N * 2 / t / 1e6
    gwte = torch.zeros(V, N, device=dev); gwpe = torch.zeros(T, N, device=dev)
    table = torch.empty(2 * V, dtype=torch.int32, device=dev)
    t = time_ms(lambda: ops.embed_bwd(tok, dy, gwte, gwpe, R // T, T, table=table), flush=fl)
    res["embed_bwd_ms"] = t
    # pipeline mailbox put of one [2048, N] message (8 MB at N = 2048), local loop-back
    msg = torch.randn(2048, N, device=dev).bfloat16(); box = torch.empty_like(msg)
    flag = torch.zeros(1, device=dev, dtype=torch.int32); state = torch.zeros(2, device=dev, dtype=torch.int32)
    t = time_ms(lambda: ops.p2p_put(msg, box.data_ptr(), flag.data_ptr(), state), flush=fl)
    res["p2p_put_local_GBs"] = 2 * msg.numel() * 2 / t / 1e6
    n = 64 << 20
    p = torch.randn(n, device=dev); g = torch.randn(n, device=dev); m = torch.zeros(n, device=dev); v = torch.zeros(n, device=dev)
    pb = torch.empty(n, device=dev, dtype=torch.bfloat16)
    t = time_ms(lambda: ops.adamw(p, g, m, v, pb, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1, step=1), iters=10)
    res["adamw_GBs"] = n * 34 / t / 1e6
    res["rows"], res["n"] = R, N
    print(json.dumps(res))
    return res


if __name__ == "__main__":
    main()
