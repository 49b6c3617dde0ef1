"""``python -m kharon_b200.bench.bench_fused ROWS N`` (default 8192 2048, reference bench/bench_fused.c:30-31):
memory-bound kernels as achieved HBM bandwidth: LayerNorm fwd/bwd, column sum, cross-entropy
(fwd+bwd in place), AdamW."""
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
