"""``python -m kharon_b200.bench.bench_bf16 M N K`` (default 8192 8192 2048, reference bench/bench_bf16.c:11-13):
the tcgen05 bf16 GEMM against torch.matmul (cuBLAS) in bf16 and fp32; relative Frobenius error vs fp32."""
import json
import sys

import torch

from .. import ops
from . import l2_flush_buffer, time_ms


def main(argv=None):
    a = [int(x) for x in (sys.argv[1:] if argv is None else argv) if x.isdigit()]
    M, N, K = (a + [8192, 8192, 2048][len(a):])[:3]
    dev = "cuda"
    x = torch.randn(M, K, device=dev)
    w = torch.randn(N, K, device=dev)
    xb, wb = x.bfloat16(), w.bfloat16()
    out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    fl = l2_flush_buffer() if (M * K + N * K + M * N) * 2 < (126 << 20) else None
    t_ours = time_ms(lambda: ops.gemm(xb, wb, out), flush=fl)
    t_cublas = time_ms(lambda: torch.matmul(xb, wb.t()), flush=fl)
    t_fp32 = time_ms(lambda: torch.matmul(x, w.t()), iters=5, flush=fl)
    ref = x @ w.t()
    err = ((out.float() - ref).norm() / ref.norm()).item()
    fl_ = 2.0 * M * N * K
    res = dict(M=M, N=N, K=K, ours_ms=t_ours, ours_tflops=fl_ / t_ours / 1e9, cublas_bf16_tflops=fl_ / t_cublas / 1e9,
               fp32_tflops=fl_ / t_fp32 / 1e9, speedup_vs_fp32=t_fp32 / t_ours, rel_frobenius=err,
               l2="flushed between iterations" if fl is not None else "operands larger than L2")
    print(json.dumps(res))
    return res


if __name__ == "__main__":
    main()
