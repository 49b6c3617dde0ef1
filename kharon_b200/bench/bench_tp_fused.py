"""Fused compute + collective kernels against their rooflines, on the ranks torchrun started
(TP = world size; the first two ranks also act as two pipeline stages for the mailbox put):

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m kharon_b200.bench.bench_tp_fused

For every shape of the 1.2B model's row-parallel products (micro-batch rows 2048 and fused rows
16384, N = 2048, K = 1024 / 4096 per rank at TP2):

  fused      ``FusedTP.gemm_ar``: GEMM + push of the bf16 partial over NVLink + ordered reduction
  gemm       the same product alone on one GPU (no communication)
  gemm+nccl  product followed by an NCCL all-reduce on the same stream (the reference's sequence,
             src/core/gpt.c:686-687)

roofline = max(2MNK / measured bf16 peak, bytes each rank must push / 770 GB/s peer-copy rate),
where every rank pushes its whole partial tile (tp - 1 times).  Device-timed (CUDA events), max
over ranks; inputs are rewritten between calls only by the kernels themselves (working sets of
the 16384-row shapes exceed L2, the 2048-row shapes are what the pipeline path really sees:
L2-resident activations).
"""
import json
import os

import torch
import torch.distributed as dist

from .. import ops
from ..parallel.fused import FusedTP
from ..parallel.mesh import Mesh, init_distributed

LINK_GBS = 770.0


def _peak_tflops():
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        return float(json.load(open(os.path.join(root, "MEASURED_PEAKS.json")))["bf16_tflops_sustained"])
    except Exception:
        return 1400.0


def _bench(fn, dev, n=50, w=10):
    for _ in range(w):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(n):
        fn()
    e.record()
    torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e) / n * 1e3], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main():
    rank, world, dev = init_distributed()
    mesh = Mesh(world, 1, 1)
    f = FusedTP(mesh, dev)
    peak = _peak_tflops() * 1e12
    rows = []
    N = 2048
    for M in (2048, 16384):
        for K in (1024, 4096):
            a = torch.randn(M, K, device=dev).bfloat16()
            b = (torch.randn(N, K, device=dev) * 0.05).bfloat16()
            out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
            bias = torch.zeros(N, device=dev).bfloat16()
            res = torch.zeros(M, N, device=dev).bfloat16()
            t_f = _bench(lambda: f.gemm_ar(a, b, out, bias=bias, resid=res), dev)
            t_g = _bench(lambda: ops.gemm(a, b, out, epi=ops.EPI_BIAS_RESID, bias=bias, aux=res), dev)
            t_n = _bench(lambda: (ops.gemm(a, b, out, epi=ops.EPI_BIAS_RESID, bias=bias, aux=res), dist.all_reduce(out)), dev)
            t_c = 2.0 * M * N * K / peak * 1e6
            t_l = (world - 1) * M * N * 2 / (LINK_GBS * 1e3)
            roof = max(t_c, t_l)
            rows.append(dict(op="gemm_ar", M=M, N=N, K=K, fused_us=round(t_f, 1), gemm_us=round(t_g, 1),
                             gemm_nccl_us=round(t_n, 1), compute_floor_us=round(t_c, 1), link_floor_us=round(t_l, 1),
                             roofline_frac=round(roof / t_f, 3)))
            # reduce-scatter form: every rank receives and reduces only its row block
            shard = torch.empty(M // world, N, device=dev, dtype=torch.bfloat16)
            t_rs = _bench(lambda: f.gemm_rs(a, b, shard, bias=bias, resid=res[:M // world]), dev)
            t_l2 = (world - 1) / world * M * N * 2 / (LINK_GBS * 1e3)
            rows.append(dict(op="gemm_rs", M=M, N=N, K=K, fused_us=round(t_rs, 1), compute_floor_us=round(t_c, 1),
                             link_floor_us=round(t_l2, 1), roofline_frac=round(max(t_c, t_l2) / t_rs, 3)))
    # all-gather -> GEMM: A rows live in the ranks' shards, remote tiles come in by TMA
    for M, K, Ng in ((2048, 2048, 3072), (16384, 2048, 3072)):
        sh, ptrs, h = f.symmetric_rows(M // world, K)
        sh.copy_(torch.randn(M // world, K, device=dev).bfloat16())
        w = (torch.randn(Ng, K, device=dev) * 0.05).bfloat16()
        out = torch.empty(M, Ng, device=dev, dtype=torch.bfloat16)
        torch.cuda.synchronize()
        dist.barrier()
        t_ag = _bench(lambda: f.ag_gemm(ptrs, K, M // world, w, out), dev)
        full = torch.randn(M, K, device=dev).bfloat16()
        t_g = _bench(lambda: ops.gemm(full, w, out), dev)
        t_c = 2.0 * M * Ng * K / peak * 1e6
        t_l = (world - 1) / world * M * K * 2 / (LINK_GBS * 1e3)
        rows.append(dict(op="ag_gemm", M=M, N=Ng, K=K, fused_us=round(t_ag, 1), gemm_us=round(t_g, 1),
                         compute_floor_us=round(t_c, 1), link_floor_us=round(t_l, 1),
                         roofline_frac=round(max(t_c, t_l) / t_ag, 3)))
    # pipeline mailbox: one [2048, 2048] bf16 activation from rank 0 into rank 1's memory
    if world >= 2:
        import torch.distributed._symmetric_memory as symm_mem
        nbytes = 2048 * 2048 * 2
        buf = symm_mem.empty(nbytes + 256, dtype=torch.uint8, device=dev)
        hh = symm_mem.rendezvous(buf, mesh.tp_group.group_name)
        buf.zero_()
        torch.cuda.synchronize()
        hh.barrier()
        peer = int(hh.buffer_ptrs[(rank + 1) % world])
        msg = torch.randn(2048, 2048, device=dev).bfloat16()
        state = torch.zeros(2, device=dev, dtype=torch.int32)
        t_p = _bench(lambda: ops.p2p_put(msg, peer, peer + nbytes, state), dev)
        rows.append(dict(op="p2p_put", bytes=nbytes, us=round(t_p, 1), GBs=round(nbytes / t_p / 1e3, 1),
                         roofline_frac=round(nbytes / t_p / 1e3 / LINK_GBS, 3)))
        torch.cuda.synchronize()
        dist.barrier()
    word = ops.error_word()
    if rank == 0:
        print(json.dumps(dict(world=world, peak_tflops=peak / 1e12, link_GBs=LINK_GBS, error_word=word, rows=rows)))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
