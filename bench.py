#!/usr/bin/env python
"""Headline benchmark: training throughput of the 1.2B GPT (24 layers, d 2048, 16 heads, MLP
8192, tied vocab 50257, seq 512, micro-batch 4, M = 8 micro-batches per replica and step;
bf16 compute, fp32 master + AdamW), the configuration of the reference's 3-D-parallel run
(scripts/ice_m7_3d.sbatch:35-36, bench/results.json:34).

    python bench.py --gpus N --steps K --warmup W            # one rank per GPU under torchrun for N > 1
    python bench.py --impl reference ...                     # the unmodified reference, same metric

Mesh per GPU count (override with --tp/--pp/--dp): 1 -> single GPU, 2 -> TP2, 4 -> TP2 x PP2,
8 -> TP2 x PP2 x ZeRO-1 DP2 (the named configuration).  Rank 0 prints one JSON line.

Two timed regions of K steps each, both on the device with CUDA events between barriers,
maximum over ranks:
  value   inputs already resident on the device (kernel-only figure)
  e2e     TrainEngine.train_step fed from pinned host memory every step and the loss read
          back to the host every step (what a user of the API sees)

Further keys of the line:
  fused_check         (N > 1) every in-kernel collective the mesh uses, run on small problems on
                      these ranks before the timed region and compared with NCCL / PyTorch
                      (kharon_b200/parallel/selfcheck.py); a failure makes the exit code non-zero
  at_reference_shape  the same engine and mesh with the shape the reference binary hard-codes
                      (vocab 256, untied head, src/pp_train.c:77), for a like-for-like ratio
  decode              paged-KV decode tok/s of the 24-layer d1024 model at G = 1 / 8 / 32 on one GPU
                      (rank 0; BASELINE's second metric), KV bytes paged vs full-sequence
Skip the extras with --no-extras.
"""
from __future__ import annotations

import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

PUBLISHED_TOK_S = 30549.0     # 8x L40S, bench/results.json:34 of the reference


def arg(name, default, conv=int):
    key = "--" + name
    if key in sys.argv:
        i = sys.argv.index(key)
        if i + 1 < len(sys.argv):
            return conv(sys.argv[i + 1])
    return default


def default_mesh(n):
    return {1: (1, 1, 1), 2: (2, 1, 1), 4: (2, 2, 1), 8: (2, 2, 2)}.get(n, (1, 1, n))


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 200 ms while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.p = None
        self.idx = gpu_index
        try:
            self.p = subprocess.Popen(["nvidia-smi", "-i", str(gpu_index), "--query-gpu=" + self.Q,
                                       "--format=csv,noheader,nounits", "-lms", "200"], stdout=subprocess.PIPE,
                                      stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.p = None

    def stop(self):
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.p.terminate()
        try:
            out, _ = self.p.communicate(timeout=5)
        except Exception:
            self.p.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def run_ours():
    import torch
    import torch.distributed as dist
    from kharon_b200 import ops
    from kharon_b200.engine import TrainEngine
    from kharon_b200.models.layout import matmul_params
    from kharon_b200.parallel.mesh import Mesh, init_distributed
    from kharon_b200.utils.rng import Rng

    n = arg("gpus", 1)
    K, W = arg("steps", 10), max(arg("warmup", 3), 3)
    rank, world, device = init_distributed()
    if world != n:
        if rank == 0:
            print(json.dumps({"error": "--gpus %d but WORLD_SIZE=%d: launch with torchrun --nproc-per-node %d" % (n, world, n)}))
        return 1
    tp0, pp0, dp0 = default_mesh(n)
    tp, pp, dp = arg("tp", tp0), arg("pp", pp0), arg("dp", dp0)
    L, d, H, V = arg("layers", 24), arg("d", 2048), arg("heads", 16), arg("vocab", 50257)
    S, mb, M = arg("seq", 512), arg("mbatch", 4), arg("M", 8)
    fuse = "--no-fuse" not in sys.argv
    pp_fuse = arg("pp-fuse", 2 if fuse else 1)          # pipeline meshes: micro-batches that travel through the stages together
    fused_comm = "--no-fused-comm" not in sys.argv     # in-kernel NVLink collectives (product path) vs NCCL baseline
    mesh = Mesh(tp, pp, dp) if world > 1 else Mesh.single()
    extras = "--no-extras" not in sys.argv
    fused_check = None
    if world > 1 and fused_comm and device.type == "cuda" and extras:
        import gc
        from kharon_b200.parallel import selfcheck
        fused_check = selfcheck.fused_check(mesh, device)
        gc.collect()
    eng = TrainEngine(L, d, H, V, S, mb, M, mesh=mesh, device=device, lr=3e-4, wd=0.1, fuse_microbatches=fuse,
                      init=arg("init", "device", str), fused_comm=fused_comm, pp_split=arg("pp-split", "auto", str),
                      sp="--sp" in sys.argv, pp_fuse=pp_fuse)
    seq_par = bool(eng.sp)
    pp_fused = int(eng.pp_fuse)
    ntok = M * mb * S                                    # per replica and step
    data = Rng(42 + mesh.c.dp_rank)
    pin = device.type == "cuda"
    host_idx = [torch.empty(ntok, dtype=torch.int32, pin_memory=pin) for _ in range(2)]
    host_tgt = [torch.empty(ntok, dtype=torch.int32, pin_memory=pin) for _ in range(2)]
    dev_idx = torch.empty(ntok, dtype=torch.int32, device=device)
    dev_tgt = torch.empty(ntok, dtype=torch.int32, device=device)

    def barrier():
        if world > 1:
            dist.barrier()
        if device.type == "cuda":
            torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        if device.type == "cuda":
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        t0 = time.perf_counter()
        for i in range(steps):
            fn(i)
        if device.type == "cuda":
            e1.record()
        barrier()
        ms = e0.elapsed_time(e1) if device.type == "cuda" else (time.perf_counter() - t0) * 1e3
        t = torch.tensor([ms], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def step_device(i):
        data.batch_into(host_idx[0], host_tgt[0], V)      # fresh synthetic ids every step
        dev_idx.copy_(host_idx[0]); dev_tgt.copy_(host_tgt[0])
        eng.train_step(dev_idx, dev_tgt)

    losses = []

    def step_e2e(i):
        b = i & 1
        data.batch_into(host_idx[b], host_tgt[b], V)
        eng.train_step(host_idx[b], host_tgt[b])          # H2D from pinned memory inside the call
        losses.append(eng.loss())                         # D2H read of the step's loss

    for i in range(W):
        step_e2e(i)
    # --- kernel-only region: inputs staged on the device outside the timing
    data.batch_into(host_idx[0], host_tgt[0], V)
    dev_idx.copy_(host_idx[0]); dev_tgt.copy_(host_tgt[0])
    gpu_index = device.index if device.type == "cuda" else 0
    sampler = ClockSampler(gpu_index) if rank == 0 and device.type == "cuda" else None
    l0 = ops.launch_count
    ms_dev = timed(lambda i: eng.train_step(dev_idx, dev_tgt), K)
    launches = ops.launch_count - l0
    ms_e2e = timed(step_e2e, K)
    clocks = sampler.stop() if sampler else {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
    if device.type == "cuda":
        ops.check_device_status()
    final_loss = losses[-1] if losses else float("nan")
    if world > 1:   # the loss lives on the last stage
        t = torch.tensor([final_loss if mesh.c.last else 0.0], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        final_loss = float(t.item())
    # ---- extras: none of them touches the numbers above
    ref_shape = decode = None
    if extras and device.type == "cuda":
        import gc
        stage_layers = eng.stage_layers
        fused_mb = bool(eng.fused_mb)
        del eng
        gc.collect()
        torch.cuda.empty_cache()
        try:
            Kr = min(K, 10)
            e2 = TrainEngine(L, d, H, 256, S, mb, M, mesh=mesh, device=device, lr=3e-4, wd=0.1, fuse_microbatches=fuse,
                             init=arg("init", "device", str), fused_comm=fused_comm, untied_head=True,
                             pp_split=arg("pp-split", "auto", str), sp="--sp" in sys.argv, pp_fuse=pp_fuse)
            data.batch_into(host_idx[0], host_tgt[0], 256)
            dev_idx.copy_(host_idx[0]); dev_tgt.copy_(host_tgt[0])
            for _ in range(W):
                e2.train_step(dev_idx, dev_tgt)
            ms_r = timed(lambda i: e2.train_step(dev_idx, dev_tgt), Kr)
            ops.check_device_status()
            ref_shape = {"value": round(ntok * dp * Kr / (ms_r / 1e3), 1), "unit": "tok/s", "ms_per_step": round(ms_r / Kr, 3),
                         "steps": Kr, "model": "GPT L%d d%d H%d V256 untied head" % (L, d, H),
                         "layers_per_stage": e2.stage_layers}
            del e2
            gc.collect()
            torch.cuda.empty_cache()
        except Exception as ex:       # the headline numbers stand on their own
            ref_shape = {"error": "%s: %s" % (type(ex).__name__, str(ex)[:200])}
        if rank == 0:
            try:
                decode = decode_numbers(device)
            except Exception as ex:
                decode = {"error": "%s: %s" % (type(ex).__name__, str(ex)[:200])}
        barrier()
    else:
        stage_layers, fused_mb = eng.stage_layers, bool(eng.fused_mb)
    if rank == 0:
        tokens = ntok * dp * K
        value = tokens / (ms_dev / 1e3)
        e2e = tokens / (ms_e2e / 1e3)
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except Exception:
            pass
        peak = peaks.get("bf16_tflops_sustained", 1400.0) * 1e12
        flops_tok = 6.0 * matmul_params(Config_like(L, d, V))
        out = {
            "metric": "1.2B GPT train tok/s", "value": round(value, 1), "unit": "tok/s", "n_gpus": n, "steps": K,
            "warmup": W, "ms_per_step": round(ms_dev / K, 3), "higher_is_better": True,
            "scaling": "weak" if n == 8 else "strong", "vs_baseline": round(value / PUBLISHED_TOK_S, 3),
            "dtype": "bf16", "data": "synthetic uniform token ids, random-init N(0,0.02) weights",
            "impl": "ours",
            "mfu": round(value * flops_tok / (n * peak), 4),
            "mfu_peak_tflops_per_gpu": round(peak / 1e12, 1),
            "config": {"model": "GPT L%d d%d H%d V%d tied" % (L, d, H, V), "global_batch": mb * M * dp, "seq_len": S,
                       "micro_batch": mb, "micro_batches": M, "parallelism": "tp%d pp%d dp%d(zero1)" % (tp, pp, dp),
                       "microbatches_fused_on_single_stage": fused_mb, "microbatches_per_pipeline_turn": pp_fused,
                       "fused_comm": fused_comm,
                       "sequence_parallel": seq_par, "layers_per_stage": stage_layers,
                       "l2": "inputs larger than L2 (step working set > 20 GB)", "loss_last_step": round(final_loss, 4)},
            "clocks": clocks,
            "e2e": {"value": round(e2e, 1), "unit": "tok/s", "ms_per_step": round(ms_e2e / K, 3),
                    "h2d_bytes_per_step": 2 * ntok * 4, "d2h_bytes_per_step": 4},
            "gpu_launches": launches,
        }
        if fused_check is not None:
            out["fused_check"] = fused_check
        if ref_shape is not None:
            out["at_reference_shape"] = ref_shape
        if decode is not None:
            out["decode"] = decode
        print(json.dumps(out), flush=True)
    rc = 0
    if fused_check is not None:
        from kharon_b200.parallel import selfcheck
        rc = 0 if selfcheck.passed(fused_check) else 3
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return rc


def decode_numbers(device):
    """Paged-KV decode of BASELINE's inference configuration on one GPU: L24 d1024 H16 V50257, prompt
    128, 256 new greedy tokens, block 16, G identical prompts through continuous batching
    (bench/bench_infer.c:43-58 of the reference; tok/s = tokens_decoded / wall time, prefill included)."""
    import torch
    from kharon_b200.infer import InferEngine
    from kharon_b200.models import GPT, Config
    L, d, H, V, seq, plen, n_new, bs = 24, 1024, 16, 50257, 1024, 128, 256, 16
    m = GPT(Config(L, d, H, V, seq, 1), device, torch.bfloat16)
    m.init_weights_device(1234)
    prompt = [(i * 131 + 7) % V for i in range(plen)]
    max_lb = (seq + bs - 1) // bs
    out = {}
    for G in (1, 8, 32):
        eng = InferEngine(m, bs, G * max_lb + 16, max(G, plen) + G * plen + 64, G + 1)
        best = None
        for _ in range(2):              # the first pass captures the CUDA graphs
            _, st, ms = eng.generate([prompt] * G, n_new, max_active=G)
            best = ms if best is None else min(best, ms)
        out["G%d_tok_s" % G] = round(st["tokens_decoded"] * 1000.0 / best, 1)
        out["kv_ratio"] = round(G * seq / (st["blocks_peak"] * bs), 2)
        eng.close()
    out["config"] = ("L24 d1024 H16 V50257 prompt 128 new 256 block 16 bf16, 1 GPU, CUDA-graph decode steps, device sampler; "
                     "up to %d sequences a step is one persistent kernel" % (eng.persistent_max if eng.persistent else 0))
    return out


class Config_like:
    def __init__(self, L, d, V):
        self.n_layer, self.d_model, self.vocab = L, d, V


def run_reference():
    from baseline import reference_run
    return reference_run.main(sys.argv[1:])


if __name__ == "__main__":
    impl = arg("impl", "ours", str)
    sys.exit(run_reference() if impl == "reference" else run_ours())
