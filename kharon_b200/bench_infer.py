"""Paged-KV decode benchmark with the flags of the reference's ``bench_infer`` (bench/bench_infer.c:16-40):
``--layers 12 --d 1024 --heads 16 --vocab 50257 --seq 1024 --prompt 128 --new 256 --block 16
--bf16 1``; additions ``--G`` (comma list, default 1,8,16,32), ``--json`` and ``--init host|device``.

Per G: G identical prompts through continuous batching -> decode tok/s (tokens_decoded /
wall time, the prefill step included, bench_infer.c:56) and KV bytes paged vs reserving ``seq``
positions per sequence; then G samples from one shared prompt -> prefix blocks saved.
"""
from __future__ import annotations

import json
import sys

import torch

from .infer import InferEngine
from .models import GPT, Config
from .utils.cli import Flags


def run(argv=None):
    f = Flags(argv, "bench_infer")
    L, d, H, V = f.int("layers", 12), f.int("d", 1024), f.int("heads", 16), f.int("vocab", 50257)
    seq, plen, n_new, bs = f.int("seq", 1024), f.int("prompt", 128), f.int("new", 256), f.int("block", 16)
    bf16 = f.int("bf16", 1)
    Gs = [int(x) for x in f.str("G", "1,8,16,32").split(",")]
    device = f.str("device", "cuda" if torch.cuda.is_available() else "cpu")
    init = f.str("init", "host")
    as_json = f.has("json")
    reps = f.int("reps", 2, "timed repetitions per G (best is reported); the first warms graphs up")
    tp_flag = f.int("tp", 0, "tensor-parallel degree (0 = world size under torchrun)")
    fused = not f.has("no-fused-comm")
    graphs = not f.has("no-graphs")
    f.maybe_help()
    cfg = Config(L, d, H, V, seq, 1)
    import torch.distributed as dist
    from .parallel.mesh import Mesh, init_distributed
    rank, world, dev = init_distributed(None if device != "cpu" else "cpu")
    tp = tp_flag or world
    mesh = None
    if world > 1:
        device = str(dev)
        mesh = Mesh(tp, 1, world // tp)
    m = GPT(cfg, device, torch.bfloat16 if bf16 else torch.float32, tp=tp if mesh else 1,
            tp_rank=mesh.c.tp_rank if mesh else 0)
    if mesh is not None and tp > 1:
        grp = mesh.tp_group
        m.tp_allreduce = lambda t: dist.all_reduce(t, group=grp)
        if fused and m.device.type == "cuda":
            from .parallel import fused as fused_mod
            fused_mod.install(m, mesh)
    say = print if rank == 0 else (lambda *a, **k: None)
    if init == "device" and device != "cpu":
        m.init_weights_device(1234)
    else:
        m.init_weights(1234)
    say("infer bench: L=%d d=%d H=%d V=%d seq=%d  prompt=%d new=%d block=%d %s" %
          (L, d, H, V, seq, plen, n_new, bs, "bf16" if bf16 else "fp32"))
    prompt = [(i * 131 + 7) % V for i in range(plen)]
    max_lb = (seq + bs - 1) // bs
    results = {"decode": [], "prefix": []}
    for G in Gs:
        eng = InferEngine(m, bs, G * max_lb + 16, max(G, plen) * 1 + G * plen + 64, G + 1, use_graphs=graphs)
        best = None
        for _ in range(max(1, reps)):
            outs, st, ms = eng.generate([prompt] * G, n_new, max_active=G)
            if best is None or ms < best[2]:
                best = (outs, st, ms)
        outs, st, ms = best
        per_pos = eng.kv_bytes_per_position()
        naive, paged = G * seq * per_pos, st["blocks_peak"] * bs * per_pos
        tps = st["tokens_decoded"] * 1000.0 / ms
        say("  G=%2d: %.0f tok/s (%d toks, %.1f ms)  KV paged %.1f MB vs naive %.1f MB (%.2fx)  blocks %d/%d" %
              (G, tps, st["tokens_decoded"], ms, paged / 1e6, naive / 1e6, naive / paged, st["blocks_peak"],
               st["blocks_total"]), flush=True)
        results["decode"].append(dict(G=G, tok_s=tps, ms=ms, kv_paged_mb=paged / 1e6, kv_naive_mb=naive / 1e6,
                                      ratio=naive / paged))
        eng.close()
    for G in [g for g in Gs if g > 1]:
        eng = InferEngine(m, bs, G * max_lb + 16, plen + 64 + G, G + 1)
        best = None
        for _ in range(max(1, reps)):
            outs, st, ms = eng.generate_group(prompt, G, n_new)
            if best is None or ms < best[2]:
                best = (outs, st, ms)
        outs, st, ms = best
        saved_mb = st["prefix_blocks_saved"] * bs * eng.kv_bytes_per_position() / 1e6
        say("  prefix-share G=%2d: blocks saved %d (%.1f MB), %.0f tok/s  peak %d/%d" %
              (G, st["prefix_blocks_saved"], saved_mb, st["tokens_decoded"] * 1000.0 / ms, st["blocks_peak"],
               st["blocks_total"]), flush=True)
        results["prefix"].append(dict(G=G, saved_blocks=st["prefix_blocks_saved"], saved_mb=saved_mb,
                                      tok_s=st["tokens_decoded"] * 1000.0 / ms))
        eng.close()
    if as_json:
        say(json.dumps(results))
    return results


if __name__ == "__main__":
    run()
