"""Runs the reference's own ``pp_train`` binary (built unchanged for sm_100 by
``baseline/build_reference.sh``) on the headline configuration and converts its final report
into the benchmark's JSON line.

What is and is not comparable: the binary hard-codes vocab 256 and an untied head
(src/pp_train.c:77, src/core/gpt.c:162), reads a byte corpus (a file of uniform random bytes is
generated for it), trains on the same M micro-batches every step, and times 20 pipeline steps
itself with host-recorded CUDA events on rank 0, adding the separately timed optimizer
communication (src/pp_train.c:137-164).  Its "tok/s mesh" figure is reported as ``value``.
"""
from __future__ import annotations

import json
import os
import re
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def _arg(argv, name, default):
    key = "--" + name
    if key in argv:
        i = argv.index(key)
        if i + 1 < len(argv):
            return int(argv[i + 1])
    return default


def run(argv):
    n = _arg(argv, "gpus", 1)
    K, W = _arg(argv, "steps", 10), max(_arg(argv, "warmup", 3), 3)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    mesh = {1: (1, 1, 1), 2: (2, 1, 1), 4: (2, 2, 1), 8: (2, 2, 2)}.get(n, (1, 1, n))
    tp, dp = _arg(argv, "tp", mesh[0]), _arg(argv, "dp", mesh[2])
    exe = os.path.join(HERE, "_ref", "build", "pp_train.exe")
    corpus = "/tmp/kh_ref_corpus_%d.bin" % os.getuid()
    if not os.path.exists(corpus):
        import random
        rnd = random.Random(42)
        tmp = corpus + ".%d" % os.getpid()
        with open(tmp, "wb") as f:
            f.write(bytes(rnd.getrandbits(8) for _ in range(1 << 20)))
        os.replace(tmp, corpus)
    env = dict(os.environ)
    env["LD_LIBRARY_PATH"] = "/usr/local/cuda/lib64:" + env.get("LD_LIBRARY_PATH", "")
    env.setdefault("RANK", str(rank))
    env.setdefault("WORLD_SIZE", str(world))
    cmd = [exe, "--tp", str(tp), "--dp", str(dp), "--layers", "24", "--d", "2048", "--heads", "16", "--seq", "512",
           "--mbatch", "4", "--M", "8", "--steps", str(W + K), "--log", "100000", "--data", corpus]
    try:
        p = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=1500)
    except subprocess.TimeoutExpired:
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": "reference pp_train did not finish within 1500 s"}))
        return 0
    if rank != 0:
        return 0
    out = p.stdout
    m = re.search(r"step ([\d.]+) ms .*\n\s*throughput: ([\d.]+) tok/s/replica, ([\d.]+) tok/s mesh", out)
    if p.returncode != 0 or not m:
        print(json.dumps({"impl": "reference", "unavailable": "reference pp_train failed (rc %d): %s" %
                          (p.returncode, out.strip().splitlines()[-1][:160] if out.strip() else "no output")}))
        return 0
    mfu = re.search(r"MFU ([\d.]+)%", out)
    bd = re.search(r"breakdown/step: (.*)", out)
    print(json.dumps({
        "impl": "reference", "metric": "1.2B GPT train tok/s", "value": float(m.group(3)), "unit": "tok/s", "n_gpus": n,
        "steps": K, "warmup": W, "ms_per_step": float(m.group(1)), "higher_is_better": True,
        "scaling": "weak" if n == 8 else "strong", "vs_baseline": round(float(m.group(3)) / 30549.0, 3), "dtype": "bf16",
        "data": "uniform random bytes (vocab 256), random-init N(0,0.02) weights",
        "config": {"model": "GPT L24 d2048 H16 V256 untied head (hard-coded in the reference)", "global_batch": 32 * dp,
                   "seq_len": 512, "micro_batch": 4, "micro_batches": 8, "parallelism": "tp%d pp%d dp%d(zero1)" %
                   (tp, world // (tp * dp), dp),
                   "timing": "the binary's own report: 20 steps, host-recorded CUDA events on rank 0 + optimizer comm",
                   "mfu_vs_181TF_reported": float(mfu.group(1)) if mfu else None,
                   "breakdown": bd.group(1) if bd else None}}))
    return 0
