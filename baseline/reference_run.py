"""``bench.py --impl reference``: runs the reference's own binaries (built unchanged for sm_100 by
``baseline/build_reference.sh``) on the headline configuration through their stock command lines
and converts what they print into the benchmark's JSON line.

Three numbers come out of one ``pp_train`` run plus one ``bench_infer`` run:

``value``   the binary's own "tok/s mesh" figure: 20 pipeline steps timed by the binary with
            host-recorded CUDA events on rank 0, plus the separately timed optimizer communication
            (src/pp_train.c:137-164).  That window leaves out AdamW, the bf16 weight sync and the
            loss read-back.
``e2e``     the rate of the binary's real training loop (src/pp_train.c:108-114), which per step
            casts the weights to bf16, clears the gradients, copies every micro-batch's ids from host
            memory (model_set_input), reads the per-row losses back and runs AdamW.  The loop prints
            one ``step N loss`` line per step with ``--log 1``; the binary's stdout is a pseudo
            terminal, so the C library flushes every line, and the arrival times of those lines
            give the step period: (t[W+K] - t[W]) / K.
``decode``  ``bench_infer.exe --layers 24`` (L24 d1024 H16 V50257, prompt 128, new 256, block 16),
            the reference's own paged-KV decode benchmark, on one GPU.

What cannot be made equal without editing the reference: it hard-codes vocab 256 and an untied
head (src/pp_train.c:77, src/core/gpt.c:162), reads a byte corpus (a file of uniform random bytes is
generated for it) and trains on the same M micro-batches every step.
"""
from __future__ import annotations

import json
import os
import pty
import re
import select
import subprocess
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
BUILD = os.path.join(HERE, "_ref", "build")


def _arg(argv, name, default):
    key = "--" + name
    if key in argv:
        i = argv.index(key)
        if i + 1 < len(argv):
            return int(argv[i + 1])
    return default


def _run_with_line_times(cmd, env, timeout):
    """Run ``cmd`` with a pseudo terminal as stdout/stderr; returns (rc, [(seconds, line), ...])."""
    master, slave = pty.openpty()
    p = subprocess.Popen(cmd, env=env, stdin=subprocess.DEVNULL, stdout=slave, stderr=slave, close_fds=True)
    os.close(slave)
    lines, buf, t_end = [], b"", time.monotonic() + timeout
    while True:
        left = t_end - time.monotonic()
        if left <= 0:
            p.kill()
            p.wait()
            os.close(master)
            return None, lines
        r, _, _ = select.select([master], [], [], min(left, 1.0))
        if r:
            try:
                chunk = os.read(master, 65536)
            except OSError:          # the child closed its side
                chunk = b""
            now = time.perf_counter()
            if not chunk:
                break
            buf += chunk
            while b"\n" in buf:
                ln, buf = buf.split(b"\n", 1)
                lines.append((now, ln.decode(errors="replace").rstrip("\r")))
        elif p.poll() is not None:
            break
    rc = p.wait()
    os.close(master)
    if buf:
        lines.append((time.perf_counter(), buf.decode(errors="replace")))
    return rc, lines


def _corpus():
    path = "/tmp/kh_ref_corpus_%d.bin" % os.getuid()
    if not os.path.exists(path):
        import random
        rnd = random.Random(42)
        tmp = path + ".%d" % os.getpid()
        with open(tmp, "wb") as f:
            f.write(bytes(rnd.getrandbits(8) for _ in range(1 << 20)))
        os.replace(tmp, path)
    return path


def step_period_ms(lines, W, K):
    """Step period of the training loop from the arrival times of its ``step N loss`` lines."""
    t = {}
    for ts, ln in lines:
        m = re.match(r"\s*step\s+(\d+)\s+loss", ln)
        if m:
            t[int(m.group(1))] = ts
    if W in t and W + K in t and K > 0:
        return (t[W + K] - t[W]) * 1e3 / K
    return None


def decode_numbers(env, timeout=600):
    exe = os.path.join(BUILD, "bench_infer.exe")
    if not os.path.exists(exe):
        return {"unavailable": "bench_infer.exe not built"}
    try:
        p = subprocess.run([exe, "--layers", "24"], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                           timeout=timeout)
    except subprocess.TimeoutExpired:
        return {"unavailable": "bench_infer.exe did not finish within %d s" % timeout}
    out = {}
    for m in re.finditer(r"^\s*G=\s*(\d+): ([\d.]+) tok/s .*\(([\d.]+)x\)", p.stdout, re.M):
        out["G%d_tok_s" % int(m.group(1))] = float(m.group(2))
        out["kv_ratio"] = float(m.group(3))
    if p.returncode != 0 or not out:
        return {"unavailable": "bench_infer.exe failed (rc %d)" % p.returncode}
    out["config"] = "L24 d1024 H16 V50257 prompt 128 new 256 block 16 bf16, 1 GPU, bench_infer.exe --layers 24"
    return out


def run(argv):
    n = _arg(argv, "gpus", 1)
    K, W = _arg(argv, "steps", 10), max(_arg(argv, "warmup", 3), 3)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    mesh = {1: (1, 1, 1), 2: (2, 1, 1), 4: (2, 2, 1), 8: (2, 2, 2)}.get(n, (1, 1, n))
    tp, dp = _arg(argv, "tp", mesh[0]), _arg(argv, "dp", mesh[2])
    exe = os.path.join(BUILD, "pp_train.exe")
    if not os.path.exists(exe):
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": "reference build not present under baseline/_ref "
                              "(run baseline/build_reference.sh <reference checkout>)"}))
        return 0
    env = dict(os.environ)
    env["LD_LIBRARY_PATH"] = "/usr/local/cuda/lib64:" + env.get("LD_LIBRARY_PATH", "")
    env.setdefault("RANK", str(rank))
    env.setdefault("WORLD_SIZE", str(world))
    handoff = "/tmp/kh_ref_e2e_%d_%s.json" % (os.getuid(), os.environ.get("MASTER_PORT", "0"))
    if rank == 0 and os.path.exists(handoff):
        os.remove(handoff)
    cmd = [exe, "--tp", str(tp), "--dp", str(dp), "--layers", "24", "--d", "2048", "--heads", "16", "--seq", "512",
           "--mbatch", "4", "--M", "8", "--steps", str(W + K), "--log", "1", "--data", _corpus()]
    rc, lines = _run_with_line_times(cmd, env, timeout=1500)
    period = step_period_ms(lines, W, K)
    if period is not None and world > 1:        # the loss lines are printed by the last rank
        tmp = handoff + ".%d" % os.getpid()
        with open(tmp, "w") as f:
            json.dump({"ms_per_step": period}, f)
        os.replace(tmp, handoff)
    if rank != 0:
        return 0
    if rc is None:
        print(json.dumps({"impl": "reference", "unavailable": "reference pp_train did not finish within 1500 s"}))
        return 0
    out = "\n".join(ln for _, ln in lines)
    m = re.search(r"step ([\d.]+) ms .*\n\s*throughput: ([\d.]+) tok/s/replica, ([\d.]+) tok/s mesh", out)
    if rc != 0 or not m:
        print(json.dumps({"impl": "reference", "unavailable": "reference pp_train failed (rc %d): %s" %
                          (rc, out.strip().splitlines()[-1][:160] if out.strip() else "no output")}))
        return 0
    if period is None and world > 1:
        for _ in range(60):
            if os.path.exists(handoff):
                try:
                    period = json.load(open(handoff))["ms_per_step"]
                    break
                except (ValueError, KeyError):
                    pass
            time.sleep(0.5)
    mfu = re.search(r"MFU ([\d.]+)%", out)
    bd = re.search(r"breakdown/step: (.*)", out)
    tokens = 8 * 4 * 512 * dp
    line = {
        "impl": "reference", "metric": "1.2B GPT train tok/s", "value": float(m.group(3)), "unit": "tok/s", "n_gpus": n,
        "steps": K, "warmup": W, "ms_per_step": float(m.group(1)), "higher_is_better": True,
        "scaling": "weak" if n == 8 else "strong", "vs_baseline": round(float(m.group(3)) / 30549.0, 3), "dtype": "bf16",
        "data": "uniform random bytes (vocab 256), random-init N(0,0.02) weights",
        "config": {"model": "GPT L24 d2048 H16 V256 untied head (hard-coded in the reference)", "global_batch": 32 * dp,
                   "seq_len": 512, "micro_batch": 4, "micro_batches": 8, "parallelism": "tp%d pp%d dp%d(zero1)" %
                   (tp, world // (tp * dp), dp),
                   "timing": "value: the binary's own report (20 steps, host-recorded CUDA events on rank 0 + optimizer "
                             "comm); e2e: period of its training loop from the arrival times of its per-step loss lines",
                   "mfu_vs_181TF_reported": float(mfu.group(1)) if mfu else None,
                   "breakdown": bd.group(1).strip() if bd else None}}
    if period is not None:
        # per step and replica the loop copies M micro-batches of ids and targets to the device
        # (model_set_input) and reads R per-row losses per micro-batch back (src/core/gpt.c:702-707)
        line["e2e"] = {"value": round(tokens / (period / 1e3), 1), "unit": "tok/s", "ms_per_step": round(period, 3),
                       "h2d_bytes_per_step": 2 * 8 * 2048 * 4 * dp, "d2h_bytes_per_step": 8 * 2048 * 4 * dp}
    if "--no-decode" not in argv:
        line["decode"] = decode_numbers(env)
    print(json.dumps(line), flush=True)
    return 0


def main(argv):
    return run(argv)
