"""GRPO trainer entry point; flags of the reference's ``grpo_train`` (src/grpo_train.c:68-79):
``--layers 4 --d 256 --heads 8 --G 8 --prompts 16 --steps 400 --lr 1e-3 --temp 1.0 --beta 0.02
--log 20 --sft 200 --rllr 1e-4``.  Additions: ``--task add|reverse`` (single-digit addition as in
the reference, or reversing a random 8-digit string with a 1/0 reward), ``--seq`` and data
parallelism over prompts when launched under torchrun (``--prompts`` is per step over all ranks).
Log lines keep the reference's wording (grpo_train.c:181-182)."""
from __future__ import annotations

import torch
import torch.distributed as dist

from .parallel.mesh import init_distributed
from .rl import AddTask, GRPOTrainer, ReverseTask
from .utils.cli import Flags


def main(argv=None):
    f = Flags(argv, "grpo_train")
    L, d, H = f.int("layers", 4), f.int("d", 256), f.int("heads", 8)
    G, NP, steps = f.int("G", 8), f.int("prompts", 16), f.int("steps", 400)
    lr, temp, beta = f.float("lr", 1e-3), f.float("temp", 1.0), f.float("beta", 0.02)
    log, sft, rllr = f.int("log", 20), f.int("sft", 200), f.float("rllr", 1e-4)
    task_name = f.str("task", "add")
    seq = f.int("seq", 0)
    hb_s = f.float("heartbeat", 0.0, "seconds after which a silent rank counts as dead (0 = off)")
    dev_flag = f.str("device", "")
    f.maybe_help()
    rank, world, device = init_distributed(dev_flag or None)
    task = ReverseTask() if task_name == "reverse" else AddTask()
    if NP % world:
        raise SystemExit("--prompts must be divisible by the number of ranks")
    tr = GRPOTrainer(task, L, d, H, seq or None, G, NP // world, lr, rllr, temp, beta, device=device,
                     dtype=torch.bfloat16 if device.type == "cuda" else torch.float32,
                     dp_group=dist.group.WORLD if world > 1 else None, dp_rank=rank, dp=world)
    hb = None
    if hb_s > 0 and world > 1:      # checked before every step's gradient exchange
        from .utils.watchdog import Heartbeat
        hb = Heartbeat(rank, world, interval_s=min(1.0, hb_s / 4), timeout_s=hb_s)
    tr.heartbeat = hb
    say = print if rank == 0 else (lambda *a, **k: None)
    say("GRPO %s: L=%d d=%d H=%d  G=%d prompts=%d (B=%d per rank, %d ranks) T=%d  lr=%g temp=%g beta=%g sft=%d" %
        (task_name, L, d, H, G, NP, tr.B, world, tr.T, lr, temp, beta, sft))
    say("step %4d  acc %.3f (random init)" % (0, tr.eval_accuracy()))
    for s in range(1, sft + 1):
        tr.sft_step()
        if s % log == 0 or s == sft:
            say("sft  %4d  acc %.3f" % (s, tr.eval_accuracy()), flush=True)
    tr.snapshot_reference()
    for step in range(1, steps + 1):
        st = tr.grpo_step(step)
        if step % log == 0:
            say("step %4d  mean-reward %.3f  greedy-acc %.3f  | rollout %.0f tok/s, prefix saved %.0f blk/step" %
                (step, st["mean_reward"], tr.eval_accuracy(), st["rollout_tok_s"], st["prefix_saved_per_prompt"]),
                flush=True)
    say("final greedy-acc %.3f" % tr.eval_accuracy())
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return tr


if __name__ == "__main__":
    main()
