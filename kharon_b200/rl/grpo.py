"""Critic-free GRPO: supervised warm start, group rollouts through the paged-KV engine with
prefix sharing, group-relative advantages, KL penalty (k3 estimator gradient) to a frozen
snapshot of the SFT policy, one AdamW step per rollout batch (on-policy, ratio = 1).

Behaviour follows the reference's src/grpo_train.c:67-191 and src/core/grpo.c:7-20:

    adv      = (r - mean_group) / (std_group_population + 1e-4)
    coef[t]  = mask[t] * (adv[row] - beta * (1 - p_ref / max(p_cur, 1e-8))) / N_completion_tokens
    dlogits  = coef * (softmax - onehot)          (fused into the cross-entropy kernel)

with mask = the positions whose logits predict completion tokens.  Additions: a second task
(reverse an 8-digit string, reward 1 / 0), rollouts of all prompts of a step in one engine batch,
and data parallelism over prompts (gradients averaged over the DP group, every rank steps the
same replicated policy) -- the reference is single-GPU only.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from .. import _native, ops
from ..infer import InferEngine
from ..models import GPT, Config
from ..utils.rng import Rng


def advantages(rewards: torch.Tensor, n_groups: int, group: int, eps: float = 1e-4) -> torch.Tensor:
    r = rewards.detach().to("cpu", torch.float32).contiguous()
    out = torch.empty_like(r)
    _native.rt().kh_grpo_advantages(r.data_ptr(), n_groups, group, eps, out.data_ptr())
    return out


def coefficients(adv, p_cur, p_ref, rows, T, t0, t1, beta) -> torch.Tensor:
    a = adv.detach().to("cpu", torch.float32).contiguous()
    pc = p_cur.detach().to("cpu", torch.float32).contiguous()
    pr = p_ref.detach().to("cpu", torch.float32).contiguous()
    out = torch.empty(rows * T, dtype=torch.float32)
    _native.rt().kh_grpo_coef(a.data_ptr(), pc.data_ptr(), pr.data_ptr(), rows, T, t0, t1, beta, out.data_ptr())
    return out


class AddTask:
    """Single-digit addition ``a+b=`` -> one digit (the reference's task, grpo_train.c:23-44):
    reward 0.1 for any digit plus 1.0 for the exact answer."""
    plen, nnew, vocab = 4, 1, 256

    def sample(self, rng: Rng):
        while True:
            a, b = rng.u32() % 10, rng.u32() % 10
            if a + b <= 9:
                return [48 + a, ord("+"), 48 + b, ord("=")], [48 + a + b]

    def reward(self, completion, answer):
        r = 0.1 if 48 <= completion[0] <= 57 else 0.0
        return r + (1.0 if completion[0] == answer[0] else 0.0)

    def eval_set(self):
        return [([48 + a, ord("+"), 48 + b, ord("=")], [48 + a + b]) for a in range(10) for b in range(10) if a + b <= 9]


class ReverseTask:
    """Reverse a random 8-digit string: prompt = 8 digits + separator, completion = the digits
    reversed + EOS; reward 1 on an exact match, else 0."""
    n, sep, eos, vocab = 8, ord("|"), ord("\n"), 256
    plen, nnew = 9, 9

    def sample(self, rng: Rng):
        digs = [48 + rng.u32() % 10 for _ in range(self.n)]
        return digs + [self.sep], digs[::-1] + [self.eos]

    def reward(self, completion, answer):
        return 1.0 if list(completion) == list(answer) else 0.0

    def eval_set(self):
        r = Rng(999)
        return [self.sample(r) for _ in range(64)]


class GRPOTrainer:
    def __init__(self, task, layers=4, d_model=256, heads=8, seq=None, G=8, prompts=16, lr=1e-3, rllr=1e-4, temp=1.0,
                 beta=0.02, device="cuda", dtype=torch.bfloat16, dp_group=None, dp_rank=0, dp=1, seed=1337,
                 task_seed=20260530):
        self.task, self.G, self.NP = task, G, prompts
        self.T = task.plen + task.nnew
        self.B = prompts * G
        self.lr, self.rllr, self.temp, self.beta = lr, rllr, temp, beta
        self.dp_group, self.dp, self.dp_rank = dp_group, dp, dp_rank
        self.device = torch.device(device)
        # the model sequence length is the trained window; ``seq`` only sizes the position table
        self.cfg = Config(layers, d_model, heads, task.vocab, self.T if seq is None else max(seq, self.T), self.B)
        train_cfg = Config(layers, d_model, heads, task.vocab, self.T, self.B)
        self.train_cfg = train_cfg
        self.policy = self._make(seed, dtype)
        self.ref = self._make(seed, dtype)
        self.engine = InferEngine(self.policy, block_size=2, n_blocks=self.B * self.T + 64 + prompts * 8,
                                  max_tokens=self.B * self.T + 64, max_seqs=self.B + prompts + 1)
        self.rng = Rng(task_seed + dp_rank)
        pin = self.device.type == "cuda"
        self.h_idx = torch.zeros(self.B * self.T, dtype=torch.int32, pin_memory=pin)
        self.h_tgt = torch.zeros(self.B * self.T, dtype=torch.int32, pin_memory=pin)
        self.d_coef = torch.zeros(self.B * self.T, dtype=torch.float32, device=self.device)
        self.h_rew = torch.zeros(self.B, dtype=torch.float32, pin_memory=pin)
        self.d_rew = torch.zeros(self.B, dtype=torch.float32, device=self.device)
        self.d_adv = torch.zeros(self.B, dtype=torch.float32, device=self.device)
        self.d_pcur = torch.zeros(self.B * self.T, dtype=torch.float32, device=self.device)
        self.stats = {}

    def _make(self, seed, dtype):
        # positions: the engine needs wpe rows up to cfg.seq, training uses rows [0, T)
        m = GPT(Config(self.train_cfg.n_layer, self.train_cfg.d_model, self.train_cfg.n_head, self.train_cfg.vocab,
                       self.T, self.B), self.device, dtype)
        m.init_weights(seed)
        return m

    # ------------------------------------------------------------------ helpers
    def _fill_rows(self, rows):
        """Token rows -> the pinned input / target staging buffers (target = next token, 0 after the last)."""
        t = torch.tensor(rows, dtype=torch.int32)                     # [B, T]
        self.h_idx.view(self.B, self.T).copy_(t)
        tg = self.h_tgt.view(self.B, self.T)
        tg[:, :-1].copy_(t[:, 1:])
        tg[:, -1].zero_()

    heartbeat = None        # utils.watchdog.Heartbeat of the job, when the entry point set one up

    def _sync_grads(self):
        if self.dp > 1:
            if self.heartbeat is not None:
                from ..utils.watchdog import guarded
                self.heartbeat.check()
                guarded(dist.all_reduce(self.policy.params.g, group=self.dp_group, async_op=True), self.heartbeat,
                        timeout_s=120.0, group=self.dp_group, what="gradient all-reduce")
            else:
                dist.all_reduce(self.policy.params.g, group=self.dp_group)
            self.policy.params.g.div_(self.dp)

    def sft_step(self):
        rows = []
        for _ in range(self.B):
            p, a = self.task.sample(self.rng)
            rows.append(p + a)
        self._fill_rows(rows)
        m = self.policy
        m.set_input(self.h_idx, self.h_tgt)
        m.forward(compute_loss=False)
        m.backward(loss_scale=1.0)
        self._sync_grads()
        m.adamw_step(self.lr, 0.9, 0.95, 1e-8, 0.0)
        return m.loss()

    def snapshot_reference(self):
        """Freeze the current policy as the KL reference (grpo_train.c:126-127)."""
        self.ref.params.w.copy_(self.policy.params.w)
        self.ref.sync_bf16()

    def eval_accuracy(self):
        self.engine.set_sampling(0.0, 1)
        es = self.task.eval_set()
        outs, _, _ = self.engine.generate([p for p, _ in es], self.task.nnew, max_active=min(len(es), self.B))
        ok = sum(1 for (p, a), o in zip(es, outs) if o[len(p):len(p) + len(a)] == list(a))
        return ok / len(es)

    def grpo_step(self, step: int):
        task, G, NP, T, B = self.task, self.G, self.NP, self.T, self.B
        self.engine.set_sampling(self.temp, 0x1234 * step + 1 + 7919 * self.dp_rank)
        probs = [task.sample(self.rng) for _ in range(NP)]
        outs, st, ms = self.engine.generate_groups([p for p, _ in probs], G, task.nnew)
        rows, rew = [], self.h_rew
        for pi, (p, ans) in enumerate(probs):
            for g in range(G):
                seq = (outs[pi][g] + [0] * T)[:T]
                rows.append(seq)
                rew[pi * G + g] = task.reward(seq[task.plen:task.plen + task.nnew], ans)
        # rewards go up (B floats); advantages, p(action) of both models and the coefficients stay on the device
        self.d_rew.copy_(rew, non_blocking=True)
        ops.grpo_advantages(self.d_rew, NP, G, 1e-4, self.d_adv)
        self._fill_rows(rows)
        m, ref = self.policy, self.ref
        m.set_input(self.h_idx, self.h_tgt)
        m.forward(compute_loss=False)
        self.d_pcur.copy_(m.gather_prob())
        ref.set_input(self.h_idx, self.h_tgt)
        ref.forward(compute_loss=False)
        p_ref = ref.gather_prob()
        ops.grpo_coef(self.d_adv, self.d_pcur, p_ref, B, T, task.plen - 1, T - 2, self.beta, self.d_coef)
        m.backward(coef=self.d_coef)
        self._sync_grads()
        m.adamw_step(self.rllr, 0.9, 0.95, 1e-8, 0.0)
        self.stats = dict(mean_reward=float(rew.mean()), rollout_tok_s=st["tokens_decoded"] * 1000.0 / max(ms, 1e-9),
                          prefix_saved_per_prompt=st["prefix_blocks_saved"] / NP, rollout_ms=ms)
        if self.dp > 1:
            t = torch.tensor([self.stats["mean_reward"]], device=self.device)
            dist.all_reduce(t, group=self.dp_group)
            self.stats["mean_reward"] = float(t.item()) / self.dp
        return self.stats
