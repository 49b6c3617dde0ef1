#!/usr/bin/env bash
# One-node counterparts of the reference's eleven cluster jobs (scripts/ice_m1.sbatch ...
# scripts/ice_m10_torch.sbatch): the exact command lines that produce each published kind of number,
# with torchrun in place of mpirun and no batch scheduler.
#
#   bash kharon_b200/bench/milestones.sh m7        # one job
#   bash kharon_b200/bench/milestones.sh all       # everything the visible GPUs allow
#
# Run from the repository root.  Flags written --kh-<name> are the torchrun-safe spelling of --<name>.
set -euo pipefail
PY=${PYTHON:-python}
NGPU=$($PY -c 'import torch; print(torch.cuda.device_count())')
run() { # run <nproc> <module> args...
  local n=$1 mod=$2; shift 2
  if [ "$n" -gt "$NGPU" ]; then echo "skip ($n GPUs needed, $NGPU visible): $mod $*"; return 0; fi
  if [ "$n" -eq 1 ]; then $PY -m "$mod" "$@"
  else $PY -m torch.distributed.run --nnodes=1 --nproc-per-node "$n" --master-addr 127.0.0.1 \
         --master-port "${MASTER_PORT:-29533}" -m "$mod" "$@"; fi
}
data() { [ -f data/input.bin ] || $PY -m kharon_b200.utils.prep_data data/input.bin; }

m1() { $PY -m pytest tests -q -m "not gpu" -k "model or runtime or resume"; run 1 kharon_b200.bench.bench_step 50; }
m2() { $PY -m pytest tests/test_kernels_gpu.py -q -m gpu -k flash; run 1 kharon_b200.bench.bench_flash 4 8 512 64; }
m3() { data; $PY -m pytest tests -q -m gpu -k "bf16 or model"
       run 1 kharon_b200.train --layers 8 --d 512 --heads 8 --seq 256 --batch 32 --steps 1000 --log 100 \
           --ckptevery 0 --lr 3e-4 --data data/input.bin --ckpt checkpoints/m3.ckpt
       run 1 kharon_b200.bench.bench_bf16 8192 8192 2048; run 1 kharon_b200.bench.bench_fused 8192 2048; }
m4_comms() { run 2 kharon_b200.bench.bench_allreduce; }
m4_tp() { data; local CFG="--layers 8 --kh-d 512 --heads 8 --seq 256 --batch 32 --steps 300 --kh-log 50 --lr 3e-4 --data data/input.bin"
          run 1 kharon_b200.train $CFG --ckptevery 0 --ckpt checkpoints/sg.ckpt; run 2 kharon_b200.tp_train $CFG; }
m5_pp() { data; local BASE="--layers 8 --kh-d 512 --heads 8 --seq 256 --mbatch 16 --data data/input.bin"
          run 1 kharon_b200.pp_train $BASE --M 16 --steps 200 --kh-log 50
          run 2 kharon_b200.pp_train $BASE --M 16 --steps 200 --kh-log 50
          for MB in 8 16 32 64; do run 2 kharon_b200.pp_train $BASE --M $MB --steps 1 --kh-log 1000; done
          for MB in 16 32 64; do run 4 kharon_b200.pp_train $BASE --M $MB --steps 1 --kh-log 1000; done; }
m6_tppp() { data; local BASE="--layers 8 --kh-d 512 --heads 8 --seq 256 --mbatch 16 --M 16 --data data/input.bin"
            run 1 kharon_b200.pp_train $BASE --tp 1 --steps 200 --kh-log 50
            run 4 kharon_b200.pp_train $BASE --tp 2 --steps 200 --kh-log 50
            run 2 kharon_b200.pp_train $BASE --tp 2 --steps 1 --kh-log 1000
            run 2 kharon_b200.pp_train $BASE --tp 1 --steps 1 --kh-log 1000; }
m7_3d() { data; local SMALL="--layers 8 --kh-d 512 --heads 8 --seq 256 --mbatch 16 --data data/input.bin"
          run 1 kharon_b200.pp_train $SMALL --tp 1 --dp 1 --M 32 --steps 200 --kh-log 50
          run 2 kharon_b200.pp_train $SMALL --tp 1 --dp 2 --M 16 --steps 200 --kh-log 50
          run 8 kharon_b200.pp_train $SMALL --tp 2 --dp 2 --M 16 --steps 200 --kh-log 50
          rm -f /tmp/m7ck.r0 /tmp/m7ck.r1 /tmp/m7ck.r2 /tmp/m7ck.r3 /tmp/m7ck.r4 /tmp/m7ck.r5 /tmp/m7ck.r6 /tmp/m7ck.r7
          run 8 kharon_b200.pp_train $SMALL --tp 2 --dp 2 --M 16 --steps 40 --kh-log 40                     # continuous
          run 8 kharon_b200.pp_train $SMALL --tp 2 --dp 2 --M 16 --steps 20 --kh-log 20 --ckpt /tmp/m7ck    # split: first half
          run 8 kharon_b200.pp_train $SMALL --tp 2 --dp 2 --M 16 --steps 40 --kh-log 20 --ckpt /tmp/m7ck --resume
          # the headline: 1.2B, TP2 x PP2 x ZeRO-1 DP2
          run 8 kharon_b200.pp_train --tp 2 --dp 2 --layers 24 --kh-d 2048 --heads 16 --seq 512 --mbatch 4 --M 8 \
              --steps 200 --kh-log 50 --vocab 50257 --synthetic
          # same, micro-batches travelling through the stages in pairs (identical math, larger kernels)
          run 8 kharon_b200.pp_train --tp 2 --dp 2 --layers 24 --kh-d 2048 --heads 16 --seq 512 --mbatch 4 --M 8 \
              --steps 200 --kh-log 50 --vocab 50257 --synthetic --pp-fuse 2; }
m8_infer() { $PY -m pytest tests/test_infer_gpu.py -q -m gpu
             run 1 kharon_b200.bench_infer --layers 24 --d 1024 --heads 16 --vocab 50257 --seq 1024 --prompt 128 --new 256 --block 16 --bf16 1
             run 1 kharon_b200.bench_infer --layers 24 --d 2048 --heads 16 --vocab 50257 --seq 1024 --prompt 256 --new 256 --block 16 --bf16 1
             for B in 8 16 32 64; do run 1 kharon_b200.bench_infer --layers 24 --block $B --G 16 | grep "G=16:"; done
             run 2 kharon_b200.bench_infer --layers 24 --tp 2; run 4 kharon_b200.bench_infer --layers 24 --tp 4
             KHARON_PERSISTENT_DECODE=0 $PY -m kharon_b200.bench_infer --layers 24; }      # the five-kernel chain for comparison
m9_grpo() { $PY -m pytest tests/test_grpo_cpu.py -q
            run 1 kharon_b200.grpo_train --layers 6 --d 512 --heads 8 --G 16 --prompts 32 --sft 200 --steps 400 --log 50 \
                --lr 1e-3 --rllr 1e-4 --temp 0.7 --beta 0.02
            run 1 kharon_b200.grpo_train --task reverse --layers 6 --d 512 --heads 8 --G 16 --prompts 32 --beta 0.04 --sft 200 --steps 400
            run 8 kharon_b200.grpo_train --task reverse --layers 6 --kh-d 512 --heads 8 --G 16 --prompts 32 --beta 0.04 --sft 200 --steps 400; }
m10_torch() { run 1 kharon_b200.bench.torch_baseline --layers 8 --d 512 --heads 8 --vocab 256 --seq 256 --batch 32 --steps 100; }

case "${1:-}" in
  all) for j in m1 m2 m3 m4_comms m4_tp m5_pp m6_tppp m7_3d m8_infer m9_grpo m10_torch; do echo "==== $j"; $j; done ;;
  m1|m2|m3|m4_comms|m4_tp|m5_pp|m6_tppp|m7_3d|m8_infer|m9_grpo|m10_torch) "$1" ;;
  m4) m4_comms; m4_tp ;; m5) m5_pp ;; m6) m6_tppp ;; m7) m7_3d ;; m8) m8_infer ;; m9) m9_grpo ;; m10) m10_torch ;;
  *) echo "usage: $0 {m1|m2|m3|m4|m5|m6|m7|m8|m9|m10|all}"; exit 2 ;;
esac
