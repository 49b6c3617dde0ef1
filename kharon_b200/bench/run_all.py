"""Runs the single-GPU micro-benchmarks and writes their JSON lines into one results file
(``python -m kharon_b200.bench.run_all [out.json]``; counterpart of the reference's bench/run_all.sh +
bench/results.json).  Multi-GPU numbers come from ``bench.py`` / ``pp_train`` under torchrun."""
import json
import sys

import torch


def main(argv=None):
    from . import bench_bf16, bench_flash, bench_fused, bench_step, torch_baseline
    from .. import bench_infer
    out = (sys.argv[1:] if argv is None else argv) or ["bench_results.json"]
    res = {"gpu": torch.cuda.get_device_name(), "torch": torch.__version__}
    res["bf16_gemm"] = [bench_bf16.main([str(x) for x in s]) for s in ((8192, 8192, 2048), (16384, 2048, 8192), (2048, 8192, 2048))]
    res["flash"] = [bench_flash.main([str(x) for x in s]) for s in ((4, 8, 512, 64), (32, 16, 512, 128))]
    res["fused"] = bench_fused.main(["8192", "2048"])
    res["step_m1"] = bench_step.main(["50"])
    res["torch_proxy"] = torch_baseline.main(["--vocab", "50257"])
    res["infer"] = bench_infer.run(["--layers", "24", "--init", "device", "--G", "1,8,32"])
    with open(out[0], "w") as f:
        json.dump(res, f, indent=1)
    print("wrote", out[0])


if __name__ == "__main__":
    main()
