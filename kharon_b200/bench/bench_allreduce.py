"""All-reduce sweep 4 KiB .. 64 MiB fp32 with a sum check (reference bench/bench_allreduce.c:18-41), NCCL,
device-timed, maximum over ranks; bus bandwidth = 2(n-1)/n * bytes / time.  Launch with torchrun."""
import json

import torch
import torch.distributed as dist

from ..parallel.mesh import init_distributed


def main():
    rank, world, dev = init_distributed()
    x = torch.full((1024,), float(rank + 1), device=dev)
    dist.all_reduce(x)
    assert x[0].item() == world * (world + 1) / 2
    rows = []
    n = 1024
    while n * 4 <= 64 << 20:
        x = torch.ones(n, device=dev)
        for _ in range(5):
            dist.all_reduce(x)
        torch.cuda.synchronize(); dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(20):
            dist.all_reduce(x)
        e1.record(); torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / 20], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        rows.append(dict(bytes=n * 4, us=ms * 1e3, busbw_GBs=2 * (world - 1) / world * n * 4 / ms / 1e6))
        n *= 4
    if rank == 0:
        print(json.dumps(dict(world=world, sweep=rows)))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
