"""Micro-benchmarks with the command lines of the reference's bench/*.c programs."""
import torch


def time_ms(fn, iters=20, warmup=5, flush=None):
    """CUDA-event time per call.  ``flush`` (a CUDA tensor larger than L2) is rewritten between
    timed iterations when the working set is smaller than L2."""
    from .. import ops
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    tot = 0.0
    for _ in range(iters):
        if flush is not None:
            ops.flush_l2(flush)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        tot += e0.elapsed_time(e1)
    return tot / iters


def l2_flush_buffer(device="cuda"):
    return torch.empty(256 << 20, dtype=torch.uint8, device=device)
