"""``python -m kharon_b200.bench.bench_flash B H T HD`` (default 4 8 512 64, reference bench/bench_flash.c:40-43):
FlashAttention forward and backward, causal FLOP rate (4*B*H*T*T*hd/2 forward, 2.5x that backward)."""
import json
import sys

import torch

from .. import ops
from . import l2_flush_buffer, time_ms


def main(argv=None):
    a = [int(x) for x in (sys.argv[1:] if argv is None else argv) if x.isdigit()]
    B, H, T, hd = (a + [4, 8, 512, 64][len(a):])[:4]
    d = H * hd
    dev = "cuda"
    qkv = torch.randn(B * T, 3 * d, device=dev).bfloat16()
    out = torch.empty(B * T, d, device=dev, dtype=torch.bfloat16)
    lse = torch.empty(B, H, T, device=dev)
    dout = torch.randn(B * T, d, device=dev).bfloat16()
    dqkv = torch.empty_like(qkv)
    delta = torch.empty(B, H, T, device=dev)
    fl = l2_flush_buffer() if qkv.numel() * 2 * 3 < (126 << 20) else None
    tf = time_ms(lambda: ops.flash_fwd(qkv, out, lse, B, T, H, hd), flush=fl)
    tb = time_ms(lambda: ops.flash_bwd(qkv, out, dout, lse, dqkv, delta, B, T, H, hd), flush=fl)
    flops = 4.0 * B * H * T * T * hd / 2
    res = dict(B=B, H=H, T=T, hd=hd, fwd_ms=tf, fwd_tflops=flops / tf / 1e9, bwd_ms=tb, bwd_tflops=2.5 * flops / tb / 1e9,
               l2="flushed between iterations" if fl is not None else "operands larger than L2")
    print(json.dumps(res))
    return res


if __name__ == "__main__":
    main()
