"""Target for timeline profilers: warm-up outside, then steady iterations fenced by
``cudaProfilerStart/Stop`` with one NVTX range per iteration (role of the reference's
stream_ep/stream_moe/nsys_pipeline.py:121-128).  Use with ``--capture-range=cudaProfilerApi``;
set ``STREAM_EP_NVTX=1`` to get the per-stage ranges of the layer as well.
"""
from __future__ import annotations

import argparse
import sys

import torch

from ._harness_common import add_shape_args, barrier, build_layers, init_distributed, rank_zero_print


def main():
    ap = argparse.ArgumentParser()
    add_shape_args(ap)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=5)
    args = ap.parse_args()
    rank, world, local, dev, group = init_distributed()
    buf, layers, _ = build_layers(args, group, world, dev)
    torch.manual_seed(1 + rank)
    x = torch.randn(args.tokens, args.hidden, device=dev).to(torch.bfloat16)
    dy = (torch.randn(args.tokens, args.hidden, device=dev) * 0.1).to(torch.bfloat16)

    def step():
        h = x.detach().requires_grad_(True)
        cur = h
        for layer in layers:
            cur = layer(cur)
        cur.backward(dy)
        for layer in layers:
            layer.w1.grad = None
            layer.w2.grad = None

    for _ in range(args.warmup):
        step()
    barrier(world, local)
    torch.cuda.profiler.start()
    for i in range(args.iters):
        torch.cuda.nvtx.range_push(f"iter_{i}")
        step()
        torch.cuda.nvtx.range_pop()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    barrier(world, local)
    buf.check_status()
    rank_zero_print(rank, f"profiled {args.iters} steady iterations after {args.warmup} warm-up iterations")
    if world > 1:
        torch.distributed.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
