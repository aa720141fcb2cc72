"""Smoke run of the layer: a few forward+backward iterations, wall-clock and device ms per
iteration, finiteness of every output (role of the reference's
stream_ep/stream_moe/smoke_pipeline.py).

    python -m streamep_b200.stream_moe.smoke_pipeline --tokens 4096 --iters 10
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29551 -m streamep_b200.stream_moe.smoke_pipeline
"""
from __future__ import annotations

import argparse
import sys
import time

import torch

from ._harness_common import add_shape_args, barrier, build_layers, init_distributed, rank_zero_print


def main():
    ap = argparse.ArgumentParser()
    add_shape_args(ap)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args()
    rank, world, local, dev, group = init_distributed()
    buf, layers, E = build_layers(args, group, world, dev)
    torch.manual_seed(1 + rank)
    x = torch.randn(args.tokens, args.hidden, device=dev).to(torch.bfloat16)
    dy = (torch.randn(args.tokens, args.hidden, device=dev) * 0.1).to(torch.bfloat16)

    def step():
        h = x.detach().requires_grad_(True)
        cur = h
        for layer in layers:
            cur = layer(cur)
        cur.backward(dy)
        grads = [h.grad] + [p.grad for layer in layers for p in (layer.w1, layer.w2)]
        ok = all(torch.isfinite(g.float()).all().item() for g in grads) and torch.isfinite(cur.float()).all().item()
        for layer in layers:
            layer.w1.grad = None
            layer.w2.grad = None
        return ok

    for _ in range(args.warmup):
        step()
    barrier(world, local)
    buf.check_status()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    finite = True
    for _ in range(args.iters):
        finite &= step()
    e1.record()
    barrier(world, local)
    wall = (time.perf_counter() - t0) / args.iters * 1e3
    buf.check_status()
    rank_zero_print(rank, f"smoke: world={world} tokens/rank={args.tokens} H={args.hidden} I={args.ffn} E={E} top{args.topk} "
                          f"layers={args.layers} fused={args.fused} ckpt={args.ckpt_level}: "
                          f"{wall:.3f} ms/iter wall, {e0.elapsed_time(e1) / args.iters:.3f} ms/iter device "
                          f"(includes the per-iteration finiteness checks), outputs finite: {finite}")
    if world > 1:
        torch.distributed.destroy_process_group()
    return 0 if finite else 1


if __name__ == "__main__":
    sys.exit(main())
