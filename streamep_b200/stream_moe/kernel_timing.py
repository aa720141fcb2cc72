"""Where the time of the fused kernels goes: per-CTA time stamps of one training step.

    python -m streamep_b200.stream_moe.kernel_timing
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29571 \\
        -m streamep_b200.stream_moe.kernel_timing --capacity-factor 1.5

The GEMM kernels can record, per CTA, %globaltimer stamps (``Runtime.set_kernel_timing``): kernel start and end,
nanoseconds the operand pipeline stood still for tile gates, when the first tile became ready, how many tiles the
CTA had finished when its push ended, when the CTA's push
warps claimed their first chunk and finished their last, and which share of its tile loop the thread that issues
the MMAs spent waiting for operands (TMA not there yet) and for a free accumulator (epilogue not done yet).  This harness runs a few steps of the layer with the
stamps on and prints, for each kind of launch, the split the reference's profile harness cannot give (its kernels
carry no stamps; stream_ep/stream_moe/profile_pipeline.py:502-560 only has whole-kernel durations).
All times are microseconds relative to the earliest CTA start of that launch on that rank.
"""
from __future__ import annotations

import argparse
import sys

import torch
import torch.distributed as dist

from ._harness_common import add_shape_args, barrier, build_layers, init_distributed, rank_zero_print

KINDS = {1: "GEMM-A SwiGLU", 6: "dispatch (+) GEMM-A SwiGLU", 2: "GEMM-Y (+ combine)", 3: "GEMM-Y_bwd dSwiGLU",
         8: "dispatch_grads (+) GEMM-Y_bwd", 7: "GEMM-A_bwd (+ combine_grads)", 5: "preact recompute",
         0: "dW1 + dW2 (last launch wins)"}


def summarise(t: torch.Tensor) -> dict:
    """``t``: [num_sms, 12] int64 stamps of one launch."""
    live = t[:, 0] > 0
    if not bool(live.any()):
        return {}
    t = t[live].double()
    t0 = t[:, 0].min()
    us = lambda v: float(v) / 1e3   # noqa: E731
    out = {"ctas": int(live.sum()), "kernel_us": us(t[:, 6].max() - t0), "start_skew_us": us(t[:, 0].max() - t0),
           "gate_wait_us_mean": us(t[:, 1].mean()), "gate_wait_us_max": us(t[:, 1].max()),
           "tiles_per_cta": float(t[:, 7].mean())}
    mma = t[:, 8] > 0
    if bool(mma.any()):     # shares of the MMA-issuing thread's tile loop (SM cycles)
        out["mma_wait_operands_frac"] = float((t[mma, 9] / t[mma, 8]).mean())
        out["mma_wait_accumulator_frac"] = float((t[mma, 10] / t[mma, 8]).mean())
    gated = t[:, 2] > 0
    if bool(gated.any()):
        out["first_tile_ready_us_mean"] = us((t[gated, 2] - t0).mean())
    pushed = t[:, 5] > 0
    if bool(pushed.any()):
        out["push_start_us_mean"] = us((t[pushed, 4] - t0).mean())
        out["push_end_us_mean"] = us((t[pushed, 5] - t0).mean())
        out["push_end_us_max"] = us((t[pushed, 5] - t0).max())
        out["tiles_done_at_push_end"] = float(t[pushed, 3].mean())
    return out


def run_steps(args, buf, layers, routes, x, dy, world, local):
    stamps = None
    for step in range(args.steps):
        if step == args.steps - 1:
            barrier(world, local)
            stamps = buf.runtime.set_kernel_timing(True)
        h = x.detach().requires_grad_(True)
        cur = h
        for layer, r in zip(layers, routes):
            cur = layer.experts(cur, *r)
        cur.backward(dy)
        for layer in layers:
            layer.w1.grad = None
            layer.w2.grad = None
    torch.cuda.synchronize()
    buf.check_status()
    buf.runtime.set_kernel_timing(False)
    return stamps


def sweep(args, buf, layers, routes, x, dy, rank, world, local):
    cols = ("kernel_us", "gate_wait_us_mean", "first_tile_ready_us_mean", "push_end_us_max", "tiles_done_at_push_end")
    rank_zero_print(rank, f"config: tokens/rank={args.tokens} hidden={args.hidden} ffn={args.ffn} top{args.topk} world={world} "
                          f"capacity_factor={args.capacity_factor}; columns: mean over ranks of " + ", ".join(cols))
    for setting in args.sweep.split(","):
        f = [int(v) for v in setting.split(":")]
        f += [2, 0, 0, 0, 0][len(f) - 3:] if len(f) < 8 else []
        ppc, warps, order, hp, hc, pctas, bulk, split = f[:8]
        buf.runtime.set_push_ctas(pctas)
        buf.runtime.set_bulk_push(bool(bulk))
        buf.runtime.set_split_local(bool(split))
        buf.runtime.set_pairs_per_chunk(ppc); buf.runtime.set_active_push_warps(warps); buf.runtime.set_push_order(order)
        buf.runtime.set_push_head(hp, hc)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        stamps = run_steps(args, buf, layers, routes, x, dy, world, local)
        barrier(world, local)
        e0.record()
        for _ in range(5):
            h = x.detach().requires_grad_(True)
            cur = h
            for layer, r in zip(layers, routes):
                cur = layer.experts(cur, *r)
            cur.backward(dy)
            for layer in layers:
                layer.w1.grad = None
                layer.w2.grad = None
        e1.record()
        torch.cuda.synchronize()
        vals = []
        for k in (6, 8):
            sm = summarise(stamps[k].cpu())
            vals += [sm.get(c, 0.0) for c in cols]
        vals.append(e0.elapsed_time(e1) / 5 * 1e3)
        t = torch.tensor(vals, device=x.device, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t)
            t /= world
        v = t.tolist()
        rank_zero_print(rank, f"chunk={ppc:2d} warps={warps:2d} order={order} head={hp}x{hc:5d} push_ctas={pctas:2d} bulk={bulk} split={split}: A[" + " ".join(f"{a:7.1f}" for a in v[0:5]) +
                        "]  Y_bwd[" + " ".join(f"{a:7.1f}" for a in v[5:10]) + f"]  step {v[10]:7.1f} us")
    barrier(world, local)
    if world > 1:
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    add_shape_args(ap)
    ap.add_argument("--steps", type=int, default=6)
    ap.add_argument("--sweep", default="", help="comma-separated push settings 'pairs_per_chunk:push_warps:push_order[:head_pairs:head_chunks[:push_ctas[:bulk[:split_local]]]]' "
                    "(push_warps 0 = all); prints one line per setting and kind, averaged over ranks")
    args = ap.parse_args()
    rank, world, local, dev, group = init_distributed()
    buf, layers, E = build_layers(args, group, world, dev)
    T, H = args.tokens, args.hidden
    torch.manual_seed(5 + rank)
    x = torch.randn(T, H, device=dev).to(torch.bfloat16)
    dy = (torch.randn(T, H, device=dev) * 0.1).to(torch.bfloat16)
    routes = [layer.route(x) for layer in layers]
    if args.sweep:
        return sweep(args, buf, layers, routes, x, dy, rank, world, local)
    stamps = None
    for step in range(args.steps):
        if step == args.steps - 1:
            barrier(world, local)
            stamps = buf.runtime.set_kernel_timing(True)
        h = x.detach().requires_grad_(True)
        cur = h
        for layer, r in zip(layers, routes):
            cur = layer.experts(cur, *r)
        cur.backward(dy)
        for layer in layers:
            layer.w1.grad = None
            layer.w2.grad = None
    torch.cuda.synchronize()
    buf.check_status()
    buf.runtime.set_kernel_timing(False)
    rows = {k: summarise(stamps[k].cpu()) for k in KINDS}
    every = [None] * world
    if world > 1:
        dist.all_gather_object(every, rows)
    else:
        every = [rows]
    rank_zero_print(rank, f"config: tokens/rank={T} hidden={H} ffn={args.ffn} experts={E} top{args.topk} world={world} "
                          f"fused={args.fused} capacity_factor={args.capacity_factor}")
    for k, name in KINDS.items():
        if not every[0].get(k):
            continue
        rank_zero_print(rank, f"\n{name}")
        keys = list(every[0][k].keys())
        rank_zero_print(rank, "rank " + " ".join(f"{c:>24}" for c in keys))
        for r, rr in enumerate(every):
            if rr.get(k):
                rank_zero_print(rank, f"{r:4d} " + " ".join(
                    f"{rr[k].get(c, float('nan')):24.3f}" if c.endswith("_frac") else f"{rr[k].get(c, float('nan')):24.1f}" for c in keys))
    barrier(world, local)
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
