"""Profile harness for the layer: CUDA-event step times, a per-kernel table from
``torch.profiler`` and the serial-sum vs end-to-end comparison that shows how much overlap the
pipeline buys (role of the reference's stream_ep/stream_moe/profile_pipeline.py:191-269,394-456,
502-560,623-709).

    python -m streamep_b200.stream_moe.profile_pipeline --tokens 8192 --hidden 2048 --ffn 1408 \
        --experts-per-rank 8 --topk 6 --steps 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29541 -m streamep_b200.stream_moe.profile_pipeline --fused 1

Rank 0 prints the table and (with ``--out DIR``) writes ``full_kernel_table.txt`` plus chrome
traces.  All times are device times; the e2e number is the max over ranks.
"""
from __future__ import annotations

import argparse
import os
import statistics
import sys

import torch
import torch.distributed as dist

LOGICAL = [  # substring of the kernel name -> logical name (template args: BN, A_MN, B_MN, EPI, PUSH)
    ("dispatch_metadata_kernel", "metadata"),
    ("fill_tile_metadata_kernel", "tile fill"),
    ("dispatch_push_kernel", "dispatch / dispatch_grads (stand-alone push)"),
    ("combine_pull_kernel", "combine / combine_grads (stand-alone pull)"),
    ("false, false, 1, true>", "dispatch (+) GEMM-A SwiGLU (fused)"),
    ("false, false, 1, false>", "GEMM-A SwiGLU"),
    ("false, false, 2, false>", "GEMM-Y (+ combine when remote)"),
    ("false, true, 3, true>", "dispatch_grads (+) GEMM-Y_bwd dSwiGLU (fused)"),
    ("false, true, 3, false>", "GEMM-Y_bwd dSwiGLU"),
    ("false, true, 2, false>", "GEMM-A_bwd (+ combine_grads when remote)"),
    ("true, true, 0, false>", "dW grouped GEMM"),
    ("false, false, 0, false>", "preact recompute GEMM"),
    ("false, false, 4, false>", "router logits GEMM (fp32 store)"),
    ("router_finish_kernel", "router softmax / top-k"),
    ("pool_rows_kernel", "pool compress / expand"),
    ("router_kernel", "router (SIMT path)"),
    ("device_barrier_kernel", "barrier / tail handshake"),
]


def classify(name: str) -> str:
    name = name.replace(", 0, 0,", ", false, false,").replace(", 0, 1,", ", false, true,").replace(", 1, 1,", ", true, true,")
    for key, label in LOGICAL:
        if key in name:
            return label
    for epi, push, label in ((1, 1, 4), (1, 0, 5), (2, 0, 6), (3, 1, 7), (3, 0, 8)):
        if name.endswith(f"{epi}, {push}>") or f", {epi}, {push}>(" in name:
            return LOGICAL[label][1]
    if "Memset" in name or "memset" in name or "FillFunctor" in name:
        return "memset / fill (torch)"
    return "other: " + name[:60]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--ffn", type=int, default=1408)
    ap.add_argument("--experts-per-rank", type=int, default=8)
    ap.add_argument("--topk", type=int, default=6)
    ap.add_argument("--layers", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--fused", type=int, default=1)
    ap.add_argument("--ckpt-level", type=int, default=0)
    ap.add_argument("--capacity-factor", type=float, default=0.0,
                    help="> 0: capacity mode (fixed receive regions, no host read per forward); 0: exact sizing")
    ap.add_argument("--out", default=None)
    ap.add_argument("--with-router", action="store_true", help="profile the module call (router + experts) and a scalar loss")
    args = ap.parse_args()

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD

    from ..models.moe_layer import StreamMoE, make_buffer

    T, H, I, K = args.tokens, args.hidden, args.ffn, args.topk
    E = args.experts_per_rank * world
    torch.manual_seed(1 + rank)
    buf = make_buffer(group, T, H, K, E, layers_in_flight=args.layers, world_size=world,
                      capacity_factor=args.capacity_factor if args.capacity_factor > 0 else None)
    layers = [StreamMoE(H, I, E, K, buf, fused=bool(args.fused), activation_checkpoint_level=args.ckpt_level,
                        device=dev, seed=10 + i) for i in range(args.layers)]
    x = torch.randn(T, H, device=dev).to(torch.bfloat16)
    dy = (torch.randn(T, H, device=dev) * 0.1).to(torch.bfloat16)
    routing = [layer.route(x) for layer in layers]

    def step():
        h = x.detach().requires_grad_(True)
        cur = h
        if args.with_router:
            for layer in layers:
                cur = layer(cur)
            ((cur * dy).sum(dtype=torch.float32) * (1.0 / cur.numel())).backward()
        else:
            for layer, (idx, w, in_rank) in zip(layers, routing):
                cur = layer.experts(cur, idx, w, in_rank)
            cur.backward(dy)
        for layer in layers:
            layer.w1.grad = None
            layer.w2.grad = None

    def sync():
        if world > 1:
            dist.barrier(device_ids=[local])
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    sync()
    buf.check_status()
    times = []
    for _ in range(args.steps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); step(); e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    med = statistics.median(times)
    t = torch.tensor([med], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    sync()

    from torch.profiler import ProfilerActivity, profile
    handler = None
    if args.out and rank == 0:
        os.makedirs(args.out, exist_ok=True)
        handler = torch.profiler.tensorboard_trace_handler(args.out)
    # two steps inside the profiler are thrown away: starting it takes a different time on every rank, and a rank
    # that is ahead would book that difference as time inside its first kernel that waits for peers
    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU], on_trace_ready=handler,
                 schedule=torch.profiler.schedule(wait=1, warmup=1, active=args.steps)) as prof:
        for i in range(args.steps + 2):
            if i == 2:
                sync()
            step()
            torch.cuda.synchronize()
            prof.step()
    sync()
    buf.check_status()
    if rank == 0:
        agg = {}
        for ev in prof.key_averages():
            dt = getattr(ev, "device_time_total", 0.0) or getattr(ev, "cuda_time_total", 0.0)
            if dt <= 0 or ev.device_type is None or "cuda" not in str(ev.device_type).lower():
                continue
            if ev.key.startswith("ProfilerStep") or ev.key.startswith("nccl:"):
                continue    # the profiler's own step range and NCCL's user annotations are spans, not kernels
            label = classify(ev.key)
            a = agg.setdefault(label, [0, 0.0])
            a[0] += ev.count
            a[1] += dt
        lines = []
        total = 0.0
        lines.append(f"config: tokens/rank={T} hidden={H} ffn={I} experts={E} ({args.experts_per_rank}/rank) top{K} "
                     f"layers={args.layers} world={world} fused={args.fused} ckpt_level={args.ckpt_level} "
                     f"capacity_factor={args.capacity_factor}")
        from ..utils.roofline import layer_rooflines, load_peaks
        peaks = load_peaks()
        roof = layer_rooflines(T, H, I, K, world, peaks, experts_per_rank=args.experts_per_rank,
                               store_preact=args.ckpt_level == 0)
        lines.append(f"{'kernel':58s} {'calls/step':>10s} {'us/step':>10s} {'roofline us':>12s} {'fraction':>9s}  bound")
        for label, (n, us) in sorted(agg.items(), key=lambda kv: -kv[1][1]):
            row = f"{label:58s} {n / args.steps:10.1f} {us / args.steps:10.1f}"
            if label in roof and us > 0:
                r = roof[label]
                want = r.roofline_us * args.layers
                row += f" {want:12.1f} {want / (us / args.steps):9.2f}  {r.bound}"
            lines.append(row)
            total += us / args.steps
        lines.append(f"(roofline per kernel = slowest of its GEMM at {peaks.tflops:.0f} TFLOP/s, its HBM bytes at "
                     f"{peaks.hbm_gbs:.0f} GB/s and its NVLink bytes at {peaks.nvlink_gbs:.0f} GB/s, {peaks.label}; balanced routing assumed)")
        lines.append(f"{'serial sum of device kernels':58s} {'':10s} {total:10.1f}")
        lines.append(f"{'end-to-end step (median, max over ranks)':58s} {'':10s} {float(t[0]) * 1e3:10.1f}")
        lines.append(f"{'overlap saved (serial sum - e2e)':58s} {'':10s} {total - float(t[0]) * 1e3:10.1f}")
        lines.append(f"step times (ms): min {min(times):.3f} median {med:.3f} max {max(times):.3f}")
        lines.append(f"peak torch allocated {torch.cuda.max_memory_allocated() / 2**20:.0f} MiB, reserved "
                     f"{torch.cuda.max_memory_reserved() / 2**20:.0f} MiB; symmetric arena high water "
                     f"{buf.runtime.arena_high_water() / 2**20:.0f} MiB of {buf.runtime.arena_capacity() / 2**20:.0f} MiB")
        text = "\n".join(lines)
        print(text, flush=True)
        if args.out:
            with open(os.path.join(args.out, "full_kernel_table.txt"), "w") as f:
                f.write(text + "\n")
    if world > 1:
        dist.barrier(device_ids=[local])
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
