"""End-to-end numerical validator: streaming layer stack vs the eager fp32 full-MoE oracle, output
and all four gradients, over several iterations and layers, with optional stress knobs (role of the
reference's stream_ep/stream_moe/validate_multi_iter.py:118-186,216-263,288-294,559-575).

    python -m streamep_b200.stream_moe.validate_multi_iter --tokens 2048 --layers 2 --iters 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 \
        --master-port 29561 -m streamep_b200.stream_moe.validate_multi_iter --routing power_law --lag-us 200

    # the reference validator's own data recipe, fail rule and tolerances at the flagship shape, capacity mode:
    python -m torch.distributed.run ... -m streamep_b200.stream_moe.validate_multi_iter --ref-tolerances \
        --tokens 8192 --hidden 2048 --ffn 1408 --experts-per-rank 8 --topk 6 --capacity-factor 1.5
    # depth stress (role of tests/test_pipeline_depth_stress.py and tests/test_dispatch_grads_stress.py of the
    # reference): 44 layers, GPU-side lag on odd ranks, NCCL all-reduce side load, no oracle:
    python -m torch.distributed.run ... -m streamep_b200.stream_moe.validate_multi_iter --layers 44 --no-ref \
        --lag-us 300 --side-ar-mb 64 --side-matmul 4096

Every rank gathers all ranks' inputs and evaluates the global fp32 oracle itself (about 20 TFLOP of fp32 and
12 GB at the flagship shape on 8 ranks).  Fail rule per element: ``|diff| > atol`` AND ``|diff| > rtol * |want|``.
Default tolerances are relative to the data: (atol, rtol) = (2e-2 * max|want|, 2e-2) for out / dx / dtopk and
(3e-2 * max|want|, 3e-2) for dW.  ``--ref-tolerances`` switches to the reference validator's recipe
(stream_ep/stream_moe/validate_multi_iter.py:86-92,320-354,559-575): x and dL/dy scaled by 0.1, weights
N(0, 0.02), top-k weights a softmax of N(0, 1), absolute tolerances (1e-3, 1e-2) for out / dx / dtopk and
(8e-2, 8e-2) for dW with ``rel = diff / (|ref| + 1e-3)``.  All tolerances are scaled by sqrt(layers).

``--no-ref`` skips the oracle (deep stacks): it checks that every output and gradient is finite, that results
repeat bit-for-bit in the deterministic parts (``dL/dtopk_weights`` per layer is reduced in a fixed order) and
within bf16 noise elsewhere from iteration to iteration when the inputs repeat, that no bounded wait gave up,
that no step takes longer than ``--max-step-ratio`` x the median, and that the symmetric arena is back to its
starting level after every iteration.
"""
from __future__ import annotations

import argparse
import math
import sys

import torch
import torch.distributed as dist

from ..models.reference import check_close, moe_reference_forward
from ._harness_common import add_shape_args, barrier, build_layers, init_distributed, rank_zero_print

ROUTINGS = ("router", "uniform_rotating", "half_empty_experts", "per_rank_imbalance", "power_law", "all_to_first_k")


def make_routing(kind, layer, x, T, K, E, world, rank, it, dev):
    """Deterministic stress routings of the reference's tests/test_skewed_experts.py."""
    g = torch.Generator(device="cpu").manual_seed(1000 * it + 17 * rank + 3)
    if kind == "router":
        idx, w, _ = layer.route(x)
        return idx, w
    if kind == "uniform_rotating":
        base = (torch.arange(T)[:, None] * K + torch.arange(K)[None, :] + it) % E
    elif kind == "half_empty_experts":
        base = ((torch.arange(T)[:, None] * K + torch.arange(K)[None, :]) % (E // 2)) * 2
    elif kind == "per_rank_imbalance":
        hot = torch.rand(T, K, generator=g) < 0.9
        el = E // world
        base = torch.where(hot, torch.randint(0, el, (T, K), generator=g), torch.randint(0, E, (T, K), generator=g))
    elif kind == "power_law":
        p = 1.0 / torch.arange(1, E + 1).float() ** 1.2
        base = torch.multinomial(p.expand(T, E), K, replacement=False, generator=g)
    elif kind == "all_to_first_k":
        base = torch.arange(K).expand(T, K)
    else:
        raise ValueError(kind)
    w = torch.rand(T, K, generator=g)
    w = w / w.sum(-1, keepdim=True)
    return base.to(torch.int64).contiguous().to(dev), w.to(dev)


def gather_cat(t, world):
    if world == 1:
        return t
    sizes = [torch.zeros(1, dtype=torch.long, device=t.device) for _ in range(world)]
    dist.all_gather(sizes, torch.tensor([t.shape[0]], device=t.device))
    mx = int(max(s.item() for s in sizes))
    pad = torch.zeros((mx,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
    pad[:t.shape[0]] = t
    outs = [torch.empty_like(pad) for _ in range(world)]
    dist.all_gather(outs, pad)
    return torch.cat([o[:int(s.item())] for o, s in zip(outs, sizes)])


def main():
    ap = argparse.ArgumentParser()
    add_shape_args(ap)
    ap.set_defaults(tokens=2048, hidden=512, ffn=384, experts_per_rank=4, topk=4)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--routing", default="router", choices=ROUTINGS)
    ap.add_argument("--uneven", action="store_true", help="rank 0 gets 128 tokens, the others --tokens")
    ap.add_argument("--lag-us", type=float, default=0.0, help="GPU-side delay injected on odd ranks before each layer")
    ap.add_argument("--side-ar-mb", type=int, default=0, help="NCCL all-reduce of this many MiB per iteration on a side stream")
    ap.add_argument("--side-matmul", type=int, default=0, help="square bf16 matmul of this size per layer on a side stream (SM contention)")
    ap.add_argument("--ref-tolerances", action="store_true", help="the reference validator's data recipe, fail rule and tolerances")
    ap.add_argument("--no-ref", action="store_true", help="no oracle: finiteness, repeatability, status and arena level only")
    ap.add_argument("--imbalance", type=float, default=1.5, help="arena sizing factor for skewed routings")
    ap.add_argument("--max-step-ratio", type=float, default=0.0, help="> 0: fail when a step takes longer than this many medians")
    args = ap.parse_args()
    if args.no_ref:
        return stress_main(args)
    rank, world, local, dev, group = init_distributed()
    T = 128 if (args.uneven and rank == 0) else args.tokens
    buf, layers, E = build_layers(args, group, world, dev)
    H, K, L = args.hidden, args.topk, args.layers
    side = torch.cuda.Stream()
    ballast = torch.empty(args.side_ar_mb << 20, dtype=torch.uint8, device=dev) if args.side_ar_mb else None
    scale = math.sqrt(L)
    fails = 0
    ref_tol = args.ref_tolerances
    x_scale = 0.1 if ref_tol else 1.0
    for it in range(args.iters):
        torch.manual_seed(100 * it + rank)
        x0 = (torch.randn(T, H, device=dev) * x_scale).to(torch.bfloat16)
        dy = (torch.randn(T, H, device=dev) * 0.1).to(torch.bfloat16)
        x = x0.clone().requires_grad_(True)
        routes, ws = [], []
        cur = x
        if ballast is not None and world > 1:
            with torch.cuda.stream(side):
                dist.all_reduce(ballast.view(torch.int8))
        for layer in layers:
            if args.lag_us > 0 and rank % 2 == 1:
                torch.cuda._sleep(int(args.lag_us * 1900))
            idx, w = make_routing(args.routing, layer, cur.detach(), T, K, E, world, rank, it, dev)
            if ref_tol:     # the reference draws the top-k weights as a softmax of N(0, 1) logits
                w = torch.softmax(torch.randn(T, K, device=dev), dim=-1)
            w = w.clone().requires_grad_(True)
            routes.append(idx); ws.append(w)
            cur = layer.experts(cur, idx, w, None)
        cur.backward(dy)
        torch.cuda.synchronize()
        buf.check_status()
        # ---- global oracle (fp32, all ranks' tokens, all experts)
        Xg = gather_cat(x0, world).float().requires_grad_(True)
        DYg = gather_cat(dy, world).float()
        w1_full = [gather_cat(layer.w1.detach(), world).float().requires_grad_(True) for layer in layers]
        w2_full = [gather_cat(layer.w2.detach(), world).float().requires_grad_(True) for layer in layers]
        Wg = [gather_cat(w.detach(), world).float().requires_grad_(True) for w in ws]
        Ig = [gather_cat(i, world) for i in routes]
        ref = Xg
        for l in range(L):
            # the streaming stack rounds every layer's output to bf16; mirror it
            ref = moe_reference_forward(ref, Ig[l], Wg[l], w1_full[l], w2_full[l], out_dtype=torch.float32)
            ref = ref + (ref.to(torch.bfloat16).float() - ref).detach()
        grads = torch.autograd.grad(ref, [Xg] + Wg + w1_full + w2_full, DYg)
        sizes = [T] if world == 1 else None
        off = 0
        if world > 1:
            all_T = [torch.zeros(1, dtype=torch.long, device=dev) for _ in range(world)]
            dist.all_gather(all_T, torch.tensor([T], device=dev))
            off = int(sum(t.item() for t in all_T[:rank]))
        sl = slice(off, off + T)
        el = E // world
        esl = slice(rank * el, (rank + 1) * el)
        s = lambda t: max(float(t.abs().max()), 1e-6)   # noqa: E731
        checks = [("out", cur, ref.detach()[sl], 2e-2), ("dL_dx", x.grad, grads[0][sl], 2e-2)]
        for l in range(L):
            checks.append((f"dL_dtopk_weights[{l}]", ws[l].grad, grads[1 + l][sl], 2e-2))
            checks.append((f"dW1[{l}]", layers[l].w1.grad, grads[1 + L + l][esl], 3e-2))
            checks.append((f"dW2[{l}]", layers[l].w2.grad, grads[1 + 2 * L + l][esl], 3e-2))
        msgs = []
        worst = []
        for name, got, want, tol in checks:
            try:
                if ref_tol:
                    atol, rtol = (8e-2, 8e-2) if name.startswith("dW") else (1e-3, 1e-2)
                    check_close(name, got, want, atol=atol * scale, rtol=rtol * scale, rel_floor=1e-3)
                else:
                    check_close(name, got, want, atol=tol * s(want) * scale, rtol=tol * scale)
            except AssertionError as e:
                msgs.append(str(e))
            worst.append(f"{name} max|diff| {float((got.detach().float() - want.detach().to(got.device).float()).abs().max()):.2e} of max|ref| {s(want):.2e}")
        for layer in layers:
            layer.w1.grad = None
            layer.w2.grad = None
        flag = torch.tensor([len(msgs)], device=dev)
        if world > 1:
            dist.all_reduce(flag)
        fails += int(flag.item())
        if rank == 0 and it == 0:
            print("[rank 0] " + "; ".join(worst), flush=True)
        print(f"[rank {rank}] iter {it}: {'PASS' if not msgs else 'FAIL ' + ' | '.join(msgs)}  "
              f"(torch peak {torch.cuda.max_memory_allocated() / 2**20:.0f} MiB, arena high water "
              f"{buf.runtime.arena_high_water() / 2**20:.0f} MiB)", flush=True)
        _ = sizes
    barrier(world, local)
    rank_zero_print(rank, f"config: tokens/rank={args.tokens} hidden={H} ffn={args.ffn} experts={E} top{K} layers={L} world={world} "
                          f"fused={args.fused} ckpt={args.ckpt_level} capacity_factor={args.capacity_factor} routing={args.routing} "
                          f"tolerances={'reference (1e-3,1e-2)/(8e-2,8e-2), rel floor 1e-3' if ref_tol else 'relative 2e-2 / 3e-2 of max|ref|'}")
    rank_zero_print(rank, "ALL PASS" if fails == 0 else f"FAILED checks: {fails}")
    if world > 1:
        dist.destroy_process_group()
    return 0 if fails == 0 else 1


def stress_main(args):
    """Deep stack under injected lag and side load, without the oracle (see the module docstring)."""
    import statistics

    rank, world, local, dev, group = init_distributed()
    T = 128 if (args.uneven and rank == 0) else args.tokens
    buf, layers, E = build_layers(args, group, world, dev)
    H, K, L = args.hidden, args.topk, args.layers
    side, side2 = torch.cuda.Stream(), torch.cuda.Stream()
    ballast = torch.empty(args.side_ar_mb << 20, dtype=torch.uint8, device=dev) if args.side_ar_mb else None
    mm = torch.randn(args.side_matmul, args.side_matmul, device=dev).to(torch.bfloat16) if args.side_matmul else None
    torch.manual_seed(7 + rank)
    x0 = (torch.randn(T, H, device=dev) * 0.5).to(torch.bfloat16)
    dy = (torch.randn(T, H, device=dev) * 0.1).to(torch.bfloat16)
    routes = [make_routing(args.routing, layer, x0, T, K, E, world, rank, 0, dev) for layer in layers]
    torch.cuda.synchronize()
    base_level = buf.runtime.arena_bytes_in_use()
    first, fails, times = None, [], []
    for it in range(args.iters):
        x = x0.clone().requires_grad_(True)
        ws = [w.clone().requires_grad_(True) for _, w in routes]
        barrier(world, local)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        if ballast is not None and world > 1:
            with torch.cuda.stream(side):
                dist.all_reduce(ballast.view(torch.int8))
        cur = x
        for l, layer in enumerate(layers):
            if args.lag_us > 0 and rank % 2 == 1 and l % 3 == 0:
                torch.cuda._sleep(int(args.lag_us * 1900))
            if mm is not None and l % 4 == 0:
                with torch.cuda.stream(side2):
                    torch.matmul(mm, mm)
            # residual stack: a residual-free chain of random layers is chaotic (bf16 reduction-order noise of one
            # layer is amplified by the next), which would make "results repeat" meaningless at this depth
            cur = cur + layer.experts(cur, routes[l][0], ws[l], None)
        cur.backward(dy)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
        try:
            buf.check_status()
        except Exception as e:  # noqa: BLE001
            fails.append(f"iter {it}: {e}")
        outs = [cur.detach(), x.grad] + [w.grad for w in ws] + [p.grad for layer in layers for p in (layer.w1, layer.w2)]
        if not all(torch.isfinite(t.float()).all() for t in outs):
            fails.append(f"iter {it}: non-finite values")
        snap = [cur.detach().float().clone(), x.grad.float().clone(), layers[0].w1.grad.float().clone()]
        if first is None:
            first = snap
        else:
            for name, a, b in zip(("out", "dL_dx", "dW1[0]"), snap, first):
                sc = max(float(b.abs().max()), 1e-6)
                if float((a - b).abs().max()) > 5e-2 * sc * math.sqrt(L):
                    fails.append(f"iter {it}: {name} does not repeat (max|diff| {float((a - b).abs().max()):.3e} of {sc:.3e})")
        for layer in layers:
            layer.w1.grad = None
            layer.w2.grad = None
        del cur, x, ws, outs, snap
        import gc
        gc.collect()
        if buf.runtime.arena_bytes_in_use() != base_level:
            fails.append(f"iter {it}: arena level {buf.runtime.arena_bytes_in_use()} != {base_level}")
    med = statistics.median(times)
    if args.max_step_ratio > 0 and len(times) > 2 and max(times[1:]) > args.max_step_ratio * med:
        fails.append(f"slowest step {max(times[1:]):.2f} ms > {args.max_step_ratio} x median {med:.2f} ms")
    flag = torch.tensor([len(fails)], device=dev)
    if world > 1:
        dist.all_reduce(flag)
    print(f"[rank {rank}] stress: {'PASS' if not fails else 'FAIL ' + ' | '.join(fails)} (steps ms: "
          f"{' '.join(f'{t:.1f}' for t in times)}; arena high water {buf.runtime.arena_high_water() / 2**20:.0f} MiB)", flush=True)
    barrier(world, local)
    rank_zero_print(rank, f"config: stress layers={L} iters={args.iters} tokens/rank={args.tokens} hidden={H} ffn={args.ffn} experts={E} "
                          f"top{K} world={world} fused={args.fused} ckpt={args.ckpt_level} capacity_factor={args.capacity_factor} "
                          f"routing={args.routing} lag_us={args.lag_us} side_ar_mb={args.side_ar_mb} side_matmul={args.side_matmul}")
    rank_zero_print(rank, "ALL PASS" if int(flag.item()) == 0 else f"FAILED checks: {int(flag.item())}")
    if world > 1:
        dist.destroy_process_group()
    return 0 if int(flag.item()) == 0 else 1


if __name__ == "__main__":
    sys.exit(main())
