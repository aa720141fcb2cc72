"""End-to-end numerical validator: streaming layer stack vs the eager fp32 full-MoE oracle, output
and all four gradients, over several iterations and layers, with optional stress knobs (role of the
reference's stream_ep/stream_moe/validate_multi_iter.py:118-186,216-263,288-294,559-575).

    python -m streamep_b200.stream_moe.validate_multi_iter --tokens 2048 --layers 2 --iters 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 \
        --master-port 29561 -m streamep_b200.stream_moe.validate_multi_iter --routing power_law --lag-us 200

Every rank gathers all ranks' inputs and evaluates the global oracle itself, so keep the shapes
moderate.  Fail rule per element: ``|diff| > atol`` AND ``|diff| > rtol * |want|`` with
(atol, rtol) = (2e-2 * max|want|, 2e-2) for out / dx / dtopk and (3e-2 * max|want|, 3e-2) for dW,
scaled by sqrt(layers).
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
    args = ap.parse_args()
    rank, world, local, dev, group = init_distributed()
    T = 128 if (args.uneven and rank == 0) else args.tokens
    buf, layers, E = build_layers(args, group, world, dev)
    H, K, L = args.hidden, args.topk, args.layers
    side = torch.cuda.Stream()
    ballast = torch.empty(args.side_ar_mb << 20, dtype=torch.uint8, device=dev) if args.side_ar_mb else None
    scale = math.sqrt(L)
    fails = 0
    for it in range(args.iters):
        torch.manual_seed(100 * it + rank)
        x0 = torch.randn(T, H, device=dev).to(torch.bfloat16)
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
        for name, got, want, tol in checks:
            try:
                check_close(name, got, want, atol=tol * s(want) * scale, rtol=tol * scale)
            except AssertionError as e:
                msgs.append(str(e))
        for layer in layers:
            layer.w1.grad = None
            layer.w2.grad = None
        flag = torch.tensor([len(msgs)], device=dev)
        if world > 1:
            dist.all_reduce(flag)
        fails += int(flag.item())
        print(f"[rank {rank}] iter {it}: {'PASS' if not msgs else 'FAIL ' + ' | '.join(msgs)}  "
              f"(torch peak {torch.cuda.max_memory_allocated() / 2**20:.0f} MiB, arena high water "
              f"{buf.runtime.arena_high_water() / 2**20:.0f} MiB)", flush=True)
        _ = sizes
    barrier(world, local)
    rank_zero_print(rank, "ALL PASS" if fails == 0 else f"FAILED checks: {fails}")
    if world > 1:
        dist.destroy_process_group()
    return 0 if fails == 0 else 1


if __name__ == "__main__":
    sys.exit(main())
