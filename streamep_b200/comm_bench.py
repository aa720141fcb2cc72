"""Stand-alone dispatch / combine bandwidth (forward and grads directions).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29551 -m streamep_b200.comm_bench --tokens 4096 --hidden 7168 \
        --experts-per-rank 32 --topk 8

Plays the role of the bandwidth print-outs of the reference's torchrun scripts
(tests/test_dispatch.py, tests/test_combine.py, tests/test_dispatch_grads.py,
tests/test_combine_grads.py): uniform-random distinct experts per token, weights from a softmax
of N(0,1) logits.  Every op is timed on the device (CUDA events on the launching stream, median
over iterations, max over ranks) through the public ``Buffer`` calls, so a dispatch time includes
the metadata kernel, the host read of the receive sizes and the push kernel.

Bytes: ``pair`` counts one bf16 row per (token, expert) pair that leaves the rank (what the push
dispatch writes over NVLink: every pair lands in its own pool slot); ``dedup`` counts one row per
(token, distinct remote rank), the reference's wire model and what the pull combine reads.
``--impl nccl`` times ``all_to_all_single`` on the same pair rows as the library baseline.
One JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

import torch
import torch.distributed as dist


def make_uniform_routing(T, K, E, seed, dev):
    g = torch.Generator(device="cpu").manual_seed(seed)
    idx = torch.rand(T, E, generator=g).argsort(dim=1)[:, :K].contiguous()
    w = torch.softmax(torch.randn(T, K, generator=g), dim=-1)
    return idx.to(dev), w.to(dev)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--experts-per-rank", type=int, default=32)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="streamep_b200", choices=["streamep_b200", "nccl"])
    args = ap.parse_args()

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    group = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD

    T, H, K = args.tokens, args.hidden, args.topk
    EL = args.experts_per_rank
    E = EL * world
    torch.manual_seed(5 + rank)
    x = torch.randn(T, H, device=dev).to(torch.bfloat16)
    dy = torch.randn(T, H, device=dev).to(torch.bfloat16)
    idx, w = make_uniform_routing(T, K, E, 900 + rank, dev)
    dest = idx // EL
    remote_pairs = int((dest != rank).sum())
    in_rank = torch.zeros(T, world, dtype=torch.bool, device=dev)
    in_rank.scatter_(1, dest, True)
    remote_dedup = int(in_rank.sum()) - int(in_rank[:, rank].sum())
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def sync():
        if world > 1:
            dist.barrier(device_ids=[local])
        torch.cuda.synchronize()

    def timed(fn):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        flush.zero_()
        sync()
        e0.record()
        r = fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1), r

    times = {"dispatch": [], "combine": [], "dispatch_grads": [], "combine_grads": []}
    launches = 0
    if args.impl == "streamep_b200":
        from .models.moe_layer import make_buffer
        buf = make_buffer(group, T, H, K, E, world_size=world)
        l0 = buf.runtime.launch_count()
        for it in range(args.warmup + args.iters):
            t_d, (pool, h, _) = timed(lambda: buf.dispatch(x, idx, w, in_rank, E))
            h.o.fill_(1.0)
            h.y_done_per_token.fill_(h.dispatch_seq)
            t_c, _ = timed(lambda: buf.combine(h.o, h))
            t_g, _ = timed(lambda: buf.dispatch_grads(h, dy))
            dx_r = torch.ones(h.num_recv_tokens, H, dtype=torch.bfloat16, device=dev)
            wg = torch.ones(h.TK_padded, device=dev)
            done = torch.full((h.num_recv_tokens,), h.dispatch_seq, dtype=torch.int64, device=dev)
            t_cg, _ = timed(lambda: buf.combine_grads(dx_r, h, wg, done))
            sync()
            buf.check_status()
            del pool, h, dx_r, wg, done
            if it >= args.warmup:
                for k, v in zip(times, (t_d, t_c, t_g, t_cg)):
                    times[k].append(v)
        launches = buf.runtime.launch_count() - l0
    else:
        order = torch.argsort(dest.reshape(-1), stable=True)
        send_splits = torch.bincount(dest.reshape(-1), minlength=world)
        recv_splits = torch.empty_like(send_splits)
        if world > 1:
            dist.all_to_all_single(recv_splits, send_splits, group=group)
        else:
            recv_splits.copy_(send_splits)
        ss, rs = send_splits.tolist(), recv_splits.tolist()

        def a2a(src, out_splits, in_splits):
            out = src.new_empty(sum(out_splits), H)
            if world > 1:
                dist.all_to_all_single(out, src, out_splits, in_splits, group=group)
            else:
                out.copy_(src)
            return out

        for it in range(args.warmup + args.iters):
            t_d, recv = timed(lambda: a2a(x[order // K], rs, ss))
            t_c, _ = timed(lambda: a2a(recv, ss, rs))
            t_g, recv_g = timed(lambda: a2a(dy[order // K], rs, ss))
            t_cg, _ = timed(lambda: a2a(recv_g, ss, rs))
            if it >= args.warmup:
                for k, v in zip(times, (t_d, t_c, t_g, t_cg)):
                    times[k].append(v)

    med = torch.tensor([statistics.median(times[k]) for k in times], device=dev)
    counts = torch.tensor([remote_pairs, remote_dedup], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(med, op=dist.ReduceOp.MAX)
        dist.all_reduce(counts, op=dist.ReduceOp.SUM)
        counts /= world
    if rank == 0:
        row = H * 2
        out = {"metric": "dispatch_combine_bandwidth", "impl": args.impl, "n_gpus": world, "dtype": "bf16",
               "config": {"tokens_per_rank": T, "hidden": H, "experts": E, "experts_per_rank": EL, "topk": K,
                          "routing": "uniform random distinct experts", "l2_flush": "256 MiB rewritten before every op"},
               "remote_pairs_per_rank": float(counts[0]), "remote_token_rank_rows_per_rank": float(counts[1]),
               "iters": args.iters, "warmup": args.warmup, "gpu_launches": int(launches), "ops": {}}
        for i, k in enumerate(times):
            ms = float(med[i])
            # the push directions move one row per pair, the pull directions one per (token, rank);
            # the library all-to-all moves pair rows both ways
            pair_dir = k in ("dispatch", "dispatch_grads") or args.impl == "nccl"
            rows = float(counts[0] if pair_dir else counts[1])
            out["ops"][k] = {"ms": round(ms, 4), "nvlink_rows_per_rank": rows,
                             "gbs_per_rank": round(rows * row / (ms * 1e-3) / 1e9, 1) if ms > 0 else None,
                             "dedup_model_gbs_per_rank": round(float(counts[1]) * row / (ms * 1e-3) / 1e9, 1) if ms > 0 else None}
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier(device_ids=[local])
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
