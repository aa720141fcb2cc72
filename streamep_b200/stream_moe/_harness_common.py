"""Shared set-up of the layer harnesses: process group, buffer, layers, synthetic inputs."""
from __future__ import annotations

import os

import torch
import torch.distributed as dist


def init_distributed():
    """Returns ``(rank, world, local_rank, device, group)``; a single process needs no launcher."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    group = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if not dist.is_initialized():
            dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD
    return rank, world, local, dev, group


def barrier(world, local):
    if world > 1:
        dist.barrier(device_ids=[local])
    torch.cuda.synchronize()


def rank_zero_print(rank, *a, **k):
    if rank == 0:
        print(*a, flush=True, **k)


def add_shape_args(ap):
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--ffn", type=int, default=1408)
    ap.add_argument("--experts-per-rank", type=int, default=8)
    ap.add_argument("--topk", type=int, default=6)
    ap.add_argument("--layers", type=int, default=1)
    ap.add_argument("--fused", type=int, default=1)
    ap.add_argument("--ckpt-level", type=int, default=0)
    ap.add_argument("--capacity-factor", type=float, default=0.0,
                    help="> 0: capacity mode (fixed receive regions of this many times the balanced load, no host read "
                         "per forward); 0: exact host-sized buffers")


def build_layers(args, group, world, dev):
    from ..models.moe_layer import StreamMoE, make_buffer
    E = args.experts_per_rank * world
    cf = getattr(args, "capacity_factor", 0.0)
    buf = make_buffer(group, args.tokens, args.hidden, args.topk, E, layers_in_flight=args.layers, world_size=world,
                      imbalance=getattr(args, "imbalance", 1.5), capacity_factor=cf if cf > 0 else None)
    layers = [StreamMoE(args.hidden, args.ffn, E, args.topk, buf, fused=bool(args.fused),
                        activation_checkpoint_level=args.ckpt_level, device=dev, seed=10 + i)
              for i in range(args.layers)]
    return buf, layers, E
