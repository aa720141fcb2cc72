"""Multi-process, one rank per GPU, checks of the real NVLink paths (launched by torchrun).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29533 tests/multigpu/layer_check.py [--scenario all|layer|comm|lopsided|missing_rank]

Covers what the reference's torchrun scripts cover (tests/test_dispatch.py, test_combine.py,
test_dispatch_grads.py, test_combine_grads.py, stream_ep/stream_moe/validate_multi_iter.py) plus a
host-made failure: a rank that does not join a dispatch.  Prints one PASS/FAIL line per check on
rank 0 and exits non-zero on any failure.
"""
import argparse
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from helpers import make_routing  # noqa: E402
from streamep_b200 import Buffer, StreamEPError  # noqa: E402
from streamep_b200.models.reference import (check_close, dispatch_layout_reference,  # noqa: E402
                                            moe_reference_grads, pool_reference)
from streamep_b200.stream_moe import make_streams, stream_moe_func  # noqa: E402

FAILS = []


def report(name, fn, rank):
    try:
        fn()
        ok, msg = True, ""
    except Exception as e:  # noqa: BLE001
        ok, msg = False, f"{type(e).__name__}: {e}"
    flags = [None] * dist.get_world_size()
    dist.all_gather_object(flags, (ok, msg))
    all_ok = all(f[0] for f in flags)
    if rank == 0:
        print(("PASS " if all_ok else "FAIL ") + name + ("" if all_ok else " :: " + " | ".join(
            f"rank {i}: {m}" for i, (o, m) in enumerate(flags) if not o)), flush=True)
    if not all_ok:
        FAILS.append(name)


def gather_list(t):
    out = [None] * dist.get_world_size()
    dist.all_gather_object(out, t.cpu())
    return out


def comm_checks(buf, rank, R, dev):
    T, H, K, E = 384 + 17 * rank, 512, 6, 8 * R
    g = torch.Generator(device="cpu").manual_seed(100 + rank)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16).to(dev)
    idx, w = make_routing(T, K, E, 200 + rank, dev, sentinel_p=0.05)
    xs, idxs, ws = gather_list(x), gather_list(idx), gather_list(w)
    layouts, sends = dispatch_layout_reference(idxs, E, buf.num_channels, 128, ws)
    L, S = layouts[rank], sends[rank]
    state = {}

    def dispatch():
        pool, h, _ = buf.dispatch(x, idx, w, None, E)
        torch.cuda.synchronize(); buf.check_status()
        state["h"] = h
        assert h.total_tiles == L.total_tiles
        for name in ("expert_frequency", "expert_pool_block_offset", "base_pool", "seen_per_substream",
                     "tile_id_to_expert", "pool_arrival_target", "pool_recv_token", "pool_k_slot",
                     "recv_token_to_slots", "k_local_total"):
            assert torch.equal(getattr(h, name).cpu(), getattr(L, name)), name
        assert torch.equal(h.pool_arrival_count.cpu(), L.pool_arrival_target)
        valid = L.pool_recv_token >= 0
        assert torch.equal(h.pool.cpu()[valid], pool_reference(L, xs)[valid]), "pool rows"
        assert torch.equal(h._dispatch_out.pair_slot.cpu(), S.pair_slot)

    def combine():
        h = state["h"]
        h.o.fill_(float(rank + 1)); h.y_done_per_token.fill_(h.dispatch_seq)
        out, _ = buf.combine(h.o, h)
        torch.cuda.synchronize(); buf.check_status()
        sent = (S.send_recv_token >= 0).float()
        want = (sent * torch.arange(1, R + 1).float()).sum(-1)
        assert torch.equal(out.float().cpu(), want[:, None].expand(T, H).contiguous())

    def grads():
        h = state["h"]
        dy = torch.randn(T, H, generator=g).to(torch.bfloat16).to(dev)
        dys = gather_list(dy)
        pool, cnt, _ = buf.dispatch_grads(h, dy)
        torch.cuda.synchronize(); buf.check_status()
        valid = L.pool_recv_token >= 0
        assert torch.equal(pool.cpu()[valid], pool_reference(L, dys)[valid])
        assert torch.equal(cnt.cpu(), L.pool_arrival_target)
        dx_r = torch.full((h.num_recv_tokens, H), float(rank + 1), dtype=torch.bfloat16, device=dev)
        wg = torch.full((h.TK_padded,), float(rank + 1), device=dev)
        done = torch.full((h.num_recv_tokens,), h.dispatch_seq, dtype=torch.int64, device=dev)
        dx, dw = buf.combine_grads(dx_r, h, wg, done)
        torch.cuda.synchronize(); buf.check_status()
        sent = (S.send_recv_token >= 0).float()
        want = (sent * torch.arange(1, R + 1).float()).sum(-1)
        assert torch.equal(dx.float().cpu(), want[:, None].expand(T, H).contiguous())
        EL = E // R
        want_w = torch.where(idx >= 0, (idx // EL + 1).float(), torch.zeros_like(w))
        assert torch.equal(dw, want_w)

    for rep in range(2):
        report(f"dispatch bit-exact (rep {rep})", dispatch, rank)
        report(f"combine closed form (rep {rep})", combine, rank)
        report(f"dispatch_grads + combine_grads (rep {rep})", grads, rank)


def layer_checks(buf, rank, R, dev, lopsided=False, tag0=""):
    """Layer forward + backward against the global fp32 oracle.  ``lopsided``: the last rank has no tokens
    and every pair goes to rank 0's experts, so every other rank receives nothing (empty pools, no tiles)
    but still takes part in every collective."""
    H, I, K = 512, 384, 4
    EL = 4
    E = EL * R
    T = 700 + 64 * rank
    if lopsided:
        T = 0 if rank == R - 1 else 300 + 32 * rank
    g = torch.Generator(device="cpu").manual_seed(7)
    w1_full = (torch.randn(E, 2 * I, H, generator=g) * 0.05).to(torch.bfloat16)
    w2_full = (torch.randn(E, H, I, generator=g) * 0.05).to(torch.bfloat16)
    gr = torch.Generator(device="cpu").manual_seed(300 + rank)
    x0 = torch.randn(T, H, generator=gr).to(torch.bfloat16).to(dev)
    idx, w0 = make_routing(T, K, E, 400 + rank, dev, sentinel_p=0.03)
    if lopsided:
        idx = torch.where(idx >= 0, idx % EL, idx)       # experts 0..EL-1 live on rank 0 (duplicates allowed)
    w0 = w0 / w0.sum(-1, keepdim=True).clamp_min(1e-6)
    dy = torch.randn(T, H, generator=gr).to(torch.bfloat16).to(dev)
    xs, idxs, ws, dys = gather_list(x0), gather_list(idx), gather_list(w0), gather_list(dy)
    # global oracle on this rank's device: all tokens of all ranks
    X, IDX, W, DY = (torch.cat(v).to(dev) for v in (xs, idxs, ws, dys))
    want_out, want_dx, want_dw, want_dw1, want_dw2 = moe_reference_grads(X, IDX, W, w1_full.to(dev), w2_full.to(dev), DY)
    off = sum(t.shape[0] for t in xs[:rank])
    sl = slice(off, off + T)
    streams = make_streams()
    s = lambda t: max(float(t.abs().max()), 1e-6)   # noqa: E731

    tag = tag0 + ("lopsided " if lopsided else "")
    for fused in ((True,) if buf.capacity_mode else (True, False)):
        for level in ((0, 2) if lopsided else (0, 1, 2)):
            def run():
                x = x0.clone().requires_grad_(True)
                w = w0.clone().requires_grad_(True)
                w1 = w1_full[rank * EL:(rank + 1) * EL].to(dev).requires_grad_(True)
                w2 = w2_full[rank * EL:(rank + 1) * EL].to(dev).requires_grad_(True)
                for it in range(2):
                    for t in (x, w, w1, w2):
                        t.grad = None
                    out = stream_moe_func(buf, x, idx, w, None, w1, w2, streams=streams, num_experts=E,
                                          activation_checkpoint_level=level, fused=fused)
                    out.backward(dy)
                    torch.cuda.synchronize(); buf.check_status()
                    if T > 0:
                        check_close("out", out, want_out[sl], 2e-2 * s(want_out), 2e-2)
                        check_close("dx", x.grad, want_dx[sl], 2e-2 * s(want_dx), 2e-2)
                        check_close("dw_topk", w.grad, want_dw[sl], 2e-2 * s(want_dw), 2e-2)
                    check_close("dW1", w1.grad, want_dw1[rank * EL:(rank + 1) * EL], 3e-2 * s(want_dw1), 3e-2)
                    check_close("dW2", w2.grad, want_dw2[rank * EL:(rank + 1) * EL], 3e-2 * s(want_dw2), 3e-2)
            report(f"{tag}layer fwd+bwd vs fp32 oracle (fused={fused}, ckpt level {level})", run, rank)


def missing_rank_check(buf, rank, R, dev):
    """Rank R-1 skips one dispatch on the host. The others' metadata wait runs out, they get an
    exception and a usable context; after `recover()` the group works again."""
    T, H, K, E = 128, 256, 2, 2 * R
    x = torch.randn(T, H, device=dev).to(torch.bfloat16)
    idx, w = make_routing(T, K, E, 900 + rank, dev)
    old = buf.runtime.get_timeout_ms()
    buf.set_timeout_ms(800)
    state = {"raised": False}

    def skip_and_timeout():
        if rank == R - 1:
            time.sleep(0.2)          # stays alive, launches nothing
        else:
            try:
                buf.dispatch(x, idx, w, None, E)
            except StreamEPError:
                state["raised"] = True
            assert state["raised"], "dispatch without a peer must raise"
    report("a rank that does not join: the others time out with an exception", skip_and_timeout, rank)

    def recover_and_continue():
        buf.recover()
        buf.set_timeout_ms(old)
        _, h, _ = buf.dispatch(x, idx, w, None, E)
        torch.cuda.synchronize(); buf.check_status()
        assert torch.equal(h.pool_arrival_count, h.pool_arrival_target)
    report("recover(): epochs re-agreed, next dispatch completes", recover_and_continue, rank)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--scenario", default="all")
    ap.add_argument("--allocator", default=None, choices=[None, "ipc", "vmm"],
                    help="arena allocator: cudaMalloc + CUDA IPC, or cuMemCreate + file descriptors + cuMemMap")
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    buf = Buffer(dist.group.WORLD, 1 << 30, timeout_ms=5000, allocator=args.allocator)
    if rank == 0:
        print(f"arena allocator: {buf.allocator}", flush=True)
    if args.scenario in ("all", "comm"):
        comm_checks(buf, rank, world, dev)
    if args.scenario in ("all", "layer"):
        layer_checks(buf, rank, world, dev)
    if args.scenario in ("all", "lopsided"):
        layer_checks(buf, rank, world, dev, lopsided=True)
    if args.scenario in ("all", "missing_rank"):
        missing_rank_check(buf, rank, world, dev)
    if args.scenario in ("all", "capacity"):
        # the same layer checks on fixed receive regions (no host read per forward); the lopsided case sends every
        # pair to rank 0, so the regions are sized for the whole group's pairs
        cbuf = Buffer(dist.group.WORLD, Buffer.capacity_mode_bytes(700 + 64 * world, 512, 4, 4 * world, world,
                                                                   capacity_factor=float(world) + 0.5) + (256 << 20),
                      timeout_ms=5000, allocator=args.allocator)
        cbuf.enable_capacity_mode(700 + 64 * world, 512, 4, 4 * world, capacity_factor=float(world) + 0.5)
        layer_checks(cbuf, rank, world, dev, tag0="capacity mode: ")
        layer_checks(cbuf, rank, world, dev, lopsided=True, tag0="capacity mode: ")
        report("capacity mode: no dispatch overflowed", lambda: cbuf.overflow_info()["count"] == 0 or (_ for _ in ()).throw(
            AssertionError(str(cbuf.overflow_info()))), rank)
    dist.barrier(device_ids=[local])
    torch.cuda.synchronize()
    if rank == 0:
        print("ALL PASS" if not FAILS else f"FAILED: {FAILS}", flush=True)
    dist.destroy_process_group()
    sys.exit(1 if FAILS else 0)


if __name__ == "__main__":
    main()
