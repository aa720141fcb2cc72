"""Single-GPU stand-alone launches of the layer's GEMM kernels, for ``ncu`` and for roofline numbers.

Producer/consumer pairs that spin on each other cannot be replayed by a profiler, so each kernel
is launched alone on a hand-built pool with its gates already open (same idea as the reference's
stream_ep/stream_moe/ncu_microbench.py:6-21,87-91,273-279).

    python -m streamep_b200.stream_moe.ncu_microbench --kernel a --hidden 2048 --ffn 1408 \
        --experts 8 --rows-per-expert 2048 --iters 5
    ncu --set full --clock-control none -k regex:grouped_gemm -c 3 -o prof \
        python -m streamep_b200.stream_moe.ncu_microbench --kernel a --rows-per-expert 1024 --iters 1 --warmup 1

Prints one JSON line per kernel: device time (CUDA events, L2 flushed between iterations),
achieved TFLOP/s and the fraction of the measured cuBLAS bf16 peak from ``MEASURED_PEAKS.json``
(fallback 1590 TFLOP/s burst when the file is absent).
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from ..ops import grouped_gemm as gg

KERNELS = ("a", "a_preact", "y", "y_bwd", "a_bwd", "dw1", "dw2", "dw_merged", "preact", "cublas")


def _peaks():
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        with open(os.path.join(here, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return float(p["bf16_tflops"]), float(p["hbm_gbs"]), "of measured"
    except (OSError, KeyError, ValueError):
        return 1590.0, 6650.0, "of fallback"


def build_case(hidden, ffn, experts, rows_per_expert, device="cuda", seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    tiles_per_e = (rows_per_expert + 127) // 128
    total = tiles_per_e * experts
    rows = total * 128
    recv = torch.full((rows,), -1, dtype=torch.int32)
    tile_e = torch.zeros(total, dtype=torch.int32)
    for e in range(experts):
        r0 = e * tiles_per_e * 128
        recv[r0:r0 + rows_per_expert] = torch.arange(e * rows_per_expert, (e + 1) * rows_per_expert, dtype=torch.int32)
        tile_e[e * tiles_per_e:(e + 1) * tiles_per_e] = e
    c = dict(
        pool=torch.randn(rows, hidden, generator=g).to(torch.bfloat16).to(device),
        w1=(torch.randn(experts, 2 * ffn, hidden, generator=g) * 0.02).to(torch.bfloat16).to(device),
        w2=(torch.randn(experts, hidden, ffn, generator=g) * 0.02).to(torch.bfloat16).to(device),
        recv=recv.to(device), tile_e=tile_e.to(device), wts=torch.rand(rows, generator=g).to(device),
        offsets=(torch.arange(experts + 1, dtype=torch.int32) * tiles_per_e).to(device),
        freqs=torch.full((experts,), rows_per_expert, dtype=torch.int32, device=device),
        rows=rows, total_tiles=total, n_recv=experts * rows_per_expert)
    c["postact"] = torch.empty(rows, ffn, dtype=torch.bfloat16, device=device)
    c["preact"] = torch.randn(rows, 2 * ffn, generator=g).to(torch.bfloat16).to(device)
    c["dswiglu_in"] = torch.randn(rows, 2 * ffn, generator=g).to(torch.bfloat16).to(device)
    c["o"] = torch.zeros(c["n_recv"], hidden, dtype=torch.bfloat16, device=device)
    c["dlw"] = torch.zeros(rows, dtype=torch.float32, device=device)
    c["dw1"] = torch.empty(experts, 2 * ffn, hidden, dtype=torch.bfloat16, device=device)
    c["dw2"] = torch.empty(experts, hidden, ffn, dtype=torch.bfloat16, device=device)
    c["postact"].copy_(torch.randn(rows, ffn, generator=g).to(torch.bfloat16))
    return c


def make_launcher(kernel, c, tile_n=None):
    rows, H, I = c["rows"], c["pool"].shape[1], c["postact"].shape[1]
    pairs = rows
    if kernel == "a":
        return (lambda: gg.streaming_moe_a(c["pool"], c["w1"], c["tile_e"], postact_a=c["postact"], tile_n=tile_n)), \
            2.0 * pairs * H * 2 * I, pairs * (H + I) * 2 + c["w1"].numel() * 2
    if kernel == "a_preact":
        return (lambda: gg.streaming_moe_a(c["pool"], c["w1"], c["tile_e"], postact_a=c["postact"], preact_a=c["preact"],
                                           tile_n=tile_n)), 2.0 * pairs * H * 2 * I, pairs * (H + 3 * I) * 2 + c["w1"].numel() * 2
    if kernel == "preact":
        return (lambda: gg.grouped_gemm_preact(c["pool"], c["w1"], c["tile_e"], out=c["preact"], tile_n=tile_n)), \
            2.0 * pairs * H * 2 * I, pairs * (H + 2 * I) * 2 + c["w1"].numel() * 2
    if kernel == "y":
        return (lambda: gg.streaming_moe_y(c["postact"], c["w2"], c["tile_e"], c["wts"], c["recv"], o=c["o"], tile_n=tile_n)), \
            2.0 * pairs * H * I, pairs * (I + 2 * H) * 2 + c["w2"].numel() * 2
    if kernel == "y_bwd":
        return (lambda: gg.streaming_moe_y_bwd(c["pool"], c["w2"], c["preact"], c["tile_e"], c["wts"], c["recv"],
                                               dL_dswiglu_in=c["dswiglu_in"], postact_a_for_dW2=c["postact"],
                                               dL_dweight=c["dlw"], tile_n=tile_n)), \
            2.0 * pairs * H * I, pairs * (H + 5 * I) * 2 + c["w2"].numel() * 2
    if kernel == "a_bwd":
        return (lambda: gg.streaming_moe_a_bwd(c["dswiglu_in"], c["w1"], c["tile_e"], c["recv"], dL_dx_per_r=c["o"],
                                               tile_n=tile_n)), 2.0 * pairs * H * 2 * I, pairs * (2 * I + 2 * H) * 2 + c["w1"].numel() * 2
    if kernel == "dw1":
        return (lambda: gg.grouped_gemm_dw(c["dswiglu_in"], c["pool"], c["offsets"], c["freqs"], out=c["dw1"], tile_n=tile_n)), \
            2.0 * pairs * H * 2 * I, pairs * (2 * I + H) * 2 + c["w1"].numel() * 2
    if kernel == "dw2":
        return (lambda: gg.grouped_gemm_dw(c["pool"], c["postact"], c["offsets"], c["freqs"], out=c["dw2"], tile_n=tile_n)), \
            2.0 * pairs * H * I, pairs * (I + H) * 2 + c["w2"].numel() * 2
    if kernel == "dw_merged":   # dW1 and dW2 in one launch, tiles claimed from a device counter (what the layer runs)
        return (lambda: gg.grouped_gemm_dw(c["dswiglu_in"], c["pool"], c["offsets"], c["freqs"], out=c["dw1"], lhs2=c["pool"],
                                           rhs2=c["postact"], out2=c["dw2"], tile_n=tile_n or 256, dynamic_tiles=True)), \
            6.0 * pairs * H * I, pairs * (3 * I + 2 * H) * 2 + (c["w1"].numel() + c["w2"].numel()) * 2
    if kernel == "router":   # tokens = rows, experts = --router-experts, top-6
        E = c["router_experts"]
        g = torch.Generator(device="cpu").manual_seed(3)
        wg = (torch.randn(E, H, generator=g) * 0.02).to(torch.bfloat16).to(c["pool"].device)
        return (lambda: gg.router_topk(c["pool"], wg, min(6, E), num_ranks=1)), 2.0 * rows * H * E, rows * H * 2 + E * H * 2
    if kernel == "cublas":   # yardstick: the library GEMM of kernel A's FLOPs (one expert's weights)
        w = c["w1"][0]
        return (lambda: torch.matmul(c["pool"], w.t())), 2.0 * pairs * H * 2 * I, pairs * (H + 2 * I) * 2 + w.numel() * 2
    raise ValueError(kernel)


def time_kernel(fn, iters, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    ts = []
    for _ in range(iters):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); fn(); e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2] if ts else float("nan")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", default="all", help="one of %s or 'all'" % ", ".join(KERNELS))
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--ffn", type=int, default=1408)
    ap.add_argument("--experts", type=int, default=8)
    ap.add_argument("--rows-per-expert", type=int, default=6144)
    ap.add_argument("--tile-n", type=int, default=None)
    ap.add_argument("--router-experts", type=int, default=64, help="expert count of --kernel router (not part of 'all')")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args()
    peak_tf, peak_bw, label = _peaks()
    c = build_case(args.hidden, args.ffn, args.experts, args.rows_per_expert)
    c["router_experts"] = args.router_experts
    names = KERNELS if args.kernel == "all" else (args.kernel,)
    for name in names:
        fn, flops, nbytes = make_launcher(name, c, args.tile_n)
        ms = time_kernel(fn, args.iters, args.warmup)
        msg = gg.default_runtime().poll_status(True)
        tf = flops / ms / 1e9
        print(json.dumps({"kernel": name, "hidden": args.hidden, "ffn": args.ffn, "experts": args.experts,
                          "rows": c["rows"], "tile_n": args.tile_n, "ms": round(ms, 4), "tflops": round(tf, 1),
                          "frac_bf16_peak": round(tf / peak_tf, 3), "algorithmic_gbs": round(nbytes / ms / 1e6, 1),
                          "frac_hbm": round(nbytes / ms / 1e6 / peak_bw, 3), "peaks": label, "status": msg or "ok"}))


if __name__ == "__main__":
    main()
