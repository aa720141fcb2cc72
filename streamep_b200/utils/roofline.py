"""Roofline arithmetic for one MoE layer step: algorithmic FLOPs and bytes of every logical kernel, and the
time each would take at the measured peaks.

A fused compute + collective kernel is bounded by the slower of its GEMM at the tensor-core peak and the bytes
it must move over NVLink at link bandwidth; a local kernel by the slower of its GEMM and its HBM traffic.
The denominators are measured ones: ``MEASURED_PEAKS.json`` at the repository root when present (a cuBLAS bf16
GEMM and a device copy on this machine), otherwise the stated fallbacks.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Dict, Optional

NVLINK_GBS = 770.0          # measured peer copy per direction per GPU on the B200 / NVSwitch boxes used here
FALLBACK_TFLOPS = 1590.0    # cuBLAS bf16 burst, earlier measurement on the same pool
FALLBACK_HBM_GBS = 6650.0


@dataclass(frozen=True)
class Peaks:
    tflops: float
    hbm_gbs: float
    nvlink_gbs: float
    label: str               # "of measured" or "of fallback"


def load_peaks(path: Optional[str] = None, sustained: bool = False) -> Peaks:
    if path is None:
        here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        path = os.path.join(here, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        tf = d["bf16_tflops_sustained" if sustained else "bf16_tflops"]
        return Peaks(float(tf), float(d["hbm_gbs"]), NVLINK_GBS, "of measured")
    except (OSError, KeyError, ValueError):
        return Peaks(FALLBACK_TFLOPS * (0.88 if sustained else 1.0), FALLBACK_HBM_GBS, NVLINK_GBS, "of fallback")


@dataclass(frozen=True)
class KernelRoofline:
    flops: float             # algorithmic FLOPs per rank and step
    hbm_bytes: float         # algorithmic bytes read + written in local HBM
    nvlink_bytes: float      # bytes this rank sends over NVLink (balanced routing)
    gemm_us: float
    hbm_us: float
    nvlink_us: float

    @property
    def roofline_us(self) -> float:
        return max(self.gemm_us, self.hbm_us, self.nvlink_us)

    @property
    def bound(self) -> str:
        return max((self.gemm_us, "tensor cores"), (self.hbm_us, "HBM"), (self.nvlink_us, "NVLink"))[1]


def _k(flops, hbm, nvl, pk: Peaks) -> KernelRoofline:
    return KernelRoofline(flops, hbm, nvl, flops / (pk.tflops * 1e6), hbm / (pk.hbm_gbs * 1e3), nvl / (pk.nvlink_gbs * 1e3))


def layer_rooflines(tokens: int, hidden: int, ffn: int, topk: int, world: int, peaks: Optional[Peaks] = None,
                    experts_per_rank: int = 8, store_preact: bool = True) -> Dict[str, KernelRoofline]:
    """Per-kernel rooflines of one rank for balanced routing: every rank receives ``tokens * topk`` pairs, of
    which the fraction ``(world - 1) / world`` crosses NVLink in each direction.  Keys are the logical kernel
    names that ``profile_pipeline`` prints."""
    pk = peaks or load_peaks()
    P, H, I = float(tokens) * topk, float(hidden), float(ffn)
    remote = P * (world - 1) / world if world > 1 else 0.0
    w1 = experts_per_rank * 2 * I * H * 2
    w2 = experts_per_rank * H * I * 2
    row_h, row_i = H * 2, I * 2
    out: Dict[str, KernelRoofline] = {}
    # forward: push x rows into pools, pool @ W1^T -> SwiGLU (+ preact)
    out["dispatch (+) GEMM-A SwiGLU (fused)"] = _k(
        2 * P * H * 2 * I, P * row_h * 2 + P * row_h + P * row_i + (P * 2 * row_i if store_preact else 0) + w1,
        remote * row_h, pk)
    out["GEMM-Y (+ combine when remote)"] = _k(2 * P * I * H, P * row_i + w2 + (P - remote) * row_h, remote * row_h, pk)
    # backward: push dL/dy rows, dL_do @ W2 -> dSwiGLU; dswiglu_in @ W1 -> scatter; dW1, dW2
    out["dispatch_grads (+) GEMM-Y_bwd dSwiGLU (fused)"] = _k(
        2 * P * H * I, P * row_h * 2 + P * row_h + P * 2 * row_i + P * 2 * row_i + P * row_i + w2, remote * row_h, pk)
    out["GEMM-A_bwd (+ combine_grads when remote)"] = _k(2 * P * 2 * I * H, P * 2 * row_i + w1 + (P - remote) * row_h,
                                                         remote * row_h, pk)
    out["dW grouped GEMM"] = _k(2 * P * 2 * I * H + 2 * P * H * I,
                                P * (2 * row_i + row_h) + P * (row_h + row_i) + w1 + w2, 0.0, pk)
    return out


def step_flops(tokens: int, hidden: int, ffn: int, topk: int, layers: int = 1, recompute: bool = False) -> float:
    """Forward 6 + backward 12 (+ 4 when the first GEMM is recomputed) FLOPs per (pair, hidden, ffn) element."""
    return (22.0 if recompute else 18.0) * tokens * topk * hidden * ffn * layers
