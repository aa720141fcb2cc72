"""Device timing helpers shared by the harnesses: CUDA events on the launching stream, an L2
flush between iterations, max over ranks."""
from __future__ import annotations

import statistics
from typing import Callable, List

import torch

_flush_buf = None


def flush_l2(nbytes: int = 256 << 20) -> None:
    """Rewrite a buffer larger than the 126 MB L2 so the next timed iteration starts cold."""
    global _flush_buf
    if _flush_buf is None or _flush_buf.numel() < nbytes or _flush_buf.device != torch.device("cuda", torch.cuda.current_device()):
        _flush_buf = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    _flush_buf.zero_()


def time_cuda(fn: Callable[[], None], iters: int = 10, warmup: int = 3, flush: bool = True) -> List[float]:
    """Per-iteration device milliseconds of ``fn``."""
    for _ in range(max(warmup, 0)):
        fn()
    torch.cuda.synchronize()
    out = []
    for _ in range(iters):
        if flush:
            flush_l2()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); fn(); e1.record()
        torch.cuda.synchronize()
        out.append(e0.elapsed_time(e1))
    return out


def median_max_over_ranks(ms: List[float], group=None) -> float:
    import torch.distributed as dist
    t = torch.tensor([statistics.median(ms)], device="cuda")
    if group is not None and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t[0])
