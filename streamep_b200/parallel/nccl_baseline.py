"""The constructed same-box baseline: ``torch.distributed.all_to_all_single`` + per-expert
matmuls (cuBLAS on GPU), differentiable through autograd.

It is what a user would write without this library, and it is also the CPU/gloo fp32 reference
layer: it runs unchanged on ``gloo`` with fp32 tensors.  A path that only calls the library
all-to-all plus library GEMMs is the baseline, not the product.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
from torch import nn

from ..models.reference import router_reference, swiglu_interleaved


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, out_splits, in_splits, group):
        ctx.group, ctx.out_splits, ctx.in_splits = group, out_splits, in_splits
        out = x.new_empty((sum(out_splits),) + tuple(x.shape[1:]))
        if group is None or dist.get_world_size(group) == 1:
            out.copy_(x)
        else:
            dist.all_to_all_single(out, x.contiguous(), out_splits, in_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        out = g.new_empty((sum(ctx.in_splits),) + tuple(g.shape[1:]))
        if ctx.group is None or dist.get_world_size(ctx.group) == 1:
            out.copy_(g)
        else:
            dist.all_to_all_single(out, g.contiguous(), ctx.in_splits, ctx.out_splits, group=ctx.group)
        return out, None, None, None


def baseline_moe_forward(x, topk_idx, topk_weights, w1_local, w2_local, num_experts, group):
    """Dropless expert-parallel MoE forward with library collectives; autograd gives the backward."""
    ws = 1 if group is None else dist.get_world_size(group)
    rank = 0 if group is None else dist.get_rank(group)
    EL = num_experts // ws
    T, K = topk_idx.shape
    flat_e = topk_idx.reshape(-1)
    valid = flat_e >= 0
    pair_id = torch.arange(T * K, device=x.device)[valid]
    e = flat_e[valid]
    order = torch.argsort(e, stable=True)
    pair_sorted, e_sorted = pair_id[order], e[order]
    counts = torch.bincount(e_sorted, minlength=num_experts)                     # pairs per global expert
    send_splits = counts.view(ws, EL).sum(1).tolist()
    if ws > 1:
        recv_counts = torch.empty_like(counts)
        dist.all_to_all_single(recv_counts, counts, group=group)                # [src rank][local expert]
    else:
        recv_counts = counts
    recv_splits = recv_counts.view(ws, EL).sum(1).tolist()
    rows = x[pair_sorted // K]
    recv = _AllToAll.apply(rows, recv_splits, send_splits, group)               # grouped by (src, local expert)
    # regroup by local expert
    rc = recv_counts.view(ws, EL)
    src_of = torch.repeat_interleave(torch.arange(ws, device=x.device), rc.sum(1))
    el_of = torch.cat([torch.repeat_interleave(torch.arange(EL, device=x.device), rc[s]) for s in range(ws)]) \
        if recv.shape[0] > 0 else torch.zeros(0, dtype=torch.long, device=x.device)
    by_expert = torch.argsort(el_of, stable=True)
    xs = recv[by_expert]
    per_e = rc.sum(0).tolist()
    outs = []
    off = 0
    for el in range(EL):
        n = per_e[el]
        h = xs[off:off + n] @ w1_local[el].t()
        a = swiglu_interleaved(h.float()).to(x.dtype) if x.dtype != torch.float32 else swiglu_interleaved(h)
        outs.append(a @ w2_local[el].t())
        off += n
    y = torch.cat(outs) if outs else xs.new_zeros(0, x.shape[1])
    inv = torch.empty_like(by_expert)
    inv[by_expert] = torch.arange(by_expert.numel(), device=x.device)
    back = _AllToAll.apply(y[inv], send_splits, recv_splits, group)             # original (sorted pair) order
    w_sorted = topk_weights.reshape(-1)[pair_sorted].to(torch.float32)
    out = torch.zeros(T, x.shape[1], dtype=torch.float32, device=x.device)
    out = out.index_add(0, pair_sorted // K, back.float() * w_sorted[:, None])
    _ = (src_of, rank)
    return out.to(x.dtype)


class NcclBaselineMoE(nn.Module):
    """Same constructor shape and init as ``StreamMoE`` so the two can be swapped in ``bench.py``."""

    def __init__(self, hidden, ffn, num_experts, top_k, group, *, device=None, seed=0, init_std=0.02,
                 dtype=torch.bfloat16):
        super().__init__()
        self.group = group
        self.ep_size = 1 if group is None else dist.get_world_size(group)
        self.ep_rank = 0 if group is None else dist.get_rank(group)
        self.num_experts, self.top_k = num_experts, top_k
        EL = num_experts // self.ep_size
        g = torch.Generator(device="cpu").manual_seed(seed)
        w_gate = torch.randn(num_experts, hidden, generator=g) * init_std
        g_local = torch.Generator(device="cpu").manual_seed(seed * 1000003 + self.ep_rank + 1)
        w1 = torch.randn(EL, 2 * ffn, hidden, generator=g_local) * init_std
        w2 = torch.randn(EL, hidden, ffn, generator=g_local) * init_std
        self.w_gate = nn.Parameter(w_gate.to(dtype).to(device), requires_grad=False)
        self.w1 = nn.Parameter(w1.to(dtype).to(device))
        self.w2 = nn.Parameter(w2.to(dtype).to(device))

    def route(self, x):
        idx, w = router_reference(x.detach(), self.w_gate, self.top_k)
        return idx, w, None

    def experts(self, x, topk_idx, topk_weights, is_token_in_rank=None):
        return baseline_moe_forward(x, topk_idx, topk_weights, self.w1, self.w2, self.num_experts, self.group)

    def forward(self, x):
        idx, w, _ = self.route(x)
        return self.experts(x, idx, w)
