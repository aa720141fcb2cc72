"""Plain-PyTorch oracles for the streaming expert-parallel MoE layer.

Everything here is device-agnostic eager PyTorch and doubles as (a) the fp32
numerics oracle for every CUDA kernel in the package and (b) the CPU/gloo
reference layer.

Math contract (reference: stream_ep/stream_moe/validate_multi_iter.py:118-186,
stream_ep/stream_moe/kernel_y_bwd.py:3-11):

    h      = x[t] @ W1[e]^T                      W1[e]: [2I, H], rows interleaved
    gate   = h[0::2];  up = h[1::2]              (row 2i = gate_i, row 2i+1 = up_i)
    a      = silu(gate) * up                     [I]
    y      = a @ W2[e]^T                         W2[e]: [H, I]
    out[t] = sum_k  w[t,k] * y(t, e = topk_idx[t,k])      (-1 entries skipped)
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------- router

def router_reference(x: torch.Tensor, w_gate: torch.Tensor, top_k: int,
                     renormalize: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    """Linear gate -> softmax -> top-k -> renormalise, all in fp32.

    Returns ``(topk_idx int64 [T,K], topk_weights fp32 [T,K])``.  The reference
    library has no router (callers pass routing in, see
    stream_ep/stream_moe/profile_pipeline.py:102-139); this is the oracle for
    the router kernel of this package.
    """
    logits = x.float() @ w_gate.float().t()
    probs = torch.softmax(logits, dim=-1)
    w, idx = torch.topk(probs, top_k, dim=-1)
    if renormalize:
        w = w / w.sum(dim=-1, keepdim=True)
    return idx.to(torch.int64), w.to(torch.float32)


def is_token_in_rank_reference(topk_idx: torch.Tensor, num_experts: int,
                               num_ranks: int) -> torch.Tensor:
    """``[T, R]`` bool bitmap: token t has at least one expert on rank r
    (reference: tests/utils.py:60-70)."""
    e_local = num_experts // num_ranks
    rank_idx = torch.where(topk_idx >= 0, topk_idx // e_local,
                           torch.full_like(topk_idx, -1))
    out = torch.zeros((topk_idx.shape[0], num_ranks), dtype=torch.bool,
                      device=topk_idx.device)
    for r in range(num_ranks):
        out[:, r] = (rank_idx == r).any(dim=-1)
    return out


# --------------------------------------------------------------------------- expert math

def swiglu_interleaved(h: torch.Tensor) -> torch.Tensor:
    """SwiGLU on gate/up pairs stored in adjacent columns."""
    return F.silu(h[..., 0::2]) * h[..., 1::2]


def moe_reference_forward(x: torch.Tensor, topk_idx: torch.Tensor,
                          topk_weights: torch.Tensor, w1_full: torch.Tensor,
                          w2_full: torch.Tensor,
                          out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """Eager full-MoE forward over ALL experts, grouped by expert, fp32 math.

    Autograd-compatible (functional ``index_add``), so gradients of ``x``,
    ``topk_weights``, ``w1_full`` and ``w2_full`` can be taken from it.
    """
    T, H = x.shape
    E = w1_full.shape[0]
    K = topk_idx.shape[1]
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    xf = x.float()
    wf = topk_weights.float()
    flat_e = topk_idx.reshape(-1)
    flat_t = torch.arange(T, device=x.device).unsqueeze(1).expand(T, K).reshape(-1)
    flat_w = wf.reshape(-1)
    for e in range(E):
        sel = (flat_e == e).nonzero(as_tuple=False).flatten()
        if sel.numel() == 0:
            continue
        t_e = flat_t[sel]
        h = xf[t_e] @ w1_full[e].float().t()
        a = swiglu_interleaved(h)
        y = a @ w2_full[e].float().t()
        out = out.index_add(0, t_e, flat_w[sel][:, None] * y)
    return out.to(out_dtype if out_dtype is not None else x.dtype)


def moe_reference_grads(x, topk_idx, topk_weights, w1_full, w2_full, dL_dout):
    """fp32 oracle gradients ``(out, dx, dtopk_weights, dW1, dW2)``."""
    xg = x.detach().float().requires_grad_(True)
    wg = topk_weights.detach().float().requires_grad_(True)
    w1 = w1_full.detach().float().requires_grad_(True)
    w2 = w2_full.detach().float().requires_grad_(True)
    out = moe_reference_forward(xg, topk_idx, wg, w1, w2, out_dtype=torch.float32)
    dx, dw, dw1, dw2 = torch.autograd.grad(out, (xg, wg, w1, w2), dL_dout.float())
    return out.detach(), dx, dw, dw1, dw2


# --------------------------------------------------------------------------- pool layout oracle

def channel_range(num_tokens: int, num_channels: int, c: int) -> Tuple[int, int]:
    """Token range owned by channel ``c`` (reference: csrc/kernels/utils.cuh:549-553)."""
    per = (num_tokens + num_channels - 1) // num_channels
    lo = min(per * c, num_tokens)
    hi = min(lo + per, num_tokens)
    return lo, hi


@dataclass
class RankLayout:
    """Everything one destination rank should hold after a dispatch."""
    expert_frequency: torch.Tensor          # [E_local] i32
    expert_pool_block_offset: torch.Tensor  # [E_local+1] i32
    base_pool: torch.Tensor                 # [C, R, E_local] i32
    seen_per_substream: torch.Tensor        # [C, R, E_local] i32
    rank_prefix_matrix: torch.Tensor        # [R, R] i32 (own column)
    recv_channel_prefix_matrix: torch.Tensor  # [R, C] i32
    tile_id_to_expert: torch.Tensor         # [tiles] i32
    pool_arrival_target: torch.Tensor       # [tiles] i32
    total_tiles: int
    num_recv_tokens: int
    pool_src_rank: torch.Tensor             # [TK_padded] i32 (-1 pad)
    pool_src_token: torch.Tensor            # [TK_padded] i32 (-1 pad)
    pool_recv_token: torch.Tensor           # [TK_padded] i32 (-1 pad)
    pool_k_slot: torch.Tensor               # [TK_padded] i32 (-1 pad)
    pool_topk_weight: Optional[torch.Tensor]  # [TK_padded] f32
    recv_token_to_slots: torch.Tensor       # [T_recv, K] i32
    k_local_total: torch.Tensor             # [T_recv] i32
    recv_src_rank: torch.Tensor             # [T_recv] i32
    recv_src_token: torch.Tensor            # [T_recv] i32


@dataclass
class SendLayout:
    """What a source rank knows about where its pairs/tokens land."""
    pair_slot: torch.Tensor          # [T, K] i32 slot in destination pool (-1 sentinel)
    send_recv_token: torch.Tensor    # [T, R] i32 recv-token id at destination (-1 = not sent)
    send_head: torch.Tensor          # [T, R] i32 position in the (channel, dst) stream, gap-encoded
    channel_prefix_matrix: torch.Tensor  # [R, C] i32 inclusive cumulative count per (dst, channel)


def dispatch_layout_reference(topk_idx_per_rank: Sequence[torch.Tensor], num_experts: int,
                              num_channels: int, tile_m: int = 128,
                              topk_weights_per_rank: Optional[Sequence[torch.Tensor]] = None,
                              ) -> Tuple[List[RankLayout], List[SendLayout]]:
    """CPU oracle of the deterministic pool placement for every rank at once.

    Placement rule (reference: csrc/kernels/intranode.cu:838-847,953-970;
    tests/test_metadata.py:37-242; tests/test_dispatch.py:75-93):

    * the pool of a rank is expert-major, each expert block padded to a
      multiple of ``tile_m`` rows;
    * inside an expert block, rows are ordered by (channel, source rank) and,
      within one such substream, by (token, k) lexicographically;
    * recv-token ids are source-rank-major, then source token order, and count
      each (source token, destination rank) once.
    """
    R = len(topk_idx_per_rank)
    E = num_experts
    assert E % R == 0
    EL = E // R
    C = num_channels
    K = topk_idx_per_rank[0].shape[1]
    idx = [t.detach().cpu().to(torch.int64) for t in topk_idx_per_rank]
    Ts = [t.shape[0] for t in idx]

    counts = torch.zeros(R, C, E, dtype=torch.int64)     # [src, c, e]
    ucount = torch.zeros(R, C, R, dtype=torch.int64)     # [src, c, dst]
    for s in range(R):
        for c in range(C):
            lo, hi = channel_range(Ts[s], C, c)
            sub = idx[s][lo:hi]
            valid = sub[sub >= 0]
            if valid.numel():
                counts[s, c] = torch.bincount(valid, minlength=E)
            for d in range(R):
                ucount[s, c, d] = (((sub >= d * EL) & (sub < (d + 1) * EL)).any(dim=1)).sum()

    freq = counts.sum(dim=(0, 1))                         # [E]
    tiles = (freq + tile_m - 1) // tile_m
    layouts: List[RankLayout] = []
    base_all = torch.zeros(C, R, E, dtype=torch.int64)    # base slot of substream (c, src) for expert e
    offsets_all = torch.zeros(E, dtype=torch.int64)
    for d in range(R):
        off = torch.zeros(EL + 1, dtype=torch.int64)
        off[1:] = torch.cumsum(tiles[d * EL:(d + 1) * EL], 0)
        offsets_all[d * EL:(d + 1) * EL] = off[:-1]
        for el in range(EL):
            e = d * EL + el
            run = int(off[el]) * tile_m
            for c in range(C):
                for s in range(R):
                    base_all[c, s, e] = run
                    run += int(counts[s, c, e])

    U = ucount.sum(dim=1)                                  # [src, dst]
    sends: List[SendLayout] = []
    # sender view -------------------------------------------------------------
    pair_slot_all = []
    send_recv_all = []
    for s in range(R):
        T = Ts[s]
        pair_slot = torch.full((T, K), -1, dtype=torch.int64)
        send_recv = torch.full((T, R), -1, dtype=torch.int64)
        send_head = torch.full((T, R), -1, dtype=torch.int64)
        chan_prefix = torch.zeros(R, C, dtype=torch.int64)
        recv_base = torch.zeros(R, dtype=torch.int64)
        for d in range(R):
            recv_base[d] = U[:s, d].sum()
        running_recv = recv_base.clone()
        for c in range(C):
            lo, hi = channel_range(T, C, c)
            seen = torch.zeros(E, dtype=torch.int64)
            pos_in_stream = torch.zeros(R, dtype=torch.int64)
            for t in range(lo, hi):
                row = idx[s][t]
                dst_of = torch.where(row >= 0, row // EL, torch.full_like(row, -1))
                for d in range(R):
                    if (dst_of == d).any():
                        send_recv[t, d] = running_recv[d]
                        running_recv[d] += 1
                        send_head[t, d] = pos_in_stream[d]
                        pos_in_stream[d] += 1
                for k in range(K):
                    e = int(row[k])
                    if e < 0:
                        continue
                    pair_slot[t, k] = base_all[c, s, e] + seen[e]
                    seen[e] += 1
            # gap-encode: token not sent to d gets -(next valid head)-1
            nxt = pos_in_stream.clone()
            for t in range(hi - 1, lo - 1, -1):
                for d in range(R):
                    if send_head[t, d] >= 0:
                        nxt[d] = send_head[t, d]
                    else:
                        send_head[t, d] = -int(nxt[d]) - 1
            for d in range(R):
                chan_prefix[d, c] = ucount[s, :c + 1, d].sum()
        pair_slot_all.append(pair_slot)
        send_recv_all.append(send_recv)
        sends.append(SendLayout(pair_slot.to(torch.int32), send_recv.to(torch.int32),
                                send_head.to(torch.int32), chan_prefix.to(torch.int32)))

    # receiver view -----------------------------------------------------------
    for d in range(R):
        off = torch.zeros(EL + 1, dtype=torch.int64)
        off[1:] = torch.cumsum(tiles[d * EL:(d + 1) * EL], 0)
        total_tiles = int(off[-1])
        TKp = total_tiles * tile_m
        T_recv = int(U[:, d].sum())
        tile_e = torch.zeros(total_tiles, dtype=torch.int64)
        target = torch.zeros(total_tiles, dtype=torch.int64)
        for el in range(EL):
            f = int(freq[d * EL + el])
            for j in range(int(tiles[d * EL + el])):
                tid = int(off[el]) + j
                tile_e[tid] = el
                target[tid] = min(tile_m, f - j * tile_m)
        p_src_rank = torch.full((TKp,), -1, dtype=torch.int64)
        p_src_tok = torch.full((TKp,), -1, dtype=torch.int64)
        p_recv = torch.full((TKp,), -1, dtype=torch.int64)
        p_k = torch.full((TKp,), -1, dtype=torch.int64)
        p_w = torch.zeros((TKp,), dtype=torch.float32) if topk_weights_per_rank is not None else None
        r2s = torch.full((T_recv, K), -1, dtype=torch.int64)
        klt = torch.zeros((T_recv,), dtype=torch.int64)
        rsr = torch.full((T_recv,), -1, dtype=torch.int64)
        rst = torch.full((T_recv,), -1, dtype=torch.int64)
        for s in range(R):
            row_d = (idx[s] >= d * EL) & (idx[s] < (d + 1) * EL)
            for t, k in row_d.nonzero(as_tuple=False).tolist():
                slot = int(pair_slot_all[s][t, k])
                r = int(send_recv_all[s][t, d])
                p_src_rank[slot] = s
                p_src_tok[slot] = t
                p_recv[slot] = r
                p_k[slot] = k
                if p_w is not None:
                    p_w[slot] = float(topk_weights_per_rank[s][t, k])
                r2s[r, k] = slot
                klt[r] += 1
                rsr[r] = s
                rst[r] = t
        rpm = torch.zeros(R, R, dtype=torch.int64)
        rpm[:, d] = torch.cumsum(U[:, d], 0)
        rcpm = torch.zeros(R, C, dtype=torch.int64)
        for s in range(R):
            rcpm[s] = torch.cumsum(ucount[s, :, d], 0)
        layouts.append(RankLayout(
            expert_frequency=freq[d * EL:(d + 1) * EL].to(torch.int32),
            expert_pool_block_offset=off.to(torch.int32),
            base_pool=base_all[:, :, d * EL:(d + 1) * EL].to(torch.int32).contiguous(),
            seen_per_substream=counts[:, :, d * EL:(d + 1) * EL].permute(1, 0, 2).to(torch.int32).contiguous(),
            rank_prefix_matrix=rpm.to(torch.int32),
            recv_channel_prefix_matrix=rcpm.to(torch.int32),
            tile_id_to_expert=tile_e.to(torch.int32),
            pool_arrival_target=target.to(torch.int32),
            total_tiles=total_tiles,
            num_recv_tokens=T_recv,
            pool_src_rank=p_src_rank.to(torch.int32),
            pool_src_token=p_src_tok.to(torch.int32),
            pool_recv_token=p_recv.to(torch.int32),
            pool_k_slot=p_k.to(torch.int32),
            pool_topk_weight=p_w,
            recv_token_to_slots=r2s.to(torch.int32),
            k_local_total=klt.to(torch.int32),
            recv_src_rank=rsr.to(torch.int32),
            recv_src_token=rst.to(torch.int32),
        ))
    return layouts, sends


def pool_reference(layout: RankLayout, x_per_rank: Sequence[torch.Tensor]) -> torch.Tensor:
    """Expected pool contents (padding rows zero) given every rank's ``x``."""
    H = x_per_rank[0].shape[1]
    pool = torch.zeros(layout.pool_src_rank.shape[0], H, dtype=x_per_rank[0].dtype)
    for slot in (layout.pool_src_rank >= 0).nonzero(as_tuple=False).flatten().tolist():
        pool[slot] = x_per_rank[int(layout.pool_src_rank[slot])][int(layout.pool_src_token[slot])].cpu()
    return pool


# --------------------------------------------------------------------------- per-kernel oracles

def kernel_a_reference(pool, w1_local, tile_id_to_expert, tile_m):
    """``preact[TKp, 2I]`` and ``postact[TKp, I]`` in fp32
    (reference semantics: stream_ep/stream_moe/kernel_a.py:405-579)."""
    TKp = pool.shape[0]
    two_i = w1_local.shape[1]
    pre = torch.zeros(TKp, two_i, dtype=torch.float32, device=pool.device)
    for t, e in enumerate(tile_id_to_expert.tolist()):
        rows = slice(t * tile_m, (t + 1) * tile_m)
        pre[rows] = pool[rows].float() @ w1_local[e].float().t()
    return pre, swiglu_interleaved(pre)


def dswiglu_reference(gate, up, g):
    """Gradient of ``silu(gate) * up`` given upstream ``g``: ``(dgate, dup, postact)``."""
    sig = torch.sigmoid(gate)
    silu = gate * sig
    dgate = g * up * sig * (1 + gate * (1 - sig))
    dup = g * silu
    return dgate, dup, silu * up


def check_close(name: str, got: torch.Tensor, want: torch.Tensor, atol: float, rtol: float,
                rel_floor: float = 0.0) -> None:
    """Dual-threshold rule of the reference validator: an element fails only if
    BOTH ``|diff| > atol`` and ``|diff| > rtol * (|want| + rel_floor)``
    (reference: stream_ep/stream_moe/validate_multi_iter.py:559-575, which uses ``rel_floor = 1e-3``)."""
    got = got.detach().float()
    want = want.detach().float().to(got.device)
    diff = (got - want).abs()
    bad = (diff > atol) & (diff > rtol * (want.abs() + rel_floor))
    if not torch.isfinite(got).all():
        raise AssertionError(f"{name}: non-finite values in result")
    if bad.any():
        i = int(diff.flatten().argmax())
        raise AssertionError(
            f"{name}: {int(bad.sum())}/{bad.numel()} elements fail (atol={atol}, rtol={rtol}); "
            f"max |diff|={float(diff.max()):.4e} at flat index {i} "
            f"(got {float(got.flatten()[i]):.5e}, want {float(want.flatten()[i]):.5e})")
