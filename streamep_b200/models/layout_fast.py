"""Vectorised form of the pool-layout oracle, for production-scale checks.

``dispatch_layout_reference`` (models/reference.py) walks tokens and pairs in Python loops, which is
the readable statement of the placement rule but takes minutes at 8 ranks x 8192 tokens x top-13.
This module computes the same ``RankLayout`` / ``SendLayout`` objects with sorts, bincounts and
cumulative sums only (any device), and ``tests/test_reference_cpu.py`` pins it to the loop oracle on
small cases.  The rule itself is the reference's (csrc/kernels/intranode.cu:838-847,953-970;
tests/test_metadata.py:37-242 checks the same tensors at T=8192, K=13, E=384).
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

from .reference import RankLayout, SendLayout


def _excl_cumsum(x: torch.Tensor, dim: int) -> torch.Tensor:
    return torch.cumsum(x, dim) - x


def dispatch_layout_fast(topk_idx_per_rank: Sequence[torch.Tensor], num_experts: int, num_channels: int,
                         tile_m: int = 128, topk_weights_per_rank: Optional[Sequence[torch.Tensor]] = None,
                         ) -> Tuple[List[RankLayout], List[SendLayout]]:
    R, E, C = len(topk_idx_per_rank), num_experts, num_channels
    assert E % R == 0
    EL = E // R
    K = topk_idx_per_rank[0].shape[1]
    dev = topk_idx_per_rank[0].device
    idx = [t.detach().to(torch.int64) for t in topk_idx_per_rank]
    Ts = [int(t.shape[0]) for t in idx]
    i64 = dict(dtype=torch.int64, device=dev)

    # ---- per source: channel of every token, per-(channel, expert) pair counts, per-(channel, dst) token counts
    chan, hit = [], []
    counts = torch.zeros(R, C, E, **i64)          # [src, c, e]
    ucount = torch.zeros(R, C, R, **i64)          # [src, c, dst]
    for s in range(R):
        T = Ts[s]
        per = max((T + C - 1) // C, 1)
        c_of_t = torch.arange(T, **i64) // per
        chan.append(c_of_t)
        valid = idx[s] >= 0
        key = (c_of_t[:, None] * E + idx[s].clamp_min(0))[valid]
        counts[s] = torch.bincount(key, minlength=C * E).view(C, E)
        dst = torch.where(valid, idx[s] // EL, torch.full_like(idx[s], -1))
        h = (dst[:, :, None] == torch.arange(R, **i64)[None, None, :]).any(dim=1)      # [T, R]
        hit.append(h)
        ucount[s] = torch.zeros(C, R, **i64).index_add_(0, c_of_t, h.to(torch.int64))

    freq = counts.sum(dim=(0, 1))                 # [E]
    tiles = (freq + tile_m - 1) // tile_m
    off_all = _excl_cumsum(tiles.view(R, EL), 1).reshape(E)                           # tile offset inside the owner
    # base slot of substream (c, src) for expert e: exclusive scan over (c, src) in lexicographic order
    by_cs = counts.permute(1, 0, 2).reshape(C * R, E)
    base_all = (off_all[None, :] * tile_m + _excl_cumsum(by_cs, 0)).view(C, R, E)
    U = ucount.sum(dim=1)                         # [src, dst]
    return _finish(idx, Ts, chan, hit, counts, ucount, freq, tiles, off_all, base_all, U, R, E, EL, C, K, tile_m,
                   topk_weights_per_rank, dev)


def _finish(idx, Ts, chan, hit, counts, ucount, freq, tiles, off_all, base_all, U, R, E, EL, C, K, tile_m, weights, dev):
    i64 = dict(dtype=torch.int64, device=dev)
    i32 = torch.int32
    sends: List[SendLayout] = []
    pair_slot_all, send_recv_all = [], []
    for s in range(R):
        T = Ts[s]
        c_of_t = chan[s]
        valid = idx[s] >= 0
        # rank of every pair inside its (channel, expert) substream, in (token, k) order: stable sort by the key
        key = torch.where(valid, c_of_t[:, None] * E + idx[s].clamp_min(0), torch.full_like(idx[s], C * E)).reshape(-1)
        order = torch.argsort(key, stable=True)
        sorted_key = key[order]
        start_of_group = torch.searchsorted(sorted_key, sorted_key, right=False)
        rank_sorted = torch.arange(T * K, **i64) - start_of_group
        rank_in = torch.empty(T * K, **i64)
        rank_in[order] = rank_sorted
        base = base_all[c_of_t[:, None].expand(T, K), s, idx[s].clamp_min(0)]
        pair_slot = torch.where(valid, base + rank_in.view(T, K), torch.full_like(idx[s], -1))
        # recv-token ids: tokens of earlier sources first, then this source's tokens in order
        h = hit[s].to(torch.int64)
        before = _excl_cumsum(h, 0)
        send_recv = torch.where(hit[s], U[:s].sum(0)[None, :] + before, torch.full_like(h, -1))
        # position in the (channel, dst) stream; a token that is not sent records -(hits before it in the channel) - 1
        chan_start = torch.zeros(C + 1, R, **i64)
        chan_start[1:] = torch.cumsum(ucount[s], 0)
        in_chan = before - chan_start[c_of_t]
        send_head = torch.where(hit[s], in_chan, -in_chan - 1)
        chan_prefix = torch.cumsum(ucount[s], 0).t().contiguous()                    # [dst, c] inclusive
        pair_slot_all.append(pair_slot)
        send_recv_all.append(send_recv)
        sends.append(SendLayout(pair_slot.to(i32), send_recv.to(i32), send_head.to(i32), chan_prefix.to(i32)))
    return _receivers(idx, Ts, counts, ucount, freq, tiles, base_all, U, pair_slot_all, send_recv_all, sends,
                      R, E, EL, C, K, tile_m, weights, dev)


def _receivers(idx, Ts, counts, ucount, freq, tiles, base_all, U, pair_slot_all, send_recv_all, sends,
               R, E, EL, C, K, tile_m, weights, dev):
    i64 = dict(dtype=torch.int64, device=dev)
    i32 = torch.int32
    layouts: List[RankLayout] = []
    for d in range(R):
        t_d = tiles[d * EL:(d + 1) * EL]
        off = torch.zeros(EL + 1, **i64)
        off[1:] = torch.cumsum(t_d, 0)
        total_tiles = int(off[-1])
        TKp = total_tiles * tile_m
        T_recv = int(U[:, d].sum())
        tile_e = torch.repeat_interleave(torch.arange(EL, **i64), t_d)
        j = torch.arange(total_tiles, **i64) - off[:-1][tile_e]
        target = torch.minimum(torch.full_like(j, tile_m), freq[d * EL:(d + 1) * EL][tile_e] - j * tile_m)
        p_src_rank = torch.full((TKp,), -1, **i64); p_src_tok = torch.full((TKp,), -1, **i64)
        p_recv = torch.full((TKp,), -1, **i64); p_k = torch.full((TKp,), -1, **i64)
        p_w = torch.zeros((TKp,), dtype=torch.float32, device=dev) if weights is not None else None
        r2s = torch.full((T_recv, K), -1, **i64)
        klt = torch.zeros((T_recv,), **i64)
        rsr = torch.full((T_recv,), -1, **i64); rst = torch.full((T_recv,), -1, **i64)
        for s in range(R):
            mine = (idx[s] >= d * EL) & (idx[s] < (d + 1) * EL)
            tk = mine.nonzero(as_tuple=False)
            if tk.numel() == 0:
                continue
            t, k = tk[:, 0], tk[:, 1]
            slot = pair_slot_all[s][t, k]
            r = send_recv_all[s][t, d]
            p_src_rank[slot] = s; p_src_tok[slot] = t; p_recv[slot] = r; p_k[slot] = k
            if p_w is not None:
                p_w[slot] = weights[s].to(dev)[t, k].float()
            r2s[r, k] = slot
            klt.index_add_(0, r, torch.ones_like(r))
            rsr[r] = s; rst[r] = t
        rpm = torch.zeros(R, R, **i64)
        rpm[:, d] = torch.cumsum(U[:, d], 0)
        rcpm = torch.cumsum(ucount[:, :, d], 1)
        layouts.append(RankLayout(
            expert_frequency=freq[d * EL:(d + 1) * EL].to(i32), expert_pool_block_offset=off.to(i32),
            base_pool=base_all[:, :, d * EL:(d + 1) * EL].to(i32).contiguous(),
            seen_per_substream=counts[:, :, d * EL:(d + 1) * EL].permute(1, 0, 2).to(i32).contiguous(),
            rank_prefix_matrix=rpm.to(i32), recv_channel_prefix_matrix=rcpm.to(i32),
            tile_id_to_expert=tile_e.to(i32), pool_arrival_target=target.to(i32),
            total_tiles=total_tiles, num_recv_tokens=T_recv,
            pool_src_rank=p_src_rank.to(i32), pool_src_token=p_src_tok.to(i32), pool_recv_token=p_recv.to(i32),
            pool_k_slot=p_k.to(i32), pool_topk_weight=p_w, recv_token_to_slots=r2s.to(i32), k_local_total=klt.to(i32),
            recv_src_rank=rsr.to(i32), recv_src_token=rst.to(i32)))
    return layouts, sends
