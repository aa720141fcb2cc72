"""Python entry points of the tcgen05 grouped-GEMM kernels.

One native kernel template (``csrc/gemm_kernels.cu``) serves all of these; the
wrappers only assemble its argument bag.  Names and argument order follow the
reference wrappers so call sites read the same:

* ``streaming_moe_a``      stream_ep/stream_moe/kernel_a.py:405-579
* ``streaming_moe_y``      stream_ep/stream_moe/kernel_y.py:842-1007
* ``streaming_moe_y_bwd``  stream_ep/stream_moe/kernel_y_bwd.py:606-891
* ``streaming_moe_a_bwd``  stream_ep/stream_moe/kernel_a_bwd.py:320-507
* ``grouped_gemm_dw``      the ``quack.gemm`` varlen-K calls at stream_ep/stream_moe/stream_moe.py:1111-1142
* ``grouped_gemm_preact``  the recompute GEMM at stream_ep/stream_moe/stream_moe.py:993-1004
* ``fire_tiles_with_delay`` stream_ep/stream_moe/kernel_a.py:378-402
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from .. import _ext

VARLEN_M, VARLEN_K = 0, 1
EPI_STORE, EPI_SWIGLU, EPI_SCATTER, EPI_DSWIGLU = 0, 1, 2, 3
KIND_GEMM_Y_TAIL, KIND_GEMM_A_BWD_TAIL = 5, 6
GATE_KERNEL_Y, GATE_KERNEL_A_BWD = 2, 3

_default_runtime = None


def default_runtime():
    """A private single-rank runtime for callers that have no ``Buffer`` (kernel
    tests, micro-benchmarks): it owns the status block and the launch-gate flags
    the kernels report into."""
    global _default_runtime
    if _default_runtime is None:
        C = _ext.load()
        _default_runtime = C.Runtime(0, 1, 64 << 20, 4, C.MAX_EXPERTS, 2000)
        _default_runtime.sync_local([_default_runtime.get_local_base_ptr()])
    return _default_runtime


def _rt(buffer):
    if buffer is None:
        return default_runtime()
    return buffer.runtime if hasattr(buffer, "runtime") else buffer


def pick_block_n(n: int, requested: Optional[int] = None) -> int:
    """Tile width of the output.  256 (one full-width UMMA per k-step) unless the masked part of
    the last tile would waste more than 15 % of the work, in which case 128 is used."""
    if requested is not None:
        if requested not in (128, 256):
            raise ValueError(f"tile_n must be 128 or 256 on sm_100a (got {requested})")
        return requested
    if n <= 128:
        return 128
    waste256 = (-(-n // 256) * 256) / n
    waste128 = (-(-n // 128) * 128) / n
    return 256 if waste256 <= 1.15 * waste128 else 128


def _args():
    return _ext.load().GemmArgs()


def streaming_moe_a(pool: torch.Tensor, w1: torch.Tensor, tile_id_to_expert: torch.Tensor, *,
                    postact_a: Optional[torch.Tensor] = None, preact_a: Optional[torch.Tensor] = None,
                    store_preact: bool = False,
                    pool_arrival_count: Optional[torch.Tensor] = None,
                    pool_arrival_target: Optional[torch.Tensor] = None,
                    tile_n: Optional[int] = None, num_sms: Optional[int] = None, buffer=None,
                    fused_dispatch=None, push_flags: int = 3, num_tiles: Optional[int] = None,
                    live_tiles: Optional[torch.Tensor] = None):
    """``postact[TKp, I] = swiglu(pool[TKp, H] @ w1[e]^T)`` tile by tile.

    ``w1`` is ``[E_local, 2I, H]`` with gate/up rows interleaved.  With
    ``pool_arrival_count/target`` each 128-row tile is read only once its count
    reached its target.  ``fused_dispatch`` (the native state of a dispatch whose
    push was not launched) makes the same kernel ship this rank's token rows to
    the peers' pools while its tensor-core warps consume tiles as they land.
    Returns ``(postact_a, preact_a or None)``.
    """
    rows, H = pool.shape
    E, two_i, H2 = w1.shape
    assert H == H2 and two_i % 2 == 0
    if postact_a is None:
        postact_a = torch.empty(rows, two_i // 2, dtype=pool.dtype, device=pool.device)
    if store_preact and preact_a is None:
        preact_a = torch.empty(rows, two_i, dtype=pool.dtype, device=pool.device)
    a = _args()
    a.mode, a.epilogue, a.block_n = VARLEN_M, EPI_SWIGLU, pick_block_n(two_i, tile_n)
    a.a, a.b = pool, w1
    a.tile_id_to_expert = tile_id_to_expert
    if num_tiles is not None:
        a.num_m_tiles = num_tiles
    a.out0 = postact_a
    if preact_a is not None:
        a.out1 = preact_a
    if pool_arrival_count is not None:
        a.arrival_count, a.arrival_target = pool_arrival_count, pool_arrival_target
    if num_sms:
        a.num_ctas = num_sms
    if fused_dispatch is not None:
        a.fused_push = fused_dispatch
        a.push_flags = push_flags
    if live_tiles is not None and num_tiles is None:
        a.num_m_tiles_dev = live_tiles
    _rt(buffer).grouped_gemm(a)
    return postact_a, preact_a


def grouped_gemm_preact(pool: torch.Tensor, w1: torch.Tensor, tile_id_to_expert: torch.Tensor, *,
                        out: Optional[torch.Tensor] = None, tile_n: Optional[int] = None,
                        num_sms: Optional[int] = None, live_tiles: Optional[torch.Tensor] = None, buffer=None):
    """``preact[TKp, 2I] = pool @ w1[e]^T`` (activation-checkpoint recompute)."""
    rows = pool.shape[0]
    two_i = w1.shape[1]
    if out is None:
        out = torch.empty(rows, two_i, dtype=pool.dtype, device=pool.device)
    a = _args()
    a.mode, a.epilogue, a.block_n = VARLEN_M, EPI_STORE, pick_block_n(two_i, tile_n)
    a.a, a.b, a.tile_id_to_expert, a.out0 = pool, w1, tile_id_to_expert, out
    if live_tiles is not None:
        a.num_m_tiles_dev = live_tiles
    if num_sms:
        a.num_ctas = num_sms
    _rt(buffer).grouped_gemm(a)
    return out


def _scatter_common(a, *, o, pool_recv_token, tile_stripes_done, k_local_remaining, done_per_token, seq,
                    remote_offsets, pool_src, pool_k_slot, num_topk, tail_kind, tail_wait, remote_static_offset=-1,
                    live_tiles=None):
    a.row_token = pool_recv_token
    a.scatter_local = o
    if live_tiles is not None:
        a.num_m_tiles_dev = live_tiles
    if remote_offsets is not None:
        if remote_static_offset is not None and remote_static_offset >= 0:
            a.remote_out_offset = int(remote_static_offset)   # capacity mode: same arena offset on every rank
        else:
            a.remote_out = [int(v) for v in remote_offsets]
        a.row_src, a.row_k_slot, a.num_topk = pool_src, pool_k_slot, int(num_topk)
        a.tail, a.tail_kind, a.tail_wait = True, tail_kind, tail_wait
    else:
        if tile_stripes_done is not None:
            a.tile_stripes_done = tile_stripes_done
            a.k_remaining = k_local_remaining
            a.done_per_token = done_per_token
            a.seq = int(seq)


def streaming_moe_y(postact_a: torch.Tensor, w2: torch.Tensor, tile_id_to_expert: torch.Tensor,
                    pool_topk_weight: torch.Tensor, pool_recv_token: torch.Tensor, *,
                    o: Optional[torch.Tensor] = None, tile_n_stripes_done: Optional[torch.Tensor] = None,
                    k_local_remaining: Optional[torch.Tensor] = None,
                    y_done_per_token: Optional[torch.Tensor] = None, combine_seq: int = 0,
                    remote_out_offsets: Optional[Sequence[int]] = None, pool_src: Optional[torch.Tensor] = None,
                    pool_k_slot: Optional[torch.Tensor] = None, num_topk: int = 0,
                    tail_wait: bool = True, started_flag: bool = False,
                    tile_n: Optional[int] = None, num_sms: Optional[int] = None, buffer=None,
                    remote_static_offset: int = -1, live_tiles: Optional[torch.Tensor] = None):
    """``y = postact @ w2[e]^T`` scaled by the slot's top-k weight and reduced
    with 16-byte bf16x2 ``red.add`` into

    * ``o[pool_recv_token[slot]]`` on this rank (then per-token completion stamps
      ``y_done_per_token[r] = combine_seq`` once all of r's local slots are in), or
    * with ``remote_out_offsets`` (fused combine): rows whose source token lives on
      this rank are red.added into ``o`` (here ``[T, H]``, indexed by source token);
      rows of other ranks' tokens are STORED, one contiguous bf16 row per (token, k),
      into that rank's ``[T * K, H]`` landing buffer over NVLink.  The triple names
      ``(record kind, epoch, word)`` of the record in which every rank published the
      arena offset of its landing buffer.  The kernel ends with a cross-rank
      completion handshake; ``combine_reduce`` then folds the landed rows into ``o``
      in fp32.
    """
    a = _args()
    N = w2.shape[1]
    a.mode, a.epilogue, a.block_n = VARLEN_M, EPI_SCATTER, pick_block_n(N, tile_n)
    a.a, a.b, a.tile_id_to_expert = postact_a, w2, tile_id_to_expert
    a.row_weight = pool_topk_weight
    if started_flag:
        a.started_flag = GATE_KERNEL_Y
    _scatter_common(a, o=o, pool_recv_token=pool_recv_token, tile_stripes_done=tile_n_stripes_done,
                    k_local_remaining=k_local_remaining, done_per_token=y_done_per_token, seq=combine_seq,
                    remote_offsets=remote_out_offsets, pool_src=pool_src, pool_k_slot=pool_k_slot, num_topk=num_topk,
                    tail_kind=KIND_GEMM_Y_TAIL, tail_wait=tail_wait, remote_static_offset=remote_static_offset,
                    live_tiles=live_tiles)
    if num_sms:
        a.num_ctas = num_sms
    _rt(buffer).grouped_gemm(a)
    return o


def streaming_moe_a_bwd(dL_dswiglu_in: torch.Tensor, w1: torch.Tensor, tile_id_to_expert: torch.Tensor,
                        pool_recv_token: torch.Tensor, *, dL_dx_per_r: Optional[torch.Tensor] = None,
                        tile_n_stripes_done: Optional[torch.Tensor] = None,
                        bwd_k_local_remaining: Optional[torch.Tensor] = None,
                        bwd_a_done_per_token: Optional[torch.Tensor] = None, dispatch_seq: int = 0,
                        remote_out_offsets: Optional[Sequence[int]] = None, pool_src: Optional[torch.Tensor] = None,
                        pool_k_slot: Optional[torch.Tensor] = None, num_topk: int = 0,
                        tail_wait: bool = True, started_flag: bool = False,
                        tile_n: Optional[int] = None, num_sms: Optional[int] = None, buffer=None,
                        remote_static_offset: int = -1, live_tiles: Optional[torch.Tensor] = None):
    """``dpool = dL_dswiglu_in[TKp, 2I] @ w1[e]`` (NN GEMM, K = 2I) reduced into
    ``dL_dx_per_r[r]`` locally or into the source rank's ``dL_dx`` remotely
    (fused combine_grads).  No per-slot weight: it is already folded into
    ``dL_dswiglu_in``."""
    a = _args()
    N = w1.shape[2]
    a.mode, a.epilogue, a.block_n = VARLEN_M, EPI_SCATTER, pick_block_n(N, tile_n)
    a.b_mn_major = True
    a.a, a.b, a.tile_id_to_expert = dL_dswiglu_in, w1, tile_id_to_expert
    if started_flag:
        a.started_flag = GATE_KERNEL_A_BWD
    _scatter_common(a, o=dL_dx_per_r, pool_recv_token=pool_recv_token, tile_stripes_done=tile_n_stripes_done,
                    k_local_remaining=bwd_k_local_remaining, done_per_token=bwd_a_done_per_token,
                    seq=dispatch_seq, remote_offsets=remote_out_offsets, pool_src=pool_src, pool_k_slot=pool_k_slot,
                    num_topk=num_topk, tail_kind=KIND_GEMM_A_BWD_TAIL, tail_wait=tail_wait,
                    remote_static_offset=remote_static_offset, live_tiles=live_tiles)
    if num_sms:
        a.num_ctas = num_sms
    _rt(buffer).grouped_gemm(a)
    return dL_dx_per_r


def streaming_moe_y_bwd(dL_do_pool: torch.Tensor, w2: torch.Tensor, preact_a: torch.Tensor,
                        tile_id_to_expert: torch.Tensor, pool_topk_weight: torch.Tensor,
                        pool_recv_token: torch.Tensor, *, dL_dswiglu_in: Optional[torch.Tensor] = None,
                        postact_a_for_dW2: Optional[torch.Tensor] = None,
                        dL_dweight: Optional[torch.Tensor] = None,
                        arrival_count: Optional[torch.Tensor] = None,
                        arrival_target: Optional[torch.Tensor] = None,
                        remote_dw_offsets: Optional[Sequence[int]] = None,
                        pool_src: Optional[torch.Tensor] = None, pool_k_slot: Optional[torch.Tensor] = None,
                        num_topk: int = 0, tile_n_stripes_done: Optional[torch.Tensor] = None,
                        fused_dispatch_grads=None, fused_routing=None, fused_rows: Optional[torch.Tensor] = None,
                        push_flags: int = 3, num_tiles: Optional[int] = None,
                        tile_n: Optional[int] = None, num_sms: Optional[int] = None, buffer=None,
                        remote_static_offset: int = -1, live_tiles: Optional[torch.Tensor] = None):
    """``g = dL_do_pool[TKp, H] @ w2[e]`` (NN GEMM, K = H) followed by the SwiGLU
    backward on the saved ``preact_a``:

    * ``dL_dweight[slot] += sum_i postact[slot, i] * g[slot, i]`` (unweighted g),
    * ``dL_dswiglu_in[slot, 2i:2i+2] = w * (dgate_i, dup_i)``,
    * ``postact_a_for_dW2[slot, i] = w * postact[slot, i]``,
    * padding rows (``pool_recv_token < 0``) come out exactly zero.

    ``dL_dweight`` must be zero on entry.  With ``remote_dw_offsets`` (a ``(record
    kind, epoch, word)`` triple, see :func:`streaming_moe_y`) the final per-slot
    value is also stored into the source rank's ``[T, K]`` matrix.
    """
    rows, H = dL_do_pool.shape
    E, H2, I = w2.shape
    assert H == H2
    if dL_dswiglu_in is None:
        dL_dswiglu_in = torch.empty(rows, 2 * I, dtype=dL_do_pool.dtype, device=dL_do_pool.device)
    if postact_a_for_dW2 is None:
        postact_a_for_dW2 = torch.empty(rows, I, dtype=dL_do_pool.dtype, device=dL_do_pool.device)
    if dL_dweight is None:
        dL_dweight = torch.zeros(rows, dtype=torch.float32, device=dL_do_pool.device)
    a = _args()
    a.mode, a.epilogue, a.block_n = VARLEN_M, EPI_DSWIGLU, pick_block_n(I, tile_n)
    a.b_mn_major = True
    a.a, a.b, a.tile_id_to_expert = dL_do_pool, w2, tile_id_to_expert
    a.preact, a.out0, a.out1 = preact_a, dL_dswiglu_in, postact_a_for_dW2
    a.row_weight, a.row_token, a.dl_dweight = pool_topk_weight, pool_recv_token, dL_dweight
    if num_tiles is not None:
        a.num_m_tiles = num_tiles
    if arrival_count is not None:
        a.arrival_count, a.arrival_target = arrival_count, arrival_target
    if live_tiles is not None and num_tiles is None:
        a.num_m_tiles_dev = live_tiles
    if remote_dw_offsets is not None:
        if remote_static_offset is not None and remote_static_offset >= 0:
            a.remote_dw_offset = int(remote_static_offset)
        else:
            a.remote_dw = [int(v) for v in remote_dw_offsets]
        a.row_src, a.row_k_slot, a.num_topk = pool_src, pool_k_slot, num_topk
        a.tile_stripes_done = tile_n_stripes_done
    if fused_dispatch_grads is not None:
        a.fused_push_grads, a.fused_push_routing, a.fused_push_rows = fused_dispatch_grads, fused_routing, fused_rows
        a.push_flags = push_flags
    if num_sms:
        a.num_ctas = num_sms
    _rt(buffer).grouped_gemm(a)
    return dL_dswiglu_in, postact_a_for_dW2, dL_dweight


def grouped_gemm_dw(lhs: torch.Tensor, rhs: torch.Tensor, expert_pool_block_offset: torch.Tensor,
                    expert_frequency: torch.Tensor, *, out: Optional[torch.Tensor] = None,
                    tile_n: Optional[int] = None, num_sms: Optional[int] = None, buffer=None,
                    lhs2: Optional[torch.Tensor] = None, rhs2: Optional[torch.Tensor] = None,
                    out2: Optional[torch.Tensor] = None, dynamic_tiles: bool = False):
    """Per-expert weight gradient ``out[e] = lhs[rows_e]^T @ rhs[rows_e]`` with
    ``rows_e`` the expert's TRUE row range (padding rows never contribute, whatever
    they hold).  ``lhs [TKp, M]``, ``rhs [TKp, N]`` -> ``out [E, M, N]`` bf16, fp32
    accumulation in tensor memory.

    ``lhs2`` / ``rhs2`` (over the same rows) add a second problem to the same launch (dW1 and dW2 of a layer
    together: one tail wave instead of two); then ``(out, out2)`` is returned.  ``dynamic_tiles``: CTAs claim
    tiles from a device counter instead of striding by the grid size, so tiles of unequal length (experts with
    unequal row counts) balance out (reference: the ``atomicAdd`` claim of
    stream_ep/stream_moe/tile_scheduler.py:336-342)."""
    E = expert_frequency.numel()
    M, N = lhs.shape[1], rhs.shape[1]
    if out is None:
        out = torch.empty(E, M, N, dtype=lhs.dtype, device=lhs.device)
    a = _args()
    a.mode, a.epilogue, a.block_n = VARLEN_K, EPI_STORE, pick_block_n(N, tile_n)
    a.a_mn_major = a.b_mn_major = True
    a.a, a.b, a.out0 = lhs, rhs, out
    a.expert_pool_block_offset, a.expert_frequency = expert_pool_block_offset, expert_frequency
    a.dynamic_tiles = bool(dynamic_tiles)
    if lhs2 is not None:
        if out2 is None:
            out2 = torch.empty(E, lhs2.shape[1], rhs2.shape[1], dtype=lhs.dtype, device=lhs.device)
        a.a2, a.b2, a.out2 = lhs2, rhs2, out2
    if num_sms:
        a.num_ctas = num_sms
    _rt(buffer).grouped_gemm(a)
    return out if lhs2 is None else (out, out2)


def fire_tiles_with_delay(count: torch.Tensor, target: torch.Tensor, delay_us: float = 0.0, buffer=None):
    """Single-thread stand-in for dispatch: releases tile after tile
    (``count[i] += target[i]``) with ``delay_us`` between them."""
    _rt(buffer).tile_producer(count, target, float(delay_us))


def compress_pool_to_recv(pool: torch.Tensor, pool_recv_token: torch.Tensor, num_recv_tokens: int, buffer=None):
    """Gather one row per recv token out of the padded pool (checkpoint level 2;
    reference: stream_ep/stream_moe/recv_pool_compress.py:60-69)."""
    return _rt(buffer).pool_compress(pool, pool_recv_token, int(num_recv_tokens))


def reexpand_recv_to_pool(x_recv: torch.Tensor, pool_recv_token: torch.Tensor, tk_padded: int, buffer=None):
    """Inverse of :func:`compress_pool_to_recv`; padding rows come out zero
    (reference: stream_ep/stream_moe/recv_pool_compress.py:71-78)."""
    return _rt(buffer).pool_expand(x_recv, pool_recv_token, int(tk_padded))


def router_topk(x: torch.Tensor, w_gate: torch.Tensor, top_k: int, num_ranks: int = 1,
                renormalize: bool = True, return_probs: bool = False, buffer=None):
    """Fused linear gate -> softmax -> top-k -> renormalise -> rank bitmap.
    Returns ``(topk_idx int64, topk_weights f32, is_token_in_rank bool[, probs])``."""
    idx, w, in_rank, probs = _rt(buffer).router(x.contiguous(), w_gate.contiguous(), top_k, num_ranks,
                                                renormalize, return_probs)
    return (idx, w, in_rank, probs) if return_probs else (idx, w, in_rank)


def combine_reduce(out: torch.Tensor, landed_rows: torch.Tensor, topk_idx: torch.Tensor, num_experts: int,
                   dw_src: Optional[torch.Tensor] = None, dw_dst: Optional[torch.Tensor] = None,
                   sizes: Optional[torch.Tensor] = None, buffer=None):
    """``out[t] += sum_k landed_rows[t * K + k]`` over the pairs owned by other ranks, in fp32
    (second half of the fused combine; a no-op for a single rank).  With ``dw_src`` / ``dw_dst`` the same pass
    copies the per-pair scalars peers stored in ``dw_src [T, K]`` to ``dw_dst`` (0 for skipped pairs).
    ``sizes``: the device-side sizes of a capacity-mode dispatch; rows are ignored when its overflow flag is set."""
    _rt(buffer).combine_reduce(out, landed_rows, topk_idx.contiguous(), int(num_experts), dw_src, dw_dst, sizes)
    return out
