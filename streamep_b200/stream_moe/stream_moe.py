"""``stream_moe_func``: one expert-parallel MoE layer, forward and backward.

Public surface follows the reference (stream_ep/stream_moe/stream_moe.py:370-411,
:432-1260): ``StreamHolder`` / ``make_streams``, ``TileConfig``, the autograd
``StreamMoEFunc`` and ``stream_moe_func(buffer, x, topk_idx, topk_weights,
is_token_in_rank, w1_local, w2_local, *, streams, num_experts, tile_config,
activation_checkpoint_level)`` with ``w1_local [E_local, 2I, H]`` (gate/up rows
interleaved) and ``w2_local [E_local, H, I]``.

Two execution plans, selected per call (``fused=None`` reads ``STREAM_EP_FUSED``,
default on):

*fused* (the product path) - four kernels per direction, all on the compute stream:

    forward   metadata -> [host reads sizes] -> fill ->
              dispatch (+) GEMM-A/SwiGLU   one persistent kernel: push warps store this rank's
                                           token rows into the owners' pool slots over NVLink
                                           while tcgen05 warps consume 128-row tiles as they land
              GEMM-Y (+) combine           epilogue scales by the top-k weight and sends every row to
                                           the SOURCE rank: contiguous bf16 row stores over NVLink
                                           into a per-(token, k) landing buffer (bf16x2 red.add for
                                           rows of this rank's own tokens), then an fp32 reduce
    backward  dispatch_grads (+) GEMM-Y_bwd/dSwiGLU (+ dL/dweight returned to the source)
              GEMM-A_bwd (+) combine_grads (remote red.add into the source's dL/dx)
              dW2, dW1 grouped GEMMs (true-length varlen-K)

*unfused* (the reference's plan, stream_ep/stream_moe/stream_moe.py:447-1175) -
dispatch and combine are stand-alone kernels on the communicate stream, GEMMs on
the compute stream, overlapped per tile / per token through ``pool_arrival_count``
and ``y_done_per_token`` and ordered by the launch gates.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from types import SimpleNamespace
from typing import Optional

import torch

from ..ops import grouped_gemm as gg
from .tile_config import TileConfig, _resolve_tile_config, default_tile_config  # noqa: F401

KIND_DISPATCH, KIND_DISPATCH_GRADS = 1, 2
AUX0, AUX1 = 10, 11   # record words of the first two aux slots


@dataclass(frozen=True)
class StreamHolder:
    """The two caller-owned streams of a layer: ``communicate`` (stand-alone
    dispatch / combine kernels) and ``compute`` (all GEMM kernels, including the
    fused ones)."""
    communicate: torch.cuda.Stream
    compute: torch.cuda.Stream


def make_streams(device=None, prioritize_communicate: bool = False) -> StreamHolder:
    """Allocate the two streams once per process (stream_ep/stream_moe/stream_moe.py:387-411)."""
    if prioritize_communicate:
        return StreamHolder(communicate=torch.cuda.Stream(device=device, priority=-99),
                            compute=torch.cuda.Stream(device=device, priority=0))
    return StreamHolder(communicate=torch.cuda.Stream(device=device), compute=torch.cuda.Stream(device=device))


_NVTX_ENABLED = bool(os.environ.get("STREAM_EP_NVTX"))
_NVTX_FWD = 0
_NVTX_BWD = 0


def _nvtx_push(name: str) -> None:
    if _NVTX_ENABLED:
        torch.cuda.nvtx.range_push(name)


def _nvtx_pop() -> None:
    if _NVTX_ENABLED:
        torch.cuda.nvtx.range_pop()


def _fused_default() -> bool:
    return os.environ.get("STREAM_EP_FUSED", "1") not in ("0", "false", "False")


# ---------------------------------------------------------------------------------------------
# forward
# ---------------------------------------------------------------------------------------------
def moe_forward(ctx, streams, buffer, x, topk_idx, topk_weights, is_token_in_rank, w1, w2, num_experts,
                cfg: TileConfig, level: int, fused: bool):
    """Forward of one layer; fills ``ctx`` (any attribute bag) for :func:`moe_backward`."""
    global _NVTX_FWD
    _NVTX_FWD += 1
    _nvtx_push(f"moe_fwd_{_NVTX_FWD}")
    assert level in (0, 1, 2), "activation_checkpoint_level must be 0, 1 or 2"
    assert x.dtype == torch.bfloat16 and w1.dtype == torch.bfloat16 and w2.dtype == torch.bfloat16, "bf16 only"
    E_local, two_i, H = w1.shape
    I = two_i // 2
    assert w2.shape == (E_local, H, I), f"w2_local must be [E_local, H, I], got {tuple(w2.shape)}"
    assert num_experts == E_local * buffer.group_size
    T = x.shape[0]
    rt = buffer.runtime
    caller = torch.cuda.current_stream()
    comm, comp = streams.communicate, streams.compute
    x = x.contiguous()
    w1c, w2c = w1.contiguous(), w2.contiguous()

    comm.wait_stream(caller)
    comp.wait_stream(caller)
    if fused and not buffer._emulated:
        # Production path: everything after the metadata launch happens in one native call (see
        # Runtime::fused_forward) so that the GPU idles as briefly as possible after the host read.
        with torch.cuda.stream(comp):
            _nvtx_push(f"fwd_fused_{_NVTX_FWD}")
            K = topk_idx.shape[1]
            # capacity mode (Buffer.enable_capacity_mode): fixed receive regions, no host read of the sizes
            cap = rt.static_fits(T, H, K)
            landing = x.new_empty(0, H) if cap else \
                buffer.alloc_symmetric([T * K if buffer.group_size > 1 else 0, H], torch.bfloat16)
            st, seq = buffer._dispatch_begin(x, topk_idx, topk_weights, num_experts, cfg.tile_m, None, cap)
            rt.dispatch_metadata(st, 3)
            try:
                out, postact, preact = rt.fused_forward(st, w1c, w2c, landing, level == 0, cfg.tile_n_a, cfg.tile_n_y,
                                                        cfg.num_sms_a or 0, cfg.num_sms_y or 0)
            except RuntimeError as e:
                if "timed out" in str(e) or "metadata failed" in str(e):
                    from ..errors import StreamEPTimeout
                    raise StreamEPTimeout(str(e)) from None
                raise
            handle = buffer._make_handle(st, is_token_in_rank, seq, cfg.tile_m)
            TKp = handle.TK_padded
            del landing
            saved_pool = _maybe_compress(buffer, handle, level)
            _nvtx_pop()
    elif fused:
        with torch.cuda.stream(comp):
            _nvtx_push(f"fwd_dispatch_{_NVTX_FWD}")
            # rows that other ranks compute for this rank's tokens land here, one per (token, k)
            K = topk_idx.shape[1]
            cap = rt.static_fits(T, H, K)
            _, handle, _ = buffer.dispatch(x, topk_idx, topk_weights, is_token_in_rank, num_experts,
                                           tile_m=cfg.tile_m, launch_push=False, capacity_mode=cap)
            st = handle._dispatch_out
            if cap:
                landing, landing_off = rt.next_landing(T, H, K)
            else:
                landing, landing_off = buffer.alloc_symmetric([T * K if buffer.group_size > 1 else 0, H], torch.bfloat16), -1
                rt.dispatch_set_aux(st, 0, landing)
            _nvtx_pop()
        TKp = handle.TK_padded
        postact = torch.empty(TKp, I, dtype=x.dtype, device=x.device)
        preact = torch.empty(TKp, two_i, dtype=x.dtype, device=x.device) if level == 0 else None
        out = torch.zeros(T, H, dtype=x.dtype, device=x.device)
        comp.wait_stream(caller)
        with torch.cuda.stream(comp):
            _nvtx_push(f"fwd_compute_{_NVTX_FWD}")
            _launch_fused_a(buffer, handle, w1c, postact, preact, cfg)
            _nvtx_pop()
            _nvtx_push(f"fwd_combine_{_NVTX_FWD}")
            gg.streaming_moe_y(postact, w2c, handle.tile_id_to_expert, handle.pool_topk_weight,
                               handle.pool_recv_token, o=out, remote_out_offsets=(KIND_DISPATCH, st.push_epoch, AUX0),
                               remote_static_offset=landing_off, live_tiles=st.dev_sizes if cap else None,
                               pool_src=handle.pool_src, pool_k_slot=handle.pool_k_slot, num_topk=K,
                               tail_wait=not buffer._emulated, tile_n=cfg.tile_n_y, num_sms=cfg.num_sms_y, buffer=buffer)
            buffer._phase()
            gg.combine_reduce(out, landing, st.topk_idx, num_experts, sizes=st.dev_sizes if cap else None, buffer=buffer)
            buffer._phase()     # (emulated ranks) nobody reuses a landing buffer before every reduce is enqueued
            del landing
            _nvtx_pop()
            saved_pool = _maybe_compress(buffer, handle, level)
    else:
        with torch.cuda.stream(comm):
            _nvtx_push(f"fwd_dispatch_{_NVTX_FWD}")
            _, handle, meta_ev = buffer.dispatch(x, topk_idx, topk_weights, is_token_in_rank, num_experts,
                                                 tile_m=cfg.tile_m)
            st = handle._dispatch_out
            _nvtx_pop()
        TKp = handle.TK_padded
        postact = torch.empty(TKp, I, dtype=x.dtype, device=x.device)
        preact = torch.empty(TKp, two_i, dtype=x.dtype, device=x.device) if level == 0 else None
        stripes = torch.zeros(max(handle.total_tiles, 1), dtype=torch.int32, device=x.device)
        comp.wait_stream(caller)
        meta_ev.wait_on(comp.cuda_stream, x.device.index if x.device.index is not None else torch.cuda.current_device())
        buffer.wait_dispatch_main_started(comp)
        with torch.cuda.stream(comp):
            _nvtx_push(f"fwd_compute_{_NVTX_FWD}")
            if handle.total_tiles > 0:
                gg.streaming_moe_a(handle.pool, w1c, handle.tile_id_to_expert, postact_a=postact, preact_a=preact,
                                   pool_arrival_count=handle.pool_arrival_count,
                                   pool_arrival_target=handle.pool_arrival_target, tile_n=cfg.tile_n_a,
                                   num_sms=cfg.num_sms_a, buffer=buffer)
                buffer.bump_kernel_y_issued()
                gg.streaming_moe_y(postact, w2c, handle.tile_id_to_expert, handle.pool_topk_weight,
                                   handle.pool_recv_token, o=handle.o, tile_n_stripes_done=stripes,
                                   k_local_remaining=handle.k_local_remaining,
                                   y_done_per_token=handle.y_done_per_token, combine_seq=handle.dispatch_seq,
                                   started_flag=True, tile_n=cfg.tile_n_y, num_sms=cfg.num_sms_y, buffer=buffer)
            _nvtx_pop()
        buffer.wait_kernel_y_started(comm)
        if buffer._emulated:
            buffer._phase()          # every rank's kernel Y is enqueued before any gather
        with torch.cuda.stream(comm):
            _nvtx_push(f"fwd_combine_{_NVTX_FWD}")
            out, _ = buffer.combine(handle.o, handle)
            _nvtx_pop()
        with torch.cuda.stream(comp):
            saved_pool = _maybe_compress(buffer, handle, level)
        handle.o = None
        st.release_o()
    caller.wait_stream(comm)
    caller.wait_stream(comp)

    ctx.buffer, ctx.streams, ctx.handle, ctx.cfg, ctx.level, ctx.fused = buffer, streams, handle, cfg, level, fused
    ctx.shapes = (T, H, I, E_local)
    ctx.saved = SimpleNamespace(preact=preact, pool=saved_pool, w1=w1c, w2=w2c)
    _nvtx_pop()
    return out


def _launch_fused_a(buffer, handle, w1, postact, preact, cfg):
    """dispatch (+) GEMM-A.  One launch per rank in production; for ranks emulated on one device
    the same kernel runs three times (publish records / push rows / consume tiles) so that no
    launch ever waits for a later one."""
    st = handle._dispatch_out
    common = dict(postact_a=postact, preact_a=preact, pool_arrival_count=handle.pool_arrival_count,
                  pool_arrival_target=handle.pool_arrival_target, tile_n=cfg.tile_n_a, num_sms=cfg.num_sms_a,
                  buffer=buffer, fused_dispatch=st, live_tiles=st.dev_sizes if st.region_id >= 0 else None)
    if not buffer._emulated:
        gg.streaming_moe_a(handle.pool, w1, handle.tile_id_to_expert, push_flags=3, **common)
        return
    buffer.runtime.dispatch_push(st, 1, 1)
    buffer._phase()
    gg.streaming_moe_a(handle.pool, w1, handle.tile_id_to_expert, push_flags=2, num_tiles=0, **common)
    buffer._phase()
    gg.streaming_moe_a(handle.pool, w1, handle.tile_id_to_expert, push_flags=0, **common)


def _maybe_compress(buffer, handle, level):
    """What backward needs of the dispatched rows: the pool itself (levels 0/1) or, at level 2, one
    compact row per recv token (stream_ep/stream_moe/stream_moe.py:661-678)."""
    if level < 2:
        return handle.pool
    x_recv = gg.compress_pool_to_recv(handle.pool, handle.pool_recv_token, handle.num_recv_tokens, buffer=buffer) \
        if handle.TK_padded > 0 else handle.pool.new_empty(handle.num_recv_tokens, handle.pool.shape[1])
    handle.pool = None
    handle._dispatch_out.release_pool()
    return x_recv


# ---------------------------------------------------------------------------------------------
# backward
# ---------------------------------------------------------------------------------------------
def moe_backward(ctx, dL_dy):
    """Returns ``(dL_dx [T, H] bf16, dL_dtopk_weights [T, K] f32, dW1, dW2)``."""
    global _NVTX_BWD
    _NVTX_BWD += 1
    _nvtx_push(f"moe_bwd_{_NVTX_BWD}")
    buffer, streams, handle, cfg, level, fused = ctx.buffer, ctx.streams, ctx.handle, ctx.cfg, ctx.level, ctx.fused
    T, H, I, E_local = ctx.shapes
    sv = ctx.saved
    st = handle._dispatch_out
    rt = buffer.runtime
    K = st.num_topk
    dev = dL_dy.device
    caller = torch.cuda.current_stream()
    comm, comp = streams.communicate, streams.compute
    dL_dy = dL_dy.contiguous().to(torch.bfloat16)
    TKp, tiles = handle.TK_padded, handle.total_tiles
    if fused and not buffer._emulated:
        # Production path: one native call (Runtime::fused_backward) issues the whole backward.
        comp.wait_stream(caller)
        with torch.cuda.stream(comp):
            dL_dx, dL_dw, dW1, dW2 = rt.fused_backward(
                st, dL_dy, sv.w1, sv.w2, sv.pool, sv.preact, level, cfg.tile_n_a, cfg.tile_n_y_bwd, cfg.tile_n_a_bwd,
                cfg.tile_n_dW1, cfg.tile_n_dW2, cfg.num_sms_y_bwd or 0, cfg.num_sms_a_bwd or 0)
        caller.wait_stream(comp)
        _nvtx_pop()
        return dL_dx, dL_dw, dW1, dW2

    dswiglu_in = torch.empty(TKp, 2 * I, dtype=torch.bfloat16, device=dev)
    postact_dw2 = torch.empty(TKp, I, dtype=torch.bfloat16, device=dev)
    dW1 = torch.empty_like(sv.w1)
    dW2 = torch.empty_like(sv.w2)
    zeros_i32 = torch.zeros(max(tiles, 1) * 2 + TKp, dtype=torch.int32, device=dev)
    stripes_y = zeros_i32[:max(tiles, 1)]
    stripes_a = zeros_i32[max(tiles, 1):2 * max(tiles, 1)]
    dl_dweight = zeros_i32[2 * max(tiles, 1):].view(torch.float32)
    comm.wait_stream(caller)
    comp.wait_stream(caller)

    def rebuild_inputs():
        pool = sv.pool
        if level == 2:
            pool = gg.reexpand_recv_to_pool(sv.pool, handle.pool_recv_token, TKp, buffer=buffer) if TKp > 0 \
                else sv.pool.new_empty(0, H)
        preact = sv.preact
        if preact is None:
            preact = gg.grouped_gemm_preact(pool, sv.w1, handle.tile_id_to_expert, tile_n=cfg.tile_n_a,
                                            live_tiles=st.dev_sizes if st.region_id >= 0 else None,
                                            buffer=buffer) if tiles > 0 else pool.new_empty(0, 2 * I)
        return pool, preact

    if fused:
        with torch.cuda.stream(comp):
            dx = torch.zeros(T, H, dtype=torch.bfloat16, device=dev)
            dl_do_pool, bwd_count, _ = buffer.dispatch_grads(handle, dL_dy, launch_push=False, fused_buffers=True)
            g = handle._grads_state
            landing, dwt = g.landing, g.dwt
            cap = g.is_static
            live = st.dev_sizes if cap else None
            pool, preact = rebuild_inputs()
            ykw = dict(dL_dswiglu_in=dswiglu_in, postact_a_for_dW2=postact_dw2, dL_dweight=dl_dweight,
                       arrival_count=bwd_count, arrival_target=handle.pool_arrival_target,
                       remote_dw_offsets=(KIND_DISPATCH_GRADS, g.epoch, AUX1), remote_static_offset=g.dwt_off,
                       live_tiles=live, pool_src=handle.pool_src,
                       pool_k_slot=handle.pool_k_slot, num_topk=K, tile_n_stripes_done=stripes_y,
                       fused_dispatch_grads=g, fused_routing=st, fused_rows=dL_dy, tile_n=cfg.tile_n_y_bwd,
                       num_sms=cfg.num_sms_y_bwd, buffer=buffer)
            yargs = (dl_do_pool, sv.w2, preact, handle.tile_id_to_expert, handle.pool_topk_weight, handle.pool_recv_token)
            if not buffer._emulated:
                gg.streaming_moe_y_bwd(*yargs, push_flags=3, **ykw)
            else:
                rt.grads_push(st, g, dL_dy, 1, 1)
                buffer._phase()
                gg.streaming_moe_y_bwd(*yargs, push_flags=2, num_tiles=0, **ykw)
                buffer._phase()
                gg.streaming_moe_y_bwd(*yargs, push_flags=0, **ykw)
            gg.streaming_moe_a_bwd(dswiglu_in, sv.w1, handle.tile_id_to_expert, handle.pool_recv_token,
                                   dL_dx_per_r=dx, remote_out_offsets=(KIND_DISPATCH_GRADS, g.epoch, AUX0),
                                   remote_static_offset=g.landing_off, live_tiles=live,
                                   pool_src=handle.pool_src, pool_k_slot=handle.pool_k_slot, num_topk=K,
                                   tail_wait=not buffer._emulated, tile_n=cfg.tile_n_a_bwd,
                                   num_sms=cfg.num_sms_a_bwd, buffer=buffer)
            buffer._phase()
            if cap:     # copy the per-pair dL/dweight out of its fixed region in the same pass
                dwt_out = torch.empty(T, K, dtype=torch.float32, device=dev)
                gg.combine_reduce(dx, landing, st.topk_idx, st.num_experts, dw_src=dwt, dw_dst=dwt_out, sizes=live, buffer=buffer)
                dwt = dwt_out
                rt.grads_finish(g)
            else:
                gg.combine_reduce(dx, landing, st.topk_idx, st.num_experts, buffer=buffer)
            buffer._phase()
            del landing
            _launch_dw(buffer, handle, cfg, dl_do_pool, postact_dw2, dswiglu_in, pool, dW1, dW2)
        dL_dx, dL_dw = dx, dwt
    else:
        with torch.cuda.stream(comm):
            dl_do_pool, bwd_count, started_ev = buffer.dispatch_grads(handle, dL_dy)
        dx_per_r = buffer.alloc_symmetric([handle.num_recv_tokens, H], torch.bfloat16)
        a_done = buffer.alloc_symmetric([handle.num_recv_tokens], torch.int64)
        dlw_sym = buffer.alloc_symmetric([TKp], torch.float32)
        started_ev.wait_on(comp.cuda_stream, dev.index if dev.index is not None else torch.cuda.current_device())
        buffer.wait_dispatch_grads_started(comp)
        with torch.cuda.stream(comp):
            dx_per_r.zero_(); a_done.zero_(); dlw_sym.zero_()
            k_rem = handle.k_local_total.clone()
            pool, preact = rebuild_inputs()
            if tiles > 0:
                gg.streaming_moe_y_bwd(dl_do_pool, sv.w2, preact, handle.tile_id_to_expert, handle.pool_topk_weight,
                                       handle.pool_recv_token, dL_dswiglu_in=dswiglu_in,
                                       postact_a_for_dW2=postact_dw2, dL_dweight=dlw_sym, arrival_count=bwd_count,
                                       arrival_target=handle.pool_arrival_target, tile_n=cfg.tile_n_y_bwd,
                                       num_sms=cfg.num_sms_y_bwd, buffer=buffer)
                buffer.bump_kernel_a_bwd_issued()
                gg.streaming_moe_a_bwd(dswiglu_in, sv.w1, handle.tile_id_to_expert, handle.pool_recv_token,
                                       dL_dx_per_r=dx_per_r, tile_n_stripes_done=stripes_a,
                                       bwd_k_local_remaining=k_rem, bwd_a_done_per_token=a_done,
                                       dispatch_seq=handle.dispatch_seq, started_flag=True,
                                       tile_n=cfg.tile_n_a_bwd, num_sms=cfg.num_sms_a_bwd, buffer=buffer)
        buffer.wait_kernel_a_bwd_started(comm)
        if buffer._emulated:
            buffer._phase()
        with torch.cuda.stream(comm):
            dL_dx, dL_dw = buffer.combine_grads(dx_per_r, handle, dlw_sym, a_done)
        with torch.cuda.stream(comp):
            _launch_dw(buffer, handle, cfg, dl_do_pool, postact_dw2, dswiglu_in, pool, dW1, dW2)
    caller.wait_stream(comm)
    caller.wait_stream(comp)
    _nvtx_pop()
    return dL_dx, dL_dw, dW1, dW2


def _launch_dw(buffer, handle, cfg, dl_do_pool, postact_dw2, dswiglu_in, pool, dW1, dW2):
    """dW2[e] = dL_do_pool[rows_e]^T @ (w * postact)[rows_e];  dW1[e] = dL_dswiglu_in[rows_e]^T @ pool[rows_e]
    (stream_ep/stream_moe/stream_moe.py:1107-1146, including the empty-rank guard)."""
    buffer.runtime.mark_local_phase()
    if handle.total_tiles > 0:
        if cfg.tile_n_dW1 == cfg.tile_n_dW2:      # one launch for both, tiles claimed dynamically
            gg.grouped_gemm_dw(dswiglu_in, pool, handle.expert_pool_block_offset, handle.expert_frequency, out=dW1,
                               lhs2=dl_do_pool, rhs2=postact_dw2, out2=dW2, tile_n=cfg.tile_n_dW1, dynamic_tiles=True,
                               buffer=buffer)
        else:
            gg.grouped_gemm_dw(dl_do_pool, postact_dw2, handle.expert_pool_block_offset, handle.expert_frequency,
                               out=dW2, tile_n=cfg.tile_n_dW2, dynamic_tiles=True, buffer=buffer)
            gg.grouped_gemm_dw(dswiglu_in, pool, handle.expert_pool_block_offset, handle.expert_frequency,
                               out=dW1, tile_n=cfg.tile_n_dW1, dynamic_tiles=True, buffer=buffer)
    else:
        dW1.zero_()
        dW2.zero_()


class StreamMoEFunc(torch.autograd.Function):
    """Autograd boundary of the layer (stream_ep/stream_moe/stream_moe.py:432-1175)."""

    @staticmethod
    def forward(ctx, streams, buffer, x, topk_idx, topk_weights, is_token_in_rank, w1_local, w2_local,
                num_experts, cfg, activation_checkpoint_level, fused):
        ctx.state = SimpleNamespace()
        out = moe_forward(ctx.state, streams, buffer, x, topk_idx, topk_weights, is_token_in_rank, w1_local,
                          w2_local, num_experts, cfg, activation_checkpoint_level, fused)
        return out

    @staticmethod
    def backward(ctx, dL_dy):
        dL_dx, dL_dw, dW1, dW2 = moe_backward(ctx.state, dL_dy)
        ctx.state = None
        return None, None, dL_dx, None, dL_dw, None, dW1, dW2, None, None, None, None


def stream_moe_func(buffer, x: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor,
                    is_token_in_rank: Optional[torch.Tensor], w1_local: torch.Tensor, w2_local: torch.Tensor, *,
                    streams: StreamHolder, num_experts: int, tile_config: Optional[TileConfig] = None,
                    activation_checkpoint_level: int = 0, fused: Optional[bool] = None) -> torch.Tensor:
    """One MoE layer: dispatch, SwiGLU expert MLP, combine; differentiable in ``x``,
    ``topk_weights``, ``w1_local`` and ``w2_local``.  Returns ``[num_tokens, hidden]`` bf16 for
    this rank's tokens (signature and semantics: stream_ep/stream_moe/stream_moe.py:1178-1260).

    ``activation_checkpoint_level``: 0 keeps ``preact_a`` and the pool; 1 keeps the pool and
    recomputes ``preact_a`` in backward; 2 keeps one compact row per recv token and re-expands the
    pool in backward.
    """
    _, two_i, H = w1_local.shape
    cfg = _resolve_tile_config(tile_config, two_i // 2, H)
    if fused is None:
        fused = _fused_default()
    return StreamMoEFunc.apply(streams, buffer, x, topk_idx, topk_weights, is_token_in_rank, w1_local, w2_local,
                               num_experts, cfg, activation_checkpoint_level, fused)
