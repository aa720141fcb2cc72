"""``StreamMoE``: router + expert-parallel SwiGLU experts as an ``nn.Module``.

This is the model-side wrapper a user of the reference writes around
``stream_moe_func`` (its harnesses build one inline: stream_ep/stream_moe/
profile_pipeline.py:102-139,338-348 for routing, :300-336 for ``make_buffer``).
Weights use the reference's layout: ``w1 [E_local, 2I, H]`` with gate/up rows
interleaved, ``w2 [E_local, H, I]``.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from ..buffer import Buffer
from ..ops.grouped_gemm import router_topk
from ..stream_moe import StreamHolder, TileConfig, make_streams, stream_moe_func


def make_buffer(group, num_tokens: int, hidden: int, num_topk: int, num_experts: int, *,
                layers_in_flight: int = 1, world_size: Optional[int] = None, imbalance: float = 1.5,
                timeout_ms: Optional[int] = None, capacity_factor: Optional[float] = None) -> Buffer:
    """Size and construct the symmetric buffer for ``layers_in_flight`` layers whose forward
    state is alive at the same time (reference: ``make_buffer`` in
    stream_ep/stream_moe/profile_pipeline.py).

    ``capacity_factor`` (e.g. 1.5) switches the fused layer to fixed receive regions of that many times the
    balanced load, which removes the per-forward host read of the receive sizes
    (:meth:`Buffer.enable_capacity_mode`); ``None`` keeps exact, dropless sizing."""
    ws = world_size if world_size is not None else (group.size() if group is not None else 1)
    if capacity_factor is not None:
        # the fixed regions hold the pools; the rest of the arena only serves the occasional exact-mode call
        arena = Buffer.capacity_mode_bytes(num_tokens, hidden, num_topk, num_experts, ws, capacity_factor=capacity_factor,
                                           layers_in_flight=layers_in_flight) + (64 << 20)
    else:
        arena = Buffer.get_arena_size_hint(num_tokens, hidden, num_topk, ws, max(num_experts // ws, 1),
                                           layers_in_flight=layers_in_flight, imbalance=imbalance)
    if group is None:
        from ..buffer import LocalWorld
        buf = LocalWorld(1, arena_bytes=arena, timeout_ms=timeout_ms or 10000).buffers[0]
    else:
        buf = Buffer(group, arena, timeout_ms=timeout_ms)
    if capacity_factor is not None:
        buf.enable_capacity_mode(num_tokens, hidden, num_topk, num_experts, capacity_factor=capacity_factor,
                                 layers_in_flight=layers_in_flight)
    return buf


class StreamMoE(nn.Module):
    def __init__(self, hidden: int, ffn: int, num_experts: int, top_k: int, buffer: Buffer, *,
                 streams: Optional[StreamHolder] = None, tile_config: Optional[TileConfig] = None,
                 activation_checkpoint_level: int = 0, fused: Optional[bool] = None, renormalize: bool = True,
                 device=None, seed: int = 0, init_std: float = 0.02):
        super().__init__()
        self.hidden, self.ffn, self.num_experts, self.top_k = hidden, ffn, num_experts, top_k
        self.buffer = buffer
        self.ep_size, self.ep_rank = buffer.group_size, buffer.rank
        assert num_experts % self.ep_size == 0
        self.num_local_experts = num_experts // self.ep_size
        self.tile_config = tile_config
        self.level = activation_checkpoint_level
        self.fused = fused
        self.renormalize = renormalize
        self._streams = streams
        g = torch.Generator(device="cpu").manual_seed(seed)
        # the router is replicated; expert weights are this rank's shard of the global init
        w_gate = torch.randn(num_experts, hidden, generator=g) * init_std
        g_local = torch.Generator(device="cpu").manual_seed(seed * 1000003 + self.ep_rank + 1)
        w1 = torch.randn(self.num_local_experts, 2 * ffn, hidden, generator=g_local) * init_std
        w2 = torch.randn(self.num_local_experts, hidden, ffn, generator=g_local) * init_std
        self.w_gate = nn.Parameter(w_gate.to(torch.bfloat16).to(device), requires_grad=False)
        self.w1 = nn.Parameter(w1.to(torch.bfloat16).to(device))
        self.w2 = nn.Parameter(w2.to(torch.bfloat16).to(device))

    @property
    def streams(self) -> StreamHolder:
        if self._streams is None:
            self._streams = make_streams(self.w1.device)
        return self._streams

    def route(self, x: torch.Tensor):
        """``(topk_idx, topk_weights, is_token_in_rank)`` from the fused router kernel."""
        return router_topk(x.detach(), self.w_gate, self.top_k, num_ranks=self.ep_size,
                           renormalize=self.renormalize, buffer=self.buffer)

    def experts(self, x, topk_idx, topk_weights, is_token_in_rank):
        return stream_moe_func(self.buffer, x, topk_idx, topk_weights, is_token_in_rank, self.w1, self.w2,
                               streams=self.streams, num_experts=self.num_experts, tile_config=self.tile_config,
                               activation_checkpoint_level=self.level, fused=self.fused)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        idx, w, in_rank = self.route(x)
        return self.experts(x, idx, w, in_rank)
