"""Tile configuration of the layer's GEMM kernels.

Same public surface as the reference (stream_ep/stream_moe/stream_moe.py:126-367):
a frozen, all-optional ``TileConfig`` of overrides, ``default_tile_config(I, H)``
and ``_resolve_tile_config``.  The values differ because the kernels do: on
sm_100a one CTA drives a 128 x tile_n UMMA with the accumulator in tensor
memory, so

* ``tile_m`` is structurally 128 (one UMMA M tile == the pool padding grain);
* every ``tile_n`` is 128 or 256 (two accumulator buffers of ``tile_n`` fp32
  columns fill at most the 512 TMEM columns);
* output widths need not be multiples of ``tile_n`` - partial tiles are
  masked in the epilogue and zero-filled by TMA - but must be multiples of 8;
* the ``cluster_*``, ``pingpong_*`` and ``swizzle_*`` fields are accepted for
  source compatibility and ignored: the kernels never use cluster multicast
  loads, and the epilogue/mainloop overlap that "pingpong" buys on Hopper comes
  from the double-buffered TMEM accumulator here.
"""
from __future__ import annotations

from dataclasses import dataclass, fields, replace
from typing import Optional

_VALID_TILE_N = (128, 256)


def _pick(n: int) -> int:
    """256 unless masking the last 256-wide tile wastes over 15 % more work than 128-wide tiles."""
    if n <= 128:
        return 128
    waste256 = (-(-n // 256) * 256) / n
    waste128 = (-(-n // 128) * 128) / n
    return 256 if waste256 <= 1.15 * waste128 else 128


@dataclass(frozen=True)
class TileConfig:
    tile_m: Optional[int] = None
    tile_n_a: Optional[int] = None        # fwd kernel A, output width 2I
    tile_n_y: Optional[int] = None        # fwd kernel Y, output width H
    tile_n_y_bwd: Optional[int] = None    # bwd kernel Y, output width I
    tile_n_a_bwd: Optional[int] = None    # bwd kernel A, output width H
    tile_m_dW1: Optional[int] = None
    tile_n_dW1: Optional[int] = None      # dW1 [2I, H]: width H
    tile_m_dW2: Optional[int] = None
    tile_n_dW2: Optional[int] = None      # dW2 [H, I]: width I
    cluster_m_dW1: Optional[int] = None
    cluster_n_dW1: Optional[int] = None
    cluster_m_dW2: Optional[int] = None
    cluster_n_dW2: Optional[int] = None
    pingpong_dW1: Optional[bool] = None
    pingpong_dW2: Optional[bool] = None
    swizzle_dW1: Optional[int] = None
    swizzle_dW2: Optional[int] = None
    num_sms_a: Optional[int] = None
    num_sms_y: Optional[int] = None
    num_sms_a_bwd: Optional[int] = None
    num_sms_y_bwd: Optional[int] = None

    def validate(self, I: int, H: int) -> None:
        """Raise ``ValueError`` when a knob cannot be honoured for weights
        ``w1 [E, 2I, H]`` / ``w2 [E, H, I]``.  ``None`` fields are skipped."""
        errs = []
        for name in ("tile_m", "tile_m_dW1", "tile_m_dW2"):
            v = getattr(self, name)
            if v is not None and v != 128:
                errs.append(f"{name}={v}: the M tile is one 128-row UMMA (and the pool padding grain)")
        for name in ("tile_n_a", "tile_n_y", "tile_n_y_bwd", "tile_n_a_bwd", "tile_n_dW1", "tile_n_dW2"):
            v = getattr(self, name)
            if v is not None and v not in _VALID_TILE_N:
                errs.append(f"{name}={v}: must be 128 or 256")
        if I % 8 != 0 or H % 8 != 0:
            errs.append(f"I={I} and H={H} must be multiples of 8 (16-byte rows for TMA)")
        for name in ("num_sms_a", "num_sms_y", "num_sms_a_bwd", "num_sms_y_bwd"):
            v = getattr(self, name)
            if v is not None and v <= 0:
                errs.append(f"{name}={v} must be positive")
        if errs:
            raise ValueError(f"TileConfig invalid for (I={I}, H={H}): " + "; ".join(errs))


def default_tile_config(I: int, H: int) -> TileConfig:
    """Shape-picked baseline: 256-wide tiles unless the masked tail costs too much."""
    return TileConfig(
        tile_m=128,
        tile_n_a=_pick(2 * I), tile_n_y=_pick(H), tile_n_y_bwd=_pick(I), tile_n_a_bwd=_pick(H),
        tile_m_dW1=128, tile_n_dW1=_pick(H), tile_m_dW2=128, tile_n_dW2=_pick(I),
        cluster_m_dW1=1, cluster_n_dW1=1, cluster_m_dW2=1, cluster_n_dW2=1,
        pingpong_dW1=False, pingpong_dW2=False, swizzle_dW1=1, swizzle_dW2=1,
        num_sms_a=None, num_sms_y=None, num_sms_a_bwd=None, num_sms_y_bwd=None,
    )


def _resolve_tile_config(tile_config: Optional[TileConfig], I: int, H: int) -> TileConfig:
    """Overlay the caller's non-``None`` fields on the baseline and validate."""
    cfg = default_tile_config(I, H)
    if tile_config is not None:
        over = {f.name: getattr(tile_config, f.name) for f in fields(tile_config)
                if getattr(tile_config, f.name) is not None}
        if over:
            cfg = replace(cfg, **over)
    cfg.validate(I, H)
    return cfg
