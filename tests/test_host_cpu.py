"""CPU-only checks of the host-side pieces: tile configuration, the symmetric-arena allocator,
the native Config, failure detection on the host (stall watchdog, heartbeat rank monitor) and
the package surface.  (Tile-config cases mirror stream_ep/stream_moe/tests/test_tile_config.py.)
"""
import io
import os
import sys
import time

import pytest
import torch
import torch.multiprocessing as mp

from streamep_b200 import _ext
from streamep_b200.stream_moe.tile_config import TileConfig, _resolve_tile_config, default_tile_config

needs_ext = pytest.mark.skipif(not _ext.available(), reason="native extension not built")


# ------------------------------------------------------------------ tile config
def test_default_tile_config_flagship_shape():
    cfg = default_tile_config(1408, 2048)
    assert cfg.tile_m == 128 and cfg.tile_n_a == 256 and cfg.tile_n_y == 256 and cfg.tile_n_a_bwd == 256
    assert cfg.tile_n_y_bwd == 256 and cfg.tile_n_dW2 == 256      # 1408 = 5.5 x 256: 9 % masked, still wider wins
    cfg.validate(1408, 2048)


def test_default_tile_config_small_and_awkward_widths():
    assert default_tile_config(64, 128).tile_n_a == 128
    assert default_tile_config(64, 128).tile_n_y == 128
    assert default_tile_config(640, 384).tile_n_y == 128            # 384 = 3 x 128 exactly, 1.5 x 256 wastes 33 %
    assert default_tile_config(14336, 4096).tile_n_a == 256


def test_all_fields_default_to_none():
    t = TileConfig()
    assert all(getattr(t, f) is None for f in t.__dataclass_fields__)


def test_override_only_touches_named_fields():
    cfg = _resolve_tile_config(TileConfig(tile_n_a=128, num_sms_a=120), 1408, 2048)
    assert cfg.tile_n_a == 128 and cfg.num_sms_a == 120
    assert cfg.tile_n_y == default_tile_config(1408, 2048).tile_n_y


def test_none_config_returns_baseline():
    assert _resolve_tile_config(None, 768, 3072) == default_tile_config(768, 3072)


@pytest.mark.parametrize("bad", [dict(tile_n_a=192), dict(tile_n_y=64), dict(tile_n_y_bwd=512), dict(tile_m=256),
                                 dict(tile_m=192), dict(tile_m=320), dict(tile_m_dW1=64), dict(num_sms_y=0)])
def test_invalid_overrides_raise(bad):
    with pytest.raises(ValueError, match="TileConfig invalid"):
        _resolve_tile_config(TileConfig(**bad), 1408, 2048)


def test_validate_rejects_unaligned_widths():
    with pytest.raises(ValueError):
        default_tile_config(1412, 2048).validate(1412, 2048)   # not a multiple of 8


def test_legacy_fields_are_accepted_and_ignored():
    cfg = _resolve_tile_config(TileConfig(cluster_m_dW1=2, cluster_n_dW1=2, pingpong_dW2=True, swizzle_dW1=8), 768, 3072)
    assert cfg.cluster_m_dW1 == 2 and cfg.pingpong_dW2 is True


def test_tile_config_is_frozen():
    with pytest.raises(Exception):
        TileConfig().tile_m = 64


# ------------------------------------------------------------------ arena
@needs_ext
def test_arena_best_fit_and_merge():
    C = _ext.load()
    a = C.ArenaProbe(0, 1 << 20)
    x = a.allocate(10_000); y = a.allocate(20_000); z = a.allocate(5_000)
    assert x % 1024 == 0 and y % 1024 == 0 and z % 1024 == 0 and len({x, y, z}) == 3
    used = a.in_use()
    a.release(y)
    assert a.in_use() < used
    w = a.allocate(18_000)          # fits the hole left by y
    assert w == y
    a.release(x); a.release(w); a.release(z)
    assert a.in_use() == 0 and a.free_blocks() == 1     # everything merged back into one block
    assert a.high_water() >= used


@needs_ext
def test_arena_zero_size_and_exhaustion():
    C = _ext.load()
    a = C.ArenaProbe(4096, 8192)
    p = a.allocate(0)
    assert a.in_use() == 1024       # empty tensors still own a block so that offsets stay unique
    with pytest.raises(RuntimeError, match="arena exhausted"):
        a.allocate(1 << 20)
    a.release(p)
    a.release(p)                    # double release is ignored
    assert a.in_use() == 0


@needs_ext
def test_arena_deferred_release_waits_for_its_fence():
    """A block whose tensor died while work on it may still be queued is not handed out again before its
    fence completes; when nothing else fits, allocate() waits for the fence instead of failing."""
    C = _ext.load()
    a = C.ArenaProbe(0, 64 * 1024)
    x = a.allocate(40_000)
    a.release_deferred(x)
    assert a.in_use() == 0 and a.parked() == 1          # logically free, physically held back
    y = a.allocate(20_000)
    assert y != x and not (x <= y < x + 40_000)          # served from the untouched remainder
    a.open_fences()
    assert a.parked() == 0
    z = a.allocate(40_000)
    assert z == x                                        # reusable once the fence is ready
    a.release_deferred(z)
    w = a.allocate(40_000)                               # only fits by waiting for z's fence
    assert w == x and a.parked() == 0
    a.release(w); a.release(y)
    assert a.in_use() == 0 and a.free_blocks() == 1


@needs_ext
def test_arena_random_stress_keeps_blocks_disjoint():
    import random
    C = _ext.load()
    a = C.ArenaProbe(0, 8 << 20)
    rnd = random.Random(0)
    live = {}
    for _ in range(2000):
        if live and rnd.random() < 0.45:
            off = rnd.choice(list(live))
            a.release(off); del live[off]
        else:
            n = rnd.randint(1, 60_000)
            try:
                off = a.allocate(n)
            except RuntimeError:
                continue
            for o, m in live.items():
                assert off + n <= o or o + m <= off, "overlapping blocks"
            live[off] = n
    for off in list(live):
        a.release(off)
    assert a.in_use() == 0 and a.free_blocks() == 1


# ------------------------------------------------------------------ native Config / package surface
@needs_ext
def test_config_validation_and_fields():
    import streamep_b200
    cfg = streamep_b200.Config(80, 6, 256, 6, 128)
    assert (cfg.num_sms, cfg.num_max_nvl_chunked_send_tokens, cfg.num_max_nvl_chunked_recv_tokens) == (80, 6, 256)
    with pytest.raises(ValueError):
        streamep_b200.Config(80, 256, 6, 6, 128)        # send must be smaller than recv
    # the ring-size hints of the reference keep their call shape; the value covers a stated workload
    small, large = cfg.get_nvl_buffer_size_hint(2048 * 2, 8), cfg.get_nvl_buffer_size_hint(7168 * 2, 8)
    assert 0 < small < large and large >= streamep_b200.Buffer.get_arena_size_hint(8192, 7168, 8, 8, 32)
    assert cfg.get_rdma_buffer_size_hint(7168 * 2, 8) == 0
    with pytest.raises(ValueError):
        cfg.get_nvl_buffer_size_hint(14336, 9)


def test_buffer_policy_tables_without_gpu():
    from streamep_b200 import Buffer
    old = (Buffer.num_sms, Buffer._num_sms_explicit)
    try:
        Buffer._num_sms_explicit = False
        assert Buffer.autopick_num_sms(8) == 80 and Buffer.autopick_num_sms(32) == 64
        Buffer.set_num_sms(24)
        assert Buffer.autopick_num_sms(8) == 24
        with pytest.raises(AssertionError):
            Buffer.set_num_sms(25)
    finally:
        Buffer.num_sms, Buffer._num_sms_explicit = old
    assert not Buffer.is_sm90_compiled()


def test_compat_package_reexports():
    import stream_ep
    from stream_ep.stream_moe.stream_moe import TileConfig as T2, stream_moe_func  # noqa: F401
    assert stream_ep.Buffer is __import__("streamep_b200").Buffer
    assert stream_ep.topk_idx_t == torch.int64


# ------------------------------------------------------------------ failure detection on the host
def test_stall_watchdog_fires_and_recovers():
    from streamep_b200.utils.watchdog import StallWatchdog
    reports = []
    sink = io.StringIO()
    with StallWatchdog(0.15, on_stall=reports.append, stream=sink) as w:
        for _ in range(5):
            time.sleep(0.05); w.heartbeat()
        assert not reports
        time.sleep(0.4)                     # "hang"
    assert reports and "no heartbeat" in reports[0] and "test_stall_watchdog_fires_and_recovers" in reports[0]
    assert w.stalls >= 1


def _monitor_worker(rank, world, path, q):
    import torch.distributed as dist
    from streamep_b200.errors import StreamEPError
    from streamep_b200.utils.watchdog import RankMonitor
    store = dist.FileStore(path, world)
    mon = RankMonitor(store, rank, world, period_s=0.05).start()
    store.set(f"ready/{rank}", "1")
    store.wait([f"ready/{r}" for r in range(world)])
    if rank == 1:
        time.sleep(0.3)
        mon.mark_leaving()                   # leaves between steps, nothing in flight
        q.put((rank, "left"))
        return
    try:
        assert mon.dead_ranks(1.0) == []
        deadline = time.time() + 10
        while not mon.dead_ranks(1.0) and time.time() < deadline:
            time.sleep(0.05)
        try:
            mon.assert_all_alive(1.0)
            q.put((rank, "no error raised"))
        except StreamEPError as e:
            q.put((rank, "detected" if "[1]" in str(e) else str(e)))
    finally:
        mon.stop()


def test_rank_monitor_detects_a_rank_that_left(tmp_path):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    path = str(tmp_path / "store")
    procs = [ctx.Process(target=_monitor_worker, args=(r, 2, path, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=30)
    assert res == {0: "detected", 1: "left"}, res


def test_errors_hierarchy():
    from streamep_b200 import StreamEPError, StreamEPTimeout
    assert issubclass(StreamEPTimeout, StreamEPError) and issubclass(StreamEPError, RuntimeError)


# ------------------------------------------------------------------ roofline arithmetic
def test_roofline_model_of_the_flagship_layer():
    from streamep_b200.utils.roofline import Peaks, layer_rooflines, step_flops
    pk = Peaks(tflops=1600.0, hbm_gbs=6400.0, nvlink_gbs=800.0, label="of test")
    one = layer_rooflines(8192, 2048, 1408, 6, 1, pk)
    eight = layer_rooflines(8192, 2048, 1408, 6, 8, pk)
    a1, a8 = one["dispatch (+) GEMM-A SwiGLU (fused)"], eight["dispatch (+) GEMM-A SwiGLU (fused)"]
    pairs = 8192 * 6
    assert a1.flops == 2.0 * pairs * 2048 * 2 * 1408 and a1.nvlink_bytes == 0 and a1.bound == "tensor cores"
    assert a8.nvlink_bytes == pairs * 7 / 8 * 2048 * 2                       # 7 of 8 rows leave the rank
    assert abs(a8.nvlink_us - a8.nvlink_bytes / 800e3) < 1e-9 and a8.roofline_us == a8.gemm_us
    y8 = eight["GEMM-Y (+ combine when remote)"]
    assert y8.bound == "NVLink" and y8.roofline_us == y8.nvlink_us           # half the FLOPs, same bytes on the wire
    total = sum(v.flops for v in one.values())
    assert total == step_flops(8192, 2048, 1408, 6)                          # 18 FLOPs per (pair, hidden, ffn) element
    assert step_flops(8192, 2048, 1408, 6, recompute=True) == total / 18 * 22
