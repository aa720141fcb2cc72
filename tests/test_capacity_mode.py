"""Capacity mode of the fused layer: fixed receive regions, live sizes read on the device, no host read per
forward.  Checked against the fp32 eager oracle like the exact-size mode (tests/test_layer_local.py), plus what
is specific to it: region reuse over several steps and layers, the two alternating gradient / landing regions,
the overflow fallback (every rank runs the dispatch as an empty one and the host hears about it one step late),
and the fall-back to exact sizing for shapes the regions were not built for.
"""
from types import SimpleNamespace

import pytest
import torch

from test_layer_local import _check, _make
from streamep_b200.errors import StreamEPError, StreamEPOverflow
from streamep_b200.models.reference import check_close

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("level", [0, 1, 2])
def test_capacity_mode_ep1_autograd(native, level):
    from streamep_b200 import LocalWorld
    from streamep_b200.stream_moe import make_streams, stream_moe_func
    T, H, I, E, K = 700, 256, 192, 8, 4
    w1, w2, xs, idxs, ws, dys = _make(1, T, H, I, E, K, seed=11, sentinel_p=0.05)
    world = LocalWorld(1, arena_bytes=256 << 20)
    buf = world.buffers[0]
    buf.enable_capacity_mode(T, H, K, E, capacity_factor=1.3)
    assert buf.capacity_mode
    streams = make_streams()
    x = xs[0].clone().requires_grad_(True)
    w = ws[0].clone().requires_grad_(True)
    w1p, w2p = w1.clone().requires_grad_(True), w2.clone().requires_grad_(True)
    base = buf.runtime.arena_bytes_in_use()
    for it in range(3):     # the third step is back on the first gradient / landing region
        for t in (x, w, w1p, w2p):
            t.grad = None
        out = stream_moe_func(buf, x, idxs[0], w, None, w1p, w2p, streams=streams, num_experts=E,
                              activation_checkpoint_level=level, fused=True)
        out.backward(dys[0])
        torch.cuda.synchronize()
        buf.check_status()
        acc = [None, None]
        _check(0, out, (x.grad, w.grad, None, None), xs[0], idxs[0], ws[0], dys[0], w1, w2, E, acc)
        check_close("dW1", w1p.grad, acc[0], atol=3e-2 * float(acc[0].abs().max()), rtol=3e-2)
        check_close("dW2", w2p.grad, acc[1], atol=3e-2 * float(acc[1].abs().max()), rtol=3e-2)
        del out
    assert buf.runtime.arena_bytes_in_use() == base, "capacity mode must not allocate arena blocks per step"
    assert buf.overflow_info()["count"] == 0


@pytest.mark.parametrize("R,level,routing,tokens", [
    (2, 0, "uniform", 300),
    (4, 1, "uniform", [260, 17, 0, 400]),        # uneven, one rank without tokens
    (4, 2, "first_k", 200),                      # all pairs to rank 0: needs a generous capacity factor
    (8, 0, "uniform", 130),
    (4, 0, "power_law", [300, 40, 512, 129]),
])
def test_capacity_mode_emulated_ranks(native, R, level, routing, tokens):
    from streamep_b200 import LocalWorld
    from streamep_b200.stream_moe import _resolve_tile_config, moe_backward, moe_forward
    H, I, E, K = 256, 128, 16, 4
    EL = E // R
    w1, w2, xs, idxs, ws, dys = _make(R, tokens, H, I, E, K, seed=12, sentinel_p=0.03, routing=routing)
    world = LocalWorld(R, arena_bytes=192 << 20)
    t_max = max(tokens) if isinstance(tokens, (list, tuple)) else tokens
    world.enable_capacity_mode(t_max, H, K, E, capacity_factor=float(R) if routing in ("first_k", "power_law") else 1.6)
    streams = world.make_streams()
    cfg = _resolve_tile_config(None, I, H)

    def rank_fn(r, buf):
        ctx = SimpleNamespace()
        w1l, w2l = w1[r * EL:(r + 1) * EL].contiguous(), w2[r * EL:(r + 1) * EL].contiguous()
        out = moe_forward(ctx, streams, buf, xs[r], idxs[r], ws[r], None, w1l, w2l, E, cfg, level, True)
        assert ctx.handle._dispatch_out.region_id == 0
        grads = moe_backward(ctx, dys[r])
        return out, grads

    for it in range(3):
        res = world.run(rank_fn)
        torch.cuda.synchronize()
        world.check_status()
        acc = [None, None]
        for r in range(R):
            out, grads = res[r]
            if xs[r].shape[0] == 0:
                continue
            _check(r, out, grads, xs[r], idxs[r], ws[r], dys[r], w1, w2, EL, acc)
        got_dw1 = torch.cat([res[r][1][2] for r in range(R)])
        got_dw2 = torch.cat([res[r][1][3] for r in range(R)])
        check_close("dW1", got_dw1, acc[0], atol=3e-2 * float(acc[0].abs().max()), rtol=3e-2)
        check_close("dW2", got_dw2, acc[1], atol=3e-2 * float(acc[1].abs().max()), rtol=3e-2)
        del res


def test_capacity_mode_layer_stack_uses_one_region_per_live_layer(native):
    from streamep_b200 import LocalWorld
    from streamep_b200.stream_moe import make_streams, stream_moe_func
    T, H, I, E, K, L = 400, 256, 128, 8, 2, 3
    w1, w2, xs, idxs, ws, dys = _make(1, T, H, I, E, K, seed=13, sentinel_p=0.02)
    g = torch.Generator(device="cpu").manual_seed(14)
    w1s = [(torch.randn(E, 2 * I, H, generator=g) * 0.08).to(torch.bfloat16).to(DEV).requires_grad_(True) for _ in range(L)]
    w2s = [(torch.randn(E, H, I, generator=g) * 0.08).to(torch.bfloat16).to(DEV).requires_grad_(True) for _ in range(L)]
    ref = LocalWorld(1, arena_bytes=256 << 20).buffers[0]          # exact-size mode, same layers: the yardstick
    buf = LocalWorld(1, arena_bytes=256 << 20).buffers[0]
    buf.enable_capacity_mode(T, H, K, E, capacity_factor=1.5, layers_in_flight=L)
    streams = make_streams()

    def run(b):
        x = xs[0].clone().requires_grad_(True)
        cur = x
        for l in range(L):
            cur = stream_moe_func(b, cur, idxs[0], ws[0], None, w1s[l], w2s[l], streams=streams, num_experts=E,
                                  activation_checkpoint_level=l % 3)
        cur.backward(dys[0])
        torch.cuda.synchronize()
        b.check_status()
        grads = [w.grad.float().clone() for w in w1s + w2s]
        for w in w1s + w2s:
            w.grad = None
        return cur.detach().float(), x.grad.float(), grads

    want = run(ref)
    for step in range(3):
        got = run(buf)
        check_close("out", got[0], want[0], atol=2e-2 * float(want[0].abs().max()), rtol=2e-2)
        check_close("dx", got[1], want[1], atol=2e-2 * float(want[1].abs().max()), rtol=2e-2)
        for a, b in zip(got[2], want[2]):
            check_close("dW", a, b, atol=3e-2 * float(b.abs().max()), rtol=3e-2)
    # one more live layer than regions: refused on the host, before anything is launched
    small = LocalWorld(1, arena_bytes=256 << 20).buffers[0]
    small.enable_capacity_mode(T, H, K, E, capacity_factor=1.5, layers_in_flight=1)
    x = xs[0].clone().requires_grad_(True)
    h1 = stream_moe_func(small, x, idxs[0], ws[0], None, w1s[0], w2s[0], streams=streams, num_experts=E)
    with pytest.raises((ValueError, StreamEPError), match="region"):
        stream_moe_func(small, h1, idxs[0], ws[0], None, w1s[1], w2s[1], streams=streams, num_experts=E)
    torch.cuda.synchronize()


def test_capacity_overflow_runs_empty_and_is_reported_one_step_late(native):
    from streamep_b200 import LocalWorld
    from streamep_b200.stream_moe import _resolve_tile_config, moe_backward, moe_forward
    R, H, I, E, K, T = 2, 256, 128, 8, 4, 256
    EL = E // R
    # every pair goes to rank 0's experts: rank 0 needs 2 x T x K rows, the capacity is 1.2 x T x K
    w1, w2, xs, idxs, ws, dys = _make(R, T, H, I, E, K, seed=15, routing="first_k")
    fit = _make(R, T, H, I, E, K, seed=16, routing="uniform")
    world = LocalWorld(R, arena_bytes=128 << 20)
    world.enable_capacity_mode(T, H, K, E, capacity_factor=1.2)
    streams = world.make_streams()
    cfg = _resolve_tile_config(None, I, H)

    def make_fn(data):
        _, _, x_, i_, w_, d_ = data

        def rank_fn(r, buf):
            ctx = SimpleNamespace()
            w1l, w2l = w1[r * EL:(r + 1) * EL].contiguous(), w2[r * EL:(r + 1) * EL].contiguous()
            out = moe_forward(ctx, streams, buf, x_[r], i_[r], w_[r], None, w1l, w2l, E, cfg, 0, True)
            return out, moe_backward(ctx, d_[r])
        return rank_fn

    res = world.run(make_fn((w1, w2, xs, idxs, ws, dys)))
    # nothing has synchronised so far; the host can already see the record without a sync once the kernel ran
    torch.cuda.synchronize()
    info = world.buffers[0].overflow_info()
    assert info["count"] == 1 and info["needed_tiles"] * 128 >= 2 * T * K
    for r in range(R):
        out, (dx, dtw, dw1, dw2) = res[r]
        assert float(out.float().abs().max()) == 0.0 and float(dx.float().abs().max()) == 0.0
        assert float(dw1.float().abs().max()) == 0.0 and float(dw2.float().abs().max()) == 0.0
        assert float(dtw.abs().max()) == 0.0
    with pytest.raises(StreamEPOverflow, match="capacity overflow"):
        world.check_status()
    # the buffer stays usable: a dispatch that fits runs normally afterwards
    res = world.run(make_fn(fit))
    torch.cuda.synchronize()
    world.check_status()
    acc = [None, None]
    for r in range(R):
        _check(r, res[r][0], res[r][1], fit[2][r], fit[3][r], fit[4][r], fit[5][r], w1, w2, EL, acc)


def test_other_shapes_fall_back_to_exact_sizing(native):
    from streamep_b200 import LocalWorld
    from streamep_b200.stream_moe import make_streams, stream_moe_func
    T, H, I, E, K = 300, 256, 128, 8, 2
    w1, w2, xs, idxs, ws, dys = _make(1, 2 * T, H, I, E, K, seed=17)
    buf = LocalWorld(1, arena_bytes=256 << 20).buffers[0]
    buf.enable_capacity_mode(T, H, K, E)        # built for T tokens; the call below brings 2 T
    x = xs[0].clone().requires_grad_(True)
    w1p, w2p = w1.clone().requires_grad_(True), w2.clone().requires_grad_(True)
    out = stream_moe_func(buf, x, idxs[0], ws[0], None, w1p, w2p, streams=make_streams(), num_experts=E)
    out.backward(dys[0])
    torch.cuda.synchronize()
    buf.check_status()
    from streamep_b200.models.reference import moe_reference_grads
    want_out, want_dx, _, _, _ = moe_reference_grads(xs[0], idxs[0], ws[0], w1, w2, dys[0])
    check_close("out", out, want_out, atol=2e-2 * float(want_out.abs().max()), rtol=2e-2)
    check_close("dx", x.grad, want_dx, atol=2e-2 * float(want_dx.abs().max()), rtol=2e-2)
