"""Full layer forward + backward against the fp32 eager oracle, on one GPU.

EP = 1 runs the production path (one fused launch per stage, real autograd); EP = 2 / 4 run the
same kernels with the ranks emulated in threads.  Mirrors the reference's end-to-end validator
(stream_ep/stream_moe/validate_multi_iter.py) and tests/test_activation_checkpoint.py,
tests/test_skewed_experts.py, tests/test_uneven_tokens_per_rank.py.
"""
import gc
from types import SimpleNamespace

import pytest
import torch

from helpers import make_routing
from streamep_b200.models.reference import check_close, moe_reference_grads

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _make(R, tokens, H, I, E, K, seed, sentinel_p=0.0, routing="uniform"):
    g = torch.Generator(device="cpu").manual_seed(seed)
    w1 = (torch.randn(E, 2 * I, H, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    w2 = (torch.randn(E, H, I, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    xs, idxs, ws, dys = [], [], [], []
    for r in range(R):
        T = tokens[r] if isinstance(tokens, (list, tuple)) else tokens
        xs.append(torch.randn(T, H, generator=g).to(torch.bfloat16).to(DEV))
        idx, w = make_routing(T, K, E, seed * 31 + r, DEV, sentinel_p=sentinel_p)
        if routing == "first_k":
            idx = torch.arange(K, device=DEV).expand(T, K).contiguous()
        elif routing == "half_empty":
            idx = torch.where(idx >= 0, idx % (E // 2), idx)
            idx = torch.where(idx >= 0, idx * 2, idx)      # only even experts; duplicates within a token allowed
        elif routing == "uniform_rotating":
            idx = ((torch.arange(T, device=DEV)[:, None] * K + torch.arange(K, device=DEV)[None, :] + r) % E).contiguous()
        elif routing == "per_rank_imbalance":              # 90 % of the tokens send every pair to rank 0's experts
            hot = torch.rand(T, generator=g) < 0.9
            hot_idx = torch.stack([torch.randperm(E // R, generator=g)[:K] for _ in range(T)]) if T else idx.cpu()
            idx = torch.where(hot[:, None].to(DEV), hot_idx.to(DEV), idx)
        elif routing == "power_law":                       # Zipf(1.2) over expert ids, distinct per token
            prob = torch.arange(1, E + 1, dtype=torch.float64).pow(-1.2)
            idx = torch.multinomial((prob / prob.sum()).expand(max(T, 1), E), K, replacement=False, generator=g)[:T].to(DEV)
        w = w / w.sum(-1, keepdim=True)
        idxs.append(idx); ws.append(w)
        dys.append(torch.randn(T, H, generator=g).to(torch.bfloat16).to(DEV))
    return w1, w2, xs, idxs, ws, dys


def _check(r, out, grads, x, idx, w, dy, w1, w2, EL, dw_want_acc):
    want_out, want_dx, want_dw, want_dw1, want_dw2 = moe_reference_grads(x, idx, w, w1, w2, dy)
    s = lambda t: max(float(t.abs().max()), 1e-6)   # noqa: E731
    check_close(f"rank {r} out", out, want_out, atol=2e-2 * s(want_out), rtol=2e-2)
    dx, dtw, _, _ = grads
    check_close(f"rank {r} dL_dx", dx, want_dx, atol=2e-2 * s(want_dx), rtol=2e-2)
    check_close(f"rank {r} dL_dtopk_weights", dtw, want_dw, atol=2e-2 * s(want_dw), rtol=2e-2)
    dw_want_acc[0] = dw_want_acc[0] + want_dw1 if dw_want_acc[0] is not None else want_dw1
    dw_want_acc[1] = dw_want_acc[1] + want_dw2 if dw_want_acc[1] is not None else want_dw2


@pytest.mark.parametrize("fused", [True, False])
@pytest.mark.parametrize("level", [0, 1, 2])
def test_layer_ep1_autograd(native, fused, level):
    from streamep_b200 import LocalWorld
    from streamep_b200.stream_moe import make_streams, stream_moe_func
    T, H, I, E, K = 700, 256, 192, 8, 4
    w1, w2, xs, idxs, ws, dys = _make(1, T, H, I, E, K, seed=1, sentinel_p=0.05)
    world = LocalWorld(1, arena_bytes=256 << 20)
    buf = world.buffers[0]
    streams = make_streams()
    x = xs[0].clone().requires_grad_(True)
    w = ws[0].clone().requires_grad_(True)
    w1p, w2p = w1.clone().requires_grad_(True), w2.clone().requires_grad_(True)
    for it in range(2):     # second iteration reuses the arena and the counters
        for t in (x, w, w1p, w2p):
            t.grad = None
        out = stream_moe_func(buf, x, idxs[0], w, None, w1p, w2p, streams=streams, num_experts=E,
                              activation_checkpoint_level=level, fused=fused)
        out.backward(dys[0])
        torch.cuda.synchronize()
        buf.check_status()
        acc = [None, None]
        _check(0, out, (x.grad, w.grad, None, None), xs[0], idxs[0], ws[0], dys[0], w1, w2, E, acc)
        check_close("dW1", w1p.grad, acc[0], atol=3e-2 * float(acc[0].abs().max()), rtol=3e-2)
        check_close("dW2", w2p.grad, acc[1], atol=3e-2 * float(acc[1].abs().max()), rtol=3e-2)


@pytest.mark.parametrize("R,fused,level,routing,tokens", [
    (2, True, 0, "uniform", 300),
    (2, False, 0, "uniform", 300),
    (4, True, 1, "uniform", [260, 17, 0, 400]),      # uneven, one rank without tokens
    (4, False, 2, "uniform", 256),
    (4, True, 2, "first_k", 200),                    # all pairs to rank 0: three ranks compute nothing
    (4, True, 0, "half_empty", 300),
    (8, True, 0, "uniform", 130),
    (4, True, 0, "uniform_rotating", 256),
    (4, True, 1, "per_rank_imbalance", 300),
    (4, False, 0, "per_rank_imbalance", 300),
    (4, True, 0, "power_law", [300, 40, 512, 129]),
])
def test_layer_emulated_ranks(native, R, fused, level, routing, tokens):
    from streamep_b200 import LocalWorld
    from streamep_b200.stream_moe import _resolve_tile_config, moe_backward, moe_forward
    H, I, E, K = 256, 128, 16, 4
    EL = E // R
    w1, w2, xs, idxs, ws, dys = _make(R, tokens, H, I, E, K, seed=2, sentinel_p=0.03, routing=routing)
    world = LocalWorld(R, arena_bytes=128 << 20)
    streams = world.make_streams()
    cfg = _resolve_tile_config(None, I, H)

    def rank_fn(r, buf):
        ctx = SimpleNamespace()
        w1l, w2l = w1[r * EL:(r + 1) * EL].contiguous(), w2[r * EL:(r + 1) * EL].contiguous()
        out = moe_forward(ctx, streams, buf, xs[r], idxs[r], ws[r], None, w1l, w2l, E, cfg, level, fused)
        grads = moe_backward(ctx, dys[r])
        return out, grads

    for it in range(2):
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


@pytest.mark.parametrize("R", [1, 4])
def test_layer_on_the_vmm_allocator(native, R):
    """The arena taken from the virtual-memory-management API (cuMemCreate / cuMemMap / cuMemSetAccess) instead of
    cudaMalloc: same layer, same checks, plus a capacity-mode region on it."""
    from streamep_b200 import LocalWorld
    from streamep_b200.stream_moe import _resolve_tile_config, moe_backward, moe_forward
    H, I, E, K, T = 256, 128, 16, 4, 300
    EL = E // R
    w1, w2, xs, idxs, ws, dys = _make(R, T, H, I, E, K, seed=9, sentinel_p=0.03)
    world = LocalWorld(R, arena_bytes=128 << 20, allocator="vmm")
    assert all(b.runtime.uses_vmm() for b in world.buffers)
    streams = world.make_streams()
    cfg = _resolve_tile_config(None, I, H)
    for capacity in (False, True):
        if capacity:
            world.enable_capacity_mode(T, H, K, E, capacity_factor=1.6)

        def rank_fn(r, buf):
            ctx = SimpleNamespace()
            w1l, w2l = w1[r * EL:(r + 1) * EL].contiguous(), w2[r * EL:(r + 1) * EL].contiguous()
            out = moe_forward(ctx, streams, buf, xs[r], idxs[r], ws[r], None, w1l, w2l, E, cfg, 0, True)
            return out, moe_backward(ctx, dys[r])
        res = world.run(rank_fn)
        torch.cuda.synchronize()
        world.check_status()
        acc = [None, None]
        for r in range(R):
            _check(r, res[r][0], res[r][1], xs[r], idxs[r], ws[r], dys[r], w1, w2, EL, acc)
        del res


def test_layer_stack_depth_and_arena_reuse(native):
    """Several layers back to back for several steps on one buffer (the reference's
    tests/test_pipeline_depth_stress.py without the fault injection): every layer's forward state
    stays alive until its backward, results repeat from step to step, and the symmetric arena is
    back to its starting level after each step."""
    from streamep_b200 import LocalWorld
    from streamep_b200.stream_moe import make_streams, stream_moe_func
    T, H, I, E, K, L = 400, 256, 128, 8, 2, 6
    w1, w2, xs, idxs, ws, dys = _make(1, T, H, I, E, K, seed=5, sentinel_p=0.02)
    g = torch.Generator(device="cpu").manual_seed(6)
    w1s = [(torch.randn(E, 2 * I, H, generator=g) * 0.08).to(torch.bfloat16).to(DEV).requires_grad_(True) for _ in range(L)]
    w2s = [(torch.randn(E, H, I, generator=g) * 0.08).to(torch.bfloat16).to(DEV).requires_grad_(True) for _ in range(L)]
    world = LocalWorld(1, arena_bytes=256 << 20)
    buf = world.buffers[0]
    streams = make_streams()
    base = buf.runtime.arena_bytes_in_use()
    outs, dxs = [], []
    for step in range(3):
        x = xs[0].clone().requires_grad_(True)
        cur = x
        for l in range(L):
            cur = stream_moe_func(buf, cur, idxs[0], ws[0], None, w1s[l], w2s[l], streams=streams, num_experts=E,
                                  activation_checkpoint_level=l % 3)
        cur.backward(dys[0])
        torch.cuda.synchronize()
        buf.check_status()
        assert torch.isfinite(cur.float()).all() and torch.isfinite(x.grad.float()).all()
        for w in w1s + w2s:
            assert w.grad is not None and torch.isfinite(w.grad.float()).all()
            w.grad = None
        outs.append(cur.detach().float()); dxs.append(x.grad.float())
        del cur, x
        gc.collect()
        assert buf.runtime.arena_bytes_in_use() == base, "a layer leaked symmetric memory"
    s = float(outs[0].abs().max())
    for o, d in zip(outs[1:], dxs[1:]):
        check_close("out repeats", o, outs[0], atol=2e-2 * s, rtol=2e-2)
        check_close("dx repeats", d, dxs[0], atol=2e-2 * float(dxs[0].abs().max()), rtol=2e-2)
