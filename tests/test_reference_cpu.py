"""CPU checks of the pure-PyTorch oracles and of the constructed baseline layer (gloo, 2 ranks).

Includes the repository's CPU reference configuration: world_size 2, fp32, 256 tokens per rank,
hidden 512, 8 experts (4 per rank), top-2, SwiGLU ffn 1024, x ~ N(0,1), router / w1 / w2 ~
N(0, 0.02), renormalised softmax top-k weights, seed 0.
"""
import os
import sys
import time

import pytest
import torch
import torch.multiprocessing as mp

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from streamep_b200.models.reference import (check_close, dispatch_layout_reference, dswiglu_reference,  # noqa: E402
                                            is_token_in_rank_reference, kernel_a_reference,
                                            moe_reference_forward, moe_reference_grads, pool_reference,
                                            router_reference, swiglu_interleaved)


def _naive_moe(x, idx, w, w1, w2):
    out = torch.zeros(x.shape[0], x.shape[1])
    for t in range(x.shape[0]):
        for k in range(idx.shape[1]):
            e = int(idx[t, k])
            if e < 0:
                continue
            h = w1[e] @ x[t]
            a = torch.nn.functional.silu(h[0::2]) * h[1::2]
            out[t] += w[t, k] * (w2[e] @ a)
    return out


def test_oracle_matches_naive_loop():
    g = torch.Generator().manual_seed(0)
    T, H, I, E, K = 37, 16, 24, 6, 3
    x = torch.randn(T, H, generator=g)
    w1 = torch.randn(E, 2 * I, H, generator=g) * 0.3
    w2 = torch.randn(E, H, I, generator=g) * 0.3
    idx = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)])
    idx[3, 1] = -1
    w = torch.rand(T, K, generator=g)
    got = moe_reference_forward(x, idx, w, w1, w2)
    assert torch.allclose(got, _naive_moe(x, idx, w, w1, w2), atol=1e-5)


def test_oracle_grads_match_finite_differences():
    g = torch.Generator().manual_seed(1)
    T, H, I, E, K = 5, 8, 6, 4, 2
    x = torch.randn(T, H, generator=g, dtype=torch.float64)
    w1 = torch.randn(E, 2 * I, H, generator=g, dtype=torch.float64) * 0.3
    w2 = torch.randn(E, H, I, generator=g, dtype=torch.float64) * 0.3
    idx = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)])
    w = torch.rand(T, K, generator=g, dtype=torch.float64)

    def f(x_, w_, w1_, w2_):
        out = torch.zeros(T, H, dtype=torch.float64)
        for e in range(E):
            sel = (idx == e).nonzero()
            if sel.numel() == 0:
                continue
            t_e, k_e = sel[:, 0], sel[:, 1]
            h = x_[t_e] @ w1_[e].t()
            out = out.index_add(0, t_e, w_[t_e, k_e][:, None] * (swiglu_interleaved(h) @ w2_[e].t()))
        return out
    assert torch.autograd.gradcheck(f, (x.requires_grad_(), w.requires_grad_(), w1.requires_grad_(), w2.requires_grad_()),
                                    atol=1e-6)


def test_dswiglu_reference_is_the_gradient_of_swiglu():
    g = torch.Generator().manual_seed(2)
    gate = torch.randn(7, 5, generator=g, dtype=torch.float64, requires_grad=True)
    up = torch.randn(7, 5, generator=g, dtype=torch.float64, requires_grad=True)
    up_g = torch.randn(7, 5, generator=g, dtype=torch.float64)
    post = torch.nn.functional.silu(gate) * up
    dg, du = torch.autograd.grad(post, (gate, up), up_g)
    rg, ru, rp = dswiglu_reference(gate.detach(), up.detach(), up_g)
    assert torch.allclose(rg, dg) and torch.allclose(ru, du) and torch.allclose(rp, post.detach())


def test_router_reference_properties():
    g = torch.Generator().manual_seed(3)
    x = torch.randn(50, 32, generator=g)
    wg = torch.randn(16, 32, generator=g)
    idx, w = router_reference(x, wg, 4)
    assert idx.shape == (50, 4) and w.dtype == torch.float32
    assert torch.allclose(w.sum(-1), torch.ones(50), atol=1e-6)
    assert (idx.sort(-1).values[:, 1:] != idx.sort(-1).values[:, :-1]).all()      # distinct experts
    in_rank = is_token_in_rank_reference(idx, 16, 4)
    assert in_rank.shape == (50, 4) and (in_rank.sum(-1) >= 1).all()


@pytest.mark.parametrize("R,C,T,K,E", [(1, 4, 50, 2, 4), (2, 3, 77, 3, 8), (4, 5, [10, 0, 33, 64], 4, 16)])
def test_layout_reference_invariants(R, C, T, K, E):
    """Properties the reference's dispatch tests assert (tests/test_dispatch.py:95-233)."""
    g = torch.Generator().manual_seed(4)
    Ts = T if isinstance(T, list) else [T] * R
    idxs = []
    for r in range(R):
        idx = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(Ts[r])]) if Ts[r] else torch.zeros(0, K, dtype=torch.int64)
        if Ts[r]:
            idx[torch.rand(Ts[r], K, generator=g) < 0.1] = -1
        idxs.append(idx)
    xs = [torch.randn(Ts[r], 8, generator=g) for r in range(R)]
    layouts, sends = dispatch_layout_reference(idxs, E, C, 128)
    EL = E // R
    total_pairs = sum(int((i >= 0).sum()) for i in idxs)
    assert sum(int(L.expert_frequency.sum()) for L in layouts) == total_pairs
    for d, L in enumerate(layouts):
        valid = (L.pool_recv_token >= 0).nonzero().flatten()
        assert valid.numel() == int(L.expert_frequency.sum())
        for el in range(EL):        # every slot inside its expert block, valid rows form a prefix
            lo = int(L.expert_pool_block_offset[el]) * 128
            f = int(L.expert_frequency[el])
            assert (L.pool_recv_token[lo:lo + f] >= 0).all()
            hi = int(L.expert_pool_block_offset[el + 1]) * 128
            assert (L.pool_recv_token[lo + f:hi] == -1).all()
        # (r, k) -> slot is the inverse of slot -> (r, k)
        for slot in valid.tolist():
            assert int(L.recv_token_to_slots[int(L.pool_recv_token[slot]), int(L.pool_k_slot[slot])]) == slot
        assert int(L.k_local_total.sum()) == valid.numel()
        assert int(L.seen_per_substream.sum()) == valid.numel()
        assert int(L.pool_arrival_target.sum()) == valid.numel()
        # recv-token ids are source-rank-major, then source token order
        order = torch.stack([L.recv_src_rank, L.recv_src_token], 1).tolist()
        assert order == sorted(order)
        pool = pool_reference(L, xs)
        for slot in valid.tolist()[:20]:
            assert torch.equal(pool[slot], xs[int(L.pool_src_rank[slot])][int(L.pool_src_token[slot])])
    for s, S in enumerate(sends):
        assert ((S.pair_slot >= 0) == (idxs[s] >= 0)).all()
        assert ((S.send_recv_token >= 0) == is_token_in_rank_reference(idxs[s], E, R)).all() if Ts[s] else True


def test_kernel_a_reference_shapes():
    pool = torch.randn(256, 16)
    w1 = torch.randn(2, 24, 16)
    pre, post = kernel_a_reference(pool, w1, torch.tensor([1, 0]), 128)
    assert pre.shape == (256, 24) and post.shape == (256, 12)
    assert torch.allclose(pre[:128], pool[:128] @ w1[1].t(), atol=1e-5)


def test_check_close_dual_threshold():
    want = torch.tensor([1.0, 100.0, 0.0])
    check_close("ok", torch.tensor([1.0005, 100.5, 0.0005]), want, atol=1e-3, rtol=1e-2)
    with pytest.raises(AssertionError):
        check_close("bad", torch.tensor([1.5, 100.0, 0.0]), want, atol=1e-3, rtol=1e-2)
    with pytest.raises(AssertionError):
        check_close("nan", torch.tensor([float("nan"), 100.0, 0.0]), want, atol=1e-3, rtol=1e-2)


# ------------------------------------------------------------------ gloo, world_size 2
def _gloo_worker(rank, world, port, result_q):
    import torch.distributed as dist
    from streamep_b200.parallel.nccl_baseline import baseline_moe_forward
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        T, H, E, K, I = 256, 512, 8, 2, 1024
        g = torch.Generator().manual_seed(0)
        w_gate = torch.randn(E, H, generator=g) * 0.02
        w1 = torch.randn(E, 2 * I, H, generator=g) * 0.02
        w2 = torch.randn(E, H, I, generator=g) * 0.02
        xs = [torch.randn(T, H, generator=g) for _ in range(world)]
        dys = [torch.randn(T, H, generator=g) for _ in range(world)]
        EL = E // world
        x = xs[rank].clone().requires_grad_(True)
        idx, w = router_reference(x.detach(), w_gate, K)
        w = w.clone().requires_grad_(True)
        w1l = w1[rank * EL:(rank + 1) * EL].clone().requires_grad_(True)
        w2l = w2[rank * EL:(rank + 1) * EL].clone().requires_grad_(True)
        t0 = time.perf_counter()
        out = baseline_moe_forward(x, idx, w, w1l, w2l, E, dist.group.WORLD)
        out.backward(dys[rank])
        dt = time.perf_counter() - t0
        # global oracle
        X = torch.cat(xs)
        IDX, W = router_reference(X, w_gate, K)
        want_out, want_dx, want_dw, want_dw1, want_dw2 = moe_reference_grads(X, IDX, W, w1, w2, torch.cat(dys))
        sl = slice(rank * T, (rank + 1) * T)
        check_close("out", out, want_out[sl], 1e-5, 1e-4)
        check_close("dx", x.grad, want_dx[sl], 1e-5, 1e-4)
        check_close("dw", w.grad, want_dw[sl], 1e-5, 1e-4)
        check_close("dW1", w1l.grad, want_dw1[rank * EL:(rank + 1) * EL], 1e-4, 1e-4)
        check_close("dW2", w2l.grad, want_dw2[rank * EL:(rank + 1) * EL], 1e-4, 1e-4)
        result_q.put((rank, "ok", T / dt))
    except Exception as e:  # noqa: BLE001
        result_q.put((rank, f"{type(e).__name__}: {e}", 0.0))
    finally:
        dist.destroy_process_group()


def test_gloo_world2_reference_layer_fwd_bwd():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29650 + os.getpid() % 200
    procs = [ctx.Process(target=_gloo_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert all(r[1] == "ok" for r in results), results


@pytest.mark.parametrize("R,tokens,K,E,C,sentinel", [(1, [300], 4, 8, 5, 0.05), (2, [257, 100], 4, 8, 7, 0.1),
                                                     (4, [260, 17, 0, 400], 6, 64, 10, 0.03), (8, [50] * 8, 13, 384, 40, 0.0)])
def test_vectorised_layout_oracle_equals_the_loop_oracle(R, tokens, K, E, C, sentinel):
    """The production-scale metadata check runs against layout_fast; here it is pinned, field by field, to the
    loop oracle that states the placement rule."""
    import dataclasses
    from helpers import make_routing
    from streamep_b200.models.layout_fast import dispatch_layout_fast
    from streamep_b200.models.reference import dispatch_layout_reference
    idxs, ws = [], []
    for r, T in enumerate(tokens):
        i, w = make_routing(T, K, E, 7 * r + 1, "cpu", sentinel_p=sentinel)
        idxs.append(i); ws.append(w)
    a = dispatch_layout_reference(idxs, E, C, 128, ws)
    b = dispatch_layout_fast(idxs, E, C, 128, ws)
    for la, lb in zip(a[0] + a[1], b[0] + b[1]):
        for f in dataclasses.fields(la):
            x, y = getattr(la, f.name), getattr(lb, f.name)
            if isinstance(x, torch.Tensor):
                assert torch.equal(x, y.to(x.dtype)), f.name
            else:
                assert x == y, f.name
