"""Dispatch / dispatch_grads / combine / combine_grads with several ranks emulated on one GPU.

The checks are the closed-form and bit-exact ones of the reference's multi-GPU scripts
(tests/test_dispatch.py:95-256, tests/test_multi_dispatch.py, tests/test_metadata.py:389-412,
tests/test_dispatch_grads.py, tests/test_combine.py:69-106, tests/test_combine_grads.py,
tests/test_uneven_tokens_per_rank.py), run against the CPU oracle of the pool layout.
"""
import pytest
import torch

from helpers import make_routing
from streamep_b200.models.reference import dispatch_layout_reference, pool_reference

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _world(R, arena_mb=192):
    from streamep_b200 import LocalWorld
    return LocalWorld(R, arena_bytes=arena_mb << 20, timeout_ms=1500)


def _inputs(R, tokens, H, K, E, seed, sentinel_p=0.0, empty_expert=None, kind="randn"):
    xs, idxs, ws = [], [], []
    for r in range(R):
        T = tokens[r] if isinstance(tokens, (list, tuple)) else tokens
        g = torch.Generator(device="cpu").manual_seed(seed * 100 + r)
        if kind == "rank_tag":
            x = torch.full((T, H), float(r + 1))
        else:
            x = torch.randn(T, H, generator=g)
        idx, w = make_routing(T, K, E, seed * 100 + r, DEV, sentinel_p=sentinel_p, empty_expert=empty_expert)
        xs.append(x.to(torch.bfloat16).to(DEV)); idxs.append(idx); ws.append(w)
    return xs, idxs, ws


def _check_dispatch(world, handles, xs, idxs, ws, E):
    R = world.num_ranks
    C = world.buffers[0].num_channels
    torch.cuda.synchronize()
    world.check_status()
    layouts, sends = dispatch_layout_reference([i.cpu() for i in idxs], E, C, 128, [w.cpu() for w in ws])
    for r in range(R):
        h, L, S = handles[r], layouts[r], sends[r]
        st = h._dispatch_out
        assert h.total_tiles == L.total_tiles and st.num_recv_tokens == L.num_recv_tokens
        for name in ("expert_frequency", "expert_pool_block_offset", "base_pool", "seen_per_substream",
                     "tile_id_to_expert", "pool_arrival_target", "pool_recv_token", "pool_k_slot",
                     "recv_token_to_slots", "k_local_total", "recv_channel_prefix_matrix"):
            assert torch.equal(getattr(h, name).cpu(), getattr(L, name)), f"rank {r}: {name}"
        assert torch.equal(h.rank_prefix_matrix.cpu()[:, r], L.rank_prefix_matrix[:, r])
        assert torch.equal(h.pool_arrival_count.cpu(), L.pool_arrival_target), f"rank {r}: arrival counts"
        assert torch.equal(h.k_local_remaining.cpu(), L.k_local_total)
        assert torch.equal(h.pool_src.cpu()[:, 0], L.pool_src_rank) and torch.equal(h.pool_src.cpu()[:, 1], L.pool_src_token)
        assert torch.equal(st.pair_slot.cpu(), S.pair_slot), f"rank {r}: pair_slot"
        assert torch.equal(st.send_recv_token.cpu(), S.send_recv_token)
        assert torch.equal(h.send_head.cpu(), S.send_head)
        assert torch.equal(h.channel_prefix_matrix.cpu(), S.channel_prefix_matrix)
        valid = L.pool_recv_token >= 0
        assert torch.equal(h.pool.cpu()[valid], pool_reference(L, xs)[valid]), f"rank {r}: pool rows"
        assert torch.equal(h.pool_topk_weight.cpu()[valid], L.pool_topk_weight[valid])
        assert (h.o == 0).all() and (h.y_done_per_token == 0).all()
        assert h.TK_padded == h.pool.shape[0] == L.total_tiles * 128
    return layouts, sends


@pytest.mark.parametrize("R,T,H,K,E", [(1, 300, 256, 4, 8), (2, 257, 256, 4, 8), (4, 512, 512, 6, 64), (8, 384, 256, 8, 256)])
def test_dispatch_layout_bit_exact(native, R, T, H, K, E):
    world = _world(R)
    xs, idxs, ws = _inputs(R, T, H, K, E, seed=1, sentinel_p=0.05, empty_expert=E - 1)
    handles = world.dispatch(xs, idxs, ws, E)
    _check_dispatch(world, handles, xs, idxs, ws, E)
    # determinism + no state leak: same inputs again, then different routing on the same buffers
    handles2 = world.dispatch(xs, idxs, ws, E)
    torch.cuda.synchronize()
    for a, b in zip(handles, handles2):
        assert torch.equal(a.pool_recv_token, b.pool_recv_token) and torch.equal(a.pool_k_slot, b.pool_k_slot)
        valid = a.pool_recv_token >= 0
        assert torch.equal(a.pool[valid], b.pool[valid])
    xs3, idxs3, ws3 = _inputs(R, T, H, K, E, seed=2)
    handles3 = world.dispatch(xs3, idxs3, ws3, E)
    _check_dispatch(world, handles3, xs3, idxs3, ws3, E)


def test_dispatch_uneven_and_empty_rank(native):
    R, H, K, E = 4, 256, 4, 16
    world = _world(R)
    xs, idxs, ws = _inputs(R, [16, 700, 0, 333], H, K, E, seed=3)
    handles = world.dispatch(xs, idxs, ws, E)
    _check_dispatch(world, handles, xs, idxs, ws, E)


def test_dispatch_all_to_first_expert(native):
    """Every pair goes to expert 0: one rank receives everything, the others get empty pools."""
    R, T, H, K, E = 4, 200, 256, 1, 8
    world = _world(R)
    xs, _, ws = _inputs(R, T, H, K, E, seed=4)
    idxs = [torch.zeros(T, K, dtype=torch.int64, device=DEV) for _ in range(R)]
    handles = world.dispatch(xs, idxs, ws, E)
    _check_dispatch(world, handles, xs, idxs, ws, E)
    assert handles[1].total_tiles == 0 and handles[1].pool.shape[0] == 0


@pytest.mark.parametrize("R", [2, 4])
def test_dispatch_grads_bit_exact(native, R):
    T, H, K, E = 300, 256, 4, 16
    world = _world(R)
    xs, idxs, ws = _inputs(R, T, H, K, E, seed=5, sentinel_p=0.05)
    handles = world.dispatch(xs, idxs, ws, E)
    layouts, _ = _check_dispatch(world, handles, xs, idxs, ws, E)
    g = torch.Generator(device="cpu").manual_seed(6)
    dys = [torch.randn(T, H, generator=g).to(torch.bfloat16).to(DEV) for _ in range(R)]
    for rep in range(2):   # second call re-fires fresh counters
        outs = world.dispatch_grads(handles, dys)
        torch.cuda.synchronize()
        world.check_status()
        for r in range(R):
            pool, cnt = outs[r]
            valid = layouts[r].pool_recv_token >= 0
            assert torch.equal(pool.cpu()[valid], pool_reference(layouts[r], dys)[valid])
            assert torch.equal(cnt.cpu(), layouts[r].pool_arrival_target)


@pytest.mark.parametrize("R", [1, 2, 4])
def test_combine_closed_form(native, R):
    """o[r] = (rank + 1) everywhere: token t gets sum over the ranks it was sent to."""
    T, H, K, E = 300, 256, 4, 16
    world = _world(R)
    xs, idxs, ws = _inputs(R, T, H, K, E, seed=7, sentinel_p=0.1)
    handles = world.dispatch(xs, idxs, ws, E)
    torch.cuda.synchronize()
    for seq_rep in range(2):
        seq = 10 + seq_rep
        for r, h in enumerate(handles):
            h.o.fill_(float(r + 1))
            h.y_done_per_token.fill_(seq)
        outs = world.combine([h.o for h in handles], handles, seqs=[seq] * R)
        torch.cuda.synchronize()
        world.check_status()
        for r in range(R):
            sent = handles[r]._dispatch_out.send_recv_token >= 0          # [T, R]
            want = (sent.float() * torch.arange(1, R + 1, device=DEV).float()).sum(-1)
            assert torch.equal(outs[r].float(), want[:, None].expand(T, H).contiguous()), f"rank {r}"


def test_combine_random_rows_fp32_reduce(native):
    R, T, H, K, E = 4, 200, 512, 4, 16
    world = _world(R)
    xs, idxs, ws = _inputs(R, T, H, K, E, seed=8)
    handles = world.dispatch(xs, idxs, ws, E)
    torch.cuda.synchronize()
    g = torch.Generator(device="cpu").manual_seed(9)
    os_ = []
    for h in handles:
        o = torch.randn(h.o.shape, generator=g).to(torch.bfloat16).to(DEV)   # NOT in the arena: staged copy path
        os_.append(o)
        h.y_done_per_token.fill_(h.dispatch_seq)
    outs = world.combine(os_, handles)
    torch.cuda.synchronize()
    world.check_status()
    for r in range(R):
        srt = handles[r]._dispatch_out.send_recv_token
        want = torch.zeros(T, H, device=DEV)
        for d in range(R):
            m = srt[:, d] >= 0
            want[m] += os_[d][srt[m, d].long()].float()
        assert torch.equal(outs[r], want.to(torch.bfloat16))


def test_combine_grads_closed_form(native):
    R, T, H, K, E = 4, 200, 256, 4, 16
    world = _world(R)
    xs, idxs, ws = _inputs(R, T, H, K, E, seed=10, sentinel_p=0.1)
    handles = world.dispatch(xs, idxs, ws, E)
    torch.cuda.synchronize()
    dxs, wgs, dones = [], [], []
    for r, h in enumerate(handles):
        dxs.append(torch.full((h.num_recv_tokens, H), float(r + 1), dtype=torch.bfloat16, device=DEV))
        wgs.append(torch.full((h.TK_padded,), float(r + 1), dtype=torch.float32, device=DEV))
        dones.append(torch.full((h.num_recv_tokens,), h.dispatch_seq, dtype=torch.int64, device=DEV))
    outs = world.combine_grads(dxs, handles, wgs, dones)
    torch.cuda.synchronize()
    world.check_status()
    EL = E // R
    for r in range(R):
        dx, dw = outs[r]
        sent = handles[r]._dispatch_out.send_recv_token >= 0
        want = (sent.float() * torch.arange(1, R + 1, device=DEV).float()).sum(-1)
        assert torch.equal(dx.float(), want[:, None].expand(T, H).contiguous())
        want_w = torch.where(idxs[r] >= 0, (idxs[r] // EL + 1).float(), torch.zeros_like(ws[r]))
        assert torch.equal(dw, want_w)


def test_combine_gate_timeout_is_reported(native):
    """A stamp that never arrives: combine gives up within its budget and reports it."""
    from streamep_b200 import StreamEPTimeout
    R, T, H, K, E = 2, 64, 256, 2, 4
    world = _world(R)
    for b in world.buffers:
        b.set_timeout_ms(200)
    xs, idxs, ws = _inputs(R, T, H, K, E, seed=11)
    handles = world.dispatch(xs, idxs, ws, E)
    torch.cuda.synchronize()
    world.combine([h.o for h in handles], handles)     # y_done stays 0 < seq
    with pytest.raises(StreamEPTimeout, match="token gate timeout"):
        world.check_status()
    # the buffers still work afterwards
    for h in handles:
        h.y_done_per_token.fill_(h.dispatch_seq)
    world.combine([h.o for h in handles], handles)
    torch.cuda.synchronize()
    world.check_status()


def test_event_handle_and_stream_handles(native):
    """``EventHandle`` behaves like a ``torch.cuda.Event`` for ``Stream.wait_event`` and the buffer
    keeps the stream handles that the layer registers (csrc/event.hpp:9-35, csrc/stream_ep.cpp:387-456)."""
    from streamep_b200 import EventHandle
    world = _world(1)
    buf = world.buffers[0]
    side = torch.cuda.Stream()
    a = torch.zeros(1 << 20, device=DEV)
    a.add_(1.0)
    ev = EventHandle()                       # recorded on the current stream, after the add
    side.wait_event(ev)                      # duck-typed: calls ev.wait(side)
    with torch.cuda.stream(side):
        b = a * 2
    side.synchronize()
    assert float(b.sum()) == 2.0 * (1 << 20)
    buf.set_compute_stream_handle(side)
    buf.set_default_stream_handle(torch.cuda.current_stream())
    assert buf._raw(None) == side.cuda_stream
    buf.set_compute_stream_handle(None)
    assert buf._raw(None) == torch.cuda.current_stream().cuda_stream


def test_handle_stats(native):
    R, T, H, K, E = 2, 200, 256, 4, 8
    world = _world(R)
    xs, idxs, ws = _inputs(R, T, H, K, E, seed=21, sentinel_p=0.05)
    handles = world.dispatch(xs, idxs, ws, E)
    torch.cuda.synchronize()
    total_pairs = sum(int((i >= 0).sum()) for i in idxs)
    got = [h.stats(rank=r) for r, h in enumerate(handles)]
    assert sum(g["pairs_received"] for g in got) == total_pairs
    for r, g in enumerate(got):
        assert g["rows_padded"] == handles[r].TK_padded and 0.0 <= g["padding_ratio"] < 1.0
        want_remote = int(((idxs[r] >= 0) & (idxs[r] // (E // R) != r)).sum())
        assert g["pairs_sent_remote"] == want_remote and g["dispatch_bytes_out"] == want_remote * H * 2


def test_three_dispatches_three_routings_one_buffer(native):
    """Three dispatches with three different routings (and token counts) through ONE buffer, all three handles kept
    alive and each checked in full against the oracle afterwards: nothing of one dispatch may leak into another
    (the reference's tests/test_multi_dispatch.py)."""
    R, H, K, E = 4, 256, 6, 32
    world = _world(R, arena_mb=256)
    cases = [_inputs(R, [300, 128, 512, 77], H, K, E, seed=21, sentinel_p=0.05),
             _inputs(R, [64, 700, 33, 256], H, K, E, seed=22, empty_expert=3),
             _inputs(R, 400, H, K, E, seed=23, sentinel_p=0.2)]
    handles = [world.dispatch(xs, idxs, ws, E) for xs, idxs, ws in cases]
    seqs = [h[0].dispatch_seq for h in handles]
    assert seqs == sorted(seqs) and len(set(seqs)) == 3
    for (xs, idxs, ws), hs in zip(cases, handles):
        _check_dispatch(world, hs, xs, idxs, ws, E)


def test_metadata_at_production_scale_top13(native):
    """Every metadata tensor at the size the reference checks (tests/test_metadata.py:289-292: 8192 tokens per
    rank, top-13, 384 experts, 128-row tiles) on 8 emulated ranks, against the vectorised form of the layout
    oracle (pinned to the loop oracle on small cases by tests/test_reference_cpu.py)."""
    from streamep_b200.models.layout_fast import dispatch_layout_fast
    R, T, H, K, E = 8, 8192, 64, 13, 384
    world = _world(R, arena_mb=160)
    g = torch.Generator(device="cpu").manual_seed(99)
    xs, idxs, ws = [], [], []
    for r in range(R):
        # distinct experts per token from a random permutation; 3 % of the pairs are skipped (-1)
        idx = torch.rand(T, E, generator=g).argsort(dim=1)[:, :K].contiguous()
        idx = torch.where(torch.rand(T, K, generator=g) < 0.03, torch.full_like(idx, -1), idx)
        xs.append(torch.randn(T, H, generator=g).to(torch.bfloat16).to(DEV))
        idxs.append(idx.to(DEV)); ws.append(torch.rand(T, K, generator=g).to(DEV))
    handles = world.dispatch(xs, idxs, ws, E)
    torch.cuda.synchronize()
    world.check_status()
    layouts, sends = dispatch_layout_fast(idxs, E, world.buffers[0].num_channels, 128, ws)
    for r in range(R):
        h, L, S = handles[r], layouts[r], sends[r]
        st = h._dispatch_out
        assert h.total_tiles == L.total_tiles and st.num_recv_tokens == L.num_recv_tokens
        for name in ("expert_frequency", "expert_pool_block_offset", "base_pool", "seen_per_substream",
                     "tile_id_to_expert", "pool_arrival_target", "pool_recv_token", "pool_k_slot",
                     "recv_token_to_slots", "k_local_total", "recv_channel_prefix_matrix"):
            assert torch.equal(getattr(h, name), getattr(L, name)), f"rank {r}: {name}"
        assert torch.equal(h.rank_prefix_matrix[:, r], L.rank_prefix_matrix[:, r])
        assert torch.equal(h.pool_arrival_count, L.pool_arrival_target)
        assert torch.equal(h.pool_src[:, 0], L.pool_src_rank) and torch.equal(h.pool_src[:, 1], L.pool_src_token)
        assert torch.equal(st.pair_slot, S.pair_slot) and torch.equal(st.send_recv_token, S.send_recv_token)
        assert torch.equal(h.send_head, S.send_head) and torch.equal(h.channel_prefix_matrix, S.channel_prefix_matrix)
        valid = (L.pool_recv_token >= 0).nonzero().squeeze(1)
        all_x = torch.stack(xs)                                      # [R, T, H]
        want_rows = all_x[L.pool_src_rank[valid].long(), L.pool_src_token[valid].long()]
        assert torch.equal(h.pool[valid], want_rows), f"rank {r}: pool rows"
        assert torch.equal(h.pool_topk_weight[valid], L.pool_topk_weight[valid])
