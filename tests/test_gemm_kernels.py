"""tcgen05 grouped-GEMM kernels against plain fp32 PyTorch.

Single GPU, hand-built pools, gates pre-fired or fired by the stand-in producer
(test tiers of the reference: stream_ep/stream_moe/tests/test_kernel_a.py,
test_kernel_y.py, test_kernel_y_bwd.py, test_kernel_a_bwd.py).
"""
import pytest
import torch

from helpers import make_pool_case
from streamep_b200.models.reference import check_close, dswiglu_reference, swiglu_interleaved

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _ops():
    from streamep_b200.ops import grouped_gemm as gg
    return gg


def _check_status():
    from streamep_b200.ops.grouped_gemm import default_runtime
    msg = default_runtime().poll_status(True)
    assert msg == "", msg


def _weights(E, n, k, seed, scale=0.05):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(E, n, k, generator=g) * scale).to(torch.bfloat16).to(DEV)


@pytest.mark.parametrize("H,I,freqs", [
    (128, 128, [128]),                      # single tile, single k-pass of two blocks
    (256, 256, [100, 0, 300, 128]),         # multi tile, empty expert, partial tiles
    (512, 704, [260, 130, 5]),              # N = 1408: 5.5 x 256 -> masked last tile; I not multiple of 128
    (2048, 1408, [700, 900, 300, 650]),     # flagship-like shape, > 148 tiles
])
def test_kernel_a_swiglu(native, H, I, freqs):
    gg = _ops()
    E = len(freqs)
    case = make_pool_case(E, freqs, H, seed=1, device=DEV)
    w1 = _weights(E, 2 * I, H, seed=2)
    post, pre = gg.streaming_moe_a(case["pool"], w1, case["tile_e"], store_preact=True)
    torch.cuda.synchronize()
    _check_status()
    want_pre = torch.zeros(case["tkp"], 2 * I, device=DEV)
    for t in range(case["total_tiles"]):
        e = int(case["tile_e"][t])
        rows = slice(t * 128, (t + 1) * 128)
        want_pre[rows] = case["pool"][rows].float() @ w1[e].float().t()
    check_close("preact", pre, want_pre, atol=2e-2, rtol=2e-2)
    check_close("postact", post, swiglu_interleaved(want_pre), atol=2e-2, rtol=2e-2)
    # without preact store, and with the alternative tile width
    for tn in (128, 256):
        post2, pre2 = gg.streaming_moe_a(case["pool"], w1, case["tile_e"], tile_n=tn)
        torch.cuda.synchronize()
        _check_status()
        assert pre2 is None
        check_close(f"postact tile_n={tn}", post2, swiglu_interleaved(want_pre), atol=2e-2, rtol=2e-2)


def test_kernel_a_producer_consumer(native):
    """Tiles are released one by one by a single-thread producer on another stream."""
    gg = _ops()
    H, I, freqs = 256, 128, [128, 200, 64, 128, 128, 300]
    case = make_pool_case(len(freqs), freqs, H, seed=3, device=DEV)
    w1 = _weights(len(freqs), 2 * I, H, seed=4)
    count = torch.zeros_like(case["target"])
    side = torch.cuda.Stream()
    torch.cuda.synchronize()
    with torch.cuda.stream(side):
        gg.fire_tiles_with_delay(count, case["target"], delay_us=20.0)
    post, _ = gg.streaming_moe_a(case["pool"], w1, case["tile_e"], pool_arrival_count=count,
                                 pool_arrival_target=case["target"])
    torch.cuda.synchronize()
    _check_status()
    want = torch.zeros(case["tkp"], 2 * I, device=DEV)
    for t in range(case["total_tiles"]):
        e = int(case["tile_e"][t])
        want[t * 128:(t + 1) * 128] = case["pool"][t * 128:(t + 1) * 128].float() @ w1[e].float().t()
    check_close("postact", post, swiglu_interleaved(want), atol=2e-2, rtol=2e-2)
    assert torch.equal(count, case["target"])


def test_gate_timeout_reports_status(native):
    """A tile that nothing ever releases: the kernel gives up after the budget, reports it and
    returns; the context stays usable."""
    gg = _ops()
    rt = gg.default_runtime()
    old = rt.get_timeout_ms()
    rt.set_timeout_ms(200)
    try:
        case = make_pool_case(1, [128], 128, seed=5, device=DEV)
        w1 = _weights(1, 256, 128, seed=6)
        count = torch.zeros_like(case["target"])
        gg.streaming_moe_a(case["pool"], w1, case["tile_e"], pool_arrival_count=count,
                           pool_arrival_target=case["target"])
        msg = rt.poll_status(True)
        assert "tile gate timeout" in msg, msg
    finally:
        rt.set_timeout_ms(old)
    # still healthy
    post, _ = gg.streaming_moe_a(case["pool"], w1, case["tile_e"])
    torch.cuda.synchronize()
    _check_status()
    assert torch.isfinite(post.float()).all()


@pytest.mark.parametrize("H,I,freqs", [(128, 128, [128]), (512, 704, [260, 130, 5]), (2048, 1408, [700, 300, 650])])
def test_preact_recompute(native, H, I, freqs):
    gg = _ops()
    E = len(freqs)
    case = make_pool_case(E, freqs, H, seed=7, device=DEV)
    w1 = _weights(E, 2 * I, H, seed=8)
    pre = gg.grouped_gemm_preact(case["pool"], w1, case["tile_e"])
    torch.cuda.synchronize()
    _check_status()
    want = torch.zeros(case["tkp"], 2 * I, device=DEV)
    for t in range(case["total_tiles"]):
        e = int(case["tile_e"][t])
        want[t * 128:(t + 1) * 128] = case["pool"][t * 128:(t + 1) * 128].float() @ w1[e].float().t()
    check_close("preact", pre, want, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("H,I,freqs,klocal", [(128, 128, [128], 1), (256, 192, [100, 0, 300, 128], 2),
                                               (2048, 1408, [700, 300, 650], 3)])
def test_kernel_y_scatter(native, H, I, freqs, klocal):
    """y = postact @ W2^T, weighted, accumulated into o[r]; klocal slots share one recv token."""
    gg = _ops()
    E = len(freqs)
    case = make_pool_case(E, freqs, I, seed=9, device=DEV, garbage_padding=True)
    postact = case["pool"]                      # [TKp, I], padding rows = +inf must be ignored
    w2 = _weights(E, H, I, seed=10)
    nvalid = case["num_valid"]
    n_recv = (nvalid + klocal - 1) // klocal
    recv_token = torch.where(case["recv_token"] >= 0, case["recv_token"] // klocal, case["recv_token"])
    g = torch.Generator(device="cpu").manual_seed(11)
    wts = torch.rand(case["tkp"], generator=g).to(DEV)
    k_rem = torch.bincount(recv_token[recv_token >= 0].long(), minlength=n_recv).to(torch.int32)
    k_total = k_rem.clone()
    o = torch.zeros(n_recv, H, dtype=torch.bfloat16, device=DEV)
    done = torch.zeros(n_recv, dtype=torch.int64, device=DEV)
    stripes = torch.zeros(case["total_tiles"], dtype=torch.int32, device=DEV)
    gg.streaming_moe_y(postact, w2, case["tile_e"], wts, recv_token, o=o, tile_n_stripes_done=stripes,
                       k_local_remaining=k_rem, y_done_per_token=done, combine_seq=7)
    torch.cuda.synchronize()
    _check_status()
    want = torch.zeros(n_recv, H, device=DEV)
    for t in range(case["total_tiles"]):
        e = int(case["tile_e"][t])
        rows = torch.arange(t * 128, (t + 1) * 128, device=DEV)
        ok = recv_token[rows] >= 0
        rows = rows[ok]
        y = postact[rows].float() @ w2[e].float().t()
        want.index_add_(0, recv_token[rows].long(), wts[rows, None] * y)
    # klocal bf16 partial sums are rounded to bf16 after every red.add: scale atol with the data
    check_close("o", o, want, atol=2e-2 * float(want.abs().max()) ** 0.5 * klocal, rtol=3e-2)
    assert (k_rem == 0).all()
    assert (done[k_total > 0] == 7).all()


@pytest.mark.parametrize("H,I,freqs", [(128, 128, [128]), (256, 192, [100, 0, 300, 128]), (2048, 1408, [700, 300, 650])])
def test_kernel_y_bwd(native, H, I, freqs):
    gg = _ops()
    E = len(freqs)
    case = make_pool_case(E, freqs, H, seed=12, device=DEV, garbage_padding=True)
    dl_do = case["pool"]                        # padding rows = +inf
    w2 = _weights(E, H, I, seed=13)
    g = torch.Generator(device="cpu").manual_seed(14)
    preact = torch.randn(case["tkp"], 2 * I, generator=g).to(torch.bfloat16).to(DEV)
    wts = torch.rand(case["tkp"], generator=g).to(DEV)
    din = torch.full((case["tkp"], 2 * I), float("nan"), dtype=torch.bfloat16, device=DEV)
    pw = torch.full((case["tkp"], I), float("nan"), dtype=torch.bfloat16, device=DEV)
    dlw = torch.zeros(case["tkp"], dtype=torch.float32, device=DEV)
    gg.streaming_moe_y_bwd(dl_do, w2, preact, case["tile_e"], wts, case["recv_token"], dL_dswiglu_in=din,
                           postact_a_for_dW2=pw, dL_dweight=dlw)
    torch.cuda.synchronize()
    _check_status()
    valid = case["recv_token"] >= 0
    assert (din[~valid] == 0).all() and (pw[~valid] == 0).all(), "padding rows must come out exactly zero"
    gref = torch.zeros(case["tkp"], I, device=DEV)
    for t in range(case["total_tiles"]):
        e = int(case["tile_e"][t])
        rows = torch.arange(t * 128, (t + 1) * 128, device=DEV)
        rows = rows[valid[rows]]
        gref[rows] = dl_do[rows].float() @ w2[e].float()
    pf = preact.float()
    dgate, dup, post = dswiglu_reference(pf[:, 0::2], pf[:, 1::2], gref)
    want_in = torch.stack([dgate, dup], dim=-1).reshape(case["tkp"], 2 * I) * wts[:, None]
    check_close("dL_dswiglu_in", din[valid], want_in[valid], atol=3e-2, rtol=3e-2)
    check_close("postact_for_dW2", pw[valid], (post * wts[:, None])[valid], atol=3e-2, rtol=3e-2)
    check_close("dL_dweight", dlw[valid], (post * gref).sum(-1)[valid], atol=5e-2 * (I ** 0.5) / 8, rtol=3e-2)


@pytest.mark.parametrize("H,I,freqs", [(128, 128, [128]), (256, 192, [100, 0, 300, 128]), (2048, 1408, [700, 300, 650])])
def test_kernel_a_bwd(native, H, I, freqs):
    gg = _ops()
    E = len(freqs)
    case = make_pool_case(E, freqs, 2 * I, seed=15, device=DEV, garbage_padding=True)
    din = case["pool"]
    w1 = _weights(E, 2 * I, H, seed=16)
    n_recv = case["num_valid"]
    dx = torch.zeros(n_recv, H, dtype=torch.bfloat16, device=DEV)
    krem = torch.ones(n_recv, dtype=torch.int32, device=DEV)
    done = torch.zeros(n_recv, dtype=torch.int64, device=DEV)
    stripes = torch.zeros(case["total_tiles"], dtype=torch.int32, device=DEV)
    gg.streaming_moe_a_bwd(din, w1, case["tile_e"], case["recv_token"], dL_dx_per_r=dx,
                           tile_n_stripes_done=stripes, bwd_k_local_remaining=krem, bwd_a_done_per_token=done,
                           dispatch_seq=3)
    torch.cuda.synchronize()
    _check_status()
    want = torch.zeros(n_recv, H, device=DEV)
    for t in range(case["total_tiles"]):
        e = int(case["tile_e"][t])
        rows = torch.arange(t * 128, (t + 1) * 128, device=DEV)
        rows = rows[case["recv_token"][rows] >= 0]
        want[case["recv_token"][rows].long()] = din[rows].float() @ w1[e].float()
    check_close("dL_dx_per_r", dx, want, atol=3e-2, rtol=3e-2)
    assert (done == 3).all() and (krem == 0).all()


@pytest.mark.parametrize("M,N,freqs", [(128, 128, [64]), (128, 256, [130, 0, 63, 257]), (320, 200, [100, 300]),
                                        (2816, 2048, [700, 300])])
def test_grouped_gemm_dw(native, M, N, freqs):
    """dW[e] = lhs[rows_e]^T @ rhs[rows_e]; padding rows hold +inf and must not contribute."""
    gg = _ops()
    E = len(freqs)
    lhs_case = make_pool_case(E, freqs, M, seed=17, device=DEV, garbage_padding=True)
    rhs_case = make_pool_case(E, freqs, N, seed=18, device=DEV, garbage_padding=True)
    out = gg.grouped_gemm_dw(lhs_case["pool"], rhs_case["pool"], lhs_case["offsets"], lhs_case["freqs"])
    torch.cuda.synchronize()
    _check_status()
    want = torch.zeros(E, M, N, device=DEV)
    for e, f in enumerate(freqs):
        r0 = int(lhs_case["offsets"][e]) * 128
        want[e] = lhs_case["pool"][r0:r0 + f].float().t() @ rhs_case["pool"][r0:r0 + f].float()
    scale = max(freqs) ** 0.5
    check_close("dW", out, want, atol=2e-2 * scale, rtol=2e-2)


@pytest.mark.parametrize("M,N,M2,N2,freqs", [(256, 128, 128, 256, [130, 0, 63, 257]), (2816, 2048, 2048, 1408, [700, 90, 1300]),
                                              (320, 200, 200, 72, [100, 300])])
def test_grouped_gemm_dw_two_problems_dynamic_claim(native, M, N, M2, N2, freqs):
    """dW1 and dW2 in one launch with tiles claimed from a device counter (experts of very unequal length, one
    empty), twice in a row (the kernel puts the counter back to zero), against fp32 and against the static launch."""
    gg = _ops()
    E = len(freqs)
    cases = [make_pool_case(E, freqs, w, seed=40 + i, device=DEV, garbage_padding=True) for i, w in enumerate((M, N, M2, N2))]
    off, fr = cases[0]["offsets"], cases[0]["freqs"]
    for rep in range(2):
        o1, o2 = gg.grouped_gemm_dw(cases[0]["pool"], cases[1]["pool"], off, fr, lhs2=cases[2]["pool"], rhs2=cases[3]["pool"],
                                    tile_n=256, dynamic_tiles=True)
        torch.cuda.synchronize()
        _check_status()
        for out, (l, r) in ((o1, (cases[0], cases[1])), (o2, (cases[2], cases[3]))):
            want = torch.zeros_like(out, dtype=torch.float32)
            for e, f in enumerate(freqs):
                r0 = int(off[e]) * 128
                want[e] = l["pool"][r0:r0 + f].float().t() @ r["pool"][r0:r0 + f].float()
            check_close(f"dW (rep {rep})", out, want, atol=2e-2 * max(freqs) ** 0.5, rtol=2e-2)
    static = gg.grouped_gemm_dw(cases[0]["pool"], cases[1]["pool"], off, fr, tile_n=256)
    torch.cuda.synchronize()
    assert torch.equal(static, o1), "dynamic claim must not change the result of a tile"


def test_pool_compress_roundtrip(native):
    gg = _ops()
    case = make_pool_case(3, [100, 0, 300], 520, seed=19, device=DEV)
    n_recv = case["num_valid"]
    x_recv = gg.compress_pool_to_recv(case["pool"], case["recv_token"], n_recv)
    pool2 = gg.reexpand_recv_to_pool(x_recv, case["recv_token"], case["tkp"])
    torch.cuda.synchronize()
    assert torch.equal(pool2, case["pool"])      # padding rows of the hand-built pool are zero
    valid = case["recv_token"] >= 0
    assert torch.equal(x_recv[case["recv_token"][valid].long()], case["pool"][valid])


@pytest.mark.parametrize("T,H,E,K,R", [(300, 256, 64, 6, 8), (515, 2048, 8, 6, 1), (130, 200, 24, 4, 2),
                                       (257, 1032, 256, 8, 8), (64, 512, 136, 3, 1)])
@pytest.mark.parametrize("tensor_cores", [True, False])
def test_router(native, T, H, E, K, R, tensor_cores):
    """Both router paths - logits from the tcgen05 grouped GEMM with the fp32 store epilogue plus the finishing
    kernel, and the SIMT kernel in every expert-width instance (16 / 32 / 64 experts per pass, several passes,
    widths that are not a multiple of the chunk) - against softmax -> top-k -> renormalise in fp32."""
    from streamep_b200.models.reference import router_reference
    gg = _ops()
    g = torch.Generator(device="cpu").manual_seed(20)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16).to(DEV)
    wg = (torch.randn(E, H, generator=g) * 0.1).to(torch.bfloat16).to(DEV)
    gg.default_runtime().set_router_on_tensor_cores(tensor_cores)
    try:
        idx, w, in_rank, probs = gg.router_topk(x, wg, K, num_ranks=R, return_probs=True)
        torch.cuda.synchronize()
    finally:
        gg.default_runtime().set_router_on_tensor_cores(True)
    _check_status()
    ridx, rw = router_reference(x, wg, K)
    check_close("probs", probs, torch.softmax(x.float() @ wg.float().t(), -1), atol=1e-5, rtol=1e-3)
    # compare as sets per token (near-ties may order differently) through the weights gathered by expert id
    dense = torch.zeros(T, E, device=DEV).scatter_(1, idx, w)
    rdense = torch.zeros(T, E, device=DEV).scatter_(1, ridx, rw)
    check_close("topk weights", dense, rdense, atol=1e-4, rtol=1e-3)
    want_rank = torch.zeros(T, R, dtype=torch.bool, device=DEV)
    want_rank.scatter_(1, idx // (E // R), True)
    assert torch.equal(in_rank, want_rank)
