"""The allocation-free variant of kernel Y, called through its exported C symbol.

Some callers cannot allocate device memory when they launch the kernel (they run inside another
framework's memory plan, or get fixed input/output buffers and nothing else).  For them the
library exports ``streamep_gemm_y_scatter_noalloc``: same math as
``streamep_b200.ops.streaming_moe_y``, with the per-tile stripe counters that the regular entry
point takes as a caller-allocated tensor kept in a static device array inside the library.

The test calls the symbol with ctypes on raw device pointers, twice in a row (the second call
must not see the first call's counters), and compares with the regular entry point.
This file sorts last on purpose so that a failure here cannot hide any other test.
"""
import ctypes

import pytest
import torch

from helpers import make_pool_case
from streamep_b200.models.reference import check_close

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _lib():
    from streamep_b200 import _ext
    _ext.load()
    lib = ctypes.CDLL(str(_ext._so_path()))
    fn = lib.streamep_gemm_y_scatter_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 8 + [ctypes.c_int] * 4 + [ctypes.c_longlong, ctypes.c_void_p]
    lib.streamep_noalloc_last_error.restype = ctypes.c_char_p
    lib.streamep_noalloc_device_status.restype = ctypes.c_int
    lib.streamep_noalloc_device_status.argtypes = [ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)]
    return lib


def _case(H, I, freqs, klocal, seed):
    E = len(freqs)
    case = make_pool_case(E, freqs, I, seed=seed, device=DEV, garbage_padding=True)
    g = torch.Generator(device="cpu").manual_seed(seed + 1)
    w2 = (torch.randn(E, H, I, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    wts = torch.rand(case["tkp"], generator=g).to(DEV)
    recv_token = torch.where(case["recv_token"] >= 0, case["recv_token"] // klocal, case["recv_token"]).contiguous()
    n_recv = (case["num_valid"] + klocal - 1) // klocal
    k_total = torch.bincount(recv_token[recv_token >= 0].long(), minlength=n_recv).to(torch.int32)
    return case, w2, wts, recv_token, n_recv, k_total


@pytest.mark.parametrize("H,I,freqs,klocal", [(256, 192, [100, 0, 300, 128], 2), (2048, 1408, [700, 300, 650], 3)])
def test_no_alloc_entry_matches_regular_entry(native, H, I, freqs, klocal):
    from streamep_b200.ops import grouped_gemm as gg
    lib = _lib()
    case, w2, wts, recv_token, n_recv, k_total = _case(H, I, freqs, klocal, seed=31)
    # regular entry point: caller-allocated scratch
    o_ref = torch.zeros(n_recv, H, dtype=torch.bfloat16, device=DEV)
    gg.streaming_moe_y(case["pool"], w2, case["tile_e"], wts, recv_token, o=o_ref,
                       tile_n_stripes_done=torch.zeros(case["total_tiles"], dtype=torch.int32, device=DEV),
                       k_local_remaining=k_total.clone(), y_done_per_token=torch.zeros(n_recv, dtype=torch.int64, device=DEV),
                       combine_seq=5)
    torch.cuda.synchronize()
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):
        o = torch.zeros(n_recv, H, dtype=torch.bfloat16, device=DEV)
        k_rem = k_total.clone()
        done = torch.zeros(n_recv, dtype=torch.int64, device=DEV)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        rc = lib.streamep_gemm_y_scatter_noalloc(
            case["pool"].data_ptr(), w2.data_ptr(), case["tile_e"].data_ptr(), wts.data_ptr(), recv_token.data_ptr(),
            o.data_ptr(), k_rem.data_ptr(), done.data_ptr(), case["total_tiles"], H, I, len(freqs), 9 + call, stream)
        assert rc == 0, lib.streamep_noalloc_last_error().decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        # both entry points reduce with bf16 atomics in arbitrary order: same tolerance as the kernel test
        scale = float(o_ref.float().abs().max()) ** 0.5
        check_close(f"o (call {call})", o, o_ref.float(), atol=2e-2 * scale * klocal, rtol=3e-2)
        assert (k_rem == 0).all()
        assert (done[k_total > 0] == 9 + call).all()
        # a return of 0 only means "enqueued": the status block in the static array says whether a device wait gave up
        code, where = ctypes.c_int(-1), ctypes.c_int(-1)
        assert lib.streamep_noalloc_device_status(ctypes.byref(code), ctypes.byref(where)) == 0
        assert code.value == 0


def test_no_alloc_entry_rejects_oversize(native):
    lib = _lib()
    rc = lib.streamep_gemm_y_scatter_noalloc(1, 1, 1, 1, 1, 1, 1, 1, 32769, 256, 256, 1, 0, None)
    assert rc == -1
    assert b"kNoAllocMaxTiles" in lib.streamep_noalloc_last_error()
    rc = lib.streamep_gemm_y_scatter_noalloc(None, 1, 1, 1, 1, 1, 1, 1, 4, 256, 256, 1, 0, None)
    assert rc == -2
    rc = lib.streamep_gemm_y_scatter_noalloc(1, 1, 1, 1, 1, 1, 1, 1, -3, 256, 256, 1, 0, None)
    assert rc == -2 and b"negative" in lib.streamep_noalloc_last_error()
