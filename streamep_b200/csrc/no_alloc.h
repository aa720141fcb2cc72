// Allocation-free entry point for the down-projection + scatter kernel ("kernel Y").
//
// This entry point has no counterpart in the reference library.
//
// Who needs it: code that must not touch the CUDA allocator at the moment it runs the kernel -
// a host thread inside another framework's memory-planning phase, a plugin that is handed
// pre-sized input/output buffers and nothing else, a real-time loop where cudaMalloc's implicit
// device synchronisation is not acceptable.  The regular path (streamep_b200.ops.streaming_moe_y)
// takes a caller-allocated `tile_n_stripes_done` scratch tensor, which in practice comes from
// torch's caching allocator; this variant keeps that scratch inside the library image instead.
//
// Scratch: one `static __device__` array of kNoAllocMaxTiles 32-bit counters plus a 256-byte
// status block (128.25 KiB in all), aligned to 256 bytes.  Every GPU that loads the library holds
// it until the process exits.  All calls on a device share it and it keeps the previous call's
// contents, so every call clears the part it uses (stream-ordered memsets) before the kernel
// starts.  Two calls that overlap on the same GPU (different streams, or different host threads)
// race on it: serialise them.
//
// First call on a device: resolves the device address of the scratch array
// (cudaGetSymbolAddress, under a lock, so two host threads may make "the first call" at once) and
// raises the kernel's dynamic shared-memory limit on that device.  Make that first call before
// starting any stream capture on that device.
//
// The call performs no cudaMalloc / cudaFree and calls no allocating library routine.
//
// The call is asynchronous: a return value of 0 means "enqueued on `stream`", not "finished".  Every
// wait inside the kernel is bounded (2 s); a wait that gives up makes the kernel return early with
// `o`, `k_local_remaining` and `y_done_per_token` only partly written.  After synchronising the
// stream, completion shows as y_done_per_token[r] == seq for every recv token that has slots, and
// streamep_noalloc_device_status() reports whether a wait gave up.  The status is cleared by the
// next call on that device, so read it first.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

enum { kNoAllocMaxTiles = 32768 };   // 4,194,304 pool rows

// y = postact[rows, I] @ w2[e]^T, scaled by pool_topk_weight[slot], accumulated with bf16x2
// red.add into o[pool_recv_token[slot], :H]; after the last slot of recv token r:
// k_local_remaining[r] reaches 0 and y_done_per_token[r] = seq.
//
//   postact            [total_tiles * 128, ffn]   bf16, row-major, device
//   w2                 [num_local_experts, hidden, ffn] bf16, device
//   tile_id_to_expert  [total_tiles] int32, device
//   pool_topk_weight   [total_tiles * 128] float32, device
//   pool_recv_token    [total_tiles * 128] int32, device (-1 = padding row, skipped)
//   o                  [num_recv_tokens, hidden] bf16, device; the caller zeroes it
//   k_local_remaining  [num_recv_tokens] int32, device; in: slots per token, out: 0
//   y_done_per_token   [num_recv_tokens] int64, device
//   stream             a cudaStream_t (0 = default stream)
//
// Returns 0 when the work was enqueued.  Negative, with nothing enqueued: -1 size beyond
// kNoAllocMaxTiles, -2 bad argument (null pointer, negative size, hidden or ffn not a multiple of
// 8, misaligned base), -3 CUDA error.  The message of the last failure on the calling thread is
// available from streamep_noalloc_last_error().
int streamep_gemm_y_scatter_noalloc(const void* postact, const void* w2, const int* tile_id_to_expert,
                                    const float* pool_topk_weight, const int* pool_recv_token, void* o,
                                    int* k_local_remaining, long long* y_done_per_token, int total_tiles,
                                    int hidden, int ffn, int num_local_experts, long long seq, void* stream);

const char* streamep_noalloc_last_error(void);

// Waits for the work already enqueued on the current device, then reads the status block of the
// last no-alloc call there: *code == 0 when no device-side wait gave up (otherwise a StatusCode of
// status.h, e.g. 5 = pipeline wait), *where = the tile it concerned.  Either pointer may be null.
// Returns 0, or -3 on a CUDA error.  Allocates nothing.
int streamep_noalloc_device_status(int* code, int* where);

#ifdef __cplusplus
}
#endif
