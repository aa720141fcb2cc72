// Host <-> kernel interface of the library: plain parameter structs and C++ launchers.
// No torch headers here, so the .cu files compile fast and stand alone.
//
// Reference counterpart: csrc/kernels/api.cuh (launcher declarations) and
// csrc/kernels/configs.cuh (compile-time limits).
#pragma once

#include <cstdint>
#include <cuda_runtime.h>

#include "status.h"

namespace sep {

constexpr int kMaxRanks = 8;            // one NVSwitch domain (reference: NUM_MAX_NVL_PEERS)
constexpr int kMaxExperts = 1024;       // total experts across ranks handled by the metadata kernel
constexpr int kMaxTopK = 32;
constexpr int kMaxChannels = 64;
constexpr int kTileM = 128;
constexpr int kMailboxWords = 16;       // 64-bit words per published buffer record

// ---------------------------------------------------------------------------------------------
// Control region: a fixed-layout block at the head of every rank's symmetric arena.  Peers write
// into it (count inboxes, barrier flags, buffer records); its offsets are the same on all ranks.
// ---------------------------------------------------------------------------------------------
// Every collective kernel belongs to one "kind"; each kind has its own monotonic epoch counter, flag
// row and record slots, so kinds that run on different streams never share a control word.
enum OpKind : int {
  kKindMetadata = 0, kKindDispatch = 1, kKindDispatchGrads = 2, kKindCombine = 3,
  kKindCombineGrads = 4, kKindGemmYTail = 5, kKindGemmABwdTail = 6, kKindBarrier = 7, kNumKinds = 8,
};
struct ControlLayout {
  int num_ranks, num_channels, num_experts_cap;
  size_t flags;              // int[kNumKinds][kMaxRanks]                    peer p stores its epoch at [kind][p]
  size_t mailbox;            // uint64[kNumKinds][2][kMaxRanks][kMailboxWords] parity-double-buffered records
  size_t inbox_counts;       // int[2][kMaxRanks][C][E_cap]                  per (src, channel, expert) pair counts
  size_t inbox_tokens;       // int[2][kMaxRanks][C][kMaxRanks]              per (src, channel, dst) token counts
  size_t inbox_misc;         // int[2][kMaxRanks][4]                          per src: region id of a capacity-mode dispatch (-1 = exact mode)
  size_t total_bytes;
};
ControlLayout make_control_layout(int num_ranks, int num_channels, int num_experts_cap);

// Record a rank publishes to every peer before peers may write into its freshly allocated buffers.
// All fields are byte offsets from the owner's arena base (so one peer base pointer suffices).
struct BufferRecord {
  unsigned long long pool, pool_topk_weight, pool_recv_token, pool_k_slot, pool_src,
      recv_token_to_slots, k_local_total, k_local_remaining, arrival_count, recv_src,
      aux0, aux1, aux2, aux3, aux4;
  unsigned long long stamp;   // written last with release semantics
};
static_assert(sizeof(BufferRecord) == kMailboxWords * 8, "record size");

// Host-mapped (pinned) words the metadata kernel writes for the host poll.
struct HostCounters {
  volatile int epoch;          // == the dispatch epoch once the values below are valid
  volatile int total_tiles;
  volatile int num_recv_tokens;
  volatile int reserved;
  volatile int recv_per_expert[kMaxExperts];
};

// Capacity mode: written by the metadata kernel when a layout does not fit; read by the host whenever it likes.
struct HostOverflow {
  volatile int count;          // number of dispatches that overflowed since the buffer was created
  volatile int epoch;          // metadata epoch of the most recent one
  volatile int needed_tiles;   // largest per-rank tile count of that dispatch
  volatile int needed_recv;    // largest per-rank recv-token count of that dispatch
};

// ---------------------------------------------------------------------------------------------
// Metadata kernel (count exchange + layout synthesis)
// ---------------------------------------------------------------------------------------------
struct MetadataParams {
  // inputs
  const long long* topk_idx;     // [T, K] int64, -1 = skip
  int num_tokens, num_topk, num_experts, num_ranks, rank, num_channels, tile_m;
  int epoch;                     // monotonic per-buffer collective counter
  int phase_mask;                // bit0: count + exchange + signal; bit1: wait + synthesize; bit2: materialise (own launch)
  int push_order;                // order of send_list: 0 = (local expert, rotated dst, channel), 1 = (local expert, channel, rotated dst)
  // symmetric memory
  void* peer_base[kMaxRanks];    // arena bases (own entry included)
  ControlLayout ctl;
  // sender-side outputs (local)
  int* pair_rank;                // [T, K] rank of the pair inside its (channel, expert) substream
  int* pair_slot;                // [T, K] destination pool slot (-1 for skipped pairs)
  int* token_rank_in_channel;    // [T, R] rank of token among the channel's tokens sent to dst (-1)
  int* send_recv_token;          // [T, R] recv-token id at dst (-1 = not sent)
  int* send_head;                // [T, R] gap-encoded stream position (handle ABI)
  unsigned char* is_token_in_rank;  // [T, R] derived bitmap (bool)
  int* channel_prefix_matrix;    // [R, C]
  int* send_base;                // [C, E] scratch: base slot at the owner for (channel, expert), src = this rank
  int* send_token_base;          // [C, R] scratch: first recv-token id at dst for (channel, dst)
  int* send_order_base;          // [C, E] scratch: first position in `send_list` of this rank's (channel, expert) pairs
  int* send_list;                // [T * K] pair ids (t * K + k) in push order (see push_order), then (t, k)
  int* num_send;                 // [1] number of valid pairs == used length of send_list
  int* peer_total_tiles;         // [R]
  int* peer_num_recv;            // [R]
  // receiver-side outputs (local)
  int* expert_frequency;         // [E_local]
  int* expert_pool_block_offset; // [E_local + 1]
  int* base_pool;                // [C, R, E_local]
  int* seen_per_substream;       // [C, R, E_local]
  int* rank_prefix_matrix;       // [R, R]
  int* recv_channel_prefix_matrix;  // [R, C]
  int* blocks_done;              // device counter, zero on entry, reset by the kernel
  HostCounters* host;            // mapped pinned memory (device pointer)
  StatusBlock* status;
  unsigned long long wait_budget_ns;
  // Capacity mode (no host read of the sizes): the receive buffers are fixed regions of `tiles_cap` tiles and
  // `recv_cap` recv tokens, the same on every rank.  The kernel checks every rank's layout against the capacity
  // and every rank's region id against its own; on a violation every rank (they all see the same counts) turns
  // the dispatch into an empty one and records kStatusOverflow / kStatusRegionMismatch.
  int region_id;                 // -1: exact mode
  int tiles_cap, recv_cap;
  int* dev_sizes;                // [4] device: total_tiles, num_recv_tokens, overflow flag, reserved (capacity mode)
  int* tile_id_to_expert;        // [tiles_cap] filled by the materialise launch in capacity mode
  int* pool_arrival_target;      // [tiles_cap]
  HostOverflow* host_overflow;   // mapped pinned memory: where the host learns of an overflow without a sync
};
void launch_dispatch_metadata(const MetadataParams& p, cudaStream_t stream);

struct FillParams {
  int total_tiles, tile_m, num_local_experts, tk_padded, num_recv_tokens, num_topk;
  const int* expert_frequency;
  const int* expert_pool_block_offset;
  int* tile_id_to_expert;
  int* pool_arrival_target;
  int* pool_arrival_count;
  int* pool_recv_token;        // -> -1
  int* pool_k_slot;            // -> -1
  int2* pool_src;              // -> (-1, -1)
  float* pool_topk_weight;     // -> 0
  int* recv_token_to_slots;    // -> -1
  int* k_local_total;          // -> 0
  int* k_local_remaining;      // -> 0
  long long* y_done_per_token; // -> 0
  int2* recv_src;              // -> (-1, -1)
};
void launch_fill_tile_metadata(const FillParams& p, cudaStream_t stream);

// ---------------------------------------------------------------------------------------------
// Push dispatch (forward rows or backward gradient rows) into peers' pool slots
// ---------------------------------------------------------------------------------------------
struct PushParams {
  const void* x;                 // [T, H] bf16 rows to ship
  const long long* topk_idx;     // [T, K]
  const float* topk_weights;     // [T, K] (forward only)
  const int* pair_slot;          // [T, K]
  const int* send_recv_token;    // [T, R]
  const int* send_list;          // [num_send] pair ids in push order
  const int* num_send;           // [1]
  int num_tokens, hidden, num_topk, num_experts, num_ranks, rank, tile_m;
  int is_grads;                  // 1: rows only (no per-slot / per-token scalars)
  int kind;                      // kKindDispatch or kKindDispatchGrads
  int epoch;
  int flags;                     // bit0 publish own record, bit1 push, bit2 tail wait for own tiles
  int static_targets;            // 1: every rank's buffers sit at the offsets of `own` (capacity mode): no records
  int pairs_per_chunk;           // pairs one warp ships between two counter releases (<= 32)
  int head_pairs_per_chunk;      // the first `head_chunks` chunks are this small, so that the first tiles complete early
  int head_chunks;               // (0 = every chunk has pairs_per_chunk pairs)
  int active_push_warps;         // push warps per CTA of the fused kernels that take chunks (0 = all)
  int row_filter;                // which pairs this launch / CTA ships: 0 all, 1 only those that stay on this rank, 2 only remote ones
  int split_local;               // with push-only CTAs: they ship the remote pairs, the push warps of the GEMM CTAs the local ones
  int* work_counter_local;       // chunk claim of the local-pair walkers (zero on entry, reset by the kernel)
  int bulk_push;                 // push-only CTAs copy rows through the bulk-copy engine (shared-memory ring) instead of ld/st
  int push_ctas;                 // fused kernels: this many CTAs only push and the others only multiply (0 = every CTA does both)
  void* peer_base[kMaxRanks];
  ControlLayout ctl;
  BufferRecord own;              // offsets of this rank's freshly allocated buffers (grads: only `pool`
                                 // = the gradient pool and `arrival_count` = its tile counters are used)
  // own tiles, for the tail wait
  const int* own_arrival_count;
  const int* own_arrival_target;
  int own_total_tiles;
  int* started_flag;             // bumped once when the kernel is resident
  int* work_counter;             // dynamic chunk claim, zero on entry, reset by the kernel
  int* blocks_done;
  StatusBlock* status;
  unsigned long long wait_budget_ns;
};
void launch_dispatch_push(const PushParams& p, int num_blocks, cudaStream_t stream);

// ---------------------------------------------------------------------------------------------
// Pull combine: each source rank gathers its tokens' partial rows from the expert ranks
// ---------------------------------------------------------------------------------------------
struct CombineParams {
  int num_tokens, hidden, num_topk, num_ranks, rank, num_experts;
  int is_fwd;                    // 0: also gather K per-slot fp32 weight grads
  long long seq;                 // gate value: done_per_token[r] >= seq
  int kind;                      // kKindCombine or kKindCombineGrads
  int epoch;
  int flags;                     // bit0 publish, bit1 gather, bit2 tail barrier
  const int* send_recv_token;    // [T, R]
  const int* pair_slot;          // [T, K]
  const long long* topk_idx;     // [T, K]
  void* out;                     // [T, H] bf16
  float* out_topk_weights;       // [T, K] (bwd)
  void* peer_base[kMaxRanks];
  ControlLayout ctl;
  BufferRecord own;              // aux0 = x rows, aux1 = done stamps, aux2 = per-slot weights
  int* blocks_done;
  StatusBlock* status;
  unsigned long long wait_budget_ns;
};
void launch_combine_pull(const CombineParams& p, int num_blocks, cudaStream_t stream);

// ---------------------------------------------------------------------------------------------
// Small utility kernels
// ---------------------------------------------------------------------------------------------
struct BarrierParams {
  int num_ranks, rank, epoch;
  int kind;                      // flag row (kKindBarrier, or a GEMM tail kind when a rank has no tiles)
  int wait;                      // 0: signal only
  void* peer_base[kMaxRanks];
  ControlLayout ctl;
  StatusBlock* status;
  unsigned long long wait_budget_ns;
};
void launch_device_barrier(const BarrierParams& p, cudaStream_t stream);

// Test stand-in for dispatch: fires `count[i] += target[i]` tile by tile with a delay in between
// (reference: stream_ep/stream_moe/kernel_a.py:310-402).
void launch_tile_producer(int* count, const int* target, int num_tiles, long long delay_ns,
                          cudaStream_t stream);

// Row gather/scatter between the padded pool and the compact per-recv-token matrix
// (reference: stream_ep/stream_moe/recv_pool_compress.py:29-78).
void launch_pool_compress(const void* pool, void* recv, const int* pool_recv_token, int tk_padded,
                          int hidden, cudaStream_t stream);
void launch_pool_expand(const void* recv, void* pool, const int* pool_recv_token, int tk_padded,
                        int hidden, cudaStream_t stream);

// out[t, :] += sum over the pairs (t, k) owned by OTHER ranks of rows[t * K + k, :], accumulated in fp32.
// Second half of the fused combine: expert ranks store one bf16 row per remote (token, k) pair into the
// source rank's `rows`; pairs owned by the source rank itself were already reduced into `out`.
// Optionally also copies the per-pair scalars peers stored into `dw_src` [T, K] to `dw_dst` (0 for skipped pairs),
// so that a persistent landing area never has to be zeroed.  `skip_rows` (optional, device): when it reads non-zero
// the landed rows are stale (a capacity-mode dispatch that ran empty) and `out` is left untouched.
void launch_combine_reduce(void* out, const void* rows, const long long* topk_idx, int num_tokens, int hidden,
                           int num_topk, int num_experts, int num_ranks, int rank, cudaStream_t stream,
                           const float* dw_src = nullptr, float* dw_dst = nullptr, const int* skip_rows = nullptr);

struct RouterParams {
  const void* x;        // [T, H] bf16
  const void* w_gate;   // [E, H] bf16
  int num_tokens, hidden, num_experts, num_topk, num_ranks, renormalize;
  long long* topk_idx;  // [T, K]
  float* topk_weights;  // [T, K]
  unsigned char* is_token_in_rank;  // [T, R]
  float* probs;         // optional [T, E] softmax output (for the backward), may be null
};
void launch_router(const RouterParams& p, cudaStream_t stream);
// Second half of the tensor-core router: softmax / top-k / rank bitmap from fp32 logits [T, ld_logits] that the
// grouped GEMM wrote with its fp32 store epilogue (p.x / p.w_gate are not read).
void launch_router_finish(const RouterParams& p, const float* logits, int ld_logits, cudaStream_t stream);

// ---------------------------------------------------------------------------------------------
// Grouped GEMM on tcgen05 / TMEM
// ---------------------------------------------------------------------------------------------
enum GemmMode : int { kVarlenM = 0, kVarlenK = 1 };
enum GemmEpilogue : int { kEpiStore = 0, kEpiSwiglu = 1, kEpiScatter = 2, kEpiDswiglu = 3, kEpiStoreF32 = 4 };

struct TailSignal {              // end-of-kernel "all my remote writes are done" handshake
  int enabled;
  int kind;                      // kKindGemmYTail or kKindGemmABwdTail
  int epoch;
  int wait;                      // 0: signal only (emulated ranks run one after another)
  int* ctas_done;                // zero on entry, reset by the kernel
};

// Where a GEMM epilogue finds a buffer that lives on every rank at a rank-specific arena offset:
// word `field` of the record that rank published for (`kind`, `epoch`).
struct RemoteRef {
  int enabled, kind, epoch, field;
  int is_static;                 // 1: the buffer sits at `offset` of every rank's arena (capacity mode), no record
  unsigned long long offset;
};

struct GemmParams {
  int mode, epilogue;
  int block_n;                   // 128 or 256
  int a_mn_major, b_mn_major;
  int N;                         // output columns (per expert)
  int K;                         // reduction length (VarlenM)
  int M_out;                     // output rows per expert (VarlenK)
  int num_experts;               // local experts
  int num_m_tiles, num_n_tiles;
  const int* num_m_tiles_dev;    // VarlenM, optional: the live tile count in device memory (<= num_m_tiles, which is
                                 // then the capacity the tensor maps were built for)
  int total_rows;                // rows of A / outputs (TK_padded)
  const int* tile_id_to_expert;          // [tiles]            (VarlenM)
  const int* expert_pool_block_offset;   // [E + 1] tile units (VarlenK)
  const int* expert_frequency;           // [E] true row count (VarlenK)
  // streaming gate (VarlenM): tile t may be read once count[t] == target[t]
  const int* arrival_count;
  const int* arrival_target;
  int* started_flag;
  // outputs
  void* out0; long long ld0;     // store / postact / dswiglu_in
  void* out1; long long ld1;     // optional preact (swiglu) / weighted postact (dswiglu)
  long long out_expert_stride;   // elements between experts (VarlenK outputs)
  // epilogue inputs
  const void* preact; long long ld_preact;   // dswiglu
  const float* row_weight;       // pool_topk_weight, may be null (unweighted scatter)
  const int* row_token;          // pool_recv_token (-1 = padding row)
  float* dl_dweight;             // [rows] fp32, red.add per (row, n-tile)
  // scatter targets
  void* scatter_local;           // [T_recv, N] bf16 (local variant)
  const int2* row_src;           // per-slot (src_rank, src_token) (remote variant)
  RemoteRef remote_out;          // remote variant: each source rank's [T * K, N] bf16 rows, one per (token, k);
                                 // rows whose source is this rank are red.added into scatter_local instead
  // remote return of per-slot scalars (dswiglu, fused backward): final dl_dweight -> source [T, K] fp32
  RemoteRef remote_dw;
  const int* row_k_slot;
  int num_topk;
  // symmetric memory (needed by remote refs and the tail handshake)
  int num_ranks;
  void* peer_base[kMaxRanks];
  ControlLayout ctl;
  // per-token completion (local scatter)
  int* tile_stripes_done;        // [tiles], zero on entry
  int* k_remaining;              // [T_recv]
  long long* done_per_token;     // [T_recv]
  long long seq;
  TailSignal tail;
  int rank;
  StatusBlock* status;
  unsigned long long wait_budget_ns;
  // VarlenK, optional second problem in the same launch (dW1 and dW2 together: one tail instead of two) and dynamic
  // tile claim.  Tiles of problem 2 follow those of problem 1 in the linear order; its operands, output and sizes:
  int N2, M_out2, num_m_tiles2, num_n_tiles2;      // num_m_tiles2 == 0: no second problem
  // tile_counter != null: CTAs claim tiles with atomicAdd(tile_counter) instead of striding by the grid size, so
  // tiles of unequal length (experts of unequal row counts) and the last wave balance out.  Two ints, zero on
  // entry, reset by the kernel: [0] next tile, [1] CTAs done.
  int* tile_counter;
  // Optional per-CTA time stamps, [gridDim.x][kTimingCols] int64 of %globaltimer nanoseconds (null = off):
  // 0 kernel start, 1 ns the operand pipeline stood still for tile gates, 2 first tile ready, 3 tiles this CTA had
  // finished when its push ended, 4 first push chunk
  // claimed, 5 last push chunk done, 6 kernel end, 7 tiles this CTA multiplied; and in SM clock cycles, of the
  // thread that issues the MMAs: 8 its whole tile loop, 9 of that waiting for operands to land in shared memory,
  // 10 of that waiting for the epilogue to give an accumulator back (11 unused).
  long long* timing;
};
constexpr int kTimingCols = 12;

// tmap_a / tmap_b: 128-byte CUtensorMap blobs (3-D, bf16, 128-byte swizzle) built by the host.
// tmap_o0 / tmap_o1: output maps for the TMA-store epilogues (store, swiglu, dswiglu); box 32 rows x one
// staging row (32, 64 or 128 bytes) with the matching swizzle.  Null for the scatter epilogue.
// Returns false, launching nothing, when no kernel instance exists for the mode / layout / epilogue combination.
// `setup_error` (optional) receives the error of the per-device kernel set-up (shared-memory attribute); when it is
// not cudaSuccess nothing was launched either.
// `maps2`: three more 128-byte maps (A, B, output) of the second VarlenK problem, or null.
bool launch_grouped_gemm(const GemmParams& p, const void* tmap_a, const void* tmap_b, const void* tmap_o0,
                         const void* tmap_o1, const PushParams* fused_push, int num_ctas, cudaStream_t stream,
                         cudaError_t* setup_error = nullptr, const void* maps2 = nullptr);
size_t grouped_gemm_smem_bytes(int block_n);

}  // namespace sep
