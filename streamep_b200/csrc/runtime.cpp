// Host runtime of the library (pybind module `_C`): symmetric arena + peer mapping, the dispatch /
// dispatch_grads / combine host paths split into phases, launch gates, grouped-GEMM launch with
// TMA descriptors, and the status block every bounded device wait reports into.
//
// Reference counterpart: csrc/stream_ep.cpp (Buffer ctor/sync :129-264,458-543; launch gates
// :387-456; intranode_dispatch :1125-1330; dispatch_grads :1332-1451; combine :1453-1561; pybind
// :2070-2156), csrc/config.hpp, csrc/event.hpp.
#include <ATen/cuda/CUDAContext.h>
#include <ATen/cuda/CUDAEvent.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <cuda.h>
#include <cuda_runtime.h>
#include <pybind11/functional.h>
#include <pybind11/stl.h>
#include <torch/extension.h>

#include <atomic>
#include <chrono>
#include <cstring>
#include <optional>
#include <sstream>
#include <thread>

#include "api.h"
#include "arena.h"

namespace py = pybind11;

namespace sep {

#define SEP_CUDA_CHECK(expr)                                                                        \
  do {                                                                                              \
    cudaError_t e__ = (expr);                                                                       \
    if (e__ != cudaSuccess) {                                                                       \
      std::ostringstream os__;                                                                      \
      os__ << "CUDA error " << cudaGetErrorName(e__) << " (" << cudaGetErrorString(e__) << ") at "  \
           << __FILE__ << ":" << __LINE__ << " in " #expr;                                          \
      throw std::runtime_error(os__.str());                                                         \
    }                                                                                               \
  } while (0)

#define SEP_ASSERT(cond, msg)                                                         \
  do {                                                                                \
    if (!(cond)) {                                                                    \
      std::ostringstream os__;                                                        \
      os__ << "streamep_b200: " << msg << " (" #cond ") at " << __FILE__ << ":" << __LINE__; \
      throw std::invalid_argument(os__.str());                                        \
    }                                                                                 \
  } while (0)

// ---------------------------------------------------------------------------------------------
// Driver entry points fetched at run time (the extension does not link libcuda).
// ---------------------------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
using StreamWaitValue32Fn = CUresult (*)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);

template <class Fn>
static Fn driver_fn(const char* name) {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  SEP_CUDA_CHECK(cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &q));
  if (q != cudaDriverEntryPointSuccess || fn == nullptr)
    throw std::runtime_error(std::string("streamep_b200: driver entry point not found: ") + name);
  return reinterpret_cast<Fn>(fn);
}

// 3-D bf16 tensor map, 128-byte swizzle, OOB reads return zero.  dims/box are innermost-first.
static CUtensorMap make_tmap(const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t stride1_elems,
                             uint64_t stride2_elems, uint32_t b0, uint32_t b1,
                             CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
  static EncodeTiledFn encode = driver_fn<EncodeTiledFn>("cuTensorMapEncodeTiled");
  CUtensorMap m;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {stride1_elems * 2, stride2_elems * 2};
  cuuint32_t box[3] = {b0, b1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  SEP_ASSERT(reinterpret_cast<uintptr_t>(base) % 16 == 0, "TMA base address must be 16-byte aligned");
  SEP_ASSERT(strides[0] % 16 == 0 && strides[1] % 16 == 0, "TMA row pitch must be a multiple of 16 bytes");
  CUresult r = encode(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) throw std::runtime_error("streamep_b200: cuTensorMapEncodeTiled failed with code " + std::to_string(r));
  return m;
}

// ---------------------------------------------------------------------------------------------
// Peer-shareable device memory through the virtual-memory-management driver API: cuMemCreate with a POSIX file
// descriptor as the shareable handle, cuMemAddressReserve + cuMemMap + cuMemSetAccess on the owner, and
// cuMemImportFromShareableHandle + map on every peer (the descriptor travels between the processes of a node over a
// Unix socket, see buffer.py).  Second allocator next to cudaMalloc + CUDA IPC, like the reference's
// SharedMemoryAllocator (csrc/stream_ep.cpp:52-124, which uses fabric handles for multi-node NVLink); it is also
// what a multicast (NVLS) binding of the arena would need.
// ---------------------------------------------------------------------------------------------
struct VmmApi {
  CUresult (*create)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long);
  CUresult (*release)(CUmemGenericAllocationHandle);
  CUresult (*reserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
  CUresult (*addr_free)(CUdeviceptr, size_t);
  CUresult (*map)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
  CUresult (*unmap)(CUdeviceptr, size_t);
  CUresult (*set_access)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
  CUresult (*export_handle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long);
  CUresult (*import_handle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType);
  CUresult (*granularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags);
  static const VmmApi& get() {
    static VmmApi api = [] {
      VmmApi a{};
      a.create = driver_fn<decltype(a.create)>("cuMemCreate");
      a.release = driver_fn<decltype(a.release)>("cuMemRelease");
      a.reserve = driver_fn<decltype(a.reserve)>("cuMemAddressReserve");
      a.addr_free = driver_fn<decltype(a.addr_free)>("cuMemAddressFree");
      a.map = driver_fn<decltype(a.map)>("cuMemMap");
      a.unmap = driver_fn<decltype(a.unmap)>("cuMemUnmap");
      a.set_access = driver_fn<decltype(a.set_access)>("cuMemSetAccess");
      a.export_handle = driver_fn<decltype(a.export_handle)>("cuMemExportToShareableHandle");
      a.import_handle = driver_fn<decltype(a.import_handle)>("cuMemImportFromShareableHandle");
      a.granularity = driver_fn<decltype(a.granularity)>("cuMemGetAllocationGranularity");
      return a;
    }();
    return api;
  }
};
#define SEP_CU_CHECK(expr)                                                                                   \
  do {                                                                                                       \
    CUresult r__ = (expr);                                                                                   \
    if (r__ != CUDA_SUCCESS)                                                                                 \
      throw std::runtime_error(std::string("streamep_b200: driver call failed with code ") + std::to_string(r__) + \
                               " in " #expr);                                                                \
  } while (0)

// One mapped range: a physical allocation (own or imported) behind a reserved virtual address range.
struct VmmRange {
  CUmemGenericAllocationHandle handle = 0;
  CUdeviceptr va = 0;
  size_t bytes = 0;
  bool mapped = false;
  void map_for(int device) {
    const VmmApi& api = VmmApi::get();
    SEP_CU_CHECK(api.reserve(&va, bytes, 0, 0, 0));
    SEP_CU_CHECK(api.map(va, bytes, 0, handle, 0));
    mapped = true;
    CUmemAccessDesc acc{};
    acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE; acc.location.id = device;
    acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    SEP_CU_CHECK(api.set_access(va, bytes, &acc, 1));
  }
  void destroy() {
    const VmmApi& api = VmmApi::get();
    if (mapped) { api.unmap(va, bytes); mapped = false; }
    if (va != 0) { api.addr_free(va, bytes); va = 0; }
    if (handle != 0) { api.release(handle); handle = 0; }
  }
};

// ---------------------------------------------------------------------------------------------
// Config (reference: csrc/config.hpp:23-132).  The five-tuple is kept for source compatibility;
// this implementation has no rings, so the chunk sizes only bound the size hints.
// ---------------------------------------------------------------------------------------------
struct Config {
  int num_sms, num_max_nvl_chunked_send_tokens, num_max_nvl_chunked_recv_tokens,
      num_max_rdma_chunked_send_tokens, num_max_rdma_chunked_recv_tokens;
  Config(int sms, int nvl_send, int nvl_recv, int rdma_send, int rdma_recv)
      : num_sms(sms), num_max_nvl_chunked_send_tokens(nvl_send), num_max_nvl_chunked_recv_tokens(nvl_recv),
        num_max_rdma_chunked_send_tokens(rdma_send), num_max_rdma_chunked_recv_tokens(rdma_recv) {
    SEP_ASSERT(sms >= 0, "num_sms must be non-negative");
    SEP_ASSERT(nvl_send > 0 && nvl_recv > 0 && nvl_send < nvl_recv, "NVL chunk sizes must satisfy 0 < send < recv");
    SEP_ASSERT(rdma_send > 0 && rdma_recv > 0, "RDMA chunk sizes must be positive");
  }
  // Same call shape as the reference's ring-size hints (csrc/config.hpp:52-87).  There are no rings
  // here: the arena holds the pools themselves, whose size depends on the token count, so the hint
  // covers a stated workload (8192 tokens per rank, top-8, 1.5x imbalance, two layers in flight).
  // Callers that know their shapes use Buffer.get_arena_size_hint instead.
  size_t get_nvl_buffer_size_hint(size_t hidden_bytes, int num_ranks) const;
  size_t get_rdma_buffer_size_hint(int64_t, int) const { return 0; }   // no RDMA tier on one NVSwitch domain
};

struct ArenaSizeHint {
  // Bytes of symmetric memory one MoE layer keeps alive between its forward and its backward at
  // `level` of activation checkpointing, for `tokens` source tokens per rank routed top-`k`.
  static size_t layer_bytes(int64_t tokens, int64_t hidden, int64_t topk, int num_ranks, int64_t experts_local,
                            double imbalance) {
    const double pairs = static_cast<double>(tokens) * topk * imbalance;
    const double rows = pairs + 128.0 * experts_local;
    const double recv = std::min<double>(static_cast<double>(tokens) * num_ranks, pairs);
    double b = rows * hidden * 2 /*pool*/ + rows * 24 /*per-slot*/ + recv * (topk * 4 + 32) /*per-token*/ +
               recv * hidden * 2 /*o*/ + static_cast<double>(tokens) * hidden * 2 /*out*/;
    return static_cast<size_t>(b * 1.05) + (8u << 20);
  }
};

size_t Config::get_nvl_buffer_size_hint(size_t hidden_bytes, int num_ranks) const {
  SEP_ASSERT(num_ranks >= 1 && num_ranks <= kMaxRanks && hidden_bytes % 2 == 0, "bad hint arguments");
  const size_t per_layer = ArenaSizeHint::layer_bytes(8192, static_cast<int64_t>(hidden_bytes / 2), 8, num_ranks, 32, 1.5);
  return per_layer * 7 / 2;
}

// ---------------------------------------------------------------------------------------------
// Event handle (reference: csrc/event.hpp:9-35)
// ---------------------------------------------------------------------------------------------
struct EventHandle {
  std::shared_ptr<at::cuda::CUDAEvent> event;
  EventHandle() : event(std::make_shared<at::cuda::CUDAEvent>()) { event->record(at::cuda::getCurrentCUDAStream()); }
  explicit EventHandle(const at::cuda::CUDAStream& s) : event(std::make_shared<at::cuda::CUDAEvent>()) { event->record(s); }
  void current_stream_wait() const { event->block(at::cuda::getCurrentCUDAStream()); }
  void wait_on(int64_t raw_stream, int device) const {
    event->block(at::cuda::getStreamFromExternal(reinterpret_cast<cudaStream_t>(raw_stream), device));
  }
};

// ---------------------------------------------------------------------------------------------
// Stream-safe release of arena blocks.  When the last reference to an arena tensor dies, kernels that
// use the block may still be queued on any stream the runtime launched on (the two-stream plan, or a
// caller of Buffer.alloc_symmetric).  The deleter records one event on each of those streams and parks
// the block behind them (Arena::release_deferred); allocate() only reuses it once they have completed.
// ---------------------------------------------------------------------------------------------
struct ReleaseCtx {
  std::mutex mu;
  std::vector<cudaStream_t> streams;     // every stream the runtime has launched or allocated on
  std::vector<cudaEvent_t> event_pool;
  std::shared_ptr<Arena> arena;
  int device = 0;
  bool dead = false;                     // runtime destroyed (device drained): release at once

  void note_stream(cudaStream_t s) {
    std::lock_guard<std::mutex> g(mu);
    for (cudaStream_t t : streams) if (t == s) return;
    streams.push_back(s);
  }
  ~ReleaseCtx() { for (cudaEvent_t e : event_pool) cudaEventDestroy(e); }
};

struct CudaFence : ArenaFence {
  std::shared_ptr<ReleaseCtx> ctx;
  std::vector<cudaEvent_t> events;
  bool ready() override {
    for (cudaEvent_t e : events) {
      const cudaError_t r = cudaEventQuery(e);
      if (r == cudaErrorNotReady) return false;
      if (r != cudaSuccess) cudaGetLastError();   // context going away: nothing can still be running
    }
    return true;
  }
  void wait() override {
    for (cudaEvent_t e : events) if (cudaEventSynchronize(e) != cudaSuccess) cudaGetLastError();
  }
  ~CudaFence() override {
    std::lock_guard<std::mutex> g(ctx->mu);
    for (cudaEvent_t e : events) ctx->event_pool.push_back(e);
  }
};

// Deleter of arena tensors.
static void release_block(const std::shared_ptr<ReleaseCtx>& ctx, size_t off) {
  std::shared_ptr<CudaFence> fence;
  {
    std::unique_lock<std::mutex> g(ctx->mu);
    if (ctx->dead || ctx->streams.empty()) { g.unlock(); ctx->arena->release(off); return; }
    fence = std::make_shared<CudaFence>();
    fence->ctx = ctx;
    int prev = -1;
    cudaGetDevice(&prev);
    if (prev != ctx->device) cudaSetDevice(ctx->device);
    for (size_t i = 0; i < ctx->streams.size();) {
      cudaEvent_t e = nullptr;
      if (!ctx->event_pool.empty()) { e = ctx->event_pool.back(); ctx->event_pool.pop_back(); }
      else if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) { cudaGetLastError(); e = nullptr; }
      if (e != nullptr && cudaEventRecord(e, ctx->streams[i]) == cudaSuccess) {
        fence->events.push_back(e);
        ++i;
      } else {
        // a stream that was destroyed by its owner (or a context that is shutting down) has nothing queued
        cudaGetLastError();
        if (e != nullptr) ctx->event_pool.push_back(e);
        ctx->streams.erase(ctx->streams.begin() + static_cast<long>(i));
      }
    }
    if (prev >= 0 && prev != ctx->device) cudaSetDevice(prev);
  }
  ctx->arena->release_deferred(off, fence);   // (the fence's destructor takes ctx->mu: call it unlocked)
}

// ---------------------------------------------------------------------------------------------
// Per-dispatch state shared between the phases of one dispatch (and kept by the handle)
// ---------------------------------------------------------------------------------------------
struct DispatchState {
  // inputs
  at::Tensor x, topk_idx, topk_weights;
  int num_tokens = 0, hidden = 0, num_topk = 0, num_experts = 0, tile_m = kTileM;
  int64_t seq = 0;
  int meta_epoch = 0, push_epoch = 0;
  int64_t slab_off[11] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0};   // byte offsets of the arrays inside meta_slab
  // sender side (regular device memory)
  at::Tensor sender_slab;
  at::Tensor pair_rank, pair_slot, token_rank_in_channel, send_recv_token, send_head, is_token_in_rank,
      channel_prefix_matrix, send_base, send_token_base, peer_total_tiles, peer_num_recv, send_order_base, send_list,
      num_send;
  // receiver side metadata (regular device memory)
  at::Tensor expert_frequency, expert_pool_block_offset, base_pool, seen_per_substream, rank_prefix_matrix,
      recv_channel_prefix_matrix, tile_id_to_expert, pool_arrival_target;
  // receiver side, written by peers (symmetric arena)
  at::Tensor meta_slab;
  at::Tensor pool, pool_topk_weight, pool_recv_token, pool_k_slot, pool_src, recv_token_to_slots, k_local_total,
      k_local_remaining, pool_arrival_count, recv_src, y_done_per_token, o;
  int total_tiles = 0, num_recv_tokens = 0;
  std::vector<int> recv_per_expert;
  std::optional<EventHandle> metadata_done_event;
  BufferRecord record{};
  std::vector<at::Tensor> aux_keepalive;
  // capacity mode (no host read of the sizes): the receive buffers are a fixed region of the arena
  int region_id = -1;                  // -1: exact mode
  at::Tensor dev_sizes;                // int32 [4] device: live total_tiles, live num_recv_tokens, overflow flag
  std::shared_ptr<void> region_guard;  // keeps the region claimed while this state (or a view of the region) lives

  void release_o() { o = at::Tensor(); }
  void release_pool() { pool = at::Tensor(); }
};

struct GradsState {
  at::Tensor dl_do_pool, bwd_dispatch_arrival_count, slab;
  at::Tensor landing, dwt;             // fused backward: landing rows [T * K, H] and per-pair dL/dweight [T, K] peers write
  int64_t landing_off = -1, dwt_off = -1;   // their arena offsets when they are fixed regions (capacity mode), else -1
  bool is_static = false;
  int epoch = 0;
  BufferRecord record{};
  std::optional<EventHandle> started_event;
};

struct CombineState {
  at::Tensor x_sym, done_sym, w_sym;   // arena-resident views/copies the peers read
  at::Tensor out, out_topk_weights;
  int epoch = 0;
  BufferRecord record{};
};

// Optional-tensor bag for the grouped GEMM launcher.
struct GemmArgs {
  int mode = kVarlenM, epilogue = kEpiStore, block_n = 256, num_ctas = 0;
  bool a_mn_major = false, b_mn_major = false;
  at::Tensor a, b;                                  // operands
  // VarlenK: a second problem (A2 [rows, M2], B2 [rows, N2] -> out2 [E, M2, N2]) multiplied in the same launch, and
  // dynamic tile claim (CTAs take the next tile from a counter instead of striding by the grid size)
  std::optional<at::Tensor> a2, b2, out2;
  bool dynamic_tiles = false;
  std::optional<at::Tensor> tile_id_to_expert, expert_pool_block_offset, expert_frequency;
  std::optional<at::Tensor> arrival_count, arrival_target;
  std::optional<at::Tensor> out0, out1, preact, row_weight, row_token, dl_dweight;
  std::optional<at::Tensor> scatter_local, row_src, row_k_slot;
  std::optional<at::Tensor> tile_stripes_done, k_remaining, done_per_token;
  // remote scatter / remote dL/dweight return: (record kind, epoch, word) naming the buffer on every rank
  std::vector<int> remote_out;
  std::vector<int> remote_dw;
  // capacity mode: the buffer sits at this arena offset on every rank (no record look-up); -1 = use the record
  int64_t remote_out_offset = -1, remote_dw_offset = -1;
  std::optional<at::Tensor> num_m_tiles_dev;        // VarlenM: live tile count in device memory (capacity mode)
  int num_topk = 0;
  int64_t seq = 0;
  int num_m_tiles = -1;                             // VarlenM: total tiles (defaults to len(tile_id_to_expert))
  int started_flag = -1;                            // index of the launch-gate flag to bump (-1 = none)
  bool tail = false; int tail_kind = kKindGemmYTail; bool tail_wait = true;
  std::shared_ptr<DispatchState> fused_push;        // dispatch fused into this GEMM (forward rows)
  std::shared_ptr<GradsState> fused_push_grads;     // dispatch_grads fused into this GEMM
  std::shared_ptr<DispatchState> fused_push_routing;
  at::Tensor fused_push_rows;
  int push_flags = 7;
};

// Fixed regions of the arena for the capacity mode of the fused layer.  Every rank builds the same plan with the
// same arguments right after constructing its runtime, so every region sits at the same arena offset on every
// rank and no buffer record has to be exchanged per dispatch.
struct StaticPlan {
  int num_regions = 0, hidden = 0, topk = 0;
  int64_t tokens_cap = 0, rows_cap = 0, tiles_cap = 0, recv_cap = 0;
  // byte offsets of the arrays inside one forward region
  size_t o_pool = 0, o_w = 0, o_rt = 0, o_ks = 0, o_src = 0, o_r2s = 0, o_klt = 0, o_klr = 0, o_cnt = 0, o_rsrc = 0, o_done = 0;
  size_t region_bytes = 0;
  size_t base_off = 0;                    // arena offset of the whole block
  std::vector<size_t> region_off;         // forward regions (one per layer whose forward state is alive)
  size_t bwd_pool_off[2] = {0, 0}, bwd_cnt_off[2] = {0, 0};   // backward: gradient pool + its tile counters
  size_t landing_off[2] = {0, 0};         // rows other ranks computed for this rank's tokens, [tokens_cap * topk, hidden]
  size_t dwt_off[2] = {0, 0};             // per-pair dL/dweight other ranks return, [tokens_cap, topk] fp32
  size_t total_bytes = 0;
  at::Tensor block;                       // owns the arena block
  std::mutex mu;
  std::vector<char> busy;
  uint64_t landing_calls = 0, bwd_calls = 0;
};

class Runtime {
 public:
  // `use_vmm`: take the arena from the virtual-memory-management API (shareable by file descriptor) instead of
  // cudaMalloc + CUDA IPC.
  Runtime(int rank, int num_ranks, int64_t arena_bytes, int num_channels, int num_experts_cap, int64_t timeout_ms,
          bool use_vmm = false)
      : rank_(rank), num_ranks_(num_ranks), num_channels_(num_channels), use_vmm_(use_vmm) {
    SEP_ASSERT(num_ranks >= 1 && num_ranks <= kMaxRanks, "1..8 ranks supported inside one NVSwitch domain");
    SEP_ASSERT(num_channels >= 1 && num_channels <= kMaxChannels, "num_channels out of range");
    SEP_ASSERT(num_experts_cap >= 1 && num_experts_cap <= kMaxExperts, "num_experts_cap out of range");
    SEP_CUDA_CHECK(cudaGetDevice(&device_));
    // Rows are pushed in chunks of this many (token, expert) pairs, each followed by the arrival signals of
    // the tiles it touched.  Small chunks let remote tiles complete progressively; with one rank only the
    // signalling overhead matters and larger chunks measured faster.
    pairs_per_chunk_ = num_ranks == 1 ? 16 : 8;
    // Several ranks (measured with the kernels' per-CTA time stamps): remote stores that wait for NVLink credit back
    // up in an SM's load/store path and starve the epilogue warps of the same SM, so a push spread over all SMs
    // slows the GEMM to a third while it lasts.  On 8 ranks, 28 SMs that only push (about 20 GB/s each) keep the
    // links busy while the other 120 multiply at their stand-alone rate (dispatch (+) GEMM-A 680 -> 570-590 us,
    // dispatch_grads (+) GEMM-Y_bwd 510 -> 435-460 us).  On 4 ranks the whole step measured 2.73-2.76 ms with 28
    // (and with 36) push-only CTAs against 2.84-2.86 ms with none, 2.79 ms with 20 and 2.80 ms with 44; on 2 ranks,
    // where half of the push stays local, the two ways measured the same and every CTA keeps doing both.  The send
    // list is walked tile by tile (order 1) and its first chunks are small: the consumers' first tiles complete after
    // ~30 us instead of ~130.
    if (num_ranks > 1) { push_order_ = 1; head_pairs_per_chunk_ = 2; head_chunks_ = 3000; }
    if (num_ranks > 2) push_ctas_ = 28;
    ctl_ = make_control_layout(num_ranks, num_channels, num_experts_cap);
    arena_bytes_ = static_cast<size_t>(arena_bytes) + ctl_.total_bytes;
    arena_bytes_ = (arena_bytes_ + (2u << 20) - 1) / (2u << 20) * (2u << 20);
    if (use_vmm_) {
      SEP_CUDA_CHECK(cudaFree(nullptr));     // make sure the primary context exists before driver calls
      CUmemAllocationProp prop{};
      prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
      prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE; prop.location.id = device_;
      prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
      size_t gran = 0;
      SEP_CU_CHECK(VmmApi::get().granularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
      arena_bytes_ = (arena_bytes_ + gran - 1) / gran * gran;
      own_range_.bytes = arena_bytes_;
      SEP_CU_CHECK(VmmApi::get().create(&own_range_.handle, arena_bytes_, &prop, 0));
      own_range_.map_for(device_);
      base_ = reinterpret_cast<void*>(own_range_.va);
    } else {
      SEP_CUDA_CHECK(cudaMalloc(&base_, arena_bytes_));
    }
    SEP_CUDA_CHECK(cudaMemset(base_, 0, ctl_.total_bytes));
    arena_ = std::make_shared<Arena>(ctl_.total_bytes, arena_bytes_ - ctl_.total_bytes);
    release_ctx_ = std::make_shared<ReleaseCtx>();
    release_ctx_->arena = arena_;
    release_ctx_->device = device_;
    for (int i = 0; i < kMaxRanks; ++i) peer_base_[i] = nullptr;
    peer_base_[rank] = base_;
    // device scratch: status block, launch-gate flags, launch-local counters
    SEP_CUDA_CHECK(cudaMalloc(&scratch_, 4096));
    SEP_CUDA_CHECK(cudaMemset(scratch_, 0, 4096));
    status_ = reinterpret_cast<StatusBlock*>(scratch_);
    gate_flags_ = reinterpret_cast<int*>(static_cast<char*>(scratch_) + 256);       // [8]
    counters_ = reinterpret_cast<int*>(static_cast<char*>(scratch_) + 512);          // [64]
    SEP_CUDA_CHECK(cudaHostAlloc(reinterpret_cast<void**>(&host_), sizeof(HostCounters), cudaHostAllocMapped));
    std::memset(reinterpret_cast<void*>(host_), 0, sizeof(HostCounters));
    host_->epoch = -1;
    SEP_CUDA_CHECK(cudaHostGetDevicePointer(reinterpret_cast<void**>(&host_dev_), host_, 0));
    set_timeout_ms(timeout_ms);
    for (int k = 0; k < kNumKinds; ++k) epochs_[k] = 0;
    for (int g = 0; g < 8; ++g) gate_issued_[g] = 0;
    SEP_CUDA_CHECK(cudaDeviceSynchronize());
  }

  ~Runtime() { destroy(); }

  void destroy() {
    if (destroyed_) return;
    destroyed_ = true;
    cudaDeviceSynchronize();
    if (release_ctx_) {
      { std::lock_guard<std::mutex> g(release_ctx_->mu); release_ctx_->dead = true; }
      arena_->sweep(true);
    }
    for (int i = 0; i < num_ranks_; ++i)
      if (i != rank_ && peer_base_[i] != nullptr && opened_[i]) {
        if (use_vmm_) peer_ranges_[i].destroy();
        else cudaIpcCloseMemHandle(peer_base_[i]);
      }
    // Tensors over arena blocks may outlive the runtime object; the slab itself is only freed when
    // the last of them is gone (they hold the shared arena, see alloc_symmetric).
    arena_guard_.reset();
    if (scratch_ != nullptr) cudaFree(scratch_);
    if (host_ != nullptr) cudaFreeHost(host_);
    if (host_overflow_ != nullptr) cudaFreeHost(host_overflow_);
    host_overflow_ = nullptr; static_.reset();
    scratch_ = nullptr; host_ = nullptr;
  }

  // ---- bootstrap ---------------------------------------------------------------------------
  int get_local_device_id() const { return device_; }
  py::bytes get_local_ipc_handle() const {
    cudaIpcMemHandle_t h;
    SEP_CUDA_CHECK(cudaIpcGetMemHandle(&h, base_));
    return py::bytes(reinterpret_cast<const char*>(&h), sizeof(h));
  }
  int64_t get_local_base_ptr() const { return reinterpret_cast<int64_t>(base_); }
  bool uses_vmm() const { return use_vmm_; }
  int64_t arena_total_bytes() const { return static_cast<int64_t>(arena_bytes_); }
  // VMM arena: a POSIX file descriptor for the physical allocation (the caller sends it to the peers and closes it).
  int export_vmm_fd() const {
    SEP_ASSERT(use_vmm_, "the arena was not allocated through the VMM API");
    int fd = -1;
    SEP_CU_CHECK(VmmApi::get().export_handle(&fd, own_range_.handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
    return fd;
  }
  // VMM arena, multi-process: import every peer's allocation from the descriptor received for it (fds[r]; own entry ignored).
  void sync_vmm(const std::vector<int>& fds, const std::vector<int64_t>& sizes) {
    SEP_ASSERT(use_vmm_ && static_cast<int>(fds.size()) == num_ranks_ && sizes.size() == fds.size(), "one descriptor and size per rank expected");
    for (int r = 0; r < num_ranks_; ++r) {
      if (r == rank_) continue;
      VmmRange& pr = peer_ranges_[r];
      pr.bytes = static_cast<size_t>(sizes[r]);
      SEP_CU_CHECK(VmmApi::get().import_handle(&pr.handle, reinterpret_cast<void*>(static_cast<uintptr_t>(fds[r])),
                                               CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR));
      pr.map_for(device_);
      peer_base_[r] = reinterpret_cast<void*>(pr.va);
      opened_[r] = true;
    }
    finish_sync();
  }

  // Multi-process: open every peer's IPC handle.  `handles[r]` is rank r's handle.
  void sync(const std::vector<int>& device_ids, const std::vector<std::optional<py::bytes>>& handles) {
    SEP_ASSERT(static_cast<int>(handles.size()) == num_ranks_, "one IPC handle per rank expected");
    for (int r = 0; r < num_ranks_; ++r) {
      if (r == rank_) continue;
      SEP_ASSERT(handles[r].has_value(), "missing IPC handle");
      std::string s = *handles[r];
      SEP_ASSERT(s.size() == sizeof(cudaIpcMemHandle_t), "malformed IPC handle");
      cudaIpcMemHandle_t h;
      std::memcpy(&h, s.data(), sizeof(h));
      SEP_CUDA_CHECK(cudaIpcOpenMemHandle(&peer_base_[r], h, cudaIpcMemLazyEnablePeerAccess));
      opened_[r] = true;
    }
    (void)device_ids;
    finish_sync();
  }
  // Single-process emulation of several ranks on one device: peers are plain pointers.
  void sync_local(const std::vector<int64_t>& base_ptrs) {
    SEP_ASSERT(static_cast<int>(base_ptrs.size()) == num_ranks_, "one base pointer per rank expected");
    for (int r = 0; r < num_ranks_; ++r) peer_base_[r] = reinterpret_cast<void*>(base_ptrs[r]);
    SEP_ASSERT(peer_base_[rank_] == base_, "own base pointer mismatch");
    finish_sync();
  }
  bool is_available() const { return available_; }

  // ---- misc ----------------------------------------------------------------------------------
  void set_timeout_ms(int64_t ms) { budget_ns_ = static_cast<unsigned long long>(std::max<int64_t>(ms, 1)) * 1000000ull; timeout_ms_ = ms; }
  int64_t get_timeout_ms() const { return timeout_ms_; }
  int rank() const { return rank_; }
  int num_ranks() const { return num_ranks_; }
  int num_channels() const { return num_channels_; }
  int64_t launch_count() const { return launches_; }
  // Event at the point of the current stream where the most recent backward left its last kernel that talks to
  // peers: what follows (the dW GEMMs) is local.  A host-to-device prefetch that waits on it stays clear of the
  // kernels that synchronise at system scope, which measured markedly slower while a PCIe copy was in flight.
  void mark_local_phase() { local_phase_ = std::make_shared<EventHandle>(stream()); }
  std::optional<EventHandle> local_phase_event() const { return local_phase_ ? std::optional<EventHandle>(*local_phase_) : std::nullopt; }
  // Per-CTA time stamps of the GEMM kernels (see GemmParams::timing).  Returns the tensor the launches that follow
  // fill: int64 [10, num_sms, 8], first index = epilogue kind (0 store, 1 SwiGLU, 2 scatter, 3 dSwiGLU, 4 fp32 store),
  // + 5 for the launches with a fused push.  Each launch overwrites the rows of its kind.  `on = false` stops it.
  at::Tensor set_kernel_timing(bool on) {
    if (!on) { timing_ = at::Tensor(); return timing_; }
    timing_ = at::zeros({10, num_sms(), kTimingCols}, at::TensorOptions().dtype(at::kLong).device(at::kCUDA, device_));
    return timing_;
  }
  void set_push_order(int n) { SEP_ASSERT(n == 0 || n == 1, "push order must be 0 or 1"); push_order_ = n; }
  void set_active_push_warps(int n) { SEP_ASSERT(n >= 0 && n <= 16, "active push warps must be 0..16"); active_push_warps_ = n; }
  // Fused dispatch + GEMM kernels: `n` CTAs only push (all their warps) and the rest only multiply; 0 = every CTA
  // does both (the default with one rank, where the push is a local copy).
  void set_push_ctas(int n) { SEP_ASSERT(n >= 0 && n < 128, "push CTAs out of range"); push_ctas_ = n; }
  int get_push_ctas() const { return push_ctas_; }
  // Push-only CTAs move rows with the bulk-copy engine (global -> shared -> owner's pool) instead of loads and stores.
  void set_bulk_push(bool on) { bulk_push_ = on; }
  // With push-only CTAs: they ship only the pairs that go to other ranks; the push warps of the GEMM CTAs ship the
  // pairs that stay on this rank (both walk the whole send list, each with its own claim counter).
  void set_split_local(bool on) { split_local_ = on; }
  // The first `chunks` chunks of every push carry `pairs` pairs each (0 chunks = off).
  void set_push_head(int pairs, int chunks) {
    SEP_ASSERT(pairs >= 1 && pairs <= 32 && chunks >= 0, "head chunks: 1..32 pairs, a non-negative count");
    head_pairs_per_chunk_ = pairs; head_chunks_ = chunks;
  }
  void set_pairs_per_chunk(int n) { SEP_ASSERT(n >= 1 && n <= 32, "pairs per chunk must be 1..32"); pairs_per_chunk_ = n; }
  // Blocks whose tensors died count as free here even while the arena still holds them back for queued work.
  int64_t arena_bytes_in_use() const { return static_cast<int64_t>(arena_->bytes_in_use()); }
  int64_t arena_blocks_parked() const { arena_->sweep(false); return static_cast<int64_t>(arena_->num_parked()); }
  int64_t arena_high_water() const { return static_cast<int64_t>(arena_->high_water()); }
  int64_t arena_capacity() const { return static_cast<int64_t>(arena_->capacity()); }

  // A tensor over a fresh arena block.  When the tensor dies the block is parked until everything queued so far on
  // the streams this runtime has used (launches and allocations) has completed, then returns to the arena: a
  // kernel that still reads or writes the block is never overtaken by the block's next owner.  Work on a stream
  // the runtime has never seen is not covered: make that stream wait for the tensor's last use, or keep a reference.
  at::Tensor alloc_symmetric(const std::vector<int64_t>& sizes, at::ScalarType dtype, bool zero, size_t* offset_out = nullptr) {
    int64_t n = 1;
    for (auto s : sizes) n *= s;
    const size_t bytes = static_cast<size_t>(n) * c10::elementSize(dtype);
    const size_t off = arena_->allocate(bytes);
    if (offset_out != nullptr) *offset_out = off;
    std::shared_ptr<ReleaseCtx> ctx = release_ctx_;
    std::shared_ptr<void> guard = arena_guard_;
    void* ptr = static_cast<char*>(base_) + off;
    auto t = at::from_blob(ptr, sizes, [ctx, guard, off](void*) { release_block(ctx, off); },
                           at::TensorOptions().dtype(dtype).device(at::kCUDA, device_));
    if (zero && bytes > 0) SEP_CUDA_CHECK(cudaMemsetAsync(ptr, 0, bytes, stream()));
    else stream();
    return t;
  }
  bool is_symmetric(const at::Tensor& t) const {
    const char* p = static_cast<const char*>(t.data_ptr());
    return t.is_cuda() && p >= static_cast<char*>(base_) && p < static_cast<char*>(base_) + arena_bytes_;
  }
  int64_t symmetric_offset(const at::Tensor& t) const {
    SEP_ASSERT(is_symmetric(t), "tensor does not live in the symmetric arena");
    return static_cast<const char*>(t.data_ptr()) - static_cast<char*>(base_);
  }

  // ---- capacity mode ---------------------------------------------------------------------------
  // Carves the fixed regions out of the arena.  Collective by convention: every rank calls it with the same
  // arguments at the same point of its allocation history; the returned arena offset must agree on all ranks
  // (the Python layer checks that).  `num_regions` = layers whose forward state is alive at the same time.
  int64_t enable_static(int num_regions, int64_t tokens_cap, int hidden, int topk, int64_t rows_cap, int64_t recv_cap) {
    SEP_ASSERT(!static_, "capacity mode is already enabled on this buffer");
    SEP_ASSERT(num_regions >= 1 && tokens_cap >= 1 && hidden % 8 == 0 && topk >= 1 && topk <= kMaxTopK, "bad capacity-mode arguments");
    SEP_ASSERT(rows_cap >= kTileM && rows_cap % kTileM == 0 && recv_cap >= 1, "rows_cap must be a positive multiple of 128, recv_cap positive");
    auto pl = std::make_shared<StaticPlan>();
    pl->num_regions = num_regions; pl->hidden = hidden; pl->topk = topk;
    pl->tokens_cap = tokens_cap; pl->rows_cap = rows_cap; pl->tiles_cap = rows_cap / kTileM; pl->recv_cap = recv_cap;
    auto al = [](size_t b) { return (b + 1023) / 1024 * 1024; };
    size_t off = 0;
    auto take = [&](size_t bytes) { size_t o = off; off += al(bytes); return o; };
    const size_t R = rows_cap, Tr = recv_cap, K = topk, H = hidden;
    pl->o_pool = take(R * H * 2); pl->o_w = take(R * 4); pl->o_rt = take(R * 4); pl->o_ks = take(R * 4); pl->o_src = take(R * 8);
    pl->o_r2s = take(Tr * K * 4); pl->o_klt = take(Tr * 4); pl->o_klr = take(Tr * 4); pl->o_cnt = take(pl->tiles_cap * 4);
    pl->o_rsrc = take(Tr * 8); pl->o_done = take(Tr * 8);
    pl->region_bytes = off;
    off = 0;
    for (int i = 0; i < num_regions; ++i) pl->region_off.push_back(take(pl->region_bytes));
    for (int i = 0; i < 2; ++i) { pl->bwd_pool_off[i] = take(R * H * 2); pl->bwd_cnt_off[i] = take(pl->tiles_cap * 4); }
    if (num_ranks_ > 1)
      for (int i = 0; i < 2; ++i) pl->landing_off[i] = take(static_cast<size_t>(tokens_cap) * K * H * 2);
    for (int i = 0; i < 2; ++i) pl->dwt_off[i] = take(static_cast<size_t>(tokens_cap) * K * 4);
    pl->total_bytes = off;
    size_t base = 0;
    pl->block = alloc_symmetric({static_cast<int64_t>(pl->total_bytes)}, at::kByte, false, &base);
    pl->base_off = base;
    for (auto& o : pl->region_off) o += base;
    for (int i = 0; i < 2; ++i) { pl->bwd_pool_off[i] += base; pl->bwd_cnt_off[i] += base; pl->landing_off[i] += base; pl->dwt_off[i] += base; }
    pl->busy.assign(num_regions, 0);
    // backward tile counters start at zero; later uses are re-zeroed at the end of the backward that used them
    for (int i = 0; i < 2; ++i)
      SEP_CUDA_CHECK(cudaMemsetAsync(static_cast<char*>(base_) + pl->bwd_cnt_off[i], 0, pl->tiles_cap * 4, stream()));
    SEP_CUDA_CHECK(cudaHostAlloc(reinterpret_cast<void**>(&host_overflow_), sizeof(HostOverflow), cudaHostAllocMapped));
    std::memset(reinterpret_cast<void*>(host_overflow_), 0, sizeof(HostOverflow));
    SEP_CUDA_CHECK(cudaHostGetDevicePointer(reinterpret_cast<void**>(&host_overflow_dev_), host_overflow_, 0));
    SEP_CUDA_CHECK(cudaStreamSynchronize(stream()));
    static_ = pl;
    return static_cast<int64_t>(base);
  }
  // After a failed collective the ranks may have made different numbers of calls: put the alternation of the
  // gradient / landing regions back to its start and re-zero the gradient tile counters.  Collective by convention
  // (Buffer.recover calls it on every rank after the device drained); regions still claimed by live handles stay so.
  void static_reset() {
    if (!static_) return;
    static_->landing_calls = 0; static_->bwd_calls = 0;
    for (int i = 0; i < 2; ++i)
      SEP_CUDA_CHECK(cudaMemsetAsync(static_cast<char*>(base_) + static_->bwd_cnt_off[i], 0, static_->tiles_cap * 4, stream()));
    SEP_CUDA_CHECK(cudaStreamSynchronize(stream()));
  }
  bool static_enabled() const { return static_ != nullptr; }
  // True when a dispatch of this shape can use the fixed regions.
  bool static_fits(int64_t tokens, int hidden, int topk) const {
    return static_ && tokens <= static_->tokens_cap && hidden == static_->hidden && topk == static_->topk;
  }
  std::vector<int64_t> static_capacity() const {
    if (!static_) return {};
    return {static_->num_regions, static_->tokens_cap, static_->rows_cap, static_->recv_cap, static_cast<int64_t>(static_->total_bytes)};
  }
  // {count of overflowed dispatches, epoch of the last one, tiles it needed, recv tokens it needed}; no device sync.
  std::vector<int64_t> overflow_info() const {
    if (host_overflow_ == nullptr) return {0, 0, 0, 0};
    return {host_overflow_->count, host_overflow_->epoch, host_overflow_->needed_tiles, host_overflow_->needed_recv};
  }
  // A non-owning tensor over a fixed region; `guard` (may be null) rides along in its deleter.
  at::Tensor region_view(size_t off, const std::vector<int64_t>& sizes, at::ScalarType dtype, std::shared_ptr<void> guard) {
    at::Tensor keep = static_->block;
    return at::from_blob(static_cast<char*>(base_) + off, sizes, [keep, guard](void*) {},
                         at::TensorOptions().dtype(dtype).device(at::kCUDA, device_));
  }
  // The landing buffer of the next fused GEMM (+) combine on this rank: two alternate.  A buffer is written by
  // peers during call c and read here right after; its next writers (call c + 2) have by then passed the
  // all-rank completion handshake of call c + 1, which this rank only joins after its read of call c.
  std::pair<at::Tensor, int64_t> next_landing(int64_t tokens, int hidden, int topk) {
    SEP_ASSERT(static_fits(tokens, hidden, topk), "shape does not fit the capacity-mode regions");
    if (num_ranks_ == 1) return {at::empty({0, hidden}, at::TensorOptions().dtype(at::kBFloat16).device(at::kCUDA, device_)), 0};
    const size_t off = static_->landing_off[static_->landing_calls++ & 1];
    return {region_view(off, {tokens * topk, static_cast<int64_t>(hidden)}, at::kBFloat16, nullptr), static_cast<int64_t>(off)};
  }

  // ---- status --------------------------------------------------------------------------------
  // Reads the device status block (synchronises the device). Returns an empty string when clean.
  std::string poll_status(bool reset) {
    SEP_CUDA_CHECK(cudaDeviceSynchronize());
    StatusBlock h;
    SEP_CUDA_CHECK(cudaMemcpy(&h, status_, sizeof(h), cudaMemcpyDeviceToHost));
    if (h.code == 0 && h.abort == 0) return "";
    if (reset) SEP_CUDA_CHECK(cudaMemset(status_, 0, sizeof(StatusBlock)));
    static const char* names[] = {"ok", "barrier timeout", "buffer-record timeout", "tile gate timeout",
                                  "token gate timeout", "GEMM pipeline timeout", "tail wait timeout", "bad index",
                                  "capacity overflow (where = region, expected = tile capacity, observed = tiles needed; the dispatch was run as an empty one)",
                                  "ranks disagree on the capacity-mode region of a dispatch"};
    std::ostringstream os;
    os << names[(h.code >= 0 && h.code < 10) ? h.code : 0] << " (code " << h.code << ") in kernel " << h.kernel_id
       << " role " << h.role << " on rank " << h.rank << ": where=" << h.where << " expected=" << h.expected
       << " observed=" << h.observed;
    return os.str();
  }

  // ---- launch gates (reference: csrc/stream_ep.cpp:387-456) -----------------------------------
  // gate ids: 0 dispatch_main, 1 dispatch_grads, 2 kernel_y, 3 kernel_a_bwd
  void gate_wait_started(int gate, int64_t raw_stream) {
    static StreamWaitValue32Fn wait_fn = driver_fn<StreamWaitValue32Fn>("cuStreamWaitValue32");
    if (gate_issued_[gate] == 0) return;
    CUresult r = wait_fn(reinterpret_cast<CUstream>(raw_stream), reinterpret_cast<CUdeviceptr>(gate_flags_ + gate),
                         static_cast<cuuint32_t>(gate_issued_[gate]), CU_STREAM_WAIT_VALUE_GEQ);
    if (r != CUDA_SUCCESS) throw std::runtime_error("streamep_b200: cuStreamWaitValue32 failed with code " + std::to_string(r));
  }
  void gate_bump_issued(int gate) { ++gate_issued_[gate]; }
  at::Tensor gate_flag_tensor(int gate) {
    return at::from_blob(gate_flags_ + gate, {1}, at::TensorOptions().dtype(at::kInt).device(at::kCUDA, device_));
  }

  // ---- dispatch: phase 0, inputs + sender-side scratch ----------------------------------------
  // `capacity_mode`: receive into a fixed region (enable_static) instead of exactly sized fresh buffers.
  std::shared_ptr<DispatchState> dispatch_begin(const at::Tensor& x, const at::Tensor& topk_idx,
                                                const at::Tensor& topk_weights, int num_experts, int tile_m,
                                                int64_t seq, bool capacity_mode = false) {
    SEP_ASSERT(available_, "Buffer.sync has not completed");
    SEP_ASSERT(x.is_cuda() && x.dim() == 2 && x.is_contiguous() && x.scalar_type() == at::kBFloat16, "x must be a contiguous [T, H] bf16 CUDA tensor");
    SEP_ASSERT(topk_idx.dim() == 2 && topk_idx.is_contiguous() && topk_idx.scalar_type() == at::kLong, "topk_idx must be contiguous [T, K] int64");
    SEP_ASSERT(topk_weights.sizes() == topk_idx.sizes() && topk_weights.is_contiguous() && topk_weights.scalar_type() == at::kFloat, "topk_weights must be contiguous [T, K] float32");
    SEP_ASSERT(x.size(0) == topk_idx.size(0), "x and topk_idx disagree on the token count");
    SEP_ASSERT(tile_m == kTileM, "tile_m must be 128 (one tcgen05 M tile)");
    SEP_ASSERT(num_experts % num_ranks_ == 0 && num_experts <= ctl_.num_experts_cap, "num_experts must divide by the rank count and fit the Buffer's expert capacity");
    SEP_ASSERT(x.size(1) % 8 == 0, "hidden must be a multiple of 8");
    SEP_ASSERT(topk_idx.size(1) <= kMaxTopK, "num_topk too large");
    auto st = std::make_shared<DispatchState>();
    st->x = x; st->topk_idx = topk_idx; st->topk_weights = topk_weights;
    st->num_tokens = x.size(0); st->hidden = x.size(1); st->num_topk = topk_idx.size(1);
    st->num_experts = num_experts; st->tile_m = tile_m; st->seq = seq;
    st->meta_epoch = ++epochs_[kKindMetadata];
    const int64_t T = st->num_tokens, K = st->num_topk, R = num_ranks_, C = num_channels_, E = num_experts, EL = E / R;
    // One int32 slab for all small tensors (each torch::empty costs microseconds on the host).
    const int64_t tiles_cap = capacity_mode ? static_->tiles_cap : 0;
    if (capacity_mode) SEP_ASSERT(static_fits(T, st->hidden, st->num_topk), "this dispatch does not fit the capacity-mode regions (tokens, hidden or top-k differ)");
    const int64_t n_i32 = T * K * 3 + T * R * 3 + (T * R + 3) / 4 + R * C + 2 * C * E + C * R + 2 * R + EL + (EL + 1) +
                          2 * C * R * EL + R * R + R * C + 2 * tiles_cap + 104;
    st->sender_slab = at::empty({n_i32}, x.options().dtype(at::kInt));
    int64_t off = 0;
    auto take = [&](std::vector<int64_t> shape) {
      int64_t n = 1; for (auto s : shape) n *= s;
      auto t = st->sender_slab.narrow(0, off, n).view(shape);
      off += (n + 3) / 4 * 4;
      return t;
    };
    st->pair_rank = take({T, K}); st->pair_slot = take({T, K});
    st->token_rank_in_channel = take({T, R}); st->send_recv_token = take({T, R}); st->send_head = take({T, R});
    st->is_token_in_rank = take({(T * R + 3) / 4}).view(at::kBool).narrow(0, 0, T * R).view({T, R});
    st->channel_prefix_matrix = take({R, C}); st->send_base = take({C, E}); st->send_token_base = take({C, R});
    st->peer_total_tiles = take({R}); st->peer_num_recv = take({R});
    st->send_order_base = take({C, E}); st->send_list = take({T * K}); st->num_send = take({1});
    st->expert_frequency = take({EL}); st->expert_pool_block_offset = take({EL + 1});
    st->base_pool = take({C, R, EL}); st->seen_per_substream = take({C, R, EL});
    st->rank_prefix_matrix = take({R, R}); st->recv_channel_prefix_matrix = take({R, C});
    if (capacity_mode) {
      st->tile_id_to_expert = take({tiles_cap}); st->pool_arrival_target = take({tiles_cap});
      st->dev_sizes = take({4});
      // claim the lowest free region: ranks that run the same program pick the same one (the metadata kernel checks)
      std::shared_ptr<StaticPlan> pl = static_;
      int id = -1;
      {
        std::lock_guard<std::mutex> g(pl->mu);
        for (int i = 0; i < pl->num_regions && id < 0; ++i) if (!pl->busy[i]) { pl->busy[i] = 1; id = i; }
      }
      SEP_ASSERT(id >= 0, "every capacity-mode region is in use: enable capacity mode with as many regions as layers keep forward state alive");
      st->region_id = id;
      st->region_guard = std::shared_ptr<void>(nullptr, [pl, id](void*) { std::lock_guard<std::mutex> g(pl->mu); pl->busy[id] = 0; });
    }
    SEP_ASSERT(off <= n_i32, "sender slab overflow");
    return st;
  }

  // ---- dispatch: phase 1, metadata kernel ------------------------------------------------------
  void dispatch_metadata(const std::shared_ptr<DispatchState>& st, int phase_mask) {
    MetadataParams p{};
    p.topk_idx = st->topk_idx.data_ptr<int64_t>() ? reinterpret_cast<const long long*>(st->topk_idx.data_ptr<int64_t>()) : nullptr;
    p.num_tokens = st->num_tokens; p.num_topk = st->num_topk; p.num_experts = st->num_experts;
    p.num_ranks = num_ranks_; p.rank = rank_; p.num_channels = num_channels_; p.tile_m = st->tile_m;
    p.epoch = st->meta_epoch; p.phase_mask = phase_mask; p.push_order = push_order_;
    fill_peers(p.peer_base); p.ctl = ctl_;
    p.pair_rank = st->pair_rank.data_ptr<int>(); p.pair_slot = st->pair_slot.data_ptr<int>();
    p.token_rank_in_channel = st->token_rank_in_channel.data_ptr<int>();
    p.send_recv_token = st->send_recv_token.data_ptr<int>(); p.send_head = st->send_head.data_ptr<int>();
    p.is_token_in_rank = reinterpret_cast<unsigned char*>(st->is_token_in_rank.data_ptr<bool>());
    p.channel_prefix_matrix = st->channel_prefix_matrix.data_ptr<int>();
    p.send_base = st->send_base.data_ptr<int>(); p.send_token_base = st->send_token_base.data_ptr<int>();
    p.send_order_base = st->send_order_base.data_ptr<int>(); p.send_list = st->send_list.data_ptr<int>();
    p.num_send = st->num_send.data_ptr<int>();
    p.peer_total_tiles = st->peer_total_tiles.data_ptr<int>(); p.peer_num_recv = st->peer_num_recv.data_ptr<int>();
    p.expert_frequency = st->expert_frequency.data_ptr<int>();
    p.expert_pool_block_offset = st->expert_pool_block_offset.data_ptr<int>();
    p.base_pool = st->base_pool.data_ptr<int>(); p.seen_per_substream = st->seen_per_substream.data_ptr<int>();
    p.rank_prefix_matrix = st->rank_prefix_matrix.data_ptr<int>();
    p.recv_channel_prefix_matrix = st->recv_channel_prefix_matrix.data_ptr<int>();
    p.blocks_done = counters_ + 0;
    p.host = host_dev_; p.status = status_; p.wait_budget_ns = budget_ns_;
    p.region_id = st->region_id;
    if (st->region_id >= 0) {
      const StaticPlan& pl = *static_;
      p.tiles_cap = static_cast<int>(pl.tiles_cap); p.recv_cap = static_cast<int>(pl.recv_cap);
      p.dev_sizes = st->dev_sizes.data_ptr<int>();
      p.tile_id_to_expert = st->tile_id_to_expert.data_ptr<int>(); p.pool_arrival_target = st->pool_arrival_target.data_ptr<int>();
      p.host_overflow = host_overflow_dev_;
      if (phase_mask & 1) {
        // Defaults of everything peers write into this region, for the whole capacity (a few MB of small arrays),
        // BEFORE this rank's count exchange: a peer pushes only after it has seen this rank's exchange flag.
        char* rb = static_cast<char*>(base_) + pl.region_off[st->region_id];
        FillParams f{};
        f.total_tiles = p.tiles_cap; f.tile_m = st->tile_m; f.num_local_experts = st->num_experts / num_ranks_;
        f.tk_padded = static_cast<int>(pl.rows_cap); f.num_recv_tokens = p.recv_cap; f.num_topk = st->num_topk;
        f.pool_topk_weight = reinterpret_cast<float*>(rb + pl.o_w); f.pool_recv_token = reinterpret_cast<int*>(rb + pl.o_rt);
        f.pool_k_slot = reinterpret_cast<int*>(rb + pl.o_ks); f.pool_src = reinterpret_cast<int2*>(rb + pl.o_src);
        f.recv_token_to_slots = reinterpret_cast<int*>(rb + pl.o_r2s); f.k_local_total = reinterpret_cast<int*>(rb + pl.o_klt);
        f.k_local_remaining = reinterpret_cast<int*>(rb + pl.o_klr); f.pool_arrival_count = reinterpret_cast<int*>(rb + pl.o_cnt);
        f.recv_src = reinterpret_cast<int2*>(rb + pl.o_rsrc); f.y_done_per_token = reinterpret_cast<long long*>(rb + pl.o_done);
        ++launches_; launch_fill_tile_metadata(f, stream());
      }
    }
    ++launches_; launch_dispatch_metadata(p, stream());
    SEP_CUDA_CHECK(cudaGetLastError());
  }

  // ---- dispatch: phase 2, host poll + receiver allocation + defaults --------------------------
  // `need_o`: allocate and zero the per-recv-token accumulator `o` (the fused layer combines in the GEMM epilogue
  // and does not use it).  `defer_views`: create only the tensors the first GEMM launch needs; the caller
  // creates the rest with dispatch_finish_views() once that launch is queued, off the GPU's critical path.
  void dispatch_allocate(const std::shared_ptr<DispatchState>& st, bool need_o = true, bool defer_views = false) {
    if (st->region_id >= 0) { dispatch_allocate_static(st, need_o); return; }
    // The metadata kernel writes the sizes to mapped pinned memory; the epoch word goes last.
    const auto t0 = std::chrono::steady_clock::now();
    bool timed_out = false;
    {
      py::gil_scoped_release nogil;
      unsigned spins = 0;
      while (host_->epoch != st->meta_epoch) {
        if ((++spins & 0x3FFu) != 0) continue;
        const auto dt = std::chrono::steady_clock::now() - t0;
        // the kernel's own waits give up after timeout_ms and then publish an error marker; the
        // extra margin only covers a kernel that never got to run
        if (std::chrono::duration_cast<std::chrono::milliseconds>(dt).count() > 2 * timeout_ms_ + 5000) { timed_out = true; break; }
      }
    }
    if (timed_out)
      throw std::runtime_error("streamep_b200: timed out waiting for dispatch metadata on rank " + std::to_string(rank_) +
                               " (did every rank call dispatch?)");
    std::atomic_thread_fence(std::memory_order_acquire);
    st->total_tiles = host_->total_tiles;
    st->num_recv_tokens = host_->num_recv_tokens;
    if (st->total_tiles < 0) {
      std::string why = poll_status(true);
      throw std::runtime_error("streamep_b200: dispatch metadata failed on rank " + std::to_string(rank_) + ": " + why);
    }
    const int EL = st->num_experts / num_ranks_;
    st->recv_per_expert.resize(EL);
    for (int e = 0; e < EL; ++e) st->recv_per_expert[e] = host_->recv_per_expert[e];

    const int64_t tiles = st->total_tiles, TKp = tiles * st->tile_m, Tr = st->num_recv_tokens, K = st->num_topk, H = st->hidden;
    auto opts = st->x.options();
    st->tile_id_to_expert = at::empty({tiles * 2}, opts.dtype(at::kInt));
    st->pool_arrival_target = st->tile_id_to_expert.narrow(0, tiles, tiles);
    st->tile_id_to_expert = st->tile_id_to_expert.narrow(0, 0, tiles);
    size_t off_pool = 0, off_slab = 0;   // empty tensors report a null data pointer, so offsets are tracked here
    st->pool = alloc_symmetric({TKp, H}, at::kBFloat16, false, &off_pool);
    st->o = need_o ? alloc_symmetric({Tr, H}, at::kBFloat16, true) : at::empty({0, H}, opts);
    // one arena block for everything small that peers write
    auto al = [](int64_t b) { return (b + 255) / 256 * 256; };
    const int64_t b_w = al(TKp * 4), b_rt = al(TKp * 4), b_ks = al(TKp * 4), b_src = al(TKp * 8), b_r2s = al(Tr * K * 4),
                  b_klt = al(Tr * 4), b_klr = al(Tr * 4), b_cnt = al(tiles * 4), b_rsrc = al(Tr * 8), b_done = al(Tr * 8);
    st->meta_slab = alloc_symmetric({b_w + b_rt + b_ks + b_src + b_r2s + b_klt + b_klr + b_cnt + b_rsrc + b_done}, at::kByte, false, &off_slab);
    const int64_t sizes[10] = {b_w, b_rt, b_ks, b_src, b_r2s, b_klt, b_klr, b_cnt, b_rsrc, b_done};
    st->slab_off[0] = 0;
    for (int i = 0; i < 10; ++i) st->slab_off[i + 1] = st->slab_off[i] + sizes[i];
    unsigned long long sub_off[10];
    for (int i = 0; i < 10; ++i) sub_off[i] = off_slab + st->slab_off[i];
    st->pool_arrival_count = slab_view(*st, 7);
    if (!defer_views) dispatch_finish_views(st);

    char* sb = st->meta_slab.numel() ? static_cast<char*>(st->meta_slab.data_ptr()) : nullptr;
    auto at_off = [&](int i) { return sb ? sb + st->slab_off[i] : nullptr; };
    FillParams f{};
    f.total_tiles = tiles; f.tile_m = st->tile_m; f.num_local_experts = EL; f.tk_padded = TKp; f.num_recv_tokens = Tr; f.num_topk = K;
    f.expert_frequency = st->expert_frequency.data_ptr<int>();
    f.expert_pool_block_offset = st->expert_pool_block_offset.data_ptr<int>();
    f.tile_id_to_expert = st->tile_id_to_expert.data_ptr<int>(); f.pool_arrival_target = st->pool_arrival_target.data_ptr<int>();
    f.pool_topk_weight = reinterpret_cast<float*>(at_off(0));
    f.pool_recv_token = reinterpret_cast<int*>(at_off(1)); f.pool_k_slot = reinterpret_cast<int*>(at_off(2));
    f.pool_src = reinterpret_cast<int2*>(at_off(3));
    f.recv_token_to_slots = reinterpret_cast<int*>(at_off(4)); f.k_local_total = reinterpret_cast<int*>(at_off(5));
    f.k_local_remaining = reinterpret_cast<int*>(at_off(6));
    f.pool_arrival_count = reinterpret_cast<int*>(at_off(7));
    f.recv_src = reinterpret_cast<int2*>(at_off(8));
    f.y_done_per_token = reinterpret_cast<long long*>(at_off(9));
    ++launches_; launch_fill_tile_metadata(f, stream());
    SEP_CUDA_CHECK(cudaGetLastError());

    BufferRecord& r = st->record;
    r.pool = off_pool; r.pool_topk_weight = sub_off[0]; r.pool_recv_token = sub_off[1]; r.pool_k_slot = sub_off[2];
    r.pool_src = sub_off[3]; r.recv_token_to_slots = sub_off[4]; r.k_local_total = sub_off[5];
    r.k_local_remaining = sub_off[6]; r.arrival_count = sub_off[7]; r.recv_src = sub_off[8];
    st->push_epoch = ++epochs_[kKindDispatch];
    st->metadata_done_event = EventHandle(stream());
  }

  // Capacity mode: no host read.  The handle's tensors are views of the whole region (`total_tiles`, `TK_padded`
  // and `num_recv_tokens` are the capacities); the live counts stay on the device in `dev_sizes`.
  void dispatch_allocate_static(const std::shared_ptr<DispatchState>& st, bool need_o) {
    const StaticPlan& pl = *static_;
    const size_t ro = pl.region_off[st->region_id];
    const int64_t R = pl.rows_cap, Tr = pl.recv_cap, K = st->num_topk, H = st->hidden, tiles = pl.tiles_cap;
    st->total_tiles = static_cast<int>(tiles); st->num_recv_tokens = static_cast<int>(Tr);
    st->recv_per_expert.clear();
    auto g = st->region_guard;
    st->pool = region_view(ro + pl.o_pool, {R, H}, at::kBFloat16, g);
    st->pool_topk_weight = region_view(ro + pl.o_w, {R}, at::kFloat, g);
    st->pool_recv_token = region_view(ro + pl.o_rt, {R}, at::kInt, g);
    st->pool_k_slot = region_view(ro + pl.o_ks, {R}, at::kInt, g);
    st->pool_src = region_view(ro + pl.o_src, {R, 2}, at::kInt, g);
    st->recv_token_to_slots = region_view(ro + pl.o_r2s, {Tr, K}, at::kInt, g);
    st->k_local_total = region_view(ro + pl.o_klt, {Tr}, at::kInt, g);
    st->k_local_remaining = region_view(ro + pl.o_klr, {Tr}, at::kInt, g);
    st->pool_arrival_count = region_view(ro + pl.o_cnt, {tiles}, at::kInt, g);
    st->recv_src = region_view(ro + pl.o_rsrc, {Tr, 2}, at::kInt, g);
    st->y_done_per_token = region_view(ro + pl.o_done, {Tr}, at::kLong, g);
    st->o = need_o ? alloc_symmetric({Tr, H}, at::kBFloat16, true) : at::empty({0, H}, st->x.options());
    BufferRecord& r = st->record;
    r.pool = ro + pl.o_pool; r.pool_topk_weight = ro + pl.o_w; r.pool_recv_token = ro + pl.o_rt; r.pool_k_slot = ro + pl.o_ks;
    r.pool_src = ro + pl.o_src; r.recv_token_to_slots = ro + pl.o_r2s; r.k_local_total = ro + pl.o_klt;
    r.k_local_remaining = ro + pl.o_klr; r.arrival_count = ro + pl.o_cnt; r.recv_src = ro + pl.o_rsrc;
    st->push_epoch = ++epochs_[kKindDispatch];
    st->metadata_done_event = EventHandle(stream());
  }

  // The i-th array of the per-dispatch slab (order: pool_topk_weight, pool_recv_token, pool_k_slot, pool_src,
  // recv_token_to_slots, k_local_total, k_local_remaining, pool_arrival_count, recv_src, y_done_per_token).
  at::Tensor slab_view(const DispatchState& st, int i) const {
    const int64_t tiles = st.total_tiles, TKp = tiles * st.tile_m, Tr = st.num_recv_tokens, K = st.num_topk;
    const int64_t used[10] = {TKp * 4, TKp * 4, TKp * 4, TKp * 8, Tr * K * 4, Tr * 4, Tr * 4, tiles * 4, Tr * 8, Tr * 8};
    const at::ScalarType dt[10] = {at::kFloat, at::kInt, at::kInt, at::kInt, at::kInt, at::kInt, at::kInt, at::kInt, at::kInt, at::kLong};
    auto t = st.meta_slab.narrow(0, st.slab_off[i], used[i]).view(dt[i]);
    if (i == 3) return t.view({TKp, 2});
    if (i == 4) return t.view({Tr, K});
    if (i == 8) return t.view({Tr, 2});
    return t;
  }
  void dispatch_finish_views(const std::shared_ptr<DispatchState>& st) {
    st->pool_topk_weight = slab_view(*st, 0); st->pool_recv_token = slab_view(*st, 1); st->pool_k_slot = slab_view(*st, 2);
    st->pool_src = slab_view(*st, 3); st->recv_token_to_slots = slab_view(*st, 4); st->k_local_total = slab_view(*st, 5);
    st->k_local_remaining = slab_view(*st, 6); st->recv_src = slab_view(*st, 8); st->y_done_per_token = slab_view(*st, 9);
  }

  // Extra words of the dispatch record: arena tensors of this rank that peers address by (rank, row),
  // e.g. the [T, H] output accumulator the fused combine reduces into.
  void dispatch_set_aux(const std::shared_ptr<DispatchState>& st, int i, const at::Tensor& t) {
    SEP_ASSERT(i >= 0 && i < 5, "aux index out of range");
    (&st->record.aux0)[i] = t.numel() ? symmetric_offset(t) : 0;
    st->aux_keepalive.push_back(t);
  }
  void grads_set_aux(const std::shared_ptr<GradsState>& g, int i, const at::Tensor& t) {
    SEP_ASSERT(i >= 0 && i < 5, "aux index out of range");
    (&g->record.aux0)[i] = t.numel() ? symmetric_offset(t) : 0;
  }

  PushParams make_push_params(const DispatchState& st, const at::Tensor& rows, bool is_grads, const BufferRecord& rec,
                              int kind, int epoch, int flags, const int* own_count, int counter_base) {
    PushParams p{};
    p.x = rows.data_ptr();
    p.topk_idx = reinterpret_cast<const long long*>(st.topk_idx.data_ptr<int64_t>());
    p.topk_weights = st.topk_weights.data_ptr<float>();
    p.pair_slot = st.pair_slot.data_ptr<int>();
    p.send_recv_token = st.send_recv_token.data_ptr<int>();
    p.send_list = st.send_list.data_ptr<int>(); p.num_send = st.num_send.data_ptr<int>();
    p.num_tokens = st.num_tokens; p.hidden = st.hidden; p.num_topk = st.num_topk; p.num_experts = st.num_experts;
    p.num_ranks = num_ranks_; p.rank = rank_; p.tile_m = st.tile_m;
    p.is_grads = is_grads ? 1 : 0; p.kind = kind; p.epoch = epoch; p.flags = flags;
    p.pairs_per_chunk = pairs_per_chunk_; p.active_push_warps = active_push_warps_;
    p.head_pairs_per_chunk = head_pairs_per_chunk_; p.head_chunks = head_chunks_;
    p.push_ctas = push_ctas_; p.bulk_push = bulk_push_ ? 1 : 0;
    p.split_local = split_local_ ? 1 : 0; p.work_counter_local = counters_ + 12 + (is_grads ? 1 : 0);
    fill_peers(p.peer_base); p.ctl = ctl_; p.own = rec;
    p.static_targets = st.region_id >= 0 ? 1 : 0;   // (a backward along a capacity-mode forward uses fixed regions too)
    p.own_arrival_count = own_count; p.own_arrival_target = st.pool_arrival_target.data_ptr<int>();
    p.own_total_tiles = st.total_tiles;
    p.started_flag = gate_flags_ + (is_grads ? 1 : 0);
    p.work_counter = counters_ + counter_base; p.blocks_done = counters_ + counter_base + 1;
    p.status = status_; p.wait_budget_ns = budget_ns_;
    return p;
  }

  // ---- dispatch: phase 3, push -----------------------------------------------------------------
  void dispatch_push(const std::shared_ptr<DispatchState>& st, int flags, int num_blocks) {
    PushParams p = make_push_params(*st, st->x, false, st->record, kKindDispatch, st->push_epoch, flags,
                                    st->pool_arrival_count.data_ptr<int>(), 2);
    if (flags & 2) ++gate_issued_[0];
    ++launches_; launch_dispatch_push(p, num_blocks, stream());
    SEP_CUDA_CHECK(cudaGetLastError());
  }

  // ---- dispatch_grads --------------------------------------------------------------------------
  // `fused_buffers`: also provide the landing rows and the per-pair dL/dweight matrix of the fused backward.
  std::shared_ptr<GradsState> grads_begin(const std::shared_ptr<DispatchState>& st, bool fused_buffers = false) {
    auto g = std::make_shared<GradsState>();
    const int64_t tiles = st->total_tiles, TKp = tiles * st->tile_m, T = st->num_tokens, K = st->num_topk, H = st->hidden;
    size_t off_pool = 0, off_cnt = 0;
    if (st->region_id >= 0) {
      // Capacity mode: two fixed gradient regions alternate.  A region used by backward call b is written again by
      // peers in call b + 2, after they passed the completion handshake of call b + 1, which this rank joins only
      // after everything of call b (dW GEMMs reading the gradient pool, the re-zeroing of the counters) is queued.
      StaticPlan& pl = *static_;
      const int par = static_cast<int>(pl.bwd_calls++ & 1);
      g->is_static = true;
      off_pool = pl.bwd_pool_off[par]; off_cnt = pl.bwd_cnt_off[par];
      g->dl_do_pool = region_view(off_pool, {TKp, H}, at::kBFloat16, nullptr);
      g->bwd_dispatch_arrival_count = region_view(off_cnt, {tiles}, at::kInt, nullptr);
      if (fused_buffers) {
        auto lo = next_landing(T, st->hidden, st->num_topk);
        g->landing = lo.first; g->landing_off = lo.second;
        g->dwt_off = static_cast<int64_t>(pl.dwt_off[par]);
        g->dwt = region_view(pl.dwt_off[par], {T, K}, at::kFloat, nullptr);
      }
    } else {
      g->dl_do_pool = alloc_symmetric({TKp, H}, at::kBFloat16, false, &off_pool);
      g->bwd_dispatch_arrival_count = alloc_symmetric({tiles}, at::kInt, true, &off_cnt);
      if (fused_buffers) {
        g->landing = alloc_symmetric({num_ranks_ > 1 ? T * K : 0, H}, at::kBFloat16, false);
        g->dwt = alloc_symmetric({T, K}, at::kFloat, true);
      }
    }
    g->record = BufferRecord{};
    g->record.pool = off_pool;
    g->record.arrival_count = off_cnt;
    if (fused_buffers && !g->is_static) {
      g->record.aux0 = g->landing.numel() ? symmetric_offset(g->landing) : 0;
      g->record.aux1 = g->dwt.numel() ? symmetric_offset(g->dwt) : 0;
    }
    g->epoch = ++epochs_[kKindDispatchGrads];
    g->started_event = EventHandle(stream());
    return g;
  }
  // Capacity mode, end of a backward: the gradient tile counters go back to zero for the call after next.  Queue it
  // behind the kernel that ends with the all-rank completion handshake (A_bwd), i.e. after every rank's push.
  void grads_finish(const std::shared_ptr<GradsState>& g) {
    if (!g->is_static || g->bwd_dispatch_arrival_count.numel() == 0) return;
    SEP_CUDA_CHECK(cudaMemsetAsync(g->bwd_dispatch_arrival_count.data_ptr(), 0, g->bwd_dispatch_arrival_count.nbytes(), stream()));
  }
  void grads_push(const std::shared_ptr<DispatchState>& st, const std::shared_ptr<GradsState>& g, const at::Tensor& dl_dy,
                  int flags, int num_blocks) {
    SEP_ASSERT(dl_dy.is_cuda() && dl_dy.is_contiguous() && dl_dy.scalar_type() == at::kBFloat16 && dl_dy.dim() == 2 &&
               dl_dy.size(0) == st->num_tokens && dl_dy.size(1) == st->hidden, "dL_dy must be contiguous [T, H] bf16");
    PushParams p = make_push_params(*st, dl_dy, true, g->record, kKindDispatchGrads, g->epoch, flags,
                                    g->bwd_dispatch_arrival_count.data_ptr<int>(), 4);
    if (flags & 2) ++gate_issued_[1];
    ++launches_; launch_dispatch_push(p, num_blocks, stream());
    SEP_CUDA_CHECK(cudaGetLastError());
  }

  // ---- combine / combine_grads -------------------------------------------------------------------
  std::shared_ptr<CombineState> combine_begin(const std::shared_ptr<DispatchState>& st, const at::Tensor& x,
                                              const at::Tensor& done, const std::optional<at::Tensor>& weights, bool is_fwd) {
    SEP_ASSERT(x.is_cuda() && x.is_contiguous() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 &&
               x.size(0) == st->num_recv_tokens && x.size(1) == st->hidden, "combine input must be contiguous [T_recv, H] bf16");
    SEP_ASSERT(done.scalar_type() == at::kLong && done.numel() == st->num_recv_tokens, "gate must be int64 [T_recv]");
    auto c = std::make_shared<CombineState>();
    auto stream = this->stream();
    // Peers read these through NVLink, so they must sit in the arena.  Tensors the caller already
    // keeps there (handle.o, handle.y_done_per_token, Buffer.alloc_symmetric results) are used in
    // place, which is what lets the gate be written while this kernel runs.
    auto to_sym = [&](const at::Tensor& t) {
      if (t.numel() == 0 || is_symmetric(t)) return t;
      auto s = alloc_symmetric(t.sizes().vec(), t.scalar_type(), false);
      if (t.numel() > 0) SEP_CUDA_CHECK(cudaMemcpyAsync(s.data_ptr(), t.data_ptr(), t.nbytes(), cudaMemcpyDeviceToDevice, stream));
      return s;
    };
    c->x_sym = to_sym(x);
    c->done_sym = to_sym(done);
    c->record = BufferRecord{};
    c->record.aux0 = x.numel() ? symmetric_offset(c->x_sym) : 0;
    c->record.aux1 = done.numel() ? symmetric_offset(c->done_sym) : 0;
    if (!is_fwd) {
      SEP_ASSERT(weights.has_value() && weights->scalar_type() == at::kFloat && weights->is_contiguous(), "combine_grads needs fp32 per-slot weight grads");
      c->w_sym = to_sym(*weights);
      c->record.aux2 = weights->numel() ? symmetric_offset(c->w_sym) : 0;
    }
    c->out = at::empty({static_cast<int64_t>(st->num_tokens), static_cast<int64_t>(st->hidden)}, x.options());
    if (!is_fwd) c->out_topk_weights = at::empty({static_cast<int64_t>(st->num_tokens), static_cast<int64_t>(st->num_topk)}, x.options().dtype(at::kFloat));
    c->epoch = ++epochs_[is_fwd ? kKindCombine : kKindCombineGrads];
    return c;
  }
  void combine_launch(const std::shared_ptr<DispatchState>& st, const std::shared_ptr<CombineState>& c, bool is_fwd,
                      int64_t seq, int flags, int num_blocks) {
    CombineParams p{};
    p.num_tokens = st->num_tokens; p.hidden = st->hidden; p.num_topk = st->num_topk; p.num_ranks = num_ranks_;
    p.rank = rank_; p.num_experts = st->num_experts; p.is_fwd = is_fwd ? 1 : 0; p.seq = seq;
    p.kind = is_fwd ? kKindCombine : kKindCombineGrads; p.epoch = c->epoch; p.flags = flags;
    p.send_recv_token = st->send_recv_token.data_ptr<int>(); p.pair_slot = st->pair_slot.data_ptr<int>();
    p.topk_idx = reinterpret_cast<const long long*>(st->topk_idx.data_ptr<int64_t>());
    p.out = c->out.data_ptr(); p.out_topk_weights = is_fwd ? nullptr : c->out_topk_weights.data_ptr<float>();
    fill_peers(p.peer_base); p.ctl = ctl_; p.own = c->record;
    p.blocks_done = counters_ + (is_fwd ? 6 : 7);
    p.status = status_; p.wait_budget_ns = budget_ns_;
    ++launches_; launch_combine_pull(p, num_blocks, stream());
    SEP_CUDA_CHECK(cudaGetLastError());
  }

  // ---- barrier ------------------------------------------------------------------------------------
  void barrier() {
    BarrierParams p{};
    p.num_ranks = num_ranks_; p.rank = rank_; p.epoch = ++epochs_[kKindBarrier]; p.kind = kKindBarrier; p.wait = 1;
    fill_peers(p.peer_base); p.ctl = ctl_; p.status = status_; p.wait_budget_ns = budget_ns_;
    ++launches_; launch_device_barrier(p, stream());
    SEP_CUDA_CHECK(cudaGetLastError());
  }
  // Emulated ranks run one after another on one device: a barrier there is "every rank bumped its
  // epoch and stored its flags", with nobody waiting.
  int next_epoch(int kind) { return ++epochs_[kind]; }
  std::vector<int> get_epochs() const { return std::vector<int>(epochs_, epochs_ + kNumKinds); }
  void set_epochs(const std::vector<int>& e) {
    SEP_ASSERT(static_cast<int>(e.size()) == kNumKinds, "one epoch per operation kind expected");
    for (int k = 0; k < kNumKinds; ++k) epochs_[k] = e[k];
  }

  // ---- grouped GEMM ---------------------------------------------------------------------------------
  void grouped_gemm(const GemmArgs& a) {
    SEP_ASSERT(a.a.is_cuda() && a.a.scalar_type() == at::kBFloat16 && a.a.is_contiguous(), "GEMM operand A must be contiguous bf16");
    SEP_ASSERT(a.b.is_cuda() && a.b.scalar_type() == at::kBFloat16 && a.b.is_contiguous(), "GEMM operand B must be contiguous bf16");
    SEP_ASSERT(a.block_n == 128 || a.block_n == 256, "block_n must be 128 or 256");
    GemmParams p{};
    p.mode = a.mode; p.epilogue = a.epilogue; p.block_n = a.block_n;
    p.a_mn_major = a.a_mn_major; p.b_mn_major = a.b_mn_major;
    p.rank = rank_; p.status = status_; p.wait_budget_ns = budget_ns_;
    CUtensorMap ta, tb, to0, to1, maps2[3];
    bool have_o0 = false, have_o1 = false, have_maps2 = false;
    const int BN = a.block_n;
    if (a.mode == kVarlenM) {
      // A: [rows, K] row-major; B: weights [E, N, K] (K-major) or [E, K, N] (MN-major)
      SEP_ASSERT(a.a.dim() == 2 && a.b.dim() == 3 && a.tile_id_to_expert.has_value(), "varlen-M GEMM needs A [rows, K], B [E, ., .] and tile_id_to_expert");
      const int64_t rows = a.a.size(0), K = a.a.size(1), E = a.b.size(0);
      const int64_t N = a.b_mn_major ? a.b.size(2) : a.b.size(1);
      SEP_ASSERT((a.b_mn_major ? a.b.size(1) : a.b.size(2)) == K, "GEMM reduction lengths disagree");
      SEP_ASSERT(K % 8 == 0 && N % 8 == 0, "K and N must be multiples of 8");
      p.N = N; p.K = K; p.num_experts = E; p.total_rows = rows;
      p.num_m_tiles = a.num_m_tiles >= 0 ? a.num_m_tiles : a.tile_id_to_expert->numel();
      // (the fp32-store epilogue guards rows itself: its last tile may hang over the end of A, TMA zero-fills it)
      SEP_ASSERT(static_cast<int64_t>(p.num_m_tiles) * BM_ <= rows || a.epilogue == kEpiStoreF32, "tile list longer than A");
      p.num_n_tiles = (N + BN - 1) / BN;
      p.tile_id_to_expert = a.tile_id_to_expert->data_ptr<int>();
      if (a.num_m_tiles_dev.has_value()) p.num_m_tiles_dev = a.num_m_tiles_dev->data_ptr<int>();
      if (rows == 0) { launch_without_tiles(a); return; }
      ta = make_tmap(a.a.data_ptr(), K, rows, 1, K, rows * K, 64, BM_);
      if (a.b_mn_major) tb = make_tmap(a.b.data_ptr(), N, K, E, N, K * N, 64, 64);
      else tb = make_tmap(a.b.data_ptr(), K, N, E, K, N * K, 64, BN);
    } else {
      // dW: A [rows, M], B [rows, N] row-major; out [E, M, N]
      SEP_ASSERT(a.a.dim() == 2 && a.b.dim() == 2 && a.a.size(0) == a.b.size(0), "varlen-K GEMM needs A [rows, M] and B [rows, N]");
      SEP_ASSERT(a.a_mn_major && a.b_mn_major && a.epilogue == kEpiStore, "varlen-K GEMM is MN-major x MN-major with the store epilogue");
      SEP_ASSERT(a.expert_pool_block_offset.has_value() && a.expert_frequency.has_value() && a.out0.has_value(), "varlen-K GEMM needs expert offsets, true lengths and an output");
      const int64_t rows = a.a.size(0), M = a.a.size(1), N = a.b.size(1), E = a.expert_frequency->numel();
      SEP_ASSERT(M % 8 == 0 && N % 8 == 0, "M and N must be multiples of 8");
      p.N = N; p.M_out = M; p.num_experts = E; p.total_rows = rows;
      p.num_m_tiles = (M + BM_ - 1) / BM_; p.num_n_tiles = (N + BN - 1) / BN;
      p.expert_pool_block_offset = a.expert_pool_block_offset->data_ptr<int>();
      p.expert_frequency = a.expert_frequency->data_ptr<int>();
      p.out_expert_stride = M * N;
      if (a.a2.has_value()) {
        SEP_ASSERT(a.b2.has_value() && a.out2.has_value() && a.a2->dim() == 2 && a.b2->dim() == 2 && a.a2->size(0) == rows &&
                   a.b2->size(0) == rows && a.a2->is_contiguous() && a.b2->is_contiguous() &&
                   a.a2->scalar_type() == at::kBFloat16 && a.b2->scalar_type() == at::kBFloat16,
                   "the second varlen-K problem needs contiguous bf16 A2 [rows, M2], B2 [rows, N2] over the same rows, and an output");
        const int64_t M2 = a.a2->size(1), N2 = a.b2->size(1);
        SEP_ASSERT(M2 % 8 == 0 && N2 % 8 == 0, "M2 and N2 must be multiples of 8");
        p.N2 = N2; p.M_out2 = M2; p.num_m_tiles2 = (M2 + BM_ - 1) / BM_; p.num_n_tiles2 = (N2 + BN - 1) / BN;
      }
      if (rows == 0) { a.out0->zero_(); if (a.out2.has_value()) a.out2->zero_(); return; }
      ta = make_tmap(a.a.data_ptr(), M, rows, 1, M, rows * M, 64, 64);
      tb = make_tmap(a.b.data_ptr(), N, rows, 1, N, rows * N, 64, 64);
      if (a.a2.has_value()) {
        maps2[0] = make_tmap(a.a2->data_ptr(), p.M_out2, rows, 1, p.M_out2, rows * p.M_out2, 64, 64);
        maps2[1] = make_tmap(a.b2->data_ptr(), p.N2, rows, 1, p.N2, rows * p.N2, 64, 64);
        have_maps2 = true;
      }
      if (a.dynamic_tiles) p.tile_counter = counters_ + 10;
    }
    if (a.arrival_count.has_value()) {
      SEP_ASSERT(a.arrival_target.has_value(), "arrival_count needs arrival_target");
      p.arrival_count = a.arrival_count->data_ptr<int>(); p.arrival_target = a.arrival_target->data_ptr<int>();
    }
    if (a.started_flag >= 0) p.started_flag = gate_flags_ + a.started_flag;
    auto ld = [](const at::Tensor& t) { return t.dim() >= 2 ? t.stride(t.dim() - 2) : t.numel(); };
    if (a.out0.has_value()) { p.out0 = a.out0->data_ptr(); p.ld0 = ld(*a.out0); }
    if (a.out1.has_value()) { p.out1 = a.out1->data_ptr(); p.ld1 = ld(*a.out1); }
    if (a.preact.has_value()) { p.preact = a.preact->data_ptr(); p.ld_preact = ld(*a.preact); }
    if (a.row_weight.has_value()) p.row_weight = a.row_weight->data_ptr<float>();
    if (a.row_token.has_value()) p.row_token = a.row_token->data_ptr<int>();
    if (a.dl_dweight.has_value()) p.dl_dweight = a.dl_dweight->data_ptr<float>();
    if (a.scatter_local.has_value()) p.scatter_local = a.scatter_local->data_ptr();
    if (a.row_src.has_value()) p.row_src = reinterpret_cast<const int2*>(a.row_src->data_ptr<int>());
    if (a.row_k_slot.has_value()) p.row_k_slot = a.row_k_slot->data_ptr<int>();
    if (a.tile_stripes_done.has_value()) p.tile_stripes_done = a.tile_stripes_done->data_ptr<int>();
    if (a.k_remaining.has_value()) p.k_remaining = a.k_remaining->data_ptr<int>();
    if (a.done_per_token.has_value()) p.done_per_token = reinterpret_cast<long long*>(a.done_per_token->data_ptr<int64_t>());
    p.seq = a.seq; p.num_topk = a.num_topk;
    if (timing_.defined()) {
      // one block of rows per kind of launch: epilogue index, +5 when a push is fused in; 5 = row-tiled store (preact
      // recompute, as opposed to dW in 0), 7 = scatter with an MN-major B (A_bwd, as opposed to Y in 2)
      int kind = a.epilogue + ((a.fused_push || a.fused_push_grads) ? 5 : 0);
      if (a.epilogue == kEpiStore && a.mode == kVarlenM) kind = 5;
      if (a.epilogue == kEpiScatter && a.b_mn_major) kind = 7;
      p.timing = reinterpret_cast<long long*>(timing_.data_ptr<int64_t>()) + static_cast<int64_t>(kind) * num_sms() * kTimingCols;
    }
    p.num_ranks = num_ranks_; fill_peers(p.peer_base); p.ctl = ctl_;
    auto set_ref = [](RemoteRef& r, const std::vector<int>& v) {
      if (v.empty()) return;
      SEP_ASSERT(v.size() == 3 && v[2] >= 0 && v[2] < kMailboxWords - 1, "remote reference must be (kind, epoch, word)");
      r.enabled = 1; r.kind = v[0]; r.epoch = v[1]; r.field = v[2];
    };
    set_ref(p.remote_out, a.remote_out);
    set_ref(p.remote_dw, a.remote_dw);
    if (a.remote_out_offset >= 0) { p.remote_out.enabled = 1; p.remote_out.is_static = 1; p.remote_out.offset = a.remote_out_offset; }
    if (a.remote_dw_offset >= 0) { p.remote_dw.enabled = 1; p.remote_dw.is_static = 1; p.remote_dw.offset = a.remote_dw_offset; }
    if (a.epilogue == kEpiScatter || a.epilogue == kEpiDswiglu) SEP_ASSERT(p.row_token != nullptr, "this epilogue needs pool_recv_token");
    if (a.epilogue == kEpiScatter) {
      SEP_ASSERT(a.scatter_local.has_value(), "scatter needs a local destination");   // may be empty (a rank without tokens)
      if (p.remote_out.enabled)
        SEP_ASSERT(p.row_src != nullptr && p.row_k_slot != nullptr && p.num_topk > 0, "remote scatter needs pool_src, pool_k_slot and num_topk");
    }
    if (a.epilogue == kEpiDswiglu) {
      SEP_ASSERT(p.preact != nullptr && p.out0 != nullptr && p.out1 != nullptr, "dswiglu epilogue needs preact and both outputs");
      if (p.remote_dw.enabled)
        SEP_ASSERT(p.row_src != nullptr && p.row_k_slot != nullptr && p.tile_stripes_done != nullptr && p.dl_dweight != nullptr,
                   "dL/dweight return needs pool_src, pool_k_slot, stripe counters and dl_dweight");
    }
    if (a.epilogue == kEpiSwiglu || a.epilogue == kEpiStore || a.epilogue == kEpiStoreF32) SEP_ASSERT(p.out0 != nullptr, "this epilogue needs out0");
    if (a.epilogue == kEpiStoreF32) SEP_ASSERT(a.out0->scalar_type() == at::kFloat && p.ld0 % 4 == 0, "the fp32 store epilogue writes float rows of a multiple of 4 elements");
    if (a.tail) {
      p.tail.enabled = 1; p.tail.kind = a.tail_kind; p.tail.epoch = ++epochs_[a.tail_kind];
      p.tail.wait = a.tail_wait ? 1 : 0;
      p.tail.ctas_done = counters_ + (a.tail_kind == kKindGemmYTail ? 8 : 9);
    }
    // Output maps of the TMA-store epilogues: one box = 32 rows x one staging row.
    auto out_map = [&](const at::Tensor& t, int64_t cols, int64_t rows, int64_t experts, uint32_t box_cols, CUtensorMapSwizzle sw) {
      SEP_ASSERT(t.scalar_type() == at::kBFloat16 && t.stride(-1) == 1, "GEMM outputs must be bf16 with contiguous rows");
      const int64_t ld = t.dim() >= 2 ? t.stride(-2) : cols;
      SEP_ASSERT(ld % 8 == 0 && cols % 8 == 0, "GEMM output rows must be multiples of 16 bytes");
      return make_tmap(t.data_ptr(), cols, rows, experts, ld, experts > 1 ? t.stride(0) : rows * ld, box_cols, 32, sw);
    };
    if (a.epilogue == kEpiStore) {
      if (a.mode == kVarlenM) to0 = out_map(*a.out0, p.N, p.total_rows, 1, 32, CU_TENSOR_MAP_SWIZZLE_64B);
      else to0 = out_map(*a.out0, p.N, p.M_out, p.num_experts, 32, CU_TENSOR_MAP_SWIZZLE_64B);
      have_o0 = true;
      if (have_maps2) maps2[2] = out_map(*a.out2, p.N2, p.M_out2, p.num_experts, 32, CU_TENSOR_MAP_SWIZZLE_64B);
    } else if (a.epilogue == kEpiSwiglu) {
      SEP_ASSERT(p.N % 16 == 0, "SwiGLU epilogue needs an output width that is a multiple of 16");
      to0 = out_map(*a.out0, p.N / 2, p.total_rows, 1, 16, CU_TENSOR_MAP_SWIZZLE_32B); have_o0 = true;
      if (a.out1.has_value()) { to1 = out_map(*a.out1, p.N, p.total_rows, 1, 32, CU_TENSOR_MAP_SWIZZLE_64B); have_o1 = true; }
    } else if (a.epilogue == kEpiDswiglu) {
      to0 = out_map(*a.out0, 2 * static_cast<int64_t>(p.N), p.total_rows, 1, 64, CU_TENSOR_MAP_SWIZZLE_128B); have_o0 = true;
      to1 = out_map(*a.out1, p.N, p.total_rows, 1, 32, CU_TENSOR_MAP_SWIZZLE_64B); have_o1 = true;
    }
    int n_ctas = a.num_ctas > 0 ? a.num_ctas : num_sms();
    const int64_t total = a.mode == kVarlenM ? static_cast<int64_t>(p.num_m_tiles) * p.num_n_tiles
        : static_cast<int64_t>(p.num_experts) * (static_cast<int64_t>(p.num_m_tiles) * p.num_n_tiles + static_cast<int64_t>(p.num_m_tiles2) * p.num_n_tiles2);
    PushParams pp{};
    const PushParams* ppp = nullptr;
    if (a.fused_push) {
      pp = make_push_params(*a.fused_push, a.fused_push->x, false, a.fused_push->record, kKindDispatch,
                            a.fused_push->push_epoch, a.push_flags, a.fused_push->pool_arrival_count.data_ptr<int>(), 2);
      pp.started_flag = nullptr;
      ppp = &pp;
    } else if (a.fused_push_grads) {
      SEP_ASSERT(a.fused_push_routing && a.fused_push_rows.defined(), "fused dispatch_grads needs the forward routing and dL_dy");
      pp = make_push_params(*a.fused_push_routing, a.fused_push_rows, true, a.fused_push_grads->record, kKindDispatchGrads,
                            a.fused_push_grads->epoch, a.push_flags, a.fused_push_grads->bwd_dispatch_arrival_count.data_ptr<int>(), 4);
      pp.started_flag = nullptr;
      ppp = &pp;
    }
    if (ppp == nullptr) n_ctas = static_cast<int>(std::min<int64_t>(n_ctas, std::max<int64_t>(total, 1)));
    if (n_ctas > num_sms()) p.timing = nullptr;   // the stamp tensor has one row per SM
    ++launches_;
    cudaError_t setup_error = cudaSuccess;
    const bool launched = launch_grouped_gemm(p, &ta, &tb, have_o0 ? &to0 : nullptr, have_o1 ? &to1 : nullptr, ppp, n_ctas,
                                              stream(), &setup_error, have_maps2 ? maps2 : nullptr);
    SEP_ASSERT(launched, "no grouped GEMM kernel for this combination of mode, operand layouts, epilogue and fused push");
    SEP_CUDA_CHECK(setup_error);
    SEP_CUDA_CHECK(cudaGetLastError());
  }

  // A rank that received no rows has nothing to multiply, but it still takes part in the collective
  // halves of the fused kernels: its own rows must be pushed and its completion flags raised.
  void launch_without_tiles(const GemmArgs& a) {
    auto stream = this->stream();
    if (a.fused_push) {
      PushParams pp = make_push_params(*a.fused_push, a.fused_push->x, false, a.fused_push->record, kKindDispatch,
                                       a.fused_push->push_epoch, a.push_flags & 3, a.fused_push->pool_arrival_count.data_ptr<int>(), 2);
      pp.started_flag = nullptr;
      ++launches_; launch_dispatch_push(pp, num_sms(), stream);
    } else if (a.fused_push_grads) {
      PushParams pp = make_push_params(*a.fused_push_routing, a.fused_push_rows, true, a.fused_push_grads->record, kKindDispatchGrads,
                                       a.fused_push_grads->epoch, a.push_flags & 3, a.fused_push_grads->bwd_dispatch_arrival_count.data_ptr<int>(), 4);
      pp.started_flag = nullptr;
      ++launches_; launch_dispatch_push(pp, num_sms(), stream);
    }
    if (a.tail) {
      BarrierParams b{};
      b.num_ranks = num_ranks_; b.rank = rank_; b.kind = a.tail_kind; b.epoch = ++epochs_[a.tail_kind]; b.wait = a.tail_wait ? 1 : 0;
      fill_peers(b.peer_base); b.ctl = ctl_; b.status = status_; b.wait_budget_ns = budget_ns_;
      ++launches_; launch_device_barrier(b, stream);
    }
    SEP_CUDA_CHECK(cudaGetLastError());
  }

  // ---- whole fused forward after the metadata launch, in one native call ----------------------------------
  // The host must read the receive sizes before it can size the pool, so the GPU has nothing queued while
  // the host works between that read and the first GEMM launch.  Doing every step of that stretch here
  // (allocation, fill, three launches) instead of ~25 Python-level calls keeps the idle gap short.
  // Returns {out, postact, preact (may be undefined)}.
  std::vector<at::Tensor> fused_forward(const std::shared_ptr<DispatchState>& st, const at::Tensor& w1, const at::Tensor& w2,
                                        const at::Tensor& landing_in, bool store_preact, int tile_n_a, int tile_n_y,
                                        int num_sms_a, int num_sms_y) {
    // Queued behind the metadata kernel, so the output is zeroed while the host waits for the sizes.
    auto opts = st->x.options();
    const bool cap = st->region_id >= 0;
    at::Tensor out = at::zeros({static_cast<int64_t>(st->num_tokens), w2.size(1)}, opts);
    dispatch_allocate(st, /*need_o=*/false, /*defer_views=*/true);
    at::Tensor landing = landing_in;
    int64_t landing_off = -1;
    if (cap) {          // fixed landing region, the same offset on every rank: no record word needed
      auto lo = next_landing(st->num_tokens, st->hidden, st->num_topk);
      landing = lo.first; landing_off = lo.second;
    } else {
      dispatch_set_aux(st, 0, landing);
    }
    const int64_t TKp = static_cast<int64_t>(st->total_tiles) * st->tile_m, I = w2.size(2);
    at::Tensor postact = at::empty({TKp, I}, opts);
    at::Tensor preact = store_preact ? at::empty({TKp, 2 * I}, opts) : at::Tensor();
    GemmArgs a;
    a.mode = kVarlenM; a.epilogue = kEpiSwiglu; a.block_n = tile_n_a; a.num_ctas = num_sms_a;
    a.a = st->pool; a.b = w1; a.tile_id_to_expert = st->tile_id_to_expert;
    a.out0 = postact; if (store_preact) a.out1 = preact;
    a.arrival_count = st->pool_arrival_count; a.arrival_target = st->pool_arrival_target;
    a.fused_push = st; a.push_flags = 3;
    if (cap) a.num_m_tiles_dev = st->dev_sizes;
    grouped_gemm(a);
    if (!cap) dispatch_finish_views(st);          // host work in the shadow of kernel A
    GemmArgs y;
    y.mode = kVarlenM; y.epilogue = kEpiScatter; y.block_n = tile_n_y; y.num_ctas = num_sms_y;
    y.a = postact; y.b = w2; y.tile_id_to_expert = st->tile_id_to_expert;
    y.row_weight = st->pool_topk_weight; y.row_token = st->pool_recv_token; y.scatter_local = out;
    if (cap) { y.remote_out_offset = landing_off; y.num_m_tiles_dev = st->dev_sizes; }
    else y.remote_out = {kKindDispatch, st->push_epoch, 10};
    y.row_src = st->pool_src; y.row_k_slot = st->pool_k_slot; y.num_topk = st->num_topk;
    y.tail = true; y.tail_kind = kKindGemmYTail; y.tail_wait = true;
    grouped_gemm(y);
    combine_reduce(out, landing, st->topk_idx, st->num_experts, std::nullopt, std::nullopt,
                   cap ? std::optional<at::Tensor>(st->dev_sizes) : std::nullopt);
    return {out, postact, preact};
  }

  // Whole fused backward in one native call (same reason as fused_forward: every host microsecond between
  // two launches is a microsecond in which a slow host holds back all ranks at the next collective).
  // `rows_saved` is the pool (checkpoint levels 0/1) or the compact per-recv-token rows (level 2).
  // Returns {dL_dx, dL_dtopk_weights, dW1, dW2}.
  std::vector<at::Tensor> fused_backward(const std::shared_ptr<DispatchState>& st, const at::Tensor& dl_dy, const at::Tensor& w1,
                                         const at::Tensor& w2, const at::Tensor& rows_saved, const std::optional<at::Tensor>& preact_saved,
                                         int level, int tile_n_a, int tile_n_y_bwd, int tile_n_a_bwd, int tile_n_dw1, int tile_n_dw2,
                                         int num_sms_y_bwd, int num_sms_a_bwd) {
    const int64_t tiles = st->total_tiles, TKp = tiles * st->tile_m, T = st->num_tokens, K = st->num_topk;
    const int64_t H = w2.size(1), I = w2.size(2);
    const bool cap = st->region_id >= 0;
    auto opts = st->x.options();
    at::Tensor dswiglu_in = at::empty({TKp, 2 * I}, opts), postact_dw2 = at::empty({TKp, I}, opts);
    at::Tensor dW1 = at::empty_like(w1), dW2 = at::empty_like(w2);
    const int64_t nt = std::max<int64_t>(tiles, 1);
    at::Tensor zeros = at::zeros({nt + TKp}, opts.dtype(at::kInt));
    at::Tensor stripes = zeros.narrow(0, 0, nt), dl_dweight = zeros.narrow(0, nt, TKp).view(at::kFloat);
    at::Tensor dx = at::zeros({T, H}, opts);
    auto g = grads_begin(st, /*fused_buffers=*/true);
    at::Tensor pool = rows_saved;
    if (level == 2) pool = TKp > 0 ? pool_expand(rows_saved, st->pool_recv_token, TKp) : at::empty({0, H}, opts);
    at::Tensor preact;
    if (preact_saved.has_value() && preact_saved->defined()) {
      preact = *preact_saved;
    } else {
      preact = at::empty({TKp, 2 * I}, opts);
      if (tiles > 0) {
        GemmArgs r;
        r.mode = kVarlenM; r.epilogue = kEpiStore; r.block_n = tile_n_a;
        r.a = pool; r.b = w1; r.tile_id_to_expert = st->tile_id_to_expert; r.out0 = preact;
        if (cap) r.num_m_tiles_dev = st->dev_sizes;
        grouped_gemm(r);
      }
    }
    GemmArgs y;
    y.mode = kVarlenM; y.epilogue = kEpiDswiglu; y.block_n = tile_n_y_bwd; y.b_mn_major = true; y.num_ctas = num_sms_y_bwd;
    y.a = g->dl_do_pool; y.b = w2; y.tile_id_to_expert = st->tile_id_to_expert;
    y.preact = preact; y.out0 = dswiglu_in; y.out1 = postact_dw2;
    y.row_weight = st->pool_topk_weight; y.row_token = st->pool_recv_token; y.dl_dweight = dl_dweight;
    y.arrival_count = g->bwd_dispatch_arrival_count; y.arrival_target = st->pool_arrival_target;
    if (cap) { y.remote_dw_offset = g->dwt_off; y.num_m_tiles_dev = st->dev_sizes; }
    else y.remote_dw = {kKindDispatchGrads, g->epoch, 11};
    y.row_src = st->pool_src; y.row_k_slot = st->pool_k_slot; y.num_topk = static_cast<int>(K); y.tile_stripes_done = stripes;
    y.fused_push_grads = g; y.fused_push_routing = st; y.fused_push_rows = dl_dy; y.push_flags = 3;
    grouped_gemm(y);
    GemmArgs a;
    a.mode = kVarlenM; a.epilogue = kEpiScatter; a.block_n = tile_n_a_bwd; a.b_mn_major = true; a.num_ctas = num_sms_a_bwd;
    a.a = dswiglu_in; a.b = w1; a.tile_id_to_expert = st->tile_id_to_expert;
    a.row_token = st->pool_recv_token; a.scatter_local = dx;
    if (cap) { a.remote_out_offset = g->landing_off; a.num_m_tiles_dev = st->dev_sizes; }
    else a.remote_out = {kKindDispatchGrads, g->epoch, 10};
    a.row_src = st->pool_src; a.row_k_slot = st->pool_k_slot; a.num_topk = static_cast<int>(K);
    a.tail = true; a.tail_kind = kKindGemmABwdTail; a.tail_wait = true;
    grouped_gemm(a);
    at::Tensor dwt = g->dwt;
    if (cap) {
      // the per-pair dL/dweight landed in a fixed region that the call after next reuses: copy it out (with zeros
      // for skipped pairs) in the same pass that folds the landed rows into dx
      dwt = at::empty({T, K}, opts.dtype(at::kFloat));
      combine_reduce(dx, g->landing, st->topk_idx, st->num_experts, g->dwt, dwt, st->dev_sizes);
      grads_finish(g);
    } else {
      combine_reduce(dx, g->landing, st->topk_idx, st->num_experts);
    }
    mark_local_phase();
    if (tiles > 0) {
      // dW1 and dW2 in one launch, tiles claimed dynamically: one tail instead of two, and experts of unequal row
      // counts (tiles of unequal length) balance out.  dW1 first: its tiles are the longer ones (K = rows, N = H).
      GemmArgs d;
      d.mode = kVarlenK; d.epilogue = kEpiStore; d.a_mn_major = d.b_mn_major = true; d.dynamic_tiles = true;
      d.expert_pool_block_offset = st->expert_pool_block_offset; d.expert_frequency = st->expert_frequency;
      if (tile_n_dw1 == tile_n_dw2) {
        d.block_n = tile_n_dw1;
        d.a = dswiglu_in; d.b = pool; d.out0 = dW1;
        d.a2 = g->dl_do_pool; d.b2 = postact_dw2; d.out2 = dW2;
        grouped_gemm(d);
      } else {
        d.block_n = tile_n_dw2; d.a = g->dl_do_pool; d.b = postact_dw2; d.out0 = dW2;
        grouped_gemm(d);
        d.block_n = tile_n_dw1; d.a = dswiglu_in; d.b = pool; d.out0 = dW1;
        grouped_gemm(d);
      }
    } else {
      dW1.zero_(); dW2.zero_();
    }
    return {dx, dwt, dW1, dW2};
  }

  // ---- small ops ---------------------------------------------------------------------------------------
  void tile_producer(const at::Tensor& count, const at::Tensor& target, double delay_us) {
    ++launches_; launch_tile_producer(count.data_ptr<int>(), target.data_ptr<int>(), count.numel(), static_cast<long long>(delay_us * 1000.0),
                         stream());
    SEP_CUDA_CHECK(cudaGetLastError());
  }
  // `dw_src` / `dw_dst`: also copy the per-pair scalars peers stored in `dw_src` [T, K] to `dw_dst` (0 for skipped
  // pairs).  `sizes` (capacity mode): the dispatch's device-side sizes; when its overflow flag is set the dispatch ran
  // empty and the landed rows are stale, so `out` is left as it is (zeros).
  void combine_reduce(const at::Tensor& out, const at::Tensor& rows, const at::Tensor& topk_idx, int num_experts,
                      const std::optional<at::Tensor>& dw_src = std::nullopt, const std::optional<at::Tensor>& dw_dst = std::nullopt,
                      const std::optional<at::Tensor>& sizes = std::nullopt) {
    SEP_ASSERT(out.is_contiguous() && out.scalar_type() == at::kBFloat16 && out.dim() == 2 && out.size(1) % 8 == 0, "out must be contiguous [T, H] bf16");
    SEP_ASSERT(topk_idx.scalar_type() == at::kLong && topk_idx.is_contiguous() && topk_idx.size(0) == out.size(0), "topk_idx must be contiguous [T, K] int64");
    const bool copy_dw = dw_dst.has_value() && dw_dst->defined();
    if (out.size(0) == 0 || (num_ranks_ == 1 && !copy_dw)) return;
    if (num_ranks_ > 1) SEP_ASSERT(rows.numel() == out.size(0) * topk_idx.size(1) * out.size(1), "rows must be [T * K, H]");
    if (copy_dw) SEP_ASSERT(dw_src.has_value() && dw_src->scalar_type() == at::kFloat && dw_dst->scalar_type() == at::kFloat &&
                            dw_src->numel() == topk_idx.numel() && dw_dst->numel() == topk_idx.numel() && topk_idx.size(1) <= 32,
                            "per-pair scalars must be fp32 [T, K] with K <= 32");
    ++launches_; launch_combine_reduce(out.data_ptr(), num_ranks_ > 1 ? rows.data_ptr() : nullptr,
                          reinterpret_cast<const long long*>(topk_idx.data_ptr<int64_t>()),
                          out.size(0), out.size(1), topk_idx.size(1), num_experts, num_ranks_, rank_, stream(),
                          copy_dw ? dw_src->data_ptr<float>() : nullptr, copy_dw ? dw_dst->data_ptr<float>() : nullptr,
                          sizes.has_value() ? sizes->data_ptr<int>() + 2 : nullptr);
    SEP_CUDA_CHECK(cudaGetLastError());
  }
  at::Tensor pool_compress(const at::Tensor& pool, const at::Tensor& pool_recv_token, int64_t num_recv) {
    SEP_ASSERT(pool.is_contiguous() && pool.scalar_type() == at::kBFloat16 && pool.size(1) % 8 == 0, "pool must be contiguous bf16 with hidden % 8 == 0");
    auto out = at::empty({num_recv, pool.size(1)}, pool.options());
    ++launches_; launch_pool_compress(pool.data_ptr(), out.data_ptr(), pool_recv_token.data_ptr<int>(), pool.size(0), pool.size(1), stream());
    SEP_CUDA_CHECK(cudaGetLastError());
    return out;
  }
  at::Tensor pool_expand(const at::Tensor& recv, const at::Tensor& pool_recv_token, int64_t tk_padded) {
    SEP_ASSERT(recv.is_contiguous() && recv.scalar_type() == at::kBFloat16 && recv.size(1) % 8 == 0, "recv must be contiguous bf16 with hidden % 8 == 0");
    auto out = at::empty({tk_padded, recv.size(1)}, recv.options());
    ++launches_; launch_pool_expand(recv.data_ptr(), out.data_ptr(), pool_recv_token.data_ptr<int>(), tk_padded, recv.size(1), stream());
    SEP_CUDA_CHECK(cudaGetLastError());
    return out;
  }
  std::vector<at::Tensor> router(const at::Tensor& x, const at::Tensor& w_gate, int top_k, int num_ranks, bool renormalize, bool want_probs) {
    SEP_ASSERT(x.is_contiguous() && w_gate.is_contiguous() && x.scalar_type() == at::kBFloat16 && w_gate.scalar_type() == at::kBFloat16, "router inputs must be contiguous bf16");
    SEP_ASSERT(x.size(1) == w_gate.size(1) && x.size(1) % 8 == 0, "router hidden mismatch");
    SEP_ASSERT(w_gate.size(0) <= 512 && top_k <= 32 && w_gate.size(0) % num_ranks == 0, "router supports up to 512 experts and top-32");
    RouterParams p{};
    p.x = x.data_ptr(); p.w_gate = w_gate.data_ptr();
    p.num_tokens = x.size(0); p.hidden = x.size(1); p.num_experts = w_gate.size(0); p.num_topk = top_k;
    p.num_ranks = num_ranks; p.renormalize = renormalize ? 1 : 0;
    auto idx = at::empty({x.size(0), top_k}, x.options().dtype(at::kLong));
    auto w = at::empty({x.size(0), top_k}, x.options().dtype(at::kFloat));
    auto in_rank = at::empty({x.size(0), num_ranks}, x.options().dtype(at::kBool));
    at::Tensor probs;
    if (want_probs) probs = at::empty({x.size(0), w_gate.size(0)}, x.options().dtype(at::kFloat));
    p.topk_idx = reinterpret_cast<long long*>(idx.data_ptr<int64_t>()); p.topk_weights = w.data_ptr<float>();
    p.is_token_in_rank = reinterpret_cast<unsigned char*>(in_rank.data_ptr<bool>());
    p.probs = want_probs ? probs.data_ptr<float>() : nullptr;
    if (p.num_tokens > 0) {
      const int64_t T = x.size(0), E = w_gate.size(0);
      if (router_on_tensor_cores_ && E % 8 == 0 && E <= 256 && x.size(1) % 64 == 0) {
        // Logits on the tensor cores: the grouped GEMM with x as the only "expert group" and W_gate as its weight,
        // fp32 accumulators stored as they are (bf16 x bf16 products are exact in fp32, so this matches an fp32
        // GEMM up to summation order); then one warp per token for softmax / top-k.
        const int64_t tiles = (T + BM_ - 1) / BM_;
        if (!router_tiles_.defined() || router_tiles_.numel() < tiles)
          router_tiles_ = at::zeros({std::max<int64_t>(tiles, 64)}, x.options().dtype(at::kInt));
        at::Tensor logits = at::empty({T, E}, x.options().dtype(at::kFloat));
        GemmArgs g;
        g.mode = kVarlenM; g.epilogue = kEpiStoreF32; g.block_n = E > 128 ? 256 : 128;
        g.a = x; g.b = w_gate.unsqueeze(0); g.tile_id_to_expert = router_tiles_.narrow(0, 0, tiles); g.out0 = logits;
        grouped_gemm(g);
        ++launches_; launch_router_finish(p, logits.data_ptr<float>(), static_cast<int>(E), stream());
      } else {
        ++launches_; launch_router(p, stream());
      }
    }
    SEP_CUDA_CHECK(cudaGetLastError());
    return {idx, w, in_rank, probs};
  }
  // false: always the SIMT router kernel (also used for expert counts the GEMM path does not take)
  void set_router_on_tensor_cores(bool on) { router_on_tensor_cores_ = on; }

 private:
  static constexpr int BM_ = kTileM;
  // The current torch stream; remembered so that released arena blocks wait for the work queued on it.
  at::cuda::CUDAStream stream() {
    auto s = at::cuda::getCurrentCUDAStream();
    if (s.stream() != last_stream_) { release_ctx_->note_stream(s.stream()); last_stream_ = s.stream(); }
    return s;
  }
  void fill_peers(void** dst) const { for (int i = 0; i < kMaxRanks; ++i) dst[i] = peer_base_[i]; }
  void finish_sync() {
    // keeps the slab alive as long as any arena tensor or the runtime itself exists
    void* base = base_;
    if (use_vmm_) {
      VmmRange own = own_range_;
      arena_guard_ = std::shared_ptr<void>(base, [own](void*) mutable { own.destroy(); });
    } else {
      arena_guard_ = std::shared_ptr<void>(base, [](void* p) { cudaFree(p); });
    }
    available_ = true;
  }
  int num_sms() {
    if (num_sms_ == 0) {
      cudaDeviceProp prop;
      SEP_CUDA_CHECK(cudaGetDeviceProperties(&prop, device_));
      num_sms_ = prop.multiProcessorCount;
    }
    return num_sms_;
  }

  int rank_, num_ranks_, num_channels_, device_ = 0, num_sms_ = 0;
  ControlLayout ctl_{};
  void* base_ = nullptr;
  size_t arena_bytes_ = 0;
  std::shared_ptr<Arena> arena_;
  std::shared_ptr<void> arena_guard_;
  std::shared_ptr<ReleaseCtx> release_ctx_;
  cudaStream_t last_stream_ = reinterpret_cast<cudaStream_t>(-1);
  void* peer_base_[kMaxRanks];
  bool opened_[kMaxRanks] = {false, false, false, false, false, false, false, false};
  bool use_vmm_ = false;
  VmmRange own_range_;
  VmmRange peer_ranges_[kMaxRanks];
  void* scratch_ = nullptr;
  StatusBlock* status_ = nullptr;
  int* gate_flags_ = nullptr;
  int* counters_ = nullptr;
  HostCounters* host_ = nullptr;
  HostCounters* host_dev_ = nullptr;
  HostOverflow* host_overflow_ = nullptr;
  HostOverflow* host_overflow_dev_ = nullptr;
  std::shared_ptr<StaticPlan> static_;
  unsigned long long budget_ns_ = 0;
  int64_t timeout_ms_ = 0;
  int epochs_[kNumKinds];
  int64_t launches_ = 0;
  int pairs_per_chunk_ = 8;
  int head_pairs_per_chunk_ = 2, head_chunks_ = 0;
  int push_ctas_ = 0;
  bool bulk_push_ = false;
  bool split_local_ = false;
  int active_push_warps_ = 0;
  bool router_on_tensor_cores_ = true;
  at::Tensor router_tiles_;            // zeros: every M tile of the router GEMM belongs to "expert" 0
  int push_order_ = 0;
  std::shared_ptr<EventHandle> local_phase_;
  at::Tensor timing_;
  int gate_issued_[8];
  bool available_ = false, destroyed_ = false;
};

}  // namespace sep

// -------------------------------------------------------------------------------------------------
// Host-only arena exerciser (no CUDA calls) so the allocator logic is testable on a CPU-only box.
// -------------------------------------------------------------------------------------------------
struct ArenaProbe {
  // A fence the test completes by hand: `open_fences()` makes every fence handed out so far ready.
  struct ManualFence : sep::ArenaFence {
    std::shared_ptr<std::atomic<int>> opened; int ticket;
    bool ready() override { return opened->load() >= ticket; }
    void wait() override { int t = opened->load(); while (t < ticket && !opened->compare_exchange_weak(t, ticket)) {} }
  };
  sep::Arena arena;
  std::shared_ptr<std::atomic<int>> opened = std::make_shared<std::atomic<int>>(0);
  int tickets = 0;
  ArenaProbe(int64_t offset, int64_t size) : arena(offset, size) {}
  int64_t allocate(int64_t bytes) { return arena.allocate(bytes); }
  void release(int64_t off) { arena.release(off); }
  void release_deferred(int64_t off) {
    auto f = std::make_shared<ManualFence>();
    f->opened = opened; f->ticket = ++tickets;
    arena.release_deferred(off, f);
  }
  void open_fences() { opened->store(tickets); }
  int64_t parked() { arena.sweep(false); return arena.num_parked(); }
  int64_t in_use() const { return arena.bytes_in_use(); }
  int64_t high_water() const { return arena.high_water(); }
  int64_t capacity() const { return arena.capacity(); }
  int64_t free_blocks() const { return arena.num_free_blocks(); }
};

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  using namespace sep;
  m.doc() = "streamep_b200 native runtime (sm_100a)";
  m.attr("TILE_M") = kTileM;
  m.attr("MAX_RANKS") = kMaxRanks;
  m.attr("MAX_CHANNELS") = kMaxChannels;
  m.attr("MAX_EXPERTS") = kMaxExperts;
  m.def("is_sm100_compiled", [] { return true; });
  m.def("layer_bytes_hint", &ArenaSizeHint::layer_bytes);

  py::class_<ArenaProbe>(m, "ArenaProbe")
      .def(py::init<int64_t, int64_t>())
      .def("allocate", &ArenaProbe::allocate).def("release", &ArenaProbe::release)
      .def("release_deferred", &ArenaProbe::release_deferred).def("open_fences", &ArenaProbe::open_fences)
      .def("parked", &ArenaProbe::parked)
      .def("in_use", &ArenaProbe::in_use).def("high_water", &ArenaProbe::high_water)
      .def("capacity", &ArenaProbe::capacity).def("free_blocks", &ArenaProbe::free_blocks);

  py::class_<Config>(m, "Config")
      .def(py::init<int, int, int, int, int>(), py::arg("num_sms") = 20, py::arg("num_max_nvl_chunked_send_tokens") = 6,
           py::arg("num_max_nvl_chunked_recv_tokens") = 256, py::arg("num_max_rdma_chunked_send_tokens") = 6,
           py::arg("num_max_rdma_chunked_recv_tokens") = 256)
      .def("get_nvl_buffer_size_hint", &Config::get_nvl_buffer_size_hint)
      .def("get_rdma_buffer_size_hint", &Config::get_rdma_buffer_size_hint)
      .def_readonly("num_sms", &Config::num_sms)
      .def_readonly("num_max_nvl_chunked_send_tokens", &Config::num_max_nvl_chunked_send_tokens)
      .def_readonly("num_max_nvl_chunked_recv_tokens", &Config::num_max_nvl_chunked_recv_tokens)
      .def_readonly("num_max_rdma_chunked_send_tokens", &Config::num_max_rdma_chunked_send_tokens)
      .def_readonly("num_max_rdma_chunked_recv_tokens", &Config::num_max_rdma_chunked_recv_tokens);

  py::class_<EventHandle>(m, "EventHandle")
      .def(py::init<>())
      .def("current_stream_wait", &EventHandle::current_stream_wait)
      .def("wait_on", &EventHandle::wait_on)
      // same duck type as torch.cuda.Event: ``stream.wait_event(handle)`` calls ``handle.wait(stream)``
      .def("wait", [](const EventHandle& e, const py::object& stream) {
        e.wait_on(stream.attr("cuda_stream").cast<int64_t>(), stream.attr("device_index").cast<int>());
      });

  py::class_<DispatchState, std::shared_ptr<DispatchState>>(m, "DispatchState")
#define RO(name) .def_readonly(#name, &DispatchState::name)
      RO(x) RO(topk_idx) RO(topk_weights) RO(num_tokens) RO(hidden) RO(num_topk) RO(num_experts) RO(tile_m) RO(seq)
      RO(pair_rank) RO(pair_slot) RO(token_rank_in_channel) RO(send_recv_token) RO(send_head) RO(is_token_in_rank)
      RO(channel_prefix_matrix) RO(send_base) RO(send_token_base) RO(peer_total_tiles) RO(peer_num_recv)
      RO(send_order_base) RO(send_list) RO(num_send)
      RO(expert_frequency) RO(expert_pool_block_offset) RO(base_pool) RO(seen_per_substream) RO(rank_prefix_matrix)
      RO(recv_channel_prefix_matrix) RO(tile_id_to_expert) RO(pool_arrival_target)
      RO(pool) RO(pool_topk_weight) RO(pool_recv_token) RO(pool_k_slot) RO(pool_src) RO(recv_token_to_slots)
      RO(k_local_total) RO(k_local_remaining) RO(pool_arrival_count) RO(recv_src) RO(y_done_per_token) RO(o)
      RO(total_tiles) RO(num_recv_tokens) RO(recv_per_expert) RO(metadata_done_event) RO(push_epoch) RO(meta_epoch)
      RO(region_id) RO(dev_sizes)
#undef RO
      .def("release_o", &DispatchState::release_o)
      .def("release_pool", &DispatchState::release_pool);

  py::class_<GradsState, std::shared_ptr<GradsState>>(m, "GradsState")
      .def_readonly("dl_do_pool", &GradsState::dl_do_pool)
      .def_readonly("bwd_dispatch_arrival_count", &GradsState::bwd_dispatch_arrival_count)
      .def_readonly("started_event", &GradsState::started_event)
      .def_readonly("landing", &GradsState::landing).def_readonly("dwt", &GradsState::dwt)
      .def_readonly("landing_off", &GradsState::landing_off).def_readonly("dwt_off", &GradsState::dwt_off)
      .def_readonly("is_static", &GradsState::is_static)
      .def_readonly("epoch", &GradsState::epoch);

  py::class_<CombineState, std::shared_ptr<CombineState>>(m, "CombineState")
      .def_readonly("out", &CombineState::out)
      .def_readonly("out_topk_weights", &CombineState::out_topk_weights);

  py::class_<GemmArgs>(m, "GemmArgs")
      .def(py::init<>())
#define RW(name) .def_readwrite(#name, &GemmArgs::name)
      RW(mode) RW(epilogue) RW(block_n) RW(num_ctas) RW(a_mn_major) RW(b_mn_major) RW(a) RW(b)
      RW(a2) RW(b2) RW(out2) RW(dynamic_tiles)
      RW(tile_id_to_expert) RW(expert_pool_block_offset) RW(expert_frequency) RW(arrival_count) RW(arrival_target)
      RW(out0) RW(out1) RW(preact) RW(row_weight) RW(row_token) RW(dl_dweight) RW(scatter_local) RW(row_src) RW(row_k_slot)
      RW(tile_stripes_done) RW(k_remaining) RW(done_per_token) RW(remote_out) RW(remote_dw) RW(remote_out_offset) RW(remote_dw_offset) RW(num_m_tiles_dev)
      RW(num_topk) RW(seq) RW(num_m_tiles) RW(started_flag)
      RW(tail) RW(tail_kind) RW(tail_wait) RW(fused_push) RW(fused_push_grads) RW(fused_push_routing) RW(fused_push_rows)
      RW(push_flags);
#undef RW

  py::class_<Runtime>(m, "Runtime")
      .def(py::init<int, int, int64_t, int, int, int64_t, bool>(), py::arg("rank"), py::arg("num_ranks"), py::arg("arena_bytes"),
           py::arg("num_channels"), py::arg("num_experts_cap"), py::arg("timeout_ms"), py::arg("use_vmm") = false)
      .def("uses_vmm", &Runtime::uses_vmm)
      .def("arena_total_bytes", &Runtime::arena_total_bytes)
      .def("export_vmm_fd", &Runtime::export_vmm_fd)
      .def("sync_vmm", &Runtime::sync_vmm)
      .def("destroy", &Runtime::destroy)
      .def("get_local_device_id", &Runtime::get_local_device_id)
      .def("get_local_ipc_handle", &Runtime::get_local_ipc_handle)
      .def("get_local_base_ptr", &Runtime::get_local_base_ptr)
      .def("sync", &Runtime::sync)
      .def("sync_local", &Runtime::sync_local)
      .def("is_available", &Runtime::is_available)
      .def("set_timeout_ms", &Runtime::set_timeout_ms)
      .def("get_timeout_ms", &Runtime::get_timeout_ms)
      .def_property_readonly("rank", &Runtime::rank)
      .def_property_readonly("num_ranks", &Runtime::num_ranks)
      .def_property_readonly("num_channels", &Runtime::num_channels)
      .def("launch_count", &Runtime::launch_count)
      .def("set_kernel_timing", &Runtime::set_kernel_timing)
      .def("set_pairs_per_chunk", &Runtime::set_pairs_per_chunk)
      .def("set_push_head", &Runtime::set_push_head)
      .def("set_push_ctas", &Runtime::set_push_ctas)
      .def("get_push_ctas", &Runtime::get_push_ctas)
      .def("set_bulk_push", &Runtime::set_bulk_push)
      .def("set_split_local", &Runtime::set_split_local)
      .def("set_active_push_warps", &Runtime::set_active_push_warps)
      .def("set_push_order", &Runtime::set_push_order)
      .def("set_router_on_tensor_cores", &Runtime::set_router_on_tensor_cores)
      .def("arena_bytes_in_use", &Runtime::arena_bytes_in_use)
      .def("arena_high_water", &Runtime::arena_high_water)
      .def("arena_blocks_parked", &Runtime::arena_blocks_parked)
      .def("arena_capacity", &Runtime::arena_capacity)
      .def("alloc_symmetric", [](Runtime& r, const std::vector<int64_t>& sizes, py::object dtype, bool zero) {
        return r.alloc_symmetric(sizes, torch::python::detail::py_object_to_dtype(dtype), zero);
      }, py::arg("sizes"), py::arg("dtype"), py::arg("zero") = false)
      .def("is_symmetric", &Runtime::is_symmetric)
      .def("symmetric_offset", &Runtime::symmetric_offset)
      .def("poll_status", &Runtime::poll_status, py::arg("reset") = true)
      .def("gate_wait_started", &Runtime::gate_wait_started)
      .def("gate_bump_issued", &Runtime::gate_bump_issued)
      .def("gate_flag_tensor", &Runtime::gate_flag_tensor)
      .def("dispatch_begin", &Runtime::dispatch_begin, py::arg("x"), py::arg("topk_idx"), py::arg("topk_weights"),
           py::arg("num_experts"), py::arg("tile_m"), py::arg("seq"), py::arg("capacity_mode") = false)
      .def("enable_static", &Runtime::enable_static)
      .def("static_enabled", &Runtime::static_enabled)
      .def("static_reset", &Runtime::static_reset)
      .def("static_fits", &Runtime::static_fits)
      .def("static_capacity", &Runtime::static_capacity)
      .def("overflow_info", &Runtime::overflow_info)
      .def("next_landing", &Runtime::next_landing)
      .def("grads_finish", &Runtime::grads_finish)
      .def("dispatch_metadata", &Runtime::dispatch_metadata)
      .def("dispatch_allocate", &Runtime::dispatch_allocate, py::arg("state"), py::arg("need_o") = true, py::arg("defer_views") = false)
      .def("dispatch_finish_views", &Runtime::dispatch_finish_views)
      .def("dispatch_push", &Runtime::dispatch_push)
      .def("grads_begin", &Runtime::grads_begin, py::arg("state"), py::arg("fused_buffers") = false)
      .def("dispatch_set_aux", &Runtime::dispatch_set_aux)
      .def("grads_set_aux", &Runtime::grads_set_aux)
      .def("grads_push", &Runtime::grads_push)
      .def("combine_begin", &Runtime::combine_begin)
      .def("combine_launch", &Runtime::combine_launch)
      .def("barrier", &Runtime::barrier)
      .def("next_epoch", &Runtime::next_epoch)
      .def("get_epochs", &Runtime::get_epochs)
      .def("set_epochs", &Runtime::set_epochs)
      .def("grouped_gemm", &Runtime::grouped_gemm)
      .def("mark_local_phase", &Runtime::mark_local_phase)
      .def("local_phase_event", &Runtime::local_phase_event)
      .def("fused_forward", &Runtime::fused_forward)
      .def("fused_backward", &Runtime::fused_backward)
      .def("tile_producer", &Runtime::tile_producer)
      .def("combine_reduce", &Runtime::combine_reduce, py::arg("out"), py::arg("rows"), py::arg("topk_idx"), py::arg("num_experts"),
           py::arg("dw_src") = std::nullopt, py::arg("dw_dst") = std::nullopt, py::arg("sizes") = std::nullopt)
      .def("pool_compress", &Runtime::pool_compress)
      .def("pool_expand", &Runtime::pool_expand)
      .def("router", &Runtime::router);
}
