// Persistent grouped GEMM for sm_100a: TMA-fed shared-memory pipeline, tcgen05.mma with fp32
// accumulators in tensor memory (two accumulator buffers so the epilogue of tile i overlaps the
// main loop of tile i+1), and fused epilogues read back with tcgen05.ld.
//
// One kernel template covers every GEMM-shaped op of the MoE layer:
//   kernel A      pool[rows,H]   x W1[e]^T  -> SwiGLU on adjacent column pairs (+ optional preact)
//   kernel Y      postact[rows,I] x W2[e]^T -> x topk weight -> bf16x2 red.add scatter (local o, or the
//                                              source rank's output over NVLink = fused combine)
//   kernel Y_bwd  dL_do[rows,H]  x W2[e]    -> dswiglu, dL/dweight, zero padding rows
//   kernel A_bwd  dswiglu[rows,2I] x W1[e]  -> red.add scatter (local, or fused combine_grads)
//   dW1 / dW2     A[rows,M]^T x B[rows,N] per expert with true-length K masking
//   preact recompute = kernel A with the plain store epilogue
// and optionally carries extra "push" warps that ship token rows into peers' pools while the
// tensor-core warps consume tiles as they complete (dispatch fused with the GEMM).
//
// Reference counterparts: stream_ep/stream_moe/kernel_a.py, kernel_y.py, kernel_y_bwd.py,
// kernel_a_bwd.py, tile_scheduler.py, epi_ops.py and the quack.gemm calls at
// stream_ep/stream_moe/stream_moe.py:993-1004,1111-1142 (all Hopper WGMMA through CuTeDSL there).
#include <atomic>
#include <cstdio>
#include <mutex>
#include <type_traits>
#include <cuda.h>

#include "comm_common.cuh"
#include "no_alloc.h"

namespace sep {

constexpr int BM = 128;          // rows per tile == pool tile_m
constexpr int BK = 64;           // bf16 elements per k-block: one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int kGemmWarps = 10;   // 0: TMA producer, 1: MMA issuer + TMEM owner, 2..9: epilogue
// The kernels that consume tiles as a dispatch completes them (A and Y_bwd) carry one more warp whose lane 0 polls
// the tile gates AHEAD of the TMA producer.  A gate poll is an acquire load at system scope, microseconds long
// while NVLink traffic is landing; done by the producer itself it stalls the operand pipeline once per tile.
constexpr bool has_gate_warp(int epi) { return epi == kEpiSwiglu || epi == kEpiDswiglu; }
constexpr int base_warps(int epi) { return kGemmWarps + (has_gate_warp(epi) ? 1 : 0); }
// extra warps of the fused variants; the dSwiGLU epilogue keeps two preact segments in registers, so it gets fewer
// (Y_bwd: 16 warps x 128 registers, A: 20 warps x 96 registers fill the register file)
constexpr int push_warps(int epi) { return epi == kEpiDswiglu ? 5 : 9; }
constexpr int kMaxDevices = 64;  // per-device host-side tables (kernel attributes, no-alloc scratch address)
constexpr int kTileQueue = 8;    // dynamic tile claim: tiles the TMA thread may be ahead of the epilogue
constexpr int kEpiThreads = 256; // two threads per accumulator row: each takes half of the tile's columns

template <int BN> struct GemmCfg {
  static constexpr int kABytes = BM * BK * 2;                 // 16 KB
  static constexpr int kBBytes = BN * BK * 2;                 // 16 / 32 KB
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (BN == 256) ? 4 : 6;
  static constexpr int kTmemCols = 2 * BN;                    // two accumulator buffers
  static constexpr int kBarrierBytes = 256;
  static constexpr int kEpiStageBytes = 4096;                 // per epilogue warp: 32 rows x 128 bytes
  static constexpr int kSmemBytes = kStages * kStageBytes + 8 * kEpiStageBytes + kBarrierBytes + 1024;  // + alignment slack
};

size_t grouped_gemm_smem_bytes(int block_n) {
  return block_n == 256 ? GemmCfg<256>::kSmemBytes : GemmCfg<128>::kSmemBytes;
}

struct SecondMaps { CUtensorMap a, b, o; };   // operands and output of the second VarlenK problem

struct TileCoord {
  int prob;        // VarlenK: 0 / 1 = first / second problem of the launch
  int m_tile, n_tile, expert;
  int row0;        // first row of A (VarlenM: m_tile * BM; VarlenK: first pool row of the expert)
  int k_blocks;    // number of BK blocks to accumulate
  int k_tail;      // VarlenK: valid rows in the last block (0 = full)
};

// Tile order.  Consecutive linear indices (= CTAs working at the same time) walk a band of kBandM row tiles
// column by column: a wave of 148 tiles then shares kBandM A tiles and ~148/kBandM B tiles instead of one A
// tile and 148 B tiles, which keeps weight traffic out of HBM when one expert's weights exceed the L2.
// Bands follow the pool order (expert-major), i.e. the order in which dispatch completes tiles.
constexpr int kBandM = 8;

__device__ __forceinline__ void band_decode(int lin, int num_m, int num_n, int& m_tile, int& n_tile) {
  const int band = lin / (kBandM * num_n);
  const int rem = lin - band * (kBandM * num_n);
  const int m0 = band * kBandM;
  const int gm = min(kBandM, num_m - m0);
  n_tile = rem / gm;
  m_tile = m0 + (rem - n_tile * gm);
}

// `num_m`: live number of M tiles (VarlenM; may come from device memory), ignored for VarlenK.
__device__ __forceinline__ TileCoord decode_tile(const GemmParams& p, int lin, int num_m) {
  TileCoord t;
  t.prob = 0;
  if (p.mode == kVarlenM) {
    band_decode(lin, num_m, p.num_n_tiles, t.m_tile, t.n_tile);
    t.expert = p.tile_id_to_expert[t.m_tile];
    t.row0 = t.m_tile * BM;
    t.k_blocks = (p.K + BK - 1) / BK;
    t.k_tail = 0;
  } else {
    int nm = p.num_m_tiles, nn = p.num_n_tiles;
    const int first = p.num_experts * nm * nn;
    if (lin >= first) { t.prob = 1; lin -= first; nm = p.num_m_tiles2; nn = p.num_n_tiles2; }
    const int per_e = nm * nn;
    t.expert = lin / per_e;
    band_decode(lin - t.expert * per_e, nm, nn, t.m_tile, t.n_tile);
    t.row0 = p.expert_pool_block_offset[t.expert] * BM;
    const int len = p.expert_frequency[t.expert];
    t.k_blocks = (len + BK - 1) / BK;
    t.k_tail = len % BK;
  }
  return t;
}

__device__ __forceinline__ void st_global_v4(void* p, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.global.v4.b32 [%0], {%1, %2, %3, %4};" :: "l"(p), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ int atom_add_acq_rel_gpu(int* p, int v) {
  int old;
  asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
  return old;
}
__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }
// OR of `pred` over the 256 epilogue threads (named barrier 1, as epi_bar_sync): every thread gets the same answer.
__device__ __forceinline__ bool epi_vote_any(bool pred) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 p, %1, 0;\n\t"
      "barrier.cta.red.or.pred q, 1, 256, p;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t}"
      : "=r"(r) : "r"(static_cast<uint32_t>(pred)) : "memory");
  return r != 0;
}

template <int BN, bool A_MN, bool B_MN, int EPI, bool PUSH>
__global__ void __launch_bounds__((base_warps(EPI) + (PUSH ? push_warps(EPI) : 0)) * 32, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CUtensorMap tmap_o0, const __grid_constant__ CUtensorMap tmap_o1,
                    const GemmParams p, const PushParams pp, const __grid_constant__ SecondMaps maps2) {
  using Cfg = GemmCfg<BN>;
  extern __shared__ unsigned char smem_dyn[];
  // 128-byte swizzle atoms are 1024 bytes: align the operand ring accordingly.
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  unsigned char* stage_base = smem;
  unsigned char* epi_stage = smem + Cfg::kStages * Cfg::kStageBytes;      // 8 x 4 KB, 1024-byte aligned
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_stage + 8 * Cfg::kEpiStageBytes);
  uint64_t* full_bar = bars;                               // [kStages]
  uint64_t* empty_bar = bars + Cfg::kStages;               // [kStages]
  uint64_t* tmem_full = bars + 2 * Cfg::kStages;           // [2]
  uint64_t* tmem_empty = bars + 2 * Cfg::kStages + 2;      // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * Cfg::kStages + 4);
  int* s_flag = reinterpret_cast<int*>(tmem_slot + 1);     // epilogue broadcast word
  __shared__ PushTargets s_tg;
  __shared__ int s_push_ok;
  __shared__ int s_gates_open;   // how many of this CTA's tiles have an open gate (-1: the gate warp gave up)
  __shared__ int s_tiles_done;   // tiles whose epilogue finished (read by the time stamps only)
  __shared__ uint64_t s_push_bar[32][2];   // push-only CTAs: two bulk-load barriers per warp
  __shared__ int s_q[kTileQueue];          // dynamic tile claim: claimed tile ids ...
  __shared__ int s_q_head, s_q_tail;       // ... how many were claimed, how many the epilogue has finished
  __shared__ char* s_remote_out[kMaxRanks];
  __shared__ float* s_remote_dw[kMaxRanks];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Capacity mode keeps the live tile count in device memory (written by the metadata kernel earlier in the stream).
  const int num_m = (p.mode == kVarlenM && p.num_m_tiles_dev != nullptr) ? min(*p.num_m_tiles_dev, p.num_m_tiles) : p.num_m_tiles;
  const int total_tiles = p.mode == kVarlenM ? num_m * p.num_n_tiles
                                             : p.num_experts * (p.num_m_tiles * p.num_n_tiles + p.num_m_tiles2 * p.num_n_tiles2);
  // Tile feed.  Static: CTA b takes tiles b, b + stride, ...  Dynamic (VarlenK with a counter): the TMA thread claims
  // the next tile and hands it to the MMA and epilogue warps through a small queue in shared memory.
  const bool dyn = p.mode == kVarlenK && p.tile_counter != nullptr;
  const unsigned long long budget = p.wait_budget_ns;
  // Fused push, two ways of sharing the GPU.  Mixed (push_ctas == 0): every CTA multiplies and its extra warps push.
  // Dedicated (push_ctas > 0): the last push_ctas CTAs only push, with all their warps, and the others only multiply.
  // Remote stores that wait for NVLink credit back up in an SM's load/store path, where the epilogue warps of
  // the same SM queue behind them: with the push on SMs of its own the GEMM runs at its stand-alone rate.
  const int num_push_ctas = PUSH ? min(max(pp.push_ctas, 0), static_cast<int>(gridDim.x) - 1) : 0;
  const int lin_stride = static_cast<int>(gridDim.x) - num_push_ctas;
  const bool is_push_cta = PUSH && static_cast<int>(blockIdx.x) >= lin_stride;
  const int first_lin = is_push_cta ? 0x7fffffff : static_cast<int>(blockIdx.x);

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    for (int s = 0; s < Cfg::kStages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tmem_full[a], 1); mbar_init(&tmem_empty[a], kEpiThreads); }
    mbar_fence_init();
    if (blockIdx.x == 0 && p.started_flag != nullptr) atomicAdd(p.started_flag, 1);
    if (PUSH) s_push_ok = 1;
    s_gates_open = 0;
    s_tiles_done = 0;
    s_q_head = 0; s_q_tail = 0;
    if (p.timing != nullptr) {
      long long* tm = p.timing + static_cast<size_t>(blockIdx.x) * kTimingCols;
      tm[0] = static_cast<long long>(globaltimer_ns());
      tm[1] = 0; tm[2] = 0; tm[3] = 0; tm[4] = 0; tm[5] = 0; tm[7] = 0; tm[8] = 0; tm[9] = 0; tm[10] = 0;
    }
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  if (PUSH) {
    if ((pp.flags & 1) && !pp.static_targets && blockIdx.x == 0 && warp == base_warps(EPI) && lane < pp.num_ranks)
      publish_record(pp.own, pp.peer_base, pp.ctl, pp.kind, pp.epoch, pp.rank, lane);
  }
  if ((EPI == kEpiScatter || EPI == kEpiDswiglu) && warp == 2 && lane < p.num_ranks) {
    // Resolve buffers that every rank allocated at its own arena offset from the published records.
    if (p.remote_out.enabled) {
      if (p.remote_out.is_static) {
        s_remote_out[lane] = static_cast<char*>(p.peer_base[lane]) + p.remote_out.offset;
      } else {
        const unsigned long long* rec = fetch_record(p.peer_base[p.rank], p.ctl, p.remote_out.kind, p.remote_out.epoch,
                                                     lane, budget, p.status, kKernelGemm, p.rank);
        s_remote_out[lane] = rec ? static_cast<char*>(p.peer_base[lane]) + rec[p.remote_out.field] : nullptr;
      }
    }
    if (p.remote_dw.enabled) {
      if (p.remote_dw.is_static) {
        s_remote_dw[lane] = reinterpret_cast<float*>(static_cast<char*>(p.peer_base[lane]) + p.remote_dw.offset);
      } else {
        const unsigned long long* rec = fetch_record(p.peer_base[p.rank], p.ctl, p.remote_dw.kind, p.remote_dw.epoch,
                                                     lane, budget, p.status, kKernelGemm, p.rank);
        s_remote_dw[lane] = rec ? reinterpret_cast<float*>(static_cast<char*>(p.peer_base[lane]) + rec[p.remote_dw.field]) : nullptr;
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (is_push_cta) {
    // ------------------------------------------------------------------ push-only CTA: every warp ships rows
    if (pp.flags & 2) {
      if (warp == 0 && lane < pp.num_ranks) {
        const unsigned long long* rec = pp.static_targets
            ? reinterpret_cast<const unsigned long long*>(&pp.own)
            : fetch_record(pp.peer_base[pp.rank], pp.ctl, pp.kind, pp.epoch, lane,
                           pp.wait_budget_ns, pp.status, kKernelDispatch, pp.rank);
        if (rec == nullptr) s_push_ok = 0;
        else resolve_push_targets(s_tg, lane, pp.peer_base[lane], rec);
      }
      // The operand ring of the GEMM is unused here: every warp takes two 4 KB slots of it for bulk copies
      // (global -> shared -> owner's pool through the copy engine, see push_chunk).
      PushRing ring{};
      ring.bar = s_push_bar[warp];
      ring.ok = true;
      if (pp.bulk_push && (warp + 1) * 2 * static_cast<int>(kPushPieceBytes) <= Cfg::kStages * Cfg::kStageBytes) {
        ring.smem = smem_u32(stage_base) + warp * 2 * kPushPieceBytes;
        if (lane == 0) { mbar_init(&ring.bar[0], 1); mbar_init(&ring.bar[1], 1); mbar_fence_init(); }
      }
      __syncthreads();
      if (s_push_ok) {
        const int num_send = *pp.num_send;
        const int num_chunks = push_num_chunks(pp, num_send);
        if (p.timing != nullptr && threadIdx.x == 0)
          p.timing[static_cast<size_t>(blockIdx.x) * kTimingCols + 4] = static_cast<long long>(globaltimer_ns());
        for (;;) {
          int chunk = 0;
          if (lane == 0) chunk = ring.ok ? atomicAdd(pp.work_counter, 1) : 0x7fffffff;
          chunk = __shfl_sync(0xffffffffu, chunk, 0);
          if (chunk >= num_chunks) break;
          int p0, p1;
          push_chunk_range(pp, num_send, chunk, p0, p1);
          push_chunk(pp, s_tg, p0, p1, lane, &ring, pp.split_local ? 2 : 0);
        }
        if (p.timing != nullptr && lane == 0)
          atomicMax(reinterpret_cast<unsigned long long*>(p.timing + static_cast<size_t>(blockIdx.x) * kTimingCols + 5), globaltimer_ns());
      }
    }
  } else if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0; int issued = 0; bool ok = true; int my_tile = 0;
      for (int it = 0; ok; ++it) {
        int lin;
        if (dyn) {
          // claim the next tile; wait for a free queue entry first (the epilogue is at most kTileQueue tiles behind)
          if (!spin_until([&] { return it - ld_acquire_cta_shared(&s_q_tail) < kTileQueue; }, budget, p.status)) {
            report_failure(p.status, kStatusTimeoutPipeline, kKernelGemm, 4, p.rank, it, 0, 0);
            ok = false;
            lin = total_tiles;
          } else {
            lin = atomicAdd(p.tile_counter, 1);
          }
          s_q[it % kTileQueue] = lin;
          st_release_cta_shared(&s_q_head, it + 1);
        } else {
          lin = first_lin + it * lin_stride;
        }
        if (lin >= total_tiles || lin < 0) break;
        const TileCoord t = decode_tile(p, lin, num_m);
        const CUtensorMap* ta = t.prob ? &maps2.a : &tmap_a;
        const CUtensorMap* tb = t.prob ? &maps2.b : &tmap_b;
        if (p.mode == kVarlenM && p.arrival_count != nullptr) {
          const unsigned long long gate_t0 = p.timing != nullptr ? globaltimer_ns() : 0ull;
          bool open;
          if constexpr (has_gate_warp(EPI)) {
            // the gate warp polls the counters ahead of this thread and publishes how far it got
            open = spin_until([&] { const int g = ld_acquire_cta_shared(&s_gates_open); return g < 0 || g > my_tile; }, budget, p.status) &&
                   ld_acquire_cta_shared(&s_gates_open) > my_tile;
          } else {
            const int target = p.arrival_target[t.m_tile];
            const int* cnt = p.arrival_count + t.m_tile;
            const bool local_only = p.num_ranks == 1;
            open = spin_until([&] { return (local_only ? ld_acquire_gpu(cnt) : ld_acquire_sys(cnt)) == target; }, budget, p.status);
            if (!open) report_failure(p.status, kStatusTimeoutTileGate, kKernelGemm, 0, p.rank, t.m_tile, target, ld_acquire_sys(cnt));
          }
          if (!open) { ok = false; break; }
          fence_proxy_async();   // rows were written through the generic proxy (possibly by a peer GPU)
          if (p.timing != nullptr) {
            long long* tm = p.timing + static_cast<size_t>(blockIdx.x) * kTimingCols;
            tm[1] += static_cast<long long>(globaltimer_ns() - gate_t0);   // time the operand pipeline stood still for gates
            tm[7] += 1;
          }
          ++my_tile;
        }
        for (int kb = 0; kb < t.k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, budget, p.status)) {
            report_failure(p.status, kStatusTimeoutPipeline, kKernelGemm, 0, p.rank, lin, kb, stage);
            ok = false; break;
          }
          unsigned char* sa = stage_base + stage * Cfg::kStageBytes;
          unsigned char* sb = sa + Cfg::kABytes;
          mbar_arrive_expect_tx(&full_bar[stage], Cfg::kStageBytes);
          const int k0 = kb * BK;
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_3d(sa + j * (BK * 128), ta, &full_bar[stage], t.m_tile * BM + j * 64, t.row0 + k0, 0);
          } else {
            tma_load_3d(sa, ta, &full_bar[stage], k0, t.row0, 0);
          }
          if (B_MN) {
            const int kz = (p.mode == kVarlenM) ? k0 : t.row0 + k0;
            const int ez = (p.mode == kVarlenM) ? t.expert : 0;
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_3d(sb + j * (BK * 128), tb, &full_bar[stage], t.n_tile * BN + j * 64, kz, ez);
          } else {
            tma_load_3d(sb, tb, &full_bar[stage], k0, t.n_tile * BN, t.expert);
          }
          ++issued;
          if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        // Drain: every copy this thread issued must have landed before the CTA may exit.
        const int pending = issued < Cfg::kStages ? issued : Cfg::kStages;
        for (int i = 0; i < pending; ++i) {
          int s = stage - 1 - i; uint32_t ph = phase;
          if (s < 0) { s += Cfg::kStages; ph ^= 1; }
          const unsigned long long t0 = globaltimer_ns();
          while (!mbar_try_wait(&full_bar[s], ph) && globaltimer_ns() - t0 < 2000000ull) {}
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
    int stage = 0; uint32_t phase = 0; int acc = 0; uint32_t acc_phase = 0; bool ok = true;
    // With time stamps on the loop also counts where this warp's time goes (SM cycles, see GemmParams::timing).  The
    // loop is compiled twice: even a predicated-off clock read between "operands have landed" and the MMA issue
    // cost 2 % of the whole step.
    long long cyc_operands = 0, cyc_accumulator = 0;
    const long long cyc_begin = p.timing != nullptr ? clock64() : 0;
    auto tile_loop = [&](auto timed) {
    constexpr bool stamp = decltype(timed)::value;
    for (int it = 0; ok; ++it) {
      int lin;
      if (dyn) {
        if (!__all_sync(0xffffffffu, spin_until([&] { return ld_acquire_cta_shared(&s_q_head) > it; }, budget, p.status))) { ok = false; break; }
        lin = s_q[it % kTileQueue];
      } else {
        lin = first_lin + it * lin_stride;
      }
      if (lin >= total_tiles || lin < 0) break;
      const TileCoord t = decode_tile(p, lin, num_m);
      if (t.k_blocks == 0) continue;   // empty expert: the epilogue writes zeros on its own
      // all 32 lanes wait; the outcome is made warp-uniform so that no lane leaves ahead of elect_one / __syncwarp
      long long c_acc = 0;
      if constexpr (stamp) c_acc = clock64();
      if (!__all_sync(0xffffffffu, mbar_wait(&tmem_empty[acc], acc_phase ^ 1, budget, p.status))) { ok = false; break; }
      if constexpr (stamp) cyc_accumulator += clock64() - c_acc;
      tc_fence_after_sync();
      const uint32_t tmem_d = tmem_base + acc * BN;
      for (int kb = 0; kb < t.k_blocks; ++kb) {
        long long c_ops = 0;
        if constexpr (stamp) c_ops = clock64();
        if (!__all_sync(0xffffffffu, mbar_wait(&full_bar[stage], phase, budget, p.status))) { ok = false; break; }
        if constexpr (stamp) cyc_operands += clock64() - c_ops;
        unsigned char* sa = stage_base + stage * Cfg::kStageBytes;
        unsigned char* sb = sa + Cfg::kABytes;
        if (p.mode == kVarlenK && t.k_tail != 0 && kb == t.k_blocks - 1) {
          // Rows past the expert's true length hold other data: zero them in both operands
          // (MN-major boxes keep one 128-byte row per k index, so whole rows are cleared).
          const int first = t.k_tail;
          constexpr int kBoxes = BM / 64 + BN / 64;
          for (int i = lane; i < kBoxes * (BK - first) * 8; i += 32) {
            const int box = i / ((BK - first) * 8);
            const int r = i - box * ((BK - first) * 8);
            *reinterpret_cast<uint4*>(sa + box * (BK * 128) + (first + r / 8) * 128 + (r % 8) * 16) = make_uint4(0, 0, 0, 0);
          }
          fence_proxy_async_smem();
          __syncwarp();
        }
        tc_fence_after_sync();
        if (elect_one()) {
          const uint32_t a_addr = smem_u32(sa), b_addr = smem_u32(sb);
#pragma unroll
          for (int j = 0; j < BK / UMMA_K; ++j) {
            const uint64_t da = A_MN ? umma_smem_desc(a_addr + j * (UMMA_K * 128), BK * 128, 1024)
                                     : umma_smem_desc(a_addr + j * (UMMA_K * 2), 16, 1024);
            const uint64_t db = B_MN ? umma_smem_desc(b_addr + j * (UMMA_K * 128), BK * 128, 1024)
                                     : umma_smem_desc(b_addr + j * (UMMA_K * 2), 16, 1024);
            umma_bf16_ss(tmem_d, da, db, idesc, (kb > 0 || j > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);                       // frees the smem stage when the MMAs retire
          if (kb == t.k_blocks - 1) umma_commit(&tmem_full[acc]);  // accumulator complete
        }
        __syncwarp();
        if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
      }
      acc ^= 1; if (acc == 0) acc_phase ^= 1;
    }
    };
    if (p.timing != nullptr) tile_loop(std::true_type{}); else tile_loop(std::false_type{});
    if (p.timing != nullptr && lane == 0) {
      long long* tm = p.timing + static_cast<size_t>(blockIdx.x) * kTimingCols;
      tm[8] = clock64() - cyc_begin; tm[9] = cyc_operands; tm[10] = cyc_accumulator;
    }
    if (!ok) report_failure(p.status, kStatusTimeoutPipeline, kKernelGemm, 1, p.rank, 0, 0, 0);
  } else if (warp < kGemmWarps) {
    // ------------------------------------------------------------------ epilogue (8 warps: a warp reads the 32 TMEM
    // lanes of its quarter; warps 2..5 take the left half of the tile's columns, warps 6..9 the right half).
    // Results go through a per-warp 4 KB swizzled staging tile so that global memory only ever sees
    // full contiguous row segments: TMA stores for dense outputs, warp-coalesced red.add / st for scatters.
    const int quarter = warp & 3;                 // TMEM lanes this warp may read
    const int row = quarter * 32 + lane;
    const int epi_tid = (warp - 2) * 32 + lane;
    const int half = (warp - 2) >> 2;
    constexpr int kChunksPerHalf = BN / 64;
    const uint32_t stg = smem_u32(epi_stage + (warp - 2) * Cfg::kEpiStageBytes);
    int acc = 0; uint32_t acc_phase = 0;
    for (int it = 0;; ++it) {
      int lin;
      if (dyn) {
        // every epilogue thread reads the queue itself; the give-up decision is taken together (see below)
        const bool got = spin_until([&] { return ld_acquire_cta_shared(&s_q_head) > it; }, budget, p.status);
        if (epi_vote_any(!got)) break;
        lin = s_q[it % kTileQueue];
      } else {
        lin = first_lin + it * lin_stride;
      }
      if (lin >= total_tiles || lin < 0) break;
      const TileCoord t = decode_tile(p, lin, num_m);
      const CUtensorMap* to0 = t.prob ? &maps2.o : &tmap_o0;
      const int prob_n = t.prob ? p.N2 : p.N;       // output width of this tile's problem
      const bool empty = (t.k_blocks == 0);
      // Everything that does not need the accumulator is fetched while the tensor cores still work on this tile.
      const int n0 = t.n_tile * BN;
      const int warp_row0 = (p.mode == kVarlenM ? t.row0 : t.m_tile * BM) + quarter * 32;   // TMA y coordinate
      const int zc = (p.mode == kVarlenK) ? t.expert : 0;
      const long long grow = static_cast<long long>(p.mode == kVarlenM ? t.row0 : t.m_tile * BM) + row;
      const int c_begin = half * kChunksPerHalf;
      int tok = 0; float w = 1.f;
      if (EPI == kEpiScatter || EPI == kEpiDswiglu) {
        tok = p.row_token[grow];
        if (p.row_weight != nullptr && tok >= 0) w = p.row_weight[grow];
      }
      // scatter: where this row goes and how (0 skip, 1 bf16x2 red.add, 2 plain store)
      char* dst_row = nullptr; int op = 0;
      if (EPI == kEpiScatter && tok >= 0) {
        if (p.remote_out.enabled) {
          const int2 src = p.row_src[grow];
          if (src.x == p.rank) {
            dst_row = static_cast<char*>(p.scatter_local) + static_cast<long long>(src.y) * p.N * 2; op = 1;
          } else {   // the source rank's per-(token, k) row: written once, reduced there in fp32
            dst_row = s_remote_out[src.x] + (static_cast<long long>(src.y) * p.num_topk + p.row_k_slot[grow]) * p.N * 2; op = 2;
          }
        } else {
          dst_row = static_cast<char*>(p.scatter_local) + static_cast<long long>(tok) * p.N * 2; op = 1;
        }
      }
      // dSwiGLU reads preact[row, 2n .. 2n+64) per chunk.  A thread-per-row read would touch 32 different lines
      // per instruction, which the load/store unit handles one line at a time; instead 8 lanes fetch one
      // row's 128 bytes (4 full lines per instruction) and the rows are handed to their threads through the
      // staging tile.  pqc = the next chunk in that fetch layout, pq = this thread's row segment.
      uint4 pq[8], pqc[8];
      const char* pre_base = nullptr;
      if (EPI == kEpiDswiglu) {
        pre_base = reinterpret_cast<const char*>(static_cast<const __nv_bfloat16*>(p.preact) +
                                                 static_cast<long long>(warp_row0 + (lane >> 3)) * p.ld_preact) + (lane & 7) * 16;
        const int nf = n0 + c_begin * 32;
        if (nf < p.N) {
#pragma unroll
          for (int i = 0; i < 8; ++i)
            pqc[i] = (2 * nf + (lane & 7) * 8 < 2 * p.N)
                         ? ld_nc_v4(pre_base + static_cast<long long>(i) * 4 * p.ld_preact * 2 + static_cast<long long>(nf) * 4)
                         : make_uint4(0, 0, 0, 0);
        }
      }
      if (!empty) {
        const bool got = mbar_wait(&tmem_full[acc], acc_phase, budget, p.status);
        if (!got) report_failure(p.status, kStatusTimeoutPipeline, kKernelGemm, 2, p.rank, lin, acc, 0);
        // The give-up decision is taken by all 256 epilogue threads together: a thread that saw the accumulator
        // must not go on to the stripe barriers (or to a warp-wide tcgen05.ld) while another one leaves the loop.
        if (epi_vote_any(!got)) break;
        tc_fence_after_sync();
      }
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(quarter * 32) << 16);
      float dw_acc = 0.f;
#pragma unroll 1
      for (int c = c_begin; c < c_begin + kChunksPerHalf; ++c) {
        const int n = n0 + c * 32;
        if (n >= prob_n) break;
        if (EPI == kEpiDswiglu) {
          // hand this chunk's preact rows to their threads, then request the next chunk (software pipeline)
#pragma unroll
          for (int i = 0; i < 8; ++i)
            st_shared_v4(stg + stage_off<128>(i * 4 + (lane >> 3), lane & 7), pqc[i].x, pqc[i].y, pqc[i].z, pqc[i].w);
          __syncwarp();
#pragma unroll
          for (int j = 0; j < 8; ++j) pq[j] = ld_shared_v4(stg + stage_off<128>(lane, j));
          __syncwarp();
          const int nn = n + 32;
          if (c + 1 < c_begin + kChunksPerHalf && nn < p.N) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
              pqc[i] = (2 * nn + (lane & 7) * 8 < 2 * p.N)
                           ? ld_nc_v4(pre_base + static_cast<long long>(i) * 4 * p.ld_preact * 2 + static_cast<long long>(nn) * 4)
                           : make_uint4(0, 0, 0, 0);
          }
        }
        uint32_t r[EPI == kEpiDswiglu ? 1 : 32];   // the dSwiGLU epilogue reads the accumulator 16 columns at a time
        if (EPI != kEpiDswiglu) {
          if (!empty) {
            tmem_ld_32x32(taddr + c * 32, reinterpret_cast<uint32_t(&)[32]>(r)); tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < (EPI == kEpiDswiglu ? 1 : 32); ++i) r[i] = 0;
          }
        }
        if (EPI == kEpiStore || EPI == kEpiSwiglu) {
          // The staging tile is reused by every chunk: the previous chunk's bulk store must have read it.
          // Waiting here, after the accumulator fetch, instead of right after the store was issued lets the
          // read overlap the TMEM load.
          if (lane == 0) bulk_wait_read();
          __syncwarp();
        }
        if (EPI == kEpiStore) {
#pragma unroll
          for (int q = 0; q < 4; ++q)
            st_shared_v4(stg + stage_off<64>(lane, q),
                         pack_bf16x2(__uint_as_float(r[q * 8 + 0]), __uint_as_float(r[q * 8 + 1])),
                         pack_bf16x2(__uint_as_float(r[q * 8 + 2]), __uint_as_float(r[q * 8 + 3])),
                         pack_bf16x2(__uint_as_float(r[q * 8 + 4]), __uint_as_float(r[q * 8 + 5])),
                         pack_bf16x2(__uint_as_float(r[q * 8 + 6]), __uint_as_float(r[q * 8 + 7])));
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) { tma_store_3d(to0, epi_stage + (warp - 2) * Cfg::kEpiStageBytes, n, warp_row0, zc); bulk_commit(); }
        } else if (EPI == kEpiSwiglu) {
          // columns (2i, 2i+1) = (gate_i, up_i); preact tile at +0 (64-byte rows), postact tile at +2048 (32-byte rows)
          if (p.out1 != nullptr) {
#pragma unroll
            for (int q = 0; q < 4; ++q)
              st_shared_v4(stg + stage_off<64>(lane, q),
                           pack_bf16x2(__uint_as_float(r[q * 8 + 0]), __uint_as_float(r[q * 8 + 1])),
                           pack_bf16x2(__uint_as_float(r[q * 8 + 2]), __uint_as_float(r[q * 8 + 3])),
                           pack_bf16x2(__uint_as_float(r[q * 8 + 4]), __uint_as_float(r[q * 8 + 5])),
                           pack_bf16x2(__uint_as_float(r[q * 8 + 6]), __uint_as_float(r[q * 8 + 7])));
          }
          float a[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float g = __uint_as_float(r[2 * i]), u = __uint_as_float(r[2 * i + 1]);
            a[i] = g * fast_sigmoid(g) * u;
          }
#pragma unroll
          for (int q = 0; q < 2; ++q)
            st_shared_v4(stg + 2048 + stage_off<32>(lane, q), pack_bf16x2(a[q * 8 + 0], a[q * 8 + 1]),
                         pack_bf16x2(a[q * 8 + 2], a[q * 8 + 3]), pack_bf16x2(a[q * 8 + 4], a[q * 8 + 5]),
                         pack_bf16x2(a[q * 8 + 6], a[q * 8 + 7]));
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            unsigned char* sb = epi_stage + (warp - 2) * Cfg::kEpiStageBytes;
            if (p.out1 != nullptr) tma_store_3d(&tmap_o1, sb, n, warp_row0, 0);
            tma_store_3d(&tmap_o0, sb + 2048, n / 2, warp_row0, 0);
            bulk_commit();
          }
        } else if (EPI == kEpiScatter) {
          // Stage two 32-column chunks side by side (128 bytes per row), then let 8 lanes handle one row so
          // that every global access - local red.add or store into a peer's landing row over NVLink - is a
          // full, contiguous 128-byte line of the destination row.
          const int hpos = (c - c_begin) & 1;
#pragma unroll
          for (int q = 0; q < 4; ++q)
            st_shared_v4(stg + stage_off<128>(lane, hpos * 4 + q),
                         pack_bf16x2(w * __uint_as_float(r[q * 8 + 0]), w * __uint_as_float(r[q * 8 + 1])),
                         pack_bf16x2(w * __uint_as_float(r[q * 8 + 2]), w * __uint_as_float(r[q * 8 + 3])),
                         pack_bf16x2(w * __uint_as_float(r[q * 8 + 4]), w * __uint_as_float(r[q * 8 + 5])),
                         pack_bf16x2(w * __uint_as_float(r[q * 8 + 6]), w * __uint_as_float(r[q * 8 + 7])));
          const bool flush = hpos == 1 || n + 32 >= p.N || c + 1 == c_begin + kChunksPerHalf;
          if (flush) {
            __syncwarp();
            const int nbase = n - hpos * 32;
            uint4 vs[8];      // shared-memory reads first: volatile asm keeps program order, see the dSwiGLU branch
#pragma unroll
            for (int i = 0; i < 8; ++i) vs[i] = ld_shared_v4(stg + stage_off<128>(i * 4 + (lane >> 3), lane & 7));
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int rr = i * 4 + (lane >> 3), piece = lane & 7;
              const uint4 v = vs[i];
              char* ptr = reinterpret_cast<char*>(__shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(dst_row), rr));
              const int o = __shfl_sync(0xffffffffu, op, rr);
              const int col = nbase + piece * 8;
              if (o != 0 && piece < (hpos + 1) * 4 && col < p.N) {
                if (o == 1) red_add_bf16x2_v4(ptr + static_cast<long long>(col) * 2, v.x, v.y, v.z, v.w);
                else st_na_v4(ptr + static_cast<long long>(col) * 2, v);
              }
            }
            __syncwarp();
          }
        } else if (EPI == kEpiStoreF32) {
          // fp32 accumulator values as they are (router logits): a thread owns a row, so its 32 columns are
          // one full 128-byte line of the output row.  Rows past the end of A are TMA zero fill: not stored.
          if (grow < p.total_rows) {
            float* dst = static_cast<float*>(p.out0) + grow * p.ld0 + n;
#pragma unroll
            for (int q = 0; q < 8; ++q)
              if (n + q * 4 < p.N) st_global_v4(dst + q * 4, r[q * 4], r[q * 4 + 1], r[q * 4 + 2], r[q * 4 + 3]);
          }
        } else {   // kEpiDswiglu: r = g[row, n..n+32) = dL/d(postact) before the topk weight
          uint32_t o_pw[16];
          unsigned char* sb = epi_stage + (warp - 2) * Cfg::kEpiStageBytes;
          uint32_t rh[16];
#pragma unroll
          for (int q = 0; q < 4; ++q) {       // 8 output columns per step; N is a multiple of 8
            if ((q & 1) == 0) {
              // One 16-column half at a time, fetched where it is used: fetching both halves up front, or the
              // first half before the preact hand-over, costs registers (spills at the 168-register cap of a
              // 10-warp CTA) and measured 7-12 % slower.
              if (!empty) { tmem_ld_32x16(taddr + c * 32 + q * 8, rh); tmem_ld_wait(); }
              else {
#pragma unroll
                for (int i = 0; i < 16; ++i) rh[i] = 0;
              }
            }
            uint32_t o_in[8];
            if (tok >= 0 && n + q * 8 < p.N) {
              const uint4 p0 = pq[q * 2], p1 = pq[q * 2 + 1];
              const uint32_t pv[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
              float post[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const float2 gu = unpack_bf16x2(pv[i]);          // (gate, up)
                const float g = __uint_as_float(rh[(q & 1) * 8 + i]);
                const float sig = fast_sigmoid(gu.x);
                const float silu = gu.x * sig;
                post[i] = silu * gu.y;
                dw_acc = fmaf(post[i], g, dw_acc);
                const float wg = w * g;
                const float dsilu = sig + fmaf(-sig, silu, silu);   // d silu / d gate = sig + silu * (1 - sig)
                o_in[i] = pack_bf16x2(wg * gu.y * dsilu, wg * silu);
              }
#pragma unroll
              for (int i = 0; i < 4; ++i) o_pw[q * 4 + i] = pack_bf16x2(w * post[2 * i], w * post[2 * i + 1]);
            } else {
#pragma unroll
              for (int i = 0; i < 8; ++i) o_in[i] = 0;
#pragma unroll
              for (int i = 0; i < 4; ++i) o_pw[q * 4 + i] = 0;
            }
            st_shared_v4(stg + stage_off<128>(lane, 2 * q), o_in[0], o_in[1], o_in[2], o_in[3]);
            st_shared_v4(stg + stage_off<128>(lane, 2 * q + 1), o_in[4], o_in[5], o_in[6], o_in[7]);
          }
          // Both outputs leave through the staging tile with plain coalesced stores (8 resp. 4 lanes per
          // 128- resp. 64-byte row segment).  No proxy fence here on purpose: a fence would wait for the
          // preact loads of the next chunk that are still in flight.
          __syncwarp();
          {
            char* din_base = reinterpret_cast<char*>(static_cast<__nv_bfloat16*>(p.out0) + static_cast<long long>(warp_row0) * p.ld0 + 2 * n);
            // all shared-memory reads first, then all global stores: the helpers are volatile asm, which the
            // compiler keeps in program order, so an interleaved loop would wait for every read in turn
            uint4 v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = ld_shared_v4(stg + stage_off<128>(i * 4 + (lane >> 3), lane & 7));
            if (2 * n + (lane & 7) * 8 < 2 * p.N) {
#pragma unroll
              for (int i = 0; i < 8; ++i)
                st_global_v4(din_base + static_cast<long long>(i * 4 + (lane >> 3)) * p.ld0 * 2 + (lane & 7) * 16,
                             v[i].x, v[i].y, v[i].z, v[i].w);
            }
          }
          __syncwarp();
#pragma unroll
          for (int q = 0; q < 4; ++q)
            st_shared_v4(stg + stage_off<64>(lane, q), o_pw[q * 4 + 0], o_pw[q * 4 + 1], o_pw[q * 4 + 2], o_pw[q * 4 + 3]);
          __syncwarp();
          {
            char* pw_base = reinterpret_cast<char*>(static_cast<__nv_bfloat16*>(p.out1) + static_cast<long long>(warp_row0) * p.ld1 + n);
            uint4 v[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) v[i] = ld_shared_v4(stg + stage_off<64>(i * 8 + (lane >> 2), lane & 3));
            if (n + (lane & 3) * 8 < p.N) {
#pragma unroll
              for (int i = 0; i < 4; ++i)
                st_global_v4(pw_base + static_cast<long long>(i * 8 + (lane >> 2)) * p.ld1 * 2 + (lane & 3) * 16,
                             v[i].x, v[i].y, v[i].z, v[i].w);
            }
          }
          __syncwarp();
        }
      }
      if (!empty) {
        tc_fence_before_sync();
        mbar_arrive(&tmem_empty[acc]);
        acc ^= 1; if (acc == 0) acc_phase ^= 1;
      }
      if (p.timing != nullptr && epi_tid == 0) *reinterpret_cast<volatile int*>(&s_tiles_done) += 1;
      if (dyn) {                    // this queue entry may be reused once every epilogue thread is done with the tile
        epi_bar_sync();
        if (epi_tid == 0) st_release_cta_shared(&s_q_tail, it + 1);
      }
      if (EPI == kEpiDswiglu) {
        if (tok >= 0 && p.dl_dweight != nullptr) red_add_f32(p.dl_dweight + grow, dw_acc);
      }
      if ((EPI == kEpiScatter && !p.remote_out.enabled && p.tile_stripes_done != nullptr) ||
          (EPI == kEpiDswiglu && p.remote_dw.enabled)) {
        // Per-M-tile completion: the CTA that finishes the last N stripe of a tile does the
        // per-row bookkeeping once every stripe's writes are visible.
        __threadfence();
        epi_bar_sync();
        if (epi_tid == 0) *s_flag = (atom_add_acq_rel_gpu(p.tile_stripes_done + t.m_tile, 1) == p.num_n_tiles - 1);
        epi_bar_sync();
        const bool last = (*s_flag != 0);
        epi_bar_sync();
        if (last && tok >= 0 && half == 0) {
          if (EPI == kEpiScatter) {
            if (atom_add_acq_rel_gpu(p.k_remaining + tok, -1) == 1) {
              // The stand-alone combine of another GPU acquires this stamp at system scope and then reads the
              // row: the release must be at system scope too (device scope is enough with one rank).
              if (p.num_ranks > 1) { fence_acq_rel_sys(); st_release_sys(p.done_per_token + tok, p.seq); }
              else st_release_gpu(p.done_per_token + tok, p.seq);
            }
          } else {
            const int2 src = p.row_src[grow];
            const float v = *reinterpret_cast<volatile float*>(p.dl_dweight + grow);
            s_remote_dw[src.x][static_cast<long long>(src.y) * p.num_topk + p.row_k_slot[grow]] = v;
          }
        }
      }
    }
    if (lane == 0) bulk_wait_all();     // every bulk store this warp issued has been performed
    if (p.tail.enabled) __threadfence_system();
  } else if (has_gate_warp(EPI) && warp == kGemmWarps) {
    // ------------------------------------------------------------------ gate warp: polls tile gates ahead of the producer
    if (lane == 0 && p.mode == kVarlenM && p.arrival_count != nullptr) {
      const bool local_only = p.num_ranks == 1;   // every writer of the counters is on this GPU: device scope is enough
      int n = 0;
      for (int lin = first_lin; lin < total_tiles; lin += lin_stride) {
        const TileCoord t = decode_tile(p, lin, num_m);
        const int target = p.arrival_target[t.m_tile];
        const int* cnt = p.arrival_count + t.m_tile;
        if (!spin_until([&] { return (local_only ? ld_acquire_gpu(cnt) : ld_acquire_sys(cnt)) == target; }, budget, p.status)) {
          report_failure(p.status, kStatusTimeoutTileGate, kKernelGemm, 0, p.rank, t.m_tile, target, ld_acquire_sys(cnt));
          st_release_cta_shared(&s_gates_open, -1);
          break;
        }
        if (p.timing != nullptr) {
          long long* tm = p.timing + static_cast<size_t>(blockIdx.x) * kTimingCols;
          const long long now = static_cast<long long>(globaltimer_ns());
          if (n == 0) tm[2] = now;
        }
        st_release_cta_shared(&s_gates_open, ++n);
      }
    }
  } else if (PUSH) {
    // ------------------------------------------------------------------ dispatch push warps (mixed mode)
    // (with push-only CTAs in the grid these warps either stay idle or, split_local, ship the pairs that stay on
    // this rank: local copies drain fast and do not back up the load/store path)
    const bool local_walker = num_push_ctas > 0 && pp.split_local && pp.work_counter_local != nullptr;
    if ((pp.flags & 2) && (num_push_ctas == 0 || local_walker)) {
      const int pw = warp - base_warps(EPI);
      if (pw == 0 && lane < pp.num_ranks) {
        const unsigned long long* rec = pp.static_targets
            ? reinterpret_cast<const unsigned long long*>(&pp.own)
            : fetch_record(pp.peer_base[pp.rank], pp.ctl, pp.kind, pp.epoch, lane,
                           pp.wait_budget_ns, pp.status, kKernelDispatch, pp.rank);
        if (rec == nullptr) s_push_ok = 0;
        else resolve_push_targets(s_tg, lane, pp.peer_base[lane], rec);
      }
      asm volatile("bar.sync 2, %0;" :: "r"(push_warps(EPI) * 32) : "memory");
      if (s_push_ok && (pp.active_push_warps <= 0 || pw < pp.active_push_warps)) {
        const int num_send = *pp.num_send;
        const int num_chunks = push_num_chunks(pp, num_send);
        if (p.timing != nullptr && pw == 0 && lane == 0)
          p.timing[static_cast<size_t>(blockIdx.x) * kTimingCols + 4] = static_cast<long long>(globaltimer_ns());
        for (;;) {
          int chunk = 0;
          if (lane == 0) chunk = atomicAdd(local_walker ? pp.work_counter_local : pp.work_counter, 1);
          chunk = __shfl_sync(0xffffffffu, chunk, 0);
          if (chunk >= num_chunks) break;
          int p0, p1;
          push_chunk_range(pp, num_send, chunk, p0, p1);
          push_chunk(pp, s_tg, p0, p1, lane, nullptr, local_walker ? 1 : 0);
        }
        if (p.timing != nullptr && lane == 0) {
          long long* tm = p.timing + static_cast<size_t>(blockIdx.x) * kTimingCols;
          const unsigned long long now = globaltimer_ns();
          if (atomicMax(reinterpret_cast<unsigned long long*>(tm + 5), now) < now)   // this warp is the CTA's last one so far
            tm[3] = *reinterpret_cast<volatile int*>(&s_tiles_done);
        }
      }
    }
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before_sync();
  __syncthreads();
  if (p.timing != nullptr && threadIdx.x == 0)
    p.timing[static_cast<size_t>(blockIdx.x) * kTimingCols + 6] = static_cast<long long>(globaltimer_ns());
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
  if (dyn && threadIdx.x == 0) {     // the last CTA puts the claim counter back to zero for the next launch
    __threadfence();
    if (atomicAdd(p.tile_counter + 1, 1) == static_cast<int>(gridDim.x) - 1) { p.tile_counter[0] = 0; p.tile_counter[1] = 0; }
  }
  if (threadIdx.x == 0) {
    int* done_ctr = p.tail.enabled ? p.tail.ctas_done : (PUSH ? pp.blocks_done : nullptr);
    if (done_ctr != nullptr) {
      __threadfence();
      const int old = atomicAdd(done_ctr, 1);
      if (old == static_cast<int>(gridDim.x) - 1) {
        *done_ctr = 0;
        if (PUSH) { *pp.work_counter = 0; if (pp.work_counter_local != nullptr) *pp.work_counter_local = 0; }
        if (p.tail.enabled) {
          // Every CTA's remote reductions were fenced at system scope before it counted itself.
          __threadfence_system();
          for (int r = 0; r < p.num_ranks; ++r)
            flags_signal(p.peer_base, p.ctl, p.tail.kind, p.tail.epoch, p.rank, r);
          if (p.tail.wait)
            for (int r = 0; r < p.num_ranks; ++r)
              if (!flags_wait(p.peer_base[p.rank], p.ctl, p.tail.kind, p.tail.epoch, r,
                              p.wait_budget_ns, p.status, kKernelGemm, p.rank, kStatusTimeoutTail))
                break;
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Host dispatch over the template instances
// ---------------------------------------------------------------------------------------------
// maps of the second problem for the launch in progress on this host thread (null: none)
static thread_local const SecondMaps* t_maps2 = nullptr;

template <int BN, bool A_MN, bool B_MN, int EPI, bool PUSH>
static cudaError_t launch_instance(const GemmParams& p, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& to0,
                            const CUtensorMap& to1, const PushParams& pp, int num_ctas, cudaStream_t stream) {
  auto kernel = grouped_gemm_kernel<BN, A_MN, B_MN, EPI, PUSH>;
  // The shared-memory limit is an attribute of the function ON A DEVICE: raise it once per device.
  static std::atomic<bool> configured[kMaxDevices];
  const int smem = GemmCfg<BN>::kSmemBytes;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  if (!configured[dev].load(std::memory_order_acquire)) {
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    configured[dev].store(true, std::memory_order_release);
  }
  const int threads = (base_warps(EPI) + (PUSH ? push_warps(EPI) : 0)) * 32;
  SecondMaps none;
  if (t_maps2 == nullptr) { none.a = ta; none.b = tb; none.o = to0; }
  kernel<<<num_ctas, threads, smem, stream>>>(ta, tb, to0, to1, p, pp, t_maps2 != nullptr ? *t_maps2 : none);
  return cudaSuccess;
}

template <int BN, bool PUSH>
static bool dispatch_layout(const GemmParams& p, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& to0,
                            const CUtensorMap& to1, const PushParams& pp, int n, cudaStream_t s, cudaError_t& err) {
  if (p.mode == kVarlenM && !p.a_mn_major && !p.b_mn_major) {
    if (p.epilogue == kEpiSwiglu) { err = launch_instance<BN, false, false, kEpiSwiglu, PUSH>(p, ta, tb, to0, to1, pp, n, s); return true; }
    if (PUSH) return false;
    if constexpr (!PUSH) {
      if (p.epilogue == kEpiStore) { err = launch_instance<BN, false, false, kEpiStore, false>(p, ta, tb, to0, to1, pp, n, s); return true; }
      if (p.epilogue == kEpiScatter) { err = launch_instance<BN, false, false, kEpiScatter, false>(p, ta, tb, to0, to1, pp, n, s); return true; }
      if (p.epilogue == kEpiStoreF32) { err = launch_instance<BN, false, false, kEpiStoreF32, false>(p, ta, tb, to0, to1, pp, n, s); return true; }
    }
  }
  if (p.mode == kVarlenM && !p.a_mn_major && p.b_mn_major) {
    if (p.epilogue == kEpiDswiglu) { err = launch_instance<BN, false, true, kEpiDswiglu, PUSH>(p, ta, tb, to0, to1, pp, n, s); return true; }
    if constexpr (!PUSH) {
      if (p.epilogue == kEpiScatter) { err = launch_instance<BN, false, true, kEpiScatter, false>(p, ta, tb, to0, to1, pp, n, s); return true; }
      if (p.epilogue == kEpiStore) { err = launch_instance<BN, false, true, kEpiStore, false>(p, ta, tb, to0, to1, pp, n, s); return true; }
    }
  }
  if constexpr (!PUSH) {
    if (p.mode == kVarlenK && p.a_mn_major && p.b_mn_major && p.epilogue == kEpiStore) {
      err = launch_instance<BN, true, true, kEpiStore, false>(p, ta, tb, to0, to1, pp, n, s); return true;
    }
  }
  return false;
}

bool launch_grouped_gemm(const GemmParams& p, const void* tmap_a, const void* tmap_b, const void* tmap_o0,
                         const void* tmap_o1, const PushParams* fused_push, int num_ctas, cudaStream_t stream,
                         cudaError_t* setup_error, const void* maps2) {
  t_maps2 = static_cast<const SecondMaps*>(maps2);
  const CUtensorMap& ta = *static_cast<const CUtensorMap*>(tmap_a);
  const CUtensorMap& tb = *static_cast<const CUtensorMap*>(tmap_b);
  const CUtensorMap& to0 = *static_cast<const CUtensorMap*>(tmap_o0 ? tmap_o0 : tmap_a);
  const CUtensorMap& to1 = *static_cast<const CUtensorMap*>(tmap_o1 ? tmap_o1 : tmap_a);
  bool ok;
  cudaError_t err = cudaSuccess;
  if (fused_push != nullptr) {
    ok = (p.block_n == 256) ? dispatch_layout<256, true>(p, ta, tb, to0, to1, *fused_push, num_ctas, stream, err)
                            : dispatch_layout<128, true>(p, ta, tb, to0, to1, *fused_push, num_ctas, stream, err);
  } else {
    PushParams none{};
    ok = (p.block_n == 256) ? dispatch_layout<256, false>(p, ta, tb, to0, to1, none, num_ctas, stream, err)
                            : dispatch_layout<128, false>(p, ta, tb, to0, to1, none, num_ctas, stream, err);
  }
  t_maps2 = nullptr;
  if (setup_error != nullptr) *setup_error = err;
  return ok;
}

}  // namespace sep

// =============================================================================================
// Allocation-free entry point (declared and documented in no_alloc.h).
// =============================================================================================
namespace {

// Scratch of the no-alloc entry point: per-M-tile "N stripes finished" counters, followed by the status block the
// kernel's bounded waits report into.  In host code this name is only a handle for cudaGetSymbolAddress; the
// device address is resolved once per device.
constexpr int kNoAllocStatusInts = 64;    // 256 bytes: keeps the status block on its own 256-byte line
static __device__ __align__(256) int g_noalloc_scratch[kNoAllocMaxTiles + kNoAllocStatusInts];
static_assert(sizeof(sep::StatusBlock) <= kNoAllocStatusInts * sizeof(int), "status block must fit its slot");

int* g_noalloc_scratch_ptr[sep::kMaxDevices] = {};
std::mutex g_noalloc_setup_mutex;
thread_local char g_noalloc_error[256] = "";

int noalloc_fail(int code, const char* what, cudaError_t e = cudaSuccess) {
  if (e != cudaSuccess) snprintf(g_noalloc_error, sizeof(g_noalloc_error), "%s: %s", what, cudaGetErrorString(e));
  else snprintf(g_noalloc_error, sizeof(g_noalloc_error), "%s", what);
  return code;
}

using NoAllocEncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                     const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                     CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

bool noalloc_tmap(CUtensorMap* m, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint32_t b0, uint32_t b1) {
  static std::atomic<NoAllocEncodeFn> encode_fn{nullptr};
  NoAllocEncodeFn encode = encode_fn.load(std::memory_order_acquire);
  if (encode == nullptr) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess || fn == nullptr)
      return false;
    encode = reinterpret_cast<NoAllocEncodeFn>(fn);
    encode_fn.store(encode, std::memory_order_release);
  }
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {d0 * 2, d0 * d1 * 2};
  cuuint32_t box[3] = {b0, b1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  return encode(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Device address of the scratch array on the current device (resolved under a lock on first use).
int* noalloc_scratch(int dev, cudaError_t* e) {
  std::lock_guard<std::mutex> g(g_noalloc_setup_mutex);
  if (g_noalloc_scratch_ptr[dev] == nullptr) {
    int* ptr = nullptr;
    *e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_scratch);
    if (*e != cudaSuccess || ptr == nullptr) return nullptr;
    g_noalloc_scratch_ptr[dev] = ptr;
  }
  return g_noalloc_scratch_ptr[dev];
}

}  // namespace

extern "C" const char* streamep_noalloc_last_error(void) { return g_noalloc_error; }

extern "C" int streamep_noalloc_device_status(int* code, int* where) {
  using namespace sep;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return noalloc_fail(-3, "cudaGetDevice", e);
  if (dev < 0 || dev >= kMaxDevices) return noalloc_fail(-2, "device ordinal out of range");
  int* scratch = noalloc_scratch(dev, &e);
  if (scratch == nullptr) return noalloc_fail(-3, "cudaGetSymbolAddress(scratch)", e);
  StatusBlock h;
  e = cudaMemcpy(&h, scratch + kNoAllocMaxTiles, sizeof(h), cudaMemcpyDeviceToHost);   // waits for earlier work
  if (e != cudaSuccess) return noalloc_fail(-3, "cudaMemcpy(status)", e);
  if (code != nullptr) *code = h.code;
  if (where != nullptr) *where = h.where;
  return 0;
}

extern "C" int streamep_gemm_y_scatter_noalloc(const void* postact, const void* w2, const int* tile_id_to_expert,
                                               const float* pool_topk_weight, const int* pool_recv_token, void* o,
                                               int* k_local_remaining, long long* y_done_per_token, int total_tiles,
                                               int hidden, int ffn, int num_local_experts, long long seq, void* stream_v) {
  using namespace sep;
  g_noalloc_error[0] = 0;
  if (total_tiles < 0) return noalloc_fail(-2, "total_tiles must not be negative");
  if (total_tiles > kNoAllocMaxTiles)
    return noalloc_fail(-1, "total_tiles exceeds kNoAllocMaxTiles (32768): split the call or use the regular entry point");
  if (total_tiles == 0) return 0;
  if (!postact || !w2 || !tile_id_to_expert || !pool_topk_weight || !pool_recv_token || !o || !k_local_remaining || !y_done_per_token)
    return noalloc_fail(-2, "null pointer argument");
  if (hidden <= 0 || ffn <= 0 || hidden % 8 != 0 || ffn % 8 != 0 || num_local_experts <= 0)
    return noalloc_fail(-2, "hidden and ffn must be positive multiples of 8, num_local_experts positive");
  if (reinterpret_cast<uintptr_t>(postact) % 16 != 0 || reinterpret_cast<uintptr_t>(w2) % 16 != 0 || reinterpret_cast<uintptr_t>(o) % 16 != 0)
    return noalloc_fail(-2, "postact, w2 and o must be 16-byte aligned");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return noalloc_fail(-3, "cudaGetDevice", e);
  if (dev < 0 || dev >= kMaxDevices) return noalloc_fail(-2, "device ordinal out of range");
  // One-time set-up for this device (with it current): the device address behind the symbol.
  int* scratch = noalloc_scratch(dev, &e);
  if (scratch == nullptr) return noalloc_fail(-3, "cudaGetSymbolAddress(scratch)", e);

  const int block_n = (hidden % 256 == 0) ? 256 : ((hidden % 128 == 0) ? 128 : (hidden > 128 ? 256 : 128));
  const long long rows = static_cast<long long>(total_tiles) * BM;
  CUtensorMap ta, tb;
  if (!noalloc_tmap(&ta, postact, ffn, rows, 1, 64, BM) || !noalloc_tmap(&tb, w2, ffn, hidden, num_local_experts, 64, block_n))
    return noalloc_fail(-3, "cuTensorMapEncodeTiled failed");
  int sms = 0;
  e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) return noalloc_fail(-3, "cudaDeviceGetAttribute", e);

  // Nothing was enqueued so far.  The array keeps the previous call's counts and status: clear the part this call
  // uses (stream-ordered, so it cannot overtake an earlier call on the same stream).
  e = cudaMemsetAsync(scratch, 0, sizeof(int) * static_cast<size_t>(total_tiles), stream);
  if (e != cudaSuccess) return noalloc_fail(-3, "cudaMemsetAsync(scratch)", e);
  e = cudaMemsetAsync(scratch + kNoAllocMaxTiles, 0, sizeof(int) * kNoAllocStatusInts, stream);
  if (e != cudaSuccess) return noalloc_fail(-3, "cudaMemsetAsync(status)", e);

  GemmParams p{};
  p.mode = kVarlenM; p.epilogue = kEpiScatter; p.block_n = block_n;
  p.N = hidden; p.K = ffn; p.num_experts = num_local_experts; p.total_rows = static_cast<int>(rows);
  p.num_m_tiles = total_tiles; p.num_n_tiles = (hidden + block_n - 1) / block_n;
  p.tile_id_to_expert = tile_id_to_expert;
  p.row_weight = pool_topk_weight; p.row_token = pool_recv_token;
  p.scatter_local = o;
  p.tile_stripes_done = scratch; p.k_remaining = k_local_remaining; p.done_per_token = y_done_per_token; p.seq = seq;
  p.num_ranks = 1; p.rank = 0;
  p.status = reinterpret_cast<StatusBlock*>(scratch + kNoAllocMaxTiles);   // read back by streamep_noalloc_device_status
  p.wait_budget_ns = 2000000000ull;
  const long long total = static_cast<long long>(p.num_m_tiles) * p.num_n_tiles;
  const int ctas = static_cast<int>(total < sms ? total : sms);
  PushParams none{};
  e = (block_n == 256) ? launch_instance<256, false, false, kEpiScatter, false>(p, ta, tb, ta, ta, none, ctas, stream)
                       : launch_instance<128, false, false, kEpiScatter, false>(p, ta, tb, ta, ta, none, ctas, stream);
  if (e != cudaSuccess) return noalloc_fail(-3, "kernel set-up (shared-memory attribute)", e);
  e = cudaGetLastError();
  if (e != cudaSuccess) return noalloc_fail(-3, "kernel launch", e);
  return 0;
}
