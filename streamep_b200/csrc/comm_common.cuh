// Device helpers shared by the communication kernels and the fused GEMM kernels: control-region
// addressing, buffer-record publish/fetch, flag barriers and the row-push worker.
#pragma once

#include "api.h"
#include "ptx.cuh"

namespace sep {

__device__ __forceinline__ int* ctl_flag(void* base, const ControlLayout& ctl, int kind, int slot) {
  return reinterpret_cast<int*>(static_cast<char*>(base) + ctl.flags) + kind * kMaxRanks + slot;
}
__device__ __forceinline__ unsigned long long* ctl_mailbox(void* base, const ControlLayout& ctl, int kind,
                                                           int parity, int src) {
  return reinterpret_cast<unsigned long long*>(static_cast<char*>(base) + ctl.mailbox) +
         ((static_cast<size_t>(kind) * 2 + parity) * kMaxRanks + src) * kMailboxWords;
}
__device__ __forceinline__ int* ctl_inbox_counts(void* base, const ControlLayout& ctl, int parity, int src, int c) {
  return reinterpret_cast<int*>(static_cast<char*>(base) + ctl.inbox_counts) +
         ((static_cast<size_t>(parity) * kMaxRanks + src) * ctl.num_channels + c) * ctl.num_experts_cap;
}
__device__ __forceinline__ int* ctl_inbox_tokens(void* base, const ControlLayout& ctl, int parity, int src, int c) {
  return reinterpret_cast<int*>(static_cast<char*>(base) + ctl.inbox_tokens) +
         ((static_cast<size_t>(parity) * kMaxRanks + src) * ctl.num_channels + c) * kMaxRanks;
}

__device__ __forceinline__ int* ctl_inbox_misc(void* base, const ControlLayout& ctl, int parity, int src) {
  return reinterpret_cast<int*>(static_cast<char*>(base) + ctl.inbox_misc) + (static_cast<size_t>(parity) * kMaxRanks + src) * 4;
}

// Thread `p` (< num_ranks) of the calling group writes this rank's record into peer p's mailbox.
// The 15 payload words are plain stores; the stamp is a system-scope release store.
__device__ __forceinline__ void publish_record(const BufferRecord& rec, void* const* peer_base,
                                               const ControlLayout& ctl, int kind, int epoch, int rank, int p) {
  unsigned long long* dst = ctl_mailbox(peer_base[p], ctl, kind, epoch & 1, rank);
  const unsigned long long* src = reinterpret_cast<const unsigned long long*>(&rec);
#pragma unroll
  for (int i = 0; i < kMailboxWords - 1; ++i) dst[i] = src[i];
  st_release_sys(reinterpret_cast<long long*>(dst + kMailboxWords - 1), static_cast<long long>(epoch));
}

// Waits (bounded) until peer p's record for `epoch` is in this rank's mailbox; returns its address.
__device__ __forceinline__ const unsigned long long* fetch_record(void* own_base, const ControlLayout& ctl,
                                                                  int kind, int epoch, int p,
                                                                  unsigned long long budget_ns, StatusBlock* st,
                                                                  int kernel_id, int rank) {
  unsigned long long* box = ctl_mailbox(own_base, ctl, kind, epoch & 1, p);
  const long long* stamp = reinterpret_cast<const long long*>(box + kMailboxWords - 1);
  bool ok = spin_until([&] { return ld_acquire_sys(stamp) == static_cast<long long>(epoch); }, budget_ns, st);
  if (!ok) {
    report_failure(st, kStatusTimeoutMailbox, kernel_id, 0, rank, p, epoch,
                   static_cast<int>(ld_acquire_sys(stamp)));
    return nullptr;
  }
  return box;
}

// Flag handshake: thread p (< num_ranks) stores `epoch` into peer p's flag row (after the caller made
// its writes visible), then waits until peer p's store to this rank's row arrived.
__device__ __forceinline__ void flags_signal(void* const* peer_base, const ControlLayout& ctl, int kind,
                                             int epoch, int rank, int p) {
  st_release_sys(ctl_flag(peer_base[p], ctl, kind, rank), epoch);
}
__device__ __forceinline__ bool flags_wait(void* own_base, const ControlLayout& ctl, int kind, int epoch,
                                           int p, unsigned long long budget_ns, StatusBlock* st,
                                           int kernel_id, int rank, int code) {
  const int* f = ctl_flag(own_base, ctl, kind, p);
  bool ok = spin_until([&] { return ld_acquire_sys(f) >= epoch; }, budget_ns, st);
  if (!ok) report_failure(st, code, kernel_id, 1, rank, p, epoch, ld_acquire_sys(f));
  return ok;
}

// ---------------------------------------------------------------------------------------------
// Row push.  Pairs are shipped in the order of the send list: local expert index first, then the
// destination rank rotated by the sender's rank, then channel and token.  Every rank therefore fills
// local expert 0 of all owners first, which is the order in which the owners' GEMM kernels consume
// tiles, and at any time the senders are spread over all destinations.  A warp copies the row of
// each pair of its chunk into the pair's pool slot at the owning rank, writes the per-slot and
// per-recv-token scalars, and finally release-adds every (rank, tile) counter the chunk touched.
// `tg` holds per-rank absolute pointers resolved from the peers' records (shared memory).
// ---------------------------------------------------------------------------------------------
struct PushTargets {
  char* pool[kMaxRanks];
  float* pool_topk_weight[kMaxRanks];
  int* pool_recv_token[kMaxRanks];
  int* pool_k_slot[kMaxRanks];
  int2* pool_src[kMaxRanks];
  int* recv_token_to_slots[kMaxRanks];
  int* k_local_total[kMaxRanks];
  int* k_local_remaining[kMaxRanks];
  int2* recv_src[kMaxRanks];
  int* arrival_count[kMaxRanks];
};

__device__ __forceinline__ void resolve_push_targets(PushTargets& tg, int p, void* peer_base,
                                                     const unsigned long long* rec) {
  char* b = static_cast<char*>(peer_base);
  tg.pool[p] = b + rec[0];
  tg.pool_topk_weight[p] = reinterpret_cast<float*>(b + rec[1]);
  tg.pool_recv_token[p] = reinterpret_cast<int*>(b + rec[2]);
  tg.pool_k_slot[p] = reinterpret_cast<int*>(b + rec[3]);
  tg.pool_src[p] = reinterpret_cast<int2*>(b + rec[4]);
  tg.recv_token_to_slots[p] = reinterpret_cast<int*>(b + rec[5]);
  tg.k_local_total[p] = reinterpret_cast<int*>(b + rec[6]);
  tg.k_local_remaining[p] = reinterpret_cast<int*>(b + rec[7]);
  tg.arrival_count[p] = reinterpret_cast<int*>(b + rec[8]);
  tg.recv_src[p] = reinterpret_cast<int2*>(b + rec[9]);
}

// Chunking of the send list.  All push warps of a rank claim chunks from one counter, so at any time (warps x chunk
// bytes) are in flight and nothing completes before a whole chunk is through.  The first `head_chunks` chunks are
// therefore small (the consumers' first tiles complete after a short time); later chunks are larger, because every
// chunk ends with a release that waits for the warp's outstanding remote stores.
__device__ __forceinline__ int push_num_chunks(const PushParams& p, int num_send) {
  const int head_pairs = min(num_send, p.head_chunks * p.head_pairs_per_chunk);
  const int head = p.head_pairs_per_chunk > 0 ? (head_pairs + p.head_pairs_per_chunk - 1) / p.head_pairs_per_chunk : 0;
  return head + (num_send - head_pairs + p.pairs_per_chunk - 1) / p.pairs_per_chunk;
}
__device__ __forceinline__ void push_chunk_range(const PushParams& p, int num_send, int chunk, int& p0, int& p1) {
  const int head_pairs = min(num_send, p.head_chunks * p.head_pairs_per_chunk);
  const int head = p.head_pairs_per_chunk > 0 ? (head_pairs + p.head_pairs_per_chunk - 1) / p.head_pairs_per_chunk : 0;
  if (chunk < head) { p0 = chunk * p.head_pairs_per_chunk; p1 = min(p0 + p.head_pairs_per_chunk, head_pairs); }
  else { p0 = head_pairs + (chunk - head) * p.pairs_per_chunk; p1 = min(p0 + p.pairs_per_chunk, num_send); }
}

// One warp ships the pairs at positions [pos_begin, pos_end) of the send list (at most 32).  Lane j
// owns pair j of the chunk for the scalar work; the row copies are done by the whole warp, one pair
// after another (plain 16-byte loads and peer stores), or - `ring` != 0, push-only CTAs - by lane 0 through the
// bulk-copy engine: row pieces of up to kPushPieceBytes are loaded into a two-slot shared-memory ring and stored
// from there into the owner's pool, the next piece's load in flight while the current one is stored.
constexpr uint32_t kPushPieceBytes = 4096;
struct PushRing {
  uint32_t smem;        // shared-memory address of this warp's two slots (2 x kPushPieceBytes, 128-byte aligned), 0 = none
  uint64_t* bar;        // two mbarriers of this warp (count 1), initialised by the caller
  uint32_t phase;       // bit s = parity the next wait on slot s expects
  bool ok;              // false after a bounded wait on a load gave up
};

__device__ __forceinline__ void push_chunk(const PushParams& p, const PushTargets& tg, int pos_begin,
                                           int pos_end, int lane, PushRing* ring = nullptr, int filter = 0) {
  const int K = p.num_topk, R = p.num_ranks;
  const int e_local = p.num_experts / R;
  const size_t row_bytes = static_cast<size_t>(p.hidden) * 2;
  const int vec_per_row = p.hidden / 8;   // 16-byte vectors
  int n = pos_end - pos_begin;

  int t = -1, k = 0, slot = -1, dst = -1;
  if (lane < n) {
    const int pair = p.send_list[pos_begin + lane];
    t = pair / K; k = pair - t * K;
    const long long e = p.topk_idx[pair];
    slot = p.pair_slot[pair];
    dst = static_cast<int>(e / e_local);
  }
  if (filter != 0) {
    // Only the pairs of one kind are this walker's: compact them to the low lanes (order kept), the rest is left to
    // the walkers of the other kind, which go through the same list with a counter of their own.
    const bool mine = lane < n && ((filter == 1) == (dst == p.rank));
    const unsigned mask = __ballot_sync(0xffffffffu, mine);
    const int src_lane = __fns(mask, 0, lane + 1);          // lane of the (lane + 1)-th pair of this kind, or -1
    const int from = src_lane < 0 ? lane : src_lane;
    const int t2 = __shfl_sync(0xffffffffu, t, from), k2 = __shfl_sync(0xffffffffu, k, from);
    const int s2 = __shfl_sync(0xffffffffu, slot, from), d2 = __shfl_sync(0xffffffffu, dst, from);
    n = __popc(mask);
    if (lane < n) { t = t2; k = k2; slot = s2; dst = d2; } else { t = -1; k = 0; slot = -1; dst = -1; }
    if (n == 0) return;
  }
  if (ring != nullptr && ring->smem != 0) {
    const int pieces = static_cast<int>((row_bytes + kPushPieceBytes - 1) / kPushPieceBytes);
    const int total = n * pieces;
    const char* src_next = nullptr; char* dst_next = nullptr; uint32_t bytes_next = 0;
    auto piece = [&](int i, const char*& src, char*& dstp, uint32_t& bytes) {
      const int j = i / pieces, q = i - j * pieces;
      const int tj = __shfl_sync(0xffffffffu, t, j);
      const int sj = __shfl_sync(0xffffffffu, slot, j);
      const int dj = __shfl_sync(0xffffffffu, dst, j);
      const size_t off = static_cast<size_t>(q) * kPushPieceBytes;
      src = static_cast<const char*>(p.x) + static_cast<size_t>(tj) * row_bytes + off;
      dstp = tg.pool[dj] + static_cast<size_t>(sj) * row_bytes + off;
      bytes = static_cast<uint32_t>(min(static_cast<size_t>(kPushPieceBytes), row_bytes - off));
    };
    if (total > 0) {
      piece(0, src_next, dst_next, bytes_next);
      if (lane == 0) {
        bulk_wait_read();                                  // both slots are free again (stores of the previous chunk)
        mbar_arrive_expect_tx(&ring->bar[0], bytes_next);
        bulk_load_1d(ring->smem, src_next, bytes_next, &ring->bar[0]);
      }
    }
    for (int i = 0; i < total; ++i) {
      const int s = i & 1;
      char* dst_cur = dst_next; const uint32_t bytes_cur = bytes_next;
      if (i + 1 < total) piece(i + 1, src_next, dst_next, bytes_next);   // (shuffles: all lanes)
      int ok = 1;
      if (lane == 0) {
        if (i + 1 < total) {
          bulk_wait_read();                                // the other slot's store (piece i - 1) has read its data
          mbar_arrive_expect_tx(&ring->bar[s ^ 1], bytes_next);
          bulk_load_1d(ring->smem + (s ^ 1) * kPushPieceBytes, src_next, bytes_next, &ring->bar[s ^ 1]);
        }
        if (mbar_wait(&ring->bar[s], (ring->phase >> s) & 1u, p.wait_budget_ns, p.status)) {
          ring->phase ^= 1u << s;
          bulk_store_1d(dst_cur, ring->smem + s * kPushPieceBytes, bytes_cur);
          bulk_commit();
        } else {
          // give up: report, let the load that is still in flight land (bounded), and ship nothing more
          report_failure(p.status, kStatusTimeoutPipeline, p.is_grads ? kKernelDispatchGrads : kKernelDispatch, 3, p.rank, i, 0, 0);
          const unsigned long long t0 = globaltimer_ns();
          while (!mbar_try_wait(&ring->bar[s], (ring->phase >> s) & 1u) && globaltimer_ns() - t0 < 2000000ull) {}
          if (i + 1 < total)
            while (!mbar_try_wait(&ring->bar[s ^ 1], (ring->phase >> (s ^ 1)) & 1u) && globaltimer_ns() - t0 < 4000000ull) {}
          ring->ok = false;
          ok = 0;
        }
      }
      if (!__shfl_sync(0xffffffffu, ok, 0)) {               // warp-uniform exit; the chunk's tiles are NOT released
        if (lane == 0) bulk_wait_all();
        __syncwarp();
        return;
      }
    }
    if (lane == 0) {
      bulk_wait_all();          // every store of this chunk has been performed ...
      fence_proxy_async();      // ... and is ordered before the generic-proxy release below
    }
    __syncwarp();
  } else {
  for (int j = 0; j < n; ++j) {
    const int tj = __shfl_sync(0xffffffffu, t, j);
    const int sj = __shfl_sync(0xffffffffu, slot, j);
    const int dj = __shfl_sync(0xffffffffu, dst, j);
    const char* src_row = static_cast<const char*>(p.x) + static_cast<size_t>(tj) * row_bytes;
    char* dst_row = tg.pool[dj] + static_cast<size_t>(sj) * row_bytes;
    int v = lane;
    for (; v + 224 < vec_per_row; v += 256) {      // 8 x 16 bytes in flight per lane: one 4 KB row per pass
      uint4 a[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) a[u] = ld_nc_v4(src_row + static_cast<size_t>(v + 32 * u) * 16);
#pragma unroll
      for (int u = 0; u < 8; ++u) st_na_v4(dst_row + static_cast<size_t>(v + 32 * u) * 16, a[u]);
    }
    for (; v + 96 < vec_per_row; v += 128) {
      uint4 a0 = ld_nc_v4(src_row + static_cast<size_t>(v) * 16);
      uint4 a1 = ld_nc_v4(src_row + static_cast<size_t>(v + 32) * 16);
      uint4 a2 = ld_nc_v4(src_row + static_cast<size_t>(v + 64) * 16);
      uint4 a3 = ld_nc_v4(src_row + static_cast<size_t>(v + 96) * 16);
      st_na_v4(dst_row + static_cast<size_t>(v) * 16, a0);
      st_na_v4(dst_row + static_cast<size_t>(v + 32) * 16, a1);
      st_na_v4(dst_row + static_cast<size_t>(v + 64) * 16, a2);
      st_na_v4(dst_row + static_cast<size_t>(v + 96) * 16, a3);
    }
    for (; v < vec_per_row; v += 32)
      st_na_v4(dst_row + static_cast<size_t>(v) * 16, ld_nc_v4(src_row + static_cast<size_t>(v) * 16));
  }
  }
  if (!p.is_grads && lane < n) {
    const int r = p.send_recv_token[static_cast<size_t>(t) * R + dst];
    tg.pool_topk_weight[dst][slot] = p.topk_weights[static_cast<size_t>(t) * K + k];
    tg.pool_recv_token[dst][slot] = r;
    tg.pool_k_slot[dst][slot] = k;
    tg.pool_src[dst][slot] = make_int2(p.rank, t);
    tg.recv_token_to_slots[dst][static_cast<size_t>(r) * K + k] = slot;   // other k of this recv token stay -1
    // per-recv-token scalars: written by the first pair of this token that goes to `dst`
    int cnt = 0; bool first = true;
    for (int kk = 0; kk < K; ++kk) {
      const long long e2 = p.topk_idx[static_cast<size_t>(t) * K + kk];
      if (e2 >= 0 && static_cast<int>(e2 / e_local) == dst) { ++cnt; if (kk < k) first = false; }
    }
    if (first) {
      tg.k_local_total[dst][r] = cnt;
      tg.k_local_remaining[dst][r] = cnt;
      tg.recv_src[dst][r] = make_int2(p.rank, t);
    }
  }
  // Release the chunk: one add per distinct (rank, tile) the chunk touched.
  __syncwarp();
  const int key = (lane < n) ? ((dst << 24) | (slot / p.tile_m)) : (-1 - lane);
  const unsigned peers = __match_any_sync(0xffffffffu, key);
  if (lane < n && (__ffs(peers) - 1) == lane) {
    // with one rank the consumer is on this GPU and acquires at device scope: release at device scope
    if (R == 1) red_release_gpu_add(tg.arrival_count[dst] + slot / p.tile_m, __popc(peers));
    else red_release_sys_add(tg.arrival_count[dst] + slot / p.tile_m, __popc(peers));
  }
}

}  // namespace sep
