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
// Row push.  One warp ships `tokens_per_chunk` consecutive tokens: each token row is read once and
// written into the pool slot of every (token, k) pair at the owning rank, followed by the per-slot
// and per-recv-token scalars, and finally one release-add per touched (rank, tile) counter.
// `dst` holds per-rank absolute pointers resolved from the peers' records (shared memory).
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

__device__ __forceinline__ void push_chunk(const PushParams& p, const PushTargets& tg, int tok_begin,
                                           int tok_end, int lane) {
  const int K = p.num_topk, R = p.num_ranks;
  const int e_local = p.num_experts / R;
  const size_t row_bytes = static_cast<size_t>(p.hidden) * 2;
  const int vec_per_row = p.hidden / 8;   // 16-byte vectors

  for (int t = tok_begin; t < tok_end; ++t) {
    // lane k (< K) owns pair (t, k)
    int slot = -1, dst = -1;
    if (lane < K) {
      long long e = p.topk_idx[static_cast<size_t>(t) * K + lane];
      slot = p.pair_slot[static_cast<size_t>(t) * K + lane];
      if (e >= 0 && slot >= 0) dst = static_cast<int>(e / e_local); else slot = -1;
    }
    // row copy: every 16-byte vector is loaded once and stored to each pair's slot
    const char* src_row = static_cast<const char*>(p.x) + static_cast<size_t>(t) * row_bytes;
    for (int k = 0; k < K; ++k) {
      const int s = __shfl_sync(0xffffffffu, slot, k);
      const int d = __shfl_sync(0xffffffffu, dst, k);
      if (s < 0) continue;
      char* dst_row = tg.pool[d] + static_cast<size_t>(s) * row_bytes;
      int v = lane;
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
    if (!p.is_grads) {
      if (slot >= 0) {
        const int r = p.send_recv_token[static_cast<size_t>(t) * R + dst];
        tg.pool_topk_weight[dst][slot] = p.topk_weights[static_cast<size_t>(t) * K + lane];
        tg.pool_recv_token[dst][slot] = r;
        tg.pool_k_slot[dst][slot] = lane;
        tg.pool_src[dst][slot] = make_int2(p.rank, t);
      }
      // per-recv-token scalars at every destination rank of this token
      for (int d = 0; d < R; ++d) {
        const int r = p.send_recv_token[static_cast<size_t>(t) * R + d];
        if (r < 0) continue;
        const unsigned mine = __ballot_sync(0xffffffffu, slot >= 0 && dst == d);
        if (lane < K) tg.recv_token_to_slots[d][static_cast<size_t>(r) * K + lane] = (dst == d) ? slot : -1;
        if (lane == 0) {
          const int cnt = __popc(mine);
          tg.k_local_total[d][r] = cnt;
          tg.k_local_remaining[d][r] = cnt;
          tg.recv_src[d][r] = make_int2(p.rank, t);
        }
      }
    }
  }
  // Release the chunk: one add per distinct (rank, tile) the chunk touched.
  __syncwarp();
  const int n_pairs = (tok_end - tok_begin) * K;
  for (int base = 0; base < n_pairs; base += 32) {
    const int i = base + lane;
    int key = -1 - lane;   // unique per lane when there is nothing to count
    int d = -1, tile = -1;
    if (i < n_pairs) {
      const size_t idx = static_cast<size_t>(tok_begin) * K + i;
      const long long e = p.topk_idx[idx];
      const int s = p.pair_slot[idx];
      if (e >= 0 && s >= 0) {
        d = static_cast<int>(e / e_local);
        tile = s / p.tile_m;
        key = (d << 24) | tile;
      }
    }
    const unsigned peers = __match_any_sync(0xffffffffu, key);
    if (d >= 0 && (__ffs(peers) - 1) == lane) red_release_sys_add(tg.arrival_count[d] + tile, __popc(peers));
  }
}

}  // namespace sep
