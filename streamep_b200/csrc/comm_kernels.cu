// Communication kernels: dispatch metadata (count exchange + deterministic pool layout), tile
// metadata fill, push dispatch (forward rows / backward gradient rows), pull combine, device
// barrier, test tile producer and pool <-> recv row copies.
//
// Design (differs from the reference on purpose): there are no ring buffers and no receiver
// CTAs.  Every rank learns all ranks' per-(channel, expert) pair counts, derives every
// destination's pool layout itself, and pushes each token row straight into its final pool slot
// in the owner's HBM with 16-byte peer stores, then release-adds the owner's per-tile arrival
// counter.  Reference counterparts: csrc/kernels/intranode.cu:124-440 (metadata), :551-599 (tile
// fill), :601-1106 (dispatch), :1161-1439 (dispatch_grads), :1505-1880 (combine),
// csrc/kernels/runtime.cu:18-31 (barrier).
#include <cstdio>

#include "comm_common.cuh"

namespace sep {

// SM count of the current device (cached per device): grids are sized from it, never from a constant.
static int sm_count() {
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 1;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 1;
    cached[dev] = n;
  }
  return cached[dev];
}

ControlLayout make_control_layout(int num_ranks, int num_channels, int num_experts_cap) {
  ControlLayout c{};
  c.num_ranks = num_ranks;
  c.num_channels = num_channels;
  c.num_experts_cap = num_experts_cap;
  size_t off = 0;
  auto take = [&](size_t bytes) { size_t o = off; off += (bytes + 255) / 256 * 256; return o; };
  c.flags = take(sizeof(int) * kNumKinds * kMaxRanks);
  c.mailbox = take(sizeof(unsigned long long) * kNumKinds * 2 * kMaxRanks * kMailboxWords);
  c.inbox_counts = take(sizeof(int) * 2 * kMaxRanks * num_channels * num_experts_cap);
  c.inbox_tokens = take(sizeof(int) * 2 * kMaxRanks * num_channels * kMaxRanks);
  c.inbox_misc = take(sizeof(int) * 2 * kMaxRanks * 4);
  c.total_bytes = off;
  return c;
}

// =============================================================================================
// Metadata
// =============================================================================================
constexpr int kMetaThreads = 1024;

__device__ __forceinline__ int warp_excl_scan(int v, int lane, int& total) {
  int x = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int y = __shfl_up_sync(0xffffffffu, x, o);
    if (lane >= o) x += y;
  }
  total = __shfl_sync(0xffffffffu, x, 31);
  return x - v;
}

__global__ void __launch_bounds__(kMetaThreads, 1) dispatch_metadata_kernel(const MetadataParams p) {
  __shared__ int s_hist[kMaxExperts];          // phase A: running per-expert count; phase B: freq
  __shared__ int s_off[kMaxExperts];           // phase B: tile offset of each expert inside its owner
  __shared__ int s_u[kMaxRanks];               // phase A: per-dst token count of this channel
  __shared__ int s_U[kMaxRanks][kMaxRanks];    // phase B: tokens from src to dst
  __shared__ int s_total_tiles[kMaxRanks];
  __shared__ int s_is_last;
  __shared__ int s_ok;
  __shared__ int s_bad;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int R = p.num_ranks, K = p.num_topk, E = p.num_experts, C = p.num_channels;
  const int EL = E / R, T = p.num_tokens;
  const int parity = p.epoch & 1;
  const int per = (T + C - 1) / C;
  void* own = p.peer_base[p.rank];

  if (p.phase_mask == 4) {
    // ---------------------------------------------------------------- materialise (own launch, any grid)
    const size_t gid = static_cast<size_t>(blockIdx.x) * blockDim.x + tid, gsz = static_cast<size_t>(gridDim.x) * blockDim.x;
    // The synthesize launch before this one gave up (a peer never arrived): the base tables were
    // never written, so there is nothing valid to materialise.
    const int num_send = *reinterpret_cast<const volatile int*>(p.num_send);
    if (num_send < 0) return;
    if (p.region_id >= 0) {
      // Capacity mode: the tile arrays cover the whole region; tiles past the live count get target 0.
      const int live = p.dev_sizes[0];
      for (size_t t = gid; t < static_cast<size_t>(p.tiles_cap); t += gsz) {
        int e = 0, target = 0;
        if (static_cast<int>(t) < live) {
          while (e + 1 < EL && p.expert_pool_block_offset[e + 1] <= static_cast<int>(t)) ++e;
          target = min(p.tile_m, p.expert_frequency[e] - (static_cast<int>(t) - p.expert_pool_block_offset[e]) * p.tile_m);
        }
        p.tile_id_to_expert[t] = e;
        p.pool_arrival_target[t] = target;
      }
      if (p.dev_sizes[2] != 0) {   // the dispatch was turned into an empty one: nothing is sent anywhere
        for (size_t i = gid; i < static_cast<size_t>(T) * K; i += gsz) p.pair_slot[i] = -1;
        for (size_t i = gid; i < static_cast<size_t>(T) * R; i += gsz) p.send_recv_token[i] = -1;
        return;
      }
    }
    for (size_t i = gid; i < static_cast<size_t>(T) * K; i += gsz) {
      const int t = static_cast<int>(i / K);
      const long long e = p.topk_idx[i];
      int slot = -1;
      if (e >= 0 && e < E) {
        const int c = t / per;
        const int rk = p.pair_rank[i];
        slot = p.send_base[static_cast<size_t>(c) * E + e] + rk;
        const int pos = p.send_order_base[static_cast<size_t>(c) * E + e] + rk;
        if (pos >= 0 && pos < num_send) p.send_list[pos] = static_cast<int>(i);
        else report_failure(p.status, kStatusBadIndex, kKernelMetadata, 4, p.rank, static_cast<int>(i), num_send, pos);
      }
      p.pair_slot[i] = slot;
    }
    for (size_t i = gid; i < static_cast<size_t>(T) * R; i += gsz) {
      const int t = static_cast<int>(i / R), d = static_cast<int>(i - static_cast<size_t>(t) * R);
      const int rk = p.token_rank_in_channel[i];
      p.send_recv_token[i] = rk < 0 ? -1 : p.send_token_base[(t / per) * R + d] + rk;
    }
    return;
  }
  if (p.phase_mask & 1) {
    const int c = blockIdx.x;
    const int lo = min(per * c, T), hi = min(lo + per, T);
    for (int e = tid; e < E; e += blockDim.x) s_hist[e] = 0;
    if (tid < kMaxRanks) s_u[tid] = 0;
    __syncthreads();
    if (warp == 0) {
      // Order-preserving rank of every pair inside its (channel, expert) substream.
      const int n = (hi - lo) * K;
      // eight steps' worth of expert ids are fetched at once: one dependent global load per step would make this
      // warp, the slowest of the block, wait ~40 times in a row
      for (int base0 = 0; base0 < n; base0 += 256) {
        long long ev[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int i = base0 + j * 32 + lane;
          ev[j] = (i < n) ? p.topk_idx[static_cast<size_t>(lo) * K + i] : -1;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int base = base0 + j * 32;
          if (base >= n) break;
          const int i = base + lane;
          const long long e = ev[j];
          const bool valid = (e >= 0 && e < E);
          const int key = valid ? static_cast<int>(e) : (-1 - lane);
          const unsigned peers = __match_any_sync(0xffffffffu, key);
          int rank_in = -1;
          if (valid) {
            rank_in = s_hist[e] + __popc(peers & ((1u << lane) - 1u));
          }
          __syncwarp();
          if (valid && (__ffs(peers) - 1) == lane) s_hist[e] += __popc(peers);
          __syncwarp();
          if (i < n) p.pair_rank[static_cast<size_t>(lo) * K + i] = rank_in;
        }
      }
    } else if (warp <= R) {
      // Order-preserving rank of every token among the channel's tokens that go to rank d.
      const int d = warp - 1;
      int run = 0;
      for (int base = lo; base < hi; base += 32) {
        const int t = base + lane;
        bool hit = false;
        if (t < hi) {
          for (int k = 0; k < K; ++k) {
            const long long e = p.topk_idx[static_cast<size_t>(t) * K + k];
            hit |= (e >= 0 && e < E && static_cast<int>(e / EL) == d);
          }
        }
        const unsigned m = __ballot_sync(0xffffffffu, hit);
        if (t < hi) {
          // position in the (channel, dst) stream; a token that is not sent records where the next
          // sent one will sit, encoded as -(position) - 1
          const int pos = run + __popc(m & ((1u << lane) - 1u));
          p.token_rank_in_channel[static_cast<size_t>(t) * R + d] = hit ? pos : -1;
          p.send_head[static_cast<size_t>(t) * R + d] = hit ? pos : -pos - 1;
          p.is_token_in_rank[static_cast<size_t>(t) * R + d] = hit ? 1 : 0;
        }
        run += __popc(m);
      }
      if (lane == 0) s_u[d] = run;
    }
    __syncthreads();
    // Ship this channel's count rows to every rank (own included).
    for (int i = tid; i < R * E; i += blockDim.x) {
      const int peer = i / E, e = i - peer * E;
      ctl_inbox_counts(p.peer_base[peer], p.ctl, parity, p.rank, c)[e] = s_hist[e];
    }
    if (tid < R * kMaxRanks) {
      const int peer = tid / kMaxRanks, d = tid % kMaxRanks;
      ctl_inbox_tokens(p.peer_base[peer], p.ctl, parity, p.rank, c)[d] = (d < R) ? s_u[d] : 0;
    }
    if (c == 0 && tid < R) ctl_inbox_misc(p.peer_base[tid], p.ctl, parity, p.rank)[0] = p.region_id;
    fence_acq_rel_sys();      // this thread's rows are ordered before the flag the last block stores below
    __syncthreads();
    if (tid == 0) {
      const int old = atomicAdd(p.blocks_done, 1);
      s_is_last = (old == static_cast<int>(gridDim.x) - 1);
    }
    __syncthreads();
    if (!s_is_last) return;
    fence_acq_rel_sys();
    if (tid < R) flags_signal(p.peer_base, p.ctl, kKindMetadata, p.epoch, p.rank, tid);
    if (tid == 0) *p.blocks_done = 0;
    if (!(p.phase_mask & 2)) return;
  } else if (blockIdx.x != 0) {
    return;
  }

  // ------------------------------------------------------------------ phase B (one block)
  if (tid == 0) { s_ok = 1; s_bad = 0; }
  __syncthreads();
  if (tid < R) {
    if (!flags_wait(own, p.ctl, kKindMetadata, p.epoch, tid, p.wait_budget_ns, p.status, kKernelMetadata,
                    p.rank, kStatusTimeoutBarrier))
      s_ok = 0;
  }
  __syncthreads();
  if (!s_ok) {
    if (tid == 0) {   // unblock the host poll with an error marker; the materialise launch must do nothing
      *p.num_send = -1;
      p.host->total_tiles = -1;
      p.host->num_recv_tokens = -1;
      __threadfence_system();
      p.host->epoch = p.epoch;
    }
    return;
  }
  const int num_warps = blockDim.x >> 5;
  // 1. expert frequencies over all sources and channels
  for (int e = warp; e < E; e += num_warps) {
    int acc = 0;
    for (int i = lane; i < R * C; i += 32) {
      const int s = i / C, c = i - s * C;
      acc += ctl_inbox_counts(own, p.ctl, parity, s, c)[e];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) s_hist[e] = acc;
  }
  // tokens from s to d
  if (tid < R * R) {
    const int s = tid / R, d = tid % R;
    int acc = 0;
    for (int c = 0; c < C; ++c) acc += ctl_inbox_tokens(own, p.ctl, parity, s, c)[d];
    s_U[s][d] = acc;
  }
  __syncthreads();
  // 2. per-owner tile offsets
  if (tid < R) {
    int run = 0;
    for (int el = 0; el < EL; ++el) {
      const int e = tid * EL + el;
      s_off[e] = run;
      run += (s_hist[e] + p.tile_m - 1) / p.tile_m;
    }
    s_total_tiles[tid] = run;
    p.peer_total_tiles[tid] = run;
    int recv = 0;
    for (int s = 0; s < R; ++s) recv += s_U[s][tid];
    p.peer_num_recv[tid] = recv;
  }
  __syncthreads();
  // 2b. every rank took the same region, and (capacity mode) every rank's layout fits it.  All ranks evaluate the
  //     same numbers, so they all come to the same conclusion and all turn a bad dispatch into an empty one.
  if (tid < R) {
    int bad = 0;
    if (ctl_inbox_misc(own, p.ctl, parity, tid)[0] != p.region_id) bad |= 2;
    if (p.region_id >= 0 && (s_total_tiles[tid] > p.tiles_cap || p.peer_num_recv[tid] > p.recv_cap)) bad |= 1;
    if (bad) atomicOr(&s_bad, bad);
  }
  __syncthreads();
  if (s_bad) {
    if (tid == 0) {
      int need_tiles = 0, need_recv = 0;
      for (int r = 0; r < R; ++r) { need_tiles = max(need_tiles, s_total_tiles[r]); need_recv = max(need_recv, p.peer_num_recv[r]); }
      report_note(p.status, (s_bad & 2) ? kStatusRegionMismatch : kStatusOverflow, kKernelMetadata, 1, p.rank,
                  p.region_id, (s_bad & 2) ? p.region_id : p.tiles_cap, need_tiles);
      *p.num_send = 0;
      if (p.dev_sizes != nullptr) { p.dev_sizes[0] = 0; p.dev_sizes[1] = 0; p.dev_sizes[2] = 1; }
      if (p.host_overflow != nullptr) {
        p.host_overflow->needed_tiles = need_tiles;
        p.host_overflow->needed_recv = need_recv;
        p.host_overflow->epoch = p.epoch;
        __threadfence_system();
        p.host_overflow->count = p.host_overflow->count + 1;
      }
      p.expert_pool_block_offset[EL] = 0;
      // an exact-mode host is polling for the sizes: hand it the error marker
      p.host->total_tiles = (p.region_id >= 0) ? 0 : -1;
      p.host->num_recv_tokens = (p.region_id >= 0) ? 0 : -1;
      __threadfence_system();
      p.host->epoch = p.epoch;
    }
    if (tid < EL) { p.expert_frequency[tid] = 0; p.expert_pool_block_offset[tid] = 0; }
    if (tid < R) { p.peer_total_tiles[tid] = 0; p.peer_num_recv[tid] = 0; }
    return;
  }
  // 3. host-visible sizes first, so the host poll overlaps the rest of this kernel
  const bool host_polls = p.region_id < 0;     // capacity mode: nobody reads the sizes on the host, skip the PCIe writes
  if (tid < EL) {
    if (host_polls) p.host->recv_per_expert[tid] = s_hist[p.rank * EL + tid];
    p.expert_frequency[tid] = s_hist[p.rank * EL + tid];
    p.expert_pool_block_offset[tid] = s_off[p.rank * EL + tid];
  }
  if (tid == 0) {
    p.expert_pool_block_offset[EL] = s_total_tiles[p.rank];
    int recv = 0;
    for (int s = 0; s < R; ++s) recv += s_U[s][p.rank];
    if (host_polls) { p.host->total_tiles = s_total_tiles[p.rank]; p.host->num_recv_tokens = recv; }
    if (p.dev_sizes != nullptr) { p.dev_sizes[0] = s_total_tiles[p.rank]; p.dev_sizes[1] = recv; p.dev_sizes[2] = 0; }
  }
  __syncthreads();
  if (tid == 0 && host_polls) {
    __threadfence_system();
    p.host->epoch = p.epoch;
  }
  // 4. substream bases: exclusive scan over (channel, source) in lexicographic order
  for (int e = warp; e < E; e += num_warps) {
    const int owner = e / EL, el = e - owner * EL;
    int carry = s_off[e] * p.tile_m;
    for (int base = 0; base < C * R; base += 32) {
      const int i = base + lane;
      int c = 0, s = 0, v = 0;
      if (i < C * R) {
        c = i / R; s = i - c * R;
        v = ctl_inbox_counts(own, p.ctl, parity, s, c)[e];
      }
      int total;
      const int excl = warp_excl_scan(v, lane, total);
      if (i < C * R) {
        if (owner == p.rank) {
          p.base_pool[(static_cast<size_t>(c) * R + s) * EL + el] = carry + excl;
          p.seen_per_substream[(static_cast<size_t>(c) * R + s) * EL + el] = v;
        }
        if (s == p.rank) p.send_base[static_cast<size_t>(c) * E + e] = carry + excl;
      }
      carry += total;
    }
  }
  // 5. token-id bases and the prefix matrices of the handle: one warp per rank, 32 channels per step (a single
  //    thread walking the channels waits for one dependent global load per channel, 2 x 40 of them)
  if (warp < R) {
    const int d = warp;            // sender view: destination d
    int before = 0;
    for (int s = 0; s < p.rank; ++s) before += s_U[s][d];
    int carry = 0;
    for (int base = 0; base < C; base += 32) {
      const int c = base + lane;
      const int u = (c < C) ? ctl_inbox_tokens(own, p.ctl, parity, p.rank, c)[d] : 0;
      int total;
      const int excl = warp_excl_scan(u, lane, total);
      if (c < C) {
        p.send_token_base[c * R + d] = before + carry + excl;
        p.channel_prefix_matrix[d * C + c] = carry + excl + u;
      }
      carry += total;
    }
    const int s = warp;            // receiver view: source s
    int cum = 0;
    for (int ss = 0; ss <= s; ++ss) cum += s_U[ss][p.rank];
    if (lane < R) p.rank_prefix_matrix[s * R + lane] = (lane == p.rank) ? cum : 0;
    carry = 0;
    for (int base = 0; base < C; base += 32) {
      const int c = base + lane;
      const int u = (c < C) ? ctl_inbox_tokens(own, p.ctl, parity, s, c)[p.rank] : 0;
      int total;
      const int excl = warp_excl_scan(u, lane, total);
      if (c < C) p.recv_channel_prefix_matrix[s * C + c] = carry + excl + u;
      carry += total;
    }
  }
  // 6. push order of this rank's pairs (p.push_order).
  //    0: experts sorted by (local index, destination rank rotated by this rank), channels in order inside an
  //       expert: long runs per destination.  s_off is reused as the per-expert base.
  //    1: local expert index, then channel, then rotated destination, see below.
  if (p.push_order == 0) {
    __syncthreads();
    for (int e = tid; e < E; e += blockDim.x) {
      int cnt = 0;
      for (int c = 0; c < C; ++c) cnt += ctl_inbox_counts(own, p.ctl, parity, p.rank, c)[e];
      const int d = e / EL, el = e - d * EL;
      s_hist[el * R + ((d - p.rank + R) % R)] = cnt;     // keyed by push order
    }
    __syncthreads();
    if (warp == 0) {
      int carry = 0;
      for (int base = 0; base < E; base += 32) {
        const int i = base + lane;
        const int v = (i < E) ? s_hist[i] : 0;
        int total;
        const int excl = warp_excl_scan(v, lane, total);
        if (i < E) s_off[i] = carry + excl;
        carry += total;
      }
      if (lane == 0) *p.num_send = carry;
    }
    __syncthreads();
    for (int e = tid; e < E; e += blockDim.x) {
      const int d = e / EL, el = e - d * EL;
      int run = s_off[el * R + ((d - p.rank + R) % R)];
      for (int c0 = 0; c0 < C; c0 += 8) {     // eight loads in flight, then eight stores (a store per load would serialise them)
        int v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = (c0 + j < C) ? ctl_inbox_counts(own, p.ctl, parity, p.rank, c0 + j)[e] : 0;
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (c0 + j < C) { p.send_order_base[static_cast<size_t>(c0 + j) * E + e] = run; run += v[j]; }
      }
    }
    return;
  }
  // 6. push order of this rank's pairs: local expert index first, then channel, then destination rank (rotated
  //    by this rank so that the sources do not all write to the same peer at once).  Slots inside an expert
  //    are laid out channel-major on every destination, so this order sends the rows of tile 0 of expert 0 of
  //    every destination first, then tile 1, ...: all sources fill the same tiles at the same time and tiles
  //    complete in the order the GEMM consumes them, from the first microseconds of the push.
  //    s_hist[el] = pairs of local expert index el over all destinations; s_off[el] = its exclusive prefix.
  __syncthreads();
  for (int el = warp; el < EL; el += num_warps) {
    int acc = 0;
    for (int i = lane; i < C * R; i += 32) {
      const int c = i / R, d = i - c * R;
      acc += ctl_inbox_counts(own, p.ctl, parity, p.rank, c)[d * EL + el];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) s_hist[el] = acc;
  }
  __syncthreads();
  if (warp == 0) {
    int carry = 0;
    for (int base = 0; base < EL; base += 32) {
      const int i = base + lane;
      const int v = (i < EL) ? s_hist[i] : 0;
      int total;
      const int excl = warp_excl_scan(v, lane, total);
      if (i < EL) s_off[i] = carry + excl;
      carry += total;
    }
    if (lane == 0) *p.num_send = carry;
  }
  __syncthreads();
  for (int el = warp; el < EL; el += num_warps) {
    int carry = s_off[el];
    for (int base = 0; base < C * R; base += 32) {
      const int i = base + lane;
      const int c = i / R, drot = i - c * R;
      const int d = (drot + p.rank) % R;
      const int v = (i < C * R) ? ctl_inbox_counts(own, p.ctl, parity, p.rank, c)[d * EL + el] : 0;
      int total;
      const int excl = warp_excl_scan(v, lane, total);
      if (i < C * R) p.send_order_base[static_cast<size_t>(c) * E + d * EL + el] = carry + excl;
      carry += total;
    }
  }
}

void launch_dispatch_metadata(const MetadataParams& p, cudaStream_t stream) {
  if (p.phase_mask & 3) {
    MetadataParams q = p;
    q.phase_mask = p.phase_mask & 3;
    const int grid = (q.phase_mask & 1) ? p.num_channels : 1;
    dispatch_metadata_kernel<<<grid, kMetaThreads, 0, stream>>>(q);
  }
  if (p.phase_mask & 2) {   // destination slots, recv-token ids and the send list, spread over many blocks
    MetadataParams q = p;
    q.phase_mask = 4;
    const long long work = static_cast<long long>(p.num_tokens) * max(p.num_topk, p.num_ranks);
    long long blocks = (work + 1023) / 1024;
    if (blocks < 1) blocks = 1;
    if (blocks > sm_count()) blocks = sm_count();
    const int grid = static_cast<int>(blocks);
    dispatch_metadata_kernel<<<grid, kMetaThreads, 0, stream>>>(q);
  }
}

// =============================================================================================
// Tile metadata + defaults of everything peers will write into
// =============================================================================================
__global__ void fill_tile_metadata_kernel(const FillParams p) {
  const int gid = blockIdx.x * blockDim.x + threadIdx.x;
  const int stride = gridDim.x * blockDim.x;
  for (int t = gid; t < p.total_tiles; t += stride) {
    if (p.tile_id_to_expert != nullptr) {   // (capacity mode fills the tile arrays in the metadata kernel)
      int e = 0;
      while (e + 1 < p.num_local_experts && p.expert_pool_block_offset[e + 1] <= t) ++e;
      const int j = t - p.expert_pool_block_offset[e];
      p.tile_id_to_expert[t] = e;
      p.pool_arrival_target[t] = min(p.tile_m, p.expert_frequency[e] - j * p.tile_m);
    }
    p.pool_arrival_count[t] = 0;
  }
  for (int i = gid; i < p.tk_padded; i += stride) {
    p.pool_recv_token[i] = -1;
    p.pool_k_slot[i] = -1;
    p.pool_src[i] = make_int2(-1, -1);
    p.pool_topk_weight[i] = 0.f;
  }
  for (int i = gid; i < p.num_recv_tokens; i += stride) {
    p.k_local_total[i] = 0;
    p.k_local_remaining[i] = 0;
    p.y_done_per_token[i] = 0;
    p.recv_src[i] = make_int2(-1, -1);
  }
  for (size_t i = gid; i < static_cast<size_t>(p.num_recv_tokens) * p.num_topk; i += stride)
    p.recv_token_to_slots[i] = -1;
}

void launch_fill_tile_metadata(const FillParams& p, cudaStream_t stream) {
  const int work = max(max(p.tk_padded, p.num_recv_tokens * p.num_topk), 1);
  const int grid = min((work + 255) / 256, 4 * sm_count());
  fill_tile_metadata_kernel<<<grid, 256, 0, stream>>>(p);
}

// =============================================================================================
// Push dispatch
// =============================================================================================
constexpr int kPushThreads = 512;

__global__ void __launch_bounds__(kPushThreads, 1) dispatch_push_kernel(const PushParams p) {
  __shared__ PushTargets s_tg;
  __shared__ int s_ok;
  const int tid = threadIdx.x, lane = tid & 31;
  const int R = p.num_ranks;
  void* own = p.peer_base[p.rank];

  if (blockIdx.x == 0 && tid == 0 && p.started_flag != nullptr) atomicAdd(p.started_flag, 1);
  if ((p.flags & 1) && !p.static_targets && blockIdx.x == 0 && tid < R)
    publish_record(p.own, p.peer_base, p.ctl, p.kind, p.epoch, p.rank, tid);
  if (tid == 0) s_ok = 1;
  __syncthreads();

  if (p.flags & 2) {
    if (tid < R) {
      const unsigned long long* rec = p.static_targets
          ? reinterpret_cast<const unsigned long long*>(&p.own)
          : fetch_record(own, p.ctl, p.kind, p.epoch, tid, p.wait_budget_ns, p.status,
                         p.is_grads ? kKernelDispatchGrads : kKernelDispatch, p.rank);
      if (rec == nullptr) s_ok = 0;
      else resolve_push_targets(s_tg, tid, p.peer_base[tid], rec);
    }
    __syncthreads();
    if (s_ok) {
      const int num_send = *p.num_send;
      const int num_chunks = push_num_chunks(p, num_send);
      for (;;) {
        int chunk = 0;
        if (lane == 0) chunk = atomicAdd(p.work_counter, 1);
        chunk = __shfl_sync(0xffffffffu, chunk, 0);
        if (chunk >= num_chunks) break;
        int p0, p1;
        push_chunk_range(p, num_send, chunk, p0, p1);
        push_chunk(p, s_tg, p0, p1, lane);
      }
    }
  }

  if ((p.flags & 4) && s_ok) {
    // All rows addressed to this rank have landed once every own tile reached its target.
    const int gid = blockIdx.x * blockDim.x + tid;
    for (int t = gid; t < p.own_total_tiles; t += gridDim.x * blockDim.x) {
      const int target = p.own_arrival_target[t];
      const int* cnt = p.own_arrival_count + t;
      if (!spin_until([&] { return ld_acquire_sys(cnt) == target; }, p.wait_budget_ns, p.status)) {
        report_failure(p.status, kStatusTimeoutTail, p.is_grads ? kKernelDispatchGrads : kKernelDispatch, 2,
                       p.rank, t, target, ld_acquire_sys(cnt));
        break;
      }
    }
  }
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    const int old = atomicAdd(p.blocks_done, 1);
    if (old == static_cast<int>(gridDim.x) - 1) {   // last block resets the launch-local counters
      *p.work_counter = 0;
      *p.blocks_done = 0;
    }
  }
}

void launch_dispatch_push(const PushParams& p, int num_blocks, cudaStream_t stream) {
  dispatch_push_kernel<<<num_blocks, kPushThreads, 0, stream>>>(p);
}

// =============================================================================================
// Pull combine
// =============================================================================================
constexpr int kCombineThreads = 512;
constexpr int kPullUnroll = 2;          // 16-byte loads in flight per lane and contributing rank

__global__ void __launch_bounds__(kCombineThreads, 1) combine_pull_kernel(const CombineParams p) {
  __shared__ const char* s_x[kMaxRanks];
  __shared__ const long long* s_done[kMaxRanks];
  __shared__ const float* s_w[kMaxRanks];
  __shared__ int s_ok;
  __shared__ int s_is_last;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int R = p.num_ranks, K = p.num_topk;
  const int kernel_id = kKernelCombine;
  void* own = p.peer_base[p.rank];

  if ((p.flags & 1) && blockIdx.x == 0 && tid < R)
    publish_record(p.own, p.peer_base, p.ctl, p.kind, p.epoch, p.rank, tid);
  if (tid == 0) s_ok = 1;
  __syncthreads();

  if (p.flags & 2) {
    if (tid < R) {
      const unsigned long long* rec =
          fetch_record(own, p.ctl, p.kind, p.epoch, tid, p.wait_budget_ns, p.status, kernel_id, p.rank);
      if (rec == nullptr) s_ok = 0;
      else {
        const char* b = static_cast<const char*>(p.peer_base[tid]);
        s_x[tid] = b + rec[10];
        s_done[tid] = reinterpret_cast<const long long*>(b + rec[11]);
        s_w[tid] = reinterpret_cast<const float*>(b + rec[12]);
      }
    }
    __syncthreads();
    const int warps_per_block = blockDim.x >> 5;
    const int e_local = p.num_experts / R;
    const size_t row_bytes = static_cast<size_t>(p.hidden) * 2;
    const int vec_per_row = p.hidden / 8;
    if (s_ok) {
      for (int t = blockIdx.x * warps_per_block + warp; t < p.num_tokens; t += gridDim.x * warps_per_block) {
        int my_r = -1;
        if (lane < R) my_r = p.send_recv_token[static_cast<size_t>(t) * R + lane];
        // gate: every contributing rank must have stamped its row
        bool ok = true;
        if (my_r >= 0) {
          const long long* g = s_done[lane] + my_r;
          ok = spin_until([&] { return ld_acquire_sys(g) >= p.seq; }, p.wait_budget_ns, p.status);
          if (!ok) report_failure(p.status, kStatusTimeoutTokenGate, kernel_id, 3, p.rank, t,
                                  static_cast<int>(p.seq), static_cast<int>(ld_acquire_sys(g)));
        }
        if (!__all_sync(0xffffffffu, ok)) break;
        // Every contributing rank's row address, warp-uniform; a lane then keeps kPullUnroll x R
        // predicated 16-byte loads in flight so that the NVLink round trip is paid once per batch,
        // not once per load.
        const char* src[kMaxRanks];
#pragma unroll
        for (int d = 0; d < kMaxRanks; ++d) {
          const int r = __shfl_sync(0xffffffffu, my_r, d);
          src[d] = (d < R && r >= 0) ? s_x[d] + static_cast<size_t>(r) * row_bytes : nullptr;
        }
        char* out_row = static_cast<char*>(p.out) + static_cast<size_t>(t) * row_bytes;
        for (int v0 = lane; v0 < vec_per_row; v0 += 32 * kPullUnroll) {
          uint4 q[kPullUnroll][kMaxRanks];
#pragma unroll
          for (int j = 0; j < kPullUnroll; ++j) {
            const int v = v0 + 32 * j;
#pragma unroll
            for (int d = 0; d < kMaxRanks; ++d)
              q[j][d] = (src[d] != nullptr && v < vec_per_row) ? ld_relaxed_sys_v4(src[d] + static_cast<size_t>(v) * 16)
                                                              : make_uint4(0, 0, 0, 0);
          }
#pragma unroll
          for (int j = 0; j < kPullUnroll; ++j) {
            const int v = v0 + 32 * j;
            if (v >= vec_per_row) break;
            float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
            for (int d = 0; d < kMaxRanks; ++d) {
              const float2 a = unpack_bf16x2(q[j][d].x), b = unpack_bf16x2(q[j][d].y), c = unpack_bf16x2(q[j][d].z),
                           e = unpack_bf16x2(q[j][d].w);
              acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
              acc[4] += c.x; acc[5] += c.y; acc[6] += e.x; acc[7] += e.y;
            }
            uint4 o;
            o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
            o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
            st_na_v4(out_row + static_cast<size_t>(v) * 16, o);
          }
        }
        if (!p.is_fwd && lane < K) {
          const long long e = p.topk_idx[static_cast<size_t>(t) * K + lane];
          const int slot = p.pair_slot[static_cast<size_t>(t) * K + lane];
          float g = 0.f;
          if (e >= 0 && slot >= 0) g = s_w[static_cast<int>(e / e_local)][slot];
          p.out_topk_weights[static_cast<size_t>(t) * K + lane] = g;
        }
      }
    }
  }

  if (p.flags & 4) {
    // Tail handshake: peers may release the rows this rank read only after it is done reading.
    __syncthreads();
    if (tid == 0) {
      __threadfence();
      const int old = atomicAdd(p.blocks_done, 1);
      s_is_last = (old == static_cast<int>(gridDim.x) - 1);
    }
    __syncthreads();
    if (s_is_last) {
      if (tid == 0) *p.blocks_done = 0;
      __threadfence_system();
      if (tid < R) {
        flags_signal(p.peer_base, p.ctl, p.kind, p.epoch, p.rank, tid);
        flags_wait(own, p.ctl, p.kind, p.epoch, tid, p.wait_budget_ns, p.status, kernel_id, p.rank,
                   kStatusTimeoutTail);
      }
    }
  }
}

void launch_combine_pull(const CombineParams& p, int num_blocks, cudaStream_t stream) {
  combine_pull_kernel<<<num_blocks, kCombineThreads, 0, stream>>>(p);
}

// =============================================================================================
// Barrier, tile producer, pool <-> recv copies
// =============================================================================================
__global__ void device_barrier_kernel(const BarrierParams p) {
  const int tid = threadIdx.x;
  __threadfence_system();
  if (tid < p.num_ranks) {
    flags_signal(p.peer_base, p.ctl, p.kind, p.epoch, p.rank, tid);
    if (p.wait)
      flags_wait(p.peer_base[p.rank], p.ctl, p.kind, p.epoch, tid, p.wait_budget_ns, p.status,
                 kKernelBarrier, p.rank, kStatusTimeoutBarrier);
  }
}
void launch_device_barrier(const BarrierParams& p, cudaStream_t stream) {
  device_barrier_kernel<<<1, 32, 0, stream>>>(p);
}

__global__ void tile_producer_kernel(int* count, const int* target, int num_tiles, long long delay_ns) {
  for (int t = 0; t < num_tiles; ++t) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < static_cast<unsigned long long>(delay_ns)) __nanosleep(100);
    red_release_gpu_add(count + t, target[t]);
  }
}
void launch_tile_producer(int* count, const int* target, int num_tiles, long long delay_ns, cudaStream_t stream) {
  tile_producer_kernel<<<1, 1, 0, stream>>>(count, target, num_tiles, delay_ns);
}

template <bool kCompress>
__global__ void pool_rows_kernel(const char* src, char* dst, const int* pool_recv_token, int tk_padded, int hidden) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const size_t row_bytes = static_cast<size_t>(hidden) * 2;
  const int vecs = hidden / 8;
  for (int slot = blockIdx.x * warps_per_block + warp; slot < tk_padded; slot += gridDim.x * warps_per_block) {
    const int r = pool_recv_token[slot];
    if (r < 0) {
      if (!kCompress)   // padding rows of a re-expanded pool are zero
        for (int v = lane; v < vecs; v += 32)
          st_na_v4(dst + static_cast<size_t>(slot) * row_bytes + static_cast<size_t>(v) * 16, make_uint4(0, 0, 0, 0));
      continue;
    }
    const char* s = kCompress ? src + static_cast<size_t>(slot) * row_bytes : src + static_cast<size_t>(r) * row_bytes;
    char* d = kCompress ? dst + static_cast<size_t>(r) * row_bytes : dst + static_cast<size_t>(slot) * row_bytes;
    for (int v = lane; v < vecs; v += 32) st_na_v4(d + static_cast<size_t>(v) * 16, ld_nc_v4(s + static_cast<size_t>(v) * 16));
  }
}
void launch_pool_compress(const void* pool, void* recv, const int* pool_recv_token, int tk_padded, int hidden,
                          cudaStream_t stream) {
  if (tk_padded == 0) return;
  const int grid = min((tk_padded + 7) / 8, sm_count() * 8);
  pool_rows_kernel<true><<<grid, 256, 0, stream>>>(static_cast<const char*>(pool), static_cast<char*>(recv),
                                                   pool_recv_token, tk_padded, hidden);
}
void launch_pool_expand(const void* recv, void* pool, const int* pool_recv_token, int tk_padded, int hidden,
                        cudaStream_t stream) {
  if (tk_padded == 0) return;
  const int grid = min((tk_padded + 7) / 8, sm_count() * 8);
  pool_rows_kernel<false><<<grid, 256, 0, stream>>>(static_cast<const char*>(recv), static_cast<char*>(pool),
                                                    pool_recv_token, tk_padded, hidden);
}

// =============================================================================================
// Second half of the fused combine: fp32 reduction of the rows that remote expert ranks stored
// =============================================================================================
__global__ void combine_reduce_kernel(char* out, const char* rows, const long long* topk_idx, int num_tokens,
                                      int hidden, int K, int e_local, int rank, const float* dw_src, float* dw_dst,
                                      const int* skip_rows) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const size_t row_bytes = static_cast<size_t>(hidden) * 2;
  const int vecs = hidden / 8;
  const bool skip = skip_rows != nullptr && *skip_rows != 0;   // the dispatch ran empty: what landed earlier is stale
  for (int t = blockIdx.x * warps_per_block + warp; t < num_tokens; t += gridDim.x * warps_per_block) {
    unsigned remote = 0;
    for (int k = 0; k < K; ++k) {
      const long long e = topk_idx[static_cast<size_t>(t) * K + k];
      if (e >= 0 && static_cast<int>(e / e_local) != rank) remote |= 1u << k;
    }
    if (dw_dst != nullptr && lane < K) {   // per-pair scalars the expert ranks stored for this token; 0 for skipped pairs
      const size_t i = static_cast<size_t>(t) * K + lane;
      dw_dst[i] = (topk_idx[i] >= 0 && !skip) ? dw_src[i] : 0.f;
    }
    if (remote == 0 || rows == nullptr || skip) continue;
    for (int v = lane; v < vecs; v += 32) {
      char* o = out + static_cast<size_t>(t) * row_bytes + static_cast<size_t>(v) * 16;
      const uint4 q0 = *reinterpret_cast<const uint4*>(o);
      float acc[8];
      { const float2 a = unpack_bf16x2(q0.x), b = unpack_bf16x2(q0.y), c = unpack_bf16x2(q0.z), d = unpack_bf16x2(q0.w);
        acc[0] = a.x; acc[1] = a.y; acc[2] = b.x; acc[3] = b.y; acc[4] = c.x; acc[5] = c.y; acc[6] = d.x; acc[7] = d.y; }
      for (int k = 0; k < K; ++k) {
        if (!((remote >> k) & 1u)) continue;
        const uint4 q = ld_nc_v4(rows + (static_cast<size_t>(t) * K + k) * row_bytes + static_cast<size_t>(v) * 16);
        const float2 a = unpack_bf16x2(q.x), b = unpack_bf16x2(q.y), c = unpack_bf16x2(q.z), d = unpack_bf16x2(q.w);
        acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y; acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
      }
      uint4 r;
      r.x = pack_bf16x2(acc[0], acc[1]); r.y = pack_bf16x2(acc[2], acc[3]);
      r.z = pack_bf16x2(acc[4], acc[5]); r.w = pack_bf16x2(acc[6], acc[7]);
      *reinterpret_cast<uint4*>(o) = r;
    }
  }
}
void launch_combine_reduce(void* out, const void* rows, const long long* topk_idx, int num_tokens, int hidden,
                           int num_topk, int num_experts, int num_ranks, int rank, cudaStream_t stream,
                           const float* dw_src, float* dw_dst, const int* skip_rows) {
  if (num_tokens == 0 || (num_ranks == 1 && dw_dst == nullptr)) return;
  const int grid = min((num_tokens + 7) / 8, sm_count() * 8);
  combine_reduce_kernel<<<grid, 256, 0, stream>>>(static_cast<char*>(out), num_ranks == 1 ? nullptr : static_cast<const char*>(rows),
                                                  topk_idx, num_tokens, hidden, num_topk, num_experts / num_ranks, rank,
                                                  dw_src, dw_dst, skip_rows);
}

// =============================================================================================
// Router: logits = x @ w_gate^T, softmax, top-k, renormalise, rank bitmap.  One warp per token.
// The reference has no router; its harnesses build routing with torch ops
// (stream_ep/stream_moe/profile_pipeline.py:102-139).
// =============================================================================================
constexpr int kRouterMaxExpertsPerLane = 16;   // up to 512 experts
constexpr int kRouterKChunk = 64;              // hidden elements per shared-memory step (128 bytes of a row)
constexpr int kRouterLd = kRouterKChunk + 4;   // padded row: float4 reads of 8 consecutive rows hit 32 different banks

// One warp finishes one token from its fp32 logits (shared or global memory): softmax over all experts, top-k by
// repeated arg-max (ties -> lowest expert id), renormalise, rank bitmap.  EPL = experts per lane.
template <int EPL>
__device__ __forceinline__ void route_token(const RouterParams& p, const float* row, int t, int lane) {
  const int E = p.num_experts, K = p.num_topk;
  const int e_local = E / p.num_ranks;
  float logit[EPL];
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < EPL; ++j) {
    const int e = j * 32 + lane;
    logit[j] = (e < E) ? row[e] : -INFINITY;
    mx = fmaxf(mx, logit[j]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < EPL; ++j) {
    const int e = j * 32 + lane;
    logit[j] = (e < E) ? __expf(logit[j] - mx) : 0.f;
    sum += logit[j];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  const float inv = 1.f / sum;
#pragma unroll
  for (int j = 0; j < EPL; ++j) {
    logit[j] *= inv;
    const int e = j * 32 + lane;
    if (p.probs != nullptr && e < E) p.probs[static_cast<size_t>(t) * E + e] = logit[j];
  }
  // top-k by repeated arg-max (ties -> lowest expert id)
  float wsum = 0.f, my_w = 0.f;
  int my_e = -1;
  unsigned rank_mask = 0;
  for (int k = 0; k < K; ++k) {
    float best = -1.f; int best_e = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      const int e = j * 32 + lane;
      if (e < E && logit[j] > best) { best = logit[j]; best_e = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
    }
#pragma unroll
    for (int j = 0; j < EPL; ++j)
      if (j * 32 + lane == best_e) logit[j] = -2.f;
    if (lane == k) { my_w = best; my_e = best_e; }
    wsum += best;
    rank_mask |= 1u << (best_e / e_local);
  }
  if (lane < K) {
    p.topk_idx[static_cast<size_t>(t) * K + lane] = my_e;
    p.topk_weights[static_cast<size_t>(t) * K + lane] = p.renormalize ? my_w / wsum : my_w;
  }
  if (lane < p.num_ranks && p.is_token_in_rank != nullptr)
    p.is_token_in_rank[static_cast<size_t>(t) * p.num_ranks + lane] = (rank_mask >> lane) & 1u;
}

// One CTA routes TOK tokens with TOK * 4 threads.  Logits: a register-tiled fp32 GEMM, (TOK / 4) x 16 threads
// with 4 tokens x JE experts each, so one pass covers 16 * JE experts (16 / 32 / 64; wider expert counts loop).
// Operands are fetched 128 contiguous bytes per row (8 lanes per row), converted to fp32 and kept row-major in
// shared memory; the global loads of the next two chunks are in flight while the current one is multiplied.
// Few experts make the kernel latency-bound, so those instances use 32 tokens per CTA (twice the CTAs); 64
// experts per pass are FMA-bound and use 64 tokens for operand reuse.  Then each warp finishes 8 tokens:
// softmax over all experts, top-k by repeated arg-max, renormalise, rank bitmap.
template <int JE, int TOK>
__global__ void __launch_bounds__(TOK * 4) router_kernel(const RouterParams p) {
  constexpr int THREADS = TOK * 4;
  constexpr int NE = 16 * JE;                                      // experts per pass
  constexpr int EPL = JE == 4 ? kRouterMaxExpertsPerLane : 1;      // experts per lane in the softmax / top-k part
  constexpr int XV = TOK * 8 / THREADS;                            // 16-byte loads of x per thread and chunk (2)
  constexpr int WV = (NE * 8 + THREADS - 1) / THREADS;             // ... of the gate weights (1 or 2)
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* xs = reinterpret_cast<float*>(smem_raw);                 // [TOK tokens][kRouterLd]
  float* ws = xs + TOK * kRouterLd;                               // [NE experts][kRouterLd]
  float* logits = ws + NE * kRouterLd;                            // [TOK tokens][e_pad]
  const int E = p.num_experts, H = p.hidden;
  const int e_pad = (E + NE - 1) / NE * NE + 1;                   // +1: rows start in different banks
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int ty = tid >> 4, tx = tid & 15;
  const __nv_bfloat16* xg = static_cast<const __nv_bfloat16*>(p.x);
  const __nv_bfloat16* wg = static_cast<const __nv_bfloat16*>(p.w_gate);
  const int t0 = blockIdx.x * TOK;

  for (int e0 = 0; e0 < E; e0 += NE) {
    float acc[4][JE];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < JE; ++j) acc[i][j] = 0.f;
    uint4 xv0[XV], wv0[WV], xv1[XV], wv1[WV];
    auto fetch = [&](int k0, uint4 (&xv)[XV], uint4 (&wv)[WV]) {
#pragma unroll
      for (int i = 0; i < XV; ++i) {
        const int idx = tid + THREADS * i, row = idx >> 3, kk = k0 + (idx & 7) * 8;
        xv[i] = (t0 + row < p.num_tokens && kk < H) ? ld_nc_v4(xg + static_cast<size_t>(t0 + row) * H + kk)
                                                    : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int i = 0; i < WV; ++i) {
        const int idx = tid + THREADS * i, row = idx >> 3, kk = k0 + (idx & 7) * 8;
        wv[i] = (row < NE && e0 + row < E && kk < H)
                    ? __ldg(reinterpret_cast<const uint4*>(wg + static_cast<size_t>(e0 + row) * H + kk))
                    : make_uint4(0, 0, 0, 0);
      }
    };
    auto stash1 = [&](float* dst, const uint4& v, int idx) {
      const float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), c = unpack_bf16x2(v.z), d = unpack_bf16x2(v.w);
      float4* o = reinterpret_cast<float4*>(dst + (idx >> 3) * kRouterLd + (idx & 7) * 8);
      o[0] = make_float4(a.x, a.y, b.x, b.y);
      o[1] = make_float4(c.x, c.y, d.x, d.y);
    };
    // one chunk: registers -> shared memory, refill the registers two chunks ahead, multiply
    auto chunk = [&](int k_next, uint4 (&xv)[XV], uint4 (&wv)[WV]) {
      __syncthreads();   // the previous chunk's tiles are no longer read
#pragma unroll
      for (int i = 0; i < XV; ++i) stash1(xs, xv[i], tid + THREADS * i);
#pragma unroll
      for (int i = 0; i < WV; ++i)
        if (tid + THREADS * i < NE * 8) stash1(ws, wv[i], tid + THREADS * i);
      __syncthreads();
      if (k_next < H) fetch(k_next, xv, wv);                       // in flight during this and the next multiply
#pragma unroll 4
      for (int k = 0; k < kRouterKChunk; k += 4) {
        float4 a[4], b[JE];
#pragma unroll
        for (int i = 0; i < 4; ++i) a[i] = *reinterpret_cast<const float4*>(xs + (ty * 4 + i) * kRouterLd + k);
#pragma unroll
        for (int j = 0; j < JE; ++j) b[j] = *reinterpret_cast<const float4*>(ws + (j * 16 + tx) * kRouterLd + k);   // lanes on consecutive rows: no bank conflict
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < JE; ++j) {
            acc[i][j] = fmaf(a[i].x, b[j].x, acc[i][j]);
            acc[i][j] = fmaf(a[i].y, b[j].y, acc[i][j]);
            acc[i][j] = fmaf(a[i].z, b[j].z, acc[i][j]);
            acc[i][j] = fmaf(a[i].w, b[j].w, acc[i][j]);
          }
      }
    };
    fetch(0, xv0, wv0);
    if (kRouterKChunk < H) fetch(kRouterKChunk, xv1, wv1);
    for (int k0 = 0; k0 < H; k0 += 2 * kRouterKChunk) {
      chunk(k0 + 2 * kRouterKChunk, xv0, wv0);
      if (k0 + kRouterKChunk >= H) break;
      chunk(k0 + 3 * kRouterKChunk, xv1, wv1);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < JE; ++j) logits[(ty * 4 + i) * e_pad + e0 + j * 16 + tx] = acc[i][j];
  }
  __syncthreads();

  for (int tt = warp; tt < TOK; tt += THREADS / 32) {
    const int t = t0 + tt;
    if (t >= p.num_tokens) break;
    route_token<EPL>(p, logits + tt * e_pad, t, lane);
  }
}

// Second half of the tensor-core router: one warp per token reads the fp32 logits the grouped GEMM stored.
template <int EPL>
__global__ void __launch_bounds__(256) router_finish_kernel(const RouterParams p, const float* __restrict__ logits, int ld) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (t >= p.num_tokens) return;
  route_token<EPL>(p, logits + static_cast<size_t>(t) * ld, t, lane);
}

void launch_router_finish(const RouterParams& p, const float* logits, int ld_logits, cudaStream_t stream) {
  const int grid = (p.num_tokens + 7) / 8;
  if (p.num_experts <= 32) router_finish_kernel<1><<<grid, 256, 0, stream>>>(p, logits, ld_logits);
  else if (p.num_experts <= 128) router_finish_kernel<4><<<grid, 256, 0, stream>>>(p, logits, ld_logits);
  else router_finish_kernel<kRouterMaxExpertsPerLane><<<grid, 256, 0, stream>>>(p, logits, ld_logits);
}

template <int JE, int TOK>
static void launch_router_je(const RouterParams& p, cudaStream_t stream) {
  constexpr int NE = 16 * JE;
  const int e_pad = (p.num_experts + NE - 1) / NE * NE + 1;
  const size_t smem = sizeof(float) * (static_cast<size_t>(TOK + NE) * kRouterLd + static_cast<size_t>(TOK) * e_pad);
  const int grid = (p.num_tokens + TOK - 1) / TOK;
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(router_kernel<JE, TOK>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  router_kernel<JE, TOK><<<grid, TOK * 4, smem, stream>>>(p);
}

void launch_router(const RouterParams& p, cudaStream_t stream) {
  if (p.num_experts <= 16) launch_router_je<1, 32>(p, stream);
  else if (p.num_experts <= 32) launch_router_je<2, 32>(p, stream);
  else launch_router_je<4, 64>(p, stream);
}

}  // namespace sep
