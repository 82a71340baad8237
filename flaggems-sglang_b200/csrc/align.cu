// Routing / alignment kernels: stable counting sort of the (token, expert) slots by
// expert with warp-match ranking and shared-memory counters.  Integer work only;
// every output is deterministic (no atomics decide an order).
#include "align.cuh"

namespace b200moe {

namespace {

constexpr int kAlignThreads = 1024;
constexpr int kAhead = 8;   // iterations of 32 slots whose ids are fetched together

__device__ __forceinline__ int load_id(const void* ids, int is64, int i) {
  return is64 ? static_cast<int>(reinterpret_cast<const long long*>(ids)[i])
              : reinterpret_cast<const int*>(ids)[i];
}

// Exclusive scan of one int per thread over the whole CTA (blockDim.x <= 1024).
// Returns the exclusive prefix; *total receives the sum.  scratch: 33 ints.
__device__ __forceinline__ int block_exclusive_scan(int v, int* scratch, int* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int inc = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    int t = __shfl_up_sync(0xffffffffu, inc, d);
    if (lane >= d) inc += t;
  }
  if (lane == 31) scratch[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    int w = (lane < (blockDim.x >> 5)) ? scratch[lane] : 0;
    int winc = w;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      int t = __shfl_up_sync(0xffffffffu, winc, d);
      if (lane >= d) winc += t;
    }
    scratch[lane] = winc - w;
    if (lane == 31) scratch[32] = winc;
  }
  __syncthreads();
  int res = inc - v + scratch[warp];
  *total = scratch[32];
  __syncthreads();
  return res;
}

// Largest e in [0, n) with offs[e] <= x, for a non-decreasing offs[0..n].
__device__ __forceinline__ int upper_expert(const int* offs, int n, int x) {
  int lo = 0, hi = n;
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (offs[mid] <= x) lo = mid; else hi = mid;
  }
  return lo;
}

// Core: stable grouping of P slots by expert.  `ids` are expert ids (already
// mapped to local experts when map != nullptr); slots with an id outside
// [0, E) are dropped.  Each expert's group starts at a multiple of `block`.
//   s_cnt   [nwarps][E] shared counters
//   s_base  [E+1] shared: padded start row of each expert
//   s_hist  [E]   shared: slots per expert
// The caller provides place(slot, pos, pre[slot]) to record a placement.
// `pre` (optional, [P]): a per-slot value fetched alongside the ids and handed to place().
template <typename Place>
__device__ __forceinline__ void group_by_expert(const void* ids, int is64, const int* map, int map_len, int P, int E,
                                                int block, int* s_cnt, int* s_base, int* s_hist,
                                                int* s_scan, int nwarps, const float* pre, Place place) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < nwarps * E; i += blockDim.x) s_cnt[i] = 0;
  __syncthreads();

  // contiguous, 32-aligned segment of slots per counting warp
  int seg = (P + nwarps - 1) / nwarps;
  seg = (seg + 31) & ~31;
  const int begin = warp * seg;
  const int end = min(P, begin + seg);

  // Both passes fetch the ids of kAhead iterations before they rank them: one dependent global
  // load per 32 slots would otherwise set the pace of the whole kernel.
  auto fetch = [&](int i) -> int {
    int e = -1;
    if (i < end) {
      e = load_id(ids, is64, i);
      if (map != nullptr && e >= 0) e = (e < map_len) ? map[e] : -1;
      if (e < 0 || e >= E) e = -1;
    }
    return e;
  };
  if (warp < nwarps) {
    for (int i0 = begin; i0 < end; i0 += 32 * kAhead) {
      int ev[kAhead];
#pragma unroll
      for (int u = 0; u < kAhead; ++u) ev[u] = fetch(i0 + 32 * u + lane);
#pragma unroll
      for (int u = 0; u < kAhead; ++u) {
        if (i0 + 32 * u >= end) break;
        const int e = ev[u];
        unsigned m = __match_any_sync(0xffffffffu, e);
        if (e >= 0 && (m & ((1u << lane) - 1)) == 0) s_cnt[warp * E + e] += __popc(m);
        __syncwarp();
      }
    }
  }
  __syncthreads();

  // per expert: totals and exclusive prefix over the counting warps
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int run = 0;
    for (int w = 0; w < nwarps; ++w) {
      int t = s_cnt[w * E + e];
      s_cnt[w * E + e] = run;
      run += t;
    }
    s_hist[e] = run;
  }
  __syncthreads();

  // padded starts: exclusive scan over experts (chunks of blockDim.x experts)
  int carry = 0;
  for (int e0 = 0; e0 < E; e0 += blockDim.x) {
    int e = e0 + threadIdx.x;
    int padded = 0;
    if (e < E) padded = (s_hist[e] + block - 1) / block * block;
    int total;
    int ex = block_exclusive_scan(padded, s_scan, &total);
    if (e < E) s_base[e] = carry + ex;
    carry += total;
  }
  if (threadIdx.x == 0) s_base[E] = carry;
  __syncthreads();

  if (warp < nwarps) {
    for (int i0 = begin; i0 < end; i0 += 32 * kAhead) {
      int ev[kAhead];
      float wv[kAhead];
#pragma unroll
      for (int u = 0; u < kAhead; ++u) {
        const int i = i0 + 32 * u + lane;
        ev[u] = fetch(i);
        wv[u] = (pre != nullptr && i < end) ? pre[i] : 0.f;
      }
#pragma unroll
      for (int u = 0; u < kAhead; ++u) {
        if (i0 + 32 * u >= end) break;
        const int i = i0 + 32 * u + lane;
        const int e = ev[u];
        unsigned m = __match_any_sync(0xffffffffu, e);
        int rank = __popc(m & ((1u << lane) - 1));
        int cur = 0;
        if (e >= 0) cur = s_cnt[warp * E + e];
        __syncwarp();
        if (e >= 0) {
          place(i, s_base[e] + cur + rank, wv[u]);
          if (rank == 0) s_cnt[warp * E + e] = cur + __popc(m);
        }
        __syncwarp();
      }
    }
  }
  __syncthreads();
}

__global__ void __launch_bounds__(kAlignThreads)
align_block_kernel(const void* ids, int is64, const int* map, int map_len, const float* weights, int P, int E,
                   int block, int cap, int nwarps, int* sorted_ids, int* expert_ids, int* num_post_pad,
                   float* row_gamma, int* blk_off, int* meta, const FlagWait fw) {
  extern __shared__ int smem[];
  griddep_wait();             // the tables written below may still be read by the kernels of the previous call
  griddep_launch_dependents();
  wait_for_peers(fw);
  int* s_cnt = smem;                    // nwarps * E
  int* s_base = s_cnt + nwarps * E;     // E + 1
  int* s_hist = s_base + (E + 1);       // E
  int* s_scan = s_hist + E;             // 33

  const int nblk_cap = (cap + block - 1) / block;
  for (int i = threadIdx.x; i < cap; i += blockDim.x) {
    sorted_ids[i] = P;
    if (row_gamma != nullptr) row_gamma[i] = 0.f;
  }
  for (int i = threadIdx.x; i < nblk_cap; i += blockDim.x) expert_ids[i] = -1;
  __syncthreads();

  group_by_expert(ids, is64, map, map_len, P, E, block, s_cnt, s_base, s_hist, s_scan, nwarps,
                  row_gamma != nullptr ? weights : nullptr, [&](int slot, int pos, float w) {
                    sorted_ids[pos] = slot;
                    if (row_gamma != nullptr) row_gamma[pos] = w;
                  });

  const int rows = s_base[E];
  const int nblk = rows / block;
  for (int b = threadIdx.x; b < nblk; b += blockDim.x) {
    int e = upper_expert(s_base, E + 1, b * block);
    expert_ids[b] = e;
  }
  if (blk_off != nullptr)
    for (int e = threadIdx.x; e <= E; e += blockDim.x) blk_off[e] = s_base[e] / block;
  if (threadIdx.x == 0) {
    num_post_pad[0] = rows;
    if (meta != nullptr) {
      meta[0] = nblk;
      meta[1] = rows;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// The same grouping spread over kAlignCtas CTAs in two launches, for tens of thousands of slots
// (one CTA pushes every store through one SM's memory pipe: 77 us at 32 k slots).  CTA c owns the
// contiguous slots [c * per, (c + 1) * per); stability follows from ordering by (CTA, warp, lane).
//   count  per-CTA slots per expert -> cnt[c][e]; all CTAs share the filling of the defaults
//   place  each CTA derives the padded expert starts and its own first rows from cnt (CTA 0 also
//          writes the block tables), recounts its chunk (cheaper than keeping the per-warp counts)
//          and writes
constexpr int kAlignCtas = 32;

// warp-private counts of the chunk [begin, end): s_cnt[w][e]
__device__ __forceinline__ void count_chunk(const void* ids, int is64, const int* map, int map_len, int begin, int end, int E,
                                            int* s_cnt, int nwarps, int* seg_begin, int* seg_end) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < nwarps * E; i += blockDim.x) s_cnt[i] = 0;
  __syncthreads();
  int seg = (max(end - begin, 0) + nwarps - 1) / nwarps;
  seg = (seg + 31) & ~31;
  const int b = begin + warp * seg;
  const int e_ = min(end, b + seg);
  *seg_begin = b;
  *seg_end = e_;
  if (warp < nwarps) {
    for (int i0 = b; i0 < e_; i0 += 32) {
      const int i = i0 + lane;
      int e = -1;
      if (i < e_) {
        e = load_id(ids, is64, i);
        if (map != nullptr && e >= 0) e = (e < map_len) ? map[e] : -1;
        if (e < 0 || e >= E) e = -1;
      }
      unsigned m = __match_any_sync(0xffffffffu, e);
      if (e >= 0 && (m & ((1u << lane) - 1)) == 0) s_cnt[warp * E + e] += __popc(m);
      __syncwarp();
    }
  }
  __syncthreads();
}

__global__ void __launch_bounds__(kAlignThreads)
align_count_kernel(const void* ids, int is64, const int* map, int map_len, int P, int E, int block, int cap, int per, int nwarps,
                   int* sorted_ids, int* expert_ids, float* row_gamma, int* cnt, const FlagWait fw) {
  extern __shared__ int smem[];
  int* s_cnt = smem;
  griddep_wait();
  griddep_launch_dependents();
  wait_for_peers(fw);
  const int nblk_cap = (cap + block - 1) / block;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < cap; i += gridDim.x * blockDim.x) {
    sorted_ids[i] = P;
    if (row_gamma != nullptr) row_gamma[i] = 0.f;
  }
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < nblk_cap; i += gridDim.x * blockDim.x) expert_ids[i] = -1;
  const int begin = min(P, static_cast<int>(blockIdx.x) * per), end = min(P, begin + per);
  int sb, se;
  count_chunk(ids, is64, map, map_len, begin, end, E, s_cnt, nwarps, &sb, &se);
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int run = 0;
    for (int w = 0; w < nwarps; ++w) run += s_cnt[w * E + e];
    cnt[blockIdx.x * E + e] = run;
  }
}

__global__ void __launch_bounds__(kAlignThreads)
align_place_kernel(const void* ids, int is64, const int* map, int map_len, const float* weights, int P, int E,
                   int block, int per, int nwarps, const int* cnt, int* sorted_ids, float* row_gamma, int* expert_ids,
                   int* num_post_pad, int* blk_off, int* meta) {
  extern __shared__ int smem[];
  int* s_cnt = smem;                      // nwarps * E
  int* s_base = s_cnt + nwarps * E;       // E + 1 padded expert starts
  int* s_mine = s_base + (E + 1);         // E: first row of this CTA's slots of each expert
  int* s_scan = s_mine + E;               // 33
  griddep_wait();
  griddep_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nctas = gridDim.x;
  // Every CTA derives the padded expert starts from the per-CTA counts by itself (a few thousand
  // integers out of L2), which saves a single-CTA launch between counting and placing.
  int carry = 0;
  for (int e0 = 0; e0 < E; e0 += blockDim.x) {
    const int e = e0 + threadIdx.x;
    int total_e = 0, before = 0;
    if (e < E) {
      for (int c = 0; c < nctas; ++c) {
        const int t = cnt[c * E + e];
        if (c < static_cast<int>(blockIdx.x)) before += t;
        total_e += t;
      }
    }
    const int padded = (total_e + block - 1) / block * block;
    int total;
    const int ex = block_exclusive_scan(padded, s_scan, &total);
    if (e < E) {
      s_base[e] = carry + ex;
      s_mine[e] = carry + ex + before;
    }
    carry += total;
  }
  if (threadIdx.x == 0) s_base[E] = carry;
  __syncthreads();
  if (blockIdx.x == 0) {
    // the block tables, once
    const int rows = s_base[E];
    const int nblk = rows / block;
    for (int b = threadIdx.x; b < nblk; b += blockDim.x) expert_ids[b] = upper_expert(s_base, E + 1, b * block);
    if (blk_off != nullptr)
      for (int e = threadIdx.x; e <= E; e += blockDim.x) blk_off[e] = s_base[e] / block;
    if (threadIdx.x == 0) {
      num_post_pad[0] = rows;
      if (meta != nullptr) {
        meta[0] = nblk;
        meta[1] = rows;
      }
    }
  }
  const int begin = min(P, static_cast<int>(blockIdx.x) * per), end = min(P, begin + per);
  int sb, se;
  count_chunk(ids, is64, map, map_len, begin, end, E, s_cnt, nwarps, &sb, &se);
  // start of (warp, expert) = this CTA's first row of the expert + the counts of the warps before it
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int run = s_mine[e];
    for (int w = 0; w < nwarps; ++w) {
      const int t = s_cnt[w * E + e];
      s_cnt[w * E + e] = run;
      run += t;
    }
  }
  __syncthreads();
  if (warp < nwarps) {
    for (int i0 = sb; i0 < se; i0 += 32) {
      const int i = i0 + lane;
      int e = -1;
      float w = 0.f;
      if (i < se) {
        e = load_id(ids, is64, i);
        if (map != nullptr && e >= 0) e = (e < map_len) ? map[e] : -1;
        if (e < 0 || e >= E) e = -1;
        if (row_gamma != nullptr) w = weights[i];
      }
      unsigned m = __match_any_sync(0xffffffffu, e);
      const int rank = __popc(m & ((1u << lane) - 1));
      int cur = 0;
      if (e >= 0) cur = s_cnt[warp * E + e];
      __syncwarp();
      if (e >= 0) {
        const int pos = cur + rank;
        sorted_ids[pos] = i;
        if (row_gamma != nullptr) row_gamma[pos] = w;
        if (rank == 0) s_cnt[warp * E + e] = cur + __popc(m);
      }
      __syncwarp();
    }
  }
}

// Internal tables from the reference's routing triple: hist[E], topk_indx[P]
// (sorted row -> slot), gate_scal[P] (sorted row order).
__global__ void __launch_bounds__(kAlignThreads)
align_from_routing_kernel(const int* hist, const int* topk_indx, const float* gate_scal, int P, int E,
                          int block, int cap, int* sorted_ids, float* row_gamma, int* blk_off,
                          int* meta) {
  extern __shared__ int smem[];
  int* s_base = smem;             // E + 1 padded starts
  int* s_raw = s_base + (E + 1);  // E + 1 raw starts
  int* s_scan = s_raw + (E + 1);  // 33

  for (int i = threadIdx.x; i < cap; i += blockDim.x) {
    sorted_ids[i] = P;
    row_gamma[i] = 0.f;
  }
  int carry_p = 0, carry_r = 0;
  for (int e0 = 0; e0 < E; e0 += blockDim.x) {
    int e = e0 + threadIdx.x;
    int h = (e < E) ? hist[e] : 0;
    int total;
    int ex = block_exclusive_scan((h + block - 1) / block * block, s_scan, &total);
    if (e < E) s_base[e] = carry_p + ex;
    carry_p += total;
    ex = block_exclusive_scan(h, s_scan, &total);
    if (e < E) s_raw[e] = carry_r + ex;
    carry_r += total;
  }
  if (threadIdx.x == 0) {
    s_base[E] = carry_p;
    s_raw[E] = carry_r;
  }
  __syncthreads();
  const int n_rows = min(P, s_raw[E]);
  for (int q = threadIdx.x; q < n_rows; q += blockDim.x) {
    int e = upper_expert(s_raw, E + 1, q);
    int pos = s_base[e] + (q - s_raw[e]);
    sorted_ids[pos] = topk_indx[q];
    row_gamma[pos] = gate_scal[q];
  }
  for (int e = threadIdx.x; e <= E; e += blockDim.x) blk_off[e] = s_base[e] / block;
  if (threadIdx.x == 0) {
    meta[0] = s_base[E] / block;
    meta[1] = s_base[E];
  }
}

// top-k -> the reference's routing tables.
__global__ void __launch_bounds__(kAlignThreads)
routing_from_topk_kernel(const float* weights, const void* ids, int is64, int M, int k, int E,
                         int max_tiles, int nwarps, int* expt_indx, int* topk_indx, int* gate_indx,
                         float* gate_scal, int* hist, int* token_offs_raw, int* token_offs_pad,
                         int* block_pid_map) {
  extern __shared__ int smem[];
  int* s_cnt = smem;
  int* s_base = s_cnt + nwarps * E;
  int* s_hist = s_base + (E + 1);
  int* s_scan = s_hist + E;
  const int P = M * k;

  // ascending (stable) insertion sort of each token's experts
  for (int t = threadIdx.x; t < M; t += blockDim.x) {
    for (int j = 0; j < k; ++j) {
      int e = load_id(ids, is64, t * k + j);
      int p = j;
      while (p > 0 && expt_indx[t * k + p - 1] > e) {
        expt_indx[t * k + p] = expt_indx[t * k + p - 1];
        --p;
      }
      expt_indx[t * k + p] = e;
    }
  }
  for (int i = threadIdx.x; i < 4 * max_tiles; i += blockDim.x) block_pid_map[i] = -1;
  __syncthreads();

  group_by_expert(expt_indx, 0, nullptr, 0, P, E, 1, s_cnt, s_base, s_hist, s_scan, nwarps, nullptr,
                  [&](int slot, int pos, float) {
                    topk_indx[pos] = slot;
                    gate_indx[slot] = pos;
                    // the weight that the per-token sort moved to rank (slot % k):
                    // the original column whose stable rank equals that position
                    const int t = slot / k, want = slot - t * k;
                    float w = 0.f;
                    for (int j = 0; j < k; ++j) {
                      int ej = load_id(ids, is64, t * k + j);
                      int rank = 0;
                      for (int i = 0; i < k; ++i) {
                        int ei = load_id(ids, is64, t * k + i);
                        rank += (ei < ej) || (ei == ej && i < j);
                      }
                      if (rank == want) w = weights[t * k + j];
                    }
                    gate_scal[pos] = w;
                  });
  for (int e = threadIdx.x; e < E; e += blockDim.x) hist[e] = s_hist[e];
  for (int e = threadIdx.x; e <= E; e += blockDim.x) token_offs_raw[e] = s_base[e];
  __syncthreads();

  // padded block tables for block sizes 16, 32, 64, 128
  for (int v = 0; v < 4; ++v) {
    const int bm = 16 << v;
    int carry = 0;
    for (int e0 = 0; e0 < E; e0 += blockDim.x) {
      int e = e0 + threadIdx.x;
      int tiles = (e < E) ? (s_hist[e] + bm - 1) / bm : 0;
      int total;
      int ex = block_exclusive_scan(tiles, s_scan, &total);
      if (e < E) {
        int off = carry + ex;
        token_offs_pad[v * (E + 1) + e] = off;
        for (int b = 0; b < tiles; ++b)
          if (off + b < max_tiles) block_pid_map[v * max_tiles + off + b] = (b << 16) + e;
      }
      carry += total;
    }
    if (threadIdx.x == 0) token_offs_pad[v * (E + 1) + E] = carry;
    __syncthreads();
  }
}

int pick_warps(int E) {
  int nw = 32;
  while (nw > 1 && static_cast<size_t>(nw) * E * 4 > 40 * 1024) nw >>= 1;
  return nw;
}

}  // namespace

int align_capacity(int n_slots, int n_experts, int block) {
  long long cap = static_cast<long long>(n_slots) + static_cast<long long>(n_experts) * (block - 1);
  if (n_slots < n_experts) {
    long long alt = static_cast<long long>(n_slots) * block;
    if (alt < cap) cap = alt;
  }
  if (cap > 0x7fffffffLL) return -1;
  return static_cast<int>(cap);
}

int routing_max_tiles(int n_slots, int n_experts) {
  if (n_slots <= n_experts) return n_slots;
  // floor division of a negative numerator, as the dependency's Python does
  int num = n_experts - n_slots - 1;  // negative
  int fl = -((-num + 15) / 16);
  return n_experts - 1 - fl;
}

int launch_align_block(const void* ids, int is64, const int* map, int map_len, const float* weights, int P, int E,
                       int block, int cap, int* sorted_ids, int* expert_ids, int* num_post_pad,
                       float* row_gamma, int* blk_off, int* meta, cudaStream_t stream, bool pdl, const FlagWait* wait) {
  if (P < 0 || E <= 0 || block <= 0 || cap < 0) return B200MOE_ERR_BAD_ARG;
  int nw = pick_warps(E);
  size_t smem = (static_cast<size_t>(nw) * E + (E + 1) + E + 40) * sizeof(int);
  if (smem > 48 * 1024) return B200MOE_ERR_TOO_LARGE;
  note_launch("align_block_kernel");
  FlagWait fw = {};
  if (wait != nullptr) fw = *wait;
  cudaError_t err = launch_kernel(align_block_kernel, dim3(1), dim3(kAlignThreads), smem, stream, pdl, ids, is64, map,
                                  map_len, weights, P, E, block, cap, nw, sorted_ids, expert_ids, num_post_pad,
                                  row_gamma, blk_off, meta, fw);
  return err == cudaSuccess ? B200MOE_OK : B200MOE_ERR_CUDA;
}

size_t align_multi_tmp_bytes(int E) { return static_cast<size_t>(kAlignCtas) * E * sizeof(int); }

int launch_align_block_multi(const void* ids, int is64, const int* map, int map_len, const float* weights, int P, int E,
                             int block, int cap, int* sorted_ids, int* expert_ids, int* num_post_pad,
                             float* row_gamma, int* blk_off, int* meta, int* tmp, cudaStream_t stream, bool pdl,
                             const FlagWait* wait) {
  if (P < 0 || E <= 0 || block <= 0 || cap < 0 || tmp == nullptr) return B200MOE_ERR_BAD_ARG;
  const int nw = pick_warps(E);
  const size_t smem = (static_cast<size_t>(nw) * E + 40) * sizeof(int);
  const size_t smem_place = (static_cast<size_t>(nw) * E + 2 * static_cast<size_t>(E) + 1 + 40) * sizeof(int);
  if (smem_place > 48 * 1024) return B200MOE_ERR_TOO_LARGE;
  int per = (P + kAlignCtas - 1) / kAlignCtas;
  per = (per + 31) & ~31;
  int* cnt = tmp;
  FlagWait fw = {};
  if (wait != nullptr) fw = *wait;
  note_launch("align_count_kernel");
  cudaError_t err = launch_kernel(align_count_kernel, dim3(kAlignCtas), dim3(kAlignThreads), smem, stream, pdl, ids,
                                  is64, map, map_len, P, E, block, cap, per, nw, sorted_ids, expert_ids, row_gamma, cnt,
                                  fw);
  if (err != cudaSuccess) return B200MOE_ERR_CUDA;
  note_launch("align_place_kernel");
  err = launch_kernel(align_place_kernel, dim3(kAlignCtas), dim3(kAlignThreads), smem_place, stream, pdl, ids, is64, map,
                      map_len, weights, P, E, block, per, nw, static_cast<const int*>(cnt), sorted_ids, row_gamma,
                      expert_ids, num_post_pad, blk_off, meta);
  return err == cudaSuccess ? B200MOE_OK : B200MOE_ERR_CUDA;
}

int launch_align_from_routing(const int* hist, const int* topk_indx, const float* gate_scal, int P,
                              int E, int block, int cap, int* sorted_ids, float* row_gamma,
                              int* blk_off, int* meta, cudaStream_t stream) {
  if (P < 0 || E <= 0 || block <= 0) return B200MOE_ERR_BAD_ARG;
  size_t smem = (2 * static_cast<size_t>(E + 1) + 40) * sizeof(int);
  if (smem > 48 * 1024) return B200MOE_ERR_TOO_LARGE;
  note_launch("align_from_routing_kernel");
  align_from_routing_kernel<<<1, kAlignThreads, smem, stream>>>(hist, topk_indx, gate_scal, P, E, block,
                                                                cap, sorted_ids, row_gamma, blk_off,
                                                                meta);
  return cudaGetLastError() == cudaSuccess ? B200MOE_OK : B200MOE_ERR_CUDA;
}

int launch_routing_from_topk(const float* weights, const void* ids, int is64, int M, int k, int E,
                             int* expt_indx, int* topk_indx, int* gate_indx, float* gate_scal,
                             int* hist, int* token_offs_raw, int* token_offs_pad, int* block_pid_map,
                             cudaStream_t stream) {
  if (M < 0 || k <= 0 || E <= 0) return B200MOE_ERR_BAD_ARG;
  int nw = pick_warps(E);
  size_t smem = (static_cast<size_t>(nw) * E + (E + 1) + E + 40) * sizeof(int);
  if (smem > 48 * 1024) return B200MOE_ERR_TOO_LARGE;
  int mt = routing_max_tiles(M * k, E);
  note_launch("routing_from_topk_kernel");
  routing_from_topk_kernel<<<1, kAlignThreads, smem, stream>>>(
      weights, ids, is64, M, k, E, mt, nw, expt_indx, topk_indx, gate_indx, gate_scal, hist,
      token_offs_raw, token_offs_pad, block_pid_map);
  return cudaGetLastError() == cudaSuccess ? B200MOE_OK : B200MOE_ERR_CUDA;
}

}  // namespace b200moe
