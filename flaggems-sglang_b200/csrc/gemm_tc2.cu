// 16-bit grouped expert GEMMs on CTA pairs (tcgen05.mma.cta_group::2), prefill sizes.
//
// Two CTAs of a cluster share one tile of 256 tokens x 256 weight rows: each CTA stages ITS 128
// token rows and HALF of the weight rows (128), the leader CTA issues one MMA for the pair and the
// tensor cores of both SMs read the weight halves from both shared memories.  Per CTA and 64-k
// stage that is 16 KiB of tokens + 16 KiB of weights instead of 16 + 32 with one CTA per tile:
// a third less shared-memory fill, L2 traffic and operand reading for the same flops.
//
//   mode 0 (gate/up):  CTA 0 stages 128 gate rows, CTA 1 the 128 matching up rows; accumulator
//                      columns 0..127 = gate, 128..255 = up, as in the single-CTA kernel.
//   mode 1 (down):     CTA r stages weight rows n0 + 128 r ..; 256 output columns per tile.
// The two token blocks of a tile are consecutive blocks of one expert; an expert with an odd number
// of blocks leaves the second half of its last tile without a block (its rows are computed on
// whatever the loads return and never stored).
//
// No load here has the cluster-multicast qualifier: every CTA loads its own operands with plain
// tiled TMA loads.  Only tcgen05.commit is multicast (to the same barrier in both CTAs).
// Synchronisation between the two CTAs:
//   * operands staged: the loads of BOTH CTAs complete on the leader's `full` barrier (the
//     cta_group::2 form of the tiled load lets the completion go to the peer CTA's barrier); each
//     producer announces its bytes there with an arrive.expect_tx of its own (remote for the second
//     CTA).  A first version that completed locally and forwarded each completion with a remote
//     arrive ran at half speed: the extra hop made the refill loop longer than the seven stages
//     of buffered work;
//   * stage free / accumulator ready: tcgen05.commit of the leader, multicast to both CTAs;
//   * accumulator drained: the epilogue warps of both CTAs arrive on the leader's `tempty`.
// Every wait is bounded (common.cuh); the cluster barriers at start and end are reached by every
// thread whatever happened in between.
//
// Status: results are bit-identical to the one-CTA-per-tile kernel, but on the Mixtral-shaped
// layer at M = 4096 this kernel takes 1.9x as long (tensor pipe 35 % active where the other shows
// 87 %), whatever the stage count (4..7), the instruction's N, the epilogue or the commit pattern;
// the cause has not been found.  It is therefore used only on request (B200MOE_FLAG_CTA_PAIR).
#include "gemm_sched.cuh"

namespace b200moe {

namespace {

constexpr int kStageBytes2 = 2 * kTileBytes;   // per CTA: 128 token rows + 128 weight rows, 64 k each

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of the same shared-memory location in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t mapa_u32(uint32_t saddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx_remote(uint32_t cluster_addr, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.release.cluster.shared::cluster.b64 _, [%0], %1;" ::"r"(cluster_addr), "r"(bytes)
               : "memory");
}
// Tiled loads into this CTA's shared memory whose completion is counted on a barrier that may live
// in the peer CTA (cluster address).  No multicast: one destination.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* m, uint32_t bar_cluster, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], "
      "[%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* m, uint32_t bar_cluster, int c0, int c1,
                                                 int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, "
      "%5}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// Arrive on the barrier at this shared-memory offset in BOTH CTAs once the pair's MMAs issued so far are done.
__device__ __forceinline__ void tc_commit2(uint32_t bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
               "h"(mask)
               : "memory");
}
__device__ __forceinline__ void tc_mma2_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void red_add_v4_2(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.v4.f32.add [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}
template <typename T>
__device__ __forceinline__ uint32_t pack2_2(float lo, float hi);
template <>
__device__ __forceinline__ uint32_t pack2_2<__nv_bfloat16>(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <>
__device__ __forceinline__ uint32_t pack2_2<__half>(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

struct PairTile {
  int e;        // expert
  int n0;       // first weight row of the tile inside the expert (mode 0: of the gate rows)
  int blk;      // this CTA's token block (index over all padded blocks)
  bool has;     // the block belongs to the expert (false: second half of an odd expert's last tile)
};

// Tile `id` in expert-major, then n-tile, then block-pair order.  s_pair_off[e] = pairs before expert e.
__device__ __forceinline__ PairTile decode_pair(int id, const int* s_pair_off, const int* s_blk_off, int E, int num_nt,
                                                int tile_n, int rank) {
  int lo = 0, hi = E;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (s_pair_off[mid] * num_nt <= id) lo = mid; else hi = mid;
  }
  PairTile t;
  t.e = lo;
  const int np = s_pair_off[lo + 1] - s_pair_off[lo];
  const int local = id - s_pair_off[lo] * num_nt;
  const int bp = local % np;
  const int nt = local / np;
  const int nb = s_blk_off[lo + 1] - s_blk_off[lo];
  t.n0 = nt * tile_n;
  t.blk = s_blk_off[lo] + 2 * bp + rank;
  t.has = 2 * bp + rank < nb;
  return t;
}

template <int MODE, typename T>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
moe_gemm_tc2_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                    const GemmArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const int stages = a.stages;
  uint8_t* ctrl_base = smem + static_cast<size_t>(stages) * kStageBytes2;
  uint64_t* bar_full = reinterpret_cast<uint64_t*>(ctrl_base);   // leader: both CTAs' operands are staged
  uint64_t* bar_empty = bar_full + stages;
  uint64_t* bar_tfull = bar_empty + stages;
  uint64_t* bar_tempty = bar_tfull + 2;          // leader: both CTAs' epilogues have drained the accumulator
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* s_blk_off = reinterpret_cast<int*>(tmem_slot + 4);   // [E+1]
  int* s_pair_off = s_blk_off + (a.E + 1);                   // [E+1]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 2);     // one arrive.expect_tx per CTA of the pair
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&bar_tfull[s]), 1);
      mbar_init(smem_u32(&bar_tempty[s]), 8);
    }
    *abort_flag = 0;
    fence_mbar_init();
    fence_proxy_async_smem();
    prefetch_tmap(&tm_w);
    prefetch_tmap(&tm_x);
  }
  // barriers of both CTAs exist before either side signals the other
  cluster_arrive();
  cluster_wait();
  if (warp == 1) {
    tmem_alloc2(smem_u32(tmem_slot), 512u);
    tmem_relinquish2();
  }
  griddep_wait();
  griddep_launch_dependents();
  for (int e = threadIdx.x; e <= a.E; e += blockDim.x) s_blk_off[e] = a.blk_off[e];
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < a.E; ++e) {
      s_pair_off[e] = run;
      run += (s_blk_off[e + 1] - s_blk_off[e] + 1) >> 1;
    }
    s_pair_off[a.E] = run;
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  constexpr int kTileN = (MODE == 1) ? 256 : 128;
  const int num_nt = a.num_nt;
  const int total = s_pair_off[a.E] * num_nt;
  const int nclusters = static_cast<int>(gridDim.x) >> 1;
  const int cluster_id = static_cast<int>(blockIdx.x) >> 1;
  // spread the tiles evenly: with w waves, ceil(total / w) clusters do w tiles each
  const int waves = (total + nclusters - 1) / nclusters;
  const int cl_eff = waves > 0 ? (total + waves - 1) / waves : 1;
  const bool active = cluster_id < cl_eff;

  if (active && warp == 0 && lane == 0) {
    // =============================== TMA producer (every CTA, its own operands) ===================
    int stage = 0;
    uint32_t phase = 0;
    long long issued = 0;
    bool ok = true;
    for (int tile = cluster_id; ok && tile < total; tile += cl_eff) {
      const PairTile t = decode_pair(tile, s_pair_off, s_blk_off, a.E, num_nt, kTileN, static_cast<int>(rank));
      const int wrow = (MODE == 0) ? (rank == 0 ? t.n0 : a.up_row_off + t.n0) : t.n0 + static_cast<int>(rank) * kTileRows;
      for (int kb = 0; kb < a.kblocks; ++kb) {
        if (!mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1, abort_flag, DEV_TIMEOUT_PRODUCER)) {
          ok = false;
          break;
        }
        const uint32_t full = mapa_u32(smem_u32(&bar_full[stage]), 0);   // the leader's barrier
        const uint32_t sx = smem_u32(smem + static_cast<size_t>(stage) * kStageBytes2);
        const int k0 = kb * (kStageKBytes / static_cast<int>(sizeof(T)));
        mbar_arrive_expect_tx_remote(full, static_cast<uint32_t>(kStageBytes2));
        tma_load_2d_pair(sx, &tm_x, full, k0, t.blk * kTileRows);
        tma_load_3d_pair(sx + kTileBytes, &tm_w, full, k0, wrow, t.e);
        ++issued;
        if (++stage == stages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
    if (!ok) {
      // let the copies still in flight land before the CTA goes away: the leader sees them on its
      // barriers; the second CTA, whose completions are counted elsewhere, simply waits a while
      if (leader) {
        const int n = static_cast<int>(issued < stages ? issued : stages);
        for (int i = 1; i <= n; ++i) {
          int s2 = stage - i;
          uint32_t ph = phase;
          if (s2 < 0) {
            s2 += stages;
            ph ^= 1;
          }
          mbar_wait_brief(smem_u32(&bar_full[s2]), ph);
        }
      } else {
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 20000ull) {
        }
      }
    }
  } else if (active && warp == 1 && lane == 0 && leader) {
    // =============================== MMA issuer (leader CTA, for the pair) ========================
    const uint32_t fmt = (a.dtype == B200MOE_DTYPE_BF16) ? 1u : 0u;
    const uint32_t idesc = make_idesc(fmt, 256u, 256u);
    constexpr int kSteps = kStageKBytes / 32;
    int stage = 0, acc = 0;
    uint32_t phase = 0, acc_phase = 0;
    bool ok = true;
    for (int tile = cluster_id; ok && tile < total; tile += cl_eff) {
      if (!mbar_wait(smem_u32(&bar_tempty[acc]), acc_phase ^ 1, abort_flag, DEV_TIMEOUT_MMA)) break;
      tc_fence_after();
      const uint32_t d0 = tmem_base + static_cast<uint32_t>(acc * 256);
      for (int kb = 0; kb < a.kblocks; ++kb) {
        if (!mbar_wait(smem_u32(&bar_full[stage]), phase, abort_flag, DEV_TIMEOUT_MMA)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t sx = smem_u32(smem + static_cast<size_t>(stage) * kStageBytes2);
        const uint64_t dx = smem_desc_k_sw128(sx);                 // token rows: the M side
        const uint64_t dw = smem_desc_k_sw128(sx + kTileBytes);    // this CTA's half of the weight rows: the N side
#pragma unroll
        for (int k = 0; k < kSteps; ++k) tc_mma2_f16(d0, dx + 2 * k, dw + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
        tc_commit2(smem_u32(&bar_empty[stage]));
        if (++stage == stages) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (!ok) break;
      tc_commit2(smem_u32(&bar_tfull[acc]));
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  } else if (active && warp >= 2) {
    // =============================== epilogue (every CTA, its own 128 token rows) =================
    const int quad = warp & 3;
    const int lrow = quad * 32 + lane;
    const bool w_on_input = (a.flags & B200MOE_FLAG_WEIGHT_ON_INPUT) != 0;
    const bool mimic = (a.flags & B200MOE_FLAG_MIMIC_ROUNDING) != 0;
    const ActParams ap = act_params(a);
    const uint32_t tempty_leader0 = mapa_u32(smem_u32(&bar_tempty[0]), 0);
    const uint32_t tempty_leader1 = mapa_u32(smem_u32(&bar_tempty[1]), 0);
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int tile = cluster_id; tile < total; tile += cl_eff) {
      const PairTile t = decode_pair(tile, s_pair_off, s_blk_off, a.E, num_nt, kTileN, static_cast<int>(rank));
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + static_cast<uint32_t>(acc * 256);
      const int r = t.blk * kTileRows + lrow;
      int slot = -1;
      float gam = 0.f;
      if (t.has) {
        slot = a.sorted_ids[r];
        if (slot >= 0 && slot < a.P) gam = a.row_gamma[r]; else slot = -1;
      }
      const bool valid = slot >= 0;
      if (!mbar_wait(smem_u32(&bar_tfull[acc]), acc_phase, abort_flag, DEV_TIMEOUT_EPILOGUE)) break;
      tc_fence_after();
      if (MODE == 0) {
        T* orow = reinterpret_cast<T*>(a.out) + static_cast<size_t>(t.has ? r : 0) * a.ld_out + t.n0;
#pragma unroll 1
        for (int c0 = 0; c0 < 128; c0 += 16) {
          float g[16], u[16];
          tmem_ld16x2_wait(taddr + c0, taddr + 128 + c0, g, u);
          uint32_t pk[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float lo = act_mul<T>(g[2 * j], u[2 * j], w_on_input, gam, mimic, ap);
            const float hi = act_mul<T>(g[2 * j + 1], u[2 * j + 1], w_on_input, gam, mimic, ap);
            pk[j] = pack2_2<T>(lo, hi);
          }
          if (t.has && t.n0 + c0 + 8 <= a.N) *reinterpret_cast<uint4*>(orow + c0) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
          if (t.has && t.n0 + c0 + 16 <= a.N)
            *reinterpret_cast<uint4*>(orow + c0 + 8) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
        }
      } else if (a.out_pairs != nullptr) {
        T* prow = reinterpret_cast<T*>(a.out_pairs) + static_cast<size_t>(valid ? slot : 0) * a.N + t.n0;
        const float scale = w_on_input ? 1.0f : gam;
#pragma unroll 1
        for (int c0 = 0; c0 < 256; c0 += 16) {
          float v[16];
          tmem_ld16_wait(taddr + c0, v);
          if (valid) {
            uint32_t pk[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) pk[j] = pack2_2<T>(v[2 * j] * scale, v[2 * j + 1] * scale);
            if (t.n0 + c0 + 8 <= a.N) *reinterpret_cast<uint4*>(prow + c0) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            if (t.n0 + c0 + 16 <= a.N) *reinterpret_cast<uint4*>(prow + c0 + 8) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
          }
        }
        if (valid && t.n0 == 0) a.pair_valid[slot] = 1;
      } else {
        float* orow = reinterpret_cast<float*>(a.out) + static_cast<size_t>(valid ? slot / a.topk : 0) * a.ld_out + t.n0;
        const float scale = w_on_input ? 1.0f : gam;
        const bool round_pair = mimic;
#pragma unroll 1
        for (int c0 = 0; c0 < 256; c0 += 16) {
          float v[16];
          tmem_ld16_wait(taddr + c0, v);
          if (valid) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              v[j] *= scale;
              if (round_pair) v[j] = to_f32<T>(from_f32<T>(v[j]));
            }
#pragma unroll
            for (int q = 0; q < 4; ++q)
              if (t.n0 + c0 + 4 * q + 4 <= a.N)
                red_add_v4_2(orow + c0 + 4 * q, v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(acc == 0 ? tempty_leader0 : tempty_leader1);
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  }

  // ---- teardown (every thread of both CTAs, aborted or not): neither CTA may leave while the other
  // can still signal its barriers or read its shared memory
  tc_fence_before();
  __syncthreads();
  cluster_arrive();
  cluster_wait();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc2(tmem_base, 512u);
  }
  if (threadIdx.x == 0 && *abort_flag != 0) atomicCAS(a.status, 0, *abort_flag);
}

size_t tc2_ctrl_bytes(const GemmArgs& a) { return 1024 + 2 * static_cast<size_t>(a.E + 1) * 4 + 64; }

int g_tc2_pairs_seen = 0;   // resident CTA pairs found for the last launch (diagnostics)

// How many CTA pairs of this kernel the device keeps resident at once.  The kernel is persistent with
// a static tile assignment, so a grid with even one pair more than that would run its last pairs as a
// second wave and take twice as long.
template <int MODE, typename T>
int max_resident_pairs(size_t smem, int num_sms) {
  static int cached = 0;
  static size_t cached_smem = 0;
  if (cached > 0 && cached_smem == smem) return cached;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(num_sms & ~1);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, moe_gemm_tc2_kernel<MODE, T>, &cfg) != cudaSuccess || n <= 0) {
    cudaGetLastError();
    n = (num_sms / 2) - 2;     // conservative guess
  }
  if (n > num_sms / 2) n = num_sms / 2;
  cached = n;
  cached_smem = smem;
  return n;
}

template <int MODE, typename T>
int launch_tc2(const CUtensorMap& tm_w, const CUtensorMap& tm_x, const GemmArgs& a, int num_sms, cudaStream_t stream) {
  const size_t smem = 1024 + static_cast<size_t>(a.stages) * kStageBytes2 + tc2_ctrl_bytes(a);
  if (smem > kSmemLimit) return B200MOE_ERR_TOO_LARGE;
  if (cudaFuncSetAttribute(moe_gemm_tc2_kernel<MODE, T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(smem)) != cudaSuccess)
    return B200MOE_ERR_CUDA;
  const int pairs = max_resident_pairs<MODE, T>(smem, num_sms);
  g_tc2_pairs_seen = pairs;
  note_launch(MODE == 0 ? "moe_gemm_tc2_kernel<gate/up>" : "moe_gemm_tc2_kernel<down>");
  cudaError_t err = launch_kernel(moe_gemm_tc2_kernel<MODE, T>, dim3(2 * pairs), dim3(kThreads), smem, stream,
                                  a.pdl != 0, tm_w, tm_x, a);
  return err == cudaSuccess ? B200MOE_OK : B200MOE_ERR_CUDA;
}

}  // namespace

int gemm_tc2_resident_pairs() { return g_tc2_pairs_seen; }

// Can this GEMM run on CTA pairs?  16-bit weights, 128-token blocks on the M side, plain epilogue,
// whole reduction in one piece.
bool gemm_tc2_ok(const GemmArgs& a) {
  return a.wmode == B200MOE_W_16BIT && a.orient == 1 && a.BT == 128 && a.bias == nullptr &&
         a.activation != B200MOE_ACT_SWIGLU_OAI && (a.mode == 0 || (a.flags & B200MOE_FLAG_NO_SPLIT_K) != 0) &&
         a.n_peers <= 1;
}

void gemm_plan_tc2(GemmArgs* a) {
  const int tile_n = (a->mode == 1) ? 256 : kTileRows;
  a->num_nt = (a->N + tile_n - 1) / tile_n;
  a->kblocks = (a->K + 63) / 64;
  a->acc_stages = 2;
  a->tmem_cols = 512;
  int st = static_cast<int>((kSmemLimit - 1024 - tc2_ctrl_bytes(*a)) / kStageBytes2);
  if (st > 8) st = 8;
  if (st < 2) st = 2;
  a->stages = st;
}

int launch_gemm_tc2(const CUtensorMap& tm_w, const CUtensorMap& tm_x, const GemmArgs& a, int num_sms,
                    cudaStream_t stream) {
  if (!gemm_tc2_ok(a)) return B200MOE_ERR_UNSUPPORTED;
  if (a.dtype == B200MOE_DTYPE_BF16)
    return a.mode == 0 ? launch_tc2<0, __nv_bfloat16>(tm_w, tm_x, a, num_sms, stream)
                       : launch_tc2<1, __nv_bfloat16>(tm_w, tm_x, a, num_sms, stream);
  return a.mode == 0 ? launch_tc2<0, __half>(tm_w, tm_x, a, num_sms, stream)
                     : launch_tc2<1, __half>(tm_w, tm_x, a, num_sms, stream);
}

}  // namespace b200moe
