// Grouped expert GEMMs on the sm_100a tensor cores (tcgen05.mma, accumulators in
// tensor memory, operands staged by TMA into a shared-memory ring).
//
// One persistent CTA per SM, six warps:
//   warp 0      one thread issues the TMA loads (weight tile(s) + token block per stage)
//   warp 1      one thread issues the MMAs and the commits; the warp owns the TMEM allocation
//   warps 2-5   epilogue: tcgen05.ld the accumulator, apply the fused tail, store
//
// mode 0 (gate/up): per stage a 128-row gate tile and the matching 128-row up tile; two
//   accumulators, so that lane i of TMEM holds gate[n0+i] and up[n0+i] for every token of
//   the block and the activation needs no data exchange.
// mode 1 (down):    one 128-row tile; the reduction may be split over CTAs; the epilogue
//   multiplies by the routing weight and adds into the fp32 combine buffer with
//   red.global.add.f32 (which also merges the top-k experts of a token), or, with many pairs on
//   128-token blocks, stores one 16-bit row per pair for the output conversion to sum.
//
// Every wait is bounded; on a time-out the CTA raises an abort flag, all roles leave their
// loops, the status word is set, TMEM is freed and the kernel returns.
#include "gemm_sched.cuh"

namespace b200moe {

namespace {

// Geometry of one pipeline stage and one accumulator for (MODE, ORIENT).
//   ORIENT 0 ("weights on M"): decode-sized token blocks (BT = 16..256 tokens on the N side).
//   ORIENT 1 ("tokens on M"):  BT = 128 tokens on the M side, 256 weight rows on the N side;
//                              every epilogue thread owns one token row and stores contiguous
//                              output columns with 16-byte accesses.
template <int MODE, int ORIENT>
struct Geo {
  static constexpr int kWBytes = (ORIENT == 1) ? 2 * kTileBytes : (MODE == 0 ? 2 : 1) * kTileBytes;
  static constexpr int kTileN = (ORIENT == 1 && MODE == 1) ? 256 : 128;  // output columns per tile
};

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.v4.f32.add [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}

template <typename T>
__device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Dequantise 32 packed uint4 weights (16 bytes: four words of eight consecutive k, element
// 2i in nibble i and element 2i+1 in nibble 4+i) into 32 fp16 values = four 16-byte chunks.
// (w >> 4i) & 0x000F000F | 0x64006400 reads as the fp16 pair (1024 + q_2i, 1024 + q_2i+1);
// subtracting (1024 + zero) is exact, the product with the scale rounds once.
__device__ __forceinline__ void dequant_w4x32(const uint4 packed, const __half2 scale, const __half2 zero1024,
                                              uint4 (&out)[4]) {
  const uint32_t w[4] = {packed.x, packed.y, packed.z, packed.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint32_t r[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t t = ((w[j] >> (4 * i)) & 0x000F000Fu) | 0x64006400u;
      __half2 h = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&t), zero1024), scale);
      r[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    out[j] = make_uint4(r[0], r[1], r[2], r[3]);
  }
}

constexpr int kDequantWarps = 8;
constexpr int kThreadsW4 = kThreads + 32 * kDequantWarps;

// W4: the weight operand is int4 (AWQ, group 128, pre-packed): TMA stages the packed rows,
// eight extra warps dequantise them into the swizzled fp16 operand tile the MMA reads.
// EXT: per-expert bias and the clamped swiglu in the epilogues (separate instantiations, so
// that the plain kernels keep their shorter epilogue loops).
template <int MODE, typename T, int ORIENT, bool W4, bool EXT>
__global__ void __launch_bounds__(W4 ? kThreadsW4 : kThreads, 1)
moe_gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                   const GemmArgs a) {

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  using G = Geo<MODE, ORIENT>;
  constexpr int W_BYTES = G::kWBytes;
  const int BT = a.BT;
  const int x_bytes = BT * kStageKBytes;
  constexpr int PK_BYTES = W4 ? W_BYTES / 4 : 0;  // packed int4 rows: 32 bytes per row and stage
  constexpr int SZ_BYTES = W4 ? 1024 : 0;         // scale / zero word of every packed row for the stage's group
  const int stage_bytes = W_BYTES + x_bytes + PK_BYTES + SZ_BYTES;
  const int stages = a.stages;

  uint8_t* ctrl_base = smem + static_cast<size_t>(stages) * stage_bytes;
  uint64_t* bar_full = reinterpret_cast<uint64_t*>(ctrl_base);
  uint64_t* bar_empty = bar_full + stages;
  uint64_t* bar_dq = bar_empty + stages;  // W4: operand tile dequantised
  uint64_t* bar_tfull = bar_dq + stages;
  uint64_t* bar_tempty = bar_tfull + 2;
  uint64_t* bar_meet = bar_tempty + 2;    // meeting point of the four epilogue warps
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_meet + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* s_col_row = reinterpret_cast<int*>(tmem_slot + 4);               // [2][kMaxBT]
  float* s_col_gam = reinterpret_cast<float*>(s_col_row + 2 * kMaxBT);  // [2][kMaxBT]
  int* s_blk_off = reinterpret_cast<int*>(s_col_gam + 2 * kMaxBT);      // [E+1]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
      mbar_init(smem_u32(&bar_dq[s]), kDequantWarps);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&bar_tfull[s]), 1);
      mbar_init(smem_u32(&bar_tempty[s]), 4);
    }
    mbar_init(smem_u32(bar_meet), 4);
    *abort_flag = 0;
    fence_mbar_init();
    fence_proxy_async_smem();
    prefetch_tmap(&tm_w);
    prefetch_tmap(&tm_x);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), static_cast<uint32_t>(a.tmem_cols));
    tmem_relinquish();
  }
  // everything above touched only shared / tensor memory and kernel parameters; the routing
  // tables and activations below come from the preceding kernels
  griddep_wait();
  griddep_launch_dependents();
  for (int e = threadIdx.x; e <= a.E; e += blockDim.x) s_blk_off[e] = a.blk_off[e];
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const Ctrl c = make_ctrl(a, MODE == 1);
  const int cols_per_acc = (ORIENT == 1) ? 256 : (MODE == 0 ? 2 : 1) * BT;
  const bool active = static_cast<int>(blockIdx.x) < c.grid_eff;

  if (active && warp == 0 && lane == 0) {
    // =============================== TMA producer ===============================
    int stage = 0;
    uint32_t phase = 0;
    long long issued = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < c.total; tile += c.grid_eff) {
      const TileCoord t = decode_tile(tile, c, s_blk_off, a.E, BT, a.num_nt, a.kblocks, G::kTileN);
      for (int kb = t.kb0; kb < t.kb1; ++kb) {
        if (!mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1, abort_flag, DEV_TIMEOUT_PRODUCER)) {
          ok = false;
          break;
        }
        const uint32_t full = smem_u32(&bar_full[stage]);
        const uint32_t sw = smem_u32(smem + static_cast<size_t>(stage) * stage_bytes);
        const int k0 = kb * (kStageKBytes / static_cast<int>(sizeof(T)));
        if (W4) {
          // packed rows: 64 k = 32 bytes per row, 128 rows per box, no swizzle; beside them the
          // scale / zero words of the rows for this stage's group (whole 128-row blocks: weight
          // rows per expert are a multiple of 128), so that the conversion never waits on a
          // global load
          const int second0 = (MODE == 0) ? a.up_row_off + t.n0 : t.n0 + kTileRows;
          const bool has_second = (MODE == 0 || ORIENT == 1);
          const bool first_in = t.n0 < a.w_rows, second_in = has_second && second0 < a.w_rows;
          mbar_arrive_expect_tx(full, static_cast<uint32_t>(PK_BYTES + x_bytes) + (first_in ? 512u : 0u) +
                                          (second_in ? 512u : 0u));
          const uint32_t spk = sw + W_BYTES + x_bytes;
          tma_load_3d(spk, &tm_w, full, kb * 32, t.n0, t.e);
          if (has_second) tma_load_3d(spk + kTileRows * 32, &tm_w, full, kb * 32, second0, t.e);
          const uint32_t* szg = reinterpret_cast<const uint32_t*>(a.w_sz) +
                                (static_cast<size_t>(t.e) * ((a.K + 127) / 128) + (kb >> 1)) * a.w_rows;
          if (first_in) bulk_copy_g2s(spk + PK_BYTES, szg + t.n0, 512, full);
          if (second_in) bulk_copy_g2s(spk + PK_BYTES + 512, szg + second0, 512, full);
        } else {
          mbar_arrive_expect_tx(full, static_cast<uint32_t>(stage_bytes));
          tma_load_3d(sw, &tm_w, full, k0, t.n0, t.e);
          if (MODE == 0) tma_load_3d(sw + kTileBytes, &tm_w, full, k0, a.up_row_off + t.n0, t.e);
        }
        tma_load_2d(sw + W_BYTES, &tm_x, full, k0, t.row0);
        ++issued;
        if (++stage == stages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
    if (!ok) {
      // let the copies still in flight land before the CTA goes away
      const int n = static_cast<int>(issued < stages ? issued : stages);
      for (int i = 1; i <= n; ++i) {
        int s = stage - i;
        uint32_t ph = phase;
        if (s < 0) {
          s += stages;
          ph ^= 1;
        }
        mbar_wait_brief(smem_u32(&bar_full[s]), ph);
      }
    }
  } else if (active && warp == 1 && lane == 0) {
    // =============================== MMA issuer =================================
    const uint32_t fmt = (a.dtype == B200MOE_DTYPE_BF16) ? 1u : 0u;
    const uint32_t idesc = make_idesc(fmt, kTileRows, ORIENT == 1 ? 256u : static_cast<uint32_t>(BT));
    constexpr int kSteps = kStageKBytes / 32;  // MMAs per stage and accumulator
    int stage = 0, acc = 0;
    uint32_t phase = 0, acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < c.total; tile += c.grid_eff) {
      const TileCoord t = decode_tile(tile, c, s_blk_off, a.E, BT, a.num_nt, a.kblocks, G::kTileN);
      if (!mbar_wait(smem_u32(&bar_tempty[acc]), acc_phase ^ 1, abort_flag, DEV_TIMEOUT_MMA)) break;
      tc_fence_after();
      const uint32_t d0 = tmem_base + static_cast<uint32_t>(acc * cols_per_acc);
      for (int kb = t.kb0; kb < t.kb1; ++kb) {
        if (!mbar_wait(smem_u32(W4 ? &bar_dq[stage] : &bar_full[stage]), phase, abort_flag, DEV_TIMEOUT_MMA)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t sw = smem_u32(smem + static_cast<size_t>(stage) * stage_bytes);
        const uint64_t dw = smem_desc_k_sw128(sw);
        const uint64_t dx = smem_desc_k_sw128(sw + W_BYTES);
#pragma unroll
        for (int k = 0; k < kSteps; ++k) {
          const uint32_t accum = (kb > t.kb0 || k > 0) ? 1u : 0u;
          // advancing 32 bytes inside the 128-byte swizzle atom = +2 in 16-byte units
          if (ORIENT == 1) {
            tc_mma_f16(d0, dx + 2 * k, dw + 2 * k, idesc, accum);
          } else {
            tc_mma_f16(d0, dw + 2 * k, dx + 2 * k, idesc, accum);
            if (MODE == 0) {
              const uint64_t du = smem_desc_k_sw128(sw + kTileBytes);
              tc_mma_f16(d0 + static_cast<uint32_t>(BT), du + 2 * k, dx + 2 * k, idesc, accum);
            }
          }
        }
        tc_commit(smem_u32(&bar_empty[stage]));
        if (++stage == stages) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (!ok) break;
      tc_commit(smem_u32(&bar_tfull[acc]));
      if (++acc == a.acc_stages) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  } else if (W4 && active && warp >= 6) {
    // =============================== int4 -> fp16 operand tile ==================
    constexpr int ROWS = (MODE == 0 || ORIENT == 1 ? 2 : 1) * kTileRows;  // packed rows per stage
    constexpr int UNITS_PER_THREAD = ROWS * 2 / (32 * kDequantWarps);  // 16-byte units per thread (2 or 1)
    const int dt = threadIdx.x - 6 * 32;                          // 0..255
    const int row = (UNITS_PER_THREAD == 2) ? dt : (dt >> 1);     // packed row this thread converts
    const int half0 = (UNITS_PER_THREAD == 2) ? 0 : (dt & 1);
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < c.total; tile += c.grid_eff) {
      const TileCoord t = decode_tile(tile, c, s_blk_off, a.E, BT, a.num_nt, a.kblocks, G::kTileN);
      // output row of this packed row inside the expert (gate rows first, then the up rows)
      const int n = (row < kTileRows || MODE == 1) ? t.n0 + row : a.up_row_off + t.n0 + (row - kTileRows);
      const bool n_ok = n < a.w_rows;
      for (int kb = t.kb0; kb < t.kb1; ++kb) {
        if (!mbar_wait(smem_u32(&bar_full[stage]), phase, abort_flag, DEV_TIMEOUT_MMA)) {
          ok = false;
          break;
        }
        // scale (low half) and 1024 + zero (high half), staged beside the packed rows
        const uint32_t szv = n_ok ? *reinterpret_cast<const uint32_t*>(smem + static_cast<size_t>(stage) * stage_bytes +
                                                                         W_BYTES + x_bytes + PK_BYTES + row * 4)
                                  : 0u;
        const __half2 sc = __half2half2(__ushort_as_half(static_cast<unsigned short>(szv & 0xFFFFu)));
        const __half2 zp = __half2half2(__ushort_as_half(static_cast<unsigned short>(szv >> 16)));
        uint8_t* sbase = smem + static_cast<size_t>(stage) * stage_bytes;
        const uint4* pk = reinterpret_cast<const uint4*>(sbase + W_BYTES + x_bytes + row * 32);
        uint8_t* orow = sbase + (row >> 7) * kTileBytes + (row & 127) * kStageKBytes;
#pragma unroll
        for (int u = 0; u < UNITS_PER_THREAD; ++u) {
          const int half = half0 + u;
          uint4 o[4];
          dequant_w4x32(pk[half], sc, zp, o);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int chunk = (half * 4 + j) ^ (row & 7);   // 128-byte swizzle of the operand tile
            *reinterpret_cast<uint4*>(orow + chunk * 16) = o[j];
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_dq[stage]));
        if (++stage == stages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (active && warp >= 2 && warp < 6) {
    // =============================== epilogue ===================================
    const int quad = warp & 3;                  // TMEM lane quadrant this warp may read
    const int ep_tid = (warp - 2) * 32 + lane;  // 0..127
    const int lrow = quad * 32 + lane;          // accumulator row (TMEM lane)
    const bool w_on_input = (a.flags & B200MOE_FLAG_WEIGHT_ON_INPUT) != 0;
    const bool mimic = (a.flags & B200MOE_FLAG_MIMIC_ROUNDING) != 0;
    const bool round_pair = mimic && c.split == 1;
    const ActParams ap = act_params(a);
    const bool has_bias = EXT && a.bias != nullptr;
    int acc = 0, iter = 0;
    uint32_t acc_phase = 0, meet_phase = 0;
    for (int tile = blockIdx.x; tile < c.total; tile += c.grid_eff, ++iter) {
      const TileCoord t = decode_tile(tile, c, s_blk_off, a.E, BT, a.num_nt, a.kblocks, G::kTileN);
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) +
                             static_cast<uint32_t>(acc * cols_per_acc);
      if (ORIENT == 1) {
        // ---- accumulator row = token: contiguous output columns per thread
        // blocks smaller than 128 tokens load only their rows; the MMA still spans 128 rows and
        // the accumulator rows beyond the block hold garbage that is never stored
        const bool in_block = lrow < BT;
        const int r = t.row0 + (in_block ? lrow : 0);
        const int slot = a.sorted_ids[r];
        const bool valid = in_block && slot >= 0 && slot < a.P;
        const float gam = valid ? a.row_gamma[r] : 0.f;
        if (!mbar_wait(smem_u32(&bar_tfull[acc]), acc_phase, abort_flag, DEV_TIMEOUT_EPILOGUE)) break;
        tc_fence_after();
        if (MODE == 0) {
          T* orow = reinterpret_cast<T*>(a.out) + static_cast<size_t>(r) * a.ld_out + t.n0;
#pragma unroll 1
          for (int c0 = 0; c0 < 128; c0 += 16) {
            float g[16], u[16];
            tmem_ld16x2_wait(taddr + c0, taddr + 128 + c0, g, u);
            if (has_bias) {
              // gate rows first, then the up / linear rows of the same expert
              const float* bg = a.bias + static_cast<size_t>(t.e) * 2 * a.N + t.n0 + c0;
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const bool in = t.n0 + c0 + j < a.N;
                g[j] += in ? __ldg(bg + j) : 0.f;
                u[j] += in ? __ldg(bg + a.N + j) : 0.f;
              }
            }
            uint32_t pk[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float lo = act_mul<T, EXT>(g[2 * j], u[2 * j], w_on_input, gam, mimic, ap);
              const float hi = act_mul<T, EXT>(g[2 * j + 1], u[2 * j + 1], w_on_input, gam, mimic, ap);
              pk[j] = pack2<T>(lo, hi);
            }
            if (in_block && t.n0 + c0 + 8 <= a.N)
              *reinterpret_cast<uint4*>(orow + c0) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            if (in_block && t.n0 + c0 + 16 <= a.N)
              *reinterpret_cast<uint4*>(orow + c0 + 8) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
          }
        } else if (a.out_pairs != nullptr) {
          // one 16-bit row per (token, choice) pair, routing weight applied; the output conversion
          // sums a token's rows in a fixed order (no atomics: a rerun gives the same bits)
          T* prow = reinterpret_cast<T*>(a.out_pairs) + static_cast<size_t>(valid ? slot : 0) * a.N + t.n0;
          const float scale = w_on_input ? 1.0f : gam;
#pragma unroll 1
          for (int c0 = 0; c0 < 256; c0 += 16) {
            float v[16];
            tmem_ld16_wait(taddr + c0, v);
            if (valid) {
              if (has_bias) {
                const float* bo = a.bias + static_cast<size_t>(t.e) * a.N + t.n0 + c0;
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] += (t.n0 + c0 + j < a.N) ? __ldg(bo + j) : 0.f;
              }
              uint32_t pk[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) pk[j] = pack2<T>(v[2 * j] * scale, v[2 * j + 1] * scale);
              if (t.n0 + c0 + 8 <= a.N) *reinterpret_cast<uint4*>(prow + c0) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
              if (t.n0 + c0 + 16 <= a.N)
                *reinterpret_cast<uint4*>(prow + c0 + 8) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
            }
          }
          if (valid && t.n0 == 0) a.pair_valid[slot] = 1;
        } else {
          const int orow_idx = valid ? slot / a.topk : 0;
          float* orow = reinterpret_cast<float*>(a.out) + static_cast<size_t>(orow_idx) * a.ld_out + t.n0;
          const float scale = w_on_input ? 1.0f : gam;
#pragma unroll 1
          for (int c0 = 0; c0 < 256; c0 += 16) {
            float v[16];
            tmem_ld16_wait(taddr + c0, v);
            if (valid) {
              if (has_bias && t.kb0 == 0) {   // the first reduction split carries the bias
                const float* bo = a.bias + static_cast<size_t>(t.e) * a.N + t.n0 + c0;
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] += (t.n0 + c0 + j < a.N) ? __ldg(bo + j) : 0.f;
              }
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                v[j] *= scale;
                if (round_pair) v[j] = to_f32<T>(from_f32<T>(v[j]));
              }
#pragma unroll
              for (int q = 0; q < 4; ++q)
                if (t.n0 + c0 + 4 * q + 4 <= a.N)
                  red_add_v4(orow + c0 + 4 * q, v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
            }
          }
        }
      } else {
        // ---- accumulator row = weight row: one output column (token) at a time
        const int buf = iter & 1;
        int* col_row = s_col_row + buf * kMaxBT;
        float* col_gam = s_col_gam + buf * kMaxBT;
        for (int cidx = ep_tid; cidx < BT; cidx += 128) {
          const int slot = a.sorted_ids[t.row0 + cidx];
          const bool valid = slot >= 0 && slot < a.P;
          col_row[cidx] = valid ? (MODE == 1 ? slot / a.topk : slot) : -1;
          col_gam[cidx] = valid ? a.row_gamma[t.row0 + cidx] : 0.f;
        }
        if (!warps_meet(smem_u32(bar_meet), meet_phase, lane, abort_flag, DEV_TIMEOUT_EPILOGUE)) break;
        if (!mbar_wait(smem_u32(&bar_tfull[acc]), acc_phase, abort_flag, DEV_TIMEOUT_EPILOGUE)) break;
        tc_fence_after();
        const int n = t.n0 + lrow;
        const bool n_ok = n < a.N;
        if (MODE == 0) {
          T* out = reinterpret_cast<T*>(a.out) + static_cast<size_t>(t.row0) * a.ld_out + n;
          float bgate = 0.f, bup = 0.f;
          if (has_bias && n_ok) {
            bgate = __ldg(a.bias + static_cast<size_t>(t.e) * 2 * a.N + n);
            bup = __ldg(a.bias + static_cast<size_t>(t.e) * 2 * a.N + a.N + n);
          }
#pragma unroll 1
          for (int c0 = 0; c0 < BT; c0 += 16) {
            float g[16], u[16];
            tmem_ld16x2_wait(taddr + c0, taddr + BT + c0, g, u);
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float av = act_mul<T, EXT>(g[j] + bgate, u[j] + bup, w_on_input, col_gam[c0 + j], mimic, ap);
              if (n_ok) out[static_cast<size_t>(c0 + j) * a.ld_out] = from_f32<T>(av);
            }
          }
        } else {
          float* out = reinterpret_cast<float*>(a.out) + n;
          const float bout = (has_bias && n_ok && t.kb0 == 0) ? __ldg(a.bias + static_cast<size_t>(t.e) * a.N + n) : 0.f;
#pragma unroll 1
          for (int c0 = 0; c0 < BT; c0 += 16) {
            float v[16];
            tmem_ld16_wait(taddr + c0, v);
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int orow = col_row[c0 + j];
              if (orow >= 0 && n_ok) {
                float y = v[j] + bout;
                if (!w_on_input) y *= col_gam[c0 + j];
                if (round_pair) y = to_f32<T>(from_f32<T>(y));
                atomicAdd(out + static_cast<size_t>(orow) * a.ld_out, y);
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_tempty[acc]));
      if (++acc == a.acc_stages) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  }

  // ---- teardown (every thread, aborted or not)
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, static_cast<uint32_t>(a.tmem_cols));
  }
  if (threadIdx.x == 0 && *abort_flag != 0) atomicCAS(a.status, 0, *abort_flag);
}

}  // namespace

static size_t stage_bytes_of(const GemmArgs& a) {
  const size_t w = (a.orient == 1) ? 2 * kTileBytes : static_cast<size_t>(a.mode == 0 ? 2 : 1) * kTileBytes;
  const size_t packed = (a.wmode == B200MOE_W_INT4_AWQ) ? w / 4 + 1024 : 0;   // + scale words of the stage
  return w + packed + static_cast<size_t>(a.BT) * kStageKBytes;
}

static size_t ctrl_bytes_of(const GemmArgs& a) {
  // with tokens on M and fewer than 128 token rows loaded, the MMA of the last stage reads up to
  // 16 KiB past its token rows: keep that inside the allocation
  const size_t overread = (a.orient == 1 && a.BT < 128) ? 16384 : 0;
  return 768 /*barriers*/ + 2 * kMaxBT * 8 + static_cast<size_t>(a.E + 1) * 4 + 64 + overread;
}

void gemm_plan(GemmArgs* a) {
  const int kelems = (a->wmode == B200MOE_W_FP8_BLOCK) ? 128 : 64;
  const int tile_n = (a->orient == 1 && a->mode == 1) ? 256 : kTileRows;
  a->num_nt = (a->N + tile_n - 1) / tile_n;
  a->kblocks = (a->K + kelems - 1) / kelems;
  const int cols = (a->orient == 1) ? 256 : (a->mode == 0 ? 2 : 1) * a->BT;
  a->acc_stages = (2 * cols <= 512) ? 2 : 1;
  int need = a->acc_stages * cols;
  int tc = 32;
  while (tc < need) tc <<= 1;
  a->tmem_cols = tc;
  int st = static_cast<int>((kSmemLimit - 1024 - ctrl_bytes_of(*a)) / stage_bytes_of(*a));
  if (st > 10) st = 10;
  if (st < 2) st = 2;
  a->stages = st;
  if (a->max_split <= 0) a->max_split = 16;
}

size_t gemm_smem_bytes(const GemmArgs& a) {
  return 1024 + static_cast<size_t>(a.stages) * stage_bytes_of(a) + ctrl_bytes_of(a);
}

template <int MODE, typename T, int ORIENT, bool W4 = false, bool EXT = false>
static int launch_one(const CUtensorMap& tm_w, const CUtensorMap& tm_x, const GemmArgs& a, int num_sms,
                      cudaStream_t stream) {
  const size_t smem = gemm_smem_bytes(a);
  if (smem > kSmemLimit) return B200MOE_ERR_TOO_LARGE;
  cudaError_t err = cudaFuncSetAttribute(moe_gemm_tc_kernel<MODE, T, ORIENT, W4, EXT>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
  if (err != cudaSuccess) return B200MOE_ERR_CUDA;
  note_launch(W4 ? (MODE == 0 ? "moe_gemm_tc_kernel<gate/up, int4 operands>" : "moe_gemm_tc_kernel<down, int4 operands>")
                 : (MODE == 0 ? "moe_gemm_tc_kernel<gate/up>" : "moe_gemm_tc_kernel<down>"));
  err = launch_kernel(moe_gemm_tc_kernel<MODE, T, ORIENT, W4, EXT>, dim3(num_sms), dim3(W4 ? kThreadsW4 : kThreads), smem,
                      stream, a.pdl != 0, tm_w, tm_x, a);
  return err == cudaSuccess ? B200MOE_OK : B200MOE_ERR_CUDA;
}

template <typename T, bool EXT>
static int launch_typed(const CUtensorMap& tm_w, const CUtensorMap& tm_x, const GemmArgs& a, int num_sms,
                        cudaStream_t stream) {
  if (a.orient == 1)
    return a.mode == 0 ? launch_one<0, T, 1, false, EXT>(tm_w, tm_x, a, num_sms, stream)
                       : launch_one<1, T, 1, false, EXT>(tm_w, tm_x, a, num_sms, stream);
  return a.mode == 0 ? launch_one<0, T, 0, false, EXT>(tm_w, tm_x, a, num_sms, stream)
                     : launch_one<1, T, 0, false, EXT>(tm_w, tm_x, a, num_sms, stream);
}

int launch_gemm_tc(const CUtensorMap& tm_w, const CUtensorMap& tm_x, const GemmArgs& a, int num_sms,
                   cudaStream_t stream) {
  if (a.BT < 16 || a.BT > kMaxBT || a.BT % 16 != 0) return B200MOE_ERR_BAD_ARG;
  if (a.orient == 1 && a.BT > 128) return B200MOE_ERR_BAD_ARG;
  if (a.wmode == B200MOE_W_INT4_AWQ) {
    if (a.dtype != B200MOE_DTYPE_FP16 || a.w_sz == nullptr) return B200MOE_ERR_UNSUPPORTED;
    const bool ext4 = a.bias != nullptr || a.activation == B200MOE_ACT_SWIGLU_OAI;
    if (a.orient == 1) {
      if (ext4)
        return a.mode == 0 ? launch_one<0, __half, 1, true, true>(tm_w, tm_x, a, num_sms, stream)
                           : launch_one<1, __half, 1, true, true>(tm_w, tm_x, a, num_sms, stream);
      return a.mode == 0 ? launch_one<0, __half, 1, true>(tm_w, tm_x, a, num_sms, stream)
                         : launch_one<1, __half, 1, true>(tm_w, tm_x, a, num_sms, stream);
    }
    if (ext4)
      return a.mode == 0 ? launch_one<0, __half, 0, true, true>(tm_w, tm_x, a, num_sms, stream)
                         : launch_one<1, __half, 0, true, true>(tm_w, tm_x, a, num_sms, stream);
    return a.mode == 0 ? launch_one<0, __half, 0, true>(tm_w, tm_x, a, num_sms, stream)
                       : launch_one<1, __half, 0, true>(tm_w, tm_x, a, num_sms, stream);
  }
  if (a.wmode != B200MOE_W_16BIT) return B200MOE_ERR_UNSUPPORTED;
  const bool ext = a.bias != nullptr || a.activation == B200MOE_ACT_SWIGLU_OAI;
  if (a.dtype == B200MOE_DTYPE_BF16)
    return ext ? launch_typed<__nv_bfloat16, true>(tm_w, tm_x, a, num_sms, stream)
               : launch_typed<__nv_bfloat16, false>(tm_w, tm_x, a, num_sms, stream);
  return ext ? launch_typed<__half, true>(tm_w, tm_x, a, num_sms, stream)
             : launch_typed<__half, false>(tm_w, tm_x, a, num_sms, stream);
}

}  // namespace b200moe
