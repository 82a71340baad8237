// Grouped expert GEMMs for FP8 (e4m3) weights with one fp32 scale per 128x128 block and
// activations quantised per token and 128-wide group.
//
// The hardware's block-scaled MMA wants power-of-two scales per 32 elements, not fp32 scales
// per 128, so the scaling is done on the CUDA cores: every 128-wide slice of the reduction
// (one pipeline stage = one swizzle row of FP8) is multiplied into a fresh partial
// accumulator in tensor memory (4 x tcgen05.mma.kind::f8f6f4, K = 32 each); the promotion
// warps read it back, scale it by a_scale[token, slice] * w_scale[row block, slice] and add it
// to accumulators they keep in registers, while the MMA thread is already filling the other
// partial buffer.  Weight rows sit on the MMA's M side, the token block (16/32/64) on N, so
// the promotion costs 2*BT FMAs per thread and slice.
//
// A tile is two 128-row weight blocks that share the token block:
//   mode 0: gate rows n0.. and up rows I+n0..; tail = SiLU*mul, rounding to the 16-bit type,
//           dynamic 1x128 quantisation (the 128 lanes are exactly one group) -> e4m3 + scale.
//   mode 1: rows n0.. and n0+128.. of the down projection; tail = routing weight and
//           red.global.add.f32 into the combine buffer (K may be split across CTAs).
//
// Warps: TMA producer, MMA issuer (owns tensor memory), four promotion warps per group of up
// to 64 tokens (one group for blocks of 16/32/64, two for blocks of 128), and a
// loader warp that prepares the next tile's per-token tables (output row, routing weight,
// activation scales by bulk copy, weight scales) in double-buffered shared memory, so that no
// global-memory latency sits between two tiles of the promotion warps.
#include "gemm_sched.cuh"

namespace b200moe {

namespace {

constexpr int kMaxKB = 64;  // 128-wide reduction slices per tile whose scales are staged in shared memory
constexpr int fp8_threads(int ng) { return 7 * 32 + (ng - 1) * 128; }

// NG = promotion groups; group g owns token columns [g * BT / NG, (g + 1) * BT / NG)
template <int MODE, int BT, int NG>
__global__ void __launch_bounds__(fp8_threads(NG), 1)
moe_gemm_fp8_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                    const GemmArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  constexpr int W_BYTES = 2 * kTileBytes;
  constexpr int X_BYTES = BT * kStageKBytes;
  constexpr int STAGE_BYTES = W_BYTES + X_BYTES;
  constexpr int PCOLS = 2 * BT;  // columns of one partial accumulator (both row blocks)
  constexpr int NPB = (512 / PCOLS) >= 4 ? 4 : 2;  // partial accumulators in flight
  const int stages = a.stages;

  uint8_t* ctrl_base = smem + static_cast<size_t>(stages) * STAGE_BYTES;
  float* s_xs = reinterpret_cast<float*>(ctrl_base);                    // [2][kMaxKB][BT] activation scales
  float* s_ws = s_xs + 2 * kMaxKB * BT;                                 // [2][2][kMaxKB] weight scales
  uint64_t* bar_full = reinterpret_cast<uint64_t*>(s_ws + 2 * 2 * kMaxKB);
  uint64_t* bar_empty = bar_full + stages;
  uint64_t* bar_pfull = bar_empty + stages;
  uint64_t* bar_pempty = bar_pfull + 4;
  uint64_t* bar_sfull = bar_pempty + 4;   // per-tile tables ready
  uint64_t* bar_sempty = bar_sfull + 2;   // per-tile tables released
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_sempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* s_col_row = reinterpret_cast<int*>(tmem_slot + 4);               // [2][128]
  float* s_col_gam = reinterpret_cast<float*>(s_col_row + 2 * 128);     // [2][128]
  float* s_red = s_col_gam + 2 * 128;                                   // [2][NG][4][64]
  int* s_blk_off = reinterpret_cast<int*>(s_red + 2 * 2 * 4 * 64);      // [E+1]
  constexpr int CPT = BT / NG;                                          // token columns per promotion thread

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    for (int s = 0; s < 4; ++s) {
      mbar_init(smem_u32(&bar_pfull[s]), 1);
      mbar_init(smem_u32(&bar_pempty[s]), 4 * NG);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&bar_sfull[s]), 1);
      mbar_init(smem_u32(&bar_sempty[s]), 4 * NG);
    }
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
  const bool active = static_cast<int>(blockIdx.x) < c.grid_eff;
  constexpr int kTileN = (MODE == 0) ? kTileRows : 2 * kTileRows;  // output rows advanced per n-tile
  // row offset of the second weight block inside the expert
  const int second_off = (MODE == 0) ? a.up_row_off : kTileRows;

  if (active && warp == 0 && lane == 0) {
    // =============================== TMA producer ===============================
    int stage = 0;
    uint32_t phase = 0;
    long long issued = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < c.total; tile += c.grid_eff) {
      const TileCoord t = decode_tile(tile, c, s_blk_off, a.E, BT, a.num_nt, a.kblocks, kTileN);
      for (int kb = t.kb0; kb < t.kb1; ++kb) {
        if (!mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1, abort_flag, DEV_TIMEOUT_PRODUCER)) {
          ok = false;
          break;
        }
        const uint32_t full = smem_u32(&bar_full[stage]);
        mbar_arrive_expect_tx(full, static_cast<uint32_t>(STAGE_BYTES));
        const uint32_t sw = smem_u32(smem + static_cast<size_t>(stage) * STAGE_BYTES);
        const int k0 = kb * kStageKBytes;  // one byte per element
        tma_load_3d(sw, &tm_w, full, k0, t.n0, t.e);
        tma_load_3d(sw + kTileBytes, &tm_w, full, k0, second_off + t.n0, t.e);  // rows past the expert zero-fill
        tma_load_2d(sw + W_BYTES, &tm_x, full, k0, t.row0);
        ++issued;
        if (++stage == stages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
    if (!ok) {
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
    const uint32_t idesc = make_idesc(0u /* e4m3 */, kTileRows, static_cast<uint32_t>(BT));
    int stage = 0;
    uint32_t phase = 0, j = 0;  // j counts reduction slices over the whole launch
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < c.total; tile += c.grid_eff) {
      const TileCoord t = decode_tile(tile, c, s_blk_off, a.E, BT, a.num_nt, a.kblocks, kTileN);
      for (int kb = t.kb0; kb < t.kb1; ++kb, ++j) {
        const uint32_t pb = j % NPB;
        if (!mbar_wait(smem_u32(&bar_full[stage]), phase, abort_flag, DEV_TIMEOUT_MMA) ||
            !mbar_wait(smem_u32(&bar_pempty[pb]), ((j / NPB) & 1u) ^ 1u, abort_flag, DEV_TIMEOUT_MMA)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d0 = tmem_base + pb * PCOLS;
        const uint32_t sw = smem_u32(smem + static_cast<size_t>(stage) * STAGE_BYTES);
        const uint64_t dw = smem_desc_k_sw128(sw);
        const uint64_t du = smem_desc_k_sw128(sw + kTileBytes);
        const uint64_t dx = smem_desc_k_sw128(sw + W_BYTES);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          tc_mma_f8(d0, dw + 2 * k, dx + 2 * k, idesc, k > 0 ? 1u : 0u);
          tc_mma_f8(d0 + BT, du + 2 * k, dx + 2 * k, idesc, k > 0 ? 1u : 0u);
        }
        tc_commit(smem_u32(&bar_empty[stage]));
        tc_commit(smem_u32(&bar_pfull[pb]));
        if (++stage == stages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (active && warp == 6) {
    // =============================== per-tile table loader ======================
    const int kb_total = a.kblocks;
    int iter = 0;
    for (int tile = blockIdx.x; tile < c.total; tile += c.grid_eff, ++iter) {
      const TileCoord t = decode_tile(tile, c, s_blk_off, a.E, BT, a.num_nt, a.kblocks, kTileN);
      const int buf = iter & 1;
      if (!mbar_wait(smem_u32(&bar_sempty[buf]), ((iter >> 1) & 1) ^ 1, abort_flag, DEV_TIMEOUT_EPILOGUE)) break;
      const int nkb = t.kb1 - t.kb0;
      for (int cidx = lane; cidx < BT; cidx += 32) {
        const int slot = a.sorted_ids[t.row0 + cidx];
        const bool valid = slot >= 0 && slot < a.P;
        s_col_row[buf * 128 + cidx] = valid ? (MODE == 1 ? slot / a.topk : slot) : -1;
        s_col_gam[buf * 128 + cidx] = valid ? a.row_gamma[t.row0 + cidx] : 0.f;
      }
      const int nb0 = t.n0 / 128, nb1 = (second_off + t.n0) / 128;
      const float* ws0 = a.w_scale + (static_cast<size_t>(t.e) * a.w_scale_rows + nb0) * kb_total + t.kb0;
      const float* ws1 = a.w_scale + (static_cast<size_t>(t.e) * a.w_scale_rows + nb1) * kb_total + t.kb0;
      const bool second_ok = nb1 < a.w_scale_rows;
      float* ws_t = s_ws + buf * 2 * kMaxKB;
      for (int i = lane; i < nkb; i += 32) {
        ws_t[i] = __ldg(ws0 + i);
        ws_t[kMaxKB + i] = second_ok ? __ldg(ws1 + i) : 0.f;
      }
      __syncwarp();
      const uint32_t sfull = smem_u32(&bar_sfull[buf]);
      if (lane == 0) mbar_arrive_expect_tx(sfull, static_cast<uint32_t>(nkb * BT * 4));
      __syncwarp();
      // one bulk copy per reduction slice: BT consecutive activation scales
      for (int i = lane; i < nkb; i += 32)
        bulk_copy_g2s(smem_u32(s_xs + (buf * kMaxKB + i) * BT),
                      a.x_scale + static_cast<size_t>(t.kb0 + i) * a.ld_xscale + t.row0, BT * 4, sfull);
    }
  } else if (active && warp >= 2 && warp != 6) {
    // =============================== promotion + tail ===========================
    const int grp = warp < 6 ? 0 : 1;               // promotion group
    const int gw = warp < 6 ? warp - 2 : warp - 7;  // warp inside the group
    const int quad = warp & 3;                      // TMEM lane quadrant (each group covers all four)
    const int ep_tid = gw * 32 + lane;
    const int lrow = quad * 32 + lane;
    const int cb = grp * CPT;                       // first token column of this thread
    const bool w_on_input = (a.flags & B200MOE_FLAG_WEIGHT_ON_INPUT) != 0;
    uint32_t j = 0;
    int iter = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < c.total; tile += c.grid_eff, ++iter) {
      const TileCoord t = decode_tile(tile, c, s_blk_off, a.E, BT, a.num_nt, a.kblocks, kTileN);
      const int buf = iter & 1;
      const int* col_row = s_col_row + buf * 128 + cb;
      const float* col_gam = s_col_gam + buf * 128 + cb;
      const float* xs_t = s_xs + buf * kMaxKB * BT;
      const float* ws_t = s_ws + buf * 2 * kMaxKB;
      if (!mbar_wait(smem_u32(&bar_sfull[buf]), (iter >> 1) & 1, abort_flag, DEV_TIMEOUT_EPILOGUE)) break;

      float acc0[CPT], acc1[CPT];
#pragma unroll
      for (int i = 0; i < CPT; ++i) {
        acc0[i] = 0.f;
        acc1[i] = 0.f;
      }

      constexpr int CH = (CPT < 32 || CPT > 32 && NG > 1) ? 16 : 32;  // columns drained from tensor memory per step
      for (int kb = t.kb0; kb < t.kb1; ++kb, ++j) {
        const float w0 = ws_t[kb - t.kb0];
        const float w1 = ws_t[kMaxKB + kb - t.kb0];
        const float4* sx = reinterpret_cast<const float4*>(xs_t + (kb - t.kb0) * BT + cb);
        const uint32_t pb = j % NPB;
        if (!mbar_wait(smem_u32(&bar_pfull[pb]), (j / NPB) & 1u, abort_flag, DEV_TIMEOUT_EPILOGUE)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + pb * PCOLS + cb;
#pragma unroll
        for (int c0 = 0; c0 < CPT; c0 += CH) {
          float g[CH], u[CH];
          if constexpr (CH == 32) tmem_ld32x2_wait(taddr + c0, taddr + BT + c0, g, u);
          else tmem_ld16x2_wait(taddr + c0, taddr + BT + c0, g, u);
#pragma unroll
          for (int q = 0; q < CH / 4; ++q) {
            const float4 s4 = sx[c0 / 4 + q];
            const float sv[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              acc0[c0 + 4 * q + i] = fmaf(g[4 * q + i], sv[i] * w0, acc0[c0 + 4 * q + i]);
              acc1[c0 + 4 * q + i] = fmaf(u[4 * q + i], sv[i] * w1, acc1[c0 + 4 * q + i]);
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_pempty[pb]));
      }
      if (!ok) break;

      const int n = t.n0 + lrow;
      if (MODE == 0) {
        // activation, rounding to the 16-bit type, then one 1x128 group per (token, tile):
        // warp maxima by redux on the bit patterns (non-negative floats order like integers),
        // one thread per token turns the four warp maxima into the scale and its reciprocal.
        float* red = s_red + (buf * 2 + grp) * 4 * 64;
#pragma unroll
        for (int i = 0; i < CPT; ++i) {
          float av = act_mul<__nv_bfloat16>(acc0[i], acc1[i], w_on_input, col_gam[i], false, a.activation);
          av = (a.dtype == B200MOE_DTYPE_BF16) ? __bfloat162float(__float2bfloat16_rn(av))
                                               : __half2float(__float2half_rn(av));
          acc0[i] = av;
          const unsigned m = __reduce_max_sync(0xffffffffu, __float_as_uint(fabsf(av)));
          if (lane == 0) red[gw * 64 + i] = __uint_as_float(m);
        }
        named_bar_sync(2 + 3 * grp, 128);
        if (ep_tid < CPT) {
          const float amax = fmaxf(fmaxf(red[ep_tid], red[64 + ep_tid]), fmaxf(red[128 + ep_tid], red[192 + ep_tid]));
          const float sc = __fdiv_rn(fmaxf(amax, 1e-10f), 448.0f);
          a.out_scale[static_cast<size_t>(t.n0 / 128) * a.ld_xscale + t.row0 + cb + ep_tid] = sc;
          red[ep_tid] = __fdiv_rn(1.0f, sc);
        }
        named_bar_sync(4 + 2 * grp, 128);
        uint8_t* outq = a.out_q + static_cast<size_t>(t.row0 + cb) * a.ld_out + n;
#pragma unroll
        for (int i = 0; i < CPT; ++i) {
          outq[static_cast<size_t>(i) * a.ld_out] =
              static_cast<uint8_t>(__nv_cvt_float_to_fp8(acc0[i] * red[i], __NV_SATFINITE, __NV_E4M3));
        }
      } else {
        float* out = reinterpret_cast<float*>(a.out) + n;
        const bool second = n + kTileRows < a.N;
#pragma unroll
        for (int i = 0; i < CPT; ++i) {
          const int orow = col_row[i];
          if (orow >= 0) {
            const float gam = w_on_input ? 1.0f : col_gam[i];
            atomicAdd(out + static_cast<size_t>(orow) * a.ld_out, acc0[i] * gam);
            if (second) atomicAdd(out + static_cast<size_t>(orow) * a.ld_out + kTileRows, acc1[i] * gam);
          }
        }
      }
      // the tables of this tile may now be overwritten
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_sempty[buf]));
    }
  }

  // ---- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, static_cast<uint32_t>(a.tmem_cols));
  }
  if (threadIdx.x == 0 && *abort_flag != 0) atomicCAS(a.status, 0, *abort_flag);
}

size_t fp8_stage_bytes(const GemmArgs& a) {
  return 2 * static_cast<size_t>(kTileBytes) + static_cast<size_t>(a.BT) * kStageKBytes;
}
size_t fp8_ctrl_bytes(const GemmArgs& a) {
  return 2 * static_cast<size_t>(kMaxKB) * a.BT * 4 + 2 * 2 * kMaxKB * 4 + 512 /*barriers*/ + 2 * 128 * 8 +
         2 * 2 * 4 * 64 * 4 + static_cast<size_t>(a.E + 1) * 4 + 64;
}

template <int MODE, int BT, int NG>
int launch_fp8(const CUtensorMap& tm_w, const CUtensorMap& tm_x, const GemmArgs& a, int num_sms,
               cudaStream_t stream) {
  const size_t smem = 1024 + static_cast<size_t>(a.stages) * fp8_stage_bytes(a) + fp8_ctrl_bytes(a);
  if (smem > kSmemLimit) return B200MOE_ERR_TOO_LARGE;
  if (cudaFuncSetAttribute(moe_gemm_fp8_kernel<MODE, BT, NG>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(smem)) != cudaSuccess)
    return B200MOE_ERR_CUDA;
  cudaError_t err = launch_kernel(moe_gemm_fp8_kernel<MODE, BT, NG>, dim3(num_sms), dim3(fp8_threads(NG)), smem,
                                  stream, a.pdl != 0, tm_w, tm_x, a);
  return err == cudaSuccess ? B200MOE_OK : B200MOE_ERR_CUDA;
}

}  // namespace

void gemm_plan_fp8(GemmArgs* a) {
  a->orient = 0;
  const int tile_n = (a->mode == 0) ? kTileRows : 2 * kTileRows;
  a->num_nt = (a->N + tile_n - 1) / tile_n;
  a->kblocks = (a->K + 127) / 128;
  const int pcols = 2 * a->BT;                       // one partial: two row blocks
  const int cols = ((512 / pcols) >= 4 ? 4 : 2) * pcols;
  int tc = 32;
  while (tc < cols) tc <<= 1;
  a->tmem_cols = tc;
  a->acc_stages = 2;
  int st = static_cast<int>((kSmemLimit - 1024 - fp8_ctrl_bytes(*a)) / fp8_stage_bytes(*a));
  if (st > 10) st = 10;
  if (st < 2) st = 2;
  a->stages = st;
  if (a->max_split <= 0) a->max_split = 16;
}

int launch_gemm_fp8(const CUtensorMap& tm_w, const CUtensorMap& tm_x, const GemmArgs& a, int num_sms,
                    cudaStream_t stream) {
  if (a.wmode != B200MOE_W_FP8_BLOCK) return B200MOE_ERR_BAD_ARG;
  if (a.K % 128 != 0 || a.N % 128 != 0 || a.K / 128 > kMaxKB) return B200MOE_ERR_UNSUPPORTED;
#define B200MOE_FP8_CASE(bt, ng)                                                          \
  case bt:                                                                                \
    return a.mode == 0 ? launch_fp8<0, bt, ng>(tm_w, tm_x, a, num_sms, stream)            \
                       : launch_fp8<1, bt, ng>(tm_w, tm_x, a, num_sms, stream);
  switch (a.BT) {
    B200MOE_FP8_CASE(16, 1)
    B200MOE_FP8_CASE(32, 1)
    B200MOE_FP8_CASE(64, 2)
    B200MOE_FP8_CASE(128, 2)
    default:
      return B200MOE_ERR_BAD_ARG;
  }
#undef B200MOE_FP8_CASE
}

}  // namespace b200moe
