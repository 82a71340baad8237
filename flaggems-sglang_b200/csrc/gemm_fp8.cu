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
  uint64_t* bar_meet = bar_sempty + 2;    // [NG] meeting point of a promotion group's four warps
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_meet + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* s_col_row = reinterpret_cast<int*>(tmem_slot + 4);               // [2][128]
  float* s_col_gam = reinterpret_cast<float*>(s_col_row + 2 * 128);     // [2][128]
  float* s_red = s_col_gam + 2 * 128;                                   // [2][NG][4][64]
  unsigned long long* s_col_ptr = reinterpret_cast<unsigned long long*>(s_red + 2 * 2 * 4 * 64);   // [2][128] mode 1: base of each token's output row
  int* s_blk_off = reinterpret_cast<int*>(s_col_ptr + 2 * 128);         // [E+1]
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
      mbar_init(smem_u32(&bar_meet[s]), 4);
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
        const int orow = valid ? (MODE == 1 ? slot / a.topk : slot) : -1;
        s_col_row[buf * 128 + cidx] = orow;
        s_col_gam[buf * 128 + cidx] = valid ? a.row_gamma[t.row0 + cidx] : 0.f;
        if (MODE == 1 && valid)
          s_col_ptr[buf * 128 + cidx] = reinterpret_cast<unsigned long long>(
              out_row_base(a, a.out, orow, static_cast<size_t>(a.ld_out) * sizeof(float)));
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
    uint32_t meet_phase = 0;
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
        // per-expert bias of this thread's gate row and up / linear row, and the clamped swiglu: the
        // rarer tail, kept out of the plain one
        const bool ext = a.bias != nullptr || a.activation == B200MOE_ACT_SWIGLU_OAI;
        float bg = 0.f, bu = 0.f;
        if (a.bias != nullptr && n < a.N) {
          bg = __ldg(a.bias + static_cast<size_t>(t.e) * 2 * a.N + n);
          bu = __ldg(a.bias + static_cast<size_t>(t.e) * 2 * a.N + a.N + n);
        }
#pragma unroll
        for (int i = 0; i < CPT; ++i) {
          float av = ext ? act_mul<__nv_bfloat16, true>(acc0[i] + bg, acc1[i] + bu, w_on_input, col_gam[i], false, act_params(a))
                         : act_mul<__nv_bfloat16>(acc0[i], acc1[i], w_on_input, col_gam[i], false, act_params(a));
          av = (a.dtype == B200MOE_DTYPE_BF16) ? __bfloat162float(__float2bfloat16_rn(av))
                                               : __half2float(__float2half_rn(av));
          acc0[i] = av;
          const unsigned m = __reduce_max_sync(0xffffffffu, __float_as_uint(fabsf(av)));
          if (lane == 0) red[gw * 64 + i] = __uint_as_float(m);
        }
        if (!warps_meet(smem_u32(&bar_meet[grp]), meet_phase, lane, abort_flag, DEV_TIMEOUT_EPILOGUE)) break;
        if (ep_tid < CPT) {
          const float amax = fmaxf(fmaxf(red[ep_tid], red[64 + ep_tid]), fmaxf(red[128 + ep_tid], red[192 + ep_tid]));
          const float sc = __fdiv_rn(fmaxf(amax, 1e-10f), 448.0f);
          a.out_scale[static_cast<size_t>(t.n0 / 128) * a.ld_xscale + t.row0 + cb + ep_tid] = sc;
          red[ep_tid] = __fdiv_rn(1.0f, sc);
        }
        if (!warps_meet(smem_u32(&bar_meet[grp]), meet_phase, lane, abort_flag, DEV_TIMEOUT_EPILOGUE)) break;
        uint8_t* outq = a.out_q + static_cast<size_t>(t.row0 + cb) * a.ld_out + n;
#pragma unroll
        for (int i = 0; i < CPT; ++i) {
          outq[static_cast<size_t>(i) * a.ld_out] =
              static_cast<uint8_t>(__nv_cvt_float_to_fp8(acc0[i] * red[i], __NV_SATFINITE, __NV_E4M3));
        }
      } else {
        const unsigned long long* col_ptr = s_col_ptr + buf * 128 + cb;
        const bool second = n + kTileRows < a.N;
        float b0 = 0.f, b1 = 0.f;      // bias of the two output columns; the first reduction split carries it
        if (a.bias != nullptr && t.kb0 == 0) {
          if (n < a.N) b0 = __ldg(a.bias + static_cast<size_t>(t.e) * a.N + n);
          if (second) b1 = __ldg(a.bias + static_cast<size_t>(t.e) * a.N + n + kTileRows);
        }
#pragma unroll
        for (int i = 0; i < CPT; ++i) {
          const int orow = col_row[i];
          if (orow >= 0) {
            const float gam = w_on_input ? 1.0f : col_gam[i];
            float* out = reinterpret_cast<float*>(col_ptr[i]) + n;   // the token's row, here or on its owner
            atomicAdd(out, (acc0[i] + b0) * gam);
            if (second) atomicAdd(out + kTileRows, (acc1[i] + b1) * gam);
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

// ------------------------------------------------------------------------------------------
// Tokens-on-M variant for 128-token blocks (prefill-sized batches).
//
// One tcgen05.mma costs about the same issue time whatever its N, so with many tokens per
// expert the token block goes on the M side (128 rows) and 256 weight rows on the N side:
// four MMAs per 128-wide reduction slice instead of sixteen.  An accumulator row is then a
// token, so the activation scale is one scalar per thread and slice, the weight scale one
// scalar per 128 columns; two promotion groups split the 256 columns (gate columns
// [64g, 64g+64) with the matching up columns for mode 0, columns [128g, 128g+128) for mode 1)
// and keep 128 accumulators per thread.  The 1x128 quantisation group of a token is the 64
// activations of its thread in group 0 plus the 64 of its thread in group 1: the two partial
// maxima meet in shared memory, no shuffles.
constexpr int kThreadsFp8TokM = 7 * 32 + 128;
constexpr int kPairStageBytes = 2 * 128 * 144;   // staging of 16-bit pair rows: two groups x 128 rows x (128 + 16) bytes

#ifdef B200MOE_STALL_STATS
__device__ unsigned long long g_stall_fp8[16];
#define STALL_ADD8(slot, v) atomicAdd(&g_stall_fp8[slot], v)
#else
#define STALL_ADD8(slot, v) ((void)0)
#endif

template <int MODE>
__global__ void __launch_bounds__(kThreadsFp8TokM, 1)
moe_gemm_fp8_tokm_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                         const GemmArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  constexpr int BT = 128;
  constexpr int W_BYTES = 2 * kTileBytes;
  constexpr int X_BYTES = BT * kStageKBytes;
  constexpr int STAGE_BYTES = W_BYTES + X_BYTES;
  constexpr int PCOLS = 256;
  const int stages = a.stages;

  const int KBS = a.kblocks;   // reduction slices of a whole row: size of the per-tile scale tables
  uint8_t* ctrl_base = smem + static_cast<size_t>(stages) * STAGE_BYTES;
  float* s_xs = reinterpret_cast<float*>(ctrl_base);                    // [2][KBS][128] activation scales
  float* s_ws = s_xs + 2 * KBS * BT;                                    // [2][2][KBS] weight scales
  // mode 1 with rows stored per pair: staging for coalesced stores, [2 groups][128 rows][144 bytes]
  uint8_t* s_stage = reinterpret_cast<uint8_t*>(s_ws + 2 * 2 * KBS);
  uint64_t* bar_full = reinterpret_cast<uint64_t*>(s_stage + ((MODE == 1 && a.out_pairs != nullptr) ? kPairStageBytes : 0));
  uint64_t* bar_empty = bar_full + stages;
  uint64_t* bar_pfull = bar_empty + stages;
  uint64_t* bar_pempty = bar_pfull + 2;
  uint64_t* bar_sfull = bar_pempty + 2;
  uint64_t* bar_sempty = bar_sfull + 2;
  uint64_t* bar_meet = bar_sempty + 2;          // [2] one per promotion group: meetings around the staged stores
  uint64_t* bar_meet8 = bar_meet + 2;           // both groups: the halves of a quantisation group's maximum
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_meet8 + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* s_col_row = reinterpret_cast<int*>(tmem_slot + 4);               // [2][128] output row of each token
  float* s_col_gam = reinterpret_cast<float*>(s_col_row + 2 * 128);     // [2][128]
  float* s_red = s_col_gam + 2 * 128;                                   // [2][2][128] partial group maxima
  unsigned long long* s_col_ptr = reinterpret_cast<unsigned long long*>(s_red + 2 * 2 * 128);   // [2][128] mode 1: base of each row's output row
  int* s_blk_off = reinterpret_cast<int*>(s_col_ptr + 2 * 128);         // [E+1]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&bar_pfull[s]), 1);
      mbar_init(smem_u32(&bar_pempty[s]), 8);
      mbar_init(smem_u32(&bar_sfull[s]), 1);
      mbar_init(smem_u32(&bar_sempty[s]), 8);
      mbar_init(smem_u32(&bar_meet[s]), 4);
    }
    mbar_init(smem_u32(bar_meet8), 8);
    *abort_flag = 0;
    fence_mbar_init();
    fence_proxy_async_smem();
    prefetch_tmap(&tm_w);
    prefetch_tmap(&tm_x);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), 512u);
    tmem_relinquish();
  }
  griddep_wait();
  griddep_launch_dependents();
  for (int e = threadIdx.x; e <= a.E; e += blockDim.x) s_blk_off[e] = a.blk_off[e];
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const Ctrl c = make_ctrl(a, MODE == 1);
  const bool active = static_cast<int>(blockIdx.x) < c.grid_eff;
  constexpr int kTileN = (MODE == 0) ? kTileRows : 2 * kTileRows;
  const int second_off = (MODE == 0) ? a.up_row_off : kTileRows;

  if (active && warp == 0 && lane == 0) {
    // =============================== TMA producer ===============================
    int stage = 0;
    uint32_t phase = 0;
    long long issued = 0;
    bool ok = true;
    unsigned long long w_empty = 0;
    const long long role_t0 = clock64();
    for (int tile = blockIdx.x; ok && tile < c.total; tile += c.grid_eff) {
      const TileCoord t = decode_tile(tile, c, s_blk_off, a.E, BT, a.num_nt, a.kblocks, kTileN);
      for (int kb = t.kb0; kb < t.kb1; ++kb) {
        if (!mbar_wait_t(smem_u32(&bar_empty[stage]), phase ^ 1, abort_flag, DEV_TIMEOUT_PRODUCER, w_empty)) {
          ok = false;
          break;
        }
        const uint32_t full = smem_u32(&bar_full[stage]);
        mbar_arrive_expect_tx(full, static_cast<uint32_t>(STAGE_BYTES));
        const uint32_t sw = smem_u32(smem + static_cast<size_t>(stage) * STAGE_BYTES);
        const int k0 = kb * kStageKBytes;
        tma_load_3d(sw, &tm_w, full, k0, t.n0, t.e);
        tma_load_3d(sw + kTileBytes, &tm_w, full, k0, second_off + t.n0, t.e);
        tma_load_2d(sw + W_BYTES, &tm_x, full, k0, t.row0);
        ++issued;
        if (++stage == stages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
    STALL_ADD8(0, w_empty);
    STALL_ADD8(8, static_cast<unsigned long long>(clock64() - role_t0));
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
    const uint32_t idesc = make_idesc(0u /* e4m3 */, kTileRows, 256u);
    int stage = 0;
    uint32_t phase = 0, j = 0;
    bool ok = true;
    unsigned long long w_full = 0, w_pempty = 0;
    const long long role_t0 = clock64();
    for (int tile = blockIdx.x; ok && tile < c.total; tile += c.grid_eff) {
      const TileCoord t = decode_tile(tile, c, s_blk_off, a.E, BT, a.num_nt, a.kblocks, kTileN);
      for (int kb = t.kb0; kb < t.kb1; ++kb, ++j) {
        const uint32_t pb = j & 1u;
        if (!mbar_wait_t(smem_u32(&bar_full[stage]), phase, abort_flag, DEV_TIMEOUT_MMA, w_full) ||
            !mbar_wait_t(smem_u32(&bar_pempty[pb]), ((j >> 1) & 1u) ^ 1u, abort_flag, DEV_TIMEOUT_MMA, w_pempty)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d0 = tmem_base + pb * PCOLS;
        const uint32_t sw = smem_u32(smem + static_cast<size_t>(stage) * STAGE_BYTES);
        const uint64_t dw = smem_desc_k_sw128(sw);             // 256 weight rows: N side
        const uint64_t dx = smem_desc_k_sw128(sw + W_BYTES);   // 128 token rows: M side
#pragma unroll
        for (int k = 0; k < 4; ++k) tc_mma_f8(d0, dx + 2 * k, dw + 2 * k, idesc, k > 0 ? 1u : 0u);
        tc_commit(smem_u32(&bar_empty[stage]));
        tc_commit(smem_u32(&bar_pfull[pb]));
        if (++stage == stages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
    STALL_ADD8(1, w_pempty);
    STALL_ADD8(2, w_full);
    STALL_ADD8(9, static_cast<unsigned long long>(clock64() - role_t0));
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
        // mode 1: output row = token, or the pair's own slot when rows are stored per pair
        const int orow = valid ? ((MODE == 1 && a.out_pairs == nullptr) ? slot / a.topk : slot) : -1;
        s_col_row[buf * 128 + cidx] = orow;
        s_col_gam[buf * 128 + cidx] = valid ? a.row_gamma[t.row0 + cidx] : 0.f;
        if (MODE == 1 && valid)
          s_col_ptr[buf * 128 + cidx] = reinterpret_cast<unsigned long long>(
              a.out_pairs != nullptr ? out_row_base(a, a.out_pairs, orow, static_cast<size_t>(a.N) * 2)
                                     : out_row_base(a, a.out, orow, static_cast<size_t>(a.ld_out) * sizeof(float)));
      }
      const int nb0 = t.n0 / 128, nb1 = (second_off + t.n0) / 128;
      const float* ws0 = a.w_scale + (static_cast<size_t>(t.e) * a.w_scale_rows + nb0) * kb_total + t.kb0;
      const float* ws1 = a.w_scale + (static_cast<size_t>(t.e) * a.w_scale_rows + nb1) * kb_total + t.kb0;
      const bool second_ok = nb1 < a.w_scale_rows;
      float* ws_t = s_ws + buf * 2 * KBS;
      for (int i = lane; i < nkb; i += 32) {
        ws_t[i] = __ldg(ws0 + i);
        ws_t[KBS + i] = second_ok ? __ldg(ws1 + i) : 0.f;
      }
      __syncwarp();
      const uint32_t sfull = smem_u32(&bar_sfull[buf]);
      if (lane == 0) mbar_arrive_expect_tx(sfull, static_cast<uint32_t>(nkb * BT * 4));
      __syncwarp();
      for (int i = lane; i < nkb; i += 32)
        bulk_copy_g2s(smem_u32(s_xs + (buf * KBS + i) * BT),
                      a.x_scale + static_cast<size_t>(t.kb0 + i) * a.ld_xscale + t.row0, BT * 4, sfull);
    }
  } else if (active && warp >= 2 && warp != 6) {
    // =============================== promotion + tail ===========================
    const int grp = warp < 6 ? 0 : 1;
    const int quad = warp & 3;
    const int lrow = quad * 32 + lane;  // token row inside the block = TMEM lane
    const bool w_on_input = (a.flags & B200MOE_FLAG_WEIGHT_ON_INPUT) != 0;
    // columns of this thread: mode 0 -> gate [64g, 64g+64) and up [128+64g, ..+64); mode 1 -> [128g, 128g+128)
    const uint32_t colA = (MODE == 0) ? 64u * grp : 128u * grp;
    const uint32_t colB = (MODE == 0) ? 128u + 64u * grp : 128u * grp + 64u;
    uint32_t j = 0;
    uint32_t meet_phase = 0, meet8_phase = 0;
    int iter = 0;
    bool ok = true;
    unsigned long long w_pfull = 0, w_sfull = 0, t_tail = 0;
    const long long role_t0 = clock64();
    for (int tile = blockIdx.x; ok && tile < c.total; tile += c.grid_eff, ++iter) {
      const TileCoord t = decode_tile(tile, c, s_blk_off, a.E, BT, a.num_nt, a.kblocks, kTileN);
      const int buf = iter & 1;
      const float* xs_t = s_xs + buf * KBS * BT;
      const float* ws_t = s_ws + buf * 2 * KBS;
      if (!mbar_wait_t(smem_u32(&bar_sfull[buf]), (iter >> 1) & 1, abort_flag, DEV_TIMEOUT_EPILOGUE, w_sfull)) break;
      const int orow = s_col_row[buf * 128 + lrow];
      const float gam = s_col_gam[buf * 128 + lrow];

      // running sums stay packed two to a 64-bit register for the whole reduction
      unsigned long long pA[32], pB[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        pA[i] = 0ull;
        pB[i] = 0ull;
      }
      for (int kb = t.kb0; kb < t.kb1; ++kb, ++j) {
        const float sx = xs_t[(kb - t.kb0) * BT + lrow];
        // mode 0: A columns belong to the first weight block, B columns to the second;
        // mode 1: group g works entirely inside weight block g
        const float fA = sx * ws_t[(MODE == 0 ? 0 : grp * KBS) + kb - t.kb0];
        const float fB = sx * ws_t[(MODE == 0 ? KBS : grp * KBS) + kb - t.kb0];
        const uint32_t pb = j & 1u;
        if (!mbar_wait_t(smem_u32(&bar_pfull[pb]), (j >> 1) & 1u, abort_flag, DEV_TIMEOUT_EPILOGUE, w_pfull)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + pb * PCOLS;
        // packed f32x2 FMAs on register pairs (one instruction per two accumulators), 16 columns of
        // each half at a time to stay inside the register budget
        const unsigned long long fA2 = pack_f32x2(fA, fA), fB2 = pack_f32x2(fB, fB);
#pragma unroll
        for (int c0 = 0; c0 < 64; c0 += 16) {
          uint32_t g[16], u[16];
          tmem_ld16x2_wait_u32(taddr + colA + c0, taddr + colB + c0, g, u);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            ffma2_packed(pA[c0 / 2 + i], g[2 * i], g[2 * i + 1], fA2);
            ffma2_packed(pB[c0 / 2 + i], u[2 * i], u[2 * i + 1], fB2);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_pempty[pb]));
      }
      if (!ok) break;
      const long long tail_t0 = clock64();
      float accA[64], accB[64];
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        unpack_f32x2(pA[i], accA[2 * i], accA[2 * i + 1]);
        unpack_f32x2(pB[i], accB[2 * i], accB[2 * i + 1]);
      }

      if (MODE == 1 && a.bias != nullptr && t.kb0 == 0) {
        // bias of columns n0 + 128 grp + [0, 128): accA holds the first 64, accB the next 64
        const float* bo = a.bias + static_cast<size_t>(t.e) * a.N + t.n0 + 128 * grp;
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          accA[i] += (t.n0 + 128 * grp + i < a.N) ? __ldg(bo + i) : 0.f;
          accB[i] += (t.n0 + 128 * grp + 64 + i < a.N) ? __ldg(bo + 64 + i) : 0.f;
        }
      }
      if (MODE == 0) {
        // 64 activations of this token; the other 64 of its quantisation group live in the
        // same lane of the other promotion group
        float amax = 0.f;
        const bool ext = a.bias != nullptr || a.activation == B200MOE_ACT_SWIGLU_OAI;
        if (a.bias != nullptr) {
          // gate columns n0 + 64 grp + i and the matching up / linear columns of the same expert
          const float* bgp = a.bias + static_cast<size_t>(t.e) * 2 * a.N + t.n0 + 64 * grp;
#pragma unroll
          for (int i = 0; i < 64; ++i) {
            const bool in = t.n0 + 64 * grp + i < a.N;
            accA[i] += in ? __ldg(bgp + i) : 0.f;
            accB[i] += in ? __ldg(bgp + a.N + i) : 0.f;
          }
        }
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          float av = ext ? act_mul<__nv_bfloat16, true>(accA[i], accB[i], w_on_input, gam, false, act_params(a))
                         : act_mul<__nv_bfloat16>(accA[i], accB[i], w_on_input, gam, false, act_params(a));
          av = (a.dtype == B200MOE_DTYPE_BF16) ? __bfloat162float(__float2bfloat16_rn(av))
                                               : __half2float(__float2half_rn(av));
          accA[i] = av;
          amax = fmaxf(amax, fabsf(av));
        }
        float* red = s_red + buf * 2 * 128;
        red[grp * 128 + lrow] = amax;
        if (!warps_meet(smem_u32(bar_meet8), meet8_phase, lane, abort_flag, DEV_TIMEOUT_EPILOGUE)) break;
        amax = fmaxf(red[lrow], red[128 + lrow]);
        const float sc = __fdiv_rn(fmaxf(amax, 1e-10f), 448.0f);
        const float inv = __fdiv_rn(1.0f, sc);
        const int r = t.row0 + lrow;
        if (grp == 0) a.out_scale[static_cast<size_t>(t.n0 / 128) * a.ld_xscale + r] = sc;
        uint32_t pk[16];
#pragma unroll
        for (int q = 0; q < 16; ++q) {
          // two values per conversion instruction
          const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(accA[4 * q] * inv, accA[4 * q + 1] * inv),
                                                       __NV_SATFINITE, __NV_E4M3);
          const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(accA[4 * q + 2] * inv, accA[4 * q + 3] * inv),
                                                       __NV_SATFINITE, __NV_E4M3);
          pk[q] = lo | (hi << 16);
        }
        uint4* dst = reinterpret_cast<uint4*>(a.out_q + static_cast<size_t>(r) * a.ld_out + t.n0 + 64 * grp);
#pragma unroll
        for (int q = 0; q < 4; ++q) dst[q] = make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);
      } else if (a.out_pairs != nullptr) {
        // The pair's row, weighted and rounded to the 16-bit type.  A thread owns 128 contiguous
        // columns of one row; storing them directly would touch 32 rows per warp instruction, so
        // the group's four warps stage 64 columns at a time in shared memory (144-byte row pitch)
        // and write them out with 16-byte stores that cover four rows per instruction.
        const float scale = w_on_input ? 1.0f : gam;
        const bool bf = a.dtype == B200MOE_DTYPE_BF16;
        uint8_t* stage_g = s_stage + grp * (128 * 144);
        const int gtid = quad * 32 + lane;            // thread within the group
        const uint32_t meet = smem_u32(&bar_meet[grp]);
        auto group_meets = [&]() -> bool { return warps_meet(meet, meet_phase, lane, abort_flag, DEV_TIMEOUT_EPILOGUE); };
#pragma unroll
        for (int round = 0; round < 2 && ok; ++round) {
          const float* src = (round == 0) ? accA : accB;
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            uint32_t w[4];
#pragma unroll
            for (int b = 0; b < 4; ++b) {
              const float lo = src[8 * q + 2 * b] * scale, hi = src[8 * q + 2 * b + 1] * scale;
              if (bf) {
                __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
                w[b] = *reinterpret_cast<uint32_t*>(&v);
              } else {
                __half2 v = __floats2half2_rn(lo, hi);
                w[b] = *reinterpret_cast<uint32_t*>(&v);
              }
            }
            *reinterpret_cast<uint4*>(stage_g + gtid * 144 + q * 16) = make_uint4(w[0], w[1], w[2], w[3]);
          }
          if (!group_meets()) {
            ok = false;
            break;
          }
          const int col0 = t.n0 + 128 * grp + 64 * round;
          if (col0 < a.N) {
#pragma unroll
            for (int it = 0; it < 8; ++it) {
              const int idx = it * 128 + gtid;
              const int row = idx >> 3, ch = idx & 7;
              const int prow = s_col_row[buf * 128 + row];
              if (prow >= 0)
                *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(s_col_ptr[buf * 128 + row]) + col0 + ch * 8) =
                    *reinterpret_cast<const uint4*>(stage_g + row * 144 + ch * 16);
            }
          }
          if (!group_meets()) {
            ok = false;
            break;
          }
        }
        if (!ok) break;
        if (orow >= 0 && t.n0 == 0 && grp == 0) mark_pair_valid(a, orow);
      } else if (orow >= 0) {
        const float scale = w_on_input ? 1.0f : gam;
        float* out = reinterpret_cast<float*>(s_col_ptr[buf * 128 + lrow]) + t.n0 + 128 * grp;
        if (t.n0 + 128 * grp < a.N) {
#pragma unroll
          for (int q = 0; q < 16; ++q) {
            asm volatile("red.global.v4.f32.add [%0], {%1, %2, %3, %4};" ::"l"(out + 4 * q), "f"(accA[4 * q] * scale),
                         "f"(accA[4 * q + 1] * scale), "f"(accA[4 * q + 2] * scale), "f"(accA[4 * q + 3] * scale)
                         : "memory");
            asm volatile("red.global.v4.f32.add [%0], {%1, %2, %3, %4};" ::"l"(out + 64 + 4 * q),
                         "f"(accB[4 * q] * scale), "f"(accB[4 * q + 1] * scale), "f"(accB[4 * q + 2] * scale),
                         "f"(accB[4 * q + 3] * scale)
                         : "memory");
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_sempty[buf]));
      t_tail += static_cast<unsigned long long>(clock64() - tail_t0);
    }
    if (threadIdx.x == 2 * 32) {
      STALL_ADD8(5, w_pfull);
      STALL_ADD8(6, w_sfull);
      STALL_ADD8(7, t_tail);
      STALL_ADD8(11, static_cast<unsigned long long>(clock64() - role_t0));
    }
  }

  // ---- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 512u);
  }
  if (threadIdx.x == 0 && *abort_flag != 0) atomicCAS(a.status, 0, *abort_flag);
}

size_t fp8_tokm_ctrl_bytes(const GemmArgs& a) {
  const size_t kbs = static_cast<size_t>(a.kblocks);
  return 2 * kbs * 128 * 4 + 2 * 2 * kbs * 4 + ((a.mode == 1 && a.out_pairs != nullptr) ? kPairStageBytes : 0) + 512 +
         2 * 128 * 8 + 2 * 2 * 128 * 4 + 2 * 128 * 8 + static_cast<size_t>(a.E + 1) * 4 + 64;
}

template <int MODE>
int launch_fp8_tokm(const CUtensorMap& tm_w, const CUtensorMap& tm_x, const GemmArgs& a, int num_sms,
                    cudaStream_t stream) {
  const size_t smem = 1024 + static_cast<size_t>(a.stages) * (3 * kTileBytes) + fp8_tokm_ctrl_bytes(a);
  if (smem > kSmemLimit) return B200MOE_ERR_TOO_LARGE;
  if (cudaFuncSetAttribute(moe_gemm_fp8_tokm_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(smem)) != cudaSuccess)
    return B200MOE_ERR_CUDA;
  note_launch(MODE == 0 ? "moe_gemm_fp8_tokm_kernel<gate/up>" : "moe_gemm_fp8_tokm_kernel<down>");
  cudaError_t err = launch_kernel(moe_gemm_fp8_tokm_kernel<MODE>, dim3(num_sms), dim3(kThreadsFp8TokM), smem, stream,
                                  a.pdl != 0, tm_w, tm_x, a);
  return err == cudaSuccess ? B200MOE_OK : B200MOE_ERR_CUDA;
}

size_t fp8_stage_bytes(const GemmArgs& a) {
  return 2 * static_cast<size_t>(kTileBytes) + static_cast<size_t>(a.BT) * kStageKBytes;
}
size_t fp8_ctrl_bytes(const GemmArgs& a) {
  return 2 * static_cast<size_t>(kMaxKB) * a.BT * 4 + 2 * 2 * kMaxKB * 4 + 512 /*barriers*/ + 2 * 128 * 8 +
         2 * 2 * 4 * 64 * 4 + 2 * 128 * 8 + static_cast<size_t>(a.E + 1) * 4 + 64;
}

template <int MODE, int BT, int NG>
int launch_fp8(const CUtensorMap& tm_w, const CUtensorMap& tm_x, const GemmArgs& a, int num_sms,
               cudaStream_t stream) {
  const size_t smem = 1024 + static_cast<size_t>(a.stages) * fp8_stage_bytes(a) + fp8_ctrl_bytes(a);
  if (smem > kSmemLimit) return B200MOE_ERR_TOO_LARGE;
  if (cudaFuncSetAttribute(moe_gemm_fp8_kernel<MODE, BT, NG>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(smem)) != cudaSuccess)
    return B200MOE_ERR_CUDA;
  note_launch(MODE == 0 ? "moe_gemm_fp8_kernel<gate/up>" : "moe_gemm_fp8_kernel<down>");
  cudaError_t err = launch_kernel(moe_gemm_fp8_kernel<MODE, BT, NG>, dim3(num_sms), dim3(fp8_threads(NG)), smem,
                                  stream, a.pdl != 0, tm_w, tm_x, a);
  return err == cudaSuccess ? B200MOE_OK : B200MOE_ERR_CUDA;
}

}  // namespace

#ifdef B200MOE_STALL_STATS
extern "C" int b200moe_debug_stalls_fp8(unsigned long long* out16, int reset) {
  if (cudaMemcpyFromSymbol(out16, g_stall_fp8, sizeof(unsigned long long) * 16) != cudaSuccess) return -1;
  if (reset) {
    unsigned long long z[16] = {0};
    cudaMemcpyToSymbol(g_stall_fp8, z, sizeof(z));
  }
  return 0;
}
#endif

void gemm_plan_fp8(GemmArgs* a) {
  if (a->BT != 128) a->orient = 0;
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
  if (a->orient == 1) {   // tokens on M, 128-token blocks
    a->tmem_cols = 512;
    st = static_cast<int>((kSmemLimit - 1024 - fp8_tokm_ctrl_bytes(*a)) / (3 * kTileBytes));
  }
  if (st > 10) st = 10;
  if (st < 2) st = 2;
  a->stages = st;
  if (a->max_split <= 0) a->max_split = 16;
}

int launch_gemm_fp8(const CUtensorMap& tm_w, const CUtensorMap& tm_x, const GemmArgs& a, int num_sms,
                    cudaStream_t stream) {
  if (a.wmode != B200MOE_W_FP8_BLOCK) return B200MOE_ERR_BAD_ARG;
  if (a.K % 128 != 0 || a.N % 128 != 0 || a.K / 128 > kMaxKB) return B200MOE_ERR_UNSUPPORTED;
  if (a.orient == 1 && a.BT == 128)
    return a.mode == 0 ? launch_fp8_tokm<0>(tm_w, tm_x, a, num_sms, stream)
                       : launch_fp8_tokm<1>(tm_w, tm_x, a, num_sms, stream);
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
