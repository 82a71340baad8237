// Grouped expert GEMMs for int4 (AWQ, group 128, zero points) weights and fp16 activations,
// decode-sized token blocks (16 / 32).
//
// Weight-only int4 at decode is a dequantisation problem: the packed weights arrive from HBM
// four times faster than fp16 ones, so the CUDA-core work per weight has to shrink with them.
// Here the dequant warps only turn each nibble into the exact small integer (q - zero) as
// fp16 (two instructions per pair) and write it into the swizzled operand tile; the MMA
// (tcgen05.mma.kind::f16, fp32 accumulate) then sums exact products over one quantisation
// group of 128 k (two pipeline stages) into a partial accumulator in tensor memory, and the
// promotion warps multiply that partial by the group's scale -- one scalar per thread, since
// a thread owns one weight row -- while adding it to accumulators in registers.  The result is
// also closer to the real-valued product than rounding (q - z) * s to fp16 per weight.
//
// Tiles are two 128-row weight blocks sharing the token block (gate | up rows for the first
// GEMM, rows n0.. | n0+128.. for the second), as in the FP8 kernels.
//
// The dequantised operand never touches shared memory: staging fp16 tiles there costs four
// times the bytes that arrive from HBM in shared-memory writes plus the same again in MMA
// operand reads, and that bandwidth (128 B/clk) caps the kernel well below the HBM rate.
// Instead each dequant thread owns one weight row = one TMEM lane and writes its 64 k-values
// of a stage into tensor memory with tcgen05.st; the MMA takes its A operand from there
// (tcgen05.mma with A in TMEM) and only the small token block as a shared-memory descriptor.
// Shared memory then holds just a deep ring of small TMA stages (8 KiB packed + token block).
//
// Warps: 0 TMA producer, 1 MMA issuer, 2-5 promotion + tail, 6 per-tile table loader,
// 7-14 dequantisation.
#include "gemm_sched.cuh"

namespace b200moe {

namespace {

#ifdef B200MOE_STALL_STATS
__device__ unsigned long long g_stall_w4[16];
#define STALL_ADD(slot, v) atomicAdd(&g_stall_w4[slot], v)
#else
#define STALL_ADD(slot, v) ((void)0)
#endif

constexpr int kDqWarps = 8;
constexpr int kOperandStages = 4;   // A-operand stages in tensor memory, 64 columns each
constexpr int kThreadsW4P = 7 * 32 + 32 * kDqWarps;  // 480

// 32 packed uint4 (16 bytes) -> 16 words of two fp16 values (q - zero) each, k ascending.
__device__ __forceinline__ void dequant_w4x32_centered(const uint4 packed, const __half2 zero1024, uint32_t* out) {
  const uint32_t w[4] = {packed.x, packed.y, packed.z, packed.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t t = ((w[j] >> (4 * i)) & 0x000F000Fu) | 0x64006400u;  // fp16 pair (1024 + q, 1024 + q')
      __half2 h = __hsub2(*reinterpret_cast<__half2*>(&t), zero1024);
      out[4 * j + i] = *reinterpret_cast<uint32_t*>(&h);
    }
  }
}

template <int MODE, int BT>
__global__ void __launch_bounds__(kThreadsW4P, 1)
moe_gemm_w4_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                   const GemmArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  constexpr int X_BYTES = BT * kStageKBytes;        // token block: BT rows x 64 k fp16
  constexpr int PK_BYTES = 2 * kTileRows * 32;      // packed rows: 256 x 32 bytes
  constexpr int STAGE_BYTES = X_BYTES + PK_BYTES;   // one stage of the TMA ring: [token block | packed rows]
  constexpr int PCOLS = 2 * BT;
  constexpr int NO = kOperandStages;
  const int stages = a.stages;                      // depth of the TMA ring

  uint8_t* pk_base = smem;                                           // TMA ring
  constexpr uint32_t A_COL0 = 4 * BT;                                // TMEM: [0, 4*BT) partial sums, then A stages
  uint8_t* ctrl_base = pk_base + static_cast<size_t>(stages) * STAGE_BYTES;
  uint64_t* bar_full = reinterpret_cast<uint64_t*>(ctrl_base);
  uint64_t* bar_empty = bar_full + stages;
  uint64_t* bar_dq = bar_empty + stages;       // [NO] operand tile written
  uint64_t* bar_oempty = bar_dq + NO;          // [NO] operand tile consumed
  uint64_t* bar_pfull = bar_oempty + NO;
  uint64_t* bar_pempty = bar_pfull + 2;
  uint64_t* bar_sfull = bar_pempty + 2;
  uint64_t* bar_sempty = bar_sfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_sempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* s_col_row = reinterpret_cast<int*>(tmem_slot + 4);           // [2][32]
  float* s_col_gam = reinterpret_cast<float*>(s_col_row + 2 * 32);  // [2][32]
  int* s_blk_off = reinterpret_cast<int*>(s_col_gam + 2 * 32);      // [E+1]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    for (int s = 0; s < NO; ++s) {
      mbar_init(smem_u32(&bar_dq[s]), kDqWarps);
      mbar_init(smem_u32(&bar_oempty[s]), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&bar_pfull[s]), 1);
      mbar_init(smem_u32(&bar_pempty[s]), 4);
      mbar_init(smem_u32(&bar_sfull[s]), 1);
      mbar_init(smem_u32(&bar_sempty[s]), 4);
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
  griddep_wait();
  griddep_launch_dependents();
  for (int e = threadIdx.x; e <= a.E; e += blockDim.x) s_blk_off[e] = a.blk_off[e];
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // the scheduler's reduction unit is one quantisation group (128 k = two pipeline stages)
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
      for (int ks = 2 * t.kb0; ks < 2 * t.kb1; ++ks) {  // ks: 64-wide k step
        if (!mbar_wait_t(smem_u32(&bar_empty[stage]), phase ^ 1, abort_flag, DEV_TIMEOUT_PRODUCER, w_empty)) {
          ok = false;
          break;
        }
        const uint32_t full = smem_u32(&bar_full[stage]);
        mbar_arrive_expect_tx(full, static_cast<uint32_t>(PK_BYTES + X_BYTES));
        const uint32_t sbase = smem_u32(pk_base + static_cast<size_t>(stage) * STAGE_BYTES);
        const uint32_t spk = sbase + X_BYTES;
        tma_load_3d(spk, &tm_w, full, ks * 32, t.n0, t.e);
        tma_load_3d(spk + kTileRows * 32, &tm_w, full, ks * 32, second_off + t.n0, t.e);
        tma_load_2d(sbase, &tm_x, full, ks * 64, t.row0);
        ++issued;
        if (++stage == stages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
    STALL_ADD(0, w_empty);
    STALL_ADD(8, static_cast<unsigned long long>(clock64() - role_t0));
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
    const uint32_t idesc = make_idesc(0u /* fp16 */, kTileRows, static_cast<uint32_t>(BT));
    int stage = 0, ost = 0;
    uint32_t phase = 0, ophase = 0, j = 0;  // j counts groups over the whole launch
    bool ok = true;
    unsigned long long w_pempty = 0, w_dq = 0;
    const long long role_t0 = clock64();
    for (int tile = blockIdx.x; ok && tile < c.total; tile += c.grid_eff) {
      const TileCoord t = decode_tile(tile, c, s_blk_off, a.E, BT, a.num_nt, a.kblocks, kTileN);
      for (int kb = t.kb0; kb < t.kb1 && ok; ++kb, ++j) {
        const uint32_t pb = j & 1u;
        if (!mbar_wait_t(smem_u32(&bar_pempty[pb]), ((j >> 1) & 1u) ^ 1u, abort_flag, DEV_TIMEOUT_MMA, w_pempty)) {
          ok = false;
          break;
        }
        const uint32_t d0 = tmem_base + pb * PCOLS;
#pragma unroll 1
        for (int h = 0; h < 2; ++h) {
          // the operand tile is written only after its TMA stage has landed, so this wait
          // also covers the token block of that stage
          if (!mbar_wait_t(smem_u32(&bar_dq[ost]), ophase, abort_flag, DEV_TIMEOUT_MMA, w_dq)) {
            ok = false;
            break;
          }
          tc_fence_after();
          // A operand: 64 TMEM columns of this stage (32 per weight block, 8 per 16-wide k slice)
          const uint32_t a0 = tmem_base + A_COL0 + static_cast<uint32_t>(ost) * 64;
          const uint64_t dx = smem_desc_k_sw128(smem_u32(pk_base + static_cast<size_t>(stage) * STAGE_BYTES));
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint32_t accum = (h > 0 || k > 0) ? 1u : 0u;
            tc_mma_f16_ts(d0, a0 + 8 * k, dx + 2 * k, idesc, accum);
            tc_mma_f16_ts(d0 + BT, a0 + 32 + 8 * k, dx + 2 * k, idesc, accum);
          }
          tc_commit(smem_u32(&bar_empty[stage]));
          tc_commit(smem_u32(&bar_oempty[ost]));
          if (++stage == stages) {
            stage = 0;
            phase ^= 1;
          }
          if (++ost == NO) {
            ost = 0;
            ophase ^= 1;
          }
        }
        if (ok) tc_commit(smem_u32(&bar_pfull[pb]));
      }
    }
    STALL_ADD(1, w_pempty);
    STALL_ADD(2, w_dq);
    STALL_ADD(9, static_cast<unsigned long long>(clock64() - role_t0));
  } else if (active && warp == 6) {
    // =============================== per-tile table loader ======================
    int iter = 0;
    for (int tile = blockIdx.x; tile < c.total; tile += c.grid_eff, ++iter) {
      const TileCoord t = decode_tile(tile, c, s_blk_off, a.E, BT, a.num_nt, a.kblocks, kTileN);
      const int buf = iter & 1;
      if (!mbar_wait(smem_u32(&bar_sempty[buf]), ((iter >> 1) & 1) ^ 1, abort_flag, DEV_TIMEOUT_EPILOGUE)) break;
      if (lane < BT) {
        const int slot = a.sorted_ids[t.row0 + lane];
        const bool valid = slot >= 0 && slot < a.P;
        s_col_row[buf * 32 + lane] = valid ? (MODE == 1 ? slot / a.topk : slot) : -1;
        s_col_gam[buf * 32 + lane] = valid ? a.row_gamma[t.row0 + lane] : 0.f;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_sfull[buf]));
    }
  } else if (active && warp >= 7) {
    // =============================== int4 -> centred fp16 operand ===============
    // warp w may touch TMEM lanes 32 * (w % 4)..: warps 7-10 convert the first weight block,
    // warps 11-14 the second, each thread the row that is its own TMEM lane
    const int wblk = (warp - 7) >> 2;
    const int quad = warp & 3;
    const int row = wblk * kTileRows + quad * 32 + lane;  // packed row of the stage
    const uint32_t* sz = reinterpret_cast<const uint32_t*>(a.w_sz);
    const int groups = a.kblocks;
    int stage = 0, ost = 0;
    uint32_t phase = 0, ophase = 0;
    bool ok = true;
    unsigned long long w_full = 0, w_oempty = 0;
    const long long role_t0 = clock64();
    for (int tile = blockIdx.x; ok && tile < c.total; tile += c.grid_eff) {
      const TileCoord t = decode_tile(tile, c, s_blk_off, a.E, BT, a.num_nt, a.kblocks, kTileN);
      const int n = (row < kTileRows) ? t.n0 + row : second_off + t.n0 + (row - kTileRows);
      const bool n_ok = n < a.w_rows;
      const uint32_t* szrow = sz + static_cast<size_t>(t.e) * groups * a.w_rows + n;
      // zero points of this row, fetched three groups ahead of their use (a dependent global
      // load per group would otherwise sit on the dequantisation's critical path);
      // 0x6400 = fp16(1024 + 0) for rows past the expert, whose output is never stored
      auto load_sz = [&](int kb) -> uint32_t {
        return (n_ok && kb < t.kb1) ? __ldg(szrow + static_cast<size_t>(kb) * a.w_rows) : 0x64000000u;
      };
      uint32_t sz_a = load_sz(t.kb0), sz_b = load_sz(t.kb0 + 1), sz_c = load_sz(t.kb0 + 2);
      for (int kb = t.kb0; kb < t.kb1 && ok; ++kb) {
        const uint32_t szv = sz_a;
        sz_a = sz_b;
        sz_b = sz_c;
        sz_c = load_sz(kb + 3);
        const __half2 zp = __half2half2(__ushort_as_half(static_cast<unsigned short>(szv >> 16)));
#pragma unroll 1
        for (int h = 0; h < 2; ++h) {
          if (!mbar_wait_t(smem_u32(&bar_full[stage]), phase, abort_flag, DEV_TIMEOUT_MMA, w_full) ||
              !mbar_wait_t(smem_u32(&bar_oempty[ost]), ophase ^ 1, abort_flag, DEV_TIMEOUT_MMA, w_oempty)) {
            ok = false;
            break;
          }
          const uint4* pk = reinterpret_cast<const uint4*>(pk_base + static_cast<size_t>(stage) * STAGE_BYTES +
                                                           X_BYTES + row * 32);
          uint32_t o[32];
          dequant_w4x32_centered(pk[0], zp, o);
          dequant_w4x32_centered(pk[1], zp, o + 16);
          tc_fence_after();
          tmem_st32_wait(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + A_COL0 +
                             static_cast<uint32_t>(ost) * 64 + static_cast<uint32_t>(wblk) * 32, o);
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&bar_dq[ost]));
          if (++stage == stages) {
            stage = 0;
            phase ^= 1;
          }
          if (++ost == NO) {
            ost = 0;
            ophase ^= 1;
          }
        }
      }
    }
    if (threadIdx.x == 8 * 32) {
      STALL_ADD(3, w_full);
      STALL_ADD(4, w_oempty);
      STALL_ADD(10, static_cast<unsigned long long>(clock64() - role_t0));
    }
  } else if (active && warp >= 2 && warp < 6) {
    // =============================== promotion + tail ===========================
    unsigned long long w_pfull = 0, w_sfull = 0;
    const long long role_t0 = clock64();
    const int quad = warp & 3;
    const int lrow = quad * 32 + lane;
    const bool w_on_input = (a.flags & B200MOE_FLAG_WEIGHT_ON_INPUT) != 0;
    const bool mimic = (a.flags & B200MOE_FLAG_MIMIC_ROUNDING) != 0;
    const bool round_pair = mimic && c.split == 1;
    const uint32_t* sz = reinterpret_cast<const uint32_t*>(a.w_sz);
    const int groups = a.kblocks;
    uint32_t j = 0;
    int iter = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < c.total; tile += c.grid_eff, ++iter) {
      const TileCoord t = decode_tile(tile, c, s_blk_off, a.E, BT, a.num_nt, a.kblocks, kTileN);
      const int buf = iter & 1;
      const int* col_row = s_col_row + buf * 32;
      const float* col_gam = s_col_gam + buf * 32;
      // scales of this thread's two weight rows, one per group
      const int n = t.n0 + lrow;
      const int n2 = second_off + t.n0 + lrow;
      const bool ok0 = n < a.w_rows, ok1 = n2 < a.w_rows;
      const uint32_t* sz0 = sz + static_cast<size_t>(t.e) * groups * a.w_rows + n;
      const uint32_t* sz1 = sz + static_cast<size_t>(t.e) * groups * a.w_rows + n2;
      auto scale_of = [](uint32_t v) { return __half2float(__ushort_as_half(static_cast<unsigned short>(v & 0xFFFFu))); };
      float s0 = ok0 ? scale_of(__ldg(sz0 + static_cast<size_t>(t.kb0) * a.w_rows)) : 0.f;
      float s1 = ok1 ? scale_of(__ldg(sz1 + static_cast<size_t>(t.kb0) * a.w_rows)) : 0.f;
      float s0n = (ok0 && t.kb0 + 1 < t.kb1) ? scale_of(__ldg(sz0 + static_cast<size_t>(t.kb0 + 1) * a.w_rows)) : 0.f;
      float s1n = (ok1 && t.kb0 + 1 < t.kb1) ? scale_of(__ldg(sz1 + static_cast<size_t>(t.kb0 + 1) * a.w_rows)) : 0.f;
      if (!mbar_wait_t(smem_u32(&bar_sfull[buf]), (iter >> 1) & 1, abort_flag, DEV_TIMEOUT_EPILOGUE, w_sfull)) break;

      float acc0[BT], acc1[BT];
#pragma unroll
      for (int i = 0; i < BT; ++i) {
        acc0[i] = 0.f;
        acc1[i] = 0.f;
      }
      for (int kb = t.kb0; kb < t.kb1; ++kb, ++j) {
        // fetch the scales two groups ahead, before waiting for this group's partial sums
        uint32_t r0 = 0, r1 = 0;
        if (kb + 2 < t.kb1) {
          if (ok0) r0 = __ldg(sz0 + static_cast<size_t>(kb + 2) * a.w_rows);
          if (ok1) r1 = __ldg(sz1 + static_cast<size_t>(kb + 2) * a.w_rows);
        }
        const uint32_t pb = j & 1u;
        if (!mbar_wait_t(smem_u32(&bar_pfull[pb]), (j >> 1) & 1u, abort_flag, DEV_TIMEOUT_EPILOGUE, w_pfull)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + pb * PCOLS;
        if constexpr (BT == 32) {
          float g[32], u[32];
          tmem_ld32x2_wait(taddr, taddr + BT, g, u);
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            acc0[i] = fmaf(g[i], s0, acc0[i]);
            acc1[i] = fmaf(u[i], s1, acc1[i]);
          }
        } else {
          float g[16], u[16];
          tmem_ld16x2_wait(taddr, taddr + BT, g, u);
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            acc0[i] = fmaf(g[i], s0, acc0[i]);
            acc1[i] = fmaf(u[i], s1, acc1[i]);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_pempty[pb]));
        s0 = s0n;
        s1 = s1n;
        s0n = scale_of(r0);   // fp16 bits 0 -> 0.0f when out of range
        s1n = scale_of(r1);
      }
      if (!ok) break;

      if (MODE == 0) {
        __half* out = reinterpret_cast<__half*>(a.out) + static_cast<size_t>(t.row0) * a.ld_out + n;
        const bool n_ok = n < a.N;
#pragma unroll
        for (int i = 0; i < BT; ++i) {
          const float av = act_mul<__half>(acc0[i], acc1[i], w_on_input, col_gam[i], mimic, act_params(a));
          if (n_ok) out[static_cast<size_t>(i) * a.ld_out] = __float2half_rn(av);
        }
      } else {
        float* out = reinterpret_cast<float*>(a.out) + n;
        const bool first = n < a.N, second = n + kTileRows < a.N;
#pragma unroll
        for (int i = 0; i < BT; ++i) {
          const int orow = col_row[i];
          if (orow >= 0) {
            const float gam = w_on_input ? 1.0f : col_gam[i];
            float y0 = acc0[i] * gam, y1 = acc1[i] * gam;
            if (round_pair) {
              y0 = __half2float(__float2half_rn(y0));
              y1 = __half2float(__float2half_rn(y1));
            }
            if (first) atomicAdd(out + static_cast<size_t>(orow) * a.ld_out, y0);
            if (second) atomicAdd(out + static_cast<size_t>(orow) * a.ld_out + kTileRows, y1);
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_sempty[buf]));
    }
    if (threadIdx.x == 2 * 32) {
      STALL_ADD(5, w_pfull);
      STALL_ADD(6, w_sfull);
      STALL_ADD(11, static_cast<unsigned long long>(clock64() - role_t0));
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

size_t w4_stage_bytes(const GemmArgs& a) {   // one stage of the TMA ring
  return static_cast<size_t>(a.BT) * kStageKBytes + 2 * kTileRows * 32;
}
size_t w4_ctrl_bytes(const GemmArgs& a) {    // barriers + tables
  return 1024 + 2 * 32 * 8 + static_cast<size_t>(a.E + 1) * 4 + 64;
}

template <int MODE, int BT>
int launch_w4(const CUtensorMap& tm_w, const CUtensorMap& tm_x, const GemmArgs& a, int num_sms, cudaStream_t stream) {
  const size_t smem = 1024 + static_cast<size_t>(a.stages) * w4_stage_bytes(a) + w4_ctrl_bytes(a);
  if (smem > kSmemLimit) return B200MOE_ERR_TOO_LARGE;
  if (cudaFuncSetAttribute(moe_gemm_w4_kernel<MODE, BT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(smem)) != cudaSuccess)
    return B200MOE_ERR_CUDA;
  cudaError_t err = launch_kernel(moe_gemm_w4_kernel<MODE, BT>, dim3(num_sms), dim3(kThreadsW4P), smem, stream,
                                  a.pdl != 0, tm_w, tm_x, a);
  return err == cudaSuccess ? B200MOE_OK : B200MOE_ERR_CUDA;
}

}  // namespace

#ifdef B200MOE_STALL_STATS
extern "C" int b200moe_debug_stalls_w4(unsigned long long* out16, int reset) {
  if (cudaMemcpyFromSymbol(out16, g_stall_w4, sizeof(unsigned long long) * 16) != cudaSuccess) return -1;
  if (reset) {
    unsigned long long z[16] = {0};
    cudaMemcpyToSymbol(g_stall_w4, z, sizeof(z));
  }
  return 0;
}
#endif

void gemm_plan_w4(GemmArgs* a) {
  a->orient = 0;
  const int tile_n = (a->mode == 0) ? kTileRows : 2 * kTileRows;
  a->num_nt = (a->N + tile_n - 1) / tile_n;
  a->kblocks = (a->K + 127) / 128;  // reduction unit = one quantisation group
  int tc = 32;
  while (tc < 4 * a->BT + 64 * kOperandStages) tc <<= 1;   // partial sums + A-operand stages
  a->tmem_cols = tc;
  a->acc_stages = 2;
  int st = static_cast<int>((kSmemLimit - 1024 - w4_ctrl_bytes(*a)) / w4_stage_bytes(*a));
  if (st > 16) st = 16;
  if (st < 2) st = 2;
  a->stages = st;
  if (a->max_split <= 0) a->max_split = 16;
}

int launch_gemm_w4(const CUtensorMap& tm_w, const CUtensorMap& tm_x, const GemmArgs& a, int num_sms,
                   cudaStream_t stream) {
  if (a.wmode != B200MOE_W_INT4_AWQ || a.dtype != B200MOE_DTYPE_FP16 || a.w_sz == nullptr) return B200MOE_ERR_BAD_ARG;
  if (a.K % 128 != 0) return B200MOE_ERR_UNSUPPORTED;
  if (a.BT == 16)
    return a.mode == 0 ? launch_w4<0, 16>(tm_w, tm_x, a, num_sms, stream) : launch_w4<1, 16>(tm_w, tm_x, a, num_sms, stream);
  if (a.BT == 32)
    return a.mode == 0 ? launch_w4<0, 32>(tm_w, tm_x, a, num_sms, stream) : launch_w4<1, 32>(tm_w, tm_x, a, num_sms, stream);
  return B200MOE_ERR_BAD_ARG;
}

}  // namespace b200moe
