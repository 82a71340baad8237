// Grouped expert GEMMs for int4 (AWQ, group 128, zero points) weights and fp16 activations,
// decode-sized token blocks (16 / 32), on the integer tensor-core path.
//
// Weight-only int4 at decode is bound by how many weights one tcgen05.mma consumes: the
// instruction walks its 128 operand rows at one row per clock whatever the width of the other
// operand, so with fp16 operands (16 k per instruction) a CTA takes in 16 weights per clock,
// a quarter of what the packed weights need to keep HBM busy.  8-bit operands double the k per
// instruction, and integer ones make the conversion almost free:
//
//   weights      the raw nibbles q (0..15) as unsigned bytes: three logic instructions per eight
//                weights, written straight into tensor memory (tcgen05.st), never into shared
//                memory.  The zero point is not subtracted here.
//   activations  per (token, 128-k group) a power-of-two scale f and the exact integers
//                v = rint(x / f), |v| < 2^19, split into three signed bytes
//                v = p0 + 256 p1 + 65536 p2.  The three byte planes of a token block are three
//                sets of columns of ONE MMA (N = 3 * BT), which costs no extra tensor time.
//   MMA          kind::i8, int32 accumulate, A from tensor memory: per group the exact sums
//                S_p = sum_k q_k p_{p,k}.
//   promotion    exact integer S = S_0 + 256 S_1 + 65536 S_2 - z * X with X = sum_k v_k (from
//                the activation tables), then acc += (s * f) * float(S): the group scale s and
//                zero z are one scalar per thread (a thread owns one weight row).
//
// Up to the rounding of x / f to 20 bits this is the real-valued product of the dequantised
// weights with the fp16 activations, accumulated in fp32 once per group: closer to it than
// rounding (q - z) * s to fp16 per weight.
//
// A tile is two 128-row weight blocks sharing the token block (gate | up rows for the first
// GEMM, rows n0.. | n0+128.. for the second).  The first GEMM's tail applies the activation,
// rounds to fp16 and re-expresses the block in the same three-plane form for the second GEMM
// (its 128 output columns are exactly one group of the second GEMM's reduction).
//
// Byte order inside each aligned run of eight k: the packed word keeps element 2i in nibble i
// and element 2i+1 in nibble 4+i, so `w & 0x0F0F0F0F` and `(w >> 4) & 0x0F0F0F0F` are the
// elements (0, 4, 1, 5) and (2, 6, 3, 7).  The activation planes are stored in that same
// order; a dot product does not care as long as both sides agree.
//
// Warps: 0 TMA producer, 1 MMA issuer, 6 per-tile table loader, 7-10 nibble -> byte conversion,
// 2-5 and 11-14 promotion + tail: a thread owns one weight row (its TMEM lane) and half of the
// token block, so that two promotion warps share each scheduler.  The group's scale / zero words
// reach the promotion through a shared-memory ring that the producer fills by bulk copy: a
// global load per group, however far ahead it is issued in the source, ends up waited for in
// the same iteration once its register is rotated, and that wait set the pace of every earlier
// version of this kernel.
#include "gemm_sched.cuh"

namespace b200moe {

namespace {

#ifdef B200MOE_STALL_STATS
__device__ unsigned long long g_stall_w4[16];
#define STALL_ADD(slot, v) atomicAdd(&g_stall_w4[slot], v)
#else
#define STALL_ADD(slot, v) ((void)0)
#endif

constexpr int kDqWarps = 4;
constexpr int kPromoWarps = 8;
constexpr int kThreadsW4P = 3 * 32 + 32 * kDqWarps + 32 * kPromoWarps;  // 480
constexpr int kPackedRowBytes = 64;                  // 128 k of one weight row
constexpr int kMaxGroupsW4 = 128;                    // reduction groups whose tables fit in shared memory
constexpr int kSzSlots = 16;                         // ring of per-group scale / zero words (1 KiB each)

// position inside an aligned run of eight k at which element e is stored
__device__ __forceinline__ int plane_pos(int e) { return ((e & 3) << 1) | ((e >> 2) & 1); }

template <int MODE, int BT>
__global__ void __launch_bounds__(kThreadsW4P, 1)
moe_gemm_w4_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                   const GemmArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  constexpr int NB = 3 * BT;                                   // MMA N: three byte planes of the token block
  constexpr int X_BYTES = NB * kStageKBytes;                   // [3 planes][BT rows][128 k] int8
  constexpr int PK_BYTES = 2 * kTileRows * kPackedRowBytes;    // packed rows: 256 x 64 bytes
  constexpr int STAGE_BYTES = X_BYTES + PK_BYTES;              // one stage = one quantisation group
  constexpr int PCOLS = 2 * NB;                                // int32 partial sums of both weight blocks
  constexpr int NO = (BT == 16) ? 4 : 2;                       // A-operand stages in tensor memory
  constexpr uint32_t A_COL0 = 2 * PCOLS;                       // TMEM: two partial buffers, then the A stages
  const int stages = a.stages;
  const int nkb_max = a.kblocks;

  uint8_t* ring = smem;
  uint8_t* ctrl_base = ring + static_cast<size_t>(stages) * STAGE_BYTES;
  float* s_xf = reinterpret_cast<float*>(ctrl_base);                       // [2][kblocks][BT] activation scales
  int* s_xsum = reinterpret_cast<int*>(s_xf + 2 * nkb_max * BT);           // [2][kblocks][BT] activation sums
  uint32_t* s_sz = reinterpret_cast<uint32_t*>(s_xsum + 2 * nkb_max * BT);  // [kSzSlots][2 blocks][128 rows]
  uint64_t* bar_full = reinterpret_cast<uint64_t*>(s_sz + kSzSlots * 256);
  uint64_t* bar_empty = bar_full + stages;
  uint64_t* bar_dq = bar_empty + stages;       // [NO] operand tile written
  uint64_t* bar_oempty = bar_dq + NO;          // [NO] operand tile consumed
  uint64_t* bar_pfull = bar_oempty + NO;
  uint64_t* bar_pempty = bar_pfull + 2;
  uint64_t* bar_sfull = bar_pempty + 2;
  uint64_t* bar_sempty = bar_sfull + 2;
  uint64_t* bar_tail = bar_sempty + 2;         // [2][2] tail: maxima complete / sums complete
  uint64_t* bar_zfull = bar_tail + 4;          // [kSzSlots] scale words landed
  uint64_t* bar_zempty = bar_zfull + kSzSlots; // [kSzSlots] scale words read by every promotion warp
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_zempty + kSzSlots);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* s_nvalid = reinterpret_cast<int*>(tmem_slot + 2);            // [2] columns up to the last valid token
  int* s_col_row = reinterpret_cast<int*>(tmem_slot + 4);           // [2][32]
  float* s_col_gam = reinterpret_cast<float*>(s_col_row + 2 * 32);  // [2][32]
  unsigned int* s_amax = reinterpret_cast<unsigned int*>(s_col_gam + 2 * 32);   // [2][32] tail: group maxima
  int* s_osum = reinterpret_cast<int*>(s_amax + 2 * 32);            // [2][32] tail: sums of the new integers
  int* s_blk_off = s_osum + 2 * 32;                                 // [E+1]

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
      mbar_init(smem_u32(&bar_pempty[s]), kPromoWarps);
      mbar_init(smem_u32(&bar_sfull[s]), 1);
      mbar_init(smem_u32(&bar_sempty[s]), kPromoWarps);
      mbar_init(smem_u32(&bar_tail[2 * s]), kPromoWarps);
      mbar_init(smem_u32(&bar_tail[2 * s + 1]), kPromoWarps);
    }
    for (int s = 0; s < kSzSlots; ++s) {
      mbar_init(smem_u32(&bar_zfull[s]), 1);
      mbar_init(smem_u32(&bar_zempty[s]), kPromoWarps);
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

  // the scheduler's reduction unit is one quantisation group (128 k = one pipeline stage)
  const Ctrl c = make_ctrl(a, MODE == 1);
  const bool active = static_cast<int>(blockIdx.x) < c.grid_eff;
  constexpr int kTileN = (MODE == 0) ? kTileRows : 2 * kTileRows;
  const int second_off = (MODE == 0) ? a.up_row_off : kTileRows;

  if (active && warp == 0 && lane == 0) {
    // =============================== TMA producer ===============================
    int stage = 0;
    uint32_t phase = 0;
    long long issued = 0;
    uint32_t jz = 0;   // groups issued over the whole launch (index into the scale ring)
    bool ok = true;
    unsigned long long w_empty = 0;
    const long long role_t0 = clock64();
    const uint32_t* szg = reinterpret_cast<const uint32_t*>(a.w_sz);
    for (int tile = blockIdx.x; ok && tile < c.total; tile += c.grid_eff) {
      const TileCoord t = decode_tile(tile, c, s_blk_off, a.E, BT, a.num_nt, a.kblocks, kTileN);
      const int xrow0 = (t.row0 / BT) * NB;   // the block's three planes are 3 * BT consecutive rows
      // whole 128-row blocks only (weight rows per expert are a multiple of 128); the second
      // block of the last tile may lie past the expert
      const bool second_in = second_off + t.n0 < a.w_rows;
      for (int kb = t.kb0; kb < t.kb1; ++kb, ++jz) {
        const uint32_t zs = jz % kSzSlots;
        if (!mbar_wait_t(smem_u32(&bar_empty[stage]), phase ^ 1, abort_flag, DEV_TIMEOUT_PRODUCER, w_empty) ||
            !mbar_wait_t(smem_u32(&bar_zempty[zs]), ((jz / kSzSlots) & 1u) ^ 1u, abort_flag, DEV_TIMEOUT_PRODUCER,
                         w_empty)) {
          ok = false;
          break;
        }
        // scale / zero words of the group's two row blocks: the promotion warps read them from
        // shared memory, so no global load sits on their critical path
        {
          const uint32_t zfull = smem_u32(&bar_zfull[zs]);
          mbar_arrive_expect_tx(zfull, second_in ? 1024u : 512u);
          const uint32_t* src = szg + (static_cast<size_t>(t.e) * a.kblocks + kb) * a.w_rows;
          bulk_copy_g2s(smem_u32(s_sz + zs * 256), src + t.n0, 512, zfull);
          if (second_in) bulk_copy_g2s(smem_u32(s_sz + zs * 256 + 128), src + second_off + t.n0, 512, zfull);
        }
        const uint32_t full = smem_u32(&bar_full[stage]);
        mbar_arrive_expect_tx(full, static_cast<uint32_t>(STAGE_BYTES));
        const uint32_t sbase = smem_u32(ring + static_cast<size_t>(stage) * STAGE_BYTES);
        const uint32_t spk = sbase + X_BYTES;
        tma_load_3d(spk, &tm_w, full, kb * kPackedRowBytes, t.n0, t.e);
        tma_load_3d(spk + kTileRows * kPackedRowBytes, &tm_w, full, kb * kPackedRowBytes, second_off + t.n0, t.e);
        tma_load_2d(sbase, &tm_x, full, kb * 128, xrow0);
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
    const uint32_t idesc = make_idesc_i8(false, true, kTileRows, static_cast<uint32_t>(NB));
    int stage = 0, ost = 0;
    uint32_t phase = 0, ophase = 0, j = 0;  // j counts groups over the whole launch
    bool ok = true;
    unsigned long long w_pempty = 0, w_dq = 0;
    const long long role_t0 = clock64();
    for (int tile = blockIdx.x; ok && tile < c.total; tile += c.grid_eff) {
      const TileCoord t = decode_tile(tile, c, s_blk_off, a.E, BT, a.num_nt, a.kblocks, kTileN);
      for (int kb = t.kb0; kb < t.kb1; ++kb, ++j) {
        const uint32_t pb = j & 1u;
        // the operand tile is written only after its TMA stage has landed, so the second wait
        // also covers the token block of that stage
        if (!mbar_wait_t(smem_u32(&bar_pempty[pb]), ((j >> 1) & 1u) ^ 1u, abort_flag, DEV_TIMEOUT_MMA, w_pempty) ||
            !mbar_wait_t(smem_u32(&bar_dq[ost]), ophase, abort_flag, DEV_TIMEOUT_MMA, w_dq)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d0 = tmem_base + pb * PCOLS;
        // A operand: 64 TMEM columns of this stage (32 per weight block, 8 per 32-wide k slice)
        const uint32_t a0 = tmem_base + A_COL0 + static_cast<uint32_t>(ost) * 64;
        const uint64_t dx = smem_desc_k_sw128(smem_u32(ring + static_cast<size_t>(stage) * STAGE_BYTES));
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          tc_mma_i8_ts(d0, a0 + 8 * k, dx + 2 * k, idesc, k > 0 ? 1u : 0u);
          tc_mma_i8_ts(d0 + NB, a0 + 32 + 8 * k, dx + 2 * k, idesc, k > 0 ? 1u : 0u);
        }
        // one commit per group: the first promotion warp passes the news on to the producer
        // (ring stage free) and to the conversion warps (operand stage free)
        tc_commit(smem_u32(&bar_pfull[pb]));
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
      s_amax[buf * 32 + lane] = 0u;
      s_osum[buf * 32 + lane] = 0;
      {
        // columns past the last valid token carry zeros: the promotion warps skip them
        int slot_ok = 0;
        if (lane < BT) {
          const int slot = a.sorted_ids[t.row0 + lane];
          slot_ok = slot >= 0 && slot < a.P;
        }
        const unsigned int m = __ballot_sync(0xffffffffu, slot_ok);
        if (lane == 0) s_nvalid[buf] = 32 - __clz(m);
      }
      __syncwarp();
      const int nkb = t.kb1 - t.kb0;
      const uint32_t sfull = smem_u32(&bar_sfull[buf]);
      if (lane == 0) mbar_arrive_expect_tx(sfull, static_cast<uint32_t>(nkb * BT * 8));
      __syncwarp();
      for (int i = lane; i < nkb; i += 32) {
        const size_t src = static_cast<size_t>(t.kb0 + i) * a.ld_xscale + t.row0;
        bulk_copy_g2s(smem_u32(s_xf + (buf * nkb_max + i) * BT), a.x_scale + src, BT * 4, sfull);
        bulk_copy_g2s(smem_u32(s_xsum + (buf * nkb_max + i) * BT), a.x_sum + src, BT * 4, sfull);
      }
    }
  } else if (active && warp >= 7 && warp < 7 + kDqWarps) {
    // =============================== nibbles -> unsigned bytes in tensor memory ==
    // warp w may touch TMEM lanes 32 * (w % 4)..; each thread converts the two rows (one per
    // weight block) that live in its own lane
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    // the packed tile is staged with the 64-byte swizzle: 16-byte chunk c of row r sits at chunk
    // c ^ ((r >> 1) & 3), which spreads the 64-byte row stride over all banks
    const int sw = (row >> 1) & 3;
    int stage = 0, ost = 0;
    uint32_t phase = 0, ophase = 0;
    bool ok = true;
    unsigned long long w_full = 0, w_oempty = 0;
    const long long role_t0 = clock64();
    for (int tile = blockIdx.x; ok && tile < c.total; tile += c.grid_eff) {
      const TileCoord t = decode_tile(tile, c, s_blk_off, a.E, BT, a.num_nt, a.kblocks, kTileN);
      for (int kb = t.kb0; kb < t.kb1; ++kb) {
        if (!mbar_wait_t(smem_u32(&bar_full[stage]), phase, abort_flag, DEV_TIMEOUT_MMA, w_full) ||
            !mbar_wait_t(smem_u32(&bar_oempty[ost]), ophase ^ 1, abort_flag, DEV_TIMEOUT_MMA, w_oempty)) {
          ok = false;
          break;
        }
        const uint8_t* pk = ring + static_cast<size_t>(stage) * STAGE_BYTES + X_BYTES;
        tc_fence_after();
#pragma unroll
        for (int b = 0; b < 2; ++b) {
          const uint4* prow = reinterpret_cast<const uint4*>(pk + (b * kTileRows + row) * kPackedRowBytes);
          uint32_t o[32];
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) {
            const uint4 v = prow[ch ^ sw];
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              o[8 * ch + 2 * q] = w[q] & 0x0F0F0F0Fu;
              o[8 * ch + 2 * q + 1] = (w[q] >> 4) & 0x0F0F0F0Fu;
            }
          }
          tmem_st32_wait(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + A_COL0 +
                             static_cast<uint32_t>(ost) * 64 + static_cast<uint32_t>(b) * 32, o);
        }
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
    if (threadIdx.x == 7 * 32) {
      STALL_ADD(3, w_full);
      STALL_ADD(4, w_oempty);
      STALL_ADD(10, static_cast<unsigned long long>(clock64() - role_t0));
    }
  } else if (active && ((warp >= 2 && warp < 6) || warp >= 7 + kDqWarps)) {
    // =============================== promotion + tail ===========================
    constexpr int HT = BT / 2;                  // tokens per thread
    unsigned long long w_pfull = 0, w_sfull = 0;
    const long long role_t0 = clock64();
    const int quad = warp & 3;
    const int lrow = quad * 32 + lane;
    const int tk0 = (warp < 6) ? 0 : HT;        // first token of this thread's half
    const bool w_on_input = (a.flags & B200MOE_FLAG_WEIGHT_ON_INPUT) != 0;
    const bool mimic = (a.flags & B200MOE_FLAG_MIMIC_ROUNDING) != 0;
    const bool round_pair = mimic && c.split == 1;
    uint32_t j = 0;
    int iter = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < c.total; tile += c.grid_eff, ++iter) {
      const TileCoord t = decode_tile(tile, c, s_blk_off, a.E, BT, a.num_nt, a.kblocks, kTileN);
      const int buf = iter & 1;
      const int* col_row = s_col_row + buf * 32 + tk0;
      const float* col_gam = s_col_gam + buf * 32 + tk0;
      // scale (fp16, low half) and 1024 + zero (fp16, high half) of this thread's two weight rows
      const int n = t.n0 + lrow;
      const int n2 = second_off + t.n0 + lrow;
      const bool ok0 = n < a.w_rows, ok1 = n2 < a.w_rows;
      auto scale_of = [](uint32_t v) { return __half2float(__ushort_as_half(static_cast<unsigned short>(v & 0xFFFFu))); };
      // fp16(1024 + z) has the bit pattern 0x6400 + z; rows past the expert carry word 0 -> scale 0
      auto zero_of = [](uint32_t v) { return static_cast<int>((v >> 16) & 0x3FFu); };
      if (!mbar_wait_t(smem_u32(&bar_sfull[buf]), (iter >> 1) & 1, abort_flag, DEV_TIMEOUT_EPILOGUE, w_sfull)) break;
      const float* xf_t = s_xf + buf * nkb_max * BT + tk0;
      const int* xs_t = s_xsum + buf * nkb_max * BT + tk0;
      // valid columns of this thread's half (the same for the whole warp): with 16-token blocks the
      // arithmetic runs in chunks of four columns and skips the chunks that hold padding only; with
      // 32-token blocks a half that holds padding only is skipped
      const int nv = s_nvalid[buf] - tk0;

      float acc0[HT], acc1[HT];
#pragma unroll
      for (int i = 0; i < HT; ++i) {
        acc0[i] = 0.f;
        acc1[i] = 0.f;
      }
      for (int kb = t.kb0; kb < t.kb1; ++kb, ++j) {
        // everything that does not depend on the MMA first: the group's scale words (staged in
        // shared memory by the producer) and its activation tables
        const uint32_t zs = j % kSzSlots;
        if (!mbar_wait_t(smem_u32(&bar_zfull[zs]), (j / kSzSlots) & 1u, abort_flag, DEV_TIMEOUT_EPILOGUE, w_sfull)) {
          ok = false;
          break;
        }
        const uint32_t c0 = ok0 ? s_sz[zs * 256 + lrow] : 0u;
        const uint32_t c1 = ok1 ? s_sz[zs * 256 + 128 + lrow] : 0u;
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_zempty[zs]));
        const float s0 = scale_of(c0), s1 = scale_of(c1);
        const int z0 = zero_of(c0), z1 = zero_of(c1);
        float xfv[HT];
        int xsv[HT];
#pragma unroll
        for (int q = 0; q < HT / 4; ++q) {
          if (nv <= (HT == 8 ? 4 * q : 0)) {   // 32-token blocks skip by halves only (register budget)
#pragma unroll
            for (int i = 4 * q; i < 4 * q + 4; ++i) {
              xfv[i] = 0.f;
              xsv[i] = 0;
            }
            continue;
          }
          const float4 fv = *reinterpret_cast<const float4*>(xf_t + (kb - t.kb0) * BT + 4 * q);
          const int4 sv = *reinterpret_cast<const int4*>(xs_t + (kb - t.kb0) * BT + 4 * q);
          xfv[4 * q] = fv.x; xfv[4 * q + 1] = fv.y; xfv[4 * q + 2] = fv.z; xfv[4 * q + 3] = fv.w;
          xsv[4 * q] = sv.x; xsv[4 * q + 1] = sv.y; xsv[4 * q + 2] = sv.z; xsv[4 * q + 3] = sv.w;
        }
        const uint32_t pb = j & 1u;
        if (!mbar_wait_t(smem_u32(&bar_pfull[pb]), (j >> 1) & 1u, abort_flag, DEV_TIMEOUT_EPILOGUE, w_pfull)) {
          ok = false;
          break;
        }
        tc_fence_after();
        if (warp == 2 && lane == 0) {
          mbar_arrive(smem_u32(&bar_empty[j % static_cast<uint32_t>(stages)]));
          mbar_arrive(smem_u32(&bar_oempty[j % NO]));
        }
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + pb * PCOLS + tk0;
        if constexpr (HT == 8) {
          if (nv > 0) {
            int p[48];   // [block][plane][8 tokens]
            tmem_ld8x6_wait_b32(taddr, taddr + BT, taddr + 2 * BT, taddr + NB, taddr + NB + BT, taddr + NB + 2 * BT, p);
#pragma unroll
            for (int q = 0; q < 2; ++q) {
              if (nv <= 4 * q) continue;
#pragma unroll
              for (int i = 4 * q; i < 4 * q + 4; ++i) {
                const int sum0 = p[i] + (p[8 + i] << 8) + (p[16 + i] << 16) - z0 * xsv[i];
                const int sum1 = p[24 + i] + (p[32 + i] << 8) + (p[40 + i] << 16) - z1 * xsv[i];
                acc0[i] = fmaf(s0 * xfv[i], static_cast<float>(sum0), acc0[i]);
                acc1[i] = fmaf(s1 * xfv[i], static_cast<float>(sum1), acc1[i]);
              }
            }
          }
        } else {
          if (nv > 0) {
            int p0[16], p1[16], p2[16];
            tmem_ld16x3_wait_b32(taddr, taddr + BT, taddr + 2 * BT, p0, p1, p2);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const int sum = p0[i] + (p1[i] << 8) + (p2[i] << 16) - z0 * xsv[i];
              acc0[i] = fmaf(s0 * xfv[i], static_cast<float>(sum), acc0[i]);
            }
            tmem_ld16x3_wait_b32(taddr + NB, taddr + NB + BT, taddr + NB + 2 * BT, p0, p1, p2);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const int sum = p0[i] + (p1[i] << 8) + (p2[i] << 16) - z1 * xsv[i];
              acc1[i] = fmaf(s1 * xfv[i], static_cast<float>(sum), acc1[i]);
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_pempty[pb]));
      }
      if (!ok) break;

      if (MODE == 0) {
        // activation, rounded to fp16 as the 16-bit path stores it, then re-expressed for the
        // second GEMM: this tile's 128 columns are one of its reduction groups
        const bool n_ok = n < a.N;
        unsigned int* amax = s_amax + buf * 32 + tk0;
        int* osum = s_osum + buf * 32 + tk0;
        // per-expert bias of this thread's gate row and up / linear row, and the clamped swiglu
        const bool ext = a.bias != nullptr || a.activation == B200MOE_ACT_SWIGLU_OAI;
        float bg = 0.f, bu = 0.f;
        if (a.bias != nullptr && n_ok) {
          bg = __ldg(a.bias + static_cast<size_t>(t.e) * 2 * a.N + n);
          bu = __ldg(a.bias + static_cast<size_t>(t.e) * 2 * a.N + a.N + n);
        }
#pragma unroll
        for (int i = 0; i < HT; ++i) {
          float av = ext ? act_mul<__half, true>(acc0[i] + bg, acc1[i] + bu, w_on_input, col_gam[i], mimic, act_params(a))
                         : act_mul<__half>(acc0[i], acc1[i], w_on_input, col_gam[i], mimic, act_params(a));
          av = n_ok ? __half2float(__float2half_rn(av)) : 0.f;
          acc0[i] = av;
          const unsigned int m = __reduce_max_sync(0xffffffffu, __float_as_uint(fabsf(av)));
          if (lane == 0) atomicMax(amax + i, m);
        }
        // the eight warps meet on a barrier with a bounded wait (a plain bar.sync would hang the
        // CTA if one of them had given up)
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_tail[2 * buf]));
        if (!mbar_wait(smem_u32(&bar_tail[2 * buf]), (iter >> 1) & 1, abort_flag, DEV_TIMEOUT_EPILOGUE)) break;
        const int kcol = (n & ~7) | plane_pos(n & 7);
        const size_t plane_stride = static_cast<size_t>(BT) * a.ld_out;
        uint8_t* obase = a.out_q + static_cast<size_t>(t.row0 / BT) * 3 * plane_stride +
                         static_cast<size_t>(tk0) * a.ld_out + kcol;
#pragma unroll
        for (int i = 0; i < HT; ++i) {
          // group maximum in [2^ex, 2^(ex+1)): integers of magnitude below 2^19
          const unsigned int mb = amax[i];
          const int ex = static_cast<int>(mb >> 23) - 127;
          const float mult = (mb == 0u) ? 0.f : __uint_as_float(static_cast<unsigned int>(127 + 18 - ex) << 23);
          const int v = __float2int_rn(acc0[i] * mult);
          const int b0 = (v << 24) >> 24;
          const int v1 = (v - b0) >> 8;
          const int b1 = (v1 << 24) >> 24;
          const int b2 = (v1 - b1) >> 8;
          if (n_ok) {
            uint8_t* o = obase + static_cast<size_t>(i) * a.ld_out;
            o[0] = static_cast<uint8_t>(b0);
            o[plane_stride] = static_cast<uint8_t>(b1);
            o[2 * plane_stride] = static_cast<uint8_t>(b2);
          }
          const int ws = __reduce_add_sync(0xffffffffu, v);
          if (lane == 0) atomicAdd(osum + i, ws);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_tail[2 * buf + 1]));
        if (!mbar_wait(smem_u32(&bar_tail[2 * buf + 1]), (iter >> 1) & 1, abort_flag, DEV_TIMEOUT_EPILOGUE)) break;
        if (warp < 6 && lrow < BT && t.n0 < a.N) {
          const unsigned int mb = s_amax[buf * 32 + lrow];
          const int ex = static_cast<int>(mb >> 23) - 127;
          const float f = (mb == 0u) ? 1.0f : __uint_as_float(static_cast<unsigned int>(127 + ex - 18) << 23);
          const size_t dst = static_cast<size_t>(t.n0 / 128) * a.ld_xscale + t.row0 + lrow;
          a.out_scale[dst] = f;
          a.out_sum[dst] = s_osum[buf * 32 + lrow];
        }
      } else {
        float* out = reinterpret_cast<float*>(a.out) + n;
        const bool first = n < a.N, second = n + kTileRows < a.N;
        float b0 = 0.f, b1 = 0.f;      // the first reduction split carries the bias
        if (a.bias != nullptr && t.kb0 == 0) {
          if (first) b0 = __ldg(a.bias + static_cast<size_t>(t.e) * a.N + n);
          if (second) b1 = __ldg(a.bias + static_cast<size_t>(t.e) * a.N + n + kTileRows);
        }
#pragma unroll
        for (int i = 0; i < HT; ++i) {
          const int orow = col_row[i];
          if (orow >= 0) {
            const float gam = w_on_input ? 1.0f : col_gam[i];
            float y0 = (acc0[i] + b0) * gam, y1 = (acc1[i] + b1) * gam;
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

size_t w4_stage_bytes(const GemmArgs& a) {   // one stage of the TMA ring: three activation planes + packed rows
  return static_cast<size_t>(3 * a.BT) * kStageKBytes + 2 * kTileRows * kPackedRowBytes;
}
size_t w4_ctrl_bytes(const GemmArgs& a) {    // activation tables, barriers, per-tile tables
  return static_cast<size_t>(2) * 2 * a.kblocks * a.BT * 4 + kSzSlots * 1024 + 1024 + 4 * 8 + 2 * kSzSlots * 8 +
         4 * 2 * 32 * 4 +
         static_cast<size_t>(a.E + 1) * 4 + 64;
}

template <int MODE, int BT>
int launch_w4(const CUtensorMap& tm_w, const CUtensorMap& tm_x, const GemmArgs& a, int num_sms, cudaStream_t stream) {
  const size_t smem = 1024 + static_cast<size_t>(a.stages) * w4_stage_bytes(a) + w4_ctrl_bytes(a);
  if (smem > kSmemLimit) return B200MOE_ERR_TOO_LARGE;
  if (cudaFuncSetAttribute(moe_gemm_w4_kernel<MODE, BT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(smem)) != cudaSuccess)
    return B200MOE_ERR_CUDA;
  note_launch(MODE == 0 ? "moe_gemm_w4_kernel<gate/up>" : "moe_gemm_w4_kernel<down>");
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

bool gemm_w4_planes_ok(int K, int BT) {
  return (BT == 16 || BT == 32) && K % 128 == 0 && K / 128 <= kMaxGroupsW4;
}

void gemm_plan_w4(GemmArgs* a) {
  a->orient = 0;
  const int tile_n = (a->mode == 0) ? kTileRows : 2 * kTileRows;
  a->num_nt = (a->N + tile_n - 1) / tile_n;
  a->kblocks = (a->K + 127) / 128;  // reduction unit = one quantisation group
  a->tmem_cols = 512;               // two partial buffers of 6 * BT int32 columns + the A-operand stages
  a->acc_stages = 2;
  int st = static_cast<int>((kSmemLimit - 1024 - w4_ctrl_bytes(*a)) / w4_stage_bytes(*a));
  if (st > 8) st = 8;
  if (st < 2) st = 2;
  a->stages = st;
  if (a->max_split <= 0) a->max_split = 16;
}

int launch_gemm_w4(const CUtensorMap& tm_w, const CUtensorMap& tm_x, const GemmArgs& a, int num_sms,
                   cudaStream_t stream) {
  if (a.wmode != B200MOE_W_INT4_AWQ || a.dtype != B200MOE_DTYPE_FP16 || a.w_sz == nullptr) return B200MOE_ERR_BAD_ARG;
  if (!gemm_w4_planes_ok(a.K, a.BT) || a.x_scale == nullptr || a.x_sum == nullptr) return B200MOE_ERR_UNSUPPORTED;
  if (a.mode == 0 && (a.out_q == nullptr || a.out_scale == nullptr || a.out_sum == nullptr)) return B200MOE_ERR_BAD_ARG;
  if (a.BT == 16)
    return a.mode == 0 ? launch_w4<0, 16>(tm_w, tm_x, a, num_sms, stream) : launch_w4<1, 16>(tm_w, tm_x, a, num_sms, stream);
  return a.mode == 0 ? launch_w4<0, 32>(tm_w, tm_x, a, num_sms, stream) : launch_w4<1, 32>(tm_w, tm_x, a, num_sms, stream);
}

}  // namespace b200moe
