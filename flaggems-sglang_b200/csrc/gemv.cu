// Matrix-vector kernels for calls with a handful of (token, choice) pairs: see gemv.cuh.
#include "gemm_sched.cuh"
#include "gemv.cuh"

namespace b200moe {
namespace {

constexpr int kUpThreads = 256;     // 8 warps, one output column (gate row + up row) per warp at a time
constexpr int kDownThreads = 512;   // 16 warps, two output elements per warp at a time
constexpr int kChunk = 256;         // elements of one warp-wide 16-byte load

// streaming 16-byte load: the weights are read once, keep them out of L1
__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
      : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
      : "l"(p));
  return v;
}

template <typename T>
__device__ __forceinline__ void unpack2(uint32_t w, float& lo, float& hi);
template <>
__device__ __forceinline__ void unpack2<__nv_bfloat16>(uint32_t w, float& lo, float& hi) {
  lo = __uint_as_float(w << 16);
  hi = __uint_as_float(w & 0xffff0000u);
}
template <>
__device__ __forceinline__ void unpack2<__half>(uint32_t w, float& lo, float& hi) {
  const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w));
  lo = f.x;
  hi = f.y;
}

// Token rows and activations are staged in shared memory as fp32 in two planes: elements 0..3 of
// every run of eight in the first half of the row, elements 4..7 in the second.  A lane that holds
// eight consecutive weights (one 16-byte load) then reads two float4 whose addresses are
// consecutive across the lanes of the warp: no bank conflicts.
__device__ __forceinline__ int plane_index(int k, int n) {
  return ((k >> 2) & 1) * (n >> 1) + ((k >> 3) << 2) + (k & 3);
}

// acc + sum of eight 16-bit weights (elements k .. k+7, k a multiple of 8) times the staged row
template <typename T>
__device__ __forceinline__ float dot8(const uint4& w, const float* row, int k, int n, float acc) {
  const float4 x0 = *reinterpret_cast<const float4*>(row + (k >> 1));
  const float4 x1 = *reinterpret_cast<const float4*>(row + (n >> 1) + (k >> 1));
  float a, b;
  unpack2<T>(w.x, a, b);
  acc = fmaf(a, x0.x, acc);
  acc = fmaf(b, x0.y, acc);
  unpack2<T>(w.y, a, b);
  acc = fmaf(a, x0.z, acc);
  acc = fmaf(b, x0.w, acc);
  unpack2<T>(w.z, a, b);
  acc = fmaf(a, x1.x, acc);
  acc = fmaf(b, x1.y, acc);
  unpack2<T>(w.w, a, b);
  acc = fmaf(a, x1.z, acc);
  acc = fmaf(b, x1.w, acc);
  return acc;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <typename T>
__device__ __forceinline__ void load4_f32(const T* p, float (&v)[4]) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  unpack2<T>(raw.x, v[0], v[1]);
  unpack2<T>(raw.y, v[2], v[3]);
}

// Local expert and routing weight of every pair, into shared memory (P <= kGemvMaxPairs).  From
// topk_ids / topk_weights (with an optional global -> local map), or from the routing triple
// hist[E] / topk_indx[P] / gate_scal[P] (sorted row -> pair slot, weights in sorted order).
// Called by every thread of the CTA; the caller synchronises before reading the tables.
__device__ __forceinline__ void stage_routing(const GemvArgs& a, int* s_e, float* s_gam) {
  const int P = a.M * a.topk;
  const int p = threadIdx.x;
  if (a.hist == nullptr) {
    if (p < P) {
      long long id = a.ids_i64 ? reinterpret_cast<const long long*>(a.topk_ids)[p]
                               : static_cast<long long>(reinterpret_cast<const int*>(a.topk_ids)[p]);
      if (a.expert_map != nullptr) id = (id >= 0 && id < a.n_global) ? a.expert_map[id] : -1;
      s_e[p] = (id >= 0 && id < a.E) ? static_cast<int>(id) : -1;
      s_gam[p] = a.topk_w[p];
    }
    return;
  }
  if (p < P) s_e[p] = -1;
  __syncthreads();
  if (p < P) {
    // sorted row p belongs to the expert whose run of hist[] covers it
    int e = -1, end = 0;
    for (int i = 0; i < a.E; ++i) {
      end += a.hist[i];
      if (p < end) {
        e = i;
        break;
      }
    }
    const int slot = (e >= 0) ? a.topk_indx[p] : -1;
    if (slot >= 0 && slot < P) {
      s_e[slot] = e;
      s_gam[slot] = a.gate_scal[p];
    }
  }
}

// ------------------------------------------------------------------------------------------
// act[p][i] = activation(w1[e_p][i] . x_t, w1[e_p][I + i] . x_t) in the 16-bit type
// U: 256-element chunks of each row that a lane keeps in flight.  4 by default (8 halves the resident
// CTAs and measured 10 % slower); 5 or 6 when that is the whole row, so that a row of 1280 or 1536
// elements does not need a second, nearly empty pass.
template <typename T, int U>
__global__ void __launch_bounds__(kUpThreads)
moe_gemv_up_kernel(const GemvArgs a) {
  extern __shared__ __align__(16) uint8_t gemv_smem[];
  const int P = a.M * a.topk;
  float* s_x = reinterpret_cast<float*>(gemv_smem);                 // [M][H], two planes per row
  int* s_e = reinterpret_cast<int*>(s_x + static_cast<size_t>(a.M) * a.H);
  float* s_gam = reinterpret_cast<float*>(s_e + kGemvMaxPairs);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  griddep_wait();
  griddep_launch_dependents();
  stage_routing(a, s_e, s_gam);
  const T* x = reinterpret_cast<const T*>(a.x);
  const int quads = a.H >> 2;
  for (int i = threadIdx.x; i < a.M * quads; i += kUpThreads) {
    const int t = i / quads, k = (i - t * quads) << 2;
    float v[4];
    load4_f32<T>(x + static_cast<size_t>(t) * a.H + k, v);
    *reinterpret_cast<float4*>(s_x + static_cast<size_t>(t) * a.H + plane_index(k, a.H)) =
        make_float4(v[0], v[1], v[2], v[3]);
  }
  __syncthreads();

  const bool w_on_input = (a.flags & B200MOE_FLAG_WEIGHT_ON_INPUT) != 0;
  const bool mimic = (a.flags & B200MOE_FLAG_MIMIC_ROUNDING) != 0;
  const bool ext = a.b1 != nullptr || a.activation == B200MOE_ACT_SWIGLU_OAI;
  ActParams ap;
  ap.activation = a.activation;
  ap.alpha = a.alpha;
  ap.limit = a.limit;
  T* act = reinterpret_cast<T*>(a.act);
  const T* w1 = reinterpret_cast<const T*>(a.w1);

  const int total = P * a.I;
  const int warps = gridDim.x * (kUpThreads / 32);
  // consecutive columns go to different SMs, so every SM streams the same share
  for (int c = warp * gridDim.x + blockIdx.x; c < total; c += warps) {
    const int p = c / a.I, i = c - p * a.I;
    const int e = s_e[p];
    if (e < 0) {
      if (lane == 0) act[c] = from_f32<T>(0.f);
      continue;
    }
    const float* xs = s_x + static_cast<size_t>(p / a.topk) * a.H;
    const T* wg = w1 + (static_cast<size_t>(e) * 2 * a.I + i) * a.H;
    const T* wu = wg + static_cast<size_t>(a.I) * a.H;
    float ag = 0.f, au = 0.f;
    for (int k0 = lane * 8; k0 < a.H; k0 += U * kChunk) {
      uint4 gq[U], uq[U];
#pragma unroll
      for (int q = 0; q < U; ++q) {
        const int k = k0 + q * kChunk;
        if (k < a.H) {
          gq[q] = ldg_stream(wg + k);
          uq[q] = ldg_stream(wu + k);
        }
      }
#pragma unroll
      for (int q = 0; q < U; ++q) {
        const int k = k0 + q * kChunk;
        if (k < a.H) {
          ag = dot8<T>(gq[q], xs, k, a.H, ag);
          au = dot8<T>(uq[q], xs, k, a.H, au);
        }
      }
    }
    ag = warp_sum(ag);
    au = warp_sum(au);
    if (lane == 0) {
      if (a.b1 != nullptr) {
        ag += __ldg(a.b1 + static_cast<size_t>(e) * 2 * a.I + i);
        au += __ldg(a.b1 + static_cast<size_t>(e) * 2 * a.I + a.I + i);
      }
      const float av = ext ? act_mul<T, true>(ag, au, w_on_input, s_gam[p], mimic, ap)
                           : act_mul<T>(ag, au, w_on_input, s_gam[p], mimic, ap);
      act[c] = from_f32<T>(av);
    }
  }
}

// ------------------------------------------------------------------------------------------
// out[t][h] = cast(routed_scaling * sum_j gamma_j * (w2[e_j][h] . act[p_j] + b2[e_j][h]))
// One warp per pair of output elements (h, h + 1) of a token: the two weight rows share every read
// of the staged activations.
template <typename T>
__global__ void __launch_bounds__(kDownThreads)
moe_gemv_down_kernel(const GemvArgs a) {
  extern __shared__ __align__(16) uint8_t gemv_smem[];
  const int P = a.M * a.topk;
  float* s_act = reinterpret_cast<float*>(gemv_smem);               // [P][I], two planes per row
  int* s_e = reinterpret_cast<int*>(s_act + static_cast<size_t>(P) * a.I);
  float* s_gam = reinterpret_cast<float*>(s_e + kGemvMaxPairs);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool w_on_input = (a.flags & B200MOE_FLAG_WEIGHT_ON_INPUT) != 0;
  const bool no_combine = (a.flags & B200MOE_FLAG_NO_COMBINE) != 0;
  // per-pair results are needed one by one when each is rounded or stored by itself; otherwise the
  // routing weight is folded into the staged activations and one running sum covers all pairs
  const bool by_pair = no_combine || a.round_pair != 0;

  const T* w2 = reinterpret_cast<const T*>(a.w2);
  const int nch = (a.I + kChunk - 1) / kChunk;
  T* out = reinterpret_cast<T*>(a.out);
  const int half_h = a.H >> 1;
  const int tasks = a.M * half_h;
  // With fewer tasks than warps, S = a.down_split warps share a task: each takes a contiguous share
  // of the (pair, chunk) slots, the partial sums meet in shared memory and are added in a fixed order.
  const int S = by_pair ? 1 : a.down_split;
  const int grp = warp / S, sub = warp - grp * S;
  const int groups = gridDim.x * ((kDownThreads / 32) / S);
  const int Q = a.topk * nch;
  const int share = (Q + S - 1) / S;
  const int q_lo = sub * share, q_hi = min(Q, q_lo + share);
  float* s_part = s_gam + kGemvMaxPairs;                            // [2 buffers][16 warps][2]

  // a run: eight (pair, chunk) slots of two rows, 16 loads of 16 bytes in flight per lane
  struct Run {
    uint4 wa[8], wb[8];
    int kk[8], pp[8];
  };
  auto load_run = [&](Run& r, int t, int h, int q0, int& j, int& ch) {
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int p = t * a.topk + j;
      const int k = ch * kChunk + lane * 8;
      const int e = (q0 + u < q_hi) ? s_e[p] : -1;
      const bool on = e >= 0 && k < a.I;
      r.kk[u] = on ? k : -1;
      r.pp[u] = p;
      if (on) {
        const T* wr = w2 + (static_cast<size_t>(e) * a.H + h) * a.I + k;
        r.wa[u] = ldg_stream(wr);
        r.wb[u] = ldg_stream(wr + a.I);
      }
      if (++ch == nch) {
        ch = 0;
        ++j;
      }
    }
  };

  // The routing tables and the weights do not depend on the up kernel: they are read before waiting
  // for it, and when the layer is small (several warps per task: the kernel is a few memory round
  // trips long) the first run of this warp's first task is put in flight as well.  With one warp per
  // task the early loads only take bandwidth from the up kernel's tail (Mixtral-shaped layer at M = 1:
  // 127 us with, 123 us without).
  stage_routing(a, s_e, s_gam);
  __syncthreads();
  Run r;                       // one register buffer: the prefetched run is consumed in place
  const int task0 = grp * gridDim.x + blockIdx.x;
  bool have_pre = false;
  int pre_j = 0, pre_ch = 0;
  if (!by_pair && S > 1 && task0 < tasks && q_lo < q_hi) {
    const int t = task0 / half_h, h = (task0 - t * half_h) << 1;
    pre_j = q_lo / nch;
    pre_ch = q_lo - pre_j * nch;
    load_run(r, t, h, q_lo, pre_j, pre_ch);
    have_pre = true;
  }
  griddep_wait();
  griddep_launch_dependents();
  const T* act = reinterpret_cast<const T*>(a.act);
  const int quads = a.I >> 2;
  for (int i = threadIdx.x; i < P * quads; i += kDownThreads) {
    const int p = i / quads, k = (i - p * quads) << 2;
    const float fold = (by_pair || w_on_input) ? 1.0f : s_gam[p];
    float v[4];
    load4_f32<T>(act + static_cast<size_t>(p) * a.I + k, v);
    *reinterpret_cast<float4*>(s_act + static_cast<size_t>(p) * a.I + plane_index(k, a.I)) =
        make_float4(v[0] * fold, v[1] * fold, v[2] * fold, v[3] * fold);
  }
  __syncthreads();

  int iter = 0;
  for (int task = task0; task < tasks; task += groups, ++iter) {
    const int t = task / half_h, h = (task - t * half_h) << 1;
    if (!by_pair) {
      float acc0 = 0.f, acc1 = 0.f;
      int j = q_lo / nch, ch = q_lo - j * nch;
      for (int q0 = q_lo; q0 < q_hi; q0 += 8) {
        if (have_pre) {
          j = pre_j;
          ch = pre_ch;
          have_pre = false;
        } else {
          load_run(r, t, h, q0, j, ch);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          if (r.kk[u] >= 0) {
            const float* av = s_act + static_cast<size_t>(r.pp[u]) * a.I;
            acc0 = dot8<T>(r.wa[u], av, r.kk[u], a.I, acc0);
            acc1 = dot8<T>(r.wb[u], av, r.kk[u], a.I, acc1);
          }
        }
      }
      acc0 = warp_sum(acc0);
      acc1 = warp_sum(acc1);
      if (S > 1) {
        float* part = s_part + (iter & 1) * 2 * (kDownThreads / 32);
        if (lane == 0) {
          part[2 * warp] = acc0;
          part[2 * warp + 1] = acc1;
        }
        named_bar_sync(1 + grp, 32 * S);   // the S warps of this task (same trip counts: no warp can be missing)
        if (sub == 0 && lane == 0) {
          acc0 = 0.f;
          acc1 = 0.f;
          for (int w = 0; w < S; ++w) {
            acc0 += part[2 * (warp + w)];
            acc1 += part[2 * (warp + w) + 1];
          }
        }
      }
      if (sub == 0 && lane == 0) {
        if (a.b2 != nullptr) {
          for (int jb = 0; jb < a.topk; ++jb) {
            const int p = t * a.topk + jb;
            if (s_e[p] >= 0) {
              const float gam = w_on_input ? 1.0f : s_gam[p];
              acc0 = fmaf(__ldg(a.b2 + static_cast<size_t>(s_e[p]) * a.H + h), gam, acc0);
              acc1 = fmaf(__ldg(a.b2 + static_cast<size_t>(s_e[p]) * a.H + h + 1), gam, acc1);
            }
          }
        }
        out[static_cast<size_t>(t) * a.H + h] = from_f32<T>(acc0 * a.routed_scaling);
        out[static_cast<size_t>(t) * a.H + h + 1] = from_f32<T>(acc1 * a.routed_scaling);
      }
    } else {
      float sum0 = 0.f, sum1 = 0.f;
      for (int jb = 0; jb < a.topk; ++jb) {
        const int p = t * a.topk + jb;
        const int e = s_e[p];
        float y0 = 0.f, y1 = 0.f;
        if (e >= 0) {
          const T* wr = w2 + (static_cast<size_t>(e) * a.H + h) * a.I;
          const float* av = s_act + static_cast<size_t>(p) * a.I;
          float acc0 = 0.f, acc1 = 0.f;
          for (int k0 = lane * 8; k0 < a.I; k0 += 4 * kChunk) {
            uint4 wa[4], wb[4];
#pragma unroll
            for (int q = 0; q < 4; ++q)
              if (k0 + q * kChunk < a.I) {
                wa[q] = ldg_stream(wr + k0 + q * kChunk);
                wb[q] = ldg_stream(wr + a.I + k0 + q * kChunk);
              }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const int k = k0 + q * kChunk;
              if (k < a.I) {
                acc0 = dot8<T>(wa[q], av, k, a.I, acc0);
                acc1 = dot8<T>(wb[q], av, k, a.I, acc1);
              }
            }
          }
          acc0 = warp_sum(acc0);
          acc1 = warp_sum(acc1);
          if (a.b2 != nullptr) {
            acc0 += __ldg(a.b2 + static_cast<size_t>(e) * a.H + h);
            acc1 += __ldg(a.b2 + static_cast<size_t>(e) * a.H + h + 1);
          }
          y0 = w_on_input ? acc0 : acc0 * s_gam[p];
          y1 = w_on_input ? acc1 : acc1 * s_gam[p];
          if (a.round_pair) {
            y0 = to_f32<T>(from_f32<T>(y0));
            y1 = to_f32<T>(from_f32<T>(y1));
          }
        }
        if (no_combine) {
          if (lane == 0) {
            out[static_cast<size_t>(p) * a.H + h] = from_f32<T>(y0);
            out[static_cast<size_t>(p) * a.H + h + 1] = from_f32<T>(y1);
          }
        } else {
          sum0 += y0;
          sum1 += y1;
        }
      }
      if (!no_combine && lane == 0) {
        out[static_cast<size_t>(t) * a.H + h] = from_f32<T>(sum0 * a.routed_scaling);
        out[static_cast<size_t>(t) * a.H + h + 1] = from_f32<T>(sum1 * a.routed_scaling);
      }
    }
  }
}

// ==========================================================================================
// int4 (AWQ) weights: the same two launches on integer dot products.
//
// The activations take the form the integer tensor-core kernels use (gemm_w4.cu): per 128-k group
// a power-of-two scale f = 2^(e-18) for a group maximum in [2^e, 2^(e+1)) and the exact integers
// v = rint(x / f), |v| < 2^19, as three signed byte planes v = p0 + 256 p1 + 65536 p2.  A packed
// word holds eight weights; `w & 0x0F0F0F0F` and `(w >> 4) & 0x0F0F0F0F` are their raw nibbles as
// unsigned bytes in the order (0, 4, 1, 5) and (2, 6, 3, 7), the planes are staged in that order,
// and one dp4a per plane and half word gives exact sums S = S0 + 256 S1 + 65536 S2.  Per 32-k
// segment (one 16-byte load of a lane, inside one quantisation group):
// acc += (s f) * float(S - z * sum(v)), s and z the group's scale and zero point of the row.
// One instruction per weight instead of a conversion and a multiply-add for each.

__device__ __forceinline__ int dp4a_u8_s8(uint32_t a, uint32_t b, int c) {
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

// A row of K staged bytes per plane is kept in two halves: bytes 0..15 of every run of 32 in the
// first, bytes 16..31 in the second, so that the two 16-byte reads of a lane (its 32 k) are
// contiguous across the warp.
__device__ __forceinline__ int half_index(int o, int K) { return ((o >> 4) & 1) * (K >> 1) + ((o >> 5) << 4) + (o & 15); }

struct StagedW4 {
  uint8_t* planes;   // [rows][3][K]
  float* f;          // [rows][K / 128] group scale (routing weight folded in where asked)
  int* vsum;         // [rows][K / 32] sum of the integers of every 32-k segment
};

// fp16 rows -> planes, scales and segment sums; one warp per (row, group), the arithmetic of
// group_split_i8_kernel (prep.cu).  fold[row] multiplies the stored scale (nullptr: 1).
__device__ __forceinline__ void stage_w4(const __half* src, int rows, int K, const StagedW4& st, const float* fold,
                                         int nthreads) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int groups = K >> 7;
  for (int w = warp; w < rows * groups; w += nthreads >> 5) {
    const int r = w / groups, g = w - r * groups;
    float v[4];
    load4_f32<__half>(src + static_cast<size_t>(r) * K + g * 128 + lane * 4, v);
    const float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
    const unsigned int mb = __reduce_max_sync(0xffffffffu, __float_as_uint(amax));
    const int ex = static_cast<int>(mb >> 23) - 127;
    const float mult = (mb == 0u) ? 0.f : __uint_as_float(static_cast<unsigned int>(127 + 18 - ex) << 23);
    const float f = (mb == 0u) ? 1.0f : __uint_as_float(static_cast<unsigned int>(127 + ex - 18) << 23);
    uint32_t pk[3] = {0u, 0u, 0u};
    int part = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int q = __float2int_rn(v[i] * mult);
      const int b0 = (q << 24) >> 24;
      const int q1 = (q - b0) >> 8;
      const int b1 = (q1 << 24) >> 24;
      const int b2 = (q1 - b1) >> 8;
      pk[0] |= static_cast<uint32_t>(b0 & 0xFF) << (8 * i);
      pk[1] |= static_cast<uint32_t>(b1 & 0xFF) << (8 * i);
      pk[2] |= static_cast<uint32_t>(b2 & 0xFF) << (8 * i);
      part += q;
    }
    // an even lane holds elements 0..3 of its run of eight, the odd neighbour 4..7; stored order
    // is (0, 4, 1, 5 | 2, 6, 3, 7)
    uint8_t* dst = st.planes + static_cast<size_t>(r) * 3 * K + half_index(g * 128 + lane * 4, K);
#pragma unroll
    for (int p = 0; p < 3; ++p) {
      const uint32_t other = __shfl_xor_sync(0xffffffffu, pk[p], 1);
      const uint32_t word = (lane & 1) ? __byte_perm(pk[p], other, 0x3726) : __byte_perm(pk[p], other, 0x5140);
      *reinterpret_cast<uint32_t*>(dst + p * K) = word;
    }
    part += __shfl_xor_sync(0xffffffffu, part, 1);
    part += __shfl_xor_sync(0xffffffffu, part, 2);
    part += __shfl_xor_sync(0xffffffffu, part, 4);
    if ((lane & 7) == 0) st.vsum[r * (K >> 5) + g * 4 + (lane >> 3)] = part;
    if (lane == 0) st.f[r * groups + g] = f * (fold != nullptr ? fold[r] : 1.0f);
  }
}

// exact integer dot of the 32 nibbles of one 16-byte load with the staged integers of its 32 k
__device__ __forceinline__ int dot32_w4(const uint4& w, const uint8_t* row_planes, int k, int K) {
  const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
  uint32_t lo[4], hi[4];
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    lo[r] = ww[r] & 0x0F0F0F0Fu;
    hi[r] = (ww[r] >> 4) & 0x0F0F0F0Fu;
  }
  int s[3];
#pragma unroll
  for (int p = 0; p < 3; ++p) {
    const uint4 xa = *reinterpret_cast<const uint4*>(row_planes + p * K + (k >> 1));
    const uint4 xb = *reinterpret_cast<const uint4*>(row_planes + p * K + (K >> 1) + (k >> 1));
    int acc = dp4a_u8_s8(lo[0], xa.x, 0);
    acc = dp4a_u8_s8(hi[0], xa.y, acc);
    acc = dp4a_u8_s8(lo[1], xa.z, acc);
    acc = dp4a_u8_s8(hi[1], xa.w, acc);
    acc = dp4a_u8_s8(lo[2], xb.x, acc);
    acc = dp4a_u8_s8(hi[2], xb.y, acc);
    acc = dp4a_u8_s8(lo[3], xb.z, acc);
    acc = dp4a_u8_s8(hi[3], xb.w, acc);
    s[p] = acc;
  }
  return s[0] + (s[1] << 8) + (s[2] << 16);
}

// acc + (s f) * float(S - z * sum(v)) for the segment at k; c is the scale word of the row and the
// segment's group (fp16 scale | fp16(1024 + zero) << 16).  The words of a row lie one table row
// apart ([E][K/128][rows]), so the callers load them together with the weights, not here.
__device__ __forceinline__ float seg_w4(const uint4& w, const uint8_t* row_planes, const float* f, const int* vsum,
                                        uint32_t c, int k, int K, float acc) {
  const float s = __half2float(__ushort_as_half(static_cast<unsigned short>(c & 0xFFFFu)));
  const int z = static_cast<int>((c >> 16) & 0x3FFu);
  const int S = dot32_w4(w, row_planes, k, K) - z * vsum[k >> 5];
  return fmaf(s * f[k >> 7], static_cast<float>(S), acc);
}

constexpr int kSeg = 32 * 32;   // k covered by one warp-wide 16-byte load of packed nibbles

__device__ __forceinline__ StagedW4 carve_w4(uint8_t* base, int rows, int K) {
  StagedW4 st;
  st.planes = base;
  st.f = reinterpret_cast<float*>(base + static_cast<size_t>(rows) * 3 * K);
  st.vsum = reinterpret_cast<int*>(st.f + rows * (K >> 7));
  return st;
}
size_t staged_w4_bytes(int rows, int K) {
  return static_cast<size_t>(rows) * (3 * K + (K >> 7) * 4 + (K >> 5) * 4);
}

// (capping the registers for three resident CTAs instead of two was slower: 74 us vs 69 us at M = 1)
__global__ void __launch_bounds__(kUpThreads)
moe_gemv_w4_up_kernel(const GemvArgs a) {
  extern __shared__ __align__(16) uint8_t gemv_smem[];
  const int P = a.M * a.topk;
  const StagedW4 st = carve_w4(gemv_smem, a.M, a.H);
  int* s_e = st.vsum + a.M * (a.H >> 5);
  float* s_gam = reinterpret_cast<float*>(s_e + kGemvMaxPairs);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  griddep_wait();
  griddep_launch_dependents();
  stage_routing(a, s_e, s_gam);
  stage_w4(reinterpret_cast<const __half*>(a.x), a.M, a.H, st, nullptr, kUpThreads);
  __syncthreads();

  const bool w_on_input = (a.flags & B200MOE_FLAG_WEIGHT_ON_INPUT) != 0;
  const bool mimic = (a.flags & B200MOE_FLAG_MIMIC_ROUNDING) != 0;
  const bool ext = a.b1 != nullptr || a.activation == B200MOE_ACT_SWIGLU_OAI;
  ActParams ap;
  ap.activation = a.activation;
  ap.alpha = a.alpha;
  ap.limit = a.limit;
  __half* act = reinterpret_cast<__half*>(a.act);
  const uint8_t* w1 = reinterpret_cast<const uint8_t*>(a.w1);
  const uint32_t* sz1 = reinterpret_cast<const uint32_t*>(a.w1_sz);
  const size_t rows = 2 * static_cast<size_t>(a.I);      // weight rows (and scale words per group) of an expert
  const int G = a.H >> 7;

  // (Two register buffers with the next item's loads in flight while the current one is multiplied
  // were tried: 89 us against 69 us for the Mixtral-shaped layer at M = 1.)
  const int total = P * a.I;
  const int warps = gridDim.x * (kUpThreads / 32);
  for (int c = warp * gridDim.x + blockIdx.x; c < total; c += warps) {
    const int p = c / a.I, i = c - p * a.I;
    const int e = s_e[p];
    if (e < 0) {
      if (lane == 0) act[c] = __float2half_rn(0.f);
      continue;
    }
    const int t = p / a.topk;
    const uint8_t* xp = st.planes + static_cast<size_t>(t) * 3 * a.H;
    const float* xf = st.f + t * G;
    const int* xv = st.vsum + t * (a.H >> 5);
    const uint8_t* wg = w1 + (static_cast<size_t>(e) * rows + i) * (a.H >> 1);
    const uint8_t* wu = wg + static_cast<size_t>(a.I) * (a.H >> 1);
    const uint32_t* szg = sz1 + static_cast<size_t>(e) * G * rows + i;
    const uint32_t* szu = szg + a.I;
    float ag = 0.f, au = 0.f;
    for (int k0 = lane * 32; k0 < a.H; k0 += 4 * kSeg) {
      uint4 gq[4], uq[4];
      uint32_t cg[4], cu[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int k = k0 + q * kSeg;
        if (k < a.H) {
          gq[q] = ldg_stream(wg + (k >> 1));
          uq[q] = ldg_stream(wu + (k >> 1));
          cg[q] = __ldg(szg + static_cast<size_t>(k >> 7) * rows);
          cu[q] = __ldg(szu + static_cast<size_t>(k >> 7) * rows);
        }
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int k = k0 + q * kSeg;
        if (k < a.H) {
          ag = seg_w4(gq[q], xp, xf, xv, cg[q], k, a.H, ag);
          au = seg_w4(uq[q], xp, xf, xv, cu[q], k, a.H, au);
        }
      }
    }
    ag = warp_sum(ag);
    au = warp_sum(au);
    if (lane == 0) {
      if (a.b1 != nullptr) {
        ag += __ldg(a.b1 + static_cast<size_t>(e) * 2 * a.I + i);
        au += __ldg(a.b1 + static_cast<size_t>(e) * 2 * a.I + a.I + i);
      }
      const float av = ext ? act_mul<__half, true>(ag, au, w_on_input, s_gam[p], mimic, ap)
                           : act_mul<__half>(ag, au, w_on_input, s_gam[p], mimic, ap);
      act[c] = __float2half_rn(av);
    }
  }
}

__global__ void __launch_bounds__(kDownThreads)
moe_gemv_w4_down_kernel(const GemvArgs a) {
  extern __shared__ __align__(16) uint8_t gemv_smem[];
  const int P = a.M * a.topk;
  const StagedW4 st = carve_w4(gemv_smem, P, a.I);
  int* s_e = st.vsum + P * (a.I >> 5);
  float* s_gam = reinterpret_cast<float*>(s_e + kGemvMaxPairs);
  float* s_fold = s_gam + kGemvMaxPairs;
  float* s_part = s_fold + kGemvMaxPairs;                           // [2 buffers][16 warps][2]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool w_on_input = (a.flags & B200MOE_FLAG_WEIGHT_ON_INPUT) != 0;
  const bool no_combine = (a.flags & B200MOE_FLAG_NO_COMBINE) != 0;
  const bool by_pair = no_combine || a.round_pair != 0;

  griddep_wait();
  griddep_launch_dependents();
  stage_routing(a, s_e, s_gam);
  __syncthreads();
  if (threadIdx.x < P) s_fold[threadIdx.x] = (by_pair || w_on_input) ? 1.0f : s_gam[threadIdx.x];
  __syncthreads();
  stage_w4(reinterpret_cast<const __half*>(a.act), P, a.I, st, s_fold, kDownThreads);
  __syncthreads();

  const uint8_t* w2 = reinterpret_cast<const uint8_t*>(a.w2);
  const uint32_t* sz2 = reinterpret_cast<const uint32_t*>(a.w2_sz);
  const size_t rows = static_cast<size_t>(a.H);
  const int G = a.I >> 7;
  const int nch = (a.I + kSeg - 1) / kSeg;
  __half* out = reinterpret_cast<__half*>(a.out);
  const int half_h = a.H >> 1;
  const int tasks = a.M * half_h;
  const int S = by_pair ? 1 : a.down_split;
  const int grp = warp / S, sub = warp - grp * S;
  const int groups = gridDim.x * ((kDownThreads / 32) / S);
  int iter = 0;
  for (int task = grp * gridDim.x + blockIdx.x; task < tasks; task += groups, ++iter) {
    const int t = task / half_h, h = (task - t * half_h) << 1;
    if (!by_pair) {
      // (pair, segment) flattened: four slots of two 16-byte loads (and their scale words) in flight
      const int Q = a.topk * nch;
      float acc0 = 0.f, acc1 = 0.f;
      int j = 0, ch = 0;
      for (int q0 = 0; q0 < Q; q0 += 4) {
        if (S > 1 && ((q0 >> 2) % S) != sub) {
          ch += 4;
          while (ch >= nch) {
            ch -= nch;
            ++j;
          }
          continue;
        }
        uint4 wa[4], wb[4];
        uint2 cc[4];
        int kk[4], pp[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int p = t * a.topk + j;
          const int k = ch * kSeg + lane * 32;
          const int e = (q0 + u < Q) ? s_e[p] : -1;
          const bool on = e >= 0 && k < a.I;
          kk[u] = on ? k : -1;
          pp[u] = p;
          if (on) {
            const uint8_t* wr = w2 + ((static_cast<size_t>(e) * rows + h) * a.I + k) / 2;
            wa[u] = ldg_stream(wr);
            wb[u] = ldg_stream(wr + (a.I >> 1));
            // rows h and h + 1 (h even) are neighbours in the scale table: one 8-byte load
            cc[u] = __ldg(reinterpret_cast<const uint2*>(sz2 + (static_cast<size_t>(e) * G + (k >> 7)) * rows + h));
          }
          if (++ch == nch) {
            ch = 0;
            ++j;
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (kk[u] >= 0) {
            const int p = pp[u];
            const uint8_t* xp = st.planes + static_cast<size_t>(p) * 3 * a.I;
            acc0 = seg_w4(wa[u], xp, st.f + p * G, st.vsum + p * (a.I >> 5), cc[u].x, kk[u], a.I, acc0);
            acc1 = seg_w4(wb[u], xp, st.f + p * G, st.vsum + p * (a.I >> 5), cc[u].y, kk[u], a.I, acc1);
          }
        }
      }
      acc0 = warp_sum(acc0);
      acc1 = warp_sum(acc1);
      if (S > 1) {
        float* part = s_part + (iter & 1) * 2 * (kDownThreads / 32);
        if (lane == 0) {
          part[2 * warp] = acc0;
          part[2 * warp + 1] = acc1;
        }
        named_bar_sync(1 + grp, 32 * S);
        if (sub == 0 && lane == 0) {
          acc0 = 0.f;
          acc1 = 0.f;
          for (int w = 0; w < S; ++w) {
            acc0 += part[2 * (warp + w)];
            acc1 += part[2 * (warp + w) + 1];
          }
        }
      }
      if (sub == 0 && lane == 0) {
        if (a.b2 != nullptr) {
          for (int jb = 0; jb < a.topk; ++jb) {
            const int p = t * a.topk + jb;
            if (s_e[p] >= 0) {
              const float gam = w_on_input ? 1.0f : s_gam[p];
              acc0 = fmaf(__ldg(a.b2 + static_cast<size_t>(s_e[p]) * a.H + h), gam, acc0);
              acc1 = fmaf(__ldg(a.b2 + static_cast<size_t>(s_e[p]) * a.H + h + 1), gam, acc1);
            }
          }
        }
        out[static_cast<size_t>(t) * a.H + h] = __float2half_rn(acc0 * a.routed_scaling);
        out[static_cast<size_t>(t) * a.H + h + 1] = __float2half_rn(acc1 * a.routed_scaling);
      }
    } else {
      float sum0 = 0.f, sum1 = 0.f;
      for (int jb = 0; jb < a.topk; ++jb) {
        const int p = t * a.topk + jb;
        const int e = s_e[p];
        float y0 = 0.f, y1 = 0.f;
        if (e >= 0) {
          const uint8_t* wr = w2 + ((static_cast<size_t>(e) * rows + h) * a.I) / 2;
          const uint32_t* sz = sz2 + static_cast<size_t>(e) * G * rows + h;
          const uint8_t* xp = st.planes + static_cast<size_t>(p) * 3 * a.I;
          float acc0 = 0.f, acc1 = 0.f;
          for (int k0 = lane * 32; k0 < a.I; k0 += 4 * kSeg) {
            uint4 wa[4], wb[4];
            uint2 cc[4];
#pragma unroll
            for (int q = 0; q < 4; ++q)
              if (k0 + q * kSeg < a.I) {
                wa[q] = ldg_stream(wr + ((k0 + q * kSeg) >> 1));
                wb[q] = ldg_stream(wr + ((a.I + k0 + q * kSeg) >> 1));
                cc[q] = __ldg(reinterpret_cast<const uint2*>(sz + static_cast<size_t>((k0 + q * kSeg) >> 7) * rows));
              }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const int k = k0 + q * kSeg;
              if (k < a.I) {
                acc0 = seg_w4(wa[q], xp, st.f + p * G, st.vsum + p * (a.I >> 5), cc[q].x, k, a.I, acc0);
                acc1 = seg_w4(wb[q], xp, st.f + p * G, st.vsum + p * (a.I >> 5), cc[q].y, k, a.I, acc1);
              }
            }
          }
          acc0 = warp_sum(acc0);
          acc1 = warp_sum(acc1);
          if (a.b2 != nullptr) {
            acc0 += __ldg(a.b2 + static_cast<size_t>(e) * a.H + h);
            acc1 += __ldg(a.b2 + static_cast<size_t>(e) * a.H + h + 1);
          }
          y0 = w_on_input ? acc0 : acc0 * s_gam[p];
          y1 = w_on_input ? acc1 : acc1 * s_gam[p];
          if (a.round_pair) {
            y0 = __half2float(__float2half_rn(y0));
            y1 = __half2float(__float2half_rn(y1));
          }
        }
        if (no_combine) {
          if (lane == 0) {
            out[static_cast<size_t>(p) * a.H + h] = __float2half_rn(y0);
            out[static_cast<size_t>(p) * a.H + h + 1] = __float2half_rn(y1);
          }
        } else {
          sum0 += y0;
          sum1 += y1;
        }
      }
      if (!no_combine && lane == 0) {
        out[static_cast<size_t>(t) * a.H + h] = __float2half_rn(sum0 * a.routed_scaling);
        out[static_cast<size_t>(t) * a.H + h + 1] = __float2half_rn(sum1 * a.routed_scaling);
      }
    }
  }
}

size_t routing_smem() { return kGemvMaxPairs * 12 + 2 * 2 * (kDownThreads / 32) * 4 + 64; }   // tables + partial sums

// resident CTAs per SM times SMs, but no more CTAs per SM than the work has warps for: the grid
// stays a multiple of the SM count, so every SM streams the same share of the weights
template <typename K>
unsigned grid_for(K kernel, size_t smem, int threads, long long items, int num_sms) {
  int per_sm = 1;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, smem) != cudaSuccess || per_sm < 1)
    per_sm = 1;
  const long long warps_per_cta = threads / 32;
  const long long need_per_sm = (items + warps_per_cta * num_sms - 1) / (warps_per_cta * num_sms);
  if (per_sm > need_per_sm) per_sm = static_cast<int>(need_per_sm < 1 ? 1 : need_per_sm);
  return static_cast<unsigned>(per_sm) * static_cast<unsigned>(num_sms);
}

template <typename K>
int launch_up(K kernel, const GemvArgs& a, int num_sms, cudaStream_t stream, bool pdl) {
  const size_t smem = gemv_up_smem(a);
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
    return B200MOE_ERR_CUDA;
  const unsigned grid = grid_for(kernel, smem, kUpThreads, static_cast<long long>(a.M) * a.topk * a.I, num_sms);
  note_launch(a.w4 ? "moe_gemv_w4_up_kernel<gate/up>" : "moe_gemv_up_kernel<gate/up>");
  return launch_kernel(kernel, dim3(grid), dim3(kUpThreads), smem, stream, pdl, a) == cudaSuccess ? B200MOE_OK
                                                                                                  : B200MOE_ERR_CUDA;
}
template <typename K>
int launch_down(K kernel, const GemvArgs& a, int num_sms, cudaStream_t stream, bool pdl) {
  const size_t smem = gemv_down_smem(a);
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
    return B200MOE_ERR_CUDA;
  // few output elements (short hidden size): several warps share one, so that every SM still has 16
  // warps' worth of loads in flight
  GemvArgs b = a;
  const long long tasks = static_cast<long long>(a.M) * (a.H / 2);
  const long long all_warps = static_cast<long long>(num_sms) * (kDownThreads / 32);
  b.down_split = 1;
  while (b.down_split < 8 && tasks * b.down_split * 2 <= all_warps) b.down_split *= 2;
  const unsigned grid = grid_for(kernel, smem, kDownThreads, tasks * b.down_split, num_sms);
  note_launch(a.w4 ? "moe_gemv_w4_down_kernel<down>" : "moe_gemv_down_kernel<down>");
  return launch_kernel(kernel, dim3(grid), dim3(kDownThreads), smem, stream, pdl, b) == cudaSuccess ? B200MOE_OK
                                                                                                    : B200MOE_ERR_CUDA;
}

}  // namespace

size_t gemv_up_smem(const GemvArgs& a) {
  return (a.w4 ? staged_w4_bytes(a.M, a.H) : static_cast<size_t>(a.M) * a.H * 4) + routing_smem();
}
size_t gemv_down_smem(const GemvArgs& a) {
  return (a.w4 ? staged_w4_bytes(a.M * a.topk, a.I) : static_cast<size_t>(a.M) * a.topk * a.I * 4) + routing_smem();
}
bool gemv_fits(const GemvArgs& a) {
  return a.M * a.topk <= kGemvMaxPairs && gemv_up_smem(a) + 1024 <= kSmemLimit && gemv_down_smem(a) + 1024 <= kSmemLimit;
}

int launch_gemv_up(const GemvArgs& a, int num_sms, cudaStream_t stream, bool pdl) {
  if (!gemv_fits(a)) return B200MOE_ERR_UNSUPPORTED;
  if (a.w4) return launch_up(moe_gemv_w4_up_kernel, a, num_sms, stream, pdl);
  const int chunks = (a.H + kChunk - 1) / kChunk;
  const bool bf = a.dtype == B200MOE_DTYPE_BF16;
  if (chunks == 5)
    return bf ? launch_up(moe_gemv_up_kernel<__nv_bfloat16, 5>, a, num_sms, stream, pdl)
              : launch_up(moe_gemv_up_kernel<__half, 5>, a, num_sms, stream, pdl);
  if (chunks == 6)
    return bf ? launch_up(moe_gemv_up_kernel<__nv_bfloat16, 6>, a, num_sms, stream, pdl)
              : launch_up(moe_gemv_up_kernel<__half, 6>, a, num_sms, stream, pdl);
  return bf ? launch_up(moe_gemv_up_kernel<__nv_bfloat16, 4>, a, num_sms, stream, pdl)
            : launch_up(moe_gemv_up_kernel<__half, 4>, a, num_sms, stream, pdl);
}
int launch_gemv_down(const GemvArgs& a, int num_sms, cudaStream_t stream, bool pdl) {
  if (!gemv_fits(a)) return B200MOE_ERR_UNSUPPORTED;
  if (a.w4) return launch_down(moe_gemv_w4_down_kernel, a, num_sms, stream, pdl);
  return a.dtype == B200MOE_DTYPE_BF16 ? launch_down(moe_gemv_down_kernel<__nv_bfloat16>, a, num_sms, stream, pdl)
                                       : launch_down(moe_gemv_down_kernel<__half>, a, num_sms, stream, pdl);
}

}  // namespace b200moe
