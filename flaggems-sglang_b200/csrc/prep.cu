// Row movers around the grouped GEMMs: gather token rows into expert-sorted,
// block-padded order (optionally quantising them to FP8 per 1x128 group),
// and turn the fp32 combine buffer into the 16-bit output.
#include "prep.cuh"

namespace b200moe {

namespace {

// One thread per 16-byte chunk of a padded row (grid-stride), so that a handful of rows at
// decode sizes still spreads over many threads.  Rows beyond meta[1] are left alone, padding
// rows are zero-filled.  The same launch clears the fp32 combine buffer (`zero`, `zero_chunks`).
// With sc_src: the rows are already quantised (one byte per element) and each has G group scales
// [tokens][G]; they are re-laid group-major for the GEMMs, sc_dst [G][ld].
__global__ void __launch_bounds__(256)
gather_rows_kernel(const uint4* __restrict__ x, uint4* __restrict__ xs, const int* __restrict__ sorted_ids,
                   const int* __restrict__ meta, int P, int topk, int chunks_per_row, int cap,
                   uint4* __restrict__ zero, long long zero_chunks, const float* __restrict__ sc_src,
                   float* __restrict__ sc_dst, int G, int ld, const FlagWait fw) {
  griddep_wait();
  griddep_launch_dependents();
  wait_for_peers(fw);     // expert parallelism: the rows come from the peers
  const int rows = min(meta[1], cap);
  const long long n_copy = static_cast<long long>(rows) * chunks_per_row;
  const long long total = n_copy + zero_chunks;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  if (sc_src != nullptr) {
    const long long n_sc = static_cast<long long>(rows) * G;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_sc; i += stride) {
      const int g = static_cast<int>(i / rows);
      const int r = static_cast<int>(i - static_cast<long long>(g) * rows);
      const int slot = sorted_ids[r];
      sc_dst[static_cast<size_t>(g) * ld + r] =
          (slot >= 0 && slot < P) ? __ldg(sc_src + static_cast<size_t>(slot / topk) * G + g) : 1.0f;
    }
  }
  // four chunks per thread and trip: first the four row ids, then the four loads, then the stores
  for (long long i0 = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < total; i0 += 4 * stride) {
    int slot[4];
    int col[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long i = i0 + u * stride;
      slot[u] = -1;
      col[u] = 0;
      if (i < n_copy) {
        const int r = static_cast<int>(i / chunks_per_row);
        col[u] = static_cast<int>(i - static_cast<long long>(r) * chunks_per_row);
        slot[u] = sorted_ids[r];
      }
    }
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      v[u] = make_uint4(0, 0, 0, 0);
      if (slot[u] >= 0 && slot[u] < P) v[u] = __ldg(x + static_cast<size_t>(slot[u] / topk) * chunks_per_row + col[u]);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long i = i0 + u * stride;
      if (i < n_copy) xs[i] = v[u];
      else if (i < total) zero[i - n_copy] = make_uint4(0, 0, 0, 0);
    }
  }
}

template <typename T>
__device__ __forceinline__ void load4(const T* p, float (&v)[4]);
template <>
__device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[4]) {
  uint2 raw = *reinterpret_cast<const uint2*>(p);
  __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162*>(&raw.x);
  __nv_bfloat162 b = *reinterpret_cast<__nv_bfloat162*>(&raw.y);
  v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
}
template <>
__device__ __forceinline__ void load4<__half>(const __half* p, float (&v)[4]) {
  uint2 raw = *reinterpret_cast<const uint2*>(p);
  __half2 a = *reinterpret_cast<__half2*>(&raw.x);
  __half2 b = *reinterpret_cast<__half2*>(&raw.y);
  v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
}

// One warp per (row, run of up to eight 128-wide groups): the loads of the run are issued
// together (one 8-byte load per lane and group in flight is too little to cover the memory
// latency), then per group amax by shuffles, scale = max(amax, eps)/448,
// q = rne_satfinite(x / scale) with an IEEE divide so that the bits match a CPU restatement.
// sorted_ids == nullptr: rows map to themselves.
// scale_t != 0: scales stored [K/128][ld_scale] (group-major) instead of [rows][K/128].
template <typename T>
__global__ void __launch_bounds__(256)
group_quant_fp8_kernel(const T* __restrict__ x, uint8_t* __restrict__ q, float* __restrict__ scales,
                       const int* __restrict__ sorted_ids, const int* __restrict__ meta, int P, int topk,
                       int n_rows_static, int K, int scale_t, int ld_scale, uint4* __restrict__ zero,
                       long long zero_chunks) {
  griddep_wait();
  griddep_launch_dependents();
  // clear the fp32 combine buffer alongside (grid-stride, 16 bytes per thread)
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < zero_chunks;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    zero[i] = make_uint4(0, 0, 0, 0);
  constexpr int RUN = 8;
  const int groups = K >> 7;
  const int runs = (groups + RUN - 1) / RUN;
  const int lane = threadIdx.x & 31;
  const int rows = (meta != nullptr) ? min(meta[1], n_rows_static) : n_rows_static;
  const long long total = static_cast<long long>(rows) * runs;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  for (long long w = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; w < total;
       w += warps) {
    const int r = static_cast<int>(w / runs);
    const int g0 = static_cast<int>(w - static_cast<long long>(r) * runs) * RUN;
    int src_row = r;
    bool pad = false;
    if (sorted_ids != nullptr) {
      int slot = sorted_ids[r];
      pad = (slot < 0 || slot >= P);
      src_row = pad ? 0 : slot / topk;
    }
    float v[RUN][4];
#pragma unroll
    for (int u = 0; u < RUN; ++u) {
      v[u][0] = v[u][1] = v[u][2] = v[u][3] = 0.f;
      if (!pad && g0 + u < groups) load4<T>(x + static_cast<size_t>(src_row) * K + (g0 + u) * 128 + lane * 4, v[u]);
    }
#pragma unroll
    for (int u = 0; u < RUN; ++u) {
      const int g = g0 + u;
      if (g >= groups) break;
      float amax = fmaxf(fmaxf(fabsf(v[u][0]), fabsf(v[u][1])), fmaxf(fabsf(v[u][2]), fabsf(v[u][3])));
      // non-negative floats order like their bit patterns: one redux instead of five shuffles
      amax = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(amax)));
      const float s = __fdiv_rn(fmaxf(amax, 1e-10f), 448.0f);
      uint32_t packed = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        __nv_fp8_storage_t b = __nv_cvt_float_to_fp8(__fdiv_rn(v[u][i], s), __NV_SATFINITE, __NV_E4M3);
        packed |= static_cast<uint32_t>(b) << (8 * i);
      }
      *reinterpret_cast<uint32_t*>(q + static_cast<size_t>(r) * K + g * 128 + lane * 4) = packed;
      if (lane == 0) {
        if (scale_t) scales[static_cast<size_t>(g) * ld_scale + r] = s;
        else scales[static_cast<size_t>(r) * groups + g] = s;
      }
    }
  }
}

// One warp per (padded row, 128-wide group): see launch_group_split_i8.
__global__ void __launch_bounds__(256)
group_split_i8_kernel(const __half* __restrict__ x, uint8_t* __restrict__ planes, float* __restrict__ scales,
                      int* __restrict__ sums, const int* __restrict__ sorted_ids, const int* __restrict__ meta,
                      int P, int topk, int cap, int K, int BT, int ld, uint4* __restrict__ zero,
                      long long zero_chunks) {
  griddep_wait();
  griddep_launch_dependents();
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < zero_chunks;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    zero[i] = make_uint4(0, 0, 0, 0);
  const int groups = K >> 7;
  const int lane = threadIdx.x & 31;
  const int rows = min(meta[1], cap);
  const long long total = static_cast<long long>(rows) * groups;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const size_t plane_stride = static_cast<size_t>(BT) * K;
  for (long long w = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; w < total; w += warps) {
    const int r = static_cast<int>(w / groups), g = static_cast<int>(w - static_cast<long long>(r) * groups);
    const int slot = sorted_ids[r];
    const bool pad = (slot < 0 || slot >= P);
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (!pad) load4<__half>(x + static_cast<size_t>(slot / topk) * K + g * 128 + lane * 4, v);
    const float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
    const unsigned int mb = __reduce_max_sync(0xffffffffu, __float_as_uint(amax));
    // group maximum in [2^ex, 2^(ex+1)): x * 2^(18-ex) has magnitude below 2^19
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
    const int xsum = __reduce_add_sync(0xffffffffu, part);
    // an even lane holds elements 0..3 of its run of eight, the odd neighbour 4..7; stored
    // order is (0, 4, 1, 5 | 2, 6, 3, 7)
    uint8_t* dst = planes + (static_cast<size_t>(r / BT) * 3) * plane_stride + static_cast<size_t>(r % BT) * K +
                   g * 128 + lane * 4;
#pragma unroll
    for (int p = 0; p < 3; ++p) {
      const uint32_t other = __shfl_xor_sync(0xffffffffu, pk[p], 1);
      const uint32_t word = (lane & 1) ? __byte_perm(pk[p], other, 0x3726) : __byte_perm(pk[p], other, 0x5140);
      *reinterpret_cast<uint32_t*>(dst + p * plane_stride) = word;
    }
    if (lane == 0) {
      scales[static_cast<size_t>(g) * ld + r] = f;
      sums[static_cast<size_t>(g) * ld + r] = xsum;
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
finalize_kernel(const float4* __restrict__ acc, T* __restrict__ out, size_t n4, float scale, const FlagWait fw) {
  griddep_wait();
  griddep_launch_dependents();
  wait_for_peers(fw);
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    float4 v = acc[i];
    T o[4] = {from_f32<T>(v.x * scale), from_f32<T>(v.y * scale), from_f32<T>(v.z * scale),
              from_f32<T>(v.w * scale)};
    *reinterpret_cast<uint2*>(out + i * 4) = *reinterpret_cast<uint2*>(o);
  }
}

// One thread per (token, run of 8 columns): fp32 sum of the token's valid pair rows.
template <typename T>
__global__ void __launch_bounds__(256)
finalize_pairs_kernel(const uint4* __restrict__ pairs, const uint8_t* __restrict__ pair_valid, uint4* __restrict__ out,
                      int M, int topk, int chunks_per_row, float scale, const FlagWait fw) {
  griddep_wait();
  griddep_launch_dependents();
  wait_for_peers(fw);
  const long long total = static_cast<long long>(M) * chunks_per_row;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(i / chunks_per_row);
    const int c = static_cast<int>(i - static_cast<long long>(t) * chunks_per_row);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    // four pairs at a time: the validity bytes first, then the row chunks, so that the loads of a
    // batch are in flight together
    for (int j0 = 0; j0 < topk; j0 += 4) {
      uint4 v[4];
      bool ok[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const size_t slot = static_cast<size_t>(t) * topk + j0 + u;
        ok[u] = (j0 + u < topk) && pair_valid[slot] != 0;
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const size_t slot = static_cast<size_t>(t) * topk + j0 + u;
        v[u] = ok[u] ? __ldg(pairs + slot * chunks_per_row + c) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const T* e = reinterpret_cast<const T*>(&v[u]);
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[k] += to_f32<T>(e[k]);   // zeros for pairs that are not there
      }
    }
    T o[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) o[k] = from_f32<T>(acc[k] * scale);
    out[i] = *reinterpret_cast<uint4*>(o);
  }
}

}  // namespace

int launch_finalize_pairs(const void* pairs, const uint8_t* pair_valid, void* out, int dtype, int M, int topk,
                          int H, float scale, int num_sms, cudaStream_t stream, bool pdl, const FlagWait* wait) {
  FlagWait fw = {};
  if (wait != nullptr) fw = *wait;
  if (H % 8 != 0) return B200MOE_ERR_UNSUPPORTED;
  const long long total = static_cast<long long>(M) * (H / 8);
  long long ctas = (total + 255) / 256;
  if (ctas > static_cast<long long>(num_sms) * 16) ctas = static_cast<long long>(num_sms) * 16;
  if (ctas < 1) ctas = 1;
  cudaError_t err;
  note_launch("finalize_pairs_kernel");
  if (dtype == B200MOE_DTYPE_BF16)
    err = launch_kernel(finalize_pairs_kernel<__nv_bfloat16>, dim3(static_cast<unsigned>(ctas)), dim3(256), 0, stream,
                        pdl, reinterpret_cast<const uint4*>(pairs), pair_valid, reinterpret_cast<uint4*>(out), M, topk,
                        H / 8, scale, fw);
  else
    err = launch_kernel(finalize_pairs_kernel<__half>, dim3(static_cast<unsigned>(ctas)), dim3(256), 0, stream, pdl,
                        reinterpret_cast<const uint4*>(pairs), pair_valid, reinterpret_cast<uint4*>(out), M, topk, H / 8,
                        scale, fw);
  return err == cudaSuccess ? B200MOE_OK : B200MOE_ERR_CUDA;
}

int launch_gather_rows(const void* x, void* xs, const int* sorted_ids, const int* meta, int P, int topk,
                       int row_bytes, int cap, void* zero, size_t zero_bytes, int num_sms,
                       cudaStream_t stream, bool pdl, const float* sc_src, float* sc_dst, int G, int ld,
                       const FlagWait* wait) {
  FlagWait fw = {};
  if (wait != nullptr) fw = *wait;
  if (row_bytes % 16 != 0 || zero_bytes % 16 != 0) return B200MOE_ERR_UNSUPPORTED;
  const long long work = static_cast<long long>(cap) * (row_bytes / 16) + static_cast<long long>(zero_bytes / 16);
  long long ctas = (work + 255) / 256;
  if (ctas > static_cast<long long>(num_sms) * 8) ctas = static_cast<long long>(num_sms) * 8;
  if (ctas < 1) ctas = 1;
  note_launch("gather_rows_kernel");
  cudaError_t err = launch_kernel(gather_rows_kernel, dim3(static_cast<unsigned>(ctas)), dim3(256), 0, stream, pdl,
                                  reinterpret_cast<const uint4*>(x), reinterpret_cast<uint4*>(xs), sorted_ids, meta,
                                  P, topk, row_bytes / 16, cap, reinterpret_cast<uint4*>(zero),
                                  static_cast<long long>(zero_bytes / 16), sc_src, sc_dst, G, ld, fw);
  return err == cudaSuccess ? B200MOE_OK : B200MOE_ERR_CUDA;
}

int launch_group_quant_fp8(const void* x, int dtype, void* q, float* scales, const int* sorted_ids,
                           const int* meta, int P, int topk, int rows, int K, int scale_t, int ld_scale,
                           void* zero, size_t zero_bytes, int num_sms, cudaStream_t stream, bool pdl) {
  if (K % 128 != 0 || zero_bytes % 16 != 0) return B200MOE_ERR_UNSUPPORTED;
  long long warps = static_cast<long long>(rows) * ((K / 128 + 7) / 8);
  long long ctas = (warps + 7) / 8;
  if (ctas > num_sms * 16) ctas = num_sms * 16;
  if (ctas < 1) ctas = 1;
  cudaError_t err;
  const long long zc = static_cast<long long>(zero_bytes / 16);
  note_launch("group_quant_fp8_kernel");
  if (dtype == B200MOE_DTYPE_BF16)
    err = launch_kernel(group_quant_fp8_kernel<__nv_bfloat16>, dim3(static_cast<unsigned>(ctas)), dim3(256), 0, stream,
                        pdl, reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<uint8_t*>(q), scales,
                        sorted_ids, meta, P, topk, rows, K, scale_t, ld_scale, reinterpret_cast<uint4*>(zero), zc);
  else
    err = launch_kernel(group_quant_fp8_kernel<__half>, dim3(static_cast<unsigned>(ctas)), dim3(256), 0, stream, pdl,
                        reinterpret_cast<const __half*>(x), reinterpret_cast<uint8_t*>(q), scales, sorted_ids, meta, P,
                        topk, rows, K, scale_t, ld_scale, reinterpret_cast<uint4*>(zero), zc);
  return err == cudaSuccess ? B200MOE_OK : B200MOE_ERR_CUDA;
}

int launch_group_split_i8(const void* x, uint8_t* planes, float* scales, int* sums, const int* sorted_ids,
                          const int* meta, int P, int topk, int cap, int K, int BT, int ld, void* zero,
                          size_t zero_bytes, int num_sms, cudaStream_t stream, bool pdl) {
  if (K % 128 != 0 || zero_bytes % 16 != 0 || BT <= 0 || cap % BT != 0) return B200MOE_ERR_UNSUPPORTED;
  long long warps = static_cast<long long>(cap) * (K / 128);
  long long ctas = (warps + 7) / 8;
  if (ctas > num_sms * 16) ctas = num_sms * 16;
  if (ctas < 1) ctas = 1;
  note_launch("group_split_i8_kernel");
  cudaError_t err = launch_kernel(group_split_i8_kernel, dim3(static_cast<unsigned>(ctas)), dim3(256), 0, stream, pdl,
                                  reinterpret_cast<const __half*>(x), planes, scales, sums, sorted_ids, meta, P, topk,
                                  cap, K, BT, ld, reinterpret_cast<uint4*>(zero),
                                  static_cast<long long>(zero_bytes / 16));
  return err == cudaSuccess ? B200MOE_OK : B200MOE_ERR_CUDA;
}

int launch_finalize(const float* acc, void* out, int dtype, size_t n, float scale, int num_sms,
                    cudaStream_t stream, bool pdl, const FlagWait* wait) {
  FlagWait fw = {};
  if (wait != nullptr) fw = *wait;
  if (n % 4 != 0) return B200MOE_ERR_UNSUPPORTED;
  size_t n4 = n / 4;
  size_t ctas = (n4 + 255) / 256;
  if (ctas > static_cast<size_t>(num_sms) * 8) ctas = static_cast<size_t>(num_sms) * 8;
  if (ctas < 1) ctas = 1;
  cudaError_t err;
  note_launch("finalize_kernel");
  if (dtype == B200MOE_DTYPE_BF16)
    err = launch_kernel(finalize_kernel<__nv_bfloat16>, dim3(static_cast<unsigned>(ctas)), dim3(256), 0, stream, pdl,
                        reinterpret_cast<const float4*>(acc), reinterpret_cast<__nv_bfloat16*>(out), n4, scale, fw);
  else
    err = launch_kernel(finalize_kernel<__half>, dim3(static_cast<unsigned>(ctas)), dim3(256), 0, stream, pdl,
                        reinterpret_cast<const float4*>(acc), reinterpret_cast<__half*>(out), n4, scale, fw);
  return err == cudaSuccess ? B200MOE_OK : B200MOE_ERR_CUDA;
}

}  // namespace b200moe
