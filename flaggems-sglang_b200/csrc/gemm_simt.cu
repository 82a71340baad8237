// Plain CUDA-core versions of the two grouped GEMMs, one CTA per padded row.
// Slow; they exist to validate the routing tables and the fused tails separately
// from the tensor-core pipeline (B200MOE_FLAG_SIMT).  16-bit weights, layer layout.
#include "gemm_sched.cuh"

namespace b200moe {

namespace {

template <int MODE, typename T>
__global__ void __launch_bounds__(256)
moe_gemm_simt_kernel(const T* __restrict__ w, const T* __restrict__ x, const GemmArgs a) {
  const int rows = a.meta[1];
  const int r = blockIdx.x;
  if (r >= rows) return;
  const int blk = r / a.BT;
  int lo = 0, hi = a.E;
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (a.blk_off[mid] <= blk) lo = mid; else hi = mid;
  }
  const int e = lo;
  const int slot = a.sorted_ids[r];
  const bool valid = slot >= 0 && slot < a.P;
  const float gam = valid ? a.row_gamma[r] : 0.f;
  const bool w_on_input = (a.flags & B200MOE_FLAG_WEIGHT_ON_INPUT) != 0;
  const bool mimic = (a.flags & B200MOE_FLAG_MIMIC_ROUNDING) != 0;
  const T* xr = x + static_cast<size_t>(r) * a.K;
  const size_t rows_per_expert = (MODE == 0) ? 2 * static_cast<size_t>(a.N) : static_cast<size_t>(a.N);
  const T* we = w + static_cast<size_t>(e) * rows_per_expert * a.K;
  for (int n = threadIdx.x; n < a.N; n += blockDim.x) {
    float g = 0.f, u = 0.f;
    const T* wg = we + static_cast<size_t>(n) * a.K;
    const T* wu = we + static_cast<size_t>(a.up_row_off + n) * a.K;
    for (int k = 0; k < a.K; ++k) {
      const float xv = to_f32<T>(xr[k]);
      g += xv * to_f32<T>(wg[k]);
      if (MODE == 0) u += xv * to_f32<T>(wu[k]);
    }
    if (MODE == 0) {
      if (a.bias != nullptr) {
        g += a.bias[static_cast<size_t>(e) * 2 * a.N + n];
        u += a.bias[static_cast<size_t>(e) * 2 * a.N + a.N + n];
      }
      const float av = act_mul<T, true>(g, u, w_on_input, gam, mimic, act_params(a));
      reinterpret_cast<T*>(a.out)[static_cast<size_t>(r) * a.ld_out + n] = from_f32<T>(av);
    } else if (valid) {
      float y = g + (a.bias != nullptr ? a.bias[static_cast<size_t>(e) * a.N + n] : 0.f);
      if (!w_on_input) y *= gam;
      if (mimic) y = to_f32<T>(from_f32<T>(y));
      atomicAdd(reinterpret_cast<float*>(a.out) + static_cast<size_t>(slot / a.topk) * a.ld_out + n, y);
    }
  }
}

}  // namespace

int launch_gemm_simt(const void* w, const void* x, const GemmArgs& a, cudaStream_t stream, int cap) {
  if (a.wmode != B200MOE_W_16BIT) return B200MOE_ERR_UNSUPPORTED;
  if (cap <= 0) return B200MOE_OK;
  note_launch("moe_gemm_simt_kernel");
  if (a.dtype == B200MOE_DTYPE_BF16) {
    const __nv_bfloat16* wp = reinterpret_cast<const __nv_bfloat16*>(w);
    const __nv_bfloat16* xp = reinterpret_cast<const __nv_bfloat16*>(x);
    if (a.mode == 0) moe_gemm_simt_kernel<0, __nv_bfloat16><<<cap, 256, 0, stream>>>(wp, xp, a);
    else moe_gemm_simt_kernel<1, __nv_bfloat16><<<cap, 256, 0, stream>>>(wp, xp, a);
  } else {
    const __half* wp = reinterpret_cast<const __half*>(w);
    const __half* xp = reinterpret_cast<const __half*>(x);
    if (a.mode == 0) moe_gemm_simt_kernel<0, __half><<<cap, 256, 0, stream>>>(wp, xp, a);
    else moe_gemm_simt_kernel<1, __half><<<cap, 256, 0, stream>>>(wp, xp, a);
  }
  return cudaGetLastError() == cudaSuccess ? B200MOE_OK : B200MOE_ERR_CUDA;
}

}  // namespace b200moe
