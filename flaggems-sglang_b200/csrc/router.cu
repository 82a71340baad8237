// Router front-end: gating logits -> (topk_weights, topk_ids), the step right before the
// block alignment.  One warp per token; the token's E scores sit in shared memory, the
// selection is k rounds of a warp-wide arg-max (larger key first, lower expert id on ties).
//
//   softmax scoring   p_e = exp(l_e - max l) / sum; the k largest.  Without a selection bias the
//                     ranking runs on the raw logits (softmax is monotone), so the ids do not
//                     depend on how exp() rounds.
//   sigmoid scoring   s_e = 1 / (1 + exp(-l_e)).
//   selection bias    key_e = score_e + bias_e ranks the experts; the weights stay score_e.
//   expert groups     the E experts form n_group contiguous groups; only the topk_group best
//                     groups stay eligible.  A group's score is its largest key, or, with a
//                     selection bias, the sum of its two largest keys (the DeepSeek-V3 rule).
//   renormalise       weights divided by their sum; then multiplied by `scale`.
#include "router.cuh"

namespace b200moe {

namespace {

constexpr int kRouterWarps = 4;
#define kNegInf (__int_as_float(0xff800000))   // -inf

template <typename TL>
__device__ __forceinline__ float logit_f32(const TL* p, size_t i);
template <>
__device__ __forceinline__ float logit_f32<float>(const float* p, size_t i) { return p[i]; }
template <>
__device__ __forceinline__ float logit_f32<__nv_bfloat16>(const __nv_bfloat16* p, size_t i) {
  return __bfloat162float(p[i]);
}
template <>
__device__ __forceinline__ float logit_f32<__half>(const __half* p, size_t i) { return __half2float(p[i]); }

// (value, index) arg-max across the warp: larger value wins, equal values -> smaller index.
__device__ __forceinline__ void warp_argmax(float& v, int& idx) {
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, d);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, d);
    if (ov > v || (ov == v && oi < idx)) {
      v = ov;
      idx = oi;
    }
  }
}

template <typename TL>
__global__ void __launch_bounds__(kRouterWarps * 32)
route_topk_kernel(const TL* __restrict__ logits, const float* __restrict__ bias, int M, int E, int topk,
                  int scoring, int renorm, int n_group, int topk_group, float scale,
                  float* __restrict__ out_w, int* __restrict__ out_ids) {
  extern __shared__ float rsm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* s_score = rsm + static_cast<size_t>(warp) * 2 * E;   // weight numerators
  float* s_key = s_score + E;                                  // selection keys
  const int gsize = n_group > 1 ? E / n_group : E;

  for (int t = blockIdx.x * kRouterWarps + warp; t < M; t += gridDim.x * kRouterWarps) {
    const size_t base = static_cast<size_t>(t) * E;
    float denom = 1.0f;
    if (scoring == B200MOE_SCORE_SOFTMAX) {
      float mx = kNegInf;
      for (int e = lane; e < E; e += 32) {
        const float l = logit_f32<TL>(logits, base + e);
        s_key[e] = l;
        mx = fmaxf(mx, l);
      }
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, d));
      float sum = 0.f;
      for (int e = lane; e < E; e += 32) {
        const float p = expf(s_key[e] - mx);
        s_score[e] = p;
        sum += p;
      }
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
      denom = sum;
      if (bias != nullptr)
        for (int e = lane; e < E; e += 32) s_key[e] = __fdiv_rn(s_score[e], sum) + bias[e];
    } else {
      for (int e = lane; e < E; e += 32) {
        const float s = __fdiv_rn(1.0f, 1.0f + expf(-logit_f32<TL>(logits, base + e)));
        s_score[e] = s;
        s_key[e] = s + (bias != nullptr ? bias[e] : 0.f);
      }
    }
    __syncwarp();

    if (n_group > 1) {
      // lane g scores group g, then topk_group rounds pick the groups that stay eligible
      float gs = kNegInf;
      if (lane < n_group) {
        float m1 = kNegInf, m2 = kNegInf;
        for (int i = 0; i < gsize; ++i) {
          const float v = s_key[lane * gsize + i];
          if (v > m1) {
            m2 = m1;
            m1 = v;
          } else if (v > m2) {
            m2 = v;
          }
        }
        gs = (bias != nullptr && gsize > 1) ? m1 + m2 : m1;
      }
      uint32_t keep = 0;
      for (int j = 0; j < topk_group; ++j) {
        float v = gs;
        int gi = lane;
        warp_argmax(v, gi);
        keep |= 1u << gi;
        if (lane == gi) gs = kNegInf;
      }
      for (int e = lane; e < E; e += 32)
        if (!((keep >> (e / gsize)) & 1u)) s_key[e] = kNegInf;
      __syncwarp();
    }

    // k rounds of arg-max; lane j keeps the j-th pick (topk <= 32)
    float my_w = 0.f;
    int my_id = 0;
    for (int j = 0; j < topk; ++j) {
      float v = kNegInf;
      int idx = 0x7fffffff;
      for (int e = lane; e < E; e += 32) {
        const float k = s_key[e];
        if (k > v) {   // ascending e: the first of equal keys stays
          v = k;
          idx = e;
        }
      }
      warp_argmax(v, idx);
      if (idx >= E) idx = 0;   // every remaining key was -inf or NaN
      if (lane == j) {
        my_w = s_score[idx];
        my_id = idx;
      }
      __syncwarp();
      if (lane == 0) s_key[idx] = kNegInf;
      __syncwarp();
    }
    // softmax probabilities divide by the full sum first, as the unfused recipe does
    if (scoring == B200MOE_SCORE_SOFTMAX) my_w = __fdiv_rn(my_w, denom);
    if (renorm) {
      float part = lane < topk ? my_w : 0.f;
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) part += __shfl_xor_sync(0xffffffffu, part, d);
      my_w = __fdiv_rn(my_w, part);
    }
    my_w *= scale;
    if (lane < topk) {
      out_ids[static_cast<size_t>(t) * topk + lane] = my_id;
      out_w[static_cast<size_t>(t) * topk + lane] = my_w;
    }
    __syncwarp();
  }
}

}  // namespace

int check_router(const b200moe_router* r, int E, int topk) {
  if (r == nullptr || r->struct_bytes != static_cast<int32_t>(sizeof(b200moe_router))) return B200MOE_ERR_BAD_ARG;
  if (r->scoring != B200MOE_SCORE_SOFTMAX && r->scoring != B200MOE_SCORE_SIGMOID) return B200MOE_ERR_BAD_ARG;
  if (r->logits_dtype < 0 || r->logits_dtype > B200MOE_DTYPE_FP32) return B200MOE_ERR_BAD_ARG;
  if (E <= 0 || topk <= 0 || topk > E) return B200MOE_ERR_BAD_ARG;
  if (topk > B200MOE_ROUTER_MAX_TOPK) return B200MOE_ERR_TOO_LARGE;
  if (E > B200MOE_ROUTER_MAX_EXPERTS) return B200MOE_ERR_TOO_LARGE;
  if (r->n_group > 1) {
    if (r->n_group > 32 || E % r->n_group != 0) return B200MOE_ERR_UNSUPPORTED;
    if (r->topk_group <= 0 || r->topk_group > r->n_group) return B200MOE_ERR_BAD_ARG;
    if (topk > r->topk_group * (E / r->n_group)) return B200MOE_ERR_BAD_ARG;
  }
  return B200MOE_OK;
}

int launch_route_topk(const b200moe_router* r, const void* logits, int M, int E, int topk, float* out_w,
                      int* out_ids, int num_sms, cudaStream_t stream) {
  int rc = check_router(r, E, topk);
  if (rc != B200MOE_OK) return rc;
  if (M == 0) return B200MOE_OK;
  if (logits == nullptr || out_w == nullptr || out_ids == nullptr) return B200MOE_ERR_BAD_ARG;
  int ctas = (M + kRouterWarps - 1) / kRouterWarps;
  if (ctas > num_sms * 8) ctas = num_sms * 8;
  const size_t smem = static_cast<size_t>(kRouterWarps) * 2 * E * sizeof(float);
  const float scale = r->scale == 0.f ? 1.0f : r->scale;
  cudaError_t err;
  note_launch("route_topk_kernel");
#define B200MOE_ROUTE(TL)                                                                                     \
  err = launch_kernel(route_topk_kernel<TL>, dim3(ctas), dim3(kRouterWarps * 32), smem, stream, false,          \
                      reinterpret_cast<const TL*>(logits), r->bias, M, E, topk, r->scoring, r->renormalize,     \
                      r->n_group, r->topk_group, scale, out_w, out_ids)
  if (r->logits_dtype == B200MOE_DTYPE_FP32) B200MOE_ROUTE(float);
  else if (r->logits_dtype == B200MOE_DTYPE_BF16) B200MOE_ROUTE(__nv_bfloat16);
  else B200MOE_ROUTE(__half);
#undef B200MOE_ROUTE
  return err == cudaSuccess ? B200MOE_OK : B200MOE_ERR_CUDA;
}

}  // namespace b200moe
