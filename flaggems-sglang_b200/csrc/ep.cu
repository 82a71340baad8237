// Expert parallelism: the kernels that move rows and flags between ranks over peer-mapped memory.
//
// A forward call under expert parallelism is, on every rank,
//   dispatch   this rank's tokens -> the ranks that hold their experts (plain peer stores of the
//              quantised row, its scales and the masked routing entries), then "ready" flags;
//   wait       until every peer's ready flag has arrived;
//   local op   alignment, gather and the two grouped GEMMs over the rows received; the down
//              projection's epilogue stores each pair's weighted row straight into the buffer of
//              the rank that owns the token (gemm.cuh: out_row_base), so the combine needs no
//              collective and overlaps the GEMM;
//   signal     "done" flags to every peer once the GEMM has completed;
//   wait       until every peer is done, then the output conversion sums the rows that arrived.
// Flags are epochs that only grow, so nothing is ever reset while a peer may look at it; each
// wait has a time limit and ends in the status word.  No load ever has a peer's memory as its
// source except these flag polls of the rank's OWN heap: data moves by stores only.
#include "ep.cuh"

namespace b200moe {

namespace {

size_t up256(size_t v) { return (v + 255) / 256 * 256; }

__device__ __forceinline__ void st_release_sys_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

template <typename T>
__device__ __forceinline__ void load4f(const T* p, float (&v)[4]);
template <>
__device__ __forceinline__ void load4f<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[4]) {
  uint2 raw = *reinterpret_cast<const uint2*>(p);
  __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162*>(&raw.x);
  __nv_bfloat162 b = *reinterpret_cast<__nv_bfloat162*>(&raw.y);
  v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
}
template <>
__device__ __forceinline__ void load4f<__half>(const __half* p, float (&v)[4]) {
  uint2 raw = *reinterpret_cast<const uint2*>(p);
  __half2 a = *reinterpret_cast<__half2*>(&raw.x);
  __half2 b = *reinterpret_cast<__half2*>(&raw.y);
  v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
}

constexpr int kDispatchWarps = 4;
// staging of one quantised row: H bytes + H/128 scales
__host__ __device__ inline size_t ep_stage_bytes(int H) { return static_cast<size_t>(H) + (((H >> 7) * 4 + 15) & ~15); }

// Where does expert choice `lane` of token i live?  (dr = rank, lid = local expert, w = routing weight;
// dr = -1: not a choice of this token, or an expert held nowhere)
__device__ __forceinline__ void ep_route(const EpDispatchArgs& a, int i, int lane, int& dr, int& lid, float& w) {
  dr = -1;
  lid = -1;
  w = 0.f;
  if (i < a.m && lane < a.topk) {
    const long long gid = a.ids_i64 ? reinterpret_cast<const long long*>(a.topk_ids)[static_cast<size_t>(i) * a.topk + lane]
                                    : reinterpret_cast<const int*>(a.topk_ids)[static_cast<size_t>(i) * a.topk + lane];
    if (gid >= 0 && gid < a.n_global_experts) {
      const int pl = a.placement[gid];
      if (pl >= 0 && (pl >> 16) < a.world) {
        dr = pl >> 16;
        lid = pl & 0xffff;
        w = a.topk_weights[static_cast<size_t>(i) * a.topk + lane];
      }
    }
  }
}

// One CTA (four warps) per token: the warps share the token's 128-wide groups, so that even a few
// hundred tokens put enough loads in flight, and then copy the staged row to every destination
// together.  Shared memory (FP8 rows): H bytes of quantised row + H/128 scales.
template <typename T>
__global__ void __launch_bounds__(kDispatchWarps * 32)
ep_dispatch_kernel(const EpDispatchArgs a) {
  extern __shared__ __align__(16) uint8_t smem[];
  __shared__ unsigned long long s_epoch;
  __shared__ int s_last;
  griddep_wait();
  griddep_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint8_t* me = a.heap[a.rank];
  const int G = a.H >> 7;

  // ---- pass 1: the routing entries of every token, masked per destination.  Every rank gets a row for
  // every token, so that it never has to guess which rows arrived; they go first and get a flag of
  // their own, so that the receivers' alignment runs while the token rows are still travelling.
  for (int i = blockIdx.x; i < a.m_cap; i += gridDim.x) {
    if (warp != 0) break;
    int dr = -1, lid = -1;
    float w = 0.f;
    ep_route(a, i, lane, dr, lid, w);
    const size_t row = static_cast<size_t>(a.rank) * a.m_cap + i;
    if (lane < a.topk) {
      for (int d = 0; d < a.world; ++d) {
        const bool mine = dr == d;
        reinterpret_cast<int*>(a.heap[d] + a.L.recv_ids)[row * a.topk + lane] = mine ? lid : -1;
        reinterpret_cast<float*>(a.heap[d] + a.L.recv_w)[row * a.topk + lane] = mine ? w : 0.f;
      }
    }
  }
  // the last CTA to get here opens a new epoch and raises "ready" on every peer (each thread's
  // stores are fenced before its CTA is counted)
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned int* cnt = reinterpret_cast<unsigned int*>(me + a.L.flags + kEpFlagCtaCount);
    const unsigned int prev = atomicAdd(cnt, 1u);
    s_last = (prev == gridDim.x - 1) ? 1 : 0;
    if (s_last) {
      *cnt = 0;
      unsigned long long* ep = reinterpret_cast<unsigned long long*>(me + a.L.flags + kEpFlagEpoch);
      s_epoch = *ep + 1;
      *ep = s_epoch;
      __threadfence_system();
    }
  }
  __syncthreads();
  if (s_last && threadIdx.x < a.world)
    st_release_sys_u64(reinterpret_cast<unsigned long long*>(a.heap[threadIdx.x] + a.L.flags + kEpFlagReady) + a.rank,
                       s_epoch);
  __syncthreads();

  // ---- this rank's result buffer starts empty (peers add to it / mark it only after they have seen
  // this rank's "rows" flag, which is raised at the end of this kernel)
  {
    uint4* z = reinterpret_cast<uint4*>(me + (a.clear_pairs ? a.L.pair_valid : a.L.out32));
    const long long n = a.clear_pairs ? (static_cast<long long>(a.m_cap) * a.topk + 15) / 16
                                      : static_cast<long long>(a.m_cap) * a.H / 4;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
         i += static_cast<long long>(gridDim.x) * blockDim.x)
      z[i] = make_uint4(0, 0, 0, 0);
  }

  // ---- pass 2: the token rows, only to the ranks that hold one of the token's experts
  uint8_t* stage = smem;
  float* stage_sc = reinterpret_cast<float*>(stage + a.H);
  for (int i = blockIdx.x; i < a.m; i += gridDim.x) {
    int dr = -1, lid = -1;
    float w = 0.f;
    ep_route(a, i, lane, dr, lid, w);      // every warp looks for itself: 32 bytes of ids
    unsigned dest_mask = 0;
    for (int d = 0; d < a.world; ++d)
      if (__any_sync(0xffffffffu, dr == d)) dest_mask |= 1u << d;
    if (dest_mask == 0) continue;     // the same in every warp of the CTA
    const size_t row = static_cast<size_t>(a.rank) * a.m_cap + i;
    const T* xrow = reinterpret_cast<const T*>(a.x) + static_cast<size_t>(i) * a.H;
    if (a.fp8_rows) {
      // 1x128 quantisation, the arithmetic of group_quant_fp8_kernel (prep.cu) so that a row
      // carries the same bits whether it is quantised here or inside a single-GPU call
      constexpr int RUN = 8;
      for (int g0 = warp * RUN; g0 < G; g0 += kDispatchWarps * RUN) {
        float v[RUN][4];
#pragma unroll
        for (int u = 0; u < RUN; ++u) {
          v[u][0] = v[u][1] = v[u][2] = v[u][3] = 0.f;
          if (g0 + u < G) load4f<T>(xrow + (g0 + u) * 128 + lane * 4, v[u]);
        }
#pragma unroll
        for (int u = 0; u < RUN; ++u) {
          const int g = g0 + u;
          if (g >= G) break;
          float amax = fmaxf(fmaxf(fabsf(v[u][0]), fabsf(v[u][1])), fmaxf(fabsf(v[u][2]), fabsf(v[u][3])));
          amax = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(amax)));
          const float s = __fdiv_rn(fmaxf(amax, 1e-10f), 448.0f);
          uint32_t packed = 0;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            __nv_fp8_storage_t b = __nv_cvt_float_to_fp8(__fdiv_rn(v[u][q], s), __NV_SATFINITE, __NV_E4M3);
            packed |= static_cast<uint32_t>(b) << (8 * q);
          }
          *reinterpret_cast<uint32_t*>(stage + g * 128 + lane * 4) = packed;
          if (lane == 0) stage_sc[g] = s;
        }
      }
      __syncthreads();
      for (int d = 0; d < a.world; ++d) {
        if (!(dest_mask & (1u << d))) continue;
        uint4* dst = reinterpret_cast<uint4*>(a.heap[d] + a.L.recv_x + row * a.L.x_row_bytes);
        const uint4* src = reinterpret_cast<const uint4*>(stage);
        for (int c = threadIdx.x; c < a.H / 16; c += blockDim.x) dst[c] = src[c];
        float* dsc = reinterpret_cast<float*>(a.heap[d] + a.L.recv_xs) + row * G;
        for (int g = threadIdx.x; g < G; g += blockDim.x) dsc[g] = stage_sc[g];
      }
      __syncthreads();     // the staging row is reused by the CTA's next token
    } else {
      const uint4* src = reinterpret_cast<const uint4*>(xrow);
      for (int c = threadIdx.x; c < a.H / 8; c += blockDim.x) {
        const uint4 v = __ldg(src + c);
        for (int d = 0; d < a.world; ++d)
          if (dest_mask & (1u << d))
            reinterpret_cast<uint4*>(a.heap[d] + a.L.recv_x + row * a.L.x_row_bytes)[c] = v;
      }
    }
  }

  // ---- the last CTA to get here tells every peer that this rank's rows are in place
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned int* cnt = reinterpret_cast<unsigned int*>(me + a.L.flags + kEpFlagCtaCount2);
    const unsigned int prev = atomicAdd(cnt, 1u);
    s_last = (prev == gridDim.x - 1) ? 1 : 0;
    if (s_last) {
      *cnt = 0;
      s_epoch = *reinterpret_cast<volatile unsigned long long*>(me + a.L.flags + kEpFlagEpoch);
      __threadfence_system();
    }
  }
  __syncthreads();
  if (s_last && threadIdx.x < a.world)
    st_release_sys_u64(reinterpret_cast<unsigned long long*>(a.heap[threadIdx.x] + a.L.flags + kEpFlagRows) + a.rank,
                       s_epoch);
}

__global__ void __launch_bounds__(32)
ep_wait_kernel(const FlagWait w) {
  griddep_wait();
  wait_for_peers(w);
  griddep_launch_dependents();
}

struct EpSignalArgs {
  uint8_t* heap[kMaxPeers];
  size_t flags_off;   // offset of the flag array (ready or done) inside a heap
  size_t epoch_off;   // offset of the epoch counter inside this rank's heap
  int world, rank;
};

__global__ void __launch_bounds__(32)
ep_signal_kernel(const EpSignalArgs a) {
  griddep_wait();   // everything launched before in this stream has completed and is visible here
  const unsigned long long e = *reinterpret_cast<const volatile unsigned long long*>(a.heap[a.rank] + a.epoch_off);
  __threadfence_system();
  if (threadIdx.x < a.world)
    st_release_sys_u64(reinterpret_cast<unsigned long long*>(a.heap[threadIdx.x] + a.flags_off) + a.rank, e);
  griddep_launch_dependents();
}

}  // namespace

EpHeap ep_heap_layout(int world, int m_cap, int H, int topk, bool fp8_rows) {
  EpHeap L;
  size_t off = 0;
  auto take = [&](size_t bytes) {
    size_t o = off;
    off = up256(off + bytes);
    return o;
  };
  const size_t rows = static_cast<size_t>(world) * m_cap;
  L.x_row_bytes = fp8_rows ? H : 2 * H;
  L.flags = take(256);
  L.recv_ids = take(rows * topk * 4);
  L.recv_w = take(rows * topk * 4);
  L.recv_x = take(rows * L.x_row_bytes);
  L.recv_xs = take(rows * ((H + 127) / 128) * 4);
  L.pairs = take(static_cast<size_t>(m_cap) * topk * H * 2);
  L.pair_valid = take((static_cast<size_t>(m_cap) * topk + 15) / 16 * 16);
  L.out32 = take(static_cast<size_t>(m_cap) * H * 4);
  L.total = off;
  return L;
}

int launch_ep_dispatch(const EpDispatchArgs& a, int num_sms, cudaStream_t stream, bool pdl) {
  if (a.world < 1 || a.world > kMaxPeers || a.rank < 0 || a.rank >= a.world || a.topk > 32) return B200MOE_ERR_BAD_ARG;
  if (a.m < 0 || a.m > a.m_cap || a.H % 8 != 0 || (a.fp8_rows && a.H % 128 != 0)) return B200MOE_ERR_BAD_ARG;
  const size_t smem = a.fp8_rows ? ep_stage_bytes(a.H) : 0;
  if (smem > 200 * 1024) return B200MOE_ERR_TOO_LARGE;
  int ctas = a.m_cap;
  if (ctas > num_sms * 8) ctas = num_sms * 8;
  if (ctas < 1) ctas = 1;
  cudaError_t err;
  note_launch("ep_dispatch_kernel");
  if (a.dtype == B200MOE_DTYPE_BF16) {
    if (cudaFuncSetAttribute(ep_dispatch_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem)) != cudaSuccess)
      return B200MOE_ERR_CUDA;
    err = launch_kernel(ep_dispatch_kernel<__nv_bfloat16>, dim3(ctas), dim3(kDispatchWarps * 32), smem, stream, pdl, a);
  } else {
    if (cudaFuncSetAttribute(ep_dispatch_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem)) != cudaSuccess)
      return B200MOE_ERR_CUDA;
    err = launch_kernel(ep_dispatch_kernel<__half>, dim3(ctas), dim3(kDispatchWarps * 32), smem, stream, pdl, a);
  }
  return err == cudaSuccess ? B200MOE_OK : B200MOE_ERR_CUDA;
}

FlagWait ep_flag_wait(uint8_t* my_heap, const EpHeap& L, size_t flag_off, int world, unsigned long long limit_ns,
                      int* status) {
  FlagWait w;
  w.flags = reinterpret_cast<const unsigned long long*>(my_heap + L.flags + flag_off);
  w.epoch = reinterpret_cast<const unsigned long long*>(my_heap + L.flags + kEpFlagEpoch);
  w.world = world;
  w.limit_ns = limit_ns;
  w.status = status;
  return w;
}

int launch_ep_wait(const FlagWait& w, cudaStream_t stream, bool pdl) {
  note_launch("ep_wait_kernel");
  cudaError_t err = launch_kernel(ep_wait_kernel, dim3(1), dim3(32), 0, stream, pdl, w);
  return err == cudaSuccess ? B200MOE_OK : B200MOE_ERR_CUDA;
}

int launch_ep_signal(uint8_t* const* heaps, const EpHeap& L, size_t flag_off, int world, int rank,
                     cudaStream_t stream, bool pdl) {
  EpSignalArgs a = {};
  for (int r = 0; r < world; ++r) a.heap[r] = heaps[r];
  a.flags_off = L.flags + flag_off;
  a.epoch_off = L.flags + kEpFlagEpoch;
  a.world = world;
  a.rank = rank;
  note_launch("ep_signal_kernel");
  cudaError_t err = launch_kernel(ep_signal_kernel, dim3(1), dim3(32), 0, stream, pdl, a);
  return err == cudaSuccess ? B200MOE_OK : B200MOE_ERR_CUDA;
}

}  // namespace b200moe
