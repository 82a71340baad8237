// C ABI: argument checks, workspace layout, tensor-map encoding and the launch sequence.
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "align.cuh"
#include "ep.cuh"
#include "gemm.cuh"
#include "gemv.cuh"
#include "prep.cuh"
#include "router.cuh"

using namespace b200moe;

namespace b200moe {
void note_launch(const char* name);
}

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

CUtensorMapDataType tmap_dtype(int dtype, int elem_bytes) {
  if (elem_bytes == 1) return CU_TENSOR_MAP_DATA_TYPE_UINT8;
  return dtype == B200MOE_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
}

// [rows, inner] row-major matrix, box = {box_inner, box_rows}, 128-byte swizzle.
int make_tmap_2d(CUtensorMap* m, CUtensorMapDataType dt, int elem_bytes, const void* base, uint64_t inner,
                 uint64_t rows, uint32_t box_inner, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return B200MOE_ERR_CUDA;
  cuuint64_t dims[2] = {inner, rows};
  cuuint64_t strides[1] = {inner * elem_bytes};
  cuuint32_t box[2] = {box_inner, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? B200MOE_OK : B200MOE_ERR_CUDA;
}

// [experts, rows, inner] tensor, box = {box_inner, box_rows, 1}.
int make_tmap_3d(CUtensorMap* m, CUtensorMapDataType dt, int elem_bytes, const void* base, uint64_t inner,
                 uint64_t rows, uint64_t experts, uint32_t box_inner, uint32_t box_rows,
                 CUtensorMapSwizzle swz = CU_TENSOR_MAP_SWIZZLE_128B) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return B200MOE_ERR_CUDA;
  cuuint64_t dims[3] = {inner, rows, experts};
  cuuint64_t strides[2] = {inner * elem_bytes, inner * rows * elem_bytes};
  cuuint32_t box[3] = {box_inner, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(m, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? B200MOE_OK : B200MOE_ERR_CUDA;
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Optional per-kernel timing for the benchmark: CUDA events recorded around the two
// GEMM launches of every forward call between profile_begin and profile_end.
struct Profile {
  std::mutex mu;
  bool on = false;
  int max_calls = 0, calls = 0;
  std::vector<cudaEvent_t> ev;  // kMarks events per call
  std::vector<char> local_marked;  // per call: marks 6 and 7 were recorded
};
Profile g_prof;

// mark index: 0 = call start, 1 = before GEMM-1, 2 = after GEMM-1, 3 = before GEMM-2, 4 = after GEMM-2, 5 = call end,
// 6 / 7 = start / end of the local operator of an expert-parallel call (after the peers' rows have
// arrived; after the down projection has completed)
constexpr int kMarks = 8;

int prof_slot() {
  if (!g_prof.on) return -1;
  std::lock_guard<std::mutex> lk(g_prof.mu);
  if (!g_prof.on || g_prof.calls >= g_prof.max_calls) return -1;
  return g_prof.calls++;
}
// The slot of the call in progress: the later phases of an expert-parallel call that was started
// by an earlier b200moe_ep_forward(phases = dispatch) continue in the slot that call took.
int prof_slot_current() {
  if (!g_prof.on) return -1;
  std::lock_guard<std::mutex> lk(g_prof.mu);
  return g_prof.calls > 0 ? g_prof.calls - 1 : -1;
}
void prof_mark(int slot, int mark, cudaStream_t st) {
  if (slot < 0) return;
  cudaEventRecord(g_prof.ev[static_cast<size_t>(slot) * kMarks + mark], st);
  if (mark == 7) g_prof.local_marked[slot] = 1;
}

// Launch accounting (see common.cuh: note_launch).
struct LaunchLog {
  std::mutex mu;
  long long total = 0;
  std::string last_call;   // kernels of the most recent forward call, comma separated
};
LaunchLog g_launches;
void launch_log_new_call() {
  std::lock_guard<std::mutex> lk(g_launches.mu);
  g_launches.last_call.clear();
}

struct Layout {
  int BT, cap, P;
  bool align_multi; // alignment on 32 CTAs (many slots)
  bool quant_once; // FP8: quantise each token once, then gather the quantised rows (many pairs per token)
  bool pair_rows; // the down projection stores one 16-bit row per pair, the output conversion sums them
  bool w4p;       // int4 decode path: integer MMAs on three-plane int8 activations
  int out_rows;   // rows of the fp32 output buffer: tokens, or pairs when nothing is combined
  int orient;     // GEMM tile orientation that goes with BT
  int act_bytes;  // bytes per activation element fed to the GEMMs
  size_t meta, blk_off, sorted_ids, expert_ids, num_post, row_gamma, xs, xs_scale, xs_sum, a2, a2_scale,
      a2_sum, out32, pairs, pair_valid, xq_tok, xq_scale, route_w, route_ids, align_tmp, total;
};

int pick_bt(const b200moe_cfg* c) {
  if (c->block_tokens > 0) return c->block_tokens;
  const double avg = static_cast<double>(c->M) * c->topk / (c->E > 0 ? c->E : 1);
  if (c->wmode == B200MOE_W_FP8_BLOCK) {
    // many-expert FP8 layers route unevenly: hot experts hold several times the average, and every
    // extra block of an expert streams its weights once more from L2, so lean towards larger blocks
    // (measured on the 256-expert zipf-skewed layer: average 2 (M = 64) -> 16 is best; average 4: 16 / 32 /
    // 64 within 4 %; average 8 (M = 256): tokens-on-M blocks of 128 and 64-token blocks beat 32-token blocks
    // by 10 %; average 12 / 16: blocks of 128 win by 20 % / 11 %)
    if (avg <= 4) return 16;
    if (avg < 8) return 32;
    return 128;  // tokens-on-M kernels
  }
  if (avg <= 10) return 16;
  if (avg <= 20) return 32;
  if (avg <= 40) return 64;
  return 128;
}

int check_cfg(const b200moe_cfg* c) {
  if (c == nullptr || c->struct_bytes != static_cast<int32_t>(sizeof(b200moe_cfg))) return B200MOE_ERR_BAD_ARG;
  if (c->M < 0 || c->H <= 0 || c->I <= 0 || c->E <= 0 || c->topk <= 0) return B200MOE_ERR_BAD_ARG;
  if (c->dtype != B200MOE_DTYPE_BF16 && c->dtype != B200MOE_DTYPE_FP16) return B200MOE_ERR_BAD_ARG;
  if (c->activation != B200MOE_ACT_SILU && c->activation != B200MOE_ACT_GELU &&
      c->activation != B200MOE_ACT_SWIGLU_OAI)
    return B200MOE_ERR_BAD_ARG;
  if (c->block_tokens != 0 && (c->block_tokens < 16 || c->block_tokens > 256 || c->block_tokens % 16))
    return B200MOE_ERR_BAD_ARG;
  if (static_cast<long long>(c->M) * c->topk > (1LL << 24)) return B200MOE_ERR_TOO_LARGE;
  if (c->H % 8 != 0 || c->I % 8 != 0) return B200MOE_ERR_UNSUPPORTED;  // 16-byte rows for TMA
  if ((c->flags & B200MOE_FLAG_X_FP8) && c->wmode != B200MOE_W_FP8_BLOCK) return B200MOE_ERR_UNSUPPORTED;
  if (c->n_global_experts < 0) return B200MOE_ERR_BAD_ARG;
  if (c->wmode == B200MOE_W_16BIT) {
    if (c->w_layout != B200MOE_LAYOUT_LAYER) return B200MOE_ERR_UNSUPPORTED;
  } else if (c->wmode == B200MOE_W_FP8_BLOCK) {
    if (c->H % 128 != 0 || c->I % 128 != 0) return B200MOE_ERR_UNSUPPORTED;
    if (c->block_tokens != 0 && c->block_tokens != 16 && c->block_tokens != 32 && c->block_tokens != 64 &&
        c->block_tokens != 128)
      return B200MOE_ERR_UNSUPPORTED;
    if (c->flags & B200MOE_FLAG_SIMT) return B200MOE_ERR_UNSUPPORTED;
  } else if (c->wmode == B200MOE_W_INT4_AWQ) {
    if (c->H % 128 != 0 || c->I % 128 != 0) return B200MOE_ERR_UNSUPPORTED;   // whole groups of 128
    if (c->dtype != B200MOE_DTYPE_FP16) return B200MOE_ERR_UNSUPPORTED;
    if (c->flags & B200MOE_FLAG_SIMT) return B200MOE_ERR_UNSUPPORTED;
  } else {
    return B200MOE_ERR_UNSUPPORTED;
  }
  return B200MOE_OK;
}

int query_sms(const b200moe_cfg* c);
bool reference_rounds_pairs(int P, int E, int n, int k, int sms);
constexpr int kAlignMultiSlots = 8192;   // from here on the alignment runs on 32 CTAs

int make_layout(const b200moe_cfg* c, Layout* L) {
  L->BT = pick_bt(c);
  // a block of 128 tokens sits on the M side of the MMA; smaller (and 256-token) blocks on the N side
  // int4 always runs tokens-on-M (one MMA then covers 256 weight rows, which halves the number of
  // MMA instructions per streamed byte; blocks below 128 tokens simply load fewer token rows)
  if (c->wmode == B200MOE_W_INT4_AWQ) L->orient = (L->BT <= 128) ? 1 : 0;
  else if (c->wmode == B200MOE_W_FP8_BLOCK)
    L->orient = (L->BT == 128) ? 1 : 0;
  else L->orient = (L->BT == 128) ? 1 : 0;
  L->P = c->M * c->topk;
  int cap = align_capacity(L->P, c->E, L->BT);
  if (cap < 0) return B200MOE_ERR_TOO_LARGE;
  cap = static_cast<int>(align_up(static_cast<size_t>(cap > 0 ? cap : 1), L->BT));
  L->cap = cap;
  const bool fp8 = c->wmode == B200MOE_W_FP8_BLOCK;
  // decode-sized int4: nibbles converted straight into tensor memory, integer MMAs, group scales
  // applied to the partial sums
  L->w4p = c->wmode == B200MOE_W_INT4_AWQ && L->BT <= 32 && !(c->flags & B200MOE_FLAG_W4_SMEM_OPERANDS) &&
           gemm_w4_planes_ok(c->H, L->BT) && gemm_w4_planes_ok(c->I, L->BT);
  L->act_bytes = fp8 ? 1 : (L->w4p ? 3 : 2);
  const bool tables = fp8 || L->w4p;   // per (128-k group, row) tables beside the activations
  size_t off = 0;
  auto take = [&](size_t bytes) {
    size_t o = off;
    off = align_up(off + bytes, 1024);
    return o;
  };
  L->meta = take(64);
  L->blk_off = take(static_cast<size_t>(c->E + 1) * 4);
  L->sorted_ids = take(static_cast<size_t>(cap) * 4);
  L->expert_ids = take(static_cast<size_t>(cap / L->BT + 1) * 4);
  L->num_post = take(16);
  L->row_gamma = take(static_cast<size_t>(cap) * 4);
  L->xs = take(static_cast<size_t>(cap) * c->H * L->act_bytes);
  L->xs_scale = take(tables ? static_cast<size_t>(cap) * (c->H / 128) * 4 : 0);
  L->xs_sum = take(L->w4p ? static_cast<size_t>(cap) * (c->H / 128) * 4 : 0);
  L->a2 = take(static_cast<size_t>(cap) * c->I * L->act_bytes);
  L->a2_scale = take(tables ? static_cast<size_t>(cap) * (c->I / 128) * 4 : 0);
  L->a2_sum = take(L->w4p ? static_cast<size_t>(cap) * (c->I / 128) * 4 : 0);
  L->out_rows = (c->flags & B200MOE_FLAG_NO_COMBINE) ? L->P : c->M;   // one fp32 row per pair when nothing is summed
  // Many pairs on 128-token blocks: fp32 atomics into the combine buffer would bound the down
  // projection's tail (every add is a read-modify-write of a row another tile also touches), and
  // its tiles fill the GPU without splitting the reduction; store one 16-bit row per pair instead
  // and let the output conversion sum a token's rows in a fixed order.  The combine buffer shrinks
  // to the pairs' validity bytes.  16-bit weights: only where the reference, too, rounds each
  // pair's row to the 16-bit type (or its rounding is not asked for).
  const int sms_l = query_sms(c);
  // (16-bit: from four waves of tiles on; below that the split reduction, which needs the atomics,
  // is what keeps the last wave full)
  const bool many_tiles = (static_cast<long long>(L->P) / L->BT) * ((c->H + 255) / 256) >=
                          (fp8 ? 2LL : 4LL) * sms_l;
  const bool pairs_ok16 = !fp8 && !L->w4p && L->orient == 1 &&
                          (!(c->flags & B200MOE_FLAG_MIMIC_ROUNDING) ||
                           reference_rounds_pairs(L->P, c->E, c->H, c->I, sms_l));
  L->pair_rows = (fp8 || pairs_ok16) && L->BT == 128 && !(c->flags & B200MOE_FLAG_NO_COMBINE) &&
                 !(c->flags & B200MOE_FLAG_SIMT) && many_tiles;
  L->out32 = take(L->pair_rows ? 16 : static_cast<size_t>(L->out_rows > 0 ? L->out_rows : 1) * c->H * 4);
  // Quantising inside the gather repeats the work topk times; beyond a few thousand pairs it pays to
  // quantise the M token rows once and gather bytes.
  L->quant_once = fp8 && L->P >= 2048 && c->topk > 1 && !(c->flags & B200MOE_FLAG_X_FP8);
  L->xq_tok = take(L->quant_once ? static_cast<size_t>(c->M) * c->H : 0);
  L->xq_scale = take(L->quant_once ? static_cast<size_t>(c->M) * (c->H / 128) * 4 : 0);
  L->pairs = take(L->pair_rows ? static_cast<size_t>(L->P) * c->H * 2 : 0);
  L->pair_valid = take(L->pair_rows ? align_up(static_cast<size_t>(L->P), 16) : 0);
  L->route_w = take(static_cast<size_t>(L->P > 0 ? L->P : 1) * 4);    // router output when the call starts from logits
  L->route_ids = take(static_cast<size_t>(L->P > 0 ? L->P : 1) * 4);
  L->align_multi = L->P >= kAlignMultiSlots && !(c->flags & B200MOE_FLAG_ALIGN_ONE_CTA);
  L->align_tmp = take(L->align_multi ? align_multi_tmp_bytes(c->E) : 0);
  L->total = off;
  return B200MOE_OK;
}

// Would the reference round each (token, expert) row of the down projection to the 16-bit
// type before the top-k sum?  It does exactly when its grouped matmul does not split the
// reduction: the dependency picks split_k = 1 for its persistent kernel (>= 2 tiles per SM)
// and otherwise min(n_sms / grid, ceil(k / 64) / 4) (triton_kernels
// matmul_ogs_details/opt_flags.py, make_default_opt_flags_nvidia, and
// opt_flags_details/opt_flags_nvidia.py, compute_split_k); with split_k > 1 the partial
// products stay in fp32 until the combined reduction (matmul_ogs.py, scratch dtype).
int next_pow2(int v) {
  int p = 1;
  while (p < v) p <<= 1;
  return p;
}
int cdiv(int a, int b) { return (a + b - 1) / b; }
bool reference_rounds_pairs(int P, int E, int n, int k, int sms) {
  const int tpe = P / E > 1 ? P / E : 1;
  int block_m = next_pow2(tpe);
  block_m = block_m < 16 ? 16 : (block_m > 128 ? 128 : block_m);
  int block_n = 256;
  if (n <= 128) {
    block_n = next_pow2(n);
    block_n = block_n < 16 ? 16 : (block_n > 128 ? 128 : block_n);
  }
  const int grid_n = cdiv(n, block_n);
  const int grid_m_routed = (P <= E) ? P : cdiv(P - E + 1 > 0 ? P - E + 1 : 0, block_m) + E - 1;
  if (static_cast<double>(grid_m_routed) * grid_n / sms >= 2.0) return true;  // persistent kernel
  const int grid = cdiv(P, block_m) * grid_n;
  int split = grid > 0 ? sms / grid : 1;
  const int by_k = cdiv(k, 64) / 4;
  if (split > by_k) split = by_k;
  return split <= 1;
}

int query_sms(const b200moe_cfg* c) {
  if (c != nullptr && c->num_sms > 0) return c->num_sms;
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

// Block alignment into the workspace tables: one CTA, or 32 CTAs in three launches for many slots.
int align_into_workspace(const b200moe_cfg* c, const Layout& L, uint8_t* ws, const void* ids, int is64,
                         const int32_t* expert_map, const float* weights, cudaStream_t st,
                         const FlagWait* wait = nullptr) {
  const bool pdl = (c->flags & B200MOE_FLAG_NO_PDL) == 0;
  int* sorted_ids = reinterpret_cast<int*>(ws + L.sorted_ids);
  int* expert_ids = reinterpret_cast<int*>(ws + L.expert_ids);
  int* num_post = reinterpret_cast<int*>(ws + L.num_post);
  float* row_gamma = reinterpret_cast<float*>(ws + L.row_gamma);
  int* blk_off = reinterpret_cast<int*>(ws + L.blk_off);
  int* meta = reinterpret_cast<int*>(ws + L.meta);
  if (L.align_multi)
    return launch_align_block_multi(ids, is64, expert_map, c->n_global_experts, weights, L.P, c->E, L.BT, L.cap, sorted_ids, expert_ids,
                                    num_post, row_gamma, blk_off, meta, reinterpret_cast<int*>(ws + L.align_tmp), st, pdl,
                                    wait);
  return launch_align_block(ids, is64, expert_map, c->n_global_experts, weights, L.P, c->E, L.BT, L.cap, sorted_ids,
                            expert_ids, num_post, row_gamma, blk_off, meta, st, pdl, wait);
}

// Expert parallelism: where the down projection's output rows go (the buffers of the ranks that
// own the tokens) instead of this call's workspace.
struct PeerOut {
  int n_peers = 0;
  int tokens_per_peer = 0;             // m_cap: rows of a rank's fp32 buffer; its pair rows: m_cap * topk
  void* out32[kMaxPeers] = {};
  void* pairs[kMaxPeers] = {};
  uint8_t* pair_valid[kMaxPeers] = {};
  const FlagWait* rows_wait = nullptr;   // the gather waits for the peers' "rows" flags in its prologue
};

// Everything after the internal routing tables exist in the workspace.  With `peers` the results
// land on their owners and nothing is cleared or converted here.
int run_experts(const b200moe_cfg* c, const Layout& L, const void* x, const void* w1, const void* w2,
                const b200moe_quant* quant, uint8_t* ws, void* out, int32_t* status, cudaStream_t st,
                int slot, const PeerOut* peers = nullptr) {
  const int sms = query_sms(c);
  int* meta = reinterpret_cast<int*>(ws + L.meta);
  int* blk_off = reinterpret_cast<int*>(ws + L.blk_off);
  int* sorted_ids = reinterpret_cast<int*>(ws + L.sorted_ids);
  float* row_gamma = reinterpret_cast<float*>(ws + L.row_gamma);
  void* xs = ws + L.xs;
  void* a2 = ws + L.a2;
  float* out32 = reinterpret_cast<float*>(ws + L.out32);
  const bool fp8 = c->wmode == B200MOE_W_FP8_BLOCK;
  const bool w4 = c->wmode == B200MOE_W_INT4_AWQ;
  const bool pdl = (c->flags & B200MOE_FLAG_NO_PDL) == 0;
  int rc;
  if (w4 && (quant == nullptr || quant->w1_sz == nullptr || quant->w2_sz == nullptr)) return B200MOE_ERR_BAD_ARG;

  // cleared alongside the first row mover: the fp32 combine buffer, or the pairs' validity bytes
  // when rows are stored per pair
  void* zero = L.pair_rows ? static_cast<void*>(ws + L.pair_valid) : static_cast<void*>(out32);
  size_t zero_bytes = L.pair_rows ? align_up(static_cast<size_t>(L.P), 16)
                                  : static_cast<size_t>(L.out_rows) * c->H * 4;
  if (peers != nullptr) zero_bytes = 0;   // the owners cleared their buffers before they signalled "ready"
  if (fp8) {
    if (quant == nullptr || quant->w1_scale == nullptr || quant->w2_scale == nullptr) return B200MOE_ERR_BAD_ARG;
    if (c->flags & B200MOE_FLAG_X_FP8) {
      // rows arrive quantised (e.g. from an expert-parallel dispatch that sends bytes): gather only
      if (quant->x_scale == nullptr) return B200MOE_ERR_BAD_ARG;
      rc = launch_gather_rows(x, xs, sorted_ids, meta, L.P, c->topk, c->H, L.cap, zero, zero_bytes, sms, st, pdl,
                              quant->x_scale, reinterpret_cast<float*>(ws + L.xs_scale), c->H / 128, L.cap,
                              peers != nullptr ? peers->rows_wait : nullptr);
    } else if (L.quant_once) {
      float* tok_scale = reinterpret_cast<float*>(ws + L.xq_scale);
      rc = launch_group_quant_fp8(x, c->dtype, ws + L.xq_tok, tok_scale, nullptr, nullptr, L.P, c->topk, c->M, c->H, 0,
                                  0, zero, zero_bytes, sms, st, pdl);
      if (rc != B200MOE_OK) return rc;
      rc = launch_gather_rows(ws + L.xq_tok, xs, sorted_ids, meta, L.P, c->topk, c->H, L.cap, zero, 0, sms, st, pdl,
                              tok_scale, reinterpret_cast<float*>(ws + L.xs_scale), c->H / 128, L.cap);
    } else {
      rc = launch_group_quant_fp8(x, c->dtype, xs, reinterpret_cast<float*>(ws + L.xs_scale), sorted_ids, meta,
                                  L.P, c->topk, L.cap, c->H, 1, L.cap, zero, zero_bytes, sms, st, pdl);
    }
  } else if (L.w4p) {
    rc = launch_group_split_i8(x, reinterpret_cast<uint8_t*>(xs), reinterpret_cast<float*>(ws + L.xs_scale),
                               reinterpret_cast<int*>(ws + L.xs_sum), sorted_ids, meta, L.P, c->topk, L.cap, c->H,
                               L.BT, L.cap, zero, zero_bytes, sms, st, pdl);
  } else {
    rc = launch_gather_rows(x, xs, sorted_ids, meta, L.P, c->topk, c->H * 2, L.cap, zero, zero_bytes, sms, st, pdl);
  }
  if (rc != B200MOE_OK) return rc;

  GemmArgs g1 = {};
  g1.mode = 0;
  g1.dtype = c->dtype;
  g1.wmode = c->wmode;
  g1.E = c->E;
  g1.K = c->H;
  g1.N = c->I;
  g1.up_row_off = c->I;
  g1.BT = L.BT;
  g1.orient = L.orient;
  g1.topk = c->topk;
  g1.P = L.P;
  g1.flags = c->flags;
  g1.activation = c->activation;
  g1.meta = meta;
  g1.blk_off = blk_off;
  g1.sorted_ids = sorted_ids;
  g1.row_gamma = row_gamma;
  g1.out = a2;
  g1.ld_out = c->I;
  g1.status = status;
  g1.pdl = pdl ? 1 : 0;
  g1.act_alpha = 1.0f;
  if (quant != nullptr) {
    g1.bias = quant->b1;
    g1.act_alpha = quant->swiglu_alpha;
    g1.act_limit = quant->swiglu_limit;
  }
  if (fp8) {
    g1.w_scale = quant->w1_scale;
    g1.w_scale_rows = (2 * c->I + 127) / 128;
    g1.x_scale = reinterpret_cast<float*>(ws + L.xs_scale);
    g1.ld_xscale = L.cap;
    g1.out_q = reinterpret_cast<uint8_t*>(a2);
    g1.out_scale = reinterpret_cast<float*>(ws + L.a2_scale);
  }
  if (w4) {
    g1.w_sz = quant->w1_sz;
    g1.w_rows = 2 * c->I;
  }
  const bool w4p = L.w4p;
  if (w4p) {
    g1.x_scale = reinterpret_cast<float*>(ws + L.xs_scale);
    g1.x_sum = reinterpret_cast<int*>(ws + L.xs_sum);
    g1.ld_xscale = L.cap;
    g1.out_q = reinterpret_cast<uint8_t*>(a2);
    g1.out_scale = reinterpret_cast<float*>(ws + L.a2_scale);
    g1.out_sum = reinterpret_cast<int*>(ws + L.a2_sum);
  }
  if (fp8) gemm_plan_fp8(&g1); else if (w4p) gemm_plan_w4(&g1); else gemm_plan(&g1);

  GemmArgs g2 = g1;
  g2.mode = 1;
  g2.K = c->I;
  g2.N = c->H;
  g2.up_row_off = 0;
  g2.out = out32;
  g2.ld_out = c->H;
  g2.max_split = 0;
  if (c->flags & B200MOE_FLAG_NO_COMBINE) g2.topk = 1;   // output row = pair slot instead of token
  g2.bias = quant != nullptr ? quant->b2 : nullptr;
  if (w4) {
    g2.w_sz = quant->w2_sz;
    g2.w_rows = c->H;
  }
  if (!fp8 && (c->flags & B200MOE_FLAG_MIMIC_ROUNDING)) {
    if (reference_rounds_pairs(L.P, c->E, c->H, c->I, sms)) g2.flags |= B200MOE_FLAG_NO_SPLIT_K;
    else g2.flags &= ~B200MOE_FLAG_MIMIC_ROUNDING;
  }
  if (L.pair_rows) {
    g2.out_pairs = ws + L.pairs;
    g2.pair_valid = ws + L.pair_valid;
    g2.flags |= B200MOE_FLAG_NO_SPLIT_K;
  }
  if (peers != nullptr) {
    if (!fp8 || (c->flags & (B200MOE_FLAG_NO_COMBINE | B200MOE_FLAG_SIMT))) return B200MOE_ERR_UNSUPPORTED;
    g2.n_peers = peers->n_peers;
    g2.rows_per_peer = L.pair_rows ? peers->tokens_per_peer * c->topk : peers->tokens_per_peer;
    for (int r = 0; r < peers->n_peers; ++r) {
      g2.peer_out[r] = L.pair_rows ? peers->pairs[r] : peers->out32[r];
      g2.peer_valid[r] = peers->pair_valid[r];
    }
    // with a single rank the "peer" is this GPU's own heap: plain local addressing through the same fields
    if (peers->n_peers == 1) {
      if (L.pair_rows) {
        g2.out_pairs = peers->pairs[0];
        g2.pair_valid = peers->pair_valid[0];
      } else {
        g2.out = peers->out32[0];
      }
    }
  }
  if (fp8) {
    g2.w_scale = quant->w2_scale;
    g2.w_scale_rows = (c->H + 127) / 128;
    g2.x_scale = reinterpret_cast<float*>(ws + L.a2_scale);
    g2.out_q = nullptr;
    g2.out_scale = nullptr;
    g2.flags &= ~B200MOE_FLAG_MIMIC_ROUNDING;
  }
  if (w4p) {
    g2.x_scale = reinterpret_cast<float*>(ws + L.a2_scale);
    g2.x_sum = reinterpret_cast<int*>(ws + L.a2_sum);
    g2.out_q = nullptr;
    g2.out_scale = nullptr;
    g2.out_sum = nullptr;
  }
  if (fp8) gemm_plan_fp8(&g2); else if (w4p) gemm_plan_w4(&g2); else gemm_plan(&g2);
  // CTA pairs for the 16-bit prefill GEMMs (each GEMM by itself: the down projection only when its
  // reduction is in one piece)
  const bool pair_flag = (c->flags & B200MOE_FLAG_CTA_PAIR) != 0 && !(c->flags & B200MOE_FLAG_SIMT) && sms >= 2;
  const bool pair1 = pair_flag && gemm_tc2_ok(g1);
  const bool pair2 = pair_flag && gemm_tc2_ok(g2);
  if (pair1) gemm_plan_tc2(&g1);
  if (pair2) gemm_plan_tc2(&g2);

  if (c->flags & B200MOE_FLAG_SIMT) {
    rc = launch_gemm_simt(w1, xs, g1, st, L.cap);
    if (rc != B200MOE_OK) return rc;
    rc = launch_gemm_simt(w2, a2, g2, st, L.cap);
    if (rc != B200MOE_OK) return rc;
  } else {
    const int eb = w4p ? 1 : L.act_bytes;
    const CUtensorMapDataType dt = tmap_dtype(c->dtype, eb);
    const uint32_t kbox = 128 / eb;
    CUtensorMap tm_w1, tm_x, tm_w2, tm_a2;
    if (w4) {
      // packed int4 rows, K/2 bytes per row.  Shared-memory-operand kernels: 32 bytes (64 k) per
      // stage, plain row-major staging; integer decode kernels: 64 bytes (one group) per stage with
      // the 64-byte swizzle, so that threads reading whole rows do not collide on banks
      const uint32_t pbox = w4p ? 64 : 32;
      const CUtensorMapSwizzle psw = w4p ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_NONE;
      if ((rc = make_tmap_3d(&tm_w1, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w1, c->H / 2, 2ull * c->I, c->E, pbox, 128,
                             psw)) != B200MOE_OK)
        return rc;
      if ((rc = make_tmap_3d(&tm_w2, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w2, c->I / 2, c->H, c->E, pbox, 128,
                             psw)) != B200MOE_OK)
        return rc;
    } else {
      if ((rc = make_tmap_3d(&tm_w1, dt, eb, w1, c->H, 2ull * c->I, c->E, kbox, 128)) != B200MOE_OK) return rc;
      if ((rc = make_tmap_3d(&tm_w2, dt, eb, w2, c->I, c->H, c->E, kbox, (L.orient == 1 && !fp8 && !pair2) ? 256 : 128)) != B200MOE_OK)
        return rc;
    }
    // int4 decode: a token block is 3 * BT consecutive rows (its three byte planes)
    const uint64_t xrows = w4p ? 3ull * L.cap : static_cast<uint64_t>(L.cap);
    const uint32_t xbox = w4p ? 3u * L.BT : static_cast<uint32_t>(L.BT);
    if ((rc = make_tmap_2d(&tm_x, dt, eb, xs, c->H, xrows, kbox, xbox)) != B200MOE_OK) return rc;
    if ((rc = make_tmap_2d(&tm_a2, dt, eb, a2, c->I, xrows, kbox, xbox)) != B200MOE_OK) return rc;
    prof_mark(slot, 1, st);
    rc = fp8 ? launch_gemm_fp8(tm_w1, tm_x, g1, sms, st)
             : (w4p ? launch_gemm_w4(tm_w1, tm_x, g1, sms, st)
                    : (pair1 ? launch_gemm_tc2(tm_w1, tm_x, g1, sms, st) : launch_gemm_tc(tm_w1, tm_x, g1, sms, st)));
    prof_mark(slot, 2, st);
    if (rc != B200MOE_OK) return rc;
    prof_mark(slot, 3, st);
    rc = fp8 ? launch_gemm_fp8(tm_w2, tm_a2, g2, sms, st)
             : (w4p ? launch_gemm_w4(tm_w2, tm_a2, g2, sms, st)
                    : (pair2 ? launch_gemm_tc2(tm_w2, tm_a2, g2, sms, st) : launch_gemm_tc(tm_w2, tm_a2, g2, sms, st)));
    prof_mark(slot, 4, st);
    if (rc != B200MOE_OK) return rc;
  }
  if (peers != nullptr) return B200MOE_OK;   // the owners convert what arrived, after the peers' "done" flags
  if (L.pair_rows)
    rc = launch_finalize_pairs(ws + L.pairs, ws + L.pair_valid, out, c->dtype, c->M, c->topk, c->H,
                               c->routed_scaling, sms, st, pdl);
  else
    rc = launch_finalize(out32, out, c->dtype, static_cast<size_t>(L.out_rows) * c->H,
                         (c->flags & B200MOE_FLAG_NO_COMBINE) ? 1.0f : c->routed_scaling, sms, st, pdl);
  prof_mark(slot, 5, st);
  return rc;
}

// A handful of (token, choice) pairs: two matrix-vector launches straight from the routing input
// instead of alignment, gather, grouped GEMMs and output conversion (gemv.cuh).  Returns
// B200MOE_ERR_UNSUPPORTED when the call does not qualify; the caller then takes the usual path.
// A caller that fixes the token block (cfg.block_tokens) asks for the grouped GEMMs.
// Does this problem take the matrix-vector path?  Host arithmetic only.
bool gemv_eligible(const b200moe_cfg* c, const Layout& L) {
  // 16-bit weights, and int4 weights on integer dot products; FP8 rows would be converted element by
  // element on the CUDA cores, which costs more than the launches saved (measured: a 32-expert FP8
  // layer at M = 1 took 152 us this way, 97 us on the grouped tensor-core path)
  const bool w4 = c->wmode == B200MOE_W_INT4_AWQ;
  if (L.P <= 0 || L.P > kGemvMaxPairs || c->block_tokens != 0) return false;
  if ((c->wmode != B200MOE_W_16BIT && !w4) || (c->flags & (B200MOE_FLAG_SIMT | B200MOE_FLAG_W4_SMEM_OPERANDS)))
    return false;
  // the pairs' 16-bit activations go where the grouped path keeps GEMM-1's output
  if (static_cast<size_t>(L.cap) * c->I * L.act_bytes < static_cast<size_t>(L.P) * c->I * 2) return false;
  // every pair streams its expert's weights by itself: two pairs of different tokens that meet in one
  // expert read it twice, which the grouped path does not.  One token's experts are distinct; with more
  // tokens the path is taken only while such meetings are rare (pairs <= experts / 4)
  if (c->M > 1 && L.P * 4 > c->E) return false;
  GemvArgs g = {};
  g.M = c->M;
  g.H = c->H;
  g.I = c->I;
  g.topk = c->topk;
  g.w4 = w4 ? 1 : 0;
  return gemv_fits(g);      // the staged rows must fit in shared memory
}

int run_gemv(const b200moe_cfg* c, const Layout& L, const void* x, const void* w1, const void* w2,
             const b200moe_quant* quant, const float* topk_weights, const void* topk_ids,
             const int32_t* expert_map, const int32_t* hist, const int32_t* topk_indx, const float* gate_scal,
             uint8_t* ws, void* out, cudaStream_t st, int slot) {
  if (!gemv_eligible(c, L)) return B200MOE_ERR_UNSUPPORTED;
  const bool w4 = c->wmode == B200MOE_W_INT4_AWQ;
  if (w4 && (quant == nullptr || quant->w1_sz == nullptr || quant->w2_sz == nullptr)) return B200MOE_ERR_BAD_ARG;
  const int sms = query_sms(c);
  GemvArgs g = {};
  g.x = x;
  g.w1 = w1;
  g.w2 = w2;
  g.topk_w = topk_weights;
  g.topk_ids = topk_ids;
  g.expert_map = expert_map;
  g.hist = hist;
  g.topk_indx = topk_indx;
  g.gate_scal = gate_scal;
  g.ids_i64 = (c->flags & B200MOE_FLAG_IDS_I64) ? 1 : 0;
  g.n_global = c->n_global_experts;
  g.M = c->M;
  g.H = c->H;
  g.I = c->I;
  g.E = c->E;
  g.topk = c->topk;
  g.dtype = c->dtype;
  g.w4 = w4 ? 1 : 0;
  g.activation = c->activation;
  g.flags = c->flags;
  g.round_pair =
      ((c->flags & B200MOE_FLAG_MIMIC_ROUNDING) && reference_rounds_pairs(L.P, c->E, c->H, c->I, sms)) ? 1 : 0;
  g.alpha = 1.0f;
  g.routed_scaling = c->routed_scaling;
  if (quant != nullptr) {
    g.alpha = quant->swiglu_alpha;
    g.limit = quant->swiglu_limit;
    g.b1 = quant->b1;
    g.b2 = quant->b2;
    g.w1_sz = quant->w1_sz;
    g.w2_sz = quant->w2_sz;
  }
  g.act = ws + L.a2;   // the pairs' activations go where the grouped path keeps GEMM-1's output (cap >= P rows)
  g.out = out;
  if (!gemv_fits(g)) return B200MOE_ERR_UNSUPPORTED;
  const bool pdl = (c->flags & B200MOE_FLAG_NO_PDL) == 0;
  prof_mark(slot, 1, st);
  int rc = launch_gemv_up(g, sms, st, pdl);
  prof_mark(slot, 2, st);
  if (rc != B200MOE_OK) return rc;
  prof_mark(slot, 3, st);
  rc = launch_gemv_down(g, sms, st, pdl);
  prof_mark(slot, 4, st);
  prof_mark(slot, 5, st);
  return rc;
}

}  // namespace

namespace b200moe {
void note_launch(const char* name) {
  std::lock_guard<std::mutex> lk(g_launches.mu);
  ++g_launches.total;
  if (g_launches.last_call.size() < 4000) {
    if (!g_launches.last_call.empty()) g_launches.last_call += ',';
    g_launches.last_call += name;
  }
}
}  // namespace b200moe

extern "C" {

int b200moe_version(void) { return B200MOE_VERSION; }

const char* b200moe_status_string(int code) {
  switch (code) {
    case B200MOE_OK: return "ok";
    case B200MOE_ERR_BAD_ARG: return "bad argument";
    case B200MOE_ERR_UNSUPPORTED: return "unsupported shape, dtype or layout";
    case B200MOE_ERR_WORKSPACE: return "workspace too small or misaligned";
    case B200MOE_ERR_CUDA: return "CUDA runtime or driver call failed";
    case B200MOE_ERR_DEVICE_TIMEOUT: return "a device-side wait ran out of time";
    case B200MOE_ERR_TOO_LARGE: return "problem too large for this build";
    default: return "unknown status";
  }
}

int b200moe_uses_matrix_vector_path(const b200moe_cfg* cfg) {
  int rc = check_cfg(cfg);
  if (rc != B200MOE_OK) return rc;
  Layout L;
  if ((rc = make_layout(cfg, &L)) != B200MOE_OK) return rc;
  return gemv_eligible(cfg, L) ? 1 : 0;
}

int b200moe_pick_block_tokens(const b200moe_cfg* cfg) {
  int rc = check_cfg(cfg);
  if (rc != B200MOE_OK) return rc;
  return pick_bt(cfg);
}

size_t b200moe_workspace_bytes(const b200moe_cfg* cfg) {
  if (check_cfg(cfg) != B200MOE_OK) return 0;
  Layout L;
  if (make_layout(cfg, &L) != B200MOE_OK) return 0;
  return L.total;
}

int b200moe_align_capacity(int n_slots, int n_experts, int block) {
  if (n_slots < 0 || n_experts <= 0 || block <= 0) return B200MOE_ERR_BAD_ARG;
  int cap = align_capacity(n_slots, n_experts, block);
  return cap < 0 ? B200MOE_ERR_TOO_LARGE : cap;
}

int b200moe_align_block_size(const void* topk_ids, int ids_are_i64, int n_slots, int n_experts, int block,
                             const int32_t* expert_map, int expert_map_len, int32_t* sorted_token_ids,
                             int32_t* expert_ids,
                             int32_t* num_tokens_post_padded, void* stream) {
  if (n_slots < 0 || n_experts <= 0 || block <= 0) return B200MOE_ERR_BAD_ARG;
  if (num_tokens_post_padded == nullptr) return B200MOE_ERR_BAD_ARG;
  if (n_slots > 0 && topk_ids == nullptr) return B200MOE_ERR_BAD_ARG;
  if (expert_map != nullptr && expert_map_len <= 0) return B200MOE_ERR_BAD_ARG;
  int cap = align_capacity(n_slots, n_experts, block);
  if (cap < 0) return B200MOE_ERR_TOO_LARGE;
  if (cap > 0 && (sorted_token_ids == nullptr || expert_ids == nullptr)) return B200MOE_ERR_BAD_ARG;
  return launch_align_block(topk_ids, ids_are_i64, expert_map, expert_map_len, nullptr, n_slots, n_experts, block, cap,
                            sorted_token_ids, expert_ids, num_tokens_post_padded, nullptr, nullptr, nullptr,
                            static_cast<cudaStream_t>(stream), false, nullptr);
}

int b200moe_routing_max_tiles(int n_slots, int n_experts) {
  if (n_slots < 0 || n_experts <= 0) return B200MOE_ERR_BAD_ARG;
  return routing_max_tiles(n_slots, n_experts);
}

int b200moe_routing_from_topk(const float* topk_weights, const void* topk_ids, int ids_are_i64, int n_tokens,
                              int topk, int n_experts, int32_t* expt_indx, int32_t* topk_indx,
                              int32_t* gate_indx, float* gate_scal, int32_t* hist, int32_t* token_offs_raw,
                              int32_t* token_offs_pad, int32_t* block_pid_map, void* stream) {
  if (n_tokens < 0 || topk <= 0 || n_experts <= 0) return B200MOE_ERR_BAD_ARG;
  if (!expt_indx || !topk_indx || !gate_indx || !gate_scal || !hist || !token_offs_raw || !token_offs_pad ||
      !block_pid_map)
    return B200MOE_ERR_BAD_ARG;
  if (n_tokens > 0 && (!topk_weights || !topk_ids)) return B200MOE_ERR_BAD_ARG;
  return launch_routing_from_topk(topk_weights, topk_ids, ids_are_i64, n_tokens, topk, n_experts, expt_indx,
                                  topk_indx, gate_indx, gate_scal, hist, token_offs_raw, token_offs_pad,
                                  block_pid_map, static_cast<cudaStream_t>(stream));
}

static int forward_common(const b200moe_cfg* cfg, const void* x, const void* w1, const void* w2, void* workspace,
                          size_t workspace_bytes, void* out, int32_t* status, Layout* L) {
  int rc = check_cfg(cfg);
  if (rc != B200MOE_OK) return rc;
  if (!x || !w1 || !w2 || !workspace || !out || !status) return B200MOE_ERR_BAD_ARG;
  if ((rc = make_layout(cfg, L)) != B200MOE_OK) return rc;
  if (workspace_bytes < L->total || (reinterpret_cast<uintptr_t>(workspace) & 255) != 0) return B200MOE_ERR_WORKSPACE;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w1) & 15) ||
      (reinterpret_cast<uintptr_t>(w2) & 15) || (reinterpret_cast<uintptr_t>(out) & 15))
    return B200MOE_ERR_BAD_ARG;
  return B200MOE_OK;
}

int b200moe_forward_topk(const b200moe_cfg* cfg, const void* x, const void* w1, const void* w2,
                         const b200moe_quant* quant, const float* topk_weights, const void* topk_ids,
                         const int32_t* expert_map, void* workspace, size_t workspace_bytes, void* out,
                         int32_t* status, void* stream) {
  Layout L;
  int rc = forward_common(cfg, x, w1, w2, workspace, workspace_bytes, out, status, &L);
  if (rc != B200MOE_OK) return rc;
  if (cfg->M == 0) return B200MOE_OK;
  if (!topk_weights || !topk_ids) return B200MOE_ERR_BAD_ARG;
  if (expert_map != nullptr && cfg->n_global_experts <= 0) return B200MOE_ERR_BAD_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
  launch_log_new_call();
  const int slot = prof_slot();
  prof_mark(slot, 0, st);
  rc = run_gemv(cfg, L, x, w1, w2, quant, topk_weights, topk_ids, expert_map, nullptr, nullptr, nullptr, ws, out, st,
                slot);
  if (rc != B200MOE_ERR_UNSUPPORTED) return rc;
  rc = align_into_workspace(cfg, L, ws, topk_ids, (cfg->flags & B200MOE_FLAG_IDS_I64) ? 1 : 0, expert_map,
                            topk_weights, st);
  if (rc != B200MOE_OK) return rc;
  return run_experts(cfg, L, x, w1, w2, quant, ws, out, status, st, slot);
}

int b200moe_route_topk(const b200moe_router* router, const void* logits, int n_tokens, int n_experts, int topk,
                       float* topk_weights, int32_t* topk_ids, void* stream) {
  if (n_tokens < 0) return B200MOE_ERR_BAD_ARG;
  return launch_route_topk(router, logits, n_tokens, n_experts, topk, topk_weights, topk_ids, query_sms(nullptr),
                           static_cast<cudaStream_t>(stream));
}

int b200moe_forward_logits(const b200moe_cfg* cfg, const b200moe_router* router, const void* x, const void* w1,
                           const void* w2, const b200moe_quant* quant, const void* logits,
                           const int32_t* expert_map, void* workspace, size_t workspace_bytes, void* out,
                           int32_t* status, void* stream) {
  Layout L;
  int rc = forward_common(cfg, x, w1, w2, workspace, workspace_bytes, out, status, &L);
  if (rc != B200MOE_OK) return rc;
  rc = check_router(router, cfg->E, cfg->topk);
  if (rc != B200MOE_OK) return rc;
  if (cfg->flags & B200MOE_FLAG_IDS_I64) return B200MOE_ERR_BAD_ARG;   // the router writes int32 ids
  if (cfg->M == 0) return B200MOE_OK;
  if (!logits) return B200MOE_ERR_BAD_ARG;
  if (expert_map != nullptr && cfg->n_global_experts <= 0) return B200MOE_ERR_BAD_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
  launch_log_new_call();
  float* tw = reinterpret_cast<float*>(ws + L.route_w);
  int* ids = reinterpret_cast<int*>(ws + L.route_ids);
  const int slot = prof_slot();
  prof_mark(slot, 0, st);
  rc = launch_route_topk(router, logits, cfg->M, cfg->E, cfg->topk, tw, ids, query_sms(cfg), st);
  if (rc != B200MOE_OK) return rc;
  rc = run_gemv(cfg, L, x, w1, w2, quant, tw, ids, expert_map, nullptr, nullptr, nullptr, ws, out, st, slot);
  if (rc != B200MOE_ERR_UNSUPPORTED) return rc;
  rc = align_into_workspace(cfg, L, ws, ids, 0, expert_map, tw, st);
  if (rc != B200MOE_OK) return rc;
  return run_experts(cfg, L, x, w1, w2, quant, ws, out, status, st, slot);
}

int b200moe_forward_routed(const b200moe_cfg* cfg, const void* x, const void* w1, const void* w2,
                           const b200moe_quant* quant, const int32_t* hist, const int32_t* topk_indx,
                           const float* gate_scal, void* workspace, size_t workspace_bytes, void* out,
                           int32_t* status, void* stream) {
  Layout L;
  int rc = forward_common(cfg, x, w1, w2, workspace, workspace_bytes, out, status, &L);
  if (rc != B200MOE_OK) return rc;
  if (cfg->M == 0) return B200MOE_OK;
  if (!hist || !topk_indx || !gate_scal) return B200MOE_ERR_BAD_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
  launch_log_new_call();
  const int slot = prof_slot();
  prof_mark(slot, 0, st);
  rc = run_gemv(cfg, L, x, w1, w2, quant, nullptr, nullptr, nullptr, hist, topk_indx, gate_scal, ws, out, st, slot);
  if (rc != B200MOE_ERR_UNSUPPORTED) return rc;
  rc = launch_align_from_routing(hist, topk_indx, gate_scal, L.P, cfg->E, L.BT, L.cap,
                                 reinterpret_cast<int*>(ws + L.sorted_ids),
                                 reinterpret_cast<float*>(ws + L.row_gamma),
                                 reinterpret_cast<int*>(ws + L.blk_off), reinterpret_cast<int*>(ws + L.meta), st);
  if (rc != B200MOE_OK) return rc;
  return run_experts(cfg, L, x, w1, w2, quant, ws, out, status, st, slot);
}

// ---------------------------------------------------------------------------------------
// Forward pass for callers that must not allocate.
//
// Some hosts of this library cannot hand over a workspace: a serving runtime that has
// already given every byte of device memory to its own pools, a plugin slot whose
// interface has no allocator and no scratch argument, or a latency-critical thread that is
// forbidden to enter the CUDA allocator (it can block on other streams and fragment a
// carefully planned heap).  For them the scratch lives inside the library image: the
// array below is part of the module, so each GPU that loads the library pays for it once,
// until the process exits.
//
// In host code the symbol `g_noalloc_scratch` only names the array; it is not a device
// address.  The address is looked up once per device, with that device current, and only
// that looked-up pointer is ever handed to kernels.
static __device__ __align__(256) unsigned char g_noalloc_scratch[B200MOE_NOALLOC_SCRATCH_BYTES];

namespace {
std::mutex g_noalloc_mu;
void* g_noalloc_ptr[64] = {nullptr};

// Device address of the scratch array on the current device (nullptr on failure).
void* noalloc_scratch_for_current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lk(g_noalloc_mu);
  if (g_noalloc_ptr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || p == nullptr) return nullptr;
    g_noalloc_ptr[dev] = p;
  }
  return g_noalloc_ptr[dev];
}
}  // namespace

int b200moe_forward_topk_noalloc(const b200moe_cfg* cfg, const void* x, const void* w1, const void* w2,
                                 const b200moe_quant* quant, const float* topk_weights, const void* topk_ids,
                                 const int32_t* expert_map, void* out, int32_t* status, void* stream) {
  int rc = check_cfg(cfg);
  if (rc != B200MOE_OK) return rc;
  Layout L;
  if ((rc = make_layout(cfg, &L)) != B200MOE_OK) return rc;
  if (L.total > static_cast<size_t>(B200MOE_NOALLOC_SCRATCH_BYTES)) return B200MOE_ERR_TOO_LARGE;
  void* scratch = noalloc_scratch_for_current_device();
  if (scratch == nullptr) return B200MOE_ERR_CUDA;
  return b200moe_forward_topk(cfg, x, w1, w2, quant, topk_weights, topk_ids, expert_map, scratch,
                              static_cast<size_t>(B200MOE_NOALLOC_SCRATCH_BYTES), out, status, stream);
}

// ---------------------------------------------------------------------------------------
// Expert parallelism over peer-mapped heaps (ep.cuh).
namespace {

int check_ep(const b200moe_cfg* cfg, const b200moe_ep_cfg* ep) {
  int rc = check_cfg(cfg);
  if (rc != B200MOE_OK) return rc;
  if (ep == nullptr || ep->struct_bytes != static_cast<int32_t>(sizeof(b200moe_ep_cfg))) return B200MOE_ERR_BAD_ARG;
  if (ep->world < 1 || ep->world > kMaxPeers || ep->rank < 0 || ep->rank >= ep->world) return B200MOE_ERR_BAD_ARG;
  if (ep->m_cap <= 0 || cfg->M > ep->m_cap || ep->n_global_experts <= 0) return B200MOE_ERR_BAD_ARG;
  if (cfg->wmode != B200MOE_W_FP8_BLOCK) return B200MOE_ERR_UNSUPPORTED;   // rows travel as e4m3 + 1x128 scales
  if (cfg->flags & (B200MOE_FLAG_X_FP8 | B200MOE_FLAG_NO_COMBINE | B200MOE_FLAG_SIMT)) return B200MOE_ERR_UNSUPPORTED;
  if (cfg->topk > 32 || cfg->E > 0xffff) return B200MOE_ERR_UNSUPPORTED;
  if (static_cast<long long>(ep->world) * ep->m_cap * cfg->topk > (1LL << 24)) return B200MOE_ERR_TOO_LARGE;
  return B200MOE_OK;
}

// The local operator's view: every row of every source rank (masked routing entries drop what
// is not for this rank), activations already quantised.
b200moe_cfg ep_local_cfg(const b200moe_cfg* cfg, const b200moe_ep_cfg* ep) {
  b200moe_cfg c = *cfg;
  // token block from the real load (M_global * topk over all experts), not from the row capacity
  b200moe_cfg load = *cfg;
  load.M = ep->m_cap;
  load.block_tokens = cfg->block_tokens;
  c.block_tokens = pick_bt(&load);
  c.M = ep->world * ep->m_cap;
  c.flags |= B200MOE_FLAG_X_FP8;
  c.n_global_experts = 0;
  return c;
}

}  // namespace

size_t b200moe_ep_heap_bytes(const b200moe_cfg* cfg, const b200moe_ep_cfg* ep) {
  if (check_ep(cfg, ep) != B200MOE_OK) return 0;
  return ep_heap_layout(ep->world, ep->m_cap, cfg->H, cfg->topk, true).total;
}

size_t b200moe_ep_workspace_bytes(const b200moe_cfg* cfg, const b200moe_ep_cfg* ep) {
  if (check_ep(cfg, ep) != B200MOE_OK) return 0;
  const b200moe_cfg c = ep_local_cfg(cfg, ep);
  Layout L;
  if (make_layout(&c, &L) != B200MOE_OK) return 0;
  return L.total;
}

int b200moe_ep_heap_alloc(size_t bytes, void** heap) {
  if (heap == nullptr || bytes == 0) return B200MOE_ERR_BAD_ARG;
  void* p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess) return B200MOE_ERR_CUDA;
  if (cudaMemset(p, 0, bytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) {
    cudaFree(p);
    return B200MOE_ERR_CUDA;
  }
  *heap = p;
  return B200MOE_OK;
}

int b200moe_ep_heap_free(void* heap) {
  if (heap == nullptr) return B200MOE_OK;
  return cudaFree(heap) == cudaSuccess ? B200MOE_OK : B200MOE_ERR_CUDA;
}

int b200moe_ep_ipc_export(void* heap, void* handle64) {
  if (heap == nullptr || handle64 == nullptr) return B200MOE_ERR_BAD_ARG;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, heap) != cudaSuccess) return B200MOE_ERR_CUDA;
  memcpy(handle64, &h, sizeof(h));
  return B200MOE_OK;
}

int b200moe_ep_ipc_open(const void* handle64, void** peer_heap) {
  if (handle64 == nullptr || peer_heap == nullptr) return B200MOE_ERR_BAD_ARG;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  void* p = nullptr;
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) return B200MOE_ERR_CUDA;
  *peer_heap = p;
  return B200MOE_OK;
}

int b200moe_ep_ipc_close(void* peer_heap) {
  if (peer_heap == nullptr) return B200MOE_OK;
  return cudaIpcCloseMemHandle(peer_heap) == cudaSuccess ? B200MOE_OK : B200MOE_ERR_CUDA;
}

int b200moe_ep_forward(const b200moe_cfg* cfg, const b200moe_ep_cfg* ep, void* const* heaps, int phases,
                       const void* x, const void* w1, const void* w2, const b200moe_quant* quant,
                       const float* topk_weights, const void* topk_ids, const int32_t* placement,
                       void* workspace, size_t workspace_bytes, void* out, int32_t* status, void* stream) {
  int rc = check_ep(cfg, ep);
  if (rc != B200MOE_OK) return rc;
  if (!heaps || !w1 || !w2 || !quant || !quant->w1_scale || !quant->w2_scale || !workspace || !status)
    return B200MOE_ERR_BAD_ARG;
  if ((phases & ~7) != 0 || phases == 0) return B200MOE_ERR_BAD_ARG;
  for (int r = 0; r < ep->world; ++r)
    if (heaps[r] == nullptr || (reinterpret_cast<uintptr_t>(heaps[r]) & 255) != 0) return B200MOE_ERR_BAD_ARG;
  const b200moe_cfg c = ep_local_cfg(cfg, ep);
  Layout L;
  if ((rc = make_layout(&c, &L)) != B200MOE_OK) return rc;
  if (workspace_bytes < L.total || (reinterpret_cast<uintptr_t>(workspace) & 255) != 0) return B200MOE_ERR_WORKSPACE;
  const EpHeap H = ep_heap_layout(ep->world, ep->m_cap, cfg->H, cfg->topk, true);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
  uint8_t* me = reinterpret_cast<uint8_t*>(heaps[ep->rank]);
  const bool pdl = (cfg->flags & B200MOE_FLAG_NO_PDL) == 0;
  const int sms = query_sms(cfg);
  const unsigned long long limit_ns = ep->wait_limit_ns > 0 ? ep->wait_limit_ns : kWaitLimitNs;
  int slot = -1;
  if (phases & B200MOE_EP_PHASE_DISPATCH) {
    if (!x || !topk_weights || !topk_ids || !placement) return B200MOE_ERR_BAD_ARG;
    if ((reinterpret_cast<uintptr_t>(x) & 15) != 0) return B200MOE_ERR_BAD_ARG;
    launch_log_new_call();
    slot = prof_slot();
    prof_mark(slot, 0, st);
    EpDispatchArgs d = {};
    d.world = ep->world;
    d.rank = ep->rank;
    d.m = cfg->M;
    d.m_cap = ep->m_cap;
    d.H = cfg->H;
    d.topk = cfg->topk;
    d.n_global_experts = ep->n_global_experts;
    d.dtype = cfg->dtype;
    d.fp8_rows = 1;
    d.ids_i64 = (cfg->flags & B200MOE_FLAG_IDS_I64) ? 1 : 0;
    d.clear_pairs = L.pair_rows ? 1 : 0;
    d.x = x;
    d.topk_weights = topk_weights;
    d.topk_ids = topk_ids;
    d.placement = placement;
    for (int r = 0; r < ep->world; ++r) d.heap[r] = reinterpret_cast<uint8_t*>(heaps[r]);
    d.L = H;
    if ((rc = launch_ep_dispatch(d, sms, st, pdl)) != B200MOE_OK) return rc;
  }
  if (phases & B200MOE_EP_PHASE_COMPUTE) {
    if (slot < 0 && (phases & B200MOE_EP_PHASE_DISPATCH) == 0) slot = prof_slot_current();
    // Two flags per peer: "ready" (its routing entries are in place) is what the first alignment kernel
    // waits for in its prologue, "rows" (its token rows are in place, raised later) what the gather waits
    // for, so the alignment overlaps the tail of the peers' dispatch.  Only while a benchmark is timing
    // the local operator the wait is a kernel of its own, so that the span can start after it.
    const FlagWait ready = ep_flag_wait(me, H, kEpFlagReady, ep->world, limit_ns, status);
    const FlagWait rows = ep_flag_wait(me, H, kEpFlagRows, ep->world, limit_ns, status);
    if (slot >= 0) {
      if ((rc = launch_ep_wait(rows, st, pdl)) != B200MOE_OK) return rc;    // "rows" is raised after "ready"
      prof_mark(slot, 6, st);
    }
    // alignment over every received row: ids are already local (or -1), weights already masked
    rc = align_into_workspace(&c, L, ws, me + H.recv_ids, 0, nullptr, reinterpret_cast<const float*>(me + H.recv_w), st,
                              slot >= 0 ? nullptr : &ready);
    if (rc != B200MOE_OK) return rc;
    b200moe_quant q = *quant;
    q.x_scale = reinterpret_cast<const float*>(me + H.recv_xs);
    PeerOut po;
    po.n_peers = ep->world;
    po.tokens_per_peer = ep->m_cap;
    po.rows_wait = slot >= 0 ? nullptr : &rows;
    for (int r = 0; r < ep->world; ++r) {
      uint8_t* h = reinterpret_cast<uint8_t*>(heaps[(cfg->flags & B200MOE_FLAG_EP_DIAG_LOCAL_COMBINE) ? ep->rank : r]);
      po.out32[r] = h + H.out32;
      po.pairs[r] = h + H.pairs;
      po.pair_valid[r] = h + H.pair_valid;
    }
    if ((rc = run_experts(&c, L, me + H.recv_x, w1, w2, &q, ws, nullptr, status, st, slot, &po)) != B200MOE_OK) return rc;
    uint8_t* hp[kMaxPeers];
    for (int r = 0; r < ep->world; ++r) hp[r] = reinterpret_cast<uint8_t*>(heaps[r]);
    if ((rc = launch_ep_signal(hp, H, kEpFlagDone, ep->world, ep->rank, st, pdl)) != B200MOE_OK) return rc;
    prof_mark(slot, 7, st);
  }
  if (phases & B200MOE_EP_PHASE_COMBINE) {
    if (!out || (reinterpret_cast<uintptr_t>(out) & 15) != 0) return B200MOE_ERR_BAD_ARG;
    if (slot < 0 && (phases & B200MOE_EP_PHASE_DISPATCH) == 0) slot = prof_slot_current();
    // every CTA of the output conversion waits for the peers' "done" flags in its prologue
    const FlagWait done = ep_flag_wait(me, H, kEpFlagDone, ep->world, limit_ns, status);
    if (cfg->M > 0) {
      if (L.pair_rows)
        rc = launch_finalize_pairs(me + H.pairs, me + H.pair_valid, out, cfg->dtype, cfg->M, cfg->topk, cfg->H,
                                   cfg->routed_scaling, sms, st, pdl, &done);
      else
        rc = launch_finalize(reinterpret_cast<const float*>(me + H.out32), out, cfg->dtype,
                             static_cast<size_t>(cfg->M) * cfg->H, cfg->routed_scaling, sms, st, pdl, &done);
      if (rc != B200MOE_OK) return rc;
    } else if ((rc = launch_ep_wait(done, st, pdl)) != B200MOE_OK) {
      return rc;    // a rank without tokens still takes part in the handshake
    }
    prof_mark(slot, 5, st);
  }
  return B200MOE_OK;
}

int b200moe_profile_begin(int max_calls) {
  if (max_calls <= 0 || max_calls > 4096) return B200MOE_ERR_BAD_ARG;
  std::lock_guard<std::mutex> lk(g_prof.mu);
  for (cudaEvent_t e : g_prof.ev) cudaEventDestroy(e);
  g_prof.ev.assign(static_cast<size_t>(max_calls) * kMarks, nullptr);
  g_prof.local_marked.assign(static_cast<size_t>(max_calls), 0);
  for (auto& e : g_prof.ev)
    if (cudaEventCreate(&e) != cudaSuccess) return B200MOE_ERR_CUDA;
  g_prof.max_calls = max_calls;
  g_prof.calls = 0;
  g_prof.on = true;
  return B200MOE_OK;
}

int b200moe_profile_end(double* gemm1_ms, double* gemm2_ms, double* total_ms, double* local_ms, int* calls) {
  std::lock_guard<std::mutex> lk(g_prof.mu);
  if (!g_prof.on) return B200MOE_ERR_BAD_ARG;
  g_prof.on = false;
  double g1 = 0, g2 = 0, tot = 0, loc = 0;
  int rc = B200MOE_OK;
  for (int i = 0; i < g_prof.calls; ++i) {
    cudaEvent_t* e = &g_prof.ev[static_cast<size_t>(i) * kMarks];
    float a = 0, b = 0, t = 0;
    if (cudaEventSynchronize(e[5]) != cudaSuccess || cudaEventElapsedTime(&a, e[1], e[2]) != cudaSuccess ||
        cudaEventElapsedTime(&b, e[3], e[4]) != cudaSuccess || cudaEventElapsedTime(&t, e[0], e[5]) != cudaSuccess) {
      rc = B200MOE_ERR_CUDA;
      break;
    }
    g1 += a; g2 += b; tot += t;
    // expert-parallel calls also mark their local operator; elsewhere the whole call is local
    float l = t;
    if (g_prof.local_marked[i] && cudaEventElapsedTime(&l, e[6], e[7]) != cudaSuccess) {
      rc = B200MOE_ERR_CUDA;
      break;
    }
    loc += l;
  }
  if (local_ms) *local_ms = loc;
  if (gemm1_ms) *gemm1_ms = g1;
  if (gemm2_ms) *gemm2_ms = g2;
  if (total_ms) *total_ms = tot;
  if (calls) *calls = g_prof.calls;
  for (cudaEvent_t e : g_prof.ev) cudaEventDestroy(e);
  g_prof.ev.clear();
  g_prof.calls = 0;
  return rc;
}

int b200moe_per_token_group_quant_fp8(const void* x, int dtype, int rows, int K, void* q, float* scales,
                                      void* stream) {
  if (rows < 0 || K <= 0 || !x || !q || !scales) return B200MOE_ERR_BAD_ARG;
  if (dtype != B200MOE_DTYPE_BF16 && dtype != B200MOE_DTYPE_FP16) return B200MOE_ERR_BAD_ARG;
  if (rows == 0) return B200MOE_OK;
  return launch_group_quant_fp8(x, dtype, q, scales, nullptr, nullptr, 0, 1, rows, K, 0, 0, nullptr, 0,
                                query_sms(nullptr), static_cast<cudaStream_t>(stream), false);
}

int b200moe_debug_resident_cta_pairs(void) { return gemm_tc2_resident_pairs(); }

int b200moe_launch_stats(long long* total_launches, char* last_call_names, size_t names_bytes) {
  std::lock_guard<std::mutex> lk(g_launches.mu);
  if (total_launches) *total_launches = g_launches.total;
  int n = 0;
  for (char ch : g_launches.last_call) n += ch == ',';
  if (!g_launches.last_call.empty()) ++n;
  if (last_call_names != nullptr && names_bytes > 0) {
    const size_t len = g_launches.last_call.size() < names_bytes - 1 ? g_launches.last_call.size() : names_bytes - 1;
    memcpy(last_call_names, g_launches.last_call.data(), len);
    last_call_names[len] = 0;
  }
  return n;
}

int b200moe_selftest_timeout(uint64_t limit_ns, int32_t* status, int32_t* observed, void* stream) {
  if (status == nullptr || observed == nullptr || limit_ns == 0 || limit_ns > 100000000ull) return B200MOE_ERR_BAD_ARG;
  return launch_selftest_timeout(limit_ns, status, observed, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
