// Matrix-vector path for a handful of tokens (decode with one or two tokens in flight).
//
// With M * topk <= kGemvMaxPairs every (token, choice) pair is an independent pair of
// matrix-vector products, and the whole operator is bound by streaming each chosen expert's
// weights from HBM once.  Tensor-core tiles buy nothing there; what costs is the launch chain
// (alignment, gather, two grouped GEMMs, output conversion).  Two launches replace it: the first
// reads the routing straight from topk_ids / topk_weights and writes the activations of every
// pair, the second sums a token's pairs in a fixed order and writes the output in its final
// type.  CUDA cores only; weights are read with 16-byte loads, one warp per output column (gate and
// up row together) or per two output elements.  16-bit weights, and int4 weights on integer dot
// products (dp4a on raw nibbles and three int8 activation planes, one instruction per weight); FP8
// rows would be converted element by element, which costs more than the launches saved.
#pragma once
#include "common.cuh"

namespace b200moe {

constexpr int kGemvMaxPairs = 16;

struct GemvArgs {
  const void* x;            // [M, H] 16-bit
  const void* w1;           // [E, 2I, H] 16-bit (gate rows, then up rows); int4: packed rows [E, 2I, H/8] int32
  const void* w2;           // [E, H, I]
  const float* topk_w;      // [M, topk]
  const void* topk_ids;     // [M, topk] int32 / int64
  const int* expert_map;    // global -> local expert id or -1; nullptr: ids are local
  // alternative routing input (then topk_w / topk_ids are unused): the routing triple of the
  // operator-level entry point
  const int* hist;          // [E] rows per expert, or nullptr
  const int* topk_indx;     // [P] sorted row -> pair slot
  const float* gate_scal;   // [P] routing weight of each sorted row
  int ids_i64, n_global;
  int M, H, I, E, topk;
  int dtype, w4, activation, flags;   // w4: int4 (AWQ) weights in the kernel layout, fp16 activations
  int round_pair;           // round each pair's weighted row to the 16-bit type before the sum
  int down_split;           // set by the launcher: warps that share one output task of the down kernel (1, 2, 4, 8)
  float alpha, limit, routed_scaling;
  const float* b1;          // [E, 2I] or nullptr
  const float* b2;          // [E, H] or nullptr
  const void* w1_sz;        // int4: [E, H/128, 2I] int32 = fp16 scale | fp16(1024 + zero) << 16
  const void* w2_sz;        // int4: [E, I/128, H]
  void* act;                // scratch [P, I] in the 16-bit type
  void* out;                // [M, H], or [P, H] when nothing is combined
};

size_t gemv_up_smem(const GemvArgs& a);
size_t gemv_down_smem(const GemvArgs& a);
// true if the pair count and the shared-memory staging (token rows / activations of every pair as
// fp32) allow this path; otherwise the caller takes the grouped-GEMM path
bool gemv_fits(const GemvArgs& a);
int launch_gemv_up(const GemvArgs& a, int num_sms, cudaStream_t stream, bool pdl);
int launch_gemv_down(const GemvArgs& a, int num_sms, cudaStream_t stream, bool pdl);

}  // namespace b200moe
