// Grouped expert GEMMs: argument block and launchers.
#pragma once
#include "common.cuh"

namespace b200moe {

// Orientation: the expert weight tile sits on the 128-row side of the tensor-core
// instruction and the (block of) tokens on its N side, so a decode-sized token
// block of 16 wastes nothing and a prefill block of 256 fills the widest shape.
constexpr int kMaxPeers = 8;   // ranks of one NVSwitch domain that an expert-parallel call may span

struct GemmArgs {
  int mode;        // 0: gate/up projection + activation; 1: down projection + weighted scatter-add
  int dtype;       // B200MOE_DTYPE_* of activations / 16-bit weights
  int wmode;       // B200MOE_W_*
  int E;           // local experts
  int K;           // reduction length (H for mode 0, I for mode 1)
  int N;           // output rows per expert covered by tiles of 128 (I for mode 0, H for mode 1)
  int up_row_off;  // mode 0: row of the first "up" weight inside an expert (= I)
  int orient;      // 0: weight rows on the MMA's M side (decode); 1: tokens on the M side (BT = 128)
  int BT;          // tokens per block (16..256, multiple of 16)
  int stages;      // shared-memory ring depth
  int acc_stages;  // accumulator buffers in tensor memory (1 or 2)
  int tmem_cols;   // allocated tensor-memory columns (power of two >= 32)
  int num_nt;      // ceil(N / 128)
  int kblocks;     // ceil(K / kblock elements)
  int topk;
  int P;           // M * topk
  int flags;       // B200MOE_FLAG_*
  int activation;  // B200MOE_ACT_*
  int max_split;   // mode 1: upper bound for the reduction split
  int pdl;         // launch with programmatic stream serialisation
  const int* meta;        // [0] = token blocks, [1] = padded rows
  const int* blk_off;     // [E+1] first block of each expert
  const int* sorted_ids;  // [cap] slot of each padded row (>= P: padding)
  const float* row_gamma; // [cap] routing weight of each padded row
  void* out;              // mode 0: activations [cap, N]; mode 1: fp32 combine buffer [M, N]
  long long ld_out;       // row stride of out in elements
  int* status;            // device status word
  // FP8 block-scaled mode
  const float* w_scale;   // [E, ceil(rows/128), ceil(K/128)] (rows = 2I for mode 0)
  const float* x_scale;   // [K/128][ld_xscale] group-major activation scales
  int ld_xscale;
  int w_scale_rows;       // scale rows per expert
  const float* bias;      // optional per-expert bias of this GEMM's output rows: [E, rows] fp32 (mode 0: gate rows then up rows)
  float act_alpha;        // B200MOE_ACT_SWIGLU_OAI: s = g * sigmoid(alpha * g)
  float act_limit;        // B200MOE_ACT_SWIGLU_OAI: clamp gate to <= limit and linear to [-limit, limit]; <= 0: none
  const void* w_sz;       // int4: per (expert, group of 128 k, weight row) fp16 scale | fp16 (1024 + zero)
  int w_rows;             // int4: weight rows per expert (2I for mode 0, H for mode 1)
  uint8_t* out_q;         // mode 0 FP8: quantised activations [cap, N]
  float* out_scale;       // mode 0 FP8: [N/128][ld_xscale]
  // int4 decode path (integer MMAs): activations are three int8 planes per token block
  // ([block][plane][BT rows][K], rows of one block consecutive) + per (128-k group, row) a
  // power-of-two scale (x_scale / out_scale, [K/128][ld_xscale]) and the sum of the integers
  // mode 1, optional: instead of adding into the fp32 combine buffer, store each (token, choice)
  // pair's weighted row in the 16-bit type at out_pairs[slot][N] and mark pair_valid[slot]; the
  // output conversion then sums a token's rows.  Plain 16-byte stores instead of fp32 atomics,
  // which bound the tail once M * topk * N is large.  Requires an unsplit reduction.
  void* out_pairs;
  uint8_t* pair_valid;
  const int* x_sum;       // [K/128][ld_xscale]
  int* out_sum;           // mode 0: [N/128][ld_xscale]; planes go to out_q with row stride ld_out
  // mode 1 under expert parallelism (FP8 kernels): the output row of a token (fp32 combine buffer)
  // or of a pair (16-bit pair rows) lives on the rank that owns the token.  Output row index r
  // (token, or pair slot, numbered rank-major over all ranks) -> rank r / rows_per_peer, row
  // r % rows_per_peer of that rank's buffer, reached through its peer mapping.  n_peers <= 1:
  // everything stays in `out` / `out_pairs` of this GPU.
  int n_peers;
  int rows_per_peer;
  void* peer_out[kMaxPeers];          // out (fp32) or out_pairs (16-bit) of every rank
  uint8_t* peer_valid[kMaxPeers];     // pair_valid of every rank (pair rows only)
};

// Base address of output row `orow` (row_bytes bytes per row): local, or on the owning rank.
__device__ __forceinline__ uint8_t* out_row_base(const GemmArgs& a, void* local, int orow, size_t row_bytes) {
  if (a.n_peers <= 1) return reinterpret_cast<uint8_t*>(local) + static_cast<size_t>(orow) * row_bytes;
  const int peer = orow / a.rows_per_peer;
  return reinterpret_cast<uint8_t*>(a.peer_out[peer]) + static_cast<size_t>(orow - peer * a.rows_per_peer) * row_bytes;
}
__device__ __forceinline__ void mark_pair_valid(const GemmArgs& a, int slot) {
  if (a.n_peers <= 1) {
    a.pair_valid[slot] = 1;
  } else {
    const int peer = slot / a.rows_per_peer;
    a.peer_valid[peer][slot - peer * a.rows_per_peer] = 1;
  }
}

size_t gemm_smem_bytes(const GemmArgs& a);
bool gemm_w4_planes_ok(int K, int BT);   // can the integer int4 path take this reduction length / token block?
void gemm_plan(GemmArgs* a);  // fills stages / acc_stages / tmem_cols / num_nt / kblocks from the rest

int launch_gemm_tc(const CUtensorMap& tm_w, const CUtensorMap& tm_x, const GemmArgs& a, int num_sms,
                   cudaStream_t stream);
void gemm_plan_fp8(GemmArgs* a);
int launch_gemm_fp8(const CUtensorMap& tm_w, const CUtensorMap& tm_x, const GemmArgs& a, int num_sms,
                    cudaStream_t stream);
// int4 AWQ, token blocks of 16 / 32: exact (q - zero) operands, group scales applied to partial sums
void gemm_plan_w4(GemmArgs* a);
int launch_gemm_w4(const CUtensorMap& tm_w, const CUtensorMap& tm_x, const GemmArgs& a, int num_sms,
                   cudaStream_t stream);
// 16-bit, 128-token blocks, on CTA pairs (tcgen05.mma.cta_group::2): see gemm_tc2.cu
bool gemm_tc2_ok(const GemmArgs& a);
int gemm_tc2_resident_pairs();   // CTA pairs the device kept resident for the last such launch (0: none yet)
void gemm_plan_tc2(GemmArgs* a);
int launch_gemm_tc2(const CUtensorMap& tm_w, const CUtensorMap& tm_x, const GemmArgs& a, int num_sms,
                    cudaStream_t stream);
int launch_gemm_simt(const void* w, const void* x, const GemmArgs& a, cudaStream_t stream, int cap);

}  // namespace b200moe
