// Host-callable launchers of the row movers around the grouped GEMMs.
#pragma once
#include "common.cuh"

namespace b200moe {

// xs[r] = x[sorted_ids[r] / topk] for r < meta[1]; padding rows zero-filled.  Also clears
// `zero_bytes` bytes at `zero` (the fp32 combine buffer) in the same launch.  With sc_src
// ([tokens][G] group scales of already quantised rows) the scales follow their rows into the
// group-major table sc_dst [G][ld].  `wait` (expert parallelism): every CTA first waits for the
// peers' flags (common.cuh: FlagWait).
int launch_gather_rows(const void* x, void* xs, const int* sorted_ids, const int* meta, int P, int topk,
                       int row_bytes, int cap, void* zero, size_t zero_bytes, int num_sms,
                       cudaStream_t stream, bool pdl, const float* sc_src = nullptr, float* sc_dst = nullptr,
                       int G = 0, int ld = 0, const FlagWait* wait = nullptr);

// Per-token-group (1x128) FP8 quantisation, optionally gathering rows through
// sorted_ids like launch_gather_rows.  scale_t: store scales group-major.
int launch_group_quant_fp8(const void* x, int dtype, void* q, float* scales, const int* sorted_ids,
                           const int* meta, int P, int topk, int rows, int K, int scale_t, int ld_scale,
                           void* zero, size_t zero_bytes, int num_sms, cudaStream_t stream, bool pdl);

// fp16 token rows -> the integer form the int4 decode kernels read: per (row, 128-k group) a
// power-of-two scale f (2^(e-18) for a group maximum in [2^e, 2^(e+1))), the exact integers
// v = rint(x / f) split into three signed byte planes (v = p0 + 256 p1 + 65536 p2) and their sum.
// planes: [block][plane][BT rows][K] int8, inside each aligned run of eight k the order
// (0, 4, 1, 5, 2, 6, 3, 7); scales / sums: [K/128][ld].  Rows are gathered through sorted_ids.
int launch_group_split_i8(const void* x, uint8_t* planes, float* scales, int* sums, const int* sorted_ids,
                          const int* meta, int P, int topk, int cap, int K, int BT, int ld, void* zero,
                          size_t zero_bytes, int num_sms, cudaStream_t stream, bool pdl);

// out[i] = cast(acc[i] * scale)
// `wait` (expert parallelism): every CTA first waits for the peers' flags (common.cuh: FlagWait).
int launch_finalize(const float* acc, void* out, int dtype, size_t n, float scale, int num_sms,
                    cudaStream_t stream, bool pdl, const FlagWait* wait = nullptr);

// out[t][c] = cast(scale * sum_j pairs[t * topk + j][c]) over the pairs marked valid.
int launch_finalize_pairs(const void* pairs, const uint8_t* pair_valid, void* out, int dtype, int M, int topk,
                          int H, float scale, int num_sms, cudaStream_t stream, bool pdl,
                          const FlagWait* wait = nullptr);

// Provokes a device-side time-out on purpose (see selftest.cu): observed[0] = 0 when the short wait
// ran out, observed[1] = 0 when the sibling wait was released by the abort flag, observed[2] = the
// microseconds the sibling waited; the status word receives DEV_TIMEOUT_SELFTEST.
int launch_selftest_timeout(unsigned long long limit_ns, int* status, int* observed, cudaStream_t stream);

}  // namespace b200moe
