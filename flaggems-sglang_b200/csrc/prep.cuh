// Host-callable launchers of the row movers around the grouped GEMMs.
#pragma once
#include "common.cuh"

namespace b200moe {

// xs[r] = x[sorted_ids[r] / topk] for r < meta[1]; padding rows zero-filled.  Also clears
// `zero_bytes` bytes at `zero` (the fp32 combine buffer) in the same launch.
int launch_gather_rows(const void* x, void* xs, const int* sorted_ids, const int* meta, int P, int topk,
                       int row_bytes, int cap, void* zero, size_t zero_bytes, int num_sms,
                       cudaStream_t stream, bool pdl);

// Per-token-group (1x128) FP8 quantisation, optionally gathering rows through
// sorted_ids like launch_gather_rows.  scale_t: store scales group-major.
int launch_group_quant_fp8(const void* x, int dtype, void* q, float* scales, const int* sorted_ids,
                           const int* meta, int P, int topk, int rows, int K, int scale_t, int ld_scale,
                           void* zero, size_t zero_bytes, int num_sms, cudaStream_t stream, bool pdl);

// out[i] = cast(acc[i] * scale)
int launch_finalize(const float* acc, void* out, int dtype, size_t n, float scale, int num_sms,
                    cudaStream_t stream, bool pdl);

}  // namespace b200moe
