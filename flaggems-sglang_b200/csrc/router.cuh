// Router front-end (gating logits -> top-k weights and ids).
#pragma once
#include "common.cuh"

namespace b200moe {

int check_router(const b200moe_router* r, int E, int topk);

// logits [M, E] in r->logits_dtype; out_w [M, topk] fp32, out_ids [M, topk] int32.
int launch_route_topk(const b200moe_router* r, const void* logits, int M, int E, int topk, float* out_w,
                      int* out_ids, int num_sms, cudaStream_t stream);

}  // namespace b200moe
