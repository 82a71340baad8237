// Host-callable launchers of the routing / alignment kernels.
#pragma once
#include "common.cuh"

namespace b200moe {

int align_capacity(int n_slots, int n_experts, int block);
int routing_max_tiles(int n_slots, int n_experts);

// `map` (optional, `map_len` entries): global expert id -> local expert, negative = not held here;
// ids at or beyond map_len are dropped like negative ones.
// Block-aligned grouping (+ optional internal tables for the GEMMs: per-row
// routing weight, per-expert block prefix, meta[0] = blocks, meta[1] = rows).
int launch_align_block(const void* ids, int is64, const int* map, int map_len, const float* weights, int P, int E,
                       int block, int cap, int* sorted_ids, int* expert_ids, int* num_post_pad,
                       float* row_gamma, int* blk_off, int* meta, cudaStream_t stream, bool pdl = false,
                       const FlagWait* wait = nullptr);

// `pdl`: launch with programmatic stream serialisation; `wait` (expert parallelism): the first kernel
// waits for the peers' flags before it reads the ids.
// The same tables from 32 CTAs in two launches (tens of thousands of slots); `tmp` holds
// align_multi_tmp_bytes(E) bytes of scratch.  Output identical to launch_align_block.
size_t align_multi_tmp_bytes(int E);
int launch_align_block_multi(const void* ids, int is64, const int* map, int map_len, const float* weights, int P, int E,
                             int block, int cap, int* sorted_ids, int* expert_ids, int* num_post_pad,
                             float* row_gamma, int* blk_off, int* meta, int* tmp, cudaStream_t stream,
                             bool pdl = false, const FlagWait* wait = nullptr);

// Same internal tables from hist / topk_indx / gate_scal of the routing triple.
int launch_align_from_routing(const int* hist, const int* topk_indx, const float* gate_scal, int P,
                              int E, int block, int cap, int* sorted_ids, float* row_gamma,
                              int* blk_off, int* meta, cudaStream_t stream);

int launch_routing_from_topk(const float* weights, const void* ids, int is64, int M, int k, int E,
                             int* expt_indx, int* topk_indx, int* gate_indx, float* gate_scal,
                             int* hist, int* token_offs_raw, int* token_offs_pad, int* block_pid_map,
                             cudaStream_t stream);

}  // namespace b200moe
