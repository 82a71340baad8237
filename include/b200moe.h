/*
 * b200moe.h -- C ABI of the B200 (sm_100a) fused Mixture-of-Experts library.
 *
 * Every entry point takes plain device pointers, integers and a CUDA stream
 * (passed as void* so that this header needs no CUDA include), launches
 * asynchronously on that stream, allocates nothing and never synchronises.
 * Return value: 0 on success, a negative B200MOE_ERR_* code otherwise.
 * Device-side problems (a bounded wait that ran out) are reported through the
 * caller-provided status word, which the caller reads after synchronising.
 *
 * Each declaration names the reference interface it stands in for, by the
 * file's path inside the flagos-ai/FlagGems-sglang tree.
 */
#ifndef B200MOE_H_
#define B200MOE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200MOE_VERSION 2

/* status codes */
#define B200MOE_OK 0
#define B200MOE_ERR_BAD_ARG (-1)
#define B200MOE_ERR_UNSUPPORTED (-2)
#define B200MOE_ERR_WORKSPACE (-3)
#define B200MOE_ERR_CUDA (-4)
#define B200MOE_ERR_DEVICE_TIMEOUT (-5)
#define B200MOE_ERR_TOO_LARGE (-6)

/* activation / output element type */
#define B200MOE_DTYPE_BF16 0
#define B200MOE_DTYPE_FP16 1
#define B200MOE_DTYPE_FP32 2 /* router logits only */

/* weight storage */
#define B200MOE_W_16BIT 0     /* same 16-bit type as the activations               */
#define B200MOE_W_FP8_BLOCK 1 /* e4m3fn, fp32 scale per 128x128 block              */
#define B200MOE_W_INT4_AWQ 2  /* uint4 g128 in the kernel layout (see b200moe_quant)  */

/* weight layout (16-bit weights only) */
#define B200MOE_LAYOUT_LAYER 0 /* w1 [E,2I,H], w2 [E,H,I]: reduction dim contiguous */
#define B200MOE_LAYOUT_OP 1    /* w1 [E,H,2I], w2 [E,I,H]: output dim contiguous    */

#define B200MOE_ACT_SILU 0
#define B200MOE_ACT_GELU 1
#define B200MOE_ACT_SWIGLU_OAI 2 /* s = g*sigmoid(alpha*g) with clamps; out = s*(linear + 1): the bias variant's activation */

/* cfg.flags */
#define B200MOE_FLAG_WEIGHT_ON_INPUT 1  /* router weight scales GEMM-1's output, not GEMM-2's */
#define B200MOE_FLAG_MIMIC_ROUNDING 2   /* round intermediates to the 16-bit type where the reference does */
#define B200MOE_FLAG_SIMT 4             /* plain CUDA-core GEMMs (validation aid, slow)        */
#define B200MOE_FLAG_IDS_I64 8          /* topk_ids are int64 instead of int32                 */
#define B200MOE_FLAG_NO_SPLIT_K 16      /* keep GEMM-2's reduction in one piece                */
#define B200MOE_FLAG_NO_GRID_BALANCE 32 /* tuning aid: every CTA takes tiles round-robin       */
#define B200MOE_FLAG_NO_PDL 64          /* launch every kernel fully serialised                */
#define B200MOE_FLAG_W4_SMEM_OPERANDS 128 /* int4: always stage fp16 operands in shared memory (tuning aid) */
#define B200MOE_FLAG_X_FP8 1024         /* FP8 weights only: x is already e4m3 [M, H], quantised per
                                           1 x 128 group with scales quant->x_scale [M, H/128] (what
                                           b200moe_per_token_group_quant_fp8 writes); cfg->dtype still
                                           names the 16-bit type of the intermediate and the output   */
#define B200MOE_FLAG_EP_DIAG_LOCAL_COMBINE 2048 /* tuning aid, expert parallelism: the down projection's rows stay on
                                           this GPU (WRONG results; isolates the cost of the peer stores)      */
#define B200MOE_FLAG_CTA_PAIR 4096      /* 16-bit prefill (128-token blocks): run the grouped GEMMs on CTA pairs
                                           (tcgen05.mma.cta_group::2) where the shape allows                   */
#define B200MOE_FLAG_ALIGN_ONE_CTA 512  /* tuning aid: single-CTA alignment however many slots           */
#define B200MOE_FLAG_NO_COMBINE 256     /* out is [M*topk, H]: row t*topk+j holds pair j of token t,
                                           routing weight applied, nothing summed, routed_scaling ignored
                                           (the adapter's no_combine, fused_moe.py:392-397)               */

typedef struct b200moe_cfg {
  int32_t struct_bytes;   /* sizeof(b200moe_cfg), checked                      */
  int32_t M;              /* tokens                                             */
  int32_t H;              /* hidden size                                        */
  int32_t I;              /* intermediate size (w1 has 2*I output rows)         */
  int32_t E;              /* experts held locally                               */
  int32_t topk;           /* experts per token                                  */
  int32_t dtype;          /* B200MOE_DTYPE_*                                    */
  int32_t wmode;          /* B200MOE_W_*                                        */
  int32_t w_layout;       /* B200MOE_LAYOUT_*                                   */
  int32_t activation;     /* B200MOE_ACT_*                                      */
  int32_t flags;          /* B200MOE_FLAG_*                                     */
  int32_t block_tokens;   /* token block of the GEMMs: 0 = choose, else 16..256.
                             With 0, 16-bit or int4 weights and at most 16 (token, expert)
                             pairs the forward calls run two matrix-vector kernels
                             instead of the grouped GEMMs; a non-zero value keeps
                             every call on the grouped GEMMs                     */
  float routed_scaling;   /* output multiplier (1.0f for none)                  */
  int32_t num_sms;        /* 0 = query the current device                       */
  int32_t n_global_experts; /* entries of expert_map (required > 0 when a map is passed); ids at or
                             beyond it are dropped like ids the map sends to a negative value      */
} b200moe_cfg;

/* scales / zero points for the quantised weight modes and the optional per-expert biases
 * (NULL members unused) */
typedef struct b200moe_quant {
  const float *w1_scale;  /* FP8: [E, ceil(2I/128), ceil(H/128)]                 */
  const float *w2_scale;  /* FP8: [E, ceil(H/128), ceil(I/128)]                  */
  /* int4 AWQ (fp16 activations).  w1 / w2 then point at packed rows [E, rows, K/8] int32,
   * one output row per line, eight consecutive k per word (element 2i in nibble i, element
   * 2i+1 in nibble 4+i); w*_sz are [E, K/128, rows] int32 = fp16 scale | fp16(1024 + zero) << 16.
   * flaggems_sglang_b200.quant.repack_awq_for_kernel builds both from AWQ checkpoint tensors. */
  const void *w1_sz;
  const void *w2_sz;
  /* per-expert biases (every weight mode), fp32.  b1 [E, 2I] (gate rows, then up / linear
   * rows, matching w1's row order), b2 [E, H]; added to the GEMM outputs before activation /
   * routing weight, as triton_kernel_fused_experts_with_bias does
   * (src/flaggems_sglang/ops/fused_moe.py:285-308). */
  const float *b1;
  const float *b2;
  float swiglu_alpha;     /* B200MOE_ACT_SWIGLU_OAI */
  float swiglu_limit;     /* B200MOE_ACT_SWIGLU_OAI: <= 0 disables the clamps */
  const float *x_scale;   /* B200MOE_FLAG_X_FP8: [M, H/128] activation scales    */
} b200moe_quant;

int b200moe_version(void);
const char *b200moe_status_string(int code);

/* Token block the library would pick for this problem (16, 32, 64, 128 or 256). */
int b200moe_pick_block_tokens(const b200moe_cfg *cfg);

/* 1 if the forward calls would run this problem on the two matrix-vector kernels (16-bit or int4
 * weights, block_tokens = 0, at most 16 (token, expert) pairs: one token, or several while
 * pairs <= experts / 4, and the staged rows fit in shared memory), 0 if on the grouped GEMMs,
 * negative B200MOE_ERR_* for a bad cfg.  Host arithmetic only.  No reference counterpart. */
int b200moe_uses_matrix_vector_path(const b200moe_cfg *cfg);

/* Bytes of scratch b200moe_forward_* needs for this problem (256-byte aligned base). */
size_t b200moe_workspace_bytes(const b200moe_cfg *cfg);

/*
 * Block-aligned grouping of the flat slot ids i = token*topk + j by expert.
 * Stands in for the alignment step the reference delegates to its dependency's
 * routing tables (src/flaggems_sglang/ops/fused_moe.py:103-130); the output
 * contract is the serving ecosystem's moe_align_block_size:
 *   sorted_token_ids[cap]   expert 0's slots ascending, sentinel n_slots up to a
 *                           multiple of `block`, expert 1's slots, ...; tail = n_slots
 *   expert_ids[ceil(cap/block)]  expert of each block; tail = -1
 *   num_tokens_post_padded[1]
 * cap = b200moe_align_capacity(n_slots, n_experts, block).  expert_map (may be
 * NULL; expert_map_len entries) maps global ids to local experts, negative = not
 * local (slot dropped); ids outside [0, expert_map_len) are dropped too.
 */
int b200moe_align_capacity(int n_slots, int n_experts, int block);
int b200moe_align_block_size(const void *topk_ids, int ids_are_i64, int n_slots,
                             int n_experts, int block, const int32_t *expert_map,
                             int expert_map_len, int32_t *sorted_token_ids,
                             int32_t *expert_ids, int32_t *num_tokens_post_padded,
                             void *stream);

/*
 * top-k -> routing tables.  Replaces _standard_topk_to_triton_kernels
 * (src/flaggems_sglang/ops/fused_moe.py:103-130) and the expert-data tables it
 * obtains from its dependency.  All outputs int32 unless noted:
 *   expt_indx[P], topk_indx[P], gate_indx[P], gate_scal[P] (fp32), hist[E],
 *   token_offs_raw[E+1], token_offs_pad[4][E+1], block_pid_map[4][max_tiles]
 * for block sizes 16, 32, 64, 128; max_tiles = b200moe_routing_max_tiles(P, E).
 */
int b200moe_routing_max_tiles(int n_slots, int n_experts);
int b200moe_routing_from_topk(const float *topk_weights, const void *topk_ids,
                              int ids_are_i64, int n_tokens, int topk, int n_experts,
                              int32_t *expt_indx, int32_t *topk_indx, int32_t *gate_indx,
                              float *gate_scal, int32_t *hist, int32_t *token_offs_raw,
                              int32_t *token_offs_pad, int32_t *block_pid_map,
                              void *stream);

/*
 * Fused experts from top-k routing.  Replaces triton_kernel_fused_experts
 * (src/flaggems_sglang/ops/fused_moe.py:133-216) preceded by the routing
 * conversion of fused_moe_flagos (same file, 339-350).
 *   x [M,H], out [M,H] of cfg.dtype; topk_weights [M,topk] fp32; topk_ids
 *   [M,topk] int32 (int64 with B200MOE_FLAG_IDS_I64); expert_map may be NULL.
 *   status: device int32, set non-zero if a device-side wait gave up.
 */
int b200moe_forward_topk(const b200moe_cfg *cfg, const void *x, const void *w1,
                         const void *w2, const b200moe_quant *quant,
                         const float *topk_weights, const void *topk_ids,
                         const int32_t *expert_map, void *workspace,
                         size_t workspace_bytes, void *out, int32_t *status,
                         void *stream);

/*
 * Same computation as b200moe_forward_topk for callers that cannot provide a
 * workspace and must not allocate one.  No counterpart in the reference (its
 * operator allocates every intermediate through PyTorch on each call).
 *
 * Who needs it: a runtime that has handed all device memory to its own pools, a
 * plugin interface without a scratch argument, or a thread that may not enter
 * the CUDA allocator.  The scratch is an array of B200MOE_NOALLOC_SCRATCH_BYTES
 * that is part of the library image: every GPU that loads the library holds it
 * until the process exits.  The call itself allocates nothing and frees nothing.
 *
 * Limits and rules:
 *   - b200moe_workspace_bytes(cfg) must not exceed B200MOE_NOALLOC_SCRATCH_BYTES,
 *     else B200MOE_ERR_TOO_LARGE is returned and nothing is launched (16 MiB
 *     covers decode-sized batches, e.g. 16 tokens of the Mixtral-shaped layer or
 *     64 tokens of the Qwen3-30B-A3B-shaped one).
 *   - The first call on each device looks up the array's device address (with
 *     that device current); make that first call before any stream capture.
 *   - Every call on a device uses the same array and finds the previous call's
 *     contents in it; the call re-initialises all it reads.  Two calls that
 *     overlap on the GPU (different streams) race on the array: serialise them.
 *   - The looked-up address is kept for the life of the process.  After
 *     cudaDeviceReset (or any teardown of the device's primary context) it no
 *     longer points at the array: unload and reload the library before calling again.
 */
#define B200MOE_NOALLOC_SCRATCH_BYTES (16 * 1024 * 1024)
int b200moe_forward_topk_noalloc(const b200moe_cfg *cfg, const void *x, const void *w1,
                                 const void *w2, const b200moe_quant *quant,
                                 const float *topk_weights, const void *topk_ids,
                                 const int32_t *expert_map, void *out, int32_t *status,
                                 void *stream);

/*
 * Fused experts from the reference's routing triple.  Replaces
 * triton_kernel_fused_experts (src/flaggems_sglang/ops/fused_moe.py:133-216)
 * as the reference's tests call it (tests/test_fused_moe.py:94): hist[E] =
 * routing_data.expt_hist, topk_indx[P] = gather_indx.src_indx, gate_scal[P]
 * (fp32) = routing_data.gate_scal.
 */
int b200moe_forward_routed(const b200moe_cfg *cfg, const void *x, const void *w1,
                           const void *w2, const b200moe_quant *quant,
                           const int32_t *hist, const int32_t *topk_indx,
                           const float *gate_scal, void *workspace,
                           size_t workspace_bytes, void *out, int32_t *status,
                           void *stream);

/*
 * Router front-end: gating logits -> top-k routing weights and expert ids, the
 * step in front of the alignment.  The reference leaves it to the caller
 * (recipe at tests/test_fused_moe.py:21-27: softmax, top-k, divide by the sum);
 * grouped selection with an optional selection bias is the DeepSeek-V2 / -V3
 * rule (named `grouped_topk` in
 * src/flaggems_sglang/runtime/backend/_iluvatar/op_black_list.yaml:6-11).
 * Ties go to the lower expert id.
 */
#define B200MOE_SCORE_SOFTMAX 0
#define B200MOE_SCORE_SIGMOID 1
#define B200MOE_ROUTER_MAX_EXPERTS 1024
#define B200MOE_ROUTER_MAX_TOPK 32

typedef struct b200moe_router {
  int32_t struct_bytes;  /* sizeof(b200moe_router), checked                                   */
  int32_t scoring;       /* B200MOE_SCORE_*                                                   */
  int32_t renormalize;   /* 1: divide the k weights by their sum                              */
  int32_t n_group;       /* contiguous expert groups (<= 32, divides E); 0 or 1: no grouping  */
  int32_t topk_group;    /* groups that stay eligible                                         */
  int32_t logits_dtype;  /* B200MOE_DTYPE_BF16 / FP16 / FP32                                  */
  float scale;           /* multiplies the final weights; 0 is read as 1                      */
  int32_t reserved;
  const float *bias;     /* [E] added to the scores for selection only, or NULL; with groups,
                            a group's score becomes the sum of its two best biased scores    */
} b200moe_router;

/* logits [M, E]; topk_weights [M, topk] fp32 and topk_ids [M, topk] int32 on the device. */
int b200moe_route_topk(const b200moe_router *router, const void *logits, int n_tokens,
                       int n_experts, int topk, float *topk_weights, int32_t *topk_ids,
                       void *stream);

/*
 * Whole layer from gating logits: router, alignment, both grouped GEMMs and the
 * combine, one call, no host read in between.  Arguments as b200moe_forward_topk
 * with `logits [M, E]` in place of the top-k tensors.
 */
int b200moe_forward_logits(const b200moe_cfg *cfg, const b200moe_router *router, const void *x,
                           const void *w1, const void *w2, const b200moe_quant *quant,
                           const void *logits, const int32_t *expert_map, void *workspace,
                           size_t workspace_bytes, void *out, int32_t *status, void *stream);

/*
 * Expert parallelism inside one NVSwitch domain: experts are spread over `world`
 * ranks (one process per GPU), every rank brings its own tokens with routing over
 * the GLOBAL expert ids.  No counterpart in the reference, which rejects expert_map
 * (src/flaggems_sglang/ops/fused_moe.py:160-162) and contains no communication.
 *
 * Each rank owns a "heap" (b200moe_ep_heap_bytes; allocated once, at set-up, by
 * b200moe_ep_heap_alloc) and maps the heaps of the other ranks through CUDA IPC
 * (export / open, 64-byte handles carried by whatever channel the host has, e.g.
 * torch.distributed).  A forward call then moves data with plain stores into peer
 * heaps and synchronises with epoch flags; it contains no collective, allocates
 * nothing and reads nothing on the host:
 *   B200MOE_EP_PHASE_DISPATCH  quantise this rank's tokens (e4m3, 1x128 scales) and store each
 *                              row, with its routing entries translated through `placement`,
 *                              into the heap of every rank that holds one of its experts;
 *                              clear this rank's result buffer; raise "ready" on every peer.
 *   B200MOE_EP_PHASE_COMPUTE   wait for every peer's "ready"; alignment, gather and both grouped
 *                              GEMMs over the rows received; the down projection stores each
 *                              (token, choice) row into the heap of the rank that owns the token;
 *                              raise "done" on every peer.
 *   B200MOE_EP_PHASE_COMBINE   wait for every peer's "done"; out [M, H] = sum of the rows that
 *                              arrived for each of this rank's tokens (fixed order).
 * Normal use passes all three phases in one call.  Passing them one at a time lets one process
 * drive several ranks' heaps on ONE GPU in a single stream (all dispatches, then all computes,
 * then all combines), which is how the path is tested where only one GPU is available: flags
 * are then always raised before anything waits on them.
 * Every wait is bounded by ep->wait_limit_ns (0 = two seconds): when it runs out the kernel
 * returns and *status receives code 104; the call's output is then meaningless.
 *
 * cfg: M = this rank's tokens (<= ep->m_cap), E = experts held locally, wmode must be
 * B200MOE_W_FP8_BLOCK; w1 / w2 / quant hold the local experts.  placement [n_global_experts]:
 * (rank << 16) | local expert id for every global expert (negative: held nowhere, dropped);
 * any assignment with at most cfg->E experts per rank is valid, contiguous or load-balanced.
 * heaps [world]: the heaps as mapped into this process, own heap at [rank].  All ranks must use
 * the same m_cap, H, topk and weight mode, and call in lockstep.
 */
#define B200MOE_EP_MAX_RANKS 8
#define B200MOE_EP_PHASE_DISPATCH 1
#define B200MOE_EP_PHASE_COMPUTE 2
#define B200MOE_EP_PHASE_COMBINE 4
#define B200MOE_EP_PHASE_ALL 7

typedef struct b200moe_ep_cfg {
  int32_t struct_bytes;       /* sizeof(b200moe_ep_cfg), checked                       */
  int32_t world;              /* ranks, 1..B200MOE_EP_MAX_RANKS                        */
  int32_t rank;
  int32_t m_cap;              /* token capacity per rank (same on every rank)          */
  int32_t n_global_experts;   /* entries of `placement`                                */
  int32_t reserved;
  uint64_t wait_limit_ns;     /* bound of every flag wait; 0 = 2 000 000 000           */
} b200moe_ep_cfg;

size_t b200moe_ep_heap_bytes(const b200moe_cfg *cfg, const b200moe_ep_cfg *ep);
size_t b200moe_ep_workspace_bytes(const b200moe_cfg *cfg, const b200moe_ep_cfg *ep);
/* set-up time only (these allocate / map and synchronise the device) */
int b200moe_ep_heap_alloc(size_t bytes, void **heap);
int b200moe_ep_heap_free(void *heap);
int b200moe_ep_ipc_export(void *heap, void *handle64);
int b200moe_ep_ipc_open(const void *handle64, void **peer_heap);
int b200moe_ep_ipc_close(void *peer_heap);
int b200moe_ep_forward(const b200moe_cfg *cfg, const b200moe_ep_cfg *ep, void *const *heaps, int phases,
                       const void *x, const void *w1, const void *w2, const b200moe_quant *quant,
                       const float *topk_weights, const void *topk_ids, const int32_t *placement,
                       void *workspace, size_t workspace_bytes, void *out, int32_t *status,
                       void *stream);

/*
 * Dynamic per-token-group FP8 quantisation (1 x 128 groups): the step in front
 * of the FP8 path (shapes listed at benchmark/core_shapes.yaml:311-317).
 * x [rows, K] of `dtype`; q [rows, K] e4m3fn; scales [rows, K/128] fp32.
 */
int b200moe_per_token_group_quant_fp8(const void *x, int dtype, int rows, int K,
                                      void *q, float *scales, void *stream);

/*
 * Per-kernel timing for benchmarks (no counterpart in the reference, whose
 * benchmark times the host side of an asynchronous launch,
 * benchmark/test_fused_moe.py:39-59).  Between begin and end every forward call
 * records CUDA events around its two grouped GEMMs on the caller's stream;
 * end synchronises on them and returns the summed milliseconds and the number
 * of calls seen (local_ms: for expert-parallel calls the span from "all peers'
 * rows have arrived" to "the down projection has completed", otherwise the whole
 * call).  begin creates the events (host objects), so neither belongs inside a
 * timed or captured region.
 */
int b200moe_profile_begin(int max_calls);
int b200moe_profile_end(double *gemm1_ms, double *gemm2_ms, double *total_ms, double *local_ms,
                        int *calls);

/*
 * Launch accounting for benchmarks (no counterpart in the reference): the number of
 * kernels this library has launched since it was loaded, and the kernels of the most
 * recent forward call as a comma-separated list (truncated to names_bytes - 1
 * characters).  Returns the number of kernels in that list.
 */
int b200moe_launch_stats(long long *total_launches, char *last_call_names, size_t names_bytes);
/* CTA pairs the device kept resident for the last grouped GEMM launched on CTA pairs
 * (B200MOE_FLAG_CTA_PAIR); 0 before the first such launch.  Diagnostics. */
int b200moe_debug_resident_cta_pairs(void);

/*
 * Self-test of the device-side time-out path (no counterpart in the reference, which has no
 * bounded waits).  Launches a one-CTA kernel in which one warp waits, for at most limit_ns
 * (1 .. 100 000 000), on a barrier nobody arrives on, and a second warp waits on the same
 * barrier with a limit a thousand times longer.  The first wait must run out, raise the CTA's
 * abort flag and so release the second; the kernel returns normally and writes the time-out
 * code 105 into *status (device int32, left alone if already non-zero).  observed (device
 * int32[3]): [0] = 0 when the short wait ran out, [1] = 0 when the long wait was released by
 * the flag, [2] = microseconds the second warp waited.  Nothing faults, traps or hangs.
 */
int b200moe_selftest_timeout(uint64_t limit_ns, int32_t *status, int32_t *observed, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* B200MOE_H_ */
