// Expert parallelism over peer-mapped memory (NVLink / NVSwitch): heap layout, dispatch and flags.
#pragma once
#include "gemm.cuh"

namespace b200moe {

// Every rank owns one "heap" of this layout and maps the heaps of all other ranks (CUDA IPC).
//   flags       ready[kMaxPeers], done[kMaxPeers], rows[kMaxPeers] (uint64 epochs written by the
//               peers), this rank's own epoch counter and two CTA counters
//   recv_*      what the peers dispatch to this rank: for source rank r and its token i the row
//               r * m_cap + i holds the token's activations (FP8 + 1x128 scales, or 16-bit), its
//               top-k expert ids translated to this rank's local experts (-1 = held elsewhere) and
//               the routing weights (0 where masked).  A fixed row per (source, token): no counts
//               are exchanged and nothing on the host reads device data.
//   pairs / pair_valid / out32
//               where the results of this rank's own tokens arrive: one 16-bit row per
//               (token, choice) pair written by whichever rank holds the expert, or fp32 rows that
//               the peers add into.
struct EpHeap {
  size_t flags, recv_ids, recv_w, recv_x, recv_xs, pairs, pair_valid, out32, total;
  int x_row_bytes;
};
constexpr size_t kEpFlagReady = 0;                          // byte offsets inside the flags block (256 bytes)
constexpr size_t kEpFlagDone = kMaxPeers * 8;               //   ready: the peers' routing entries are in place
constexpr size_t kEpFlagEpoch = 2 * kMaxPeers * 8;          //   rows:  the peers' token rows are in place (raised later)
constexpr size_t kEpFlagCtaCount = 2 * kMaxPeers * 8 + 8;   //   done:  the peers' down projections have completed
constexpr size_t kEpFlagCtaCount2 = 2 * kMaxPeers * 8 + 12;
constexpr size_t kEpFlagRows = 3 * kMaxPeers * 8;

EpHeap ep_heap_layout(int world, int m_cap, int H, int topk, bool fp8_rows);

struct EpDispatchArgs {
  int world, rank, m, m_cap, H, topk, n_global_experts;
  int dtype;        // B200MOE_DTYPE_* of x
  int fp8_rows;     // 1: quantise rows to e4m3 with 1x128 scales before they travel; 0: 16-bit rows as they are
  int ids_i64;
  int clear_pairs;  // which of this rank's result buffers to clear: 1 = pair_valid, 0 = out32
  const void* x;            // [m, H]
  const float* topk_weights;  // [m, topk]
  const void* topk_ids;     // [m, topk] global expert ids
  const int* placement;     // [n_global_experts] (rank << 16) | local expert, negative = nowhere
  uint8_t* heap[kMaxPeers]; // heaps of all ranks as mapped here; own heap at [rank]
  EpHeap L;
};

int launch_ep_dispatch(const EpDispatchArgs& a, int num_sms, cudaStream_t stream, bool pdl);

// Waiting for the peers' flags (common.cuh: FlagWait): as a kernel of its own, or handed to the kernel
// that consumes what the peers wrote (alignment, output conversion), which then waits in its prologue.
FlagWait ep_flag_wait(uint8_t* my_heap, const EpHeap& L, size_t flag_off, int world, unsigned long long limit_ns,
                      int* status);
int launch_ep_wait(const FlagWait& w, cudaStream_t stream, bool pdl);

// After everything before it in the stream has completed: this rank's epoch goes into its slot of
// the flag array (at flag_off) of every peer.
int launch_ep_signal(uint8_t* const* heaps, const EpHeap& L, size_t flag_off, int world, int rank,
                     cudaStream_t stream, bool pdl);

}  // namespace b200moe
