// Tile scheduler shared by the grouped GEMM kernels: constants of the pipeline, the split
// of the work into (expert, token block, n-tile, k-split) units and the decode of a unit id.
#pragma once
#include "gemm.cuh"

namespace b200moe {

constexpr int kThreads = 192;
constexpr int kTileRows = 128;           // weight rows per MMA (the instruction's M)
constexpr int kStageKBytes = 128;        // bytes of the reduction dim per stage row (one swizzle atom)
constexpr int kTileBytes = kTileRows * kStageKBytes;  // 16 KiB
constexpr int kMaxBT = 256;
constexpr size_t kSmemLimit = 232448;    // 227 KiB

struct Ctrl {
  int nblocks;
  int units_per_block;  // num_nt (* split)
  int split;
  int total;
  int grid_eff;
};

__device__ __forceinline__ int pick_split(int tiles, int kblocks, int grid, int max_split) {
  int best = 1;
  float best_eff = -1.f;
  int smax = min(max_split, max(1, kblocks / 4));
  for (int s = 1; s <= smax; ++s) {
    int total = tiles * s;
    int waves = (total + grid - 1) / grid;
    float eff = static_cast<float>(total) / static_cast<float>(waves * grid);
    if (eff > best_eff + 0.04f) {
      best_eff = eff;
      best = s;
    }
  }
  return best;
}

struct TileCoord {
  int e;      // expert
  int row0;   // first padded row of the token block
  int n0;     // first weight row inside the expert
  int kb0, kb1;  // k-block range
};

__device__ __forceinline__ TileCoord decode_tile(int id, const Ctrl& c, const int* s_blk_off, int E,
                                                 int BT, int num_nt, int kblocks, int tile_n) {
  // largest e with blk_off[e] * units <= id
  int lo = 0, hi = E;
  const int u = c.units_per_block;
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (s_blk_off[mid] * u <= id) lo = mid; else hi = mid;
  }
  TileCoord t;
  t.e = lo;
  const int first = s_blk_off[lo];
  const int nb = s_blk_off[lo + 1] - first;
  const int local = id - first * u;
  const int b = local % nb;
  const int rest = local / nb;
  const int s = rest % c.split;
  const int nt = rest / c.split;
  t.row0 = (first + b) * BT;
  t.n0 = nt * tile_n;
  t.kb0 = static_cast<int>((static_cast<long long>(s) * kblocks) / c.split);
  t.kb1 = static_cast<int>((static_cast<long long>(s + 1) * kblocks) / c.split);
  return t;
}


// Fused tail of the gate/up projection.
//   SiLU / GELU (the reference's plain op, fused_moe.py:198-206): optional routing weight on the
//   two projections, optional rounding of both to the 16-bit type (as the reference stores
//   them), activation(gate) * up.
//   B200MOE_ACT_SWIGLU_OAI (the reference's bias variant fuses its dependency's swiglu into
//   GEMM-1, fused_moe.py:258-298): gate clamped from above, linear clamped to [-limit, limit],
//   s = g / (1 + exp(-alpha * g)), result s * (linear + 1); the routing weight, if it goes on
//   the input side, multiplies the result.
struct ActParams {
  int activation;
  float alpha, limit;
};
// EXT = false compiles the SiLU / GELU tail only: the epilogues are bound by their instruction
// count, so the plain kernels must not carry the extra tests.
template <typename T, bool EXT = false>
__device__ __forceinline__ float act_mul(float g, float u, bool w_on_input, float gam, bool mimic,
                                         const ActParams& p) {
  if (EXT && p.activation == B200MOE_ACT_SWIGLU_OAI) {
    if (p.limit > 0.f) {
      g = fminf(g, p.limit);
      u = fminf(fmaxf(u, -p.limit), p.limit);
    }
    const float s = __fdividef(g, 1.0f + __expf(-p.alpha * g));
    const float r = fmaf(s, u, s);
    return w_on_input ? r * gam : r;
  }
  if (w_on_input) {
    g *= gam;
    u *= gam;
  }
  if (mimic) {
    g = to_f32<T>(from_f32<T>(g));
    u = to_f32<T>(from_f32<T>(u));
  }
  const float s = (p.activation == B200MOE_ACT_SILU) ? __fdividef(g, 1.0f + __expf(-g)) : gelu_f32(g);
  return s * u;
}
__device__ __forceinline__ ActParams act_params(const GemmArgs& a) {
  ActParams p;
  p.activation = a.activation;
  p.alpha = a.act_alpha;
  p.limit = a.act_limit;
  return p;
}

// Work decomposition for one launch; identical in every thread of every CTA.
__device__ __forceinline__ Ctrl make_ctrl(const GemmArgs& a, bool may_split) {
  Ctrl c;
  c.nblocks = a.meta[0];
  c.split = 1;
  if (may_split && !(a.flags & B200MOE_FLAG_NO_SPLIT_K))
    c.split = pick_split(c.nblocks * a.num_nt, a.kblocks, gridDim.x, a.max_split);
  c.units_per_block = a.num_nt * c.split;
  c.total = c.nblocks * c.units_per_block;
  // spread the tiles evenly: with w waves, ceil(total / w) CTAs do w tiles each
  int waves = (c.total + gridDim.x - 1) / static_cast<int>(gridDim.x);
  c.grid_eff = waves > 0 ? (c.total + waves - 1) / waves : 1;
  if (a.flags & B200MOE_FLAG_NO_GRID_BALANCE) c.grid_eff = gridDim.x;
  return c;
}

}  // namespace b200moe
