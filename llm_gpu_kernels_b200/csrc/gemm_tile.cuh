// Pieces shared by the BF16 and the W4A16 grouped GEMM kernels: the device-side
// tile enumeration over the `tasks` prefix and the TMEM -> global epilogue.
#pragma once
#include <cuda_bf16.h>
#include "sm100_ptx.cuh"

namespace b200moe {
namespace tile {

constexpr int kTileM = 128;      // output channels per tile (UMMA M)
constexpr int kBlockK = 64;      // BF16 per k-block: 128 bytes = one swizzle row
constexpr int kUmmaK = 16;
constexpr int kMaxExperts = 256;
constexpr int kSmemLimit = 232448;  // 227 KB opt-in limit per CTA

// Per-CTA copy of the dispatch metadata (shared memory).
struct Tables {
  int tasks[kMaxExperts + 1];
  int offsets[kMaxExperts];
  int counts[kMaxExperts];
};

__device__ __forceinline__ void load_tables(Tables* t, const int* g_tasks, const int* g_offsets, const int* g_counts,
                                            int E) {
  for (int i = threadIdx.x; i <= E; i += blockDim.x) t->tasks[i] = g_tasks[i];
  for (int i = threadIdx.x; i < E; i += blockDim.x) {
    t->offsets[i] = g_offsets[i];
    t->counts[i] = g_counts[i];
  }
}

struct Tile {
  int expert, ct, row0, rows, n_eff;
};

// item -> (expert, channel tile, token tile). Items of one expert are ordered
// channel tile major, token tile fastest, so CTAs running side by side share a
// weight tile (L2) when an expert has several token tiles.
__device__ __forceinline__ Tile decode_tile(const Tables* c, int item, int E, int n_ct, int token_tile) {
  int lo = 0, hi = E;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (item >= c->tasks[mid + 1] * n_ct) lo = mid + 1; else hi = mid;
  }
  Tile t;
  t.expert = lo;
  const int local = item - c->tasks[lo] * n_ct;
  const int tiles = c->tasks[lo + 1] - c->tasks[lo];
  t.ct = local / tiles;
  const int tt = local - t.ct * tiles;
  t.row0 = c->offsets[lo] + tt * token_tile;
  t.rows = min(token_tile, c->counts[lo] - tt * token_tile);
  t.n_eff = max(16, (t.rows + 15) & ~15);
  return t;
}

// One epilogue warp drains its 32 TMEM lanes (= 32 output channels) of one tile:
// D[channel][row] FP32 -> out[row0 + row][channel] BF16, SwiGLU first when kGateUp
// (gate columns at taddr, up columns at taddr + token_tile). kSumPair: the tile was accumulated as two partial
// sums over K (even and odd K steps, by two MMA-issuing threads) in the same two column ranges; they are added
// here, in FP32. The whole warp must call it.
template <bool kGateUp, bool kSumPair = false>
__device__ __forceinline__ void store_tile(const Tile& t, uint32_t taddr, int token_tile, int channel, int n_out,
                                           __nv_bfloat16* __restrict__ out) {
  const bool ch_ok = channel < n_out;
  __nv_bfloat16* dst = out + static_cast<size_t>(t.row0) * n_out + channel;
  for (int n0 = 0; n0 < t.n_eff; n0 += 16) {
    uint32_t g[16], u[16];
    ptx::tmem_ld16(taddr + n0, g);
    if (kGateUp || kSumPair) ptx::tmem_ld16(taddr + token_tile + n0, u);
    ptx::tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const int n = n0 + j;
      float v = __uint_as_float(g[j]);
      if (kGateUp) v = (v / (1.0f + __expf(-v))) * __uint_as_float(u[j]);
      else if (kSumPair) v = __fadd_rn(v, __uint_as_float(u[j]));
      if (ch_ok && n < t.rows) dst[static_cast<size_t>(n) * n_out] = __float2bfloat16_rn(v);
    }
  }
}

}  // namespace tile
}  // namespace b200moe
