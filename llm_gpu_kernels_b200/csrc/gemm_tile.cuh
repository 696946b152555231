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

// Chaining of the gate/up and the down kernel of one forward (see grouped_gemm_tcgen05.cu): the down kernel does not
// wait for the gate/up grid but for per-expert completion counters, and draws its tiles from a global counter.
constexpr int kItemRing = 16;  // tiles a dynamic producer may announce ahead of the epilogue

// Acquire load of a completion counter another SM bumps.
__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// The tile a role works on next. Static schedule: tile seq of this CTA is blockIdx.x + seq * gridDim.x.
// Dynamic schedule: the producer draws tiles from a global counter and announces them in a small ring
// (Ctrl::item / Ctrl::item_ready, kItemRing entries) that the other roles follow; -1 ends the work.
template <class Ctrl>
__device__ __forceinline__ int follow_item(Ctrl* c, bool dynamic, int seq, int total_items, int* status) {
  if (!dynamic) {
    const long long item = static_cast<long long>(blockIdx.x) + static_cast<long long>(seq) * gridDim.x;
    return item < total_items ? static_cast<int>(item) : -1;
  }
  const int q = seq % kItemRing;
  if (!ptx::mbar_wait(&c->item_ready[q], static_cast<uint32_t>((seq / kItemRing) & 1), &c->abort, status)) return -1;
  return *reinterpret_cast<volatile int*>(&c->item[q]);
}

// Producer side of the dynamic schedule: draw the next tile and announce it as tile `seq` of this CTA.
template <class Ctrl>
__device__ __forceinline__ int draw_item(Ctrl* c, int* tile_counter, int seq, int total_items) {
  int item = atomicAdd(tile_counter, 1);
  if (item >= total_items) item = -1;
  const int q = seq % kItemRing;
  *reinterpret_cast<volatile int*>(&c->item[q]) = item;
  ptx::mbar_arrive(&c->item_ready[q]);  // release: the item is visible to whoever sees the phase flip
  return item;
}

// Waits (bounded) until `done` says that every activated row of an expert is written: `need` arrivals.
// Returns false when the wait was given up (status and *abort raised) or another role raised *abort.
__device__ __forceinline__ bool wait_expert_done(const int* done, int need, int* abort, int* status) {
  const unsigned long long start = ptx::global_timer();
  uint32_t spins = 0;
  while (ld_acquire_gpu(done) < need) {
    if ((++spins & 15u) == 0) {
      if (*reinterpret_cast<volatile int*>(abort)) return false;
      if (ptx::global_timer() - start > ptx::kWaitLimitNs) {
        *reinterpret_cast<volatile int*>(abort) = 1;
        atomicOr(status, B200MOE_STATUS_TIMEOUT);
        return false;
      }
    }
  }
  return true;
}

// Head of the gate/up weights that the gate/up CTAs pull into L2 while router and dispatch still run (HBM is idle
// then). Qwen3 shape, forward at 17 / 193 / 1024 tokens: 142.4 / 197.7 / 230.7 us without, 138.0 / 192.4 / 225.8 with
// 32 MB, 137.5 / 190.8 / 223.8 with 64 MB, 135.9 / 189.6 / 226.0 with 96 MB (L2 holds 126 MB).
constexpr long long kPrefetchBytes = 64ll << 20;
constexpr uint32_t kPrefetchChunk = 8192;            // bytes per L2 prefetch instruction
inline int prefetch_head_chunks(long long weight_bytes) {
  return static_cast<int>((weight_bytes < kPrefetchBytes ? weight_bytes : kPrefetchBytes) / kPrefetchChunk);
}
// Called by every thread of every CTA of a gate/up kernel before it waits for the kernels in front of it: the grid
// shares out `chunks` prefetch instructions over the head of the weight tensor at `base`.
__device__ __forceinline__ void prefetch_head(const unsigned char* __restrict__ base, int chunks) {
  const int per_cta = (chunks + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);
  const int first = static_cast<int>(blockIdx.x) * per_cta;
  const int last = first + per_cta < chunks ? first + per_cta : chunks;
  for (int chunk = first + static_cast<int>(threadIdx.x); chunk < last; chunk += static_cast<int>(blockDim.x))
    ptx::prefetch_l2_bulk(base + static_cast<size_t>(chunk) * kPrefetchChunk, kPrefetchChunk);
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
