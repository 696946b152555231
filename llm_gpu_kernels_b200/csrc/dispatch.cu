// Ranked dispatch: per-expert count, prefix sum, deterministic route -> row
// permutation, and the row copy into expert-contiguous order.
//
// Replaces _reset + _rank_histogram + _prefix + _rank_dispatch of the
// reference (moe.py:13-43, moe_ranked.py:18-65). The reference takes the rank
// of a route inside its expert from the return value of a global atomic, so
// its permutation depends on arrival order; here the rank is the number of
// earlier routes (by flat index q = token*K + slot) that chose the same
// expert, which is the stable order of argsort(ids, stable=True). No global
// atomics are used, so counts / offsets / ranks / mapping are bit-reproducible.
//
// Up to kFusedRoutes (2048) routes one 1024-thread block does count + scan + final
// ranks / mapping in a single launch (warp histograms stay in shared memory)
// and a second kernel copies the rows; up to 8 x 2048 routes a thread-block cluster of
// 2, 4 or 8 such blocks does the same, exchanging per-expert totals through distributed
// shared memory. Above that, three kernels:
//  count   - every warp owns `warp_routes` consecutive routes and walks them 32
//            at a time in order: __match_any_sync gives the lanes with the same
//            expert, so rank-in-partition = running warp histogram + number of
//            lower lanes with that expert. Writes the rank inside the
//            partition to ranks[q] and the partition histogram to scratch.
//  scan    - one block: per expert an exclusive scan over the partitions
//            (scratch becomes the partition's base rank), counts, offsets,
//            the token-tile prefix `tasks`, cursors = 0, and the status word.
//  permute - ranks[q] += base; mapping[q] = offsets[id] + ranks[q]; one warp
//            copies the token's row to grouped_input[mapping[q]].
// A plan whose gate/up kernel gathers the token rows itself gets source_rows[mapping[q]] = q / K (the inverse
// permutation) instead of the row copy.
#include <cuda_bf16.h>
#include "plan.h"
#include "pdl.cuh"

namespace b200moe {
namespace {

constexpr int kWarps = kDispatchWarps;
constexpr int kThreads = kWarps * 32;
constexpr int kMaxExperts = 256;
constexpr int kFusedIters = kFusedRoutes / 1024;  // routes per lane of the one-block kernel

// scratch layout: int32 hist[partitions][E], int32 flags[blocks], int32 router_flag,
// then (plans only) int32 tile counter and int32 done[E] of the chained GEMM kernels
template <typename IdT>
__global__ void __launch_bounds__(kThreads)
dispatch_count_kernel(const IdT* __restrict__ ids, const float* __restrict__ rw, int* __restrict__ ranks,
                      int* __restrict__ hist, int* __restrict__ flags, const int* __restrict__ valid_routes, int R,
                      int E, int warp_routes, int partitions) {
  pdl_launch_dependents();
  pdl_wait();  // ids / routing weights may come from the router kernel just before
  const int r_eff = valid_routes ? min(R, max(*valid_routes, 0)) : R;  // routes past r_eff are padding
  __shared__ int warp_hist[kWarps][kMaxExperts];
  __shared__ int block_flags;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int part = blockIdx.x * kWarps + warp;
  if (threadIdx.x == 0) block_flags = 0;
  for (int e = lane; e < E; e += 32) warp_hist[warp][e] = 0;
  __syncthreads();
  int my_flags = 0;
  if (part < partitions) {
    const int begin = part * warp_routes;
    const int end = min(R, begin + warp_routes);
    for (int base = begin; base < end; base += 32) {
      const int q = base + lane;
      const bool in = q < end, live = in && q < r_eff;
      long long id = live ? static_cast<long long>(ids[q]) : -1;
      const float w = live ? rw[q] : 0.0f;
      const bool valid = live && id >= 0 && id < E;
      if (live && !valid) my_flags |= B200MOE_STATUS_BAD_ID;
      if (live && !(fabsf(w) < INFINITY)) my_flags |= B200MOE_STATUS_BAD_WEIGHT;  // false for NaN too
      const int key = valid ? static_cast<int>(id) : E;  // E = "no expert"
      const unsigned peers = __match_any_sync(0xffffffffu, key);
      const int below = __popc(peers & ((1u << lane) - 1u));
      int rank = -1;
      if (valid) {
        rank = warp_hist[warp][key] + below;
      }
      __syncwarp();
      if (valid && below == 0) warp_hist[warp][key] += __popc(peers);
      __syncwarp();
      if (in) ranks[q] = rank;
    }
    for (int e = lane; e < E; e += 32) hist[static_cast<size_t>(part) * E + e] = warp_hist[warp][e];
  }
  if (my_flags) atomicOr(&block_flags, my_flags);
  __syncthreads();
  if (threadIdx.x == 0) flags[blockIdx.x] = block_flags;
}

// Exclusive prefix over the experts of (count, tiles) for the first 256 threads of a block.
// Every thread of the block must call it (it synchronises); `scratch` holds 2 x 8 ints.
__device__ __forceinline__ void expert_prefix(int count, int tiles, int* scratch, int* count_excl, int* tiles_excl,
                                              int* tiles_total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int c = count, t = tiles;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int oc = __shfl_up_sync(0xffffffffu, c, o), ot = __shfl_up_sync(0xffffffffu, t, o);
    if (lane >= o) { c += oc; t += ot; }
  }
  if (warp < 8 && lane == 31) { scratch[warp] = c; scratch[8 + warp] = t; }
  __syncthreads();
  int cb = 0, tb = 0, tt = 0;
#pragma unroll
  for (int w = 0; w < 8; ++w) {
    if (w < warp) { cb += scratch[w]; tb += scratch[8 + w]; }
    tt += scratch[8 + w];
  }
  *count_excl = c - count + cb;
  *tiles_excl = t - tiles + tb;
  *tiles_total = tt;
}

__global__ void __launch_bounds__(kMaxExperts)
dispatch_scan_kernel(int* __restrict__ hist, const int* __restrict__ flags, int* __restrict__ counts,
                     int* __restrict__ offsets, int* __restrict__ cursors, int* __restrict__ tasks,
                     int* __restrict__ status, int* __restrict__ router_flag, int E, int partitions, int blocks,
                     int token_tile, int chain_words) {
  pdl_launch_dependents();
  pdl_wait();  // partition histograms come from the count kernel
  __shared__ int s_scan[16];
  __shared__ int s_flags;
  const int e = threadIdx.x;
  if (e == 0) s_flags = 0;
  __syncthreads();
  int total = 0;
  if (e < E) {
    for (int p0 = 0; p0 < partitions; p0 += 8) {  // loads first, then the dependent running sum
      int c[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) c[j] = p0 + j < partitions ? hist[static_cast<size_t>(p0 + j) * E + e] : 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (p0 + j < partitions) hist[static_cast<size_t>(p0 + j) * E + e] = total;
        total += c[j];
      }
    }
  }
  int f = 0;
  for (int b = e; b < blocks; b += blockDim.x) f |= flags[b];
  if (f) atomicOr(&s_flags, f);
  const int tiles = e < E ? (total + token_tile - 1) / token_tile : 0;
  int off, toff, ttotal;
  expert_prefix(e < E ? total : 0, tiles, s_scan, &off, &toff, &ttotal);
  if (e < E) {
    counts[e] = total;
    offsets[e] = off;
    cursors[e] = 0;
    tasks[e] = toff;
    if (e == E - 1) tasks[E] = ttotal;
  }
  // tile counter and per-expert completion counters of the chained GEMM kernels
  for (int i = e; i < chain_words; i += blockDim.x) router_flag[1 + i] = 0;
  if (e == 0) {  // the status word restarts every forward; fold in what the router raised
    *status = s_flags | *router_flag;
    *router_flag = 0;
  }
}

// Distributed shared memory: the word at the address of `local` in CTA `cta` of this cluster.
__device__ __forceinline__ int ld_cluster(const int* local, unsigned cta) {
  unsigned remote;
  int v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;"
               : "=r"(remote) : "r"(static_cast<unsigned>(__cvta_generic_to_shared(local))), "r"(cta));
  asm volatile("ld.shared::cluster.b32 %0, [%1];" : "=r"(v) : "r"(remote) : "memory");
  return v;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// One kernel does the whole dispatch metadata: a block ranks up to kFusedRoutes routes, and a thread-block cluster of
// 1, 2, 4 or 8 such blocks shares a larger forward - block c owns routes [c, c+1) x 32 x warp_routes, keeps its
// per-warp histograms in its own shared memory and reads the other blocks' per-expert totals through distributed
// shared memory, so the stable rank of a route is rank in its warp + rows of earlier warps of its block + rows of
// earlier blocks. Every block computes the expert offsets; block 0 writes the metadata.
template <typename IdT>
__global__ void __launch_bounds__(1024)
dispatch_fused_kernel(const IdT* __restrict__ ids, const float* __restrict__ rw, int* __restrict__ ranks,
                      int* __restrict__ mapping, int* __restrict__ counts, int* __restrict__ offsets,
                      int* __restrict__ cursors, int* __restrict__ tasks, int* __restrict__ status,
                      int* __restrict__ router_flag, const int* __restrict__ valid_routes, int R, int E,
                      int warp_routes, int token_tile, int chain_words, int* __restrict__ source_rows, int K) {
  pdl_launch_dependents();
  pdl_wait();  // ids / routing weights may come from the router kernel just before
  unsigned cta, ctas;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(cta));
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(ctas));
  const int r_eff = valid_routes ? min(R, max(*valid_routes, 0)) : R;  // routes past r_eff are padding
  __shared__ int warp_hist[32][kMaxExperts];
  __shared__ int s_total[kMaxExperts];   // rows of each expert among this block's routes (read by the other blocks)
  __shared__ int s_base[kMaxExperts];    // rows of each expert in the blocks before this one
  __shared__ int s_off[kMaxExperts];
  __shared__ int s_scan[16];
  __shared__ int s_flags;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) s_flags = 0;
  for (int e = lane; e < E; e += 32) warp_hist[warp][e] = 0;
  __syncthreads();
  const int part = static_cast<int>(cta) * 32 + warp;
  const int begin = static_cast<int>(min(static_cast<long long>(R), static_cast<long long>(part) * warp_routes));
  const int end = min(R, begin + warp_routes);
  const int iters = (end - begin + 31) >> 5;   // <= kFusedIters: kFusedRoutes / 32 warps / 32 lanes
  int my_flags = 0;
  int key[kFusedIters], rk[kFusedIters];
  // all loads first (one global latency for the whole range), then the in-order ranking
#pragma unroll
  for (int it = 0; it < kFusedIters; ++it) {
    const int q = begin + it * 32 + lane;
    const bool live = it < iters && q < end && q < r_eff;
    const long long id = live ? static_cast<long long>(ids[q]) : -1;
    const float w = live ? rw[q] : 0.0f;
    const bool valid = live && id >= 0 && id < E;
    if (live && !valid) my_flags |= B200MOE_STATUS_BAD_ID;
    if (live && !(fabsf(w) < INFINITY)) my_flags |= B200MOE_STATUS_BAD_WEIGHT;
    key[it] = valid ? static_cast<int>(id) : E;  // E = "no expert"
  }
#pragma unroll
  for (int it = 0; it < kFusedIters; ++it) {
    if (it < iters) {  // warp-uniform
      const unsigned peers = __match_any_sync(0xffffffffu, key[it]);
      const int below = __popc(peers & ((1u << lane) - 1u));
      const bool valid = key[it] < E;
      rk[it] = valid ? warp_hist[warp][key[it]] + below : -1;
      __syncwarp();
      if (valid && below == 0) warp_hist[warp][key[it]] += __popc(peers);
      __syncwarp();
    }
  }
  if (my_flags) atomicOr(&s_flags, my_flags);
  __syncthreads();
  const int e = threadIdx.x;
  int total = 0;
  if (e < E) {
#pragma unroll 8
    for (int w = 0; w < 32; ++w) {
      const int c = warp_hist[w][e];
      warp_hist[w][e] = total;  // base rank of warp w's partition inside expert e, within this block
      total += c;
    }
    s_total[e] = total;
  }
  int base = 0, flags = s_flags;
  if (ctas > 1) {
    cluster_sync();   // every block's s_total / s_flags is written
    if (e < E) {
      total = 0;
      for (unsigned c = 0; c < ctas; ++c) {
        const int v = ld_cluster(&s_total[e], c);
        if (c < cta) base += v;
        total += v;
      }
    }
    if (e == 0)
      for (unsigned c = 0; c < ctas; ++c) flags |= ld_cluster(&s_flags, c);
  }
  const int tiles = e < E ? (total + token_tile - 1) / token_tile : 0;
  int off, toff, ttotal;
  expert_prefix(e < E ? total : 0, tiles, s_scan, &off, &toff, &ttotal);
  if (e < E) {
    s_off[e] = off;
    s_base[e] = base;
  }
  if (cta == 0) {
    if (e < E) {
      counts[e] = total;
      offsets[e] = off;
      cursors[e] = 0;
      tasks[e] = toff;
      if (e == E - 1) tasks[E] = ttotal;
    }
    for (int i = e; i < chain_words; i += blockDim.x) router_flag[1 + i] = 0;  // see the scan kernel
    if (e == 0) {
      *status = flags | *router_flag;
      *router_flag = 0;
    }
  }
  __syncthreads();
#pragma unroll
  for (int it = 0; it < kFusedIters; ++it) {
    const int q = begin + it * 32 + lane;
    if (it < iters && q < end) {
      int rank = -1, pos = -1;
      if (key[it] < E) {
        rank = rk[it] + warp_hist[warp][key[it]] + s_base[key[it]];  // + rows of earlier warps and earlier blocks
        pos = s_off[key[it]] + rank;
      }
      ranks[q] = rank;
      mapping[q] = pos;
      if (source_rows != nullptr && pos >= 0) source_rows[pos] = q / K;
    }
  }
  if (ctas > 1) cluster_sync();   // no block leaves while another may still read its shared memory
}

// Row copy for the fused path: grouped_input[mapping[q], :] = x[q / K, :], one warp per route.
__global__ void __launch_bounds__(kThreads)
dispatch_copy_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ mapping,
                     __nv_bfloat16* __restrict__ grouped, int R, int H, int K) {
  pdl_launch_dependents();
  pdl_wait();  // mapping comes from the kernel just before
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q = blockIdx.x * kWarps + warp;
  if (q >= R) return;
  const int pos = mapping[q];
  if (pos < 0) return;
  const __nv_bfloat16* src = x + static_cast<size_t>(q / K) * H;
  __nv_bfloat16* dst = grouped + static_cast<size_t>(pos) * H;
  if ((H & 7) == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(grouped)) & 15) == 0) {
    const uint4* s4 = reinterpret_cast<const uint4*>(src);
    uint4* d4 = reinterpret_cast<uint4*>(dst);
    for (int i = lane; i < H / 8; i += 32) d4[i] = s4[i];
  } else {
    for (int i = lane; i < H; i += 32) dst[i] = src[i];
  }
}

template <typename IdT>
__global__ void __launch_bounds__(kThreads)
dispatch_permute_kernel(const __nv_bfloat16* __restrict__ x, const IdT* __restrict__ ids,
                        const int* __restrict__ hist, const int* __restrict__ offsets,
                        int* __restrict__ ranks, int* __restrict__ mapping,
                        __nv_bfloat16* __restrict__ grouped, const int* __restrict__ valid_routes, int R, int E,
                        int H, int K, int warp_routes, int* __restrict__ source_rows) {
  pdl_launch_dependents();
  pdl_wait();  // offsets and partition base ranks come from the scan kernel
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q = blockIdx.x * kWarps + warp;
  if (q >= R) return;
  const int r_eff = valid_routes ? min(R, max(*valid_routes, 0)) : R;
  const long long id = q < r_eff ? static_cast<long long>(ids[q]) : -1;
  const bool valid = id >= 0 && id < E;
  int pos = -1;
  if (lane == 0) {  // one lane owns the read-modify-write of ranks[q]
    if (valid) {
      const int part = q / warp_routes;
      const int rank = ranks[q] + hist[static_cast<size_t>(part) * E + static_cast<int>(id)];
      pos = offsets[id] + rank;
      ranks[q] = rank;
      if (source_rows != nullptr) source_rows[pos] = q / K;
    }
    mapping[q] = pos;
  }
  pos = __shfl_sync(0xffffffffu, pos, 0);
  if (!valid || grouped == nullptr) return;
  const __nv_bfloat16* src = x + static_cast<size_t>(q / K) * H;
  __nv_bfloat16* dst = grouped + static_cast<size_t>(pos) * H;
  if ((H & 7) == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(grouped)) & 15) == 0) {
    const uint4* s4 = reinterpret_cast<const uint4*>(src);
    uint4* d4 = reinterpret_cast<uint4*>(dst);
    for (int i = lane; i < H / 8; i += 32) d4[i] = s4[i];
  } else {
    for (int i = lane; i < H; i += 32) dst[i] = src[i];
  }
}

// The permute step without the row copy (the rows are gathered by the gate/up kernel or sent to other ranks):
// one thread per route.
template <typename IdT>
__global__ void __launch_bounds__(kThreads)
dispatch_map_kernel(const IdT* __restrict__ ids, const int* __restrict__ hist, const int* __restrict__ offsets,
                    int* __restrict__ ranks, int* __restrict__ mapping, const int* __restrict__ valid_routes, int R,
                    int E, int K, int warp_routes, int* __restrict__ source_rows) {
  pdl_launch_dependents();
  pdl_wait();  // offsets and partition base ranks come from the scan kernel
  const int q = blockIdx.x * kThreads + threadIdx.x;
  if (q >= R) return;
  const int r_eff = valid_routes ? min(R, max(*valid_routes, 0)) : R;
  const long long id = q < r_eff ? static_cast<long long>(ids[q]) : -1;
  int pos = -1;
  if (id >= 0 && id < E) {
    const int rank = ranks[q] + hist[static_cast<size_t>(q / warp_routes) * E + static_cast<int>(id)];
    pos = offsets[id] + rank;
    ranks[q] = rank;
    if (source_rows != nullptr) source_rows[pos] = q / K;
  }
  mapping[q] = pos;
}

}  // namespace

cudaError_t launch_dispatch(const B200MoePlan& p, cudaStream_t s) {
  const auto& sh = p.shape;
  const int R = p.routes, E = sh.experts;
  const int blocks = (p.partitions + kWarps - 1) / kWarps;
  int* hist = static_cast<int*>(p.buf.scratch);
  int* flags = hist + static_cast<size_t>(p.partitions) * E;
  int* ranks = static_cast<int*>(p.buf.ranks);
  auto* rw = static_cast<const float*>(p.buf.routing_weights);
  auto* valid = static_cast<const int*>(p.buf.valid_routes);
  if (p.dispatch_fused) {
    int* router_flag = hist + router_flag_index(p);
    auto* counts = static_cast<int*>(p.buf.counts);
    auto* offsets = static_cast<int*>(p.buf.offsets);
    auto* cursors = static_cast<int*>(p.buf.cursors);
    auto* tasks = static_cast<int*>(p.buf.tasks);
    auto* status = static_cast<int*>(p.buf.status);
    auto* mapping = static_cast<int*>(p.buf.mapping);
    int* source_rows = p.gather ? static_cast<int*>(p.buf.source_rows) : nullptr;
    if (sh.ids_are_int64) {
      launch_pdl_cluster(dispatch_fused_kernel<long long>, p.dispatch_ctas, dim3(1024), 0, s, static_cast<const long long*>(p.buf.ids), rw, ranks, mapping,
                                                          counts, offsets, cursors, tasks, status, router_flag, valid, R,
                                                          E, p.warp_routes, p.token_tile, p.chain_words, source_rows, sh.topk);
    } else {
      launch_pdl_cluster(dispatch_fused_kernel<int>, p.dispatch_ctas, dim3(1024), 0, s, static_cast<const int*>(p.buf.ids), rw, ranks, mapping, counts,
                                                    offsets, cursors, tasks, status, router_flag, valid, R, E,
                                                    p.warp_routes, p.token_tile, p.chain_words, source_rows, sh.topk);
    }
    if (sh.route_only != 2 && !p.gather)  // the rows are sent to their expert owners / gathered by gate/up instead
      launch_pdl(dispatch_copy_kernel, dim3((R + kWarps - 1) / kWarps), dim3(kThreads), 0, s,
          static_cast<const __nv_bfloat16*>(p.buf.x), static_cast<const int*>(mapping), static_cast<__nv_bfloat16*>(p.buf.grouped_input), R,
          sh.hidden, sh.topk);
    return cudaPeekAtLastError();
  }
  if (sh.ids_are_int64) {
    launch_pdl(dispatch_count_kernel<long long>, dim3(blocks), dim3(kThreads), 0, s,
        static_cast<const long long*>(p.buf.ids), rw, ranks, hist, flags, valid, R, E, p.warp_routes, p.partitions);
  } else {
    launch_pdl(dispatch_count_kernel<int>, dim3(blocks), dim3(kThreads), 0, s,
        static_cast<const int*>(p.buf.ids), rw, ranks, hist, flags, valid, R, E, p.warp_routes, p.partitions);
  }
  launch_pdl(dispatch_scan_kernel, dim3(1), dim3(kMaxExperts), 0, s,
      hist, flags, static_cast<int*>(p.buf.counts), static_cast<int*>(p.buf.offsets),
      static_cast<int*>(p.buf.cursors), static_cast<int*>(p.buf.tasks), static_cast<int*>(p.buf.status),
      hist + router_flag_index(p), E, p.partitions, blocks, p.token_tile, p.chain_words);
  auto* x = static_cast<const __nv_bfloat16*>(p.buf.x);
  auto* grouped = (sh.route_only == 2 || p.gather) ? nullptr : static_cast<__nv_bfloat16*>(p.buf.grouped_input);
  int* source_rows = p.gather ? static_cast<int*>(p.buf.source_rows) : nullptr;
  if (grouped == nullptr) {
    const int mblocks = (R + kThreads - 1) / kThreads;
    if (sh.ids_are_int64) {
      launch_pdl(dispatch_map_kernel<long long>, dim3(mblocks), dim3(kThreads), 0, s,
          static_cast<const long long*>(p.buf.ids), hist, static_cast<const int*>(p.buf.offsets), ranks,
          static_cast<int*>(p.buf.mapping), valid, R, E, sh.topk, p.warp_routes, source_rows);
    } else {
      launch_pdl(dispatch_map_kernel<int>, dim3(mblocks), dim3(kThreads), 0, s,
          static_cast<const int*>(p.buf.ids), hist, static_cast<const int*>(p.buf.offsets), ranks,
          static_cast<int*>(p.buf.mapping), valid, R, E, sh.topk, p.warp_routes, source_rows);
    }
    return cudaPeekAtLastError();
  }
  const int pblocks = (R + kWarps - 1) / kWarps;
  if (sh.ids_are_int64) {
    launch_pdl(dispatch_permute_kernel<long long>, dim3(pblocks), dim3(kThreads), 0, s,
        x, static_cast<const long long*>(p.buf.ids), hist, static_cast<const int*>(p.buf.offsets), ranks,
        static_cast<int*>(p.buf.mapping), grouped, valid, R, E, sh.hidden, sh.topk, p.warp_routes, source_rows);
  } else {
    launch_pdl(dispatch_permute_kernel<int>, dim3(pblocks), dim3(kThreads), 0, s,
        x, static_cast<const int*>(p.buf.ids), hist, static_cast<const int*>(p.buf.offsets), ranks,
        static_cast<int*>(p.buf.mapping), grouped, valid, R, E, sh.hidden, sh.topk, p.warp_routes, source_rows);
  }
  return cudaPeekAtLastError();
}

}  // namespace b200moe

// ---------------------------------------------------------------------------------------------
// b200moe_dispatch_static: the same ranked dispatch for callers that cannot allocate device
// memory (a host that owns the GPU's memory pool, a real-time loop, a plug-in that is only
// handed its input and output buffers). The partition histograms that b200moe_dispatch()
// keeps in the caller's `scratch` workspace live here in one fixed device array, sized for
// B200MOE_STATIC_DISPATCH_MAX_ROUTES routes and 256 experts: 512 partitions x 256 experts
// + 64 block flags + 1 router-flag word, rounded up = 131328 int32 (513 KiB per GPU, held
// from library load to process exit). The array is shared by every call on the device and
// keeps what the last call left in it: the histogram and block-flag words are fully rewritten
// by the counting kernel before anything reads them; the one word that must start at zero
// (the router flag the scan kernel folds into `status`) is cleared on the stream by each call.
// Calls that may overlap on the GPU race on the array. No allocation routine is called.
#include <mutex>

namespace b200moe {
namespace {

constexpr int kStaticScratchInts = 512 * 256 + 64 + 1 + 191;  // 131328
static_assert(kStaticScratchInts % 64 == 0, "keep the array a whole number of 256-byte lines");
static __device__ __align__(256) int g_static_dispatch_scratch[kStaticScratchInts];

constexpr int kMaxDevices = 64;
std::mutex g_static_mutex;
int* g_static_ptr[kMaxDevices] = {};  // device address of the array, per device, looked up once

// In host code the array's name is only a handle for the runtime; the address a kernel can
// use comes from cudaGetSymbolAddress on the device that is current.
int static_scratch_for_current_device(int** out) {
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) {
    set_error("cudaGetDevice: %s", cudaGetErrorString(e));
    return B200MOE_ERR_CUDA;
  }
  if (device < 0 || device >= kMaxDevices) {
    set_error("device index %d outside the supported range", device);
    return B200MOE_ERR_UNSUPPORTED;
  }
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (!g_static_ptr[device]) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_static_dispatch_scratch);
    if (e != cudaSuccess || !ptr) {
      set_error("cudaGetSymbolAddress(static dispatch scratch): %s", cudaGetErrorString(e));
      return B200MOE_ERR_CUDA;
    }
    g_static_ptr[device] = static_cast<int*>(ptr);
  }
  *out = g_static_ptr[device];
  return B200MOE_OK;
}

}  // namespace
}  // namespace b200moe

extern "C" int b200moe_dispatch_static(const B200MoeDispatchArgs* a, void* cuda_stream) {
  using namespace b200moe;
  if (!a) {
    set_error("null argument");
    return B200MOE_ERR_INVALID;
  }
  if (a->tokens < 0 || a->experts < 1 || a->experts > 256 || a->topk < 1 || a->topk > 32 || a->hidden <= 0 ||
      a->token_tile <= 0) {
    set_error("static dispatch: needs T >= 0, E in [1,256], K in [1,32], H > 0, token_tile > 0");
    return B200MOE_ERR_INVALID;
  }
  const long long routes = static_cast<long long>(a->tokens) * a->topk;
  if (routes > B200MOE_STATIC_DISPATCH_MAX_ROUTES) {
    set_error("static dispatch: %lld routes exceed the built-in scratch (at most %d routes); "
              "use b200moe_dispatch with a caller-provided workspace", routes, B200MOE_STATIC_DISPATCH_MAX_ROUTES);
    return B200MOE_ERR_INVALID;
  }
  if (routes == 0) return B200MOE_OK;
  const void* needed[] = {a->x, a->ids, a->routing_weights, a->counts, a->offsets, a->cursors, a->tasks,
                          a->ranks, a->mapping, a->grouped_input, a->status};
  for (const void* ptr : needed)
    if (!ptr) {
      set_error("static dispatch: null buffer");
      return B200MOE_ERR_INVALID;
    }
  // a misaligned pointer from a C caller must come back as an error, not as a device fault
  const uintptr_t ids_align = a->ids_are_int64 ? 8 : 4;
  const void* words4[] = {a->routing_weights, a->counts, a->offsets, a->cursors, a->tasks, a->ranks, a->mapping,
                          a->status};
  bool aligned = reinterpret_cast<uintptr_t>(a->ids) % ids_align == 0 &&
                 (reinterpret_cast<uintptr_t>(a->x) | reinterpret_cast<uintptr_t>(a->grouped_input)) % 2 == 0;
  for (const void* ptr : words4) aligned = aligned && reinterpret_cast<uintptr_t>(ptr) % 4 == 0;
  if (!aligned) {
    set_error("static dispatch: misaligned buffer (int32 / float32 buffers 4 bytes, int64 ids 8 bytes, BF16 rows 2 bytes)");
    return B200MOE_ERR_INVALID;
  }
  int* scratch = nullptr;
  int rc = static_scratch_for_current_device(&scratch);
  if (rc) return rc;

  B200MoePlan p;  // host-side description only; nothing is allocated
  p.shape.tokens = a->tokens;
  p.shape.experts = a->experts;
  p.shape.topk = a->topk;
  p.shape.hidden = a->hidden;
  p.shape.ids_are_int64 = a->ids_are_int64;
  p.routes = static_cast<int>(routes);
  p.token_tile = a->token_tile;
  p.dispatch_fused = false;  // the multi-kernel path: the one that uses global scratch
  const int per_warp = static_cast<int>(((routes + 511) / 512 + 31) / 32 * 32);
  p.warp_routes = per_warp < 128 ? 128 : per_warp;
  p.partitions = static_cast<int>((routes + p.warp_routes - 1) / p.warp_routes);
  if (router_flag_index(p) + 1 > static_cast<size_t>(kStaticScratchInts)) {
    set_error("static dispatch: internal scratch bound exceeded");
    return B200MOE_ERR_INVALID;
  }
  p.buf.x = a->x;
  p.buf.ids = const_cast<void*>(a->ids);
  p.buf.routing_weights = const_cast<void*>(a->routing_weights);
  p.buf.counts = a->counts;
  p.buf.offsets = a->offsets;
  p.buf.cursors = a->cursors;
  p.buf.tasks = a->tasks;
  p.buf.ranks = a->ranks;
  p.buf.mapping = a->mapping;
  p.buf.grouped_input = a->grouped_input;
  p.buf.status = a->status;
  p.buf.scratch = scratch;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  cudaError_t e = cudaMemsetAsync(scratch + router_flag_index(p), 0, sizeof(int), stream);
  if (e == cudaSuccess) e = launch_dispatch(p, stream);
  if (e != cudaSuccess) {
    set_error("static dispatch launch: %s", cudaGetErrorString(e));
    return B200MOE_ERR_CUDA;
  }
  return B200MOE_OK;
}
