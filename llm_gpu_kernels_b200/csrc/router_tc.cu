// Router on the tensor cores: logits[token][expert] = x . Wr^T as a tcgen05 GEMM per
// 128-token tile (tokens on the TMEM lanes, experts on the columns), with the K dimension
// split over the CTAs of a thread-block cluster: each CTA multiplies its K slice and parks
// its partial logits in shared memory; after a cluster barrier CTA c sums rows
// [c*128/S, (c+1)*128/S) of all S partials through distributed shared memory (fixed order,
// so the result is reproducible) and routes them. The
// epilogue warps copy the FP32 logits from tensor memory to shared memory (reusing the
// drained operand stages), then sixteen warps take rows in turn: the 32 lanes share one
// row's experts, softmax by warp reductions, top-k by k rounds of warp arg-max done with
// integer warp reductions (redux.sync) on order-preserving keys of the logits.
//
// Formula: scripts/capture_qwen3_moe_layer0.py:583-586 of the reference (FP32
// softmax, top-k, divide by the sum of the k). The k experts are taken in
// descending logit order (softmax is monotonic), ties to the lowest index;
// weights are exp(l - max) / sum over all experts, renormalised over the k.
// Columns >= E (zero-filled by TMA) and lanes >= T are masked.
#include <cuda_bf16.h>
#include "plan.h"
#include "sm100_ptx.cuh"
#include "pdl.cuh"

namespace b200moe {
namespace {

using namespace ptx;

constexpr int kRowWarps = 16;      // warps 2..17 work on rows; the first four of them also read TMEM
constexpr int kThreads = 64 + kRowWarps * 32;  // warp 0 TMA, warp 1 MMA + TMEM owner
constexpr int kMaxStages = 8;
constexpr int kTileTokens = 128;   // UMMA M
constexpr int kBlockK = 64;
constexpr int kCtrlBytes = 1024;
constexpr int kSmemLimit = 232448;

struct Ctrl {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t tmem_full;
  uint32_t tmem_base;
  int abort;
};
static_assert(sizeof(Ctrl) <= kCtrlBytes, "control block too large");

// kPerLane: experts per lane in the routing epilogue (ceil(E / 32) rounded up to 1, 2, 4 or 8): the top-k rounds
// walk exactly the keys a lane holds.
template <typename IdT, int kPerLane>
__global__ void __launch_bounds__(kThreads, 1)
router_tc_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_wr,
                 IdT* __restrict__ ids, float* __restrict__ rw, int* __restrict__ status, int T, int E, int H,
                 int K, int e_pad, int num_stages, int ksplit, int bf16_weights) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  Ctrl* c = reinterpret_cast<Ctrl*>(smem_raw);
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t stage_off = ((raw_addr + kCtrlBytes + 1023u) & ~1023u) - raw_addr;
  unsigned char* stages = smem_raw + stage_off;
  constexpr uint32_t kXBytes = kTileTokens * 128;
  const uint32_t stage_bytes = kXBytes + static_cast<uint32_t>(e_pad) * 128u;
  uint32_t tmem_cols = 32;
  while (tmem_cols < static_cast<uint32_t>(e_pad)) tmem_cols <<= 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint32_t cta_rank;  // rank inside the cluster = K slice
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(cta_rank));
  const int t0 = (blockIdx.x / ksplit) * kTileTokens;
  const int num_kb = (H + kBlockK - 1) / kBlockK;
  const int kb_per = (num_kb + ksplit - 1) / ksplit;
  const int kb0 = min(num_kb, static_cast<int>(cta_rank) * kb_per), kb1 = min(num_kb, kb0 + kb_per);

  if (threadIdx.x == 0) {
    for (int s = 0; s < num_stages; ++s) {
      mbar_init(&c->full[s], 1);
      mbar_init(&c->empty[s], 1);
    }
    mbar_init(&c->tmem_full, 1);
    c->abort = 0;
    mbar_init_fence();
  }
  pdl_launch_dependents();
  if (warp == 1) tmem_alloc(&c->tmem_base, tmem_cols);
  pdl_wait();  // x may be written by the kernel just before; ids / weights may still be read by it
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&c->tmem_base);
  const int ld = e_pad + 1;                            // row stride in floats: conflict-free column writes
  float* logits = reinterpret_cast<float*>(stages);    // [128][ld] partial logits, aliases the drained operand stages

  if (warp == 0) {
    if (lane == 0) {
      const uint64_t pol = policy_evict_last();  // x is read again by dispatch, Wr by every tile
      int stage = 0, issued = 0;
      uint32_t phase = 0;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(&c->empty[stage], phase ^ 1u, &c->abort, status)) break;
        unsigned char* st = stages + static_cast<size_t>(stage) * stage_bytes;
        mbar_expect_tx(&c->full[stage], stage_bytes);
        tma_load_2d(st, &tm_x, &c->full[stage], kb * kBlockK, t0, pol);
        tma_load_2d(st + kXBytes, &tm_wr, &c->full[stage], kb * kBlockK, 0, pol);
        ++issued;
        if (++stage == num_stages) { stage = 0; phase ^= 1u; }
      }
      for (int i = issued > num_stages ? issued - num_stages : 0; i < issued; ++i) {  // no copy left in flight
        if (!mbar_wait_plain(&c->full[i % num_stages], static_cast<uint32_t>((i / num_stages) & 1))) {
          atomicOr(status, B200MOE_STATUS_TIMEOUT);
          break;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(kTileTokens, e_pad);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(&c->full[stage], phase, &c->abort, status)) { ok = false; break; }
        tc_fence_after();
        const uint32_t x_addr = smem_u32(stages + static_cast<size_t>(stage) * stage_bytes);
        const uint32_t w_addr = x_addr + kXBytes;
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma(tmem_base, umma_desc(x_addr + k * 32), umma_desc(w_addr + k * 32), idesc, (kb > kb0 || k != 0) ? 1u : 0u);
        umma_commit(&c->empty[stage]);
        if (++stage == num_stages) { stage = 0; phase ^= 1u; }
      }
      if (kb1 > kb0) umma_commit(&c->tmem_full);  // also the drain point when the loop gave up
      else mbar_arrive(&c->tmem_full);            // empty K slice: nothing to wait for
      if (!ok) mbar_wait_plain(&c->tmem_full, 0);
    }
  } else if (warp < 6) {
    // ---------------------------------------------------------------- TMEM -> shared memory (this CTA's partial)
    const int quarter = warp & 3;                 // the TMEM lane quarter this warp may read
    const bool ready = __all_sync(0xffffffffu, mbar_wait(&c->tmem_full, 0, &c->abort, status));
    if (ready) {
      tc_fence_after();
      const int r = quarter * 32 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
      for (int c0 = 0; c0 < e_pad; c0 += 16) {
        uint32_t v[16];
        if (kb1 > kb0) {
          tmem_ld16(taddr + c0, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = 0u;  // empty K slice contributes zero
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) logits[r * ld + c0 + j] = __uint_as_float(v[j]);
      }
    }
  }
  // every CTA's partial is in its shared memory
  __syncwarp();
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  if (warp >= 2) {
    // ---------------------------------------------------------------- rows of this CTA: reduce over the cluster, route
    const int rows_live = min(kTileTokens, T - t0);
    const int rows_per_cta = kTileTokens / ksplit;
    const uint32_t logits_addr = smem_u32(logits);
    for (int rr = warp - 2; rr < rows_per_cta; rr += kRowWarps) {
      const int r = static_cast<int>(cta_rank) * rows_per_cta + rr;
      if (r >= rows_live) break;
      {
        // key(x): unsigned, monotonic in x; 0 is below every finite logit and marks "absent / taken"
        uint32_t key[kPerLane];
        uint32_t kmax_local = 0;
#pragma unroll
        for (int j = 0; j < kPerLane; ++j) {
          const int e = j * 32 + lane;
          uint32_t u = 0;
          if (e < E) {
            float sum_parts = 0.0f;
            for (int sidx = 0; sidx < ksplit; ++sidx) {  // fixed order: slice 0, 1, ...
              uint32_t remote;
              asm volatile("mapa.shared::cluster.u32 %0, %1, %2;"
                           : "=r"(remote) : "r"(logits_addr + static_cast<uint32_t>((r * ld + e) * 4)), "r"(sidx));
              float part;
              asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(part) : "r"(remote) : "memory");
              sum_parts += part;
            }
            u = __float_as_uint(sum_parts);
            u ^= (u >> 31) ? 0xffffffffu : 0x80000000u;
          }
          key[j] = u;
          kmax_local = max(kmax_local, u);
        }
        const uint32_t kmax = __reduce_max_sync(0xffffffffu, kmax_local);
        const float m = __uint_as_float((kmax >> 31) ? (kmax ^ 0x80000000u) : ~kmax);
        float sum = 0.0f;
#pragma unroll
        for (int j = 0; j < kPerLane; ++j) {
          if (key[j]) {
            const uint32_t u = key[j];
            sum += expf(__uint_as_float((u >> 31) ? (u ^ 0x80000000u) : ~u) - m);
          }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        uint32_t my_key = 0;
        int my_e = 0;
        for (int k = 0; k < K; ++k) {
          uint32_t best = 0;
#pragma unroll
          for (int j = 0; j < kPerLane; ++j) best = max(best, key[j]);
          const uint32_t top = __reduce_max_sync(0xffffffffu, best);
          int cand = 0x7fffffff;                     // lowest expert index holding the top key
#pragma unroll
          for (int j = kPerLane - 1; j >= 0; --j)
            if (key[j] == top) cand = j * 32 + lane;
          int be = __reduce_min_sync(0xffffffffu, top ? cand : 0x7fffffff);
          if (be >= E) be = min(k, E - 1);           // row exhausted (NaNs / K > finite entries): stay in range
          const int taken = (be & 31) == lane ? (be >> 5) : -1;
#pragma unroll
          for (int j = 0; j < kPerLane; ++j) key[j] = j == taken ? 0u : key[j];
          if (lane == k) { my_key = top; my_e = be; }
        }
        float p = 0.0f;
        if (lane < K && my_key)
          p = expf(__uint_as_float((my_key >> 31) ? (my_key ^ 0x80000000u) : ~my_key) - m) / sum;
        float total = p;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
        if (lane < K) {
          const size_t o = static_cast<size_t>(t0 + r) * K + lane;
          ids[o] = static_cast<IdT>(my_e);
          const float w = p / total;
          rw[o] = bf16_weights ? __bfloat162float(__float2bfloat16_rn(w)) : w;
        }
      }
    }
  }

  // no CTA may leave while another still reads its partial
  __syncwarp();
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, tmem_cols);
  }
}

}  // namespace

int router_ksplit(int hidden, int tokens) {
  const int num_kb = (hidden + kBlockK - 1) / kBlockK;
  int split = 1;
  while (split < 8 && num_kb / (split * 2) >= 2) split *= 2;  // at least two k-blocks per CTA
  // All clusters should be resident at once, or the router runs in waves. Clusters of 8 (one CTA per SM) fit about
  // two per GPC: 12 of them measured fine (21.5 us at 12 token tiles), 16 did not (35.8 us at 16 token tiles against
  // 27.6 us with clusters of 4); smaller clusters pack up to 128 CTAs (25.6 us at 32 tiles x 4, 37.9 us at 64 x 2;
  // 35.7 / 54.3 us when capped at 64 CTAs).
  const int tiles = (tokens + kTileTokens - 1) / kTileTokens;
  while (split > 1 && tiles * split > (split == 8 ? 96 : 128)) split /= 2;
  return split;
}

int configure_router_tc(B200MoePlan& p) {
  const int e_pad = (p.shape.experts + 15) / 16 * 16;
  const int stage = kTileTokens * 128 + e_pad * 128;
  const int num_kb = (p.shape.hidden + kBlockK - 1) / kBlockK;
  const int ksplit = router_ksplit(p.shape.hidden, p.shape.tokens);
  const int kb_per = (num_kb + ksplit - 1) / ksplit;
  int stages = (kSmemLimit - kCtrlBytes - 1024) / stage;
  if (stages > kMaxStages) stages = kMaxStages;
  if (stages > kb_per) stages = kb_per < 2 ? 2 : kb_per;
  while (stages * stage < kTileTokens * (e_pad + 1) * 4) ++stages;  // the partial logits reuse this space
  p.router_stages = stages;
  p.router_smem = kCtrlBytes + 1024 + stages * stage;
  p.router_ksplit = ksplit;
  const void* kernels[] = {
      reinterpret_cast<const void*>(router_tc_kernel<int, 1>), reinterpret_cast<const void*>(router_tc_kernel<int, 2>),
      reinterpret_cast<const void*>(router_tc_kernel<int, 4>), reinterpret_cast<const void*>(router_tc_kernel<int, 8>),
      reinterpret_cast<const void*>(router_tc_kernel<long long, 1>),
      reinterpret_cast<const void*>(router_tc_kernel<long long, 2>),
      reinterpret_cast<const void*>(router_tc_kernel<long long, 4>),
      reinterpret_cast<const void*>(router_tc_kernel<long long, 8>)};
  for (const void* kernel : kernels) {
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
    if (e != cudaSuccess) {
      set_error("cudaFuncSetAttribute(router shared memory) failed: %s", cudaGetErrorString(e));
      return B200MOE_ERR_CUDA;
    }
  }
  return B200MOE_OK;
}

template <typename IdT>
cudaError_t launch_router_typed(const B200MoePlan& p, cudaStream_t s, IdT* ids) {
  const auto& sh = p.shape;
  const int tiles = (sh.tokens + kTileTokens - 1) / kTileTokens;
  const int e_pad = (sh.experts + 15) / 16 * 16;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles * p.router_ksplit);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = p.router_smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = p.router_ksplit;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  int* status = static_cast<int*>(p.buf.scratch) + router_flag_index(p);  // folded into status by the dispatch
  auto* rw = static_cast<float*>(p.buf.routing_weights);
  auto launch = [&](auto kernel) {
    return cudaLaunchKernelEx(&cfg, kernel, p.tm_x, p.tm_router_w, ids, rw, status, sh.tokens, sh.experts, sh.hidden,
                              sh.topk, e_pad, p.router_stages, p.router_ksplit, sh.router_bf16_weights);
  };
  if (e_pad <= 32) return launch(router_tc_kernel<IdT, 1>);
  if (e_pad <= 64) return launch(router_tc_kernel<IdT, 2>);
  if (e_pad <= 128) return launch(router_tc_kernel<IdT, 4>);
  return launch(router_tc_kernel<IdT, 8>);
}


cudaError_t launch_router_tc(const B200MoePlan& p, cudaStream_t s) {
  cudaError_t e = p.shape.ids_are_int64 ? launch_router_typed<long long>(p, s, static_cast<long long*>(p.buf.ids))
                                        : launch_router_typed<int>(p, s, static_cast<int*>(p.buf.ids));
  return e != cudaSuccess ? e : cudaPeekAtLastError();
}

}  // namespace b200moe
