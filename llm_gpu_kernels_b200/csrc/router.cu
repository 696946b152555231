// Router: logits = x . Wr^T (BF16 operands, FP32 accumulate in a fixed order),
// FP32 softmax over the experts, top-k by repeated arg-max (ties go to the
// lowest expert index), renormalise the k probabilities to sum 1.
// Formula: the reference's capture script, scripts/capture_qwen3_moe_layer0.py:583-586;
// the operator of the reference takes ids / weights as inputs, so this kernel
// is the new first stage in front of its fixed-route contract (moe.py:227-230).
#include <cuda_bf16.h>
#include "plan.h"

namespace b200moe {
namespace {

constexpr int kRouterThreads = 512;
constexpr int kRouterTokens = 4;  // tokens per block

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <typename IdT>
__global__ void __launch_bounds__(kRouterThreads)
router_topk_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ wr,
                   IdT* __restrict__ ids, float* __restrict__ rw, int T, int E, int H, int K, int bf16_weights) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* xs = reinterpret_cast<float*>(smem_raw);               // [kRouterTokens][H]
  float* logits = xs + static_cast<size_t>(kRouterTokens) * H;   // [kRouterTokens][E]
  const int t0 = blockIdx.x * kRouterTokens;
  const int nt = min(kRouterTokens, T - t0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = kRouterThreads >> 5;

  for (int i = threadIdx.x; i < kRouterTokens * H; i += kRouterThreads) {
    const int tt = i / H, h = i - tt * H;
    xs[i] = tt < nt ? __bfloat162float(x[static_cast<size_t>(t0 + tt) * H + h]) : 0.0f;
  }
  __syncthreads();

  const bool vec = (H % 8 == 0) && ((reinterpret_cast<uintptr_t>(wr) & 15) == 0);
  for (int e = warp; e < E; e += nwarps) {
    float acc[kRouterTokens];
#pragma unroll
    for (int tt = 0; tt < kRouterTokens; ++tt) acc[tt] = 0.0f;
    const __nv_bfloat16* row = wr + static_cast<size_t>(e) * H;
    if (vec) {
#pragma unroll 4
      for (int h = lane * 8; h < H; h += 256) {
        const uint4 p = *reinterpret_cast<const uint4*>(row + h);
        const uint32_t u[4] = {p.x, p.y, p.z, p.w};
        float w[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          w[2 * j] = __uint_as_float(u[j] << 16);
          w[2 * j + 1] = __uint_as_float(u[j] & 0xffff0000u);
        }
#pragma unroll
        for (int tt = 0; tt < kRouterTokens; ++tt) {
          const float4 a = *reinterpret_cast<const float4*>(xs + tt * H + h);
          const float4 b = *reinterpret_cast<const float4*>(xs + tt * H + h + 4);
          acc[tt] = fmaf(a.x, w[0], acc[tt]); acc[tt] = fmaf(a.y, w[1], acc[tt]);
          acc[tt] = fmaf(a.z, w[2], acc[tt]); acc[tt] = fmaf(a.w, w[3], acc[tt]);
          acc[tt] = fmaf(b.x, w[4], acc[tt]); acc[tt] = fmaf(b.y, w[5], acc[tt]);
          acc[tt] = fmaf(b.z, w[6], acc[tt]); acc[tt] = fmaf(b.w, w[7], acc[tt]);
        }
      }
    } else {
      for (int h = lane; h < H; h += 32) {
        const float w = __bfloat162float(row[h]);
#pragma unroll
        for (int tt = 0; tt < kRouterTokens; ++tt) acc[tt] = fmaf(xs[tt * H + h], w, acc[tt]);
      }
    }
#pragma unroll
    for (int tt = 0; tt < kRouterTokens; ++tt) {
      const float s = warp_sum(acc[tt]);
      if (lane == 0) logits[tt * E + e] = s;
    }
  }
  __syncthreads();

  if (warp >= nt) return;
  // one warp per token: softmax, then K rounds of arg-max
  float* l = logits + warp * E;
  float m = -INFINITY;
  for (int e = lane; e < E; e += 32) m = fmaxf(m, l[e]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  float sum = 0.0f;
  for (int e = lane; e < E; e += 32) {
    const float p = expf(l[e] - m);
    l[e] = p;
    sum += p;
  }
  sum = warp_sum(sum);
  for (int e = lane; e < E; e += 32) l[e] = l[e] / sum;
  __syncwarp();

  const int token = t0 + warp;
  float chosen_w = 0.0f;  // lane k keeps the k-th pick
  int chosen_e = 0;
  float total = 0.0f;
  for (int k = 0; k < K; ++k) {
    float best = -1.0f;
    int best_e = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float p = l[e];
      if (p > best) { best = p; best_e = e; }  // ascending e: first maximum wins
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
    }
    if (best_e >= E) { best_e = min(k, E - 1); best = 0.0f; }  // NaN logits: stay in range
    if (lane == k) { chosen_w = best; chosen_e = best_e; }
    total += best;
    if (lane == (best_e & 31)) l[best_e] = -2.0f;
    __syncwarp();
  }
  if (lane < K) {
    ids[static_cast<size_t>(token) * K + lane] = static_cast<IdT>(chosen_e);
    const float w = chosen_w / total;
    rw[static_cast<size_t>(token) * K + lane] = bf16_weights ? __bfloat162float(__float2bfloat16_rn(w)) : w;
  }
}

}  // namespace

cudaError_t launch_router(const B200MoePlan& p, cudaStream_t s) {
  const auto& sh = p.shape;
  const int grid = (sh.tokens + kRouterTokens - 1) / kRouterTokens;
  const size_t smem = (static_cast<size_t>(kRouterTokens) * sh.hidden + kRouterTokens * sh.experts) * sizeof(float);
  auto* x = static_cast<const __nv_bfloat16*>(p.buf.x);
  auto* wr = static_cast<const __nv_bfloat16*>(p.buf.router_weight);
  auto* rw = static_cast<float*>(p.buf.routing_weights);
  if (sh.ids_are_int64) {
    router_topk_kernel<long long><<<grid, kRouterThreads, smem, s>>>(
        x, wr, static_cast<long long*>(p.buf.ids), rw, sh.tokens, sh.experts, sh.hidden, sh.topk, sh.router_bf16_weights);
  } else {
    router_topk_kernel<int><<<grid, kRouterThreads, smem, s>>>(
        x, wr, static_cast<int*>(p.buf.ids), rw, sh.tokens, sh.experts, sh.hidden, sh.topk, sh.router_bf16_weights);
  }
  return cudaPeekAtLastError();
}

size_t router_smem_bytes(int hidden, int experts) {
  return (static_cast<size_t>(kRouterTokens) * hidden + kRouterTokens * experts) * sizeof(float);
}

// The opt-in is an attribute of the kernel, not of a plan: always raise it to the device limit, so that binding a
// second plan with a smaller hidden size cannot lower it under the first plan's launches.
cudaError_t router_opt_in_smem() {
  constexpr int kLimit = 227 * 1024;
  cudaError_t e = cudaFuncSetAttribute(router_topk_kernel<int>, cudaFuncAttributeMaxDynamicSharedMemorySize, kLimit);
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(router_topk_kernel<long long>, cudaFuncAttributeMaxDynamicSharedMemorySize, kLimit);
}

}  // namespace b200moe
