// CUDA-core ragged grouped GEMM for shapes the TMA/tcgen05 schedule cannot take
// (H or I not a multiple of 8, unaligned bases). Same contract as the
// reference's _dynamic_grouped / _dynamic_grouped_gate_up_swiglu
// (moe.py:69-95, moe_fused.py:18-73): a host-computable upper bound of tiles is
// launched, tile -> expert by binary search over the `tasks` prefix, excess
// blocks exit; FP32 accumulation; gate and up share the activation tile and
// SwiGLU runs on the FP32 accumulators before the single BF16 rounding.
#include <cuda_bf16.h>
#include "plan.h"

namespace b200moe {
namespace {

constexpr int BM = kGenericTile, BN = 64, BK = 32, kThreads = 256;

template <bool kGateUp>
__global__ void __launch_bounds__(kThreads)
grouped_gemm_generic_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ w,
                            __nv_bfloat16* __restrict__ out, const int* __restrict__ offsets,
                            const int* __restrict__ counts, const int* __restrict__ tasks, int E, int n_out,
                            int k_dim) {
  const int task = blockIdx.x;
  if (task >= tasks[E]) return;
  int lo = 0, hi = E;
  while (lo < hi) {  // first expert whose tile range ends after `task`
    const int mid = (lo + hi) >> 1;
    if (task >= tasks[mid + 1]) lo = mid + 1; else hi = mid;
  }
  const int expert = lo;
  const int local0 = (task - tasks[expert]) * BM;
  const int row_base = offsets[expert], row_count = counts[expert];
  const int n0 = blockIdx.y * BN;
  const size_t w_rows = static_cast<size_t>(kGateUp ? 2 * n_out : n_out);
  const __nv_bfloat16* wg = w + static_cast<size_t>(expert) * w_rows * k_dim;
  const __nv_bfloat16* wu = wg + static_cast<size_t>(n_out) * k_dim;  // used when kGateUp

  __shared__ float As[BM][BK + 1];
  __shared__ float Gs[BN][BK + 1];
  __shared__ float Us[kGateUp ? BN : 1][BK + 1];
  const int ty = threadIdx.x / 16, tx = threadIdx.x % 16;  // 16 x 16 threads, 2 rows x 4 cols each
  float accg[2][4] = {}, accu[2][4] = {};

  for (int k0 = 0; k0 < k_dim; k0 += BK) {
    for (int i = threadIdx.x; i < BM * BK; i += kThreads) {
      const int r = i / BK, k = i % BK;
      const bool ok = local0 + r < row_count && k0 + k < k_dim;
      As[r][k] = ok ? __bfloat162float(a[static_cast<size_t>(row_base + local0 + r) * k_dim + k0 + k]) : 0.0f;
    }
    for (int i = threadIdx.x; i < BN * BK; i += kThreads) {
      const int c = i / BK, k = i % BK;
      const bool ok = n0 + c < n_out && k0 + k < k_dim;
      const size_t idx = static_cast<size_t>(n0 + c) * k_dim + k0 + k;
      Gs[c][k] = ok ? __bfloat162float(wg[idx]) : 0.0f;
      if (kGateUp) Us[c][k] = ok ? __bfloat162float(wu[idx]) : 0.0f;
    }
    __syncthreads();
#pragma unroll 8
    for (int k = 0; k < BK; ++k) {
      const float a0 = As[ty * 2][k], a1 = As[ty * 2 + 1][k];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float g = Gs[tx * 4 + j][k];
        accg[0][j] = fmaf(a0, g, accg[0][j]);
        accg[1][j] = fmaf(a1, g, accg[1][j]);
        if (kGateUp) {
          const float u = Us[tx * 4 + j][k];
          accu[0][j] = fmaf(a0, u, accu[0][j]);
          accu[1][j] = fmaf(a1, u, accu[1][j]);
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = local0 + ty * 2 + i;
    if (r >= row_count) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = n0 + tx * 4 + j;
      if (c >= n_out) continue;
      float v = accg[i][j];
      if (kGateUp) v = (v / (1.0f + expf(-v))) * accu[i][j];
      out[static_cast<size_t>(row_base + r) * n_out + c] = __float2bfloat16_rn(v);
    }
  }
}

inline dim3 generic_grid(const B200MoePlan& p, int n_out) {
  const int bound = (p.routes + BM - 1) / BM + p.shape.experts - 1;
  return dim3(bound, (n_out + BN - 1) / BN);
}

}  // namespace

cudaError_t launch_gate_up_generic(const B200MoePlan& p, cudaStream_t s) {
  const auto& sh = p.shape;
  grouped_gemm_generic_kernel<true><<<generic_grid(p, sh.intermediate), kThreads, 0, s>>>(
      static_cast<const __nv_bfloat16*>(p.buf.grouped_input), static_cast<const __nv_bfloat16*>(p.buf.gate_up),
      static_cast<__nv_bfloat16*>(p.buf.activated), static_cast<const int*>(p.buf.offsets),
      static_cast<const int*>(p.buf.counts), static_cast<const int*>(p.buf.tasks), sh.experts, sh.intermediate,
      sh.hidden);
  return cudaPeekAtLastError();
}

cudaError_t launch_down_generic(const B200MoePlan& p, cudaStream_t s) {
  const auto& sh = p.shape;
  grouped_gemm_generic_kernel<false><<<generic_grid(p, sh.hidden), kThreads, 0, s>>>(
      static_cast<const __nv_bfloat16*>(p.buf.activated), static_cast<const __nv_bfloat16*>(p.buf.down),
      static_cast<__nv_bfloat16*>(p.buf.down_output), static_cast<const int*>(p.buf.offsets),
      static_cast<const int*>(p.buf.counts), static_cast<const int*>(p.buf.tasks), sh.experts, sh.hidden,
      sh.intermediate);
  return cudaPeekAtLastError();
}

}  // namespace b200moe
