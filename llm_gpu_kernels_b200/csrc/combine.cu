// Weighted combine back to token order:
//   out[t,:] = bf16( sum_{slot=0..K-1} float(down_output[mapping[t*K+slot],:]) * rw[t,slot] )
// in fixed slot order, FP32, multiply and add kept as separate roundings -
// the semantics of the reference's _combine (moe.py:109-121, launched with
// enable_fp_fusion=False at moe.py:217). A gather-reduce, not a scatter with
// atomics, so the result does not depend on scheduling. Routes with
// mapping < 0 (invalid expert id) contribute nothing (moe.py:117).
// Optional residual: out = bf16(float(residual[t,:]) + float(bf16(sum))) - what the layer followed by the
// model's BF16 residual add gives, without writing and re-reading the layer output.
#include <cuda_bf16.h>
#include "plan.h"
#include "pdl.cuh"

namespace b200moe {
namespace {

constexpr int kThreads = 64;  // small blocks: T * H/512 of them even for a handful of tokens

template <bool kVec>
__global__ void __launch_bounds__(kThreads)
combine_kernel(const __nv_bfloat16* __restrict__ down_out, const int* __restrict__ mapping,
               const float* __restrict__ rw, __nv_bfloat16* __restrict__ out, const int* __restrict__ valid_routes,
               const __nv_bfloat16* __restrict__ residual, int H, int K) {
  pdl_launch_dependents();
  pdl_wait();  // down_output / mapping come from the kernels before
  const int token = blockIdx.x;
  if (valid_routes && token * K >= *valid_routes) return;  // padding rows of a fixed-capacity buffer
  __shared__ int s_pos[32];
  __shared__ float s_w[32];
  if (threadIdx.x < K) {
    s_pos[threadIdx.x] = mapping[static_cast<size_t>(token) * K + threadIdx.x];
    s_w[threadIdx.x] = rw[static_cast<size_t>(token) * K + threadIdx.x];
  }
  __syncthreads();
  if (kVec) {
    const int h = (blockIdx.y * kThreads + threadIdx.x) * 8;
    if (h >= H) return;
    float acc[8] = {};
    for (int s0 = 0; s0 < K; s0 += 8) {  // issue the (independent) row loads first, then add in slot order
      uint4 v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int slot = s0 + j;
        const int pos = slot < K ? s_pos[slot] : -1;
        v[j] = pos >= 0 ? *reinterpret_cast<const uint4*>(down_out + static_cast<size_t>(pos) * H + h)
                        : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int slot = s0 + j;
        if (slot >= K || s_pos[slot] < 0) continue;
        const float w = s_w[slot];
        const uint32_t u[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          acc[2 * i] = __fadd_rn(acc[2 * i], __fmul_rn(__uint_as_float(u[i] << 16), w));
          acc[2 * i + 1] = __fadd_rn(acc[2 * i + 1], __fmul_rn(__uint_as_float(u[i] & 0xffff0000u), w));
        }
      }
    }
    uint4 o;
    uint32_t* ou = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __nv_bfloat162 v = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
      ou[j] = *reinterpret_cast<const uint32_t*>(&v);
    }
    if (residual) {
      const uint4 r = *reinterpret_cast<const uint4*>(residual + static_cast<size_t>(token) * H + h);
      const uint32_t ru[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const __nv_bfloat162 v = __floats2bfloat162_rn(
            __fadd_rn(__uint_as_float(ru[j] << 16), __uint_as_float(ou[j] << 16)),
            __fadd_rn(__uint_as_float(ru[j] & 0xffff0000u), __uint_as_float(ou[j] & 0xffff0000u)));
        ou[j] = *reinterpret_cast<const uint32_t*>(&v);
      }
    }
    *reinterpret_cast<uint4*>(out + static_cast<size_t>(token) * H + h) = o;
  } else {
    const int h = blockIdx.y * kThreads + threadIdx.x;
    if (h >= H) return;
    float acc = 0.0f;
    for (int slot = 0; slot < K; ++slot) {
      const int pos = s_pos[slot];
      if (pos < 0) continue;
      acc = __fadd_rn(acc, __fmul_rn(__bfloat162float(down_out[static_cast<size_t>(pos) * H + h]), s_w[slot]));
    }
    __nv_bfloat16 r = __float2bfloat16_rn(acc);
    if (residual)
      r = __float2bfloat16_rn(__fadd_rn(__bfloat162float(residual[static_cast<size_t>(token) * H + h]), __bfloat162float(r)));
    out[static_cast<size_t>(token) * H + h] = r;
  }
}

}  // namespace

cudaError_t launch_combine(const B200MoePlan& p, cudaStream_t s) {
  const auto& sh = p.shape;
  auto* d = static_cast<const __nv_bfloat16*>(p.buf.down_output);
  auto* o = static_cast<__nv_bfloat16*>(p.buf.output);
  auto* res = static_cast<const __nv_bfloat16*>(p.buf.residual);
  const bool vec = sh.hidden % 8 == 0 &&
                   ((reinterpret_cast<uintptr_t>(d) | reinterpret_cast<uintptr_t>(o) | reinterpret_cast<uintptr_t>(res)) & 15) == 0;
  if (vec) {
    dim3 grid(sh.tokens, (sh.hidden / 8 + kThreads - 1) / kThreads);
    launch_pdl(combine_kernel<true>, grid, dim3(kThreads), 0, s, d, static_cast<const int*>(p.buf.mapping),
                                                   static_cast<const float*>(p.buf.routing_weights), o,
                                                   static_cast<const int*>(p.buf.valid_routes), res, sh.hidden, sh.topk);
  } else {
    dim3 grid(sh.tokens, (sh.hidden + kThreads - 1) / kThreads);
    launch_pdl(combine_kernel<false>, grid, dim3(kThreads), 0, s, d, static_cast<const int*>(p.buf.mapping),
                                                    static_cast<const float*>(p.buf.routing_weights), o,
                                                    static_cast<const int*>(p.buf.valid_routes), res, sh.hidden, sh.topk);
  }
  return cudaPeekAtLastError();
}

}  // namespace b200moe
