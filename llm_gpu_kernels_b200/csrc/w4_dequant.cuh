// W4G128 nibble decode shared by the W4A16 kernels.
//
// Format (reference moe_weight_quant.py:1-6,35-52; device decode cuda_w4_gate_up.cu:28-41): word kw of a channel row
// holds K = 8*kw .. 8*kw+7, nibble j at bits [4j,4j+4), nibble = q + 8 with q in [-7,7]; the operand fed to the MMA is
// exactly bf16_rn(float(q) * float(scale)). (w >> 4j) & 0x000F000F | 0x43004300 is the BF16 pair
// {128 + n_j, 128 + n_(j+4)}; minus 136 is the exact integer q; one BF16 multiply by the scale rounds once.
#pragma once
#include <cuda_bf16.h>
#include <cstdint>

namespace b200moe {
namespace w4 {

// The two constants of the decode as registers the compiler cannot see through. Left as immediates it spends two
// logic instructions per nibble pair; from registers the three-input form takes one. Call once per thread.
struct Consts {
  uint32_t mask, magic;
};
__device__ __forceinline__ Consts make_consts() {
  Consts c{0x000F000Fu, 0x43004300u};
  asm volatile("" : "+r"(c.mask), "+r"(c.magic));
  return c;
}

// (a & b) | c in one logic instruction
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

// One packed word -> four BF16 pairs {k_j, k_(j+4)}, j = 0..3, each bf16_rn(q * scale).
__device__ __forceinline__ void dequant_pairs(uint32_t w, __nv_bfloat162 scale2, const Consts& k, uint32_t (&pair)[4]) {
  const __nv_bfloat162 bias = __float2bfloat162_rn(136.0f);  // 128 (magic exponent) + 8 (zero point)
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint32_t v = and_or(w >> (4 * j), k.mask, k.magic);                          // {128 + n_j, 128 + n_(j+4)}
    __nv_bfloat162 q = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&v), bias);   // exact
    q = __hmul2(q, scale2);                                                       // the one rounding
    pair[j] = *reinterpret_cast<uint32_t*>(&q);
  }
}

// The same in K order: eight BF16 k0..k7 = one 16-byte chunk of an operand row.
__device__ __forceinline__ uint4 dequant_word(uint32_t w, __nv_bfloat162 scale2, const Consts& k) {
  uint32_t pair[4];
  dequant_pairs(w, scale2, k, pair);
  uint4 out;
  out.x = __byte_perm(pair[0], pair[1], 0x5410);  // k0 k1
  out.y = __byte_perm(pair[2], pair[3], 0x5410);  // k2 k3
  out.z = __byte_perm(pair[0], pair[1], 0x7632);  // k4 k5
  out.w = __byte_perm(pair[2], pair[3], 0x7632);  // k6 k7
  return out;
}

}  // namespace w4
}  // namespace b200moe
