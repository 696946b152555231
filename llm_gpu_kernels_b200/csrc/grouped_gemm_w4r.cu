// W4A16 ragged grouped GEMM for the weight-streaming regime (an expert has at most 16 rows per tile):
// packed int4 weights (the reference's W4G128 v1 format) are TMA-loaded to shared memory as stored and
// dequantised to BF16 IN REGISTERS by the warps that multiply them - the dequantised weight never touches
// shared or tensor memory.
//
// Format contract (reference moe_weight_quant.py:1-6,35-52 and the device decode of
// cuda_w4_gate_up.cu:28-41): words[e][n][kw] holds K = 8*kw .. 8*kw+7, nibble j at bits [4j,4j+4),
// nibble = q + 8 with q in [-7,7]; one BF16 scale per (expert, output channel, 128 consecutive K); the
// operand fed to the MMA is exactly bf16_rn(float(q) * float(scale)). Here: (w >> 4j) & 0x000F000F |
// 0x43004300 gives the BF16 pair {128 + n_j, 128 + n_(j+4)}, minus 136 is the exact integer q, and one
// BF16 multiply by the scale rounds once - the same value.
//
// Why not tcgen05 here. With 1-16 rows per expert the layer is bound by HBM, and with 4-bit weights one SM
// must dequantise 45 weights per clock to keep up with its share of HBM. The tcgen05 variants
// (grouped_gemm_w4t.cu, grouped_gemm_w4.cu) pass every dequantised tile from converter warps through tensor or
// shared memory to one MMA-issuing thread; that hand-over chain, not a pipe, bounded them at 0.3 of the HBM
// roofline. In this kernel a warp owns 16 output channels of the gate tile and the same 16 of the up tile:
// it reads its packed words with ldmatrix (each thread gets word t of rows g and g+8), dequantises them
// into the A fragments of mma.sync.m16n8k16 and multiplies at once. Tensor throughput is irrelevant in this
// regime (< 0.1 PFLOP/s needed), instruction issue is what counts, so:
//  * No shuffle to restore K order: a dot product does not care about the order of its terms, so the pair
//    {k_j, k_(j+4)} that falls out of one mask is fed as it is and the ACTIVATION tile is stored in shared
//    memory with every 8 K permuted to match (k0 k4 k1 k5 | k2 k6 k3 k7). Two producer warps copy the rows
//    from global memory with plain loads and apply that permutation on the way (4 byte-permutes per 16 bytes
//    of activations against 15 instructions per 4 bytes of weights).
//  * gate and up share every activation fragment; SwiGLU is applied to the FP32 accumulators of the same
//    thread. For the down projection the two weight boxes are the low and the high 128 channels of a
//    256-channel tile, so the structure is the same.
//  * 16 consumer warps in two groups: group g multiplies K half g (128 K = one scale group) of every 256-K
//    stage, so a stage is released after half the time and more of the ring is in flight; the two partial
//    sums are added in FP32 (group 0 + group 1, fixed order) before the epilogue. The scales come straight
//    from global memory (read-only path, fetched one stage ahead): the whole ring is weights and rows.
// Chaining with the other GEMM of the forward, dynamic tiles for the down projection, bounded waits and the
// status word work as in grouped_gemm_tcgen05.cu.
#include <cuda_bf16.h>
#include <cuda.h>
#include "plan.h"
#include "sm100_ptx.cuh"
#include "gemm_tile.cuh"
#include "pdl.cuh"
#include "w4_dequant.cuh"

namespace b200moe {
namespace {

using namespace ptx;
using namespace tile;

constexpr int kGroups = 2;                    // consumer groups; group g takes K half g of every stage
constexpr int kGroupWarps = 8;                // 16 channel rows of each weight box per warp: 128 rows per box
constexpr int kConsumerWarps = kGroups * kGroupWarps;
constexpr int kRowWarps = 2;                  // warps that bring the activation rows
constexpr int kFirstConsumer = 1 + kRowWarps;  // warp 0: TMA (packed words, scales)
constexpr int kThreads = 32 * (kFirstConsumer + kConsumerWarps);   // 608
constexpr int kStageK = 256;                  // K of one stage: 128 bytes of packed words per channel row
constexpr uint32_t kBoxBytes = 128 * 128;     // one box of packed words: 128 rows x 32 int32
constexpr int kMaxStages = 6;
constexpr int kMaxTile = 16;                  // rows of one expert per tile
constexpr int kMaxNT = kMaxTile / 8;          // n8 column tiles of the MMA
constexpr int kAccRegs = 2 * kMaxNT * 4;      // FP32 accumulators per thread: two boxes
constexpr uint32_t kRowBytes = kStageK * 2;   // one activation row of one stage
constexpr uint32_t kRedBytes = kGroupWarps * kAccRegs * 32 * 4;
constexpr int kCtrlBytes = 4096;
static_assert(kItemRing >= kMaxStages + 3, "producer could lap the item ring");

struct Ctrl {
  uint64_t full[kMaxStages];      // words landed (TMA) + rows written (kRowWarps arrivals)
  uint64_t empty[kMaxStages];     // all consumer warps
  uint64_t red_full;              // group 1 wrote its partial sums
  uint64_t red_empty;             // group 0 read them
  uint64_t item_ready[kItemRing];
  int item[kItemRing];
  int abort;
  Tables tables;
};
static_assert(sizeof(Ctrl) <= kCtrlBytes, "control block too large");

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
// L2 only: rows another SM may have written moments ago (chained down projection) must not come from a stale L1 line
__device__ __forceinline__ uint4 ldg_cg128(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// One consumer warp's share of one stage: 128 K (four 32-K chunks) of its 16 channel rows in both weight boxes,
// against kNT column tiles of 8 rows. w_base: the stage; b_base: the activation tile at this thread's row g.
template <int kNT>
__device__ __forceinline__ void multiply_half(float (&acc)[2][kMaxNT][4], uint32_t w_base, uint32_t b_base,
                                              const __nv_bfloat162 (&sc)[2][2], int group, uint32_t lm_row,
                                              uint32_t lm_chunk, int t4, int g, const w4::Consts& k4) {
  // all packed words of this stage half first: the loads overlap the arithmetic of the chunks before
  uint32_t wl[2][4], wh[2][4];
#pragma unroll
  for (int c2l = 0; c2l < 2; ++c2l) {
    const uint32_t c2 = static_cast<uint32_t>(group * 2 + c2l);
    const uint32_t lm = lm_row * 128u + (((c2 * 2u + lm_chunk) ^ (lm_row & 7u)) << 4);
    ldmatrix_x4(wl[c2l], w_base + lm);
    ldmatrix_x4(wh[c2l], w_base + kBoxBytes + lm);
  }
  const uint32_t flip = static_cast<uint32_t>(g & 1) << 2;
#pragma unroll
  for (int c2l = 0; c2l < 2; ++c2l) {
#pragma unroll
    for (int cc = 0; cc < 2; ++cc) {
      const uint32_t gidx = static_cast<uint32_t>(((group * 2 + c2l) * 2 + cc) * 4 + t4);
      const uint32_t b_off = (gidx ^ flip) << 4;
      uint4 b[kNT];
#pragma unroll
      for (int nt = 0; nt < kNT; ++nt) b[nt] = lds128(b_base + nt * 8 * kRowBytes + b_off);
      uint32_t a[2][2][4];   // [box][row g / g+8][pair]
      w4::dequant_pairs(wl[c2l][2 * cc], sc[0][0], k4, a[0][0]);
      w4::dequant_pairs(wl[c2l][2 * cc + 1], sc[0][1], k4, a[0][1]);
      w4::dequant_pairs(wh[c2l][2 * cc], sc[1][0], k4, a[1][0]);
      w4::dequant_pairs(wh[c2l][2 * cc + 1], sc[1][1], k4, a[1][1]);
#pragma unroll
      for (int nt = 0; nt < kNT; ++nt) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          mma_bf16(acc[h][nt], a[h][0][0], a[h][1][0], a[h][0][1], a[h][1][1], b[nt].x, b[nt].y);
          mma_bf16(acc[h][nt], a[h][0][2], a[h][1][2], a[h][0][3], a[h][1][3], b[nt].z, b[nt].w);
        }
      }
    }
  }
}

// act: the rows the tile multiplies ([R, k_dim] BF16, dense ragged expert segments). hi_offset: row distance of the
// second weight box (the up rows: n_out; the upper half of a 256-channel down tile: 128). tile_channels: output
// channels of one tile (128 gate/up, 256 down). chain_done / chain_need / tile_counter: as in the BF16 kernel.
// source_rows (gate/up of a gathering plan, else null): `act` is the token matrix x and grouped row r is its row
// source_rows[r] - the dispatch then copies no rows at all.
template <bool kGateUp>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_w4r_kernel(const __grid_constant__ CUtensorMap tm_words, const __nv_bfloat16* act,
                        const __nv_bfloat16* __restrict__ scales, __nv_bfloat16* __restrict__ out,
                        const int* __restrict__ g_offsets, const int* __restrict__ g_counts,
                        const int* __restrict__ g_tasks, int* __restrict__ status, int E, int n_out, int k_dim,
                        int w_rows_per_expert, int token_tile, int num_stages, int stream_weights, int hi_offset,
                        int tile_channels, int* chain_done, int chain_need, int* tile_counter,
                        const int* __restrict__ source_rows, const unsigned char* __restrict__ prefetch_base,
                        int prefetch_chunks) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  Ctrl* c = reinterpret_cast<Ctrl*>(smem_raw);
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t ring_off = ((raw_addr + kCtrlBytes + 1023u) & ~1023u) - raw_addr;
  const uint32_t stage_bytes = 2 * kBoxBytes + static_cast<uint32_t>(token_tile) * kRowBytes;
  const int groups = k_dim / 128;                                   // scales per channel row
  unsigned char* stages = smem_raw + ring_off;
  float* red = reinterpret_cast<float*>(stages + static_cast<size_t>(num_stages) * stage_bytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool chained = !kGateUp && chain_done != nullptr;
  const bool dynamic = !kGateUp && tile_counter != nullptr;
  if (!kGateUp) pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < num_stages; ++s) {
      mbar_init(&c->full[s], 1 + kRowWarps);
      mbar_init(&c->empty[s], kConsumerWarps);
    }
    mbar_init(&c->red_full, kGroupWarps);
    mbar_init(&c->red_empty, kGroupWarps);
    for (int q = 0; q < kItemRing; ++q) mbar_init(&c->item_ready[q], 1);
    c->abort = 0;
    mbar_init_fence();
  }
  // A chained down kernel can only be scheduled once every gate/up CTA has passed its own wait (gate/up lets its
  // dependents go after it), so the dispatch metadata is complete; activated rows are awaited per expert below.
  if (kGateUp) prefetch_head(prefetch_base, prefetch_chunks);   // packed words into L2 while router / dispatch run
  if (!chained) pdl_wait();
  if (kGateUp) pdl_launch_dependents();
  load_tables(&c->tables, g_tasks, g_offsets, g_counts, E);
  __syncthreads();

  const int n_ct = (n_out + tile_channels - 1) / tile_channels;
  const int num_ks = (k_dim + kStageK - 1) / kStageK;            // stages per tile
  const int total_items = c->tables.tasks[E] * n_ct;

  if (warp == 0) {
    if (lane == 0) {
      // ---------------------------------------------------------------- TMA producer: packed words and scales
      const uint64_t pol_w = stream_weights ? policy_evict_first() : policy_evict_last();
      int stage = 0;
      uint32_t phase = 0;
      long long issued = 0;
      bool ok = true;
      for (int seq = 0; ok; ++seq) {
        const int item = dynamic ? draw_item(c, tile_counter, seq, total_items)
                                 : follow_item(c, false, seq, total_items, status);
        if (item < 0) break;
        const Tile t = decode_tile(&c->tables, item, E, n_ct, token_tile);
        const int w_row = t.expert * w_rows_per_expert + t.ct * tile_channels;
        for (int s = 0; s < num_ks; ++s) {
          if (!mbar_wait(&c->empty[stage], phase ^ 1u, &c->abort, status)) { ok = false; break; }
          unsigned char* st = stages + static_cast<size_t>(stage) * stage_bytes;
          mbar_expect_tx(&c->full[stage], 2 * kBoxBytes);
          tma_load_2d(st, &tm_words, &c->full[stage], s * (kStageK / 8), w_row, pol_w);   // 32 int32 per row
          tma_load_2d(st + kBoxBytes, &tm_words, &c->full[stage], s * (kStageK / 8), w_row + hi_offset, pol_w);
          ++issued;
          if (++stage == num_stages) { stage = 0; phase ^= 1u; }
        }
      }
      const long long first = issued > num_stages ? issued - num_stages : 0;
      for (long long i = first; i < issued; ++i) {  // never leave with copies in flight (long done on the normal path)
        if (!mbar_wait_plain(&c->full[i % num_stages], static_cast<uint32_t>((i / num_stages) & 1))) {
          atomicOr(status, B200MOE_STATUS_TIMEOUT);
          break;
        }
      }
    }
  } else if (warp < kFirstConsumer) {
    // ------------------------------------------------------------------ activation rows, permuted into the stage
    const int rw = warp - 1;
    int stage = 0;
    uint32_t phase = 0;
    int ready_expert = -1;   // activated rows of this expert are known to be complete
    bool ok = true;
    for (int seq = 0; ok; ++seq) {
      int item = 0;
      if (lane == 0) item = follow_item(c, dynamic, seq, total_items, status);
      item = __shfl_sync(0xffffffffu, item, 0);
      if (item < 0) break;
      const Tile t = decode_tile(&c->tables, item, E, n_ct, token_tile);
      if (chained && t.expert != ready_expert) {
        int done = 1;
        if (lane == 0) {
          const int need = chain_need * (c->tables.tasks[t.expert + 1] - c->tables.tasks[t.expert]);
          done = wait_expert_done(chain_done + t.expert, need, &c->abort, status) ? 1 : 0;
        }
        done = __shfl_sync(0xffffffffu, done, 0);
        if (!done) break;
        ready_expert = t.expert;
      }
      const int n_pad = (t.rows + 7) & ~7;                 // rows of the n8 column tiles in use
      const int items = n_pad * (kStageK / 8);             // 16-byte groups of one stage
      int src_row[kMaxTile / 2];                           // the row of `act` behind each of this lane's groups
#pragma unroll
      for (int j = 0; j < kMaxTile / 2; ++j) {
        const int n = (j * kRowWarps + rw), r = t.row0 + min(n, t.rows - 1);
        src_row[j] = (n < n_pad && source_rows != nullptr) ? source_rows[r] : r;
      }
      for (int s = 0; s < num_ks; ++s) {
        int free_ok = 1;
        if (lane == 0) free_ok = mbar_wait(&c->empty[stage], phase ^ 1u, &c->abort, status) ? 1 : 0;
        free_ok = __shfl_sync(0xffffffffu, free_ok, 0);
        if (!free_ok) { ok = false; break; }
        const uint32_t b_base = smem_u32(stages + static_cast<size_t>(stage) * stage_bytes) + 2 * kBoxBytes;
        uint4 v[kMaxTile / 2];
#pragma unroll
        for (int j = 0; j < kMaxTile / 2; ++j) {           // loads first: one L2 latency for the whole stage
          const int i = (j * kRowWarps + rw) * 32 + lane;
          const int k = s * kStageK + (i & 31) * 8;
          if (i < items && k < k_dim)
            v[j] = ldg_cg128(act + static_cast<size_t>(src_row[j]) * k_dim + k);
        }
#pragma unroll
        for (int j = 0; j < kMaxTile / 2; ++j) {
          const int i = (j * kRowWarps + rw) * 32 + lane;
          const int n = i >> 5, gidx = i & 31, k = s * kStageK + gidx * 8;
          if (i < items && k < k_dim) {
            // k0 k1 | k2 k3 | k4 k5 | k6 k7  ->  k0 k4 | k1 k5 | k2 k6 | k3 k7
            const uint32_t o0 = __byte_perm(v[j].x, v[j].z, 0x5410), o1 = __byte_perm(v[j].x, v[j].z, 0x7632);
            const uint32_t o2 = __byte_perm(v[j].y, v[j].w, 0x5410), o3 = __byte_perm(v[j].y, v[j].w, 0x7632);
            const uint32_t dst = b_base + n * kRowBytes + ((gidx ^ ((n & 1) << 2)) << 4);
            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst), "r"(o0), "r"(o1), "r"(o2), "r"(o3) : "memory");
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&c->full[stage]);
        if (++stage == num_stages) { stage = 0; phase ^= 1u; }
      }
    }
  } else {
    // ------------------------------------------------------------------ consumers: dequantise in registers, multiply
    const int cw = warp - kFirstConsumer;
    const int group = cw / kGroupWarps, blk = cw % kGroupWarps;
    const int g = lane >> 2, t4 = lane & 3;
    int stage = 0;
    uint32_t phase = 0;
    const long long total_rows = static_cast<long long>(E) * w_rows_per_expert;
    // ldmatrix: lane l addresses row (l & 7) of matrix (l >> 3): matrices = rows 0-7 / 8-15 of this warp's 16 rows,
    // for two consecutive 16-byte chunks (32 K each) of the 128-byte row
    const uint32_t lm_row = static_cast<uint32_t>(blk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7));
    const uint32_t lm_chunk = static_cast<uint32_t>(lane >> 4);
    const w4::Consts k4 = w4::make_consts();
    bool ok = true;
    for (int seq = 0; ok; ++seq) {
      const int item = follow_item(c, dynamic, seq, total_items, status);
      if (__any_sync(0xffffffffu, item < 0)) break;
      const Tile t = decode_tile(&c->tables, item, E, n_ct, token_tile);
      const int n_tiles = (t.rows + 7) >> 3;
      float acc[2][kMaxNT][4];
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int nt = 0; nt < kMaxNT; ++nt)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[h][nt][j] = 0.0f;
      // scales of this thread's four channel rows ([box][row g / g+8]); rows past the last channel are never stored
      const __nv_bfloat16* sc_ptr[2][2];
      {
        const long long row = static_cast<long long>(t.expert) * w_rows_per_expert + t.ct * tile_channels + blk * 16 + g;
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int r = 0; r < 2; ++r)
            sc_ptr[h][r] = scales + min(row + h * hi_offset + r * 8, total_rows - 1) * groups + group;
      }
      __nv_bfloat16 sc_next[2][2];
      if (group * 128 < k_dim) {
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int r = 0; r < 2; ++r) sc_next[h][r] = __ldg(sc_ptr[h][r]);
      }
      for (int s = 0; s < num_ks; ++s) {
        {
          const int k_left = k_dim - s * kStageK - group * 128;   // K this group still has in this stage
          __nv_bfloat162 sc[2][2];   // the 128-K scale group of this stage half
#pragma unroll
          for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int r = 0; r < 2; ++r) sc[h][r] = __bfloat162bfloat162(sc_next[h][r]);
          if (k_left > kStageK) {   // the next stage's scales while this one is multiplied
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
              for (int r = 0; r < 2; ++r) sc_next[h][r] = __ldg(sc_ptr[h][r] + (s + 1) * 2);
          }
          if (!__all_sync(0xffffffffu, mbar_wait(&c->full[stage], phase, &c->abort, status))) { ok = false; break; }
          const uint32_t w_base = smem_u32(stages + static_cast<size_t>(stage) * stage_bytes);
          const uint32_t b_base = w_base + 2 * kBoxBytes + static_cast<uint32_t>(g) * kRowBytes;
          if (k_left > 0) {   // K is a multiple of 128: a stage half is whole or absent
            if (n_tiles == 1) multiply_half<1>(acc, w_base, b_base, sc, group, lm_row, lm_chunk, t4, g, k4);
            else multiply_half<2>(acc, w_base, b_base, sc, group, lm_row, lm_chunk, t4, g, k4);
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(&c->empty[stage]);
        }
        if (++stage == num_stages) { stage = 0; phase ^= 1u; }
      }
      if (!ok) break;
      // ---- the two groups' partial sums: group 1 hands its accumulators over, group 0 adds them and stores
      float* rbuf = red + static_cast<size_t>(blk) * kAccRegs * 32 + lane;
      const uint32_t rph = static_cast<uint32_t>(seq & 1);
      if (group == 1) {
        if (!__all_sync(0xffffffffu, mbar_wait(&c->red_empty, rph ^ 1u, &c->abort, status))) break;
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int nt = 0; nt < kMaxNT; ++nt)
#pragma unroll
            for (int j = 0; j < 4; ++j) rbuf[((h * kMaxNT + nt) * 4 + j) * 32] = acc[h][nt][j];
        __syncwarp();
        if (lane == 0) mbar_arrive(&c->red_full);
        continue;
      }
      if (!__all_sync(0xffffffffu, mbar_wait(&c->red_full, rph, &c->abort, status))) break;
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int nt = 0; nt < kMaxNT; ++nt)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[h][nt][j] = __fadd_rn(acc[h][nt][j], rbuf[((h * kMaxNT + nt) * 4 + j) * 32]);
      __syncwarp();
      if (lane == 0) mbar_arrive(&c->red_empty);
      // ---- epilogue: accumulator j of column tile nt is D[channel g (+8 for j >= 2)][row nt*8 + 2*t4 + (j & 1)]
      const int ch = t.ct * tile_channels + blk * 16 + g;
#pragma unroll
      for (int nt = 0; nt < kMaxNT; ++nt) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int n = nt * 8 + 2 * t4 + (j & 1);
          const int channel = ch + (j >> 1) * 8;
          if (nt < n_tiles && n < t.rows) {
            __nv_bfloat16* dst = out + static_cast<size_t>(t.row0 + n) * n_out;
            if (kGateUp) {
              const float v = acc[0][nt][j];
              if (channel < n_out) dst[channel] = __float2bfloat16_rn((v / (1.0f + __expf(-v))) * acc[1][nt][j]);
            } else {
              if (channel < n_out) dst[channel] = __float2bfloat16_rn(acc[0][nt][j]);
              if (channel + 128 < n_out) dst[channel + 128] = __float2bfloat16_rn(acc[1][nt][j]);
            }
          }
        }
      }
      if (kGateUp && chain_done != nullptr) {
        __threadfence();   // this lane's rows visible GPU-wide before the counter moves
        __syncwarp();
        if (lane == 0) atomicAdd(chain_done + t.expert, 1);
      }
    }
  }
  __syncthreads();
}

void ring_for(bool gate_up, int token_tile, int hidden, int inter, int* stages, int* smem_bytes) {
  const int k_dim = gate_up ? hidden : inter;
  const int stage = 2 * static_cast<int>(kBoxBytes) + token_tile * static_cast<int>(kRowBytes);
  (void)k_dim;
  const int fixed = kCtrlBytes + 1024 + static_cast<int>(kRedBytes);
  int s = (kSmemLimit - fixed) / stage;
  if (s > kMaxStages) s = kMaxStages;
  *stages = s;
  *smem_bytes = fixed + s * stage;
}

template <bool kGateUp>
cudaError_t launch_w4r(const B200MoePlan& p, cudaStream_t s, bool chained) {
  const auto& sh = p.shape;
  const int n_out = kGateUp ? sh.intermediate : sh.hidden;
  const int k_dim = kGateUp ? sh.hidden : sh.intermediate;
  const int tile_channels = kGateUp ? 128 : 256;
  const int n_ct = (n_out + tile_channels - 1) / tile_channels;
  const long long bound = (static_cast<long long>((p.routes + p.token_tile - 1) / p.token_tile) + sh.experts - 1) * n_ct;
  const int grid = static_cast<int>(bound < p.num_sms ? bound : p.num_sms);
  const int stream_weights = static_cast<long long>(p.routes) <= static_cast<long long>(sh.experts) * p.token_tile;
  launch_pdl(grouped_gemm_w4r_kernel<kGateUp>, dim3(grid), dim3(kThreads),
             static_cast<size_t>(kGateUp ? p.w4r_smem_gate_up : p.w4r_smem_down), s,
      kGateUp ? p.tm_gate_up_w : p.tm_down_w,
      static_cast<const __nv_bfloat16*>(kGateUp ? (p.gather ? p.buf.x : p.buf.grouped_input) : p.buf.activated),
      static_cast<const __nv_bfloat16*>(kGateUp ? p.buf.gate_up_scales : p.buf.down_scales),
      static_cast<__nv_bfloat16*>(kGateUp ? p.buf.activated : p.buf.down_output),
      static_cast<const int*>(p.buf.offsets), static_cast<const int*>(p.buf.counts),
      static_cast<const int*>(p.buf.tasks), static_cast<int*>(p.buf.status), sh.experts, n_out, k_dim,
      kGateUp ? 2 * sh.intermediate : sh.hidden, p.token_tile, kGateUp ? p.w4r_stages_gate_up : p.w4r_stages_down,
      stream_weights, kGateUp ? sh.intermediate : 128, tile_channels,
      chained ? static_cast<int*>(p.buf.scratch) + router_flag_index(p) + 2 : static_cast<int*>(nullptr),
      kGroupWarps * ((sh.intermediate + 127) / 128),  // storing warps x gate/up channel tiles per token tile
      chained && !kGateUp ? static_cast<int*>(p.buf.scratch) + router_flag_index(p) + 1 : static_cast<int*>(nullptr),
      kGateUp && p.gather ? static_cast<const int*>(p.buf.source_rows) : static_cast<const int*>(nullptr),
      kGateUp ? static_cast<const unsigned char*>(p.buf.gate_up) : static_cast<const unsigned char*>(nullptr),
      kGateUp ? prefetch_head_chunks(static_cast<long long>(sh.experts) * 2 * sh.intermediate * sh.hidden / 2) : 0);
  return cudaPeekAtLastError();
}

}  // namespace

bool w4r_serves(const B200MoePlan& p) { return p.token_tile <= kMaxTile; }

int configure_w4r(B200MoePlan& p) {
  ring_for(true, p.token_tile, p.shape.hidden, p.shape.intermediate, &p.w4r_stages_gate_up, &p.w4r_smem_gate_up);
  ring_for(false, p.token_tile, p.shape.hidden, p.shape.intermediate, &p.w4r_stages_down, &p.w4r_smem_down);
  if (p.w4r_stages_gate_up < 2 || p.w4r_stages_down < 2) {
    set_error("W4 weight-streaming kernel: K = %d / %d leaves fewer than 2 stages", p.shape.hidden, p.shape.intermediate);
    return B200MOE_ERR_UNSUPPORTED;
  }
  for (const void* ptr : {p.buf.gate_up_scales, p.buf.down_scales})
    if (ptr && reinterpret_cast<uintptr_t>(ptr) % 16) {
      set_error("W4G128 scales must be 16-byte aligned");
      return B200MOE_ERR_INVALID;
    }
  cudaError_t e = cudaFuncSetAttribute(grouped_gemm_w4r_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(grouped_gemm_w4r_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
  if (e != cudaSuccess) {
    set_error("cudaFuncSetAttribute(W4 shared memory) failed: %s", cudaGetErrorString(e));
    return B200MOE_ERR_CUDA;
  }
  return B200MOE_OK;
}

cudaError_t launch_gate_up_w4r(const B200MoePlan& p, cudaStream_t s, bool chained) { return launch_w4r<true>(p, s, chained); }
cudaError_t launch_down_w4r(const B200MoePlan& p, cudaStream_t s, bool chained) { return launch_w4r<false>(p, s, chained); }

}  // namespace b200moe
