// W4A16 ragged grouped GEMM: packed int4 weights (the reference's W4G128 v1
// format) are TMA-loaded to shared memory as stored, dequantised to BF16 by
// converter warps straight into the 128-byte-swizzled operand tile, and
// multiplied on tcgen05 with the accumulators in tensor memory.
//
// Format contract (reference moe_weight_quant.py:1-6,35-52 and the device decode
// of cuda_w4_gate_up.cu:28-41): words[e][n][kw] holds K = 8*kw .. 8*kw+7, nibble j
// at bits [4j,4j+4), nibble = q + 8 with q in [-7,7]; one BF16 scale per
// (expert, output channel, 128 consecutive K); the operand fed to the MMA is
// exactly bf16_rn(float(q) * float(scale)). Here: (w >> 4j) & 0x000F000F | 0x43004300
// gives the BF16 pair {128 + n_j, 128 + n_(j+4)}, minus 136 is the exact integer
// q, and one BF16 multiply by the scale rounds once - the same value.
// The reference quantises gate/up only; the same format with K = I serves down.
//
// Schedule: as grouped_gemm_tcgen05.cu (swap-AB, per-tile N, persistent,
// device-side tile list) plus eight converter warps, a second TMA warp and two rings:
//  * words ring  - packed tiles of 128 channels x 256 K (one 128-byte row of words per
//    channel, 128B-swizzled by TMA so the converters' 16-byte reads are conflict-free).
//    Whole 128-byte rows matter: 32-byte rows (64 K per box) fetch HBM in 32-byte sectors
//    and ran at a quarter of the bandwidth.
//  * operand ring - per 64 K: the BF16 weight tile(s) written by the converters plus the
//    activation rows written by the second TMA warp; consumed by the MMA warp.
// Sixteen converter warps (four per scheduler) hide the shared-memory and BF16-ALU latency of
// the dequantisation; each thread converts four (gate/up) or two (down) words per 64 K.
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

constexpr int kConverters = 512;                       // 16 warps (warps 6..21)
constexpr int kThreads = 192 + kConverters + 64;       // + words TMA, MMA, 4 epilogue, activation TMA, second MMA warp
// Two MMA-issuing threads with an accumulator each (one thread issues a tcgen05.mma only about every 100 cycles):
// the gate and the up tile, or for down the even and the odd K steps, summed in the epilogue.
constexpr int kMmaWarpB = 6 + kConverters / 32 + 1;
constexpr int kMaxWords = 6, kMaxOperand = 4;
constexpr int kWordsK = 256;                           // K covered by one words stage: 128 bytes per channel
constexpr uint32_t kWTileBytes = kTileM * kBlockK * 2;   // one BF16 weight tile of 64 K: 16 KB
constexpr uint32_t kWordsTileBytes = kTileM * kWordsK / 2;  // one packed tile of 256 K: 16 KB
constexpr int kCtrlBytes = 4096;

struct Ctrl {
  uint64_t words_full[kMaxWords];
  uint64_t words_empty[kMaxWords];
  uint64_t op_full[kMaxOperand];
  uint64_t op_empty[kMaxOperand];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t drain[2];
  uint64_t item_ready[kItemRing];
  int item[kItemRing];
  uint32_t tmem_base;
  int abort;
  Tables tables;
};
static_assert(sizeof(Ctrl) <= kCtrlBytes, "control block too large");

template <bool kGateUp>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_w4_kernel(const __grid_constant__ CUtensorMap tm_words, const __grid_constant__ CUtensorMap tm_act,
                       const __nv_bfloat16* __restrict__ scales, __nv_bfloat16* __restrict__ out,
                       const int* __restrict__ g_offsets, const int* __restrict__ g_counts,
                       const int* __restrict__ g_tasks, int* __restrict__ status, int E, int n_out, int k_dim,
                       int w_rows_per_expert, int token_tile, int num_words, int num_operand, int stream_weights,
                       int* chain_done, int chain_need, int* tile_counter) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  Ctrl* c = reinterpret_cast<Ctrl*>(smem_raw);
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t ring_off = ((raw_addr + kCtrlBytes + 1023u) & ~1023u) - raw_addr;
  constexpr uint32_t kOpWeightBytes = kGateUp ? 2 * kWTileBytes : kWTileBytes;
  constexpr uint32_t kWordsBytes = kGateUp ? 2 * kWordsTileBytes : kWordsTileBytes;  // words stage
  const uint32_t act_bytes = static_cast<uint32_t>(token_tile) * 128u;
  const uint32_t op_bytes = kOpWeightBytes + act_bytes;                               // operand stage
  unsigned char* op_ring = smem_raw + ring_off;
  unsigned char* words_ring = op_ring + static_cast<size_t>(num_operand) * op_bytes;
  const int acc_cols = 2 * token_tile;   // gate and up, or the two partial sums of down
  const int num_acc = (2 * acc_cols <= 512) ? 2 : 1;
  uint32_t tmem_cols = 32;
  while (tmem_cols < static_cast<uint32_t>(num_acc * acc_cols)) tmem_cols <<= 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // chain_done / chain_need / tile_counter: the gate/up and down kernels of one forward chained through per-expert
  // completion counters and a dynamic tile order for down, as in the BF16 kernel (grouped_gemm_tcgen05.cu)
  const bool chained = !kGateUp && chain_done != nullptr;
  const bool dynamic = !kGateUp && tile_counter != nullptr;
  if (!kGateUp) pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < num_words; ++s) {
      mbar_init(&c->words_full[s], 1);
      mbar_init(&c->words_empty[s], kConverters / 32);   // one arrival per converter warp
    }
    for (int s = 0; s < num_operand; ++s) {
      mbar_init(&c->op_full[s], kConverters / 32 + 1);   // converter warps + the activation TMA
      mbar_init(&c->op_empty[s], 2);                     // the commits of the two MMA issuers
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&c->tmem_full[a], 2);  // the two MMA issuers
      mbar_init(&c->tmem_empty[a], 4);  // one arrival per epilogue warp
    }
    mbar_init(&c->drain[0], 1);
    mbar_init(&c->drain[1], 1);
    for (int q = 0; q < kItemRing; ++q) mbar_init(&c->item_ready[q], 1);
    c->abort = 0;
    mbar_init_fence();
  }
  if (warp == 1) tmem_alloc(&c->tmem_base, tmem_cols);
  if (!chained) pdl_wait();   // a chained down kernel waits per expert instead (below)
  if (kGateUp) pdl_launch_dependents();   // after the wait: a dependent then knows the dispatch metadata is complete
  load_tables(&c->tables, g_tasks, g_offsets, g_counts, E);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&c->tmem_base);

  const int n_ct = (n_out + kTileM - 1) / kTileM;
  const int num_kb = k_dim / kBlockK;                       // K is a multiple of 128
  const int num_ws = (k_dim + kWordsK - 1) / kWordsK;       // words stages per tile
  const int groups = k_dim / 128;
  const int total_items = c->tables.tasks[E] * n_ct;

  if (warp == 0) {
    if (lane == 0) {
      // ---------------------------------------------------------------- TMA producer: packed words
      const uint64_t pol_w = stream_weights ? policy_evict_first() : policy_evict_last();
      int p = 0;
      uint32_t pph = 0;
      long long issued = 0;
      bool ok = true;
      for (int seq = 0; ok; ++seq) {
        const int item = dynamic ? draw_item(c, tile_counter, seq, total_items)
                                 : follow_item(c, false, seq, total_items, status);
        if (item < 0) break;
        const Tile t = decode_tile(&c->tables, item, E, n_ct, token_tile);
        const int w_row = t.expert * w_rows_per_expert + t.ct * kTileM;
        for (int ws = 0; ws < num_ws; ++ws) {
          if (!mbar_wait(&c->words_empty[p], pph ^ 1u, &c->abort, status)) { ok = false; break; }
          unsigned char* st = words_ring + static_cast<size_t>(p) * kWordsBytes;
          mbar_expect_tx(&c->words_full[p], kWordsBytes);
          tma_load_2d(st, &tm_words, &c->words_full[p], ws * (kWordsK / 8), w_row, pol_w);  // 32 int32 per row
          if (kGateUp)
            tma_load_2d(st + kWordsTileBytes, &tm_words, &c->words_full[p], ws * (kWordsK / 8), w_row + n_out, pol_w);
          ++issued;
          if (++p == num_words) { p = 0; pph ^= 1u; }
        }
      }
      const long long first = issued > num_words ? issued - num_words : 0;
      for (long long i = first; i < issued; ++i) {  // never leave with copies in flight
        if (!mbar_wait_plain(&c->words_full[i % num_words], static_cast<uint32_t>((i / num_words) & 1))) {
          atomicOr(status, B200MOE_STATUS_TIMEOUT);
          break;
        }
      }
    }
  } else if (warp == 6 + kConverters / 32) {
    if (lane == 0) {
      // ---------------------------------------------------------------- TMA producer: activation rows
      const uint64_t pol_act = policy_evict_last();
      int q = 0;
      uint32_t qph = 0;
      long long issued = 0;
      bool ok = true;
      int ready_expert = -1;   // activated rows of this expert are known to be complete
      for (int seq = 0; ok; ++seq) {
        const int item = follow_item(c, dynamic, seq, total_items, status);
        if (item < 0) break;
        const Tile t = decode_tile(&c->tables, item, E, n_ct, token_tile);
        if (chained && t.expert != ready_expert) {
          const int need = chain_need * (c->tables.tasks[t.expert + 1] - c->tables.tasks[t.expert]);
          if (!wait_expert_done(chain_done + t.expert, need, &c->abort, status)) { ok = false; break; }
          ready_expert = t.expert;
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&c->op_empty[q], qph ^ 1u, &c->abort, status)) { ok = false; break; }
          mbar_expect_tx(&c->op_full[q], act_bytes);
          tma_load_2d(op_ring + static_cast<size_t>(q) * op_bytes + kOpWeightBytes, &tm_act, &c->op_full[q],
                      kb * kBlockK, t.row0, pol_act);
          ++issued;
          if (++q == num_operand) { q = 0; qph ^= 1u; }
        }
      }
      const long long first = issued > num_operand ? issued - num_operand : 0;
      for (long long i = first; i < issued; ++i) {  // completes once the converters arrived too; bounded
        if (!mbar_wait_plain(&c->op_full[i % num_operand], static_cast<uint32_t>((i / num_operand) & 1))) break;
      }
    }
  } else if (warp == 1 || warp == kMmaWarpB) {
    if (lane == 0) {
      // ---------------------------------------------------------------- MMA issuers (0: gate / even K, 1: up / odd K)
      const int half = warp == 1 ? 0 : 1;
      int q = 0, acc = 0;
      uint32_t qph = 0, acc_phase = 0;
      bool ok = true;
      for (int seq = 0; ok; ++seq) {
        const int item = follow_item(c, dynamic, seq, total_items, status);
        if (item < 0) { ok = !*reinterpret_cast<volatile int*>(&c->abort); break; }
        const Tile t = decode_tile(&c->tables, item, E, n_ct, token_tile);
        const uint32_t idesc = umma_idesc(kTileM, t.n_eff);
        if (!mbar_wait(&c->tmem_empty[acc], acc_phase ^ 1u, &c->abort, status)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_gate = tmem_base + static_cast<uint32_t>(acc * acc_cols);
        const uint32_t d_up = d_gate + static_cast<uint32_t>(token_tile);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&c->op_full[q], qph, &c->abort, status)) { ok = false; break; }
          tc_fence_after();
          const uint32_t w_addr = smem_u32(op_ring + static_cast<size_t>(q) * op_bytes);
          const uint32_t w_lo = umma_desc_lo(w_addr), a_lo = umma_desc_lo(w_addr + kOpWeightBytes);
#pragma unroll
          for (int k = 0; k < kBlockK / kUmmaK; ++k) {  // a K step of 16 BF16 = 32 bytes = 2 in descriptor units
            if (kGateUp) {
              umma_lo(half ? d_up : d_gate, w_lo + half * (kWTileBytes >> 4) + 2 * k, a_lo + 2 * k, idesc,
                      (kb | k) != 0 ? 1u : 0u);
            } else if ((k & 1) == half) {
              umma_lo(half ? d_up : d_gate, w_lo + 2 * k, a_lo + 2 * k, idesc, (kb | (k >> 1)) != 0 ? 1u : 0u);
            }
          }
          umma_commit(&c->op_empty[q]);
          if (++q == num_operand) { q = 0; qph ^= 1u; }
        }
        if (!ok) break;
        umma_commit(&c->tmem_full[acc]);
        if (++acc == num_acc) { acc = 0; acc_phase ^= 1u; }
      }
      if (!ok) {
        umma_commit(&c->drain[half]);
        mbar_wait_plain(&c->drain[half], 0);
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------------ epilogue warps
    const int quarter = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int seq = 0;; ++seq) {
      const int item = follow_item(c, dynamic, seq, total_items, status);
      if (__any_sync(0xffffffffu, item < 0)) break;   // warp-uniform: the TMEM loads below need the whole warp
      const Tile t = decode_tile(&c->tables, item, E, n_ct, token_tile);
      if (!__all_sync(0xffffffffu, mbar_wait(&c->tmem_full[acc], acc_phase, &c->abort, status))) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + static_cast<uint32_t>(acc * acc_cols) + (static_cast<uint32_t>(quarter * 32) << 16);
      store_tile<kGateUp, !kGateUp>(t, taddr, token_tile, t.ct * kTileM + quarter * 32 + lane, n_out, out);
      tc_fence_before();
      if (kGateUp && chain_done != nullptr) {
        // this lane's rows: ordered for the async proxy (the down kernel reads them by TMA), then visible GPU-wide
        asm volatile("fence.proxy.async;" ::: "memory");
        __threadfence();
      }
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&c->tmem_empty[acc]);
        if (kGateUp && chain_done != nullptr) atomicAdd(chain_done + t.expert, 1);
      }
      if (++acc == num_acc) { acc = 0; acc_phase ^= 1u; }
    }
  } else {
    // ------------------------------------------------------------------ converter warps (6..13)
    const int tid = threadIdx.x - 192;
    const int row = tid & 127, part = tid >> 7;   // four threads per channel row
    // gate/up: part&1 picks the gate or up tile, part>>1 the 16-byte half of the row's 32 bytes per 64 K
    //          (four words each); down: part picks a quarter of the row's 32 bytes (two words each).
    const int half = kGateUp ? (part & 1) : 0;
    const w4::Consts k4 = w4::make_consts();
    const long long total_rows = static_cast<long long>(E) * w_rows_per_expert;
    int p = 0, q = 0;
    uint32_t pph = 0, qph = 0;
    bool ok = true;
    for (int seq = 0; ok; ++seq) {
      const int item = follow_item(c, dynamic, seq, total_items, status);
      if (__any_sync(0xffffffffu, item < 0)) break;
      const Tile t = decode_tile(&c->tables, item, E, n_ct, token_tile);
      long long srow = static_cast<long long>(t.expert) * w_rows_per_expert + t.ct * kTileM + row +
                       (kGateUp ? half * n_out : 0);
      if (srow >= total_rows) srow = total_rows - 1;  // lanes past the last channel are never stored
      const __nv_bfloat16* srow_ptr = scales + srow * groups;
      __nv_bfloat16 s0 = srow_ptr[0], s1 = srow_ptr[groups > 1 ? 1 : 0];   // the two groups of words stage 0
      for (int ws = 0; ok && ws < num_ws; ++ws) {
        const __nv_bfloat162 scale_lo = __bfloat162bfloat162(s0), scale_hi = __bfloat162bfloat162(s1);
        if (ws + 1 < num_ws) {  // prefetch the next stage's scales while this one is converted
          s0 = srow_ptr[2 * ws + 2];
          s1 = srow_ptr[min(2 * ws + 3, groups - 1)];
        }
        if (!__all_sync(0xffffffffu, mbar_wait(&c->words_full[p], pph, &c->abort, status))) { ok = false; break; }
        const unsigned char* words = words_ring + static_cast<size_t>(p) * kWordsBytes +
                                     (kGateUp ? half * kWordsTileBytes : 0) + row * 128;
        const int subs = min(kWordsK, k_dim - ws * kWordsK) / kBlockK;
        for (int j = 0; j < subs; ++j) {
          if (!__all_sync(0xffffffffu, mbar_wait(&c->op_empty[q], qph ^ 1u, &c->abort, status))) { ok = false; break; }
          const __nv_bfloat162 scale2 = j < 2 ? scale_lo : scale_hi;
          unsigned char* dst = op_ring + static_cast<size_t>(q) * op_bytes + row * 128;
          if (kGateUp) {
            dst += half * kWTileBytes;
            const int ch = part >> 1;
            const uint4 w0 = *reinterpret_cast<const uint4*>(words + (((2 * j + ch) ^ (row & 7)) << 4));
            const uint32_t w[4] = {w0.x, w0.y, w0.z, w0.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
              *reinterpret_cast<uint4*>(dst + (((ch * 4 + i) ^ (row & 7)) << 4)) = w4::dequant_word(w[i], scale2, k4);
          } else {
            const uint2 w0 = *reinterpret_cast<const uint2*>(words + (((2 * j + (part >> 1)) ^ (row & 7)) << 4) +
                                                             (part & 1) * 8);
            *reinterpret_cast<uint4*>(dst + (((part * 2) ^ (row & 7)) << 4)) = w4::dequant_word(w0.x, scale2, k4);
            *reinterpret_cast<uint4*>(dst + (((part * 2 + 1) ^ (row & 7)) << 4)) = w4::dequant_word(w0.y, scale2, k4);
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy stores -> tensor-core reads
          __syncwarp();
          if (lane == 0) mbar_arrive(&c->op_full[q]);  // one arrival per warp
          if (++q == num_operand) { q = 0; qph ^= 1u; }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&c->words_empty[p]);
        if (++p == num_words) { p = 0; pph ^= 1u; }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, tmem_cols);
  }
}

void rings_for(bool gate_up, int token_tile, int* num_words, int* num_operand, int* smem_bytes) {
  const int op = (gate_up ? 2 : 1) * static_cast<int>(kWTileBytes) + token_tile * 128;
  const int words = (gate_up ? 2 : 1) * static_cast<int>(kWordsTileBytes);
  const int budget = kSmemLimit - kCtrlBytes - 1024;
  int q = 3;
  while (q > 2 && budget - q * op < 2 * words) --q;
  int p = (budget - q * op) / words;
  if (p > kMaxWords) {  // spare room goes to the operand ring
    p = kMaxWords;
    while (q < kMaxOperand && budget - (q + 1) * op >= p * words) ++q;
  }
  *num_words = p;
  *num_operand = q;
  *smem_bytes = kCtrlBytes + 1024 + q * op + p * words;
}

template <bool kGateUp>
cudaError_t launch_w4(const B200MoePlan& p, cudaStream_t s, bool chained) {
  const auto& sh = p.shape;
  const int n_out = kGateUp ? sh.intermediate : sh.hidden;
  const int k_dim = kGateUp ? sh.hidden : sh.intermediate;
  const int n_ct = (n_out + kTileM - 1) / kTileM;
  const long long bound = (static_cast<long long>((p.routes + p.token_tile - 1) / p.token_tile) + sh.experts - 1) * n_ct;
  const int grid = static_cast<int>(bound < p.num_sms ? bound : p.num_sms);
  const int stream_weights = static_cast<long long>(p.routes) <= static_cast<long long>(sh.experts) * p.token_tile;
  launch_pdl(grouped_gemm_w4_kernel<kGateUp>, dim3(grid), dim3(kThreads),
             static_cast<size_t>(kGateUp ? p.w4_smem_gate_up : p.w4_smem_down), s,
      kGateUp ? p.tm_gate_up_w : p.tm_down_w, kGateUp ? p.tm_grouped : p.tm_activated,
      static_cast<const __nv_bfloat16*>(kGateUp ? p.buf.gate_up_scales : p.buf.down_scales),
      static_cast<__nv_bfloat16*>(kGateUp ? p.buf.activated : p.buf.down_output),
      static_cast<const int*>(p.buf.offsets), static_cast<const int*>(p.buf.counts),
      static_cast<const int*>(p.buf.tasks), static_cast<int*>(p.buf.status), sh.experts, n_out, k_dim,
      kGateUp ? 2 * sh.intermediate : sh.hidden, p.token_tile, kGateUp ? p.w4_packed_gate_up : p.w4_packed_down,
      kGateUp ? p.w4_operand_gate_up : p.w4_operand_down, stream_weights,
      chained ? static_cast<int*>(p.buf.scratch) + router_flag_index(p) + 2 : static_cast<int*>(nullptr),
      4 * ((sh.intermediate + kTileM - 1) / kTileM),  // epilogue warps x gate/up channel tiles per token tile
      chained && !kGateUp ? static_cast<int*>(p.buf.scratch) + router_flag_index(p) + 1 : static_cast<int*>(nullptr));
  return cudaPeekAtLastError();
}

}  // namespace

int configure_w4(B200MoePlan& p) {
  rings_for(true, p.token_tile, &p.w4_packed_gate_up, &p.w4_operand_gate_up, &p.w4_smem_gate_up);
  rings_for(false, p.token_tile, &p.w4_packed_down, &p.w4_operand_down, &p.w4_smem_down);
  if (p.w4_packed_gate_up < 2 || p.w4_packed_down < 2) {
    set_error("token_tile %d leaves fewer than 2 stages of packed words", p.token_tile);
    return B200MOE_ERR_INVALID;
  }
  cudaError_t e = cudaFuncSetAttribute(grouped_gemm_w4_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       kSmemLimit);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(grouped_gemm_w4_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
  if (e != cudaSuccess) {
    set_error("cudaFuncSetAttribute(W4 shared memory) failed: %s", cudaGetErrorString(e));
    return B200MOE_ERR_CUDA;
  }
  return B200MOE_OK;
}

cudaError_t launch_gate_up_w4(const B200MoePlan& p, cudaStream_t s, bool chained) { return launch_w4<true>(p, s, chained); }
cudaError_t launch_down_w4(const B200MoePlan& p, cudaStream_t s, bool chained) { return launch_w4<false>(p, s, chained); }

}  // namespace b200moe
