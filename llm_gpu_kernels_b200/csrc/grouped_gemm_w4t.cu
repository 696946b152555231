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
// This file: the dequantised weight tile never touches shared memory. The converter warps write it
// with tcgen05.st into tensor memory (channel on the lane, 128 K = 64 packed columns per tile) and the MMA
// takes its A operand from there; shared memory only carries the packed words (TMA, 128-byte rows) and the
// activation rows. That removes the 32 KB store + 36 KB operand fetch per 64 K that made the
// shared-memory-operand variant (grouped_gemm_w4.cu, used from token tile 128 up, where the accumulators
// leave no room for two sets plus operand stages in tensor memory) heavy on shared-memory bandwidth.
// Converter warp w may only touch TMEM lanes 32*(w%4)..+31, so the four warps of a lane quarter share those
// 32 channel rows by K: warp `part` converts sub-block `part` (64 K) of every 256-K words stage. An operand
// stage is 128 K (64 TMEM columns per weight tile, two 64-K row tiles in shared memory): the kernel is bound
// by the chain "stage free -> rows fetched / words converted -> 16 MMAs -> completion -> stage free", not by
// HBM (4x fewer bytes than BF16) or by any one pipe, so fewer, larger stages are faster. Measured with work
// removed selectively (Qwen shape, 17 tokens, gate/up, 64-K stages): 98 us as is, 92 without the
// dequantisation, 69 without the MMAs, 51 with neither; 128-K stages: 86 us.
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
// One thread issues a small-N tcgen05.mma about every 100 cycles whatever else the SM does (measured); two threads
// in different warps issue in parallel. So the MMAs of a stage are split between two issuers with an accumulator
// each: gate and up tiles (gate/up), even and odd K steps (down; the epilogue adds the two partial sums).
constexpr int kMmaWarpB = 6 + kConverters / 32 + 1;
constexpr int kMaxWords = 6, kMaxOperand = 4;
constexpr int kWordsK = 256;                           // K covered by one words stage: 128 bytes per channel
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

// chain_done / chain_need / tile_counter: as in the BF16 kernel (grouped_gemm_tcgen05.cu). The gate/up kernel adds
// one to chain_done[expert] per epilogue warp and tile; the down kernel, launched as a programmatic dependent, does
// not wait for the gate/up grid but, per expert, for chain_need arrivals per token tile before it loads activated
// rows, and draws its tiles from *tile_counter. Null pointers = stages separated by a kernel boundary.
template <bool kGateUp>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_w4t_kernel(const __grid_constant__ CUtensorMap tm_words, const __grid_constant__ CUtensorMap tm_act,
                       const __nv_bfloat16* __restrict__ scales, __nv_bfloat16* __restrict__ out,
                       const int* __restrict__ g_offsets, const int* __restrict__ g_counts,
                       const int* __restrict__ g_tasks, int* __restrict__ status, int E, int n_out, int k_dim,
                       int w_rows_per_expert, int token_tile, int num_words, int num_operand, int stream_weights,
                       int* chain_done, int chain_need, int* tile_counter) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  Ctrl* c = reinterpret_cast<Ctrl*>(smem_raw);
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t ring_off = ((raw_addr + kCtrlBytes + 1023u) & ~1023u) - raw_addr;
  constexpr uint32_t kOpWeightBytes = 0;  // the weight operand lives in tensor memory
  constexpr int kACols = kGateUp ? 128 : 64;  // TMEM columns of one operand stage: 128 K packed = 64 columns per tile
  constexpr uint32_t kWordsBytes = kGateUp ? 2 * kWordsTileBytes : kWordsTileBytes;  // words stage
  const uint32_t act_bytes = static_cast<uint32_t>(token_tile) * 256u;                 // rows x 128 K: two 64-K tiles
  const uint32_t op_bytes = kOpWeightBytes + act_bytes;                               // operand stage
  unsigned char* op_ring = smem_raw + ring_off;
  unsigned char* words_ring = op_ring + static_cast<size_t>(num_operand) * op_bytes;
  const int acc_cols = 2 * token_tile;   // gate and up, or the two partial sums of down
  const int num_acc = (2 * acc_cols + num_operand * kACols <= 512) ? 2 : 1;
  const uint32_t a_col0 = static_cast<uint32_t>(num_acc * acc_cols);       // operand stages follow the accumulators
  uint32_t tmem_cols = 32;
  while (tmem_cols < a_col0 + static_cast<uint32_t>(num_operand * kACols)) tmem_cols <<= 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool chained = !kGateUp && chain_done != nullptr;
  const bool dynamic = !kGateUp && tile_counter != nullptr;
  if (!kGateUp) pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < num_words; ++s) {
      mbar_init(&c->words_full[s], 1);
      mbar_init(&c->words_empty[s], kConverters / 32);   // one arrival per converter warp
    }
    for (int s = 0; s < num_operand; ++s) {
      mbar_init(&c->op_full[s], 8 + 1);                  // two converter warps per lane quarter + the activation TMA
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
  // A chained down kernel can only be scheduled once every gate/up CTA has passed its own wait (gate/up lets its
  // dependents go after it), so the dispatch metadata is complete; activated rows are awaited per expert below.
  if (!chained) pdl_wait();
  if (kGateUp) pdl_launch_dependents();
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
        for (int st = 0; st < num_kb / 2; ++st) {   // one operand stage = 128 K = two 64-K row tiles
          if (!mbar_wait(&c->op_empty[q], qph ^ 1u, &c->abort, status)) { ok = false; break; }
          mbar_expect_tx(&c->op_full[q], act_bytes);
          unsigned char* dst = op_ring + static_cast<size_t>(q) * op_bytes + kOpWeightBytes;
          tma_load_2d(dst, &tm_act, &c->op_full[q], (2 * st) * kBlockK, t.row0, pol_act);
          tma_load_2d(dst + act_bytes / 2, &tm_act, &c->op_full[q], (2 * st + 1) * kBlockK, t.row0, pol_act);
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
        for (int st = 0; st < num_kb / 2; ++st) {
          if (!mbar_wait(&c->op_full[q], qph, &c->abort, status)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_lo = umma_desc_lo(smem_u32(op_ring + static_cast<size_t>(q) * op_bytes));  // activation rows
          const uint32_t a_half = act_bytes >> 5;   // second 64-K row tile, in 16-byte descriptor units
          const uint32_t w_tmem = tmem_base + a_col0 + static_cast<uint32_t>(q * kACols);                 // weight tile(s)
#pragma unroll
          for (int k = 0; k < 2 * kBlockK / kUmmaK; ++k) {  // a K step of 16 BF16: 8 TMEM columns / 2 descriptor units
            const uint32_t b_lo = a_lo + (k >> 2) * a_half + 2 * (k & 3);
            if (kGateUp) {
              umma_tmem_a(half ? d_up : d_gate, w_tmem + 64 * half + 8 * k, b_lo, idesc, (st | k) != 0 ? 1u : 0u);
            } else if ((k & 1) == half) {
              umma_tmem_a(half ? d_up : d_gate, w_tmem + 8 * k, b_lo, idesc, (st | (k >> 1)) != 0 ? 1u : 0u);
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
    // ------------------------------------------------------------------ converter warps
    // Warp w may write TMEM lanes 32*(w%4)..+31 only, so the four warps of a lane quarter share those 32
    // channel rows by K: warp `part` converts sub-block `part` (64 K) of every words stage (256 K), gate and
    // up rows both, i.e. half `part & 1` of operand stage `part >> 1` of that words stage. One wait / fence /
    // arrival per 16 words, sixteen independent words in flight per thread.
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;          // channel row of the tile = TMEM lane
    const int part = (warp - 6) >> 2;             // 0..3: the sub-block of each words stage this warp converts
    const w4::Consts k4 = w4::make_consts();
    const long long total_rows = static_cast<long long>(E) * w_rows_per_expert;
    int p = 0, gst = 0;                           // words slot; operand stages so far (all warps count)
    uint32_t pph = 0;
    bool ok = true;
    for (int seq = 0; ok; ++seq) {
      const int item = follow_item(c, dynamic, seq, total_items, status);
      if (__any_sync(0xffffffffu, item < 0)) break;
      const Tile t = decode_tile(&c->tables, item, E, n_ct, token_tile);
      long long srow = static_cast<long long>(t.expert) * w_rows_per_expert + t.ct * kTileM + row;
      if (srow >= total_rows) srow = total_rows - 1;  // lanes past the last channel are never stored
      long long srow_up = srow + (kGateUp ? n_out : 0);
      if (srow_up >= total_rows) srow_up = total_rows - 1;
      const __nv_bfloat16* sg_ptr = scales + srow * groups + (part >> 1);   // this warp's group inside a words stage
      const __nv_bfloat16* su_ptr = scales + srow_up * groups + (part >> 1);
      const bool mine0 = part * kBlockK < min(kWordsK, k_dim);
      __nv_bfloat16 sg = mine0 ? sg_ptr[0] : __float2bfloat16(0.0f), su = mine0 ? su_ptr[0] : sg;
      for (int ws = 0; ok && ws < num_ws; ++ws) {
        const int subs = min(kWordsK, k_dim - ws * kWordsK) / kBlockK;
        const __nv_bfloat162 g2 = __bfloat162bfloat162(sg), u2 = __bfloat162bfloat162(su);
        if (ws + 1 < num_ws && part * kBlockK < min(kWordsK, k_dim - (ws + 1) * kWordsK)) {
          sg = sg_ptr[2 * ws + 2];   // next stage's scales while this one is converted
          su = su_ptr[2 * ws + 2];
        }
        if (!__all_sync(0xffffffffu, mbar_wait(&c->words_full[p], pph, &c->abort, status))) { ok = false; break; }
        if (part < subs) {
          const int g = gst + (part >> 1);
          const int q = g % num_operand;
          const uint32_t qph = static_cast<uint32_t>((g / num_operand) & 1);
          if (!__all_sync(0xffffffffu, mbar_wait(&c->op_empty[q], qph ^ 1u, &c->abort, status))) { ok = false; break; }
          tc_fence_after();  // the MMAs that read this stage last have completed (op_empty)
          const unsigned char* words = words_ring + static_cast<size_t>(p) * kWordsBytes + row * 128;
          const uint32_t dst = tmem_base + a_col0 + static_cast<uint32_t>(q * kACols) +
                               (static_cast<uint32_t>(quarter * 32) << 16);
          const int c0 = ((2 * part) ^ (row & 7)) << 4, c1 = ((2 * part + 1) ^ (row & 7)) << 4;
#pragma unroll 2
          for (int h = 0; h < (kGateUp ? 4 : 2); ++h) {   // 4 words = 32 K = 16 packed columns per store
            const __nv_bfloat162 scale2 = h < 2 ? g2 : u2;
            const uint4 w = *reinterpret_cast<const uint4*>(words + (h >> 1) * kWordsTileBytes + ((h & 1) ? c1 : c0));
            const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
            uint32_t r[16];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint4 d = w4::dequant_word(ww[i], scale2, k4);
              r[4 * i] = d.x; r[4 * i + 1] = d.y; r[4 * i + 2] = d.z; r[4 * i + 3] = d.w;
            }
            // gate columns [0,64) and up columns [64,128) of the stage (down: [0,64)), this warp's 64-K half
            tmem_st16(dst + (h >> 1) * 64 + (part & 1) * 32 + (h & 1) * 16, r);
          }
          tmem_st_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&c->op_full[q]);  // one arrival per warp: eight warps complete a stage
        }
        gst += subs / 2;
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

void rings_for_t(bool gate_up, int token_tile, int* num_words, int* num_operand, int* smem_bytes) {
  const int act = token_tile * 256;
  const int words = (gate_up ? 2 : 1) * static_cast<int>(kWordsTileBytes);
  const int a_cols = gate_up ? 128 : 64, acc_cols = 2 * token_tile;
  int q = kMaxOperand;                                   // operand stages live in TMEM next to the accumulators
  while (q > 2 && 2 * acc_cols + q * a_cols > 512) --q;  // keep two accumulator sets
  const int budget = kSmemLimit - kCtrlBytes - 1024 - q * act;
  int p = budget / words;
  if (p > kMaxWords) p = kMaxWords;
  *num_words = p;
  *num_operand = q;
  *smem_bytes = kCtrlBytes + 1024 + q * act + p * words;
}

template <bool kGateUp>
cudaError_t launch_w4t(const B200MoePlan& p, cudaStream_t s, bool chained) {
  const auto& sh = p.shape;
  const int n_out = kGateUp ? sh.intermediate : sh.hidden;
  const int k_dim = kGateUp ? sh.hidden : sh.intermediate;
  const int n_ct = (n_out + kTileM - 1) / kTileM;
  const long long bound = (static_cast<long long>((p.routes + p.token_tile - 1) / p.token_tile) + sh.experts - 1) * n_ct;
  const int grid = static_cast<int>(bound < p.num_sms ? bound : p.num_sms);
  const int stream_weights = static_cast<long long>(p.routes) <= static_cast<long long>(sh.experts) * p.token_tile;
  launch_pdl(grouped_gemm_w4t_kernel<kGateUp>, dim3(grid), dim3(kThreads),
             static_cast<size_t>(kGateUp ? p.w4t_smem_gate_up : p.w4t_smem_down), s,
      kGateUp ? p.tm_gate_up_w : p.tm_down_w, kGateUp ? p.tm_grouped : p.tm_activated,
      static_cast<const __nv_bfloat16*>(kGateUp ? p.buf.gate_up_scales : p.buf.down_scales),
      static_cast<__nv_bfloat16*>(kGateUp ? p.buf.activated : p.buf.down_output),
      static_cast<const int*>(p.buf.offsets), static_cast<const int*>(p.buf.counts),
      static_cast<const int*>(p.buf.tasks), static_cast<int*>(p.buf.status), sh.experts, n_out, k_dim,
      kGateUp ? 2 * sh.intermediate : sh.hidden, p.token_tile, kGateUp ? p.w4t_packed_gate_up : p.w4t_packed_down,
      kGateUp ? p.w4t_operand_gate_up : p.w4t_operand_down, stream_weights,
      chained ? static_cast<int*>(p.buf.scratch) + router_flag_index(p) + 2 : static_cast<int*>(nullptr),
      4 * ((sh.intermediate + kTileM - 1) / kTileM),  // epilogue warps x gate/up channel tiles per token tile
      chained && !kGateUp ? static_cast<int*>(p.buf.scratch) + router_flag_index(p) + 1 : static_cast<int*>(nullptr));
  return cudaPeekAtLastError();
}

}  // namespace

int configure_w4t(B200MoePlan& p) {
  rings_for_t(true, p.token_tile, &p.w4t_packed_gate_up, &p.w4t_operand_gate_up, &p.w4t_smem_gate_up);
  rings_for_t(false, p.token_tile, &p.w4t_packed_down, &p.w4t_operand_down, &p.w4t_smem_down);
  if (p.w4t_packed_gate_up < 2 || p.w4t_packed_down < 2) {
    set_error("token_tile %d leaves fewer than 2 stages of packed words", p.token_tile);
    return B200MOE_ERR_INVALID;
  }
  cudaError_t e = cudaFuncSetAttribute(grouped_gemm_w4t_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       kSmemLimit);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(grouped_gemm_w4t_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
  if (e != cudaSuccess) {
    set_error("cudaFuncSetAttribute(W4 shared memory) failed: %s", cudaGetErrorString(e));
    return B200MOE_ERR_CUDA;
  }
  return B200MOE_OK;
}

cudaError_t launch_gate_up_w4t(const B200MoePlan& p, cudaStream_t s, bool chained) {
  return launch_w4t<true>(p, s, chained);
}
cudaError_t launch_down_w4t(const B200MoePlan& p, cudaStream_t s, bool chained) { return launch_w4t<false>(p, s, chained); }

}  // namespace b200moe
