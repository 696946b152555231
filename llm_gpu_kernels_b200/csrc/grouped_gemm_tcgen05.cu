// Ragged grouped GEMM on the Blackwell tensor cores: TMA-fed tcgen05.mma with
// the accumulators in tensor memory, one persistent warp-specialised CTA per SM.
//
// Replaces the reference's gate/up + SwiGLU kernels (moe_fused.py:18-73,
// cuda_gate_up.cu:53-131) and its down projection (_dynamic_grouped,
// moe.py:69-95). Written for sm_100a from scratch:
//
//  * The weights are the M operand ("swap-AB"): one tile is 128 output
//    channels x `token_tile` rows of one expert. D[channel][row] lives in
//    tensor memory with the channel on the TMEM lane, so the MMA N dimension
//    is the (small, ragged) number of rows of the expert and is set per tile in
//    the instruction descriptor: an expert with 5 rows costs an N=16 MMA and
//    its weights are streamed from HBM exactly once.
//  * gate and up tiles share the activation tile and accumulate into two TMEM
//    column ranges of the same lanes, so SwiGLU needs no data exchange: the
//    thread that owns channel c reads gate[c][n] and up[c][n], and nothing is
//    rounded before silu(g)*u (one BF16 rounding, at the store).
//  * Expert segments are dense and ragged (no padding): an activation box may
//    run into the next expert's rows or past the end (zero fill); those
//    columns of D are simply not stored. A weight box may run past the
//    expert's channels; those lanes are not stored.
//  * Tiles are enumerated on the device from the `tasks` prefix the dispatch
//    wrote (tile -> expert by binary search), round-robin over the persistent
//    CTAs, so the grid is shape-only and the launch is graph-capturable.
//  * warp 0 = TMA producer, warps 1 and 6 = MMA issuers (warp 1 owns TMEM), warps 2-5 =
//    epilogue (one TMEM lane quarter each). One thread can issue a tcgen05.mma only about
//    every 100 cycles (measured, any N), two threads in different warps issue in parallel:
//    the MMAs of a stage are split between two issuers with an accumulator each - the gate
//    and the up tile, or for the down projection the even and the odd K steps, whose two
//    partial sums the epilogue adds in FP32. Shared-memory stages and the TMEM
//    accumulators are double buffered through mbarriers; every wait is bounded
//    and on expiry raises B200MOE_STATUS_TIMEOUT and leaves cleanly.
//  * Inside one forward the two GEMMs are chained by per-expert completion
//    counters instead of a kernel boundary: every gate/up epilogue warp bumps
//    done[expert] after its stores, the down kernel is launched as a programmatic
//    dependent, does not wait for the gate/up grid, takes its tiles from a global
//    counter (so CTAs that start early do more) and waits per expert until the
//    counter says that all activated rows of that expert are written. The SMs that
//    idle in gate/up's last, partial round of tiles stream down weights meanwhile.
#include <cuda_bf16.h>
#include <cuda.h>
#include "plan.h"
#include "sm100_ptx.cuh"
#include "gemm_tile.cuh"
#include "pdl.cuh"

namespace b200moe {
namespace {

using namespace ptx;
using namespace tile;

constexpr int kThreads = 224;
constexpr int kMmaWarpB = 6;  // second MMA-issuing warp
constexpr int kGatherWarps = 4;                              // warps 7..10 of the gathering gate/up kernel
constexpr int kGatherThreads = kThreads + 32 * kGatherWarps;
constexpr int kGatherMaxIters = 16;                           // 16-byte chunks per gather lane and stage: tile 256
constexpr int kMaxStages = 12;
constexpr uint32_t kWTileBytes = kTileM * kBlockK * 2;  // 16 KB
constexpr int kCtrlBytes = 4096;
static_assert(kItemRing >= kMaxStages + 3, "producer could lap the item ring");
// Staging of the epilogue that returns rows to other ranks: 16 rows x 128 channels BF16 (+16 bytes of padding per
// row), two buffers.
constexpr uint32_t kEpiRowBytes = kTileM * 2 + 16;
constexpr uint32_t kEpiBufBytes = 16 * kEpiRowBytes;

struct Ctrl {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t drain[2];
  uint64_t epi_bar[2];            // the four epilogue warps wrote their part of a staging buffer
  uint64_t item_ready[kItemRing];
  int item[kItemRing];
  uint32_t tmem_base;
  int abort;
  Tables tables;
};
static_assert(sizeof(Ctrl) <= kCtrlBytes, "control block too large");

// Epilogue of the down projection of an expert-parallel expert plan: result row r of the tile belongs to another
// rank and goes to row (row_dest[r] & 0xFFFFFF) of the buffer ret_bases[row_dest[r] >> 24], over NVLink. The
// accumulator has the channel on the TMEM lane, so a thread holds one channel of 16 rows; stored like that a warp
// would write 64-byte pieces, which NVLink moves badly. The four epilogue warps therefore transpose 16 rows x 128
// channels through shared memory and write whole 256-byte row segments, 16 bytes per lane. `chunk` counts the
// 16-row chunks this warp has staged (all four warps walk the same sequence); channel0 = first of the 128 channels
// behind `taddr`. Returns false when a wait gave up.
__device__ __forceinline__ bool return_tile_rows(const Tile& t, uint32_t taddr, int token_tile, int quarter, int lane,
                                                 int n_out, const int* __restrict__ row_dest,
                                                 const unsigned long long* __restrict__ ret_bases,
                                                 unsigned char* epi, uint64_t* epi_bar, unsigned& chunk, int* abort,
                                                 int* status, bool pair, int channel0) {
  for (int n0 = 0; n0 < t.n_eff; n0 += 16, ++chunk) {
    uint32_t g[16], u[16];
    tmem_ld16(taddr + n0, g);
    if (pair) {
      tmem_ld16(taddr + token_tile + n0, u);   // the odd-K partial sum of the second MMA issuer
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j) u[j] = 0u;
    }
    tmem_ld_wait();
    const unsigned buf = chunk & 1u;
    unsigned char* stage = epi + buf * kEpiBufBytes;
#pragma unroll
    for (int j = 0; j < 16; ++j)
      *reinterpret_cast<__nv_bfloat16*>(stage + j * kEpiRowBytes + (quarter * 32 + lane) * 2) =
          __float2bfloat16_rn(__fadd_rn(__uint_as_float(g[j]), __uint_as_float(u[j])));
    __syncwarp();
    if (lane == 0) mbar_arrive(&epi_bar[buf]);
    if (!__all_sync(0xffffffffu, mbar_wait(&epi_bar[buf], (chunk >> 1) & 1u, abort, status))) return false;
    // this warp sends rows quarter*4 .. quarter*4+3 of the chunk: two rows per instruction, 16 lanes x 16 bytes each
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
      const int row = quarter * 4 + rr * 2 + (lane >> 4), n = n0 + row;
      const int channel = channel0 + (lane & 15) * 8;
      if (n < t.rows && channel < n_out) {
        const int d = row_dest[t.row0 + n];
        __nv_bfloat16* base = reinterpret_cast<__nv_bfloat16*>(ret_bases[static_cast<unsigned>(d) >> 24]);
        const uint4 v = *reinterpret_cast<const uint4*>(stage + row * kEpiRowBytes + (lane & 15) * 16);
        *reinterpret_cast<uint4*>(base + static_cast<size_t>(d & 0xFFFFFF) * n_out + channel) = v;
      }
    }
  }
  return true;
}

// chain_done: per-expert completion counters of the gate/up stage (null = stages separated by kernel
// boundaries). The gate/up kernel adds one per epilogue warp and tile; the down kernel, given
// chain_need = arrivals per token tile of an expert, waits for them before it loads activated rows.
// tile_counter (down kernel only): global tile counter of the dynamic schedule, zero at launch.
// row_dest / ret_bases (down kernel of an expert-parallel expert plan, else null): the result rows are stored
// straight into their token owners' buffers over NVLink (see return_tile_rows).
// kGather (gate/up only): the rows of a tile are not read from an expert-contiguous copy but gathered from the
// token rows themselves: source_rows[r] = token whose row grouped row r is (written by the dispatch), x = [T, k_dim].
// Four extra warps copy 16-byte chunks with cp.async into the 128-byte-swizzled activation tile of each stage
// (what the TMA box load would have written) and arrive on the stage's barrier through
// cp.async.mbarrier.arrive, so the copies of several stages are in flight and no register holds data.
// kPair (down projection only): one tile is TWO channel tiles (256 output channels) of one token tile. The two weight
// boxes share every activation tile in shared memory, exactly as the gate and the up box do, each MMA issuer owns one
// channel tile over all of K and there are no partial sums. Once an expert has several token tiles the kernels are
// bound by what they pull out of L2 per FLOP (ncu at T=8192: 3.2 GB of operand tiles through L2 for the down
// projection, 7.7 TB/s, tensor pipe 24 % busy); sharing the activation tile cuts that by a quarter.
// kSingle (down projection at token tile 256) and kReturn (row_dest set) are template parameters as well: as run-time
// switches they left the compiler one large epilogue with every variant in it, and the plain down kernel lost a
// quarter of its speed to that.
template <bool kGateUp, bool kGather = false, bool kPair = false, bool kSingle = false, bool kReturn = false>
__global__ void __launch_bounds__(kGather ? kGatherThreads : kThreads, 1)
grouped_gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_act,
                       __nv_bfloat16* __restrict__ out, const int* __restrict__ g_offsets,
                       const int* __restrict__ g_counts, const int* __restrict__ g_tasks, int* __restrict__ status,
                       int E, int n_out, int k_dim, int w_rows_per_expert, int token_tile, int num_stages,
                       int stream_weights, int* chain_done, int chain_need, int* tile_counter,
                       const int* row_dest, const unsigned long long* ret_bases,
                       const __nv_bfloat16* __restrict__ x, const int* __restrict__ source_rows,
                       const unsigned char* __restrict__ prefetch_base, int prefetch_chunks, int chain_tile) {
  static_assert(kGateUp || !kGather, "only the gate/up projection gathers token rows");
  static_assert(!kGateUp || !(kPair || kSingle || kReturn), "schedules of the down projection");
  static_assert(!(kPair && kSingle), "the pair tile has two issuers");
  constexpr bool kTwoBoxes = kGateUp || kPair;          // two weight boxes per stage, one MMA issuer each
  constexpr int kTileChannels = kPair ? 2 * kTileM : kTileM;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  Ctrl* c = reinterpret_cast<Ctrl*>(smem_raw);
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t stage_off = ((raw_addr + kCtrlBytes + 1023u) & ~1023u) - raw_addr;
  unsigned char* stages = smem_raw + stage_off;
  constexpr uint32_t kWBytes = kTwoBoxes ? 2 * kWTileBytes : kWTileBytes;
  const uint32_t act_bytes = static_cast<uint32_t>(token_tile) * 128u;
  const uint32_t stage_bytes = kWBytes + act_bytes;
  // At token tile 256 an MMA (N = 256) takes longer than one thread needs to issue it, so the down projection runs
  // with ONE issuer and one partial sum: its accumulator is 256 columns and still double-buffered (the epilogue of
  // a K = I tile is too long to leave unoverlapped). gate/up needs gate + up = 512 columns either way.
  constexpr bool single_issuer = kSingle;
  const int acc_cols = single_issuer ? token_tile : 2 * token_tile;   // gate and up, or the two partial sums of down
  const int num_acc = (2 * acc_cols <= 512) ? 2 : 1;
  uint32_t tmem_cols = 32;
  while (tmem_cols < static_cast<uint32_t>(num_acc * acc_cols)) tmem_cols <<= 1;
  const bool chained = !kGateUp && chain_done != nullptr;  // down kernel reading a gate/up grid still running
  const bool dynamic = !kGateUp && tile_counter != nullptr;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (!kGateUp) pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < num_stages; ++s) {
      mbar_init(&c->full[s], kGather ? 1 + 32 * kGatherWarps : 1);   // TMA (+ every gather lane's copies)
      mbar_init(&c->empty[s], single_issuer ? 1 : 2);   // the commits of the MMA issuers
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&c->tmem_full[a], single_issuer ? 1 : 2);  // the MMA issuers
      mbar_init(&c->tmem_empty[a], 4);  // one arrival per epilogue warp
    }
    for (int q = 0; q < kItemRing; ++q) mbar_init(&c->item_ready[q], 1);
    mbar_init(&c->drain[0], 1);
    mbar_init(&c->drain[1], 1);
    if (kReturn) {
      mbar_init(&c->epi_bar[0], 4);
      mbar_init(&c->epi_bar[1], 4);
    }
    c->abort = 0;
    mbar_init_fence();
  }
  if (warp == 1) {
    tmem_alloc(&c->tmem_base, tmem_cols);
  }
  // gate/up: the kernels before this one (router, dispatch) leave HBM idle, and this CTA is resident long before they
  // finish. Pull the head of the weight tensor - what the grid will read first, whatever the routing turns out to
  // be - into L2 meanwhile; the TMA loads below then hit there.
  if (kGateUp) prefetch_head(prefetch_base, prefetch_chunks);
  // Everything above overlapped with the previous kernel. A chained down kernel does not wait for the
  // gate/up grid: it can only be scheduled after every gate/up CTA has passed its own wait (below), so
  // the dispatch metadata is complete, and it synchronises on activated rows through chain_done.
  if (!chained) pdl_wait();
  // gate/up lets its dependents go only now, so that a chained down kernel inherits "dispatch complete"
  if (kGateUp) pdl_launch_dependents();
  load_tables(&c->tables, g_tasks, g_offsets, g_counts, E);
  if (!kGateUp && chain_tile != token_tile) {
    // wide tiles: `tasks` was built by the dispatch for gate/up's token tile; this kernel tiles the same experts at
    // its own token_tile, so it rebuilds the prefix from the counts (one warp, E <= 256)
    __syncthreads();
    if (warp == 0) {
      int run = 0;
      for (int e0 = 0; e0 < E; e0 += 32) {
        const int e = e0 + lane;
        const int tiles = e < E ? (c->tables.counts[e] + token_tile - 1) / token_tile : 0;
        int incl = tiles;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int v = __shfl_up_sync(0xffffffffu, incl, o);
          if (lane >= o) incl += v;
        }
        if (e < E) c->tables.tasks[e] = run + incl - tiles;
        run += __shfl_sync(0xffffffffu, incl, 31);
      }
      if (lane == 0) c->tables.tasks[E] = run;
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&c->tmem_base);

  const int n_ct = (n_out + kTileChannels - 1) / kTileChannels;
  const int num_kb = (k_dim + kBlockK - 1) / kBlockK;
  const int total_items = c->tables.tasks[E] * n_ct;

  if (warp == 0) {
    if (lane == 0) {
      // ---------------------------------------------------------------- TMA producer
      const uint64_t pol_w = stream_weights ? policy_evict_first() : policy_evict_last();
      const uint64_t pol_act = policy_evict_last();
      int stage = 0;
      uint32_t phase = 0;
      long long issued = 0;
      bool ok = true;
      int ready_expert = -1;  // activated rows of this expert are known to be complete
      for (int seq = 0; ok; ++seq) {
        const int item = dynamic ? draw_item(c, tile_counter, seq, total_items)
                                 : follow_item(c, false, seq, total_items, status);
        if (item < 0) break;
        const Tile t = decode_tile(&c->tables, item, E, n_ct, token_tile);
        const int w_row = t.expert * w_rows_per_expert + t.ct * kTileChannels;
        if (chained && t.expert != ready_expert) {
          // arrivals per gate/up token tile x gate/up token tiles of the expert (gate/up tiles at chain_tile rows)
          const int need = chain_need * ((c->tables.counts[t.expert] + chain_tile - 1) / chain_tile);
          if (!wait_expert_done(chain_done + t.expert, need, &c->abort, status)) { ok = false; break; }
          ready_expert = t.expert;
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&c->empty[stage], phase ^ 1u, &c->abort, status)) { ok = false; break; }
          unsigned char* st = stages + static_cast<size_t>(stage) * stage_bytes;
          mbar_expect_tx(&c->full[stage], kGather ? kWBytes : stage_bytes);
          tma_load_2d(st, &tm_w, &c->full[stage], kb * kBlockK, w_row, pol_w);
          if (kTwoBoxes)   // the up rows of the same channels / the next 128 channels
            tma_load_2d(st + kWTileBytes, &tm_w, &c->full[stage], kb * kBlockK, w_row + (kGateUp ? n_out : kTileM), pol_w);
          if (!kGather) tma_load_2d(st + kWBytes, &tm_act, &c->full[stage], kb * kBlockK, t.row0, pol_act);
          ++issued;
          if (++stage == num_stages) { stage = 0; phase ^= 1u; }
        }
      }
      // Never leave with copies in flight: wait (bounded) for the last copy of
      // every stage. On the normal path these have long completed.
      const long long first = issued > num_stages ? issued - num_stages : 0;
      for (long long i = first; i < issued; ++i) {
        const int s = static_cast<int>(i % num_stages);
        const uint32_t ph = static_cast<uint32_t>((i / num_stages) & 1);
        if (!mbar_wait_plain(&c->full[s], ph)) { atomicOr(status, B200MOE_STATUS_TIMEOUT); break; }
      }
    }
  } else if (warp == 1 || warp == kMmaWarpB) {
    if (lane == 0 && !(single_issuer && warp == kMmaWarpB)) {
      // ---------------------------------------------------------------- MMA issuers (0: gate / even K, 1: up / odd K)
      const int half = warp == 1 ? 0 : 1;
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
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
          if (!mbar_wait(&c->full[stage], phase, &c->abort, status)) { ok = false; break; }
          tc_fence_after();
          if (kGather) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // cp.async-written rows -> MMA
          const uint32_t w_addr = smem_u32(stages + static_cast<size_t>(stage) * stage_bytes);
          const uint32_t a_addr = w_addr + kWBytes;
#pragma unroll
          for (int k = 0; k < kBlockK / kUmmaK; ++k) {
            const uint64_t bdesc = umma_desc(a_addr + k * kUmmaK * 2);
            if (kTwoBoxes) {
              umma(half ? d_up : d_gate, umma_desc(w_addr + half * kWTileBytes + k * kUmmaK * 2), bdesc, idesc,
                   (kb | k) != 0 ? 1u : 0u);
            } else if (single_issuer) {
              umma(d_gate, umma_desc(w_addr + k * kUmmaK * 2), bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
            } else if ((k & 1) == half) {
              umma(half ? d_up : d_gate, umma_desc(w_addr + k * kUmmaK * 2), bdesc, idesc, (kb | (k >> 1)) != 0 ? 1u : 0u);
            }
          }
          umma_commit(&c->empty[stage]);  // stage reusable once these MMAs have read it
          if (++stage == num_stages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma_commit(&c->tmem_full[acc]);
        if (++acc == num_acc) { acc = 0; acc_phase ^= 1u; }
      }
      if (!ok) {  // gave up: let the MMAs already issued finish before TMEM is freed
        umma_commit(&c->drain[half]);
        mbar_wait_plain(&c->drain[half], 0);
      }
    }
  } else if (kGather && warp > kMmaWarpB) {
    // ------------------------------------------------------------------ gather warps: token rows -> activation tile
    const int gt = (warp - kMmaWarpB - 1) * 32 + lane;   // 0..127
    const int chunk = gt & 7;                            // 16-byte chunk of the 128-byte k-block row
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int seq = 0; ok; ++seq) {
      const int item = follow_item(c, false, seq, total_items, status);
      if (item < 0) break;
      const Tile t = decode_tile(&c->tables, item, E, n_ct, token_tile);
      const int iters = (t.rows * 8 + 32 * kGatherWarps - 1) / (32 * kGatherWarps);   // <= kGatherMaxIters
      int src[kGatherMaxIters];   // element offset of row n = it*16 + gt/8 in x, -1 past the tile's rows
#pragma unroll
      for (int it = 0; it < kGatherMaxIters; ++it) {
        const int n = it * 16 + (gt >> 3);
        src[it] = (it < iters && n < t.rows) ? source_rows[t.row0 + n] * k_dim : -1;
      }
      for (int kb = 0; kb < num_kb; ++kb) {
        int free_ok = 1;
        if (lane == 0) free_ok = mbar_wait(&c->empty[stage], phase ^ 1u, &c->abort, status) ? 1 : 0;
        free_ok = __shfl_sync(0xffffffffu, free_ok, 0);
        if (!free_ok) { ok = false; break; }
        const uint32_t act = smem_u32(stages + static_cast<size_t>(stage) * stage_bytes) + kWBytes;
        const int k = kb * kBlockK + chunk * 8;
        const uint32_t bytes = k < k_dim ? 16u : 0u;       // a chunk past K is zero-filled, as the TMA load did
#pragma unroll
        for (int it = 0; it < kGatherMaxIters; ++it) {
          if (it < iters && src[it] >= 0) {
            const int n = it * 16 + (gt >> 3);
            const uint32_t dst = act + static_cast<uint32_t>(n) * 128u + (static_cast<uint32_t>(chunk ^ (n & 7)) << 4);
            const __nv_bfloat16* from = x + src[it] + (bytes ? k : 0);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(from), "r"(bytes) : "memory");
          }
        }
        // one arrival per lane once its copies above have landed (the barrier expects every gather lane)
        asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(&c->full[stage])) : "memory");
        if (++stage == num_stages) { stage = 0; phase ^= 1u; }
      }
    }
    asm volatile("cp.async.wait_all;" ::: "memory");   // never leave with copies in flight
  } else {
    // ------------------------------------------------------------------ epilogue warps
    const int quarter = warp & 3;  // TMEM lane quarter this warp may read
    int acc = 0;
    uint32_t acc_phase = 0;
    unsigned epi_chunk = 0;
    unsigned char* epi = stages + static_cast<size_t>(num_stages) * stage_bytes;   // reserved when row_dest is set
    for (int seq = 0;; ++seq) {
      // warp-uniform outcomes: the TMEM loads below need the whole warp
      const int item = follow_item(c, dynamic, seq, total_items, status);
      if (__any_sync(0xffffffffu, item < 0)) break;
      const Tile t = decode_tile(&c->tables, item, E, n_ct, token_tile);
      if (!__all_sync(0xffffffffu, mbar_wait(&c->tmem_full[acc], acc_phase, &c->abort, status))) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + static_cast<uint32_t>(acc * acc_cols) + (static_cast<uint32_t>(quarter * 32) << 16);
      if (kReturn) {
        bool sent = return_tile_rows(t, taddr, token_tile, quarter, lane, n_out, row_dest, ret_bases, epi, c->epi_bar,
                                     epi_chunk, &c->abort, status, !single_issuer && !kPair, t.ct * kTileChannels);
        if (sent && kPair)
          sent = return_tile_rows(t, taddr + token_tile, token_tile, quarter, lane, n_out, row_dest, ret_bases, epi,
                                  c->epi_bar, epi_chunk, &c->abort, status, false, t.ct * kTileChannels + kTileM);
        if (!sent) break;
      } else if (kPair) {
        store_tile<false, false>(t, taddr, token_tile, t.ct * kTileChannels + quarter * 32 + lane, n_out, out);
        store_tile<false, false>(t, taddr + token_tile, token_tile, t.ct * kTileChannels + kTileM + quarter * 32 + lane,
                                 n_out, out);
      } else if (single_issuer) {
        store_tile<false, false>(t, taddr, token_tile, t.ct * kTileM + quarter * 32 + lane, n_out, out);
      } else {
        store_tile<kGateUp, !kGateUp>(t, taddr, token_tile, t.ct * kTileM + quarter * 32 + lane, n_out, out);
      }
      tc_fence_before();
      if (kGateUp && chain_done != nullptr) {
        // this lane's rows were written through the generic proxy and the down kernel reads them through the
        // async proxy (TMA): order them for that proxy, then make them visible GPU-wide before the counter moves
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
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, tmem_cols);
  }
}

int stages_for(bool gate_up, int token_tile, int* smem_bytes, int reserve = 0) {
  const int stage = (gate_up ? 2 : 1) * static_cast<int>(kWTileBytes) + token_tile * 128;
  int stages = (kSmemLimit - kCtrlBytes - 1024 - reserve) / stage;
  if (stages > kMaxStages) stages = kMaxStages;
  *smem_bytes = kCtrlBytes + 1024 + stages * stage + reserve;
  return stages;
}

template <bool kGateUp, bool kGather = false, bool kPair = false, bool kSingle = false, bool kReturn = false>
cudaError_t launch_tc(const B200MoePlan& p, cudaStream_t s, bool chained) {
  const auto& sh = p.shape;
  const int n_out = kGateUp ? sh.intermediate : sh.hidden;
  const int k_dim = kGateUp ? sh.hidden : sh.intermediate;
  const int tile_channels = kPair ? 2 * kTileM : kTileM;
  const int n_ct = (n_out + tile_channels - 1) / tile_channels;
  const int token_tile = kGateUp ? p.token_tile : p.down_tile;
  const long long bound = (static_cast<long long>((p.routes + token_tile - 1) / token_tile) + sh.experts - 1) * n_ct;
  const int grid = static_cast<int>(bound < p.num_sms ? bound : p.num_sms);
  const int smem = kGateUp ? p.gemm_smem_gate_up : kPair ? p.gemm_smem_down_pair : p.gemm_smem_down;
  const int stages = kGateUp ? p.gemm_stages_gate_up : kPair ? p.gemm_stages_down_pair : p.gemm_stages_down;
  // weights are streamed (evict-first) when an expert rarely has a second token tile
  const int stream_weights = static_cast<long long>(p.routes) <= static_cast<long long>(sh.experts) * token_tile;
  const long long weight_bytes = static_cast<long long>(sh.experts) * 2 * sh.intermediate * sh.hidden * 2;
  const int prefetch_chunks = prefetch_head_chunks(weight_bytes);
  launch_pdl(grouped_gemm_tc_kernel<kGateUp, kGather, kPair, kSingle, kReturn>, dim3(grid), dim3(kGather ? kGatherThreads : kThreads), smem, s,
      kGateUp ? p.tm_gate_up_w : p.tm_down_w, kGateUp ? p.tm_grouped : p.tm_activated,
      static_cast<__nv_bfloat16*>(kGateUp ? p.buf.activated : p.buf.down_output),
      static_cast<const int*>(p.buf.offsets), static_cast<const int*>(p.buf.counts),
      static_cast<const int*>(p.buf.tasks), static_cast<int*>(p.buf.status), sh.experts, n_out, k_dim,
      kGateUp ? 2 * sh.intermediate : sh.hidden, token_tile, stages, stream_weights,
      chained ? static_cast<int*>(p.buf.scratch) + router_flag_index(p) + 2 : static_cast<int*>(nullptr),
      4 * ((sh.intermediate + kTileM - 1) / kTileM),  // epilogue warps x gate/up channel tiles per token tile
      chained && !kGateUp ? static_cast<int*>(p.buf.scratch) + router_flag_index(p) + 1 : static_cast<int*>(nullptr),
      kGateUp ? static_cast<const int*>(nullptr) : static_cast<const int*>(p.buf.ep_row_dest),
      static_cast<const unsigned long long*>(p.buf.ep_return_bases), static_cast<const __nv_bfloat16*>(p.buf.x),
      static_cast<const int*>(p.buf.source_rows),
      kGateUp ? static_cast<const unsigned char*>(p.buf.gate_up) : static_cast<const unsigned char*>(nullptr),
      kGateUp ? prefetch_chunks : 0, p.token_tile);
  return cudaPeekAtLastError();
}

}  // namespace

int configure_tc(B200MoePlan& p) {
  p.gemm_stages_gate_up = stages_for(true, p.token_tile, &p.gemm_smem_gate_up);
  const int epi_reserve = p.buf.ep_row_dest ? 2 * static_cast<int>(kEpiBufBytes) : 0;
  p.gemm_stages_down = stages_for(false, p.down_tile, &p.gemm_smem_down, epi_reserve);
  p.gemm_stages_down_pair = stages_for(true, p.down_tile, &p.gemm_smem_down_pair, epi_reserve);   // two boxes per stage

  if (p.gemm_stages_gate_up < 2 || p.gemm_stages_down < 2) {
    set_error("token_tile %d leaves fewer than 2 shared-memory stages", p.token_tile);
    return B200MOE_ERR_INVALID;
  }
  // the opt-in is per kernel, not per plan: always raise it to the device limit
  const void* kernels[] = {
      reinterpret_cast<const void*>(grouped_gemm_tc_kernel<true>),
      reinterpret_cast<const void*>(grouped_gemm_tc_kernel<true, true>),
      reinterpret_cast<const void*>(grouped_gemm_tc_kernel<false>),
      reinterpret_cast<const void*>(grouped_gemm_tc_kernel<false, false, true>),
      reinterpret_cast<const void*>(grouped_gemm_tc_kernel<false, false, false, true>),
      reinterpret_cast<const void*>(grouped_gemm_tc_kernel<false, false, false, false, true>),
      reinterpret_cast<const void*>(grouped_gemm_tc_kernel<false, false, true, false, true>),
      reinterpret_cast<const void*>(grouped_gemm_tc_kernel<false, false, false, true, true>)};
  for (const void* kernel : kernels) {
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
    if (e != cudaSuccess) {
      set_error("cudaFuncSetAttribute(shared memory) failed: %s", cudaGetErrorString(e));
      return B200MOE_ERR_CUDA;
    }
  }
  return B200MOE_OK;
}

cudaError_t launch_gate_up_tc(const B200MoePlan& p, cudaStream_t s, bool chained) {
  return p.gather ? launch_tc<true, true>(p, s, chained) : launch_tc<true>(p, s, chained);
}
cudaError_t launch_down_tc(const B200MoePlan& p, cudaStream_t s, bool chained) {
  const bool single = !p.down_pair && p.down_tile > 128;   // one MMA issuer, one partial sum (see the kernel)
  if (p.buf.ep_row_dest) {
    if (p.down_pair) return launch_tc<false, false, true, false, true>(p, s, chained);
    return single ? launch_tc<false, false, false, true, true>(p, s, chained)
                  : launch_tc<false, false, false, false, true>(p, s, chained);
  }
  if (p.down_pair) return launch_tc<false, false, true>(p, s, chained);
  return single ? launch_tc<false, false, false, true>(p, s, chained) : launch_tc<false>(p, s, chained);
}

}  // namespace b200moe
