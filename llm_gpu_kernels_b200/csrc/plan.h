// Internal plan object behind the C ABI and the launchers of each subsystem.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>
#include "../../include/b200moe.h"

struct B200MoePlan {
  B200MoeShape shape{};
  B200MoeBuffers buf{};
  B200MoeWorkspace ws{};
  bool bound = false;
  int device = -1;
  int num_sms = 0;
  int routes = 0;          // R = T*K
  int token_tile = 0;      // rows of one expert per tile (tasks granularity)
  int schedule = 0;
  // dispatch partition: each warp ranks `warp_routes` consecutive routes
  int warp_routes = 0;
  int partitions = 0;      // number of warp partitions = ceil(R / warp_routes)
  bool dispatch_fused = false;  // count + scan + mapping in one kernel (R <= kFusedRoutes per CTA of a cluster)
  int dispatch_ctas = 1;        // CTAs of that kernel's thread-block cluster
  bool gather = false;          // gate/up reads token rows through source_rows; the dispatch copies no rows
  int chain_words = 0;     // scratch words after the router flag that the dispatch zeroes: tile counter + done[E]
  // TMA descriptors (tcgen05 schedule)
  CUtensorMap tm_gate_up_w{};   // [E*2I, H] bf16, box 64 x 128  (W4: [E*2I, H/8] int32, box 8 x 128)
  CUtensorMap tm_grouped{};     // [R, H] bf16, box 64 x token_tile
  CUtensorMap tm_down_w{};      // [E*H, I] bf16, box 64 x 128   (W4: [E*H, I/8] int32, box 8 x 128)
  CUtensorMap tm_activated{};   // [R, I] bf16, box 64 x token_tile
  // router on the tensor cores (tcgen05 schedule with a router)
  bool router_tc = false;
  CUtensorMap tm_x{};           // [T, H] bf16, box 64 x 128
  CUtensorMap tm_router_w{};    // [E, H] bf16, box 64 x round_up(E,16)
  int router_smem = 0, router_stages = 0, router_ksplit = 1;  // ksplit = CTAs per cluster sharing one token tile
  int gemm_smem_gate_up = 0, gemm_stages_gate_up = 0;
  int gemm_smem_down = 0, gemm_stages_down = 0;
  int gemm_smem_down_pair = 0, gemm_stages_down_pair = 0;   // down projection over 256-channel pair tiles
  bool down_pair = false;
  int down_tile = 0;        // token tile of the down kernel (256 with wide tiles while gate/up and `tasks` keep 128)
  int down_tiles = 0;       // resolved B200MoeShape.down_tiles (0 = not the BF16 tensor-core down kernel)
  // W4A16 kernels: packed-stage ring, operand-stage ring, dynamic shared memory
  int w4_packed_gate_up = 0, w4_operand_gate_up = 0, w4_smem_gate_up = 0;
  int w4_packed_down = 0, w4_operand_down = 0, w4_smem_down = 0;
  // the same for the variant that keeps the dequantised operand in tensor memory (token tile <= 128)
  int w4t_packed_gate_up = 0, w4t_operand_gate_up = 0, w4t_smem_gate_up = 0;
  int w4t_packed_down = 0, w4t_operand_down = 0, w4t_smem_down = 0;
  // the weight-streaming W4A16 kernel (token tile <= 16): dequantisation in registers, mma.sync
  int w4r_stages_gate_up = 0, w4r_smem_gate_up = 0;
  int w4r_stages_down = 0, w4r_smem_down = 0;
};

namespace b200moe {

void set_error(const char* fmt, ...);

// Each returns a cudaError_t from the launch (cudaPeekAtLastError), never synchronises.
cudaError_t launch_router(const B200MoePlan& p, cudaStream_t s);
cudaError_t launch_router_tc(const B200MoePlan& p, cudaStream_t s);
cudaError_t launch_dispatch(const B200MoePlan& p, cudaStream_t s);
cudaError_t launch_gate_up_generic(const B200MoePlan& p, cudaStream_t s);
cudaError_t launch_down_generic(const B200MoePlan& p, cudaStream_t s);
// chained: the two BF16 GEMMs of one forward synchronise per expert through the done[E] counters in
// scratch and the down kernel draws tiles from the tile counter there (both zeroed by the dispatch).
cudaError_t launch_gate_up_tc(const B200MoePlan& p, cudaStream_t s, bool chained);
cudaError_t launch_down_tc(const B200MoePlan& p, cudaStream_t s, bool chained);
cudaError_t launch_gate_up_w4(const B200MoePlan& p, cudaStream_t s, bool chained);
cudaError_t launch_down_w4(const B200MoePlan& p, cudaStream_t s, bool chained);
cudaError_t launch_gate_up_w4t(const B200MoePlan& p, cudaStream_t s, bool chained);
cudaError_t launch_down_w4t(const B200MoePlan& p, cudaStream_t s, bool chained);
cudaError_t launch_gate_up_w4r(const B200MoePlan& p, cudaStream_t s, bool chained);
cudaError_t launch_down_w4r(const B200MoePlan& p, cudaStream_t s, bool chained);
bool w4r_serves(const B200MoePlan& p);
cudaError_t launch_combine(const B200MoePlan& p, cudaStream_t s);

size_t router_smem_bytes(int hidden, int experts);
cudaError_t router_opt_in_smem();

// One-time per-plan set-up of the tcgen05 kernels (smem opt-in, stage counts).
int configure_tc(B200MoePlan& p);
int configure_router_tc(B200MoePlan& p);
int configure_w4(B200MoePlan& p);
int configure_w4t(B200MoePlan& p);
int configure_w4r(B200MoePlan& p);

// The router raises its timeout flag in a scratch word (the dispatch folds it into the
// status word, which it resets every forward): int32 index of that word inside `scratch`.
// After it: the tile counter of the chained down kernel and done[E], also reset by the dispatch.
inline size_t router_flag_index(const B200MoePlan& p) {
  const int blocks = (p.partitions + 7) / 8;
  return static_cast<size_t>(p.partitions) * p.shape.experts + blocks;
}

constexpr int kGenericTile = 32;   // rows per tile of the CUDA-core schedule
constexpr int kFusedRoutes = 2048;   // one 1024-thread block ranks up to this many routes; a cluster of up to
constexpr int kFusedCluster = 8;     // kFusedCluster such blocks builds the dispatch metadata in one kernel (the
                                     // histograms meet through distributed shared memory); above, the ranking
                                     // is spread over many SMs by three kernels
constexpr int kDispatchWarps = 8;  // warps per block of the count / permute kernels

}  // namespace b200moe
