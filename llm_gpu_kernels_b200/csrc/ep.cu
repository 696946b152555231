// Expert parallelism over NVLink peer memory: the token dispatch and the result
// return are plain stores from this GPU's kernels into buffers that live on the
// expert owner's / token owner's GPU, at the row's final position. No staging
// copy, no collective library call, no host read of a count: every rank learns
// all per-expert counts through an all-gather done with peer stores, and from
// them computes where each of its rows goes on the remote side.
//
// The reference is single-GPU and has no counterpart; the layout it implies is
// kept: on the expert owner rows are grouped by expert (then by source rank,
// then by the stable rank inside the source's block), i.e. exactly the
// `grouped_input` the grouped GEMM kernels consume, so the owner runs no
// dispatch of its own.
//
// Ordering between ranks uses three flag barriers per forward (counts
// published, rows landed, results landed): a rank stores its epoch into every
// peer's flag word with release.sys and spins (bounded, 1 s) on its own words
// with acquire.sys. The ranks run on different GPUs, so the spins do not
// starve each other. No multicast or multimem is used: plain peer stores only.
#include <cuda_bf16.h>
#include <cstring>
#include "plan.h"

namespace b200moe {
namespace {

constexpr int kMaxRanks = B200MOE_EP_MAX_RANKS;
constexpr int kMaxExperts = 256;
constexpr int kFlagSlots = 4;
constexpr unsigned long long kWaitLimitNs = 1000000000ull;

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long global_timer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// One block, every thread calls. Flags buffer per rank: int32 [kFlagSlots][8] flags, then [kFlagSlots] epochs.
__device__ void rank_barrier(const B200MoeEpArgs& a, int slot) {
  __shared__ int s_epoch;
  __threadfence_system();
  __syncthreads();
  int* mine = static_cast<int*>(a.flags_peers[a.rank]);
  if (threadIdx.x == 0) {
    int* epoch = mine + kFlagSlots * kMaxRanks + slot;
    s_epoch = *epoch + 1;
    *epoch = s_epoch;
  }
  __syncthreads();
  if (threadIdx.x < a.world) {
    st_release_sys(static_cast<int*>(a.flags_peers[threadIdx.x]) + slot * kMaxRanks + a.rank, s_epoch);
    const int* wait_on = mine + slot * kMaxRanks + threadIdx.x;
    const unsigned long long start = global_timer();
    while (ld_acquire_sys(wait_on) - s_epoch < 0) {
      if (global_timer() - start > kWaitLimitNs) {  // a peer never arrived: report, do not hang
        atomicOr(static_cast<int*>(a.status), B200MOE_STATUS_TIMEOUT);
        break;
      }
    }
  }
  __syncthreads();
}

// tables (int32): send_base[E] | block_start[El*G + 1] | src_pos[El*G]
__global__ void __launch_bounds__(256)
ep_counts_kernel(const B200MoeEpArgs a) {
  __shared__ int A[kMaxRanks * kMaxExperts];   // counts[source][expert]
  __shared__ int P[kMaxRanks * kMaxExperts];   // exclusive prefix of A over the experts of one source
  __shared__ int colsum[kMaxExperts];          // rows of expert e over all sources
  __shared__ int owner_prefix[kMaxExperts];    // rows of earlier experts of the same owner
  const int E = a.experts, G = a.world, El = E / G, lo = a.rank * El, tid = threadIdx.x;
  const int* counts = static_cast<const int*>(a.counts);
  // the expert plan's GEMM kernels synchronise through these words and expect them zero at their start
  for (int i = tid; i < a.expert_chain_words; i += blockDim.x) static_cast<int*>(a.expert_chain)[i] = 0;
  // that plan has no dispatch of its own, so its status word restarts here (the previous forward is complete:
  // this kernel runs behind it on the stream)
  if (tid == 0 && a.expert_status) *static_cast<int*>(a.expert_status) = 0;
  if (tid < E) {
    const int c = counts[tid];
    for (int g = 0; g < G; ++g) static_cast<int*>(a.all_counts_peers[g])[a.rank * E + tid] = c;
  }
  rank_barrier(a, 0);  // every rank's counts have landed here
  const int* all_counts = static_cast<const int*>(a.all_counts_peers[a.rank]);
  for (int i = tid; i < G * E; i += blockDim.x) A[i] = ld_acquire_sys(all_counts + i);
  __syncthreads();
  if (tid < E) {
    int sum = 0;
    for (int s = 0; s < G; ++s) sum += A[s * E + tid];
    colsum[tid] = sum;
  }
  if (tid < G) {  // one thread per source: prefix over its experts
    int run = 0;
    for (int e = 0; e < E; ++e) {
      P[tid * E + e] = run;
      run += A[tid * E + e];
    }
  }
  __syncthreads();
  if (tid < E) {
    const int first = tid / El * El;
    int run = 0;
    for (int e = first; e < tid; ++e) run += colsum[e];
    owner_prefix[tid] = run;
  }
  __syncthreads();
  int* tables = static_cast<int*>(a.tables);
  int* send_base = tables;
  int* block_start = tables + E;
  int* src_pos = block_start + El * G + 1;
  if (tid < E) {
    int before = 0;
    for (int s = 0; s < a.rank; ++s) before += A[s * E + tid];
    send_base[tid] = owner_prefix[tid] + before;  // where my first row of expert `tid` lands on its owner
  }
  // More rows for some owner than its receive buffer holds: every rank sees the same [G][E] matrix, so every rank
  // takes the same decision - no expert tile runs anywhere and every rank's status says so (a sender whose own
  // rows all fit would otherwise combine rows that the overflowing owner never produced).
  bool overflow = false;
  for (int g = 0; g < G; ++g) overflow |= owner_prefix[g * El + El - 1] + colsum[g * El + El - 1] > a.capacity;
  if (overflow && tid == 0) atomicOr(static_cast<int*>(a.status), B200MOE_STATUS_EP_OVERFLOW);
  if (tid < El) {
    const int e = lo + tid;
    const int total = overflow ? 0 : colsum[e], offset = overflow ? 0 : owner_prefix[e];
    static_cast<int*>(a.expert_counts)[tid] = total;
    static_cast<int*>(a.expert_offsets)[tid] = offset;
    int tiles_before = 0;
    for (int j = lo; j < e && !overflow; ++j) tiles_before += (colsum[j] + a.token_tile - 1) / a.token_tile;
    static_cast<int*>(a.expert_tasks)[tid] = tiles_before;
    if (tid == El - 1) {
      static_cast<int*>(a.expert_tasks)[El] = tiles_before + (total + a.token_tile - 1) / a.token_tile;
      static_cast<int*>(a.expert_rows)[0] = offset + total;
      block_start[El * G] = offset + total;
    }
    int run = offset;
    for (int s = 0; s < G; ++s) {
      block_start[tid * G + s] = run;        // block (local expert, source) in my receive buffer
      src_pos[tid * G + s] = P[s * E + e];   // the same rows' grouped position at the source
      run += A[s * E + e];
    }
  }
}

__device__ __forceinline__ void copy_row(const __nv_bfloat16* src, __nv_bfloat16* dst, int H, int lane) {
  if ((H & 7) == 0 && ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0) {
    const uint4* s4 = reinterpret_cast<const uint4*>(src);
    uint4* d4 = reinterpret_cast<uint4*>(dst);
    for (int i = lane; i < H / 8; i += 32) d4[i] = s4[i];
  } else {
    for (int i = lane; i < H; i += 32) dst[i] = src[i];
  }
}

// One warp per local route: its token row goes to the owner of its expert.
__global__ void __launch_bounds__(256)
ep_send_kernel(const B200MoeEpArgs a) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q = blockIdx.x * 8 + warp;
  if (q >= a.tokens * a.topk) return;
  const long long id = a.ids_are_int64 ? static_cast<const long long*>(a.ids)[q]
                                       : static_cast<long long>(static_cast<const int*>(a.ids)[q]);
  const int rank_in_block = static_cast<const int*>(a.ranks)[q];
  if (id < 0 || id >= a.experts || rank_in_block < 0) return;  // invalid route: flagged by the dispatch
  const int El = a.experts / a.world;
  const int owner = static_cast<int>(id) / El;
  const int row = static_cast<const int*>(a.tables)[id] + rank_in_block;
  if (row >= a.capacity) {
    if (lane == 0) atomicOr(static_cast<int*>(a.status), B200MOE_STATUS_EP_OVERFLOW);
    return;
  }
  copy_row(static_cast<const __nv_bfloat16*>(a.x) + static_cast<size_t>(q / a.topk) * a.hidden,
           static_cast<__nv_bfloat16*>(a.recv_rows_peers[owner]) + static_cast<size_t>(row) * a.hidden, a.hidden, lane);
  // the way back: the owner's down projection stores this row's result at mapping[q] of my return buffer
  if (lane == 0 && a.row_dest_peers[owner] && a.mapping)
    static_cast<int*>(a.row_dest_peers[owner])[row] = (a.rank << 24) | static_cast<const int*>(a.mapping)[q];
}

// One warp per received row: its result goes back to the source rank, at the route's grouped position.
__global__ void __launch_bounds__(256)
ep_return_kernel(const B200MoeEpArgs a) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int j = blockIdx.x * 8 + warp;
  const int rows = min(static_cast<const int*>(a.expert_rows)[0], a.capacity);
  if (j >= rows) return;
  const int G = a.world, El = a.experts / G;
  const int* block_start = static_cast<const int*>(a.tables) + a.experts;
  const int* src_pos = block_start + El * G + 1;
  int lo = 0, hi = El * G - 1;  // last block whose start is <= j
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (block_start[mid] <= j) lo = mid; else hi = mid - 1;
  }
  const int source = lo % G;
  const int dst_row = src_pos[lo] + (j - block_start[lo]);
  copy_row(static_cast<const __nv_bfloat16*>(a.expert_output) + static_cast<size_t>(j) * a.hidden,
           static_cast<__nv_bfloat16*>(a.return_rows_peers[source]) + static_cast<size_t>(dst_row) * a.hidden, a.hidden,
           lane);
}

__global__ void __launch_bounds__(32) ep_barrier_kernel(const B200MoeEpArgs a, int slot) { rank_barrier(a, slot); }

int check_args(const B200MoeEpArgs* a) {
  if (!a) {
    set_error("null argument");
    return B200MOE_ERR_INVALID;
  }
  if (a->world < 1 || a->world > kMaxRanks || a->rank < 0 || a->rank >= a->world || a->experts < 1 ||
      a->experts > kMaxExperts || a->experts % a->world || a->topk < 1 || a->topk > 32 || a->hidden <= 0 ||
      a->tokens < 0 || a->capacity <= 0 || a->token_tile <= 0 ||
      static_cast<long long>(a->tokens) * a->topk >= (1 << 24)) {
    set_error("expert parallel: needs 1 <= world <= 8, experts <= 256 divisible by world, K <= 32, H > 0");
    return B200MOE_ERR_INVALID;
  }
  const void* local[] = {a->counts, a->expert_counts, a->expert_offsets, a->expert_tasks, a->expert_rows,
                         a->expert_output, a->tables, a->status};
  for (const void* p : local)
    if (!p) {
      set_error("expert parallel: null local buffer");
      return B200MOE_ERR_INVALID;
    }
  for (int g = 0; g < a->world; ++g)
    if (!a->recv_rows_peers[g] || !a->return_rows_peers[g] || !a->all_counts_peers[g] || !a->flags_peers[g]) {
      set_error("expert parallel: peer buffer of rank %d is not open", g);
      return B200MOE_ERR_INVALID;
    }
  return B200MOE_OK;
}

int launched(const char* what) {
  const cudaError_t e = cudaPeekAtLastError();
  if (e == cudaSuccess) return B200MOE_OK;
  set_error("%s: %s", what, cudaGetErrorString(e));
  return B200MOE_ERR_CUDA;
}

int cuda_rc(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return B200MOE_OK;
  set_error("%s: %s", what, cudaGetErrorString(e));
  return B200MOE_ERR_CUDA;
}

}  // namespace
}  // namespace b200moe

using namespace b200moe;

extern "C" {

size_t b200moe_ep_table_ints(int32_t world, int32_t experts) {
  (void)world;
  return static_cast<size_t>(3) * static_cast<size_t>(experts) + 8;
}

int b200moe_peer_alloc(size_t bytes, void** ptr) {
  if (!ptr || !bytes) {
    set_error("peer_alloc: bad argument");
    return B200MOE_ERR_INVALID;
  }
  int rc = cuda_rc(cudaMalloc(ptr, bytes), "cudaMalloc (peer buffer)");
  if (rc) return rc;
  return cuda_rc(cudaMemset(*ptr, 0, bytes), "cudaMemset (peer buffer)");
}

int b200moe_peer_free(void* ptr) { return cuda_rc(cudaFree(ptr), "cudaFree (peer buffer)"); }

int b200moe_peer_export(void* ptr, unsigned char handle[64]) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  cudaIpcMemHandle_t h;
  int rc = cuda_rc(cudaIpcGetMemHandle(&h, ptr), "cudaIpcGetMemHandle");
  if (rc) return rc;
  memcpy(handle, &h, 64);
  return B200MOE_OK;
}

int b200moe_peer_import(const unsigned char handle[64], void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  return cuda_rc(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
}

int b200moe_peer_close(void* ptr) { return cuda_rc(cudaIpcCloseMemHandle(ptr), "cudaIpcCloseMemHandle"); }

int b200moe_ep_exchange_counts(const B200MoeEpArgs* a, void* stream) {
  int rc = check_args(a);
  if (rc) return rc;
  ep_counts_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(*a);
  return launched("ep counts launch");
}

int b200moe_ep_send_rows(const B200MoeEpArgs* a, void* stream) {
  int rc = check_args(a);
  if (rc) return rc;
  if (!a->x || !a->ids || !a->ranks) {
    set_error("expert parallel: x / ids / ranks are required to send rows");
    return B200MOE_ERR_INVALID;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int routes = a->tokens * a->topk;
  if (routes > 0) ep_send_kernel<<<(routes + 7) / 8, 256, 0, s>>>(*a);
  ep_barrier_kernel<<<1, 32, 0, s>>>(*a, 1);
  return launched("ep send launch");
}

int b200moe_ep_return_rows(const B200MoeEpArgs* a, void* stream) {
  int rc = check_args(a);
  if (rc) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (!a->fused_return) ep_return_kernel<<<(a->capacity + 7) / 8, 256, 0, s>>>(*a);
  ep_barrier_kernel<<<1, 32, 0, s>>>(*a, 2);
  return launched("ep return launch");
}

}  // extern "C"
