/*
 * b200moe - C ABI of the B200 (sm_100a) MoE-layer forward.
 *
 * One plan = one prepared MoE layer: fixed shapes, fixed device addresses,
 * values may change in place between forwards. Nothing here allocates device
 * memory, synchronises the device or reads device memory back to the host
 * after b200moe_plan_bind(): b200moe_forward() only enqueues kernels on the
 * given stream, so it can be captured into a CUDA graph.
 *
 * Each entry point names the interface of the reference project
 * (llm-gpu-kernels, paths relative to its src/llm_gpu_kernels/) it replaces.
 * All functions return 0 on success and a negative B200MOE_ERR_* code on
 * failure; b200moe_last_error() gives the message for the calling thread.
 * Nothing throws across this boundary.
 */
#ifndef B200MOE_H_
#define B200MOE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200MOE_ABI_VERSION 4

/* error codes */
#define B200MOE_OK 0
#define B200MOE_ERR_INVALID (-1)     /* bad argument / shape / alignment */
#define B200MOE_ERR_CUDA (-2)        /* a CUDA runtime or driver call failed */
#define B200MOE_ERR_UNSUPPORTED (-3) /* device is not sm_100, or schedule impossible for the shape */
#define B200MOE_ERR_STATE (-4)       /* call order (forward before bind, ...) */

/* device status word, bits as in the reference (moe.py:21-30, docs/MOE_USAGE.md:110-113) */
#define B200MOE_STATUS_BAD_ID 1      /* an expert id outside [0,E) */
#define B200MOE_STATUS_BAD_WEIGHT 2  /* a NaN/Inf routing weight */
#define B200MOE_STATUS_TIMEOUT 4     /* a bounded wait inside a kernel gave up */
#define B200MOE_STATUS_EP_OVERFLOW 8 /* expert-parallel receive capacity exceeded */

/* weight formats */
#define B200MOE_WEIGHTS_BF16 0
#define B200MOE_WEIGHTS_W4G128 1 /* packed int4 (q+8), 8 per int32, BF16 scale per 128 along K */

/* schedules (shape-only choice, the analogue of moe_full_policy.py:132-152) */
#define B200MOE_SCHEDULE_AUTO 0
#define B200MOE_SCHEDULE_GENERIC 1 /* CUDA-core tiles, any H/I */
#define B200MOE_SCHEDULE_TCGEN05 2 /* TMA + tcgen05/TMEM tiles, needs H%8==0 and I%8==0 */

typedef struct B200MoePlan B200MoePlan;

/* Shape of one prepared layer. Replaces the shape arguments implied by
 * prepare_moe(x, gate_up, down, ids, routing_weights) (moe.py:220-235). */
typedef struct {
  int32_t tokens;         /* T >= 0 */
  int32_t experts;        /* 1 <= E <= 256 */
  int32_t topk;           /* 1 <= K <= 32 */
  int32_t hidden;         /* H > 0 */
  int32_t intermediate;   /* I > 0 */
  int32_t ids_are_int64;  /* 0: int32 ids, 1: int64 ids */
  int32_t gate_up_format; /* B200MOE_WEIGHTS_* */
  int32_t down_format;    /* B200MOE_WEIGHTS_* */
  int32_t schedule;       /* B200MOE_SCHEDULE_* */
  int32_t token_tile;     /* rows of one expert handled by one tile; 0 = choose from T*K/E */
  int32_t use_router;     /* 1: ids / routing_weights are written by the router each forward */
  int32_t route_only;     /* 1: no expert weights: forward = router + dispatch; combine reads down_output
                             filled by the caller (the token-owning side of expert parallelism);
                             2: the same, and dispatch does not copy rows (grouped_input may be NULL) */
  int32_t external_dispatch; /* 1: rows arrive already grouped by expert and counts / offsets / tasks are
                             written by someone else (the expert-owning side of expert parallelism):
                             forward = gate_up + down on grouped_input; x / ids / weights / output unused.
                             2: the same, and whoever writes the metadata also zeroes the plan's chain words
                             (b200moe_plan_chain) before every forward, so that gate_up and down may be
                             chained through them as in an ordinary plan */
  int32_t router_bf16_weights; /* 1: the router rounds its renormalised weights through BF16, as the model the
                             reference captured does (scripts/capture_qwen3_moe_layer0.py:587-588) */
  int32_t unchained;      /* 1: b200moe_forward separates gate/up and down by an ordinary kernel boundary instead of
                             chaining them through the per-expert completion counters (for A/B timing) */
  int32_t fused_gather;   /* 1: do not materialise grouped_input when the kernels allow it (BF16 tensor-core gate/up, or
                             the W4 weight-streaming kernel): the dispatch writes source_rows instead of copying rows
                             and the gate/up kernel gathers the token rows itself. B200MoeWorkspace.gathers reports
                             what the plan resolved; grouped_input may then be NULL and is left untouched.
                             1 stops gathering once experts average more than three 128-row tiles (routes > 384 x
                             experts: the materialised copy is faster there), 2 gathers at any size. */
  int32_t down_tiles;     /* BF16 tensor-core down projection: 0 = shape-only choice, 1 = pair tiles (256 output channels x
                             token tile, token tile <= 128), 2 = 128-channel tiles with an even-K and an odd-K partial
                             sum, 3 = wide tiles (128 channels x 256 rows: the down kernel re-tiles the experts at 256
                             rows while gate/up keeps token tile 128; needs token tile 128; faster as a stage, no
                             faster inside a forward, so never the choice at 0). The choice at 0: pair up to token
                             tile 128, one 128-channel tile at token tile 256. 1 and 3 keep one running FP32 sum over K, 2 adds
                             two partial sums, so its low-order bits differ; two plans that must give identical bits
                             (an expert-parallel layer and its single-GPU twin) pin the same value.
                             B200MoeWorkspace.down_tiles reports what the plan resolved. */
  int32_t reserved[1];
} B200MoeShape;

/* Bytes of every workspace buffer the caller must allocate (256-byte aligned
 * device memory). Field names follow the workspace tensors of PreparedMoE
 * (moe.py:124-155) and PreparedRankedMoE.ranks (moe_ranked.py:72). */
typedef struct {
  size_t output;        /* [T,H] bf16 */
  size_t counts;        /* [E] int32 */
  size_t offsets;       /* [E] int32 */
  size_t cursors;       /* [E] int32, kept for interface parity (zeroed) */
  size_t tasks;         /* [E+1] int32, exclusive prefix of per-expert token tiles */
  size_t mapping;       /* [R] int32 */
  size_t ranks;         /* [R] int32 */
  size_t grouped_input; /* [R,H] bf16 */
  size_t activated;     /* [R,I] bf16 */
  size_t down_output;   /* [R,H] bf16 */
  size_t status;        /* [1] int32 */
  size_t scratch;       /* dispatch partial histograms, router flag, tile counter and per-expert completion
                           counters of the chained GEMM kernels */
  size_t source_rows;   /* [R] int32: token whose row each grouped row is (inverse of mapping; 0 unless gathers) */
  int32_t token_tile;   /* resolved tile */
  int32_t schedule;     /* resolved schedule */
  int32_t launches;     /* kernels one forward enqueues */
  int32_t gathers;      /* 1: gate/up gathers token rows through source_rows; grouped_input is not written */
  int32_t down_tiles;   /* the resolved B200MoeShape.down_tiles (1, 2 or 3); 0 where that option does not apply */
  int32_t reserved;
} B200MoeWorkspace;

/* Device pointers. x, weights, ids, routing_weights belong to the caller;
 * the rest is workspace of the sizes b200moe_plan_workspace() reports. */
typedef struct {
  const void* x;               /* [T,H] bf16 */
  const void* router_weight;   /* [E,H] bf16, NULL unless use_router */
  const void* gate_up;         /* bf16 [E,2I,H]  or packed int32 [E,2I,H/8] */
  const void* gate_up_scales;  /* bf16 [E,2I,H/128] for W4G128, else NULL */
  const void* down;            /* bf16 [E,H,I]   or packed int32 [E,H,I/8] */
  const void* down_scales;     /* bf16 [E,H,I/128] for W4G128, else NULL */
  void* ids;                   /* [T,K] int32/int64 (input, or router output) */
  void* routing_weights;       /* [T,K] float32 (input, or router output) */
  void* output;
  void* counts;
  void* offsets;
  void* cursors;
  void* tasks;
  void* mapping;
  void* ranks;
  void* grouped_input;
  void* activated;
  void* down_output;
  void* status;
  void* scratch;
  const void* valid_routes;    /* optional device int32: only the first *valid_routes routes exist this forward
                                  (the rest of the fixed-capacity buffers is padding); NULL = all T*K */
  const void* residual;        /* optional [T,H] bf16: output = bf16(float(residual) + float(bf16(layer result))),
                                  i.e. the layer followed by the model's residual add in BF16, in the combine kernel.
                                  May alias `output` is NOT allowed; NULL = no residual. No reference counterpart. */
  /* Expert-owning side of expert parallelism only (external_dispatch plans, BF16 tensor-core schedule), both NULL
   * otherwise: the down projection stores each result row straight into its token owner's buffer instead of
   * down_output. ep_row_dest[row] = (owner rank << 24) | row index in that owner's return buffer, written by the
   * senders next to the row itself; ep_return_bases = device array of B200MOE_EP_MAX_RANKS addresses, entry g =
   * rank g's return buffer ([its routes, H] bf16) as mapped in this process. */
  const void* ep_row_dest;
  const void* ep_return_bases;
  void* source_rows;           /* [R] int32 workspace, required when the plan gathers (B200MoeWorkspace.gathers) */
} B200MoeBuffers;

/* ABI version of the loaded library. */
int b200moe_abi_version(void);

/* Message of the last failure on this thread ("" if none). */
const char* b200moe_last_error(void);

/* Validates the shape exactly as prepare_moe does (moe.py:221-235: ranks,
 * 1<=E<=256, 1<=K<=32, H,I>0, R*max(H,2I) < 2^31) and resolves schedule and
 * tile. Does not touch the device. */
int b200moe_plan_create(const B200MoeShape* shape, B200MoePlan** plan);

/* Workspace sizes; the allocation itself stays with the caller, as the
 * reference allocates in prepare_moe (moe.py:237-242). */
int b200moe_plan_workspace(const B200MoePlan* plan, B200MoeWorkspace* sizes);

/* Binds device addresses on the current device, checks alignment / aliasing
 * (the TORCH_CHECKs of GateUpPlan, cuda_gate_up.cu:133-165) and encodes the
 * TMA descriptors. May be called again to rebind. */
int b200moe_plan_bind(B200MoePlan* plan, const B200MoeBuffers* buffers);

/* One whole forward: PreparedRankedMoE.run() (moe_ranked.py:81-92). No-op for T == 0. */
int b200moe_forward(B200MoePlan* plan, void* cuda_stream);

/* The five subsystems one at a time, for stage tests and profiling; calling
 * them in this order equals b200moe_forward(). They replace, in order:
 * (new: formula of scripts/capture_qwen3_moe_layer0.py:583-587),
 * _reset+_rank_histogram+_prefix+_rank_dispatch (moe.py:13-43, moe_ranked.py:18-65),
 * _dynamic_grouped_gate_up_swiglu / GateUpPlan.run / W4GateUpPlan.run
 *   (moe_fused.py:18-73, cuda_gate_up.cu:167-190, cuda_w4_gate_up.cu:133-151),
 * _dynamic_grouped as down (moe.py:69-95, 209-210),
 * _combine (moe.py:109-121). */
int b200moe_router(B200MoePlan* plan, void* cuda_stream);
int b200moe_dispatch(B200MoePlan* plan, void* cuda_stream);
int b200moe_gate_up(B200MoePlan* plan, void* cuda_stream);
int b200moe_down(B200MoePlan* plan, void* cuda_stream);
int b200moe_combine(B200MoePlan* plan, void* cuda_stream);

/* Arguments of b200moe_dispatch_static(): the tensors of the dispatch stage as
 * plain device pointers. Inputs: x [T,H] bf16, ids [T,K] int32/int64,
 * routing_weights [T,K] float32. Outputs (caller-owned device memory):
 * counts/offsets/cursors [E] int32, tasks [E+1] int32, ranks/mapping [T*K] int32,
 * grouped_input [T*K,H] bf16, status [1] int32. */
typedef struct {
  int32_t tokens, experts, topk, hidden;
  int32_t ids_are_int64;
  int32_t token_tile; /* rows of one expert per tile, for the `tasks` prefix (> 0) */
  const void* x;
  const void* ids;
  const void* routing_weights;
  void* counts;
  void* offsets;
  void* cursors;
  void* tasks;
  void* ranks;
  void* mapping;
  void* grouped_input;
  void* status;
} B200MoeDispatchArgs;

/* Most routes (T*K) b200moe_dispatch_static() accepts. */
#define B200MOE_STATIC_DISPATCH_MAX_ROUTES 65536

/* Ranked dispatch for callers that must not allocate device memory. This entry
 * point has no counterpart in the reference project. It is for hosts that
 * embed the library where cudaMalloc is off limits once the process is
 * running: inside another framework's memory pool, in a real-time loop, or
 * behind a plug-in interface that hands out only the input and output buffers.
 * It gives the same counts / offsets / tasks / ranks / mapping / grouped_input /
 * status as b200moe_dispatch(), but needs no plan and no workspace from the
 * caller: the partition histograms of the counting kernels live in one
 * fixed array inside the library (about 0.5 MiB of device memory on every GPU
 * that loads the library, held until the process exits). Limits and rules:
 *  - T*K <= B200MOE_STATIC_DISPATCH_MAX_ROUTES, E <= 256, K <= 32; larger sizes are
 *    refused with B200MOE_ERR_INVALID, nothing is launched.
 *  - The first call on each device looks up the device address of that array
 *    (on the device that is current at the call); make that first call outside
 *    any stream capture. Later calls only enqueue three kernels and one
 *    4-byte memset on `cuda_stream`.
 *  - All calls on a device share the array: two calls that can overlap on the
 *    GPU (different streams, no dependency) race. Order them on one stream or
 *    with events. Nothing needs to be cleared by the caller between calls.
 *  - It calls no cudaMalloc / cudaFree or other allocating routine. */
int b200moe_dispatch_static(const B200MoeDispatchArgs* args, void* cuda_stream);

/* ---- expert parallelism over peer memory (no counterpart in the single-GPU reference) ----
 * Ranks of one node, one process per GPU. Rank r owns experts [r*E/G, (r+1)*E/G) and a slice of the
 * tokens. The buffers named *_peers are allocated with b200moe_peer_alloc() on every rank and opened on
 * the others with b200moe_peer_export()/import(): entry g is the address of rank g's buffer as seen
 * from this process (entry `rank` is the local one). Rows cross NVLink by plain stores from the
 * dispatch / return kernels; nothing is staged and the host never reads a count. */
#define B200MOE_EP_MAX_RANKS 8

typedef struct {
  int32_t rank, world;            /* 1 <= world <= 8, experts % world == 0 */
  int32_t experts, topk, hidden;  /* global E, K, H */
  int32_t tokens;                 /* tokens of this rank */
  int32_t capacity;               /* rows each rank's receive buffer holds */
  int32_t token_tile;             /* tile of the expert plan (for its `tasks` prefix) */
  int32_t ids_are_int64;
  int32_t fused_return;           /* 1: the expert plan's down projection returns the rows itself (ep_row_dest bound):
                                     b200moe_ep_return_rows then only runs the closing barrier */
  int32_t reserved[2];
  /* token-owning side (local) */
  const void* x;                  /* [tokens,H] bf16 */
  const void* ids;                /* [tokens,K] */
  const void* ranks;              /* [tokens*K] int32, from the route-only plan's dispatch */
  const void* counts;             /* [E] int32, from the route-only plan's dispatch */
  /* expert-owning side (local): metadata of the external_dispatch plan, written here */
  void* expert_counts;            /* [E/G] int32 */
  void* expert_offsets;           /* [E/G] int32 */
  void* expert_tasks;             /* [E/G+1] int32 */
  void* expert_rows;              /* [1] int32: rows received this forward */
  const void* expert_output;      /* [capacity,H] bf16: down_output of the expert plan, grouped order */
  void* tables;                   /* local int32 scratch: b200moe_ep_table_ints() entries */
  void* status;                   /* [1] int32 status word of the token plan */
  /* peer-visible buffers, one address per rank */
  void* recv_rows_peers[B200MOE_EP_MAX_RANKS];   /* [capacity,H] bf16: grouped_input of the expert plan */
  void* return_rows_peers[B200MOE_EP_MAX_RANKS]; /* [tokens*K,H] bf16: down_output of the token plan */
  void* all_counts_peers[B200MOE_EP_MAX_RANKS];  /* [G,E] int32 */
  void* flags_peers[B200MOE_EP_MAX_RANKS];       /* [4*8] int32 barrier flags + [4] local epochs */
  /* chain words of an expert plan created with external_dispatch = 2 (b200moe_plan_chain), zeroed by
   * b200moe_ep_exchange_counts every forward; NULL / 0 for external_dispatch = 1 */
  void* expert_chain;
  int32_t expert_chain_words;
  int32_t reserved2;
  void* expert_status;            /* [1] int32 status word of the expert plan, restarted by the count exchange every
                                     forward (that plan has no dispatch of its own to do it); may be NULL */
  const void* mapping;            /* [tokens*K] int32 of the route-only plan: where each route's result row belongs in
                                     this rank's return buffer; sent along with the row when row_dest_peers is set */
  void* row_dest_peers[B200MOE_EP_MAX_RANKS];    /* [capacity] int32 per rank (ep_row_dest of its expert plan), or NULL */
} B200MoeEpArgs;

/* The int32 words (inside the bound `scratch` buffer) through which the two GEMM kernels of one forward
 * synchronise: a tile counter and one completion counter per expert. An ordinary plan's dispatch zeroes
 * them; for external_dispatch = 2 the caller must, before every forward. No reference counterpart. */
int b200moe_plan_chain(B200MoePlan* plan, void** first_word, int32_t* words);

/* int32 entries of B200MoeEpArgs.tables for a given world / experts. */
size_t b200moe_ep_table_ints(int32_t world, int32_t experts);

/* cudaMalloc'd, zeroed device memory that other processes of the node may open. */
int b200moe_peer_alloc(size_t bytes, void** ptr);
int b200moe_peer_free(void* ptr);
int b200moe_peer_export(void* ptr, unsigned char handle[64]);
int b200moe_peer_import(const unsigned char handle[64], void** ptr);
int b200moe_peer_close(void* ptr);

/* Step 1: publish this rank's per-expert counts to every rank, wait for everyone's, then build the
 * expert plan's counts / offsets / tasks and the send / return address tables. */
int b200moe_ep_exchange_counts(const B200MoeEpArgs* args, void* cuda_stream);
/* Step 2: copy every local route's token row straight into its expert owner's receive buffer, at its
 * final grouped position; returns after all ranks' rows have landed (device-side barrier). */
int b200moe_ep_send_rows(const B200MoeEpArgs* args, void* cuda_stream);
/* Step 3 (after the expert plan's gate_up + down): copy every result row straight into the
 * token owner's return buffer at the route's grouped position; barrier; the owner then combines. */
int b200moe_ep_return_rows(const B200MoeEpArgs* args, void* cuda_stream);

void b200moe_plan_destroy(B200MoePlan* plan);

#ifdef __cplusplus
}
#endif
#endif /* B200MOE_H_ */
