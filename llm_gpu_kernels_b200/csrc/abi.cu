// C ABI of the MoE-layer forward: plan life cycle, argument validation, TMA
// descriptor encoding, and the launch sequence. See include/b200moe.h.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <new>
#include "plan.h"

namespace b200moe {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

namespace {

int round_up(int v, int m) { return (v + m - 1) / m * m; }
size_t align256(size_t v) { return (v + 255) / 256 * 256; }

bool is_w4(int format) { return format == B200MOE_WEIGHTS_W4G128; }

bool tc_shape_ok(const B200MoeShape& s) {
  if (is_w4(s.gate_up_format) && s.hidden % 128) return false;    // one scale per 128 along K
  if (is_w4(s.down_format) && s.intermediate % 128) return false;
  return s.hidden % 8 == 0 && s.intermediate % 8 == 0 && s.hidden >= 64 && s.intermediate >= 64;
}

int auto_token_tile(long long routes, int experts) {
  // twice the mean rows per expert, as a power of two in [16,128]; 256 (one TMEM accumulator set, no
  // epilogue overlap, but half the weight re-reads) once an expert averages 1024 rows or more
  const long long twice_mu = (2 * routes + experts - 1) / experts;
  if (twice_mu >= 2048) return 256;
  int tile = 16;
  while (tile < 128 && tile < twice_mu) tile <<= 1;
  return tile;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// Packed int4 weights as a 2-D int32 tensor [rows, words_per_row]; box = 32 words (256 nibbles, 128 bytes)
// x 128 rows, 128-byte swizzle (whole 128-byte rows keep HBM reads efficient; the swizzle keeps the
// converters' shared-memory reads conflict-free).
int encode_words(CUtensorMap* map, const void* base, uint64_t rows, uint64_t words_per_row) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) {
    set_error("cuTensorMapEncodeTiled is not available from this driver");
    return B200MOE_ERR_CUDA;
  }
  const cuuint64_t dims[2] = {words_per_row, rows};
  const cuuint64_t strides[1] = {words_per_row * 4};
  const cuuint32_t box[2] = {32, 128};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_INT32, 2, const_cast<void*>(base), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled (packed words) failed with CUresult %d", static_cast<int>(r));
    return B200MOE_ERR_CUDA;
  }
  return B200MOE_OK;
}

// 2-D BF16 row-major [rows, cols] tensor, box = 64 columns x box_rows, 128-byte swizzle.
int encode_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows, bool weights) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) {
    set_error("cuTensorMapEncodeTiled is not available from this driver");
    return B200MOE_ERR_CUDA;
  }
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * 2};
  const cuuint32_t box[2] = {64, box_rows};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        weights ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B : CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with CUresult %d (rows=%llu cols=%llu box_rows=%u)", static_cast<int>(r),
              static_cast<unsigned long long>(rows), static_cast<unsigned long long>(cols), box_rows);
    return B200MOE_ERR_CUDA;
  }
  return B200MOE_OK;
}

int check_cuda(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return B200MOE_OK;
  set_error("%s: %s", what, cudaGetErrorString(e));
  return B200MOE_ERR_CUDA;
}

int require_bound(const B200MoePlan* p) {
  if (!p) {
    set_error("null plan");
    return B200MOE_ERR_INVALID;
  }
  if (!p->bound) {
    set_error("plan has no buffers bound; call b200moe_plan_bind first");
    return B200MOE_ERR_STATE;
  }
  return B200MOE_OK;
}

}  // namespace
}  // namespace b200moe

using namespace b200moe;

extern "C" {

int b200moe_abi_version(void) { return B200MOE_ABI_VERSION; }

const char* b200moe_last_error(void) { return g_error; }

int b200moe_plan_create(const B200MoeShape* shape, B200MoePlan** out) {
  if (!shape || !out) {
    set_error("null argument");
    return B200MOE_ERR_INVALID;
  }
  const B200MoeShape& s = *shape;
  if (s.tokens < 0 || s.experts < 1 || s.experts > 256 || s.hidden <= 0 || s.intermediate <= 0) {
    set_error("invalid MoE shape; requires T >= 0, E in [1,256], H/I positive");
    return B200MOE_ERR_INVALID;
  }
  if (s.topk < 1 || s.topk > 32) {
    set_error("expected IDs[T,topk<=32]: topk=%d", s.topk);
    return B200MOE_ERR_INVALID;
  }
  const long long r = static_cast<long long>(s.tokens) * s.topk;
  const long long widest = s.hidden > 2 * s.intermediate ? s.hidden : 2LL * s.intermediate;
  if (r >= (1LL << 31) || r * widest >= (1LL << 31)) {
    set_error("routed/intermediate elements must stay below 2**31 (R=%lld)", r);
    return B200MOE_ERR_INVALID;
  }
  if (s.use_router && s.topk > s.experts) {
    set_error("router needs topk <= experts");
    return B200MOE_ERR_INVALID;
  }
  if (s.use_router && router_smem_bytes(s.hidden, s.experts) > 227 * 1024) {
    set_error("router: hidden=%d does not fit the shared-memory staging", s.hidden);
    return B200MOE_ERR_UNSUPPORTED;
  }
  for (int f : {s.gate_up_format, s.down_format}) {
    if (f != B200MOE_WEIGHTS_BF16 && f != B200MOE_WEIGHTS_W4G128) {
      set_error("unknown weight format %d", f);
      return B200MOE_ERR_INVALID;
    }
  }
  const bool any_w4 = is_w4(s.gate_up_format) || is_w4(s.down_format);
  if (any_w4 && (s.schedule == B200MOE_SCHEDULE_GENERIC || !tc_shape_ok(s))) {
    set_error("W4G128 weights need the tcgen05 schedule: K a multiple of 128 (H=%d for gate/up, I=%d for down), "
              "H and I multiples of 8", s.hidden, s.intermediate);
    return B200MOE_ERR_UNSUPPORTED;
  }
  int schedule = s.schedule;
  if (schedule == B200MOE_SCHEDULE_AUTO) schedule = tc_shape_ok(s) ? B200MOE_SCHEDULE_TCGEN05 : B200MOE_SCHEDULE_GENERIC;
  if (schedule != B200MOE_SCHEDULE_GENERIC && schedule != B200MOE_SCHEDULE_TCGEN05) {
    set_error("unknown schedule %d", s.schedule);
    return B200MOE_ERR_INVALID;
  }
  if (schedule == B200MOE_SCHEDULE_TCGEN05 && !tc_shape_ok(s)) {
    set_error("tcgen05 schedule needs H and I multiples of 8 and >= 64 (H=%d I=%d)", s.hidden,
              s.intermediate);
    return B200MOE_ERR_UNSUPPORTED;
  }
  int tile = s.token_tile;
  if (schedule == B200MOE_SCHEDULE_GENERIC) {
    if (tile != 0 && tile != kGenericTile) {
      set_error("the generic schedule uses token_tile %d", kGenericTile);
      return B200MOE_ERR_INVALID;
    }
    tile = kGenericTile;
  } else if (tile == 0) {
    tile = auto_token_tile(r, s.experts);
    // both projections W4: the weight-streaming kernel (dequantisation in registers) serves 16 rows per tile and
    // beats the tensor-memory variant at its tile 32; the few experts above 16 rows take a second tile
    if (tile == 32 && is_w4(s.gate_up_format) && is_w4(s.down_format)) tile = 16;
  } else if (tile != 16 && tile != 32 && tile != 64 && tile != 128 && tile != 256) {
    set_error("token_tile must be one of 16, 32, 64, 128, 256");
    return B200MOE_ERR_INVALID;
  }
  B200MoePlan* p = new (std::nothrow) B200MoePlan();
  if (!p) {
    set_error("out of host memory");
    return B200MOE_ERR_INVALID;
  }
  p->shape = s;
  p->routes = static_cast<int>(r);
  p->schedule = schedule;
  p->token_tile = tile;
  p->dispatch_fused = r <= static_cast<long long>(kFusedRoutes) * kFusedCluster;
  if (p->dispatch_fused) {  // the 32 warps of each block of a cluster share the routes
    p->dispatch_ctas = 1;   // 1, 2, 4 or 8
    while (static_cast<long long>(p->dispatch_ctas) * kFusedRoutes < r) p->dispatch_ctas *= 2;
    const int warps = 32 * p->dispatch_ctas;
    const int per_warp = round_up(static_cast<int>((r + warps - 1) / warps), 32);
    p->warp_routes = per_warp < 32 ? 32 : per_warp;
    p->partitions = warps;
  } else {
    const int per_warp = round_up(static_cast<int>((r + 511) / 512), 32);
    p->warp_routes = per_warp < 128 ? 128 : per_warp;
    p->partitions = static_cast<int>((r + p->warp_routes - 1) / p->warp_routes);
  }
  const int blocks = (p->partitions + kDispatchWarps - 1) / kDispatchWarps;
  p->chain_words = 1 + s.experts;
  // Down projection over pair tiles once an expert averages more than one token tile (shape-only): below that every
  // weight tile is fetched once anyway and the finer 128-channel tiles balance the SMs better.
  if (s.fused_gather < 0 || s.fused_gather > 2) {
    delete p;
    set_error("fused_gather must be 0 (materialise grouped_input), 1 (gather where it is faster) or 2 (wherever possible)");
    return B200MOE_ERR_INVALID;
  }
  if (s.down_tiles < 0 || s.down_tiles > 3) {
    delete p;
    set_error("down_tiles must be 0 (shape-only choice), 1 (pair tiles), 2 (128-channel tiles) or 3 (wide tiles)");
    return B200MOE_ERR_INVALID;
  }
  // BF16 tensor-core down projection. Pair tiles wherever two accumulator sets of two tiles fit (token tile <= 128):
  // fewer, longer tiles and no partial sums; forward 143.0 / 197.7 / 232.9 us against 145.0 / 200.0 / 240.2 us with
  // 128-channel tiles at 17 / 193 / 1024 tokens of the Qwen3 shape. Wide tiles (the down kernel re-tiles at 256 rows,
  // one issuer, two 256-column accumulators, while gate/up keeps token tile 128) are an explicit option only: alone
  // the down stage gains (106.8 / 172.7 / 257.2 us against 116.0 / 182.5 / 308.4 us with pair tiles at 2048 / 4096 /
  // 8192 tokens, half the passes over an expert's weights), inside a forward it does not (334.2 / 504.7 / 870.9 us
  // against 330.3 / 508.0 / 871.7 us): there the activated rows are still in L2 and sharing them between two
  // channel tiles, which is what pair tiles do, is worth as much.
  p->down_tile = tile;
  if (schedule == B200MOE_SCHEDULE_TCGEN05 && !is_w4(s.down_format) && !s.route_only) {
    if (s.down_tiles == 3 && tile != 128) {
      delete p;
      set_error("down_tiles = 3 (wide tiles) needs token tile 128 (resolved token tile: %d)", tile);
      return B200MOE_ERR_INVALID;
    }
    if (s.down_tiles == 3)
      p->down_tiles = 3;
    else if (tile <= 128 && s.down_tiles != 2)
      p->down_tiles = 1;
    else
      p->down_tiles = 2;
    if (p->down_tiles == 3) p->down_tile = 256;
  }
  p->down_pair = p->down_tiles == 1;
  // gathering gate/up: the BF16 tensor-core kernel, or the W4 weight-streaming kernel (token tile 16). Past about
  // three 128-row tiles per expert the kernel is bound by operand latency out of L2, the cp.async gather answers later
  // than a TMA box load and costs more than the row copy it saves (Qwen3 shape, forward with / without gather:
  // 350 / 359 us at 2048 tokens, 506 / 511 at 4096, 898 / 891 at 8192), so fused_gather = 1 stops there;
  // fused_gather = 2 gathers regardless.
  p->gather = s.fused_gather && schedule == B200MOE_SCHEDULE_TCGEN05 && !s.route_only && !s.external_dispatch &&
              r > 0 && (!is_w4(s.gate_up_format) || tile <= 16) &&
              (s.fused_gather == 2 || r <= static_cast<long long>(s.experts) * 384);

  B200MoeWorkspace& w = p->ws;
  const size_t T = s.tokens, H = s.hidden, I = s.intermediate, E = s.experts, R = r;
  w.output = T * H * 2;
  w.counts = E * 4;
  w.offsets = E * 4;
  w.cursors = E * 4;
  w.tasks = (E + 1) * 4;
  w.mapping = R * 4;
  w.ranks = R * 4;
  w.grouped_input = R * H * 2;
  w.activated = s.route_only ? 0 : R * I * 2;
  w.down_output = R * H * 2;
  w.status = 4;
  w.scratch = align256((static_cast<size_t>(p->partitions) * E + blocks + 2 + E) * 4);
  w.source_rows = p->gather ? R * 4 : 0;
  w.gathers = p->gather ? 1 : 0;
  w.down_tiles = p->down_tiles;
  if (p->gather) w.grouped_input = 0;
  w.token_tile = tile;
  w.schedule = schedule;
  w.launches = s.tokens == 0 ? 0 : (s.use_router ? 1 : 0) + (p->dispatch_fused ? 2 : 3) + (s.route_only ? 0 : 3);
  if (s.route_only == 2) w.launches -= 1;            // no row copy
  if (p->gather && p->dispatch_fused) w.launches -= 1;  // no row copy kernel
  if (s.external_dispatch) w.launches = s.tokens == 0 ? 0 : 2;  // gate_up + down only
  *out = p;
  return B200MOE_OK;
}

int b200moe_plan_workspace(const B200MoePlan* plan, B200MoeWorkspace* sizes) {
  if (!plan || !sizes) {
    set_error("null argument");
    return B200MOE_ERR_INVALID;
  }
  *sizes = plan->ws;
  return B200MOE_OK;
}

int b200moe_plan_bind(B200MoePlan* p, const B200MoeBuffers* b) {
  if (!p || !b) {
    set_error("null argument");
    return B200MOE_ERR_INVALID;
  }
  p->bound = false;
  const B200MoeShape& s = p->shape;
  int rc = check_cuda(cudaGetDevice(&p->device), "cudaGetDevice");
  if (rc) return rc;
  int major = 0;
  rc = check_cuda(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, p->device), "device attribute");
  if (rc) return rc;
  rc = check_cuda(cudaDeviceGetAttribute(&p->num_sms, cudaDevAttrMultiProcessorCount, p->device), "device attribute");
  if (rc) return rc;
  if (major != 10) {
    set_error("this library is built for sm_100a only; device %d has compute capability major %d", p->device, major);
    return B200MOE_ERR_UNSUPPORTED;
  }
  if (s.tokens > 0) {
    if (!s.route_only && (!b->gate_up || !b->down || !b->activated)) {
      set_error("gate_up, down and activated buffers are required unless the plan is route_only");
      return B200MOE_ERR_INVALID;
    }
    struct Named { const void* ptr; const char* name; };
    const Named always[] = {{b->counts, "counts"}, {b->offsets, "offsets"}, {b->tasks, "tasks"},
                            {b->down_output, "down_output"}, {b->status, "status"}};
    const Named own_dispatch[] = {{b->x, "x"}, {b->ids, "ids"}, {b->routing_weights, "routing_weights"},
                                  {b->output, "output"}, {b->cursors, "cursors"}, {b->mapping, "mapping"},
                                  {b->ranks, "ranks"}, {b->scratch, "scratch"}};
    auto check = [](const Named& n) {
      if (!n.ptr) {
        set_error("buffer '%s' is null", n.name);
        return false;
      }
      if (reinterpret_cast<uintptr_t>(n.ptr) % 4) {
        set_error("buffer '%s' is not 4-byte aligned", n.name);
        return false;
      }
      return true;
    };
    for (const Named& n : always)
      if (!check(n)) return B200MOE_ERR_INVALID;
    if (!s.external_dispatch)
      for (const Named& n : own_dispatch)
        if (!check(n)) return B200MOE_ERR_INVALID;
    if (s.route_only != 2 && !p->gather && !check({b->grouped_input, "grouped_input"})) return B200MOE_ERR_INVALID;
    if (p->gather && !check({b->source_rows, "source_rows"})) return B200MOE_ERR_INVALID;
    if (!s.external_dispatch && s.ids_are_int64 && reinterpret_cast<uintptr_t>(b->ids) % 8) {
      set_error("buffer 'ids' (int64) is not 8-byte aligned");
      return B200MOE_ERR_INVALID;
    }
    if (s.use_router && !b->router_weight) {
      set_error("use_router is set but router_weight is null");
      return B200MOE_ERR_INVALID;
    }
    // the output and the workspace must not alias the inputs (cuda_gate_up.cu:150-158)
    const void* inputs[] = {b->x, b->gate_up, b->down, b->ids, b->routing_weights, b->router_weight, b->residual};
    const void* written[] = {b->output, b->grouped_input, b->activated, b->down_output, b->mapping, b->ranks};
    for (const void* in : inputs)
      for (const void* wr : written)
        if (in && in == wr) {
          set_error("output/workspace buffer aliases an input");
          return B200MOE_ERR_INVALID;
        }
  }
  if (b->ep_row_dest || b->ep_return_bases) {
    if (!b->ep_row_dest || !b->ep_return_bases || !s.external_dispatch || p->schedule != B200MOE_SCHEDULE_TCGEN05 ||
        is_w4(s.down_format)) {
      set_error("ep_row_dest / ep_return_bases go together and need an external_dispatch plan on the BF16 "
                "tensor-core schedule");
      return B200MOE_ERR_INVALID;
    }
    if (reinterpret_cast<uintptr_t>(b->ep_row_dest) % 4 || reinterpret_cast<uintptr_t>(b->ep_return_bases) % 8) {
      set_error("ep_row_dest / ep_return_bases are misaligned");
      return B200MOE_ERR_INVALID;
    }
  }
  p->buf = *b;
  p->router_tc = false;
  if (s.tokens > 0 && s.use_router && p->schedule == B200MOE_SCHEDULE_TCGEN05 &&
      (reinterpret_cast<uintptr_t>(b->x) | reinterpret_cast<uintptr_t>(b->router_weight)) % 16 == 0) {
    const uint32_t e_pad = static_cast<uint32_t>((s.experts + 15) / 16 * 16);
    if ((rc = encode_2d(&p->tm_x, b->x, s.tokens, s.hidden, 128, false))) return rc;
    if ((rc = encode_2d(&p->tm_router_w, b->router_weight, s.experts, s.hidden, e_pad, false))) return rc;
    if ((rc = configure_router_tc(*p))) return rc;
    p->router_tc = true;
  } else if (s.tokens > 0 && s.use_router) {
    if (router_smem_bytes(s.hidden, s.experts) > 48 * 1024) {
      rc = check_cuda(router_opt_in_smem(), "router shared-memory opt-in");
      if (rc) return rc;
    }
  }
  if (s.tokens > 0 && p->schedule == B200MOE_SCHEDULE_TCGEN05 && !s.route_only) {
    const void* aligned16[] = {b->gate_up, b->down, p->gather ? b->x : b->grouped_input, b->activated};
    for (const void* ptr : aligned16)
      if (reinterpret_cast<uintptr_t>(ptr) % 16) {
        set_error("tcgen05 schedule: weights and workspace rows must be 16-byte aligned");
        return B200MOE_ERR_INVALID;
      }
    const uint64_t E = s.experts, H = s.hidden, I = s.intermediate, R = p->routes;
    if (is_w4(s.gate_up_format)) {
      if (!b->gate_up_scales) {
        set_error("W4G128 gate/up needs gate_up_scales");
        return B200MOE_ERR_INVALID;
      }
      if ((rc = encode_words(&p->tm_gate_up_w, b->gate_up, E * 2 * I, H / 8))) return rc;
    } else if ((rc = encode_2d(&p->tm_gate_up_w, b->gate_up, E * 2 * I, H, 128, true))) {
      return rc;
    }
    if (is_w4(s.down_format)) {
      if (!b->down_scales) {
        set_error("W4G128 down needs down_scales");
        return B200MOE_ERR_INVALID;
      }
      if ((rc = encode_words(&p->tm_down_w, b->down, E * H, I / 8))) return rc;
    } else if ((rc = encode_2d(&p->tm_down_w, b->down, E * H, I, 128, true))) {
      return rc;
    }
    if (!p->gather && (rc = encode_2d(&p->tm_grouped, b->grouped_input, R, H, p->token_tile, false))) return rc;
    if ((rc = encode_2d(&p->tm_activated, b->activated, R, I, p->down_tile, false))) return rc;
    if ((rc = configure_tc(*p))) return rc;
    if ((is_w4(s.gate_up_format) || is_w4(s.down_format)) && (rc = configure_w4(*p))) return rc;
    if ((is_w4(s.gate_up_format) || is_w4(s.down_format)) && p->token_tile <= 64 && (rc = configure_w4t(*p))) return rc;
    if ((is_w4(s.gate_up_format) || is_w4(s.down_format)) && w4r_serves(*p) && (rc = configure_w4r(*p))) return rc;
  }
  p->bound = true;
  return B200MOE_OK;
}

int b200moe_router(B200MoePlan* p, void* stream) {
  int rc = require_bound(p);
  if (rc) return rc;
  if (p->shape.tokens == 0 || !p->shape.use_router) return B200MOE_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return check_cuda(p->router_tc ? launch_router_tc(*p, s) : launch_router(*p, s), "router launch");
}

int b200moe_dispatch(B200MoePlan* p, void* stream) {
  int rc = require_bound(p);
  if (rc) return rc;
  if (p->shape.tokens == 0) return B200MOE_OK;
  if (p->shape.external_dispatch) {
    set_error("an external_dispatch plan receives grouped rows and metadata from outside");
    return B200MOE_ERR_STATE;
  }
  return check_cuda(launch_dispatch(*p, static_cast<cudaStream_t>(stream)), "dispatch launch");
}

// Inside b200moe_forward the two BF16 tensor-core GEMMs are chained through per-expert counters.
static bool w4_in_tmem(const B200MoePlan* p) { return p->token_tile <= 64; }
static bool chain_stages(const B200MoePlan* p) {
  if (p->shape.unchained || p->schedule != B200MOE_SCHEDULE_TCGEN05 || p->shape.external_dispatch == 1 || !p->buf.scratch)
    return false;
  const bool g4 = is_w4(p->shape.gate_up_format), d4 = is_w4(p->shape.down_format);
  return g4 == d4;   // both stages BF16 or both W4 (the two W4 variants are chosen by token tile, the same for both)
}

static int gate_up_stage(B200MoePlan* p, void* stream, bool chained);
static int down_stage(B200MoePlan* p, void* stream, bool chained);

int b200moe_gate_up(B200MoePlan* p, void* stream) { return gate_up_stage(p, stream, false); }
int b200moe_down(B200MoePlan* p, void* stream) { return down_stage(p, stream, false); }

static int gate_up_stage(B200MoePlan* p, void* stream, bool chained) {
  int rc = require_bound(p);
  if (rc) return rc;
  if (p->shape.tokens == 0) return B200MOE_OK;
  if (p->shape.route_only) {
    set_error("a route_only plan has no expert stages");
    return B200MOE_ERR_STATE;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (p->schedule != B200MOE_SCHEDULE_TCGEN05) return check_cuda(launch_gate_up_generic(*p, s), "gate_up launch");
  // W4: up to 16 rows per tile the weights are dequantised in registers (weight-streaming kernel); above, the
  // dequantised operand goes to tensor memory while two accumulator sets still fit beside it (tile <= 64), to
  // shared memory above that
  if (is_w4(p->shape.gate_up_format)) {
    if (w4r_serves(*p)) return check_cuda(launch_gate_up_w4r(*p, s, chained), "gate_up launch");
    return check_cuda(w4_in_tmem(p) ? launch_gate_up_w4t(*p, s, chained) : launch_gate_up_w4(*p, s, chained), "gate_up launch");
  }
  return check_cuda(launch_gate_up_tc(*p, s, chained), "gate_up launch");
}

static int down_stage(B200MoePlan* p, void* stream, bool chained) {
  int rc = require_bound(p);
  if (rc) return rc;
  if (p->shape.tokens == 0) return B200MOE_OK;
  if (p->shape.route_only) {
    set_error("a route_only plan has no expert stages");
    return B200MOE_ERR_STATE;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (p->schedule != B200MOE_SCHEDULE_TCGEN05) return check_cuda(launch_down_generic(*p, s), "down launch");
  if (is_w4(p->shape.down_format)) {
    if (w4r_serves(*p)) return check_cuda(launch_down_w4r(*p, s, chained), "down launch");
    return check_cuda(w4_in_tmem(p) ? launch_down_w4t(*p, s, chained) : launch_down_w4(*p, s, chained), "down launch");
  }
  return check_cuda(launch_down_tc(*p, s, chained), "down launch");
}

int b200moe_combine(B200MoePlan* p, void* stream) {
  int rc = require_bound(p);
  if (rc) return rc;
  if (p->shape.tokens == 0) return B200MOE_OK;
  if (p->shape.external_dispatch) {
    set_error("an external_dispatch plan has no combine stage");
    return B200MOE_ERR_STATE;
  }
  return check_cuda(launch_combine(*p, static_cast<cudaStream_t>(stream)), "combine launch");
}

int b200moe_forward(B200MoePlan* p, void* stream) {
  int rc;
  if (p && p->bound && p->shape.external_dispatch) {
    // external_dispatch = 2: whoever wrote the metadata zeroed the chain words, so the two GEMMs chain
    const bool chained = chain_stages(p);
    if ((rc = gate_up_stage(p, stream, chained))) return rc;
    return down_stage(p, stream, chained);
  }
  if ((rc = b200moe_router(p, stream))) return rc;
  if ((rc = b200moe_dispatch(p, stream))) return rc;
  if (p && p->shape.route_only) return B200MOE_OK;  // experts run elsewhere; the caller combines later
  const bool chained = chain_stages(p);
  if ((rc = gate_up_stage(p, stream, chained))) return rc;
  if ((rc = down_stage(p, stream, chained))) return rc;
  return b200moe_combine(p, stream);
}

int b200moe_plan_chain(B200MoePlan* p, void** first_word, int32_t* words) {
  int rc = require_bound(p);
  if (rc) return rc;
  if (!first_word || !words) {
    set_error("null output pointer");
    return B200MOE_ERR_INVALID;
  }
  if (!p->buf.scratch) {
    set_error("the plan was bound without a scratch buffer");
    return B200MOE_ERR_STATE;
  }
  *first_word = static_cast<int*>(p->buf.scratch) + router_flag_index(*p) + 1;
  *words = p->chain_words;
  return B200MOE_OK;
}

void b200moe_plan_destroy(B200MoePlan* p) { delete p; }

}  // extern "C"
