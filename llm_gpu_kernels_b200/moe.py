"""Prepared MoE layer: fixed buffers and shapes, values change in place.

Host-side mirror of the reference's ``PreparedMoE`` / ``prepare_moe``
(reference moe.py:124-245): same argument order, same validation and error
types, same attribute names for every buffer, the same life cycle (allocate
and run once at prepare, then ``run()`` enqueues kernels on the current stream
with no allocation, no host read and no synchronisation, so it can be captured
in a CUDA graph). The kernels behind it are the sm_100a library reached
through the C ABI of ``include/b200moe.h``; nothing here computes on the host.

Two additions to the reference interface, both keyword-only:
``router_weight`` ([E,H] BF16) puts the top-k softmax router in front of the
fixed-route path - ``ids`` and ``routing_weights`` then are outputs rewritten by
every ``run()``; ``schedule`` / ``token_tile`` pin the shape-only kernel choice.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field

import torch

from . import _native, _ops
from .gemm import GemmConfig

STAGE_NAMES = ("router", "dispatch", "gate_up_swiglu", "down", "combine")
_GATHER = {False: 1, True: 0, "never": 2}   # keep_grouped_input -> B200MoeShape.fused_gather
_SCHEDULES = {None: _native.SCHEDULE_AUTO, "auto": _native.SCHEDULE_AUTO,
              "generic": _native.SCHEDULE_GENERIC, "tcgen05": _native.SCHEDULE_TCGEN05}


def _input(tensor, ndim):
    # reference gemm.py:105-107
    if (not isinstance(tensor, torch.Tensor) or tensor.ndim != ndim or tensor.dtype != torch.bfloat16
            or not tensor.is_cuda or not tensor.is_contiguous()):
        raise ValueError(f"expected contiguous CUDA BF16 tensor with {ndim} dimensions")


@dataclass(frozen=True)
class StageLaunch:
    """One subsystem of the forward; ``run()`` enqueues it on the current stream."""
    name: str
    _call: object = field(repr=False)
    _plan: object = field(repr=False)
    _device: torch.device = field(repr=False)

    def run(self):
        _native.check(self._call(self._plan, torch.cuda.current_stream(self._device).cuda_stream))


@dataclass
class PreparedMoE:
    """Fixed buffers/shapes; runtime ids and values may change in place.

    Attribute names follow reference moe.py:131-149. ``projected`` (the unfused
    [R,2I] gate/up result of the reference) is never materialised here - SwiGLU
    runs on the accumulators - and is kept as an empty tensor for interface
    parity. ``ranks`` and ``scratch`` are this implementation's dispatch workspace.
    Status flags invalid runtime values; ``check_inputs`` is an explicit
    synchronising debug operation, never part of ``run``. The caller orders
    streams and never runs one workspace concurrently (docs/MOE_USAGE.md:95-108).
    """
    x: torch.Tensor
    gate_up: torch.Tensor
    down: torch.Tensor
    ids: torch.Tensor
    routing_weights: torch.Tensor
    output: torch.Tensor
    counts: torch.Tensor
    offsets: torch.Tensor
    cursors: torch.Tensor
    tasks: torch.Tensor
    mapping: torch.Tensor
    grouped_input: torch.Tensor
    projected: torch.Tensor
    activated: torch.Tensor
    down_output: torch.Tensor
    status: torch.Tensor
    config: GemmConfig
    kernels: dict = field(default_factory=dict)
    ranks: torch.Tensor = None
    scratch: torch.Tensor = None
    router_weight: torch.Tensor = None
    gate_up_scales: torch.Tensor = None  # set when gate_up holds packed W4G128 words
    down_scales: torch.Tensor = None     # set when down holds packed W4G128 words
    packed: object = None                # the PackedGateUp the plan was prepared from (reference W4Workspace.packed)
    valid_routes: torch.Tensor = None    # optional device int32: routes beyond it are padding this forward
    residual: torch.Tensor = None        # optional [T,H] bf16 added to the layer result in the combine kernel
    schedule: str = ""
    token_tile: int = 0
    launches: tuple = ()
    kernel_launches: int = 0  # kernels one run() enqueues
    chain: tuple = None       # expert-side plans: (device address, count) of the int32 words the exchange zeroes
    gathers: bool = False     # gate/up gathers token rows through source_rows; grouped_input is empty
    down_pair: bool = False   # the down projection runs over 256-channel pair tiles
    down_tiles: int = 0       # resolved BF16 down schedule: 1 pair, 2 128-channel tiles (two partial sums), 3 wide
                              # (256-row tiles); pass it as ``down_tiles=`` to a plan that must give the same bits
    source_rows: torch.Tensor = None   # [R] int32: the token behind each grouped row (only when gathers)
    fused_return: bool = False  # expert-side plans: the down projection stores result rows into their owners' buffers
    ep_tables: tuple = None
    _plan: object = field(default=None, repr=False)
    _forward: object = field(default=None, repr=False)
    _op_args: tuple = field(default=None, repr=False)

    @property
    def workspace_bytes(self):
        # the tensors reference moe.py:151-155 counts, plus this implementation's scratch
        return sum(t.numel() * t.element_size() for t in
                   (self.counts, self.offsets, self.cursors, self.tasks, self.mapping, self.grouped_input,
                    self.projected, self.activated, self.down_output, self.status, self.scratch)
                   ) + (self.source_rows.numel() * 4 if self.source_rows is not None else 0)

    def check_inputs(self):
        flags = int(self.status.item())
        if flags:
            raise ValueError(f"invalid runtime MoE inputs: GPU status={flags} "
                             "(1=IDs, 2=nonfinite weights, 4=kernel wait timeout)")

    def _stage(self, index):
        if self.launches:
            self.launches[index].run()

    def route(self):
        """Router (only when prepared with ``router_weight``)."""
        self._stage(0)

    def dispatch(self):
        self._stage(1)

    def project(self):
        """Gate/up grouped GEMM with SwiGLU fused (writes ``activated``)."""
        self._stage(2)

    def activate(self):
        """No separate launch: SwiGLU is fused into :meth:`project`."""

    def down_project(self):
        self._stage(3)

    def combine(self):
        self._stage(4)

    def run(self):
        """One forward on the current stream, through the registered PyTorch operator
        ``torch.ops.b200moe.forward`` (a thin wrapper of ``b200moe_forward``), so that graph capture and
        ``torch.compile`` see which tensors the call writes."""
        if self.x.shape[0] == 0:
            return self.output
        if self._op_args is None:
            weights = [t for t in (self.gate_up, self.down, self.router_weight, self.gate_up_scales,
                                   self.down_scales, self.valid_routes, self.residual) if t is not None]
            workspace = [self.counts, self.offsets, self.cursors, self.tasks, self.mapping, self.ranks,
                         self.grouped_input, self.activated, self.down_output, self.status, self.scratch]
            if self.source_rows is not None:
                workspace.append(self.source_rows)
            self._op_args = (self._plan.value, self.x, weights, self.ids, self.routing_weights, self.output, workspace)
            _ops.register_plan(self)
        _ops.forward(*self._op_args)
        return self.output

    def __del__(self):
        plan, self._plan = self._plan, None
        if plan is not None:
            try:
                _native.load().b200moe_plan_destroy(plan)
            except Exception:  # interpreter shutdown
                pass


def _packed_input(words, scales, name):
    """Packed W4G128 operand: int32 words [E,N,K/8] and BF16 scales [E,N,K/128] (reference moe_w4_cuda.py:101-114)."""
    if (not isinstance(words, torch.Tensor) or not isinstance(scales, torch.Tensor) or words.ndim != 3
            or scales.ndim != 3 or words.dtype != torch.int32 or scales.dtype != torch.bfloat16
            or not words.is_cuda or not scales.is_cuda or not words.is_contiguous() or not scales.is_contiguous()
            or words.shape[:2] != scales.shape[:2] or words.shape[2] * 8 != scales.shape[2] * 128):
        raise ValueError(f"{name}: packed shape/dtype mismatch (int32 words [E,N,K/8], BF16 scales [E,N,K/128])")
    if words.data_ptr() % 16:
        raise ValueError("16-byte input alignment required")


def _validate(x, gate_up, down, ids, routing_weights, router_weight, gate_up_scales=None, down_scales=None,
              route_only_experts=None):
    _input(x, 2)
    if route_only_experts is not None:
        # token-owning side of expert parallelism: no expert weights on this plan
        e, h, intermediate = int(route_only_experts), x.shape[1], 64
        gate_up_shape = (e, 2 * intermediate, h)
        gate_up = down = None
    elif gate_up_scales is None:
        _input(gate_up, 3)
        gate_up_shape = tuple(gate_up.shape)
    else:
        _packed_input(gate_up, gate_up_scales, "gate_up")
        gate_up_shape = (gate_up.shape[0], gate_up.shape[1], gate_up.shape[2] * 8)
    if route_only_experts is not None:
        pass
    elif down_scales is None:
        _input(down, 3)
        e, h, intermediate = down.shape
    else:
        _packed_input(down, down_scales, "down")
        e, h, intermediate = down.shape[0], down.shape[1], down.shape[2] * 8
    if (not 0 < e <= 256 or h <= 0 or intermediate <= 0 or x.shape[1] != h
            or gate_up_shape != (e, 2 * intermediate, h)):
        raise ValueError("invalid MoE shape; prototype requires E in [1,256], H/I positive")
    if (not isinstance(ids, torch.Tensor) or not isinstance(routing_weights, torch.Tensor) or ids.ndim != 2
            or ids.dtype not in (torch.int32, torch.int64) or ids.shape[0] != x.shape[0]
            or not 0 < ids.shape[1] <= 32 or routing_weights.shape != ids.shape
            or routing_weights.dtype != torch.float32):
        raise ValueError("expected CUDA IDs[T,topk<=32] and FP32 weights of identical shape")
    extra = [t for t in (gate_up_scales, down_scales) if t is not None]
    weights = [t for t in (gate_up, down) if t is not None]
    if any(t.device != x.device or not t.is_contiguous() for t in (*weights, ids, routing_weights, *extra)):
        raise ValueError("all MoE tensors must be contiguous and on the same CUDA device")
    r = ids.numel()
    if r >= 2**31 or r * max(h, 2 * intermediate) >= 2**31:
        raise ValueError("prototype vector indexing requires routed/intermediate elements < 2**31")
    if router_weight is not None:
        _input(router_weight, 2)
        if tuple(router_weight.shape) != (e, h) or router_weight.device != x.device:
            raise ValueError("router_weight must be [E,H] BF16 on the same device")
        if ids.shape[1] > e:
            raise ValueError("router needs topk <= experts")
    return e, h, intermediate


def _prepare(x, gate_up, down, ids, routing_weights, *, router_weight=None, schedule=None,
             token_tile=0, config=None, warm=True, gate_up_scales=None, down_scales=None,
             route_only_experts=None, valid_routes=None, copy_rows=True, workspace=None,
             router_bf16_weights=False, residual=None, unchained=False, keep_grouped_input=False, down_pair=None,
             down_tiles=None):
    """Validate, allocate the workspace, bind the native plan, run one forward.

    With ``gate_up_scales`` / ``down_scales`` the matching weight argument is the packed
    W4G128 int32 word tensor instead of a BF16 tensor. Unless ``keep_grouped_input`` is set, a plan whose
    gate/up kernel can gather token rows itself does not materialise ``grouped_input`` (it stays an empty
    tensor): the dispatch then writes ``source_rows`` (grouped row -> token) instead of copying rows.
    ``keep_grouped_input``: False = the library decides by shape (it gathers until experts average more than three
    128-row tiles), True = always materialise, "never" = gather whenever the kernels can.
    """
    if keep_grouped_input not in _GATHER:
        raise ValueError('keep_grouped_input must be False, True or "never"')
    e, h, intermediate = _validate(x, gate_up, down, ids, routing_weights, router_weight, gate_up_scales,
                                   down_scales, route_only_experts)
    if valid_routes is not None and (valid_routes.dtype != torch.int32 or valid_routes.numel() != 1
                                     or valid_routes.device != x.device):
        raise ValueError("valid_routes must be one int32 on the same device")
    if schedule not in _SCHEDULES:
        raise ValueError(f"unknown schedule {schedule!r}; expected one of auto/generic/tcgen05")
    if residual is not None and (residual.dtype != torch.bfloat16 or residual.shape != x.shape
                                 or residual.device != x.device or not residual.is_contiguous()):
        raise ValueError("residual must be a contiguous bfloat16 tensor of the shape and device of x")
    lib = _native.load()
    tokens = x.shape[0]
    topk = ids.shape[1]
    shape = _native.Shape(tokens=tokens, experts=e, topk=topk, hidden=h, intermediate=intermediate,
                          ids_are_int64=int(ids.dtype == torch.int64),
                          gate_up_format=_native.WEIGHTS_BF16 if gate_up_scales is None else _native.WEIGHTS_W4G128,
                          down_format=_native.WEIGHTS_BF16 if down_scales is None else _native.WEIGHTS_W4G128,
                          schedule=_SCHEDULES[schedule], token_tile=int(token_tile),
                          use_router=int(router_weight is not None),
                          route_only=0 if route_only_experts is None else (1 if copy_rows else 2),
                          router_bf16_weights=int(bool(router_bf16_weights)), unchained=int(bool(unchained)),
                          fused_gather=_GATHER[keep_grouped_input],
                          down_tiles=int(down_tiles) if down_tiles is not None
                          else (0 if down_pair is None else (1 if down_pair else 2)))
    handle = ctypes.c_void_p()
    _native.check(lib.b200moe_plan_create(ctypes.byref(shape), ctypes.byref(handle)))
    try:
        sizes = _native.Workspace()
        _native.check(lib.b200moe_plan_workspace(handle, ctypes.byref(sizes)))
        device = x.device
        r = ids.numel()
        bf16 = lambda shp: torch.empty(shp, device=device, dtype=torch.bfloat16)
        int32 = lambda shp: torch.zeros(shp, device=device, dtype=torch.int32)
        config = config if config is not None else GemmConfig(block_m=max(16, sizes.token_tile))
        plan = PreparedMoE(
            x, gate_up, down, ids, routing_weights, bf16((tokens, h)),
            int32((e,)), int32((e,)), int32((e,)), int32((e + 1,)), int32((r,)),
            bf16((0 if sizes.gathers else r, h)), bf16((0, 2 * intermediate)),
            bf16((0 if route_only_experts is not None else r, intermediate)), bf16((r, h)),
            int32((1,)), config,
            ranks=int32((r,)), scratch=int32((max(1, sizes.scratch // 4),)), router_weight=router_weight,
            schedule=_native.SCHEDULE_NAMES[sizes.schedule], token_tile=sizes.token_tile,
            kernel_launches=sizes.launches, gate_up_scales=gate_up_scales, down_scales=down_scales,
            valid_routes=valid_routes, residual=residual, gathers=bool(sizes.gathers), down_pair=sizes.down_tiles == 1,
            down_tiles=sizes.down_tiles,
            source_rows=int32((r,)) if sizes.gathers else None)
        for name, tensor in (workspace or {}).items():  # caller-provided workspace (peer-visible buffers)
            if tuple(tensor.shape) != tuple(getattr(plan, name).shape) or tensor.dtype != getattr(plan, name).dtype:
                raise ValueError(f"workspace override {name} has the wrong shape or dtype")
            setattr(plan, name, tensor)
        expected = {"output": plan.output, "counts": plan.counts, "offsets": plan.offsets,
                    "cursors": plan.cursors, "tasks": plan.tasks, "mapping": plan.mapping, "ranks": plan.ranks,
                    "grouped_input": plan.grouped_input, "activated": plan.activated,
                    "down_output": plan.down_output, "status": plan.status, "scratch": plan.scratch}
        for name, tensor in expected.items():
            if tensor.numel() * tensor.element_size() < getattr(sizes, name):
                raise RuntimeError(f"workspace buffer {name} smaller than the library requires")
        if sizes.gathers and plan.source_rows.numel() * 4 < sizes.source_rows:
            raise RuntimeError("workspace buffer source_rows smaller than the library requires")
        ptr = lambda t: ctypes.c_void_p(t.data_ptr()) if t is not None and t.numel() else None
        buffers = _native.Buffers(
            x=ptr(x), router_weight=ptr(router_weight), gate_up=ptr(gate_up), gate_up_scales=ptr(gate_up_scales),
            down=ptr(down), down_scales=ptr(down_scales), ids=ptr(ids), routing_weights=ptr(routing_weights),
            valid_routes=ptr(valid_routes), residual=ptr(residual), source_rows=ptr(plan.source_rows),
            **{name: ptr(tensor) for name, tensor in expected.items()})
        with torch.cuda.device(device):
            _native.check(lib.b200moe_plan_bind(handle, ctypes.byref(buffers)))
    except Exception:
        lib.b200moe_plan_destroy(handle)
        raise
    plan._plan = handle
    plan._forward = lib.b200moe_forward
    if tokens:
        calls = (lib.b200moe_router, lib.b200moe_dispatch, lib.b200moe_gate_up, lib.b200moe_down,
                 lib.b200moe_combine)
        plan.launches = tuple(StageLaunch(name, call, handle, device) for name, call in zip(STAGE_NAMES, calls))
        plan.kernels = {name: plan.schedule for name in STAGE_NAMES}
    if warm:
        # populate metadata before any capture; no device value validation here (reference moe.py:243-244)
        plan.run()
    return plan


def prepare_moe(x, gate_up, down, ids, routing_weights, *, router_weight=None, schedule=None, token_tile=0,
                router_bf16_weights=False, residual=None, keep_grouped_input=False, down_pair=None, down_tiles=None):
    """Drop-in for reference ``prepare_moe`` (moe.py:220-245). ``router_bf16_weights`` makes the router round
    its weights through BF16 like the captured model does (scripts/capture_qwen3_moe_layer0.py:587-588).
    ``residual`` ([T,H] bf16, read every forward) is added to the layer result inside the combine kernel:
    ``output = bf16(residual + bf16(layer))``, the model's residual add without a round trip through HBM.
    ``keep_grouped_input=True`` makes every forward fill the ``grouped_input`` workspace tensor as the reference's
    dispatch does; by default the gate/up kernel reads the token rows through ``source_rows`` where that is
    faster (until experts average more than three 128-row tiles); ``"never"`` gathers whenever the kernels can.
    ``down_pair`` / ``down_tiles`` pin the tile schedule of the BF16 down projection (None = shape-only choice;
    ``down_tiles`` 1 = pair tiles, 2 = 128-channel tiles with two partial sums over K, 3 = wide 256-row tiles, as
    ``PreparedMoE.down_tiles`` reports): plans that must agree to the bit pin the same one."""
    return _prepare(x, gate_up, down, ids, routing_weights, router_weight=router_weight, schedule=schedule,
                    token_tile=token_tile, router_bf16_weights=router_bf16_weights, residual=residual,
                    keep_grouped_input=keep_grouped_input, down_pair=down_pair, down_tiles=down_tiles)


def _prepare_expert_side(gate_up, down, grouped_input, *, token_tile, gate_up_scales=None, down_scales=None,
                         row_dest=None, return_bases=None):
    """Plan for the expert-owning side of expert parallelism: rows arrive already grouped by expert in
    ``grouped_input`` ([capacity,H], written by other ranks) and counts / offsets / tasks are written by the
    exchange kernels; the plan runs gate_up + down only (``launches[2]`` and ``launches[3]``). The exchange also
    zeroes the plan's chain words (``plan.chain``: address and count) every forward, which lets the two BF16
    GEMM kernels overlap as they do in an ordinary plan. ``row_dest`` ([capacity] int32, written by the senders)
    and ``return_bases`` (int64 device tensor, one address per rank) make the down projection store every result
    row straight into its token owner's buffer; ``plan.fused_return`` says whether the plan took them (BF16
    tensor-core schedule only)."""
    capacity, h = grouped_input.shape
    device = grouped_input.device
    dummy_x = grouped_input  # only shapes are taken from it
    ids = torch.zeros((capacity, 1), dtype=torch.int32, device=device)
    rw = torch.ones((capacity, 1), dtype=torch.float32, device=device)
    e, h2, intermediate = _validate(dummy_x, gate_up, down, ids, rw, None, gate_up_scales, down_scales)
    lib = _native.load()
    shape = _native.Shape(tokens=capacity, experts=e, topk=1, hidden=h, intermediate=intermediate,
                          gate_up_format=_native.WEIGHTS_BF16 if gate_up_scales is None else _native.WEIGHTS_W4G128,
                          down_format=_native.WEIGHTS_BF16 if down_scales is None else _native.WEIGHTS_W4G128,
                          schedule=_native.SCHEDULE_AUTO, token_tile=int(token_tile), external_dispatch=2)
    handle = ctypes.c_void_p()
    _native.check(lib.b200moe_plan_create(ctypes.byref(shape), ctypes.byref(handle)))
    try:
        sizes = _native.Workspace()
        _native.check(lib.b200moe_plan_workspace(handle, ctypes.byref(sizes)))
        bf16 = lambda shp: torch.empty(shp, device=device, dtype=torch.bfloat16)
        int32 = lambda shp: torch.zeros(shp, device=device, dtype=torch.int32)
        plan = PreparedMoE(
            None, gate_up, down, None, None, None, int32((e,)), int32((e,)), int32((e,)), int32((e + 1,)), None,
            grouped_input, bf16((0, 2 * intermediate)), bf16((capacity, intermediate)), bf16((capacity, h)),
            int32((1,)), GemmConfig(block_m=max(16, sizes.token_tile)),
            schedule=_native.SCHEDULE_NAMES[sizes.schedule], token_tile=sizes.token_tile,
            kernel_launches=sizes.launches, gate_up_scales=gate_up_scales, down_scales=down_scales,
            down_pair=sizes.down_tiles == 1, down_tiles=sizes.down_tiles)
        ptr = lambda t: ctypes.c_void_p(t.data_ptr()) if t is not None and t.numel() else None
        buffers = _native.Buffers(
            gate_up=ptr(gate_up), gate_up_scales=ptr(gate_up_scales), down=ptr(down), down_scales=ptr(down_scales),
            counts=ptr(plan.counts), offsets=ptr(plan.offsets), cursors=ptr(plan.cursors), tasks=ptr(plan.tasks),
            grouped_input=ptr(grouped_input), activated=ptr(plan.activated), down_output=ptr(plan.down_output),
            status=ptr(plan.status))
        plan.scratch = int32((max(1, sizes.scratch // 4),))
        buffers.scratch = ptr(plan.scratch)
        plan.fused_return = (row_dest is not None and return_bases is not None and down_scales is None
                             and sizes.schedule == _native.SCHEDULE_TCGEN05)
        if plan.fused_return:
            buffers.ep_row_dest, buffers.ep_return_bases = ptr(row_dest), ptr(return_bases)
            plan.ep_tables = (row_dest, return_bases)   # keep alive
        with torch.cuda.device(device):
            _native.check(lib.b200moe_plan_bind(handle, ctypes.byref(buffers)))
        first, words = ctypes.c_void_p(), ctypes.c_int32()
        _native.check(lib.b200moe_plan_chain(handle, ctypes.byref(first), ctypes.byref(words)))
        plan.chain = (first.value, words.value)
    except Exception:
        lib.b200moe_plan_destroy(handle)
        raise
    plan._plan = handle
    plan._forward = lib.b200moe_forward
    calls = (lib.b200moe_router, lib.b200moe_dispatch, lib.b200moe_gate_up, lib.b200moe_down, lib.b200moe_combine)
    plan.launches = tuple(StageLaunch(name, call, handle, device) for name, call in zip(STAGE_NAMES, calls))
    return plan
