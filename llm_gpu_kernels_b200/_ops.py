"""``torch.library`` registration of the forward: ``torch.ops.b200moe.forward``.

The C ABI (``b200moe_forward``) takes raw pointers bound at prepare time, so the
operator proper is "enqueue the plan's kernels on the current stream". Wrapping
that call as a PyTorch custom op tells PyTorch which tensors it writes, which is
what lets ``PreparedMoE.run()`` sit inside ``torch.cuda.graph`` capture and inside
a ``torch.compile(fullgraph=True)`` region without a graph break: the tracer sees
one opaque op that mutates ``output`` (and the workspace, and ``ids`` /
``routing_weights`` when the plan has a router) and reads the rest.

The reference reaches its native plans through pybind11 classes holding
``torch::Tensor`` members (cuda_gate_up.cu:133-191); this is the same boundary with
the tensors passed per call for the tracer's benefit and the addresses fixed in the plan.
"""
from __future__ import annotations

import weakref
from typing import List

import torch

from . import _native

_LIB_NAME = "b200moe::forward"
_PLANS = {}   # plan address -> weak reference to the PreparedMoE that owns it


def register_plan(prepared):
    """Called by ``PreparedMoE.run()`` once: lets the operator find the tensors bound into the plan."""
    key = prepared._plan.value
    _PLANS[key] = weakref.ref(prepared, lambda _ref, key=key: _PLANS.pop(key, None))


def _bound_tensors(prepared):
    bound = [prepared.ids, prepared.routing_weights, prepared.output, prepared.counts, prepared.offsets,
             prepared.cursors, prepared.tasks, prepared.mapping, prepared.ranks, prepared.grouped_input,
             prepared.activated, prepared.down_output, prepared.status, prepared.scratch]
    if prepared.source_rows is not None:
        bound.append(prepared.source_rows)
    return bound


@torch.library.custom_op(_LIB_NAME, mutates_args=("ids", "routing_weights", "output", "workspace"),
                         device_types="cuda")
def forward(plan: int, x: torch.Tensor, weights: List[torch.Tensor], ids: torch.Tensor,
            routing_weights: torch.Tensor, output: torch.Tensor, workspace: List[torch.Tensor]) -> None:
    """One forward of the prepared plan ``plan`` (the ``B200MoePlan*`` as an integer) on the current stream of
    ``x``'s device. The kernels use the addresses bound at prepare time; the tensor arguments tell PyTorch what
    is read and what is written. Normally they ARE the bound tensors and nothing else happens. A tracer that
    functionalises the call (``torch.compile`` without re-inplacing) hands in copies instead: values of passed
    inputs are then copied into the bound buffers before the forward and the bound results into the passed
    tensors after it, so the op is a function of its arguments either way."""
    device = x.device
    lib = _native.load()
    owner = _PLANS.get(plan)
    prepared = owner() if owner is not None else None
    passed = [ids, routing_weights, output, *workspace]
    bound = _bound_tensors(prepared) if prepared is not None else passed
    if prepared is not None:
        for given, real in ((x, prepared.x), (ids, prepared.ids), (routing_weights, prepared.routing_weights)):
            if given.data_ptr() != real.data_ptr():
                real.copy_(given)
    if torch.cuda.current_device() == device.index:
        _native.check(lib.b200moe_forward(plan, torch.cuda.current_stream(device).cuda_stream))
    else:
        with torch.cuda.device(device):
            _native.check(lib.b200moe_forward(plan, torch.cuda.current_stream(device).cuda_stream))
    for given, real in zip(passed, bound):
        if given.data_ptr() != real.data_ptr():
            given.copy_(real)


@forward.register_fake
def _(plan, x, weights, ids, routing_weights, output, workspace):
    return None
