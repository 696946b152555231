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

from typing import List

import torch

from . import _native

_LIB_NAME = "b200moe::forward"


@torch.library.custom_op(_LIB_NAME, mutates_args=("ids", "routing_weights", "output", "workspace"),
                         device_types="cuda")
def forward(plan: int, x: torch.Tensor, weights: List[torch.Tensor], ids: torch.Tensor,
            routing_weights: torch.Tensor, output: torch.Tensor, workspace: List[torch.Tensor]) -> None:
    """One forward of the prepared plan ``plan`` (the ``B200MoePlan*`` as an integer) on the current stream of
    ``x``'s device. The tensor arguments are the ones bound into the plan; they are passed so that PyTorch knows
    what is read and what is written - the kernels use the addresses bound at prepare time."""
    device = x.device
    lib = _native.load()
    if torch.cuda.current_device() == device.index:
        _native.check(lib.b200moe_forward(plan, torch.cuda.current_stream(device).cuda_stream))
    else:
        with torch.cuda.device(device):
            _native.check(lib.b200moe_forward(plan, torch.cuda.current_stream(device).cuda_stream))


@forward.register_fake
def _(plan, x, weights, ids, routing_weights, output, workspace):
    return None
