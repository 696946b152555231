"""Ranked-dispatch prepared MoE: the entry point the reference recommends.

Mirror of ``PreparedRankedMoE`` / ``prepare_ranked_moe_launcher`` (reference
moe_ranked.py:68-169): ``.base`` holds every buffer, ``.ranks`` the per-route
rank inside its expert, ``.launches`` the cached launch sequence (empty for
T == 0), ``run()`` replays it on the current stream. Here the rank is the
deterministic stable rank computed without global atomics, and the sequence
has five subsystems (router, dispatch, gate_up_swiglu, down, combine) instead
of the reference's seven Triton launches.
"""
from dataclasses import dataclass

import torch

from .moe import PreparedMoE, _prepare


@dataclass(frozen=True)
class PreparedRankedMoE:
    base: PreparedMoE
    ranks: torch.Tensor
    launches: tuple

    @property
    def workspace_bytes(self) -> int:
        return self.base.workspace_bytes + self.ranks.numel() * self.ranks.element_size()

    @property
    def names(self) -> tuple:
        """Names of the subsystems ``run()`` executes, in order."""
        return tuple(launch.name for launch in self.launches)

    def run(self):
        return self.base.run()

    def check_inputs(self):
        """The base workspace's explicit synchronising input check."""
        return self.base.check_inputs()


def _ranked(base: PreparedMoE) -> PreparedRankedMoE:
    launches = base.launches if base.router_weight is not None else base.launches[1:]
    return PreparedRankedMoE(base=base, ranks=base.ranks, launches=tuple(launches))


def prepare_ranked_moe_launcher(x, gate_up, down, ids, routing_weights, *, router_weight=None,
                                schedule=None, token_tile=0, router_bf16_weights=False, residual=None,
                                keep_grouped_input=False, down_pair=None, down_tiles=None):
    """Drop-in for reference ``prepare_ranked_moe_launcher`` (moe_ranked.py:99-169)."""
    return _ranked(_prepare(x, gate_up, down, ids, routing_weights, router_weight=router_weight,
                            schedule=schedule, token_tile=token_tile, router_bf16_weights=router_bf16_weights,
                            residual=residual, keep_grouped_input=keep_grouped_input, down_pair=down_pair,
                            down_tiles=down_tiles))
