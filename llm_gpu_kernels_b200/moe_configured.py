"""Explicit tile configuration over the ranked path.

Mirror of ``prepare_configured_moe`` (reference moe_configured.py:17-70): the
caller binds one ``GemmConfig`` chosen from the shape alone before any capture.
``config.block_m`` is the number of rows of one expert a tile covers; on the
tcgen05 schedule it must be one of 16/32/64/128/256 (the MMA N range), and the
remaining fields are recorded but fixed by the hardware tile.
"""
from .gemm import GemmConfig
from .moe import _prepare
from .moe_ranked import _ranked


def prepare_configured_moe(x, gate_up, down, ids, routing_weights, config, *, router_weight=None,
                           schedule=None):
    if not isinstance(config, GemmConfig):
        raise TypeError("config must be GemmConfig")
    hidden, intermediate = x.shape[1] if x.ndim == 2 else 0, down.shape[2] if down.ndim == 3 else 0
    tensor_tiles = hidden % 8 == 0 and intermediate % 8 == 0 and hidden >= 64 and intermediate >= 64
    if schedule == "generic" or (schedule in (None, "auto") and not tensor_tiles):
        token_tile = 0  # the CUDA-core schedule has one tile size
    else:
        if config.block_m > 256:
            raise ValueError("block_m above 256 exceeds the tcgen05 MMA N range")
        token_tile = config.block_m
    base = _prepare(x, gate_up, down, ids, routing_weights, router_weight=router_weight, schedule=schedule,
                    token_tile=token_tile, config=config)
    return _ranked(base)
