"""Tile configuration object of the reference interface.

Mirror of ``GemmConfig`` (reference gemm.py:13-25): same fields, same
validation and error text, so callers of ``prepare_configured_moe`` keep
working. On B200 only ``block_m`` (rows of one expert per tile, the
granularity of the ``tasks`` prefix) reaches the kernels, as the token tile;
the channel tile (128) and K step (64) are fixed by the tcgen05 tile and
``block_n`` / ``block_k`` / ``warps`` / ``stages`` are accepted and recorded only.
"""
from dataclasses import dataclass


@dataclass(frozen=True)
class GemmConfig:
    block_m: int = 32
    block_n: int = 64
    block_k: int = 32
    warps: int = 4
    stages: int = 3

    def __post_init__(self):
        if any(x < 16 or x & (x - 1) for x in (self.block_m, self.block_n, self.block_k)):
            raise ValueError("tile dimensions must be powers of two >= 16")
        if self.warps not in (4, 8) or self.stages not in (2, 3, 4):
            raise ValueError("supported warps: 4/8; stages: 2/3/4")
