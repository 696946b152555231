"""Shape-only schedule choice.

The reference freezes a tile policy keyed on ``mu = T*K/E`` with thresholds 8
and 64 (reference moe_full_policy.py:132-152, results/m7-policy.json) so that a
captured graph stays valid when routes change: nothing about the choice may
depend on ids or counts. The same rule holds here. ``select`` returns the
``GemmConfig`` whose ``block_m`` is the token tile the library would pick for
the shape, and the bucket name.
"""
from .gemm import GemmConfig

BUCKET_NAMES = ("small", "medium", "large")
THRESHOLDS_MU = (8.0, 64.0)


def token_tile_for(tokens: int, experts: int, topk: int) -> int:
    """Twice the mean rows per expert as a power of two in [16,128]; 256 from 1024 rows per expert
    (the rule in csrc/abi.cu)."""
    routes = tokens * topk
    twice_mu = -(-2 * routes // experts)
    if twice_mu >= 2048:
        return 256
    tile = 16
    while tile < 128 and tile < twice_mu:
        tile <<= 1
    return tile


def select(T, E, topk, H, I):
    """Return ``(GemmConfig, bucket)`` from dimensions only; T may be zero."""
    tokens, experts, routed = int(T), int(E), int(topk)
    if tokens < 0:
        raise ValueError("T must be nonnegative")
    mu = tokens * routed / experts
    index = 0 if mu <= THRESHOLDS_MU[0] else 1 if mu <= THRESHOLDS_MU[1] else 2
    return GemmConfig(block_m=token_tile_for(tokens, experts, routed)), BUCKET_NAMES[index]
