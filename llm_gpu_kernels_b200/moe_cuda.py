"""Hand-written CUDA gate/up path of the reference interface.

Mirror of ``prepare_cuda_moe`` (reference moe_cuda.py:54-73). The reference
swaps its Triton gate/up launch for a WMMA kernel in three variants
(sync / async / async_skip: different cp.async pipelines for SM86). On B200
all three names select the same TMA + tcgen05 kernel - the pipeline is a
property of the hardware path, not a variant - and the E128/H2048/I768 shape
restriction of the reference is dropped.
"""
from .gemm import GemmConfig
from .moe_configured import prepare_configured_moe
from .moe_ranked import prepare_ranked_moe_launcher

VARIANTS = {"sync": 0, "async": 1, "async_skip": 2}


def prepare_cuda_moe(x, gate_up, down, ids, routing_weights, *, variant="sync", down_config=None,
                     router_weight=None):
    if variant not in VARIANTS:
        raise ValueError("unsupported CUDA variant")
    if down_config is None:
        return prepare_ranked_moe_launcher(x, gate_up, down, ids, routing_weights, router_weight=router_weight,
                                           schedule="tcgen05")
    if not isinstance(down_config, GemmConfig):
        raise TypeError("down_config must be GemmConfig")
    return prepare_configured_moe(x, gate_up, down, ids, routing_weights, down_config,
                                  router_weight=router_weight, schedule="tcgen05")
