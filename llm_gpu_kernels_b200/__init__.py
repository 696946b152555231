"""B200-native MoE-layer forward behind the llm-gpu-kernels prepared-MoE interface.

Entry points are imported by module path, as in the reference:
``llm_gpu_kernels_b200.moe_ranked.prepare_ranked_moe_launcher`` and friends.
"""
from .gemm import GemmConfig

__all__ = ["GemmConfig"]
__version__ = "0.1.0"
