"""Fixed-route (or routed) W4A16 MoE behind the reference's ``prepare_w4_moe``.

Mirror of reference moe_w4_cuda.py:85-164: takes an already packed, immutable
``PackedGateUp`` (format version 1, W4G128) on the device instead of a dense
gate/up tensor, owns no dense weight copy, and keeps the prepared life cycle.
The reference quantises gate/up only and keeps down in BF16; that is the
default here too. ``packed_down`` (same container, K = I) extends the format
to the down projection. The E128/H2048/I768 restriction is dropped: any shape
with H (and I, when down is packed) a multiple of 128 works.
The packed words are consumed as stored: TMA brings them to shared memory and
converter warps dequantise to BF16 inside the tile (csrc/grouped_gemm_w4.cu).
"""
import torch

from .gemm import GemmConfig
from .moe import _prepare
from .moe_ranked import _ranked
from .moe_weight_quant import PackedGateUp


def _check_format(packed, what):
    if (not isinstance(packed, PackedGateUp) or packed.metadata.get("format_version") != 1
            or packed.metadata.get("group_size") != 128):
        raise ValueError(f"{what}: validated W4G128 format version 1 required")
    if packed.words.device.type != "cuda" or packed.scales.device != packed.words.device:
        raise ValueError(f"{what}: same-device contiguous CUDA inputs required")


def prepare_w4_moe(x, packed, down, ids, routing_weights, *, down_config=None, packed_down=None,
                   router_weight=None, keep_grouped_input=False):
    """Prepare outside timing; no dense weight reconstruction, no counts read-back.

    ``down`` is the BF16 ``[E,H,I]`` tensor, or ``None`` when ``packed_down`` is given.
    ``down_config.block_m`` (if any) is the token tile, as in ``prepare_configured_moe``.
    """
    _check_format(packed, "gate/up")
    if packed_down is not None:
        _check_format(packed_down, "down")
        if down is not None:
            raise ValueError("pass either a BF16 down tensor or packed_down, not both")
    elif not isinstance(down, torch.Tensor):
        raise ValueError("BF16 down tensor (or packed_down) required")
    token_tile = 0
    if down_config is not None:
        if not isinstance(down_config, GemmConfig):
            raise TypeError("down_config must be GemmConfig")
        if down_config.block_m > 256:
            raise ValueError("block_m above 256 exceeds the tcgen05 MMA N range")
        token_tile = down_config.block_m
    base = _prepare(
        x, packed.words, down if packed_down is None else packed_down.words, ids, routing_weights,
        router_weight=router_weight, schedule="tcgen05", token_tile=token_tile, config=down_config,
        gate_up_scales=packed.scales, down_scales=None if packed_down is None else packed_down.scales,
        keep_grouped_input=keep_grouped_input)
    base.packed = packed
    return _ranked(base)
