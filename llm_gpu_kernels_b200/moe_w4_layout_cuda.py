"""``prepare_w4_layout_moe``: the reference's entry point for its re-laid-out pack.

Mirror of reference moe_w4_layout_cuda.py:152-265. The reference's "v2" layout
reorders words so that SM86 scalar loads coalesce across output channels. The
B200 kernel reads canonical rows through TMA, so a ``RepackedGateUp`` is turned
back into the canonical v1 tensors once, on the device, at prepare time (a
bit-preserving permutation, verified by ``restore_v1_layout`` on the host
side), and then takes the same path as ``prepare_w4_moe``.
"""
from copy import deepcopy

from .moe_w4_cuda import prepare_w4_moe
from .moe_weight_layout import LAYOUT, RepackedGateUp, restore_v1_tensors
from .moe_weight_quant import PackedGateUp


def prepare_w4_layout_moe(x, repacked, down, ids, routing_weights, *, down_config=None, packed_down=None,
                          router_weight=None):
    if not isinstance(repacked, RepackedGateUp):
        raise TypeError("RepackedGateUp required")
    metadata = repacked.metadata
    if metadata.get("format_version") != 2 or metadata.get("layout") != LAYOUT or metadata.get("group_size") != 128:
        raise ValueError("unsupported physical layout metadata")
    if repacked.words.ndim != 6 or repacked.scales.ndim != 5 or repacked.words.device.type != "cuda":
        raise ValueError("physical CUDA buffers [E,2,Nt,K32,4,64] / [E,2,Nt,K128,64] required")
    words, scales = restore_v1_tensors(repacked.words, repacked.scales)
    canonical = PackedGateUp(words, scales, deepcopy(metadata["canonical_v1_metadata"]))
    prepared = prepare_w4_moe(x, canonical, down, ids, routing_weights, down_config=down_config,
                              packed_down=packed_down, router_weight=router_weight)
    prepared.base.repacked = repacked
    return prepared
