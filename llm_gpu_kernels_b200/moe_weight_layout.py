"""Bit-preserving physical re-layout of packed gate/up (the reference's "v2").

Mirror of reference moe_weight_layout.py:39-175: ``words_v2[e,p,nt,kt,w,nl] =
words_v1[e, p*I + nt*64 + nl, kt*4 + w]`` and ``scales_v2[e,p,nt,kg,nl] =
scales_v1[e, p*I + nt*64 + nl, kg]``. The reference introduced it so that
SM86 scalar loads coalesce across output channels; the B200 kernels TMA-load
the canonical v1 rows, so a ``RepackedGateUp`` handed to
``prepare_w4_layout_moe`` is restored to v1 (on the device, bit-exactly) at
prepare time. Generalised to any ``[E, 2I, K]`` with ``I % 64 == 0``.
"""
from copy import deepcopy
from dataclasses import dataclass

import torch

from .moe_weight_quant import GROUP, PackedGateUp, _check_packed, _digest

LAYOUT = ("words[E,projection,Ntile,K32,word,Nlane];"
          "scales[E,projection,Ntile,K128,Nlane];Nlane-contiguous")


@dataclass(frozen=True)
class RepackedGateUp:
    words: torch.Tensor
    scales: torch.Tensor
    metadata: dict

    def to(self, device):
        return RepackedGateUp(self.words.to(device), self.scales.to(device), deepcopy(self.metadata))


def repack_gate_up(packed: PackedGateUp) -> RepackedGateUp:
    """Permute a v1 pack without requantising or changing a bit."""
    _check_packed(packed)
    if packed.metadata.get("format_version") != 1 or packed.metadata.get("group_size") != GROUP:
        raise ValueError("v1 metadata must declare format_version=1, W4G128")
    experts, rows, word_count = packed.words.shape
    if rows % 128 or word_count % 4:
        raise ValueError("gate/up rows must be 2*I with I a multiple of 64; K a multiple of 32")
    ntiles = rows // 128
    words = packed.words.reshape(experts, 2, ntiles, 64, word_count // 4, 4).permute(0, 1, 2, 4, 5, 3).contiguous()
    groups = packed.scales.shape[2]
    scales = packed.scales.reshape(experts, 2, ntiles, 64, groups).permute(0, 1, 2, 4, 3).contiguous()
    metadata = {
        "format_version": 2, "layout": LAYOUT, "logical_shape": list(packed.metadata["logical_shape"]),
        "group_size": GROUP,
        "canonical_words_sha256": _digest(packed.words), "canonical_scales_sha256": _digest(packed.scales),
        "canonical_words_shape": list(packed.words.shape), "canonical_scales_shape": list(packed.scales.shape),
        "physical_words_shape": list(words.shape), "physical_scales_shape": list(scales.shape),
        "physical_words_sha256": _digest(words), "physical_scales_sha256": _digest(scales),
        "canonical_v1_metadata": deepcopy(packed.metadata),
    }
    if words.numel() != packed.words.numel() or scales.numel() != packed.scales.numel():
        raise RuntimeError("layout conversion changed the packed+scale size")
    return RepackedGateUp(words, scales, metadata)


def restore_v1_tensors(words_v2, scales_v2):
    """The inverse permutation on any device; returns (words_v1, scales_v1)."""
    experts, _, ntiles, k32, _, _ = words_v2.shape
    words = words_v2.permute(0, 1, 2, 5, 3, 4).contiguous().reshape(experts, 2 * ntiles * 64, k32 * 4)
    scales = scales_v2.permute(0, 1, 2, 4, 3).contiguous().reshape(experts, 2 * ntiles * 64, scales_v2.shape[3])
    return words, scales


def restore_v1_layout(repacked: RepackedGateUp) -> PackedGateUp:
    """Restore the canonical v1 bit patterns and check them against the recorded digests."""
    if not isinstance(repacked, RepackedGateUp):
        raise TypeError("restore_v1_layout requires RepackedGateUp")
    metadata = repacked.metadata
    if metadata.get("format_version") != 2 or metadata.get("layout") != LAYOUT:
        raise ValueError("unsupported physical layout metadata")
    if repacked.words.dtype != torch.int32 or repacked.scales.dtype != torch.bfloat16 or repacked.words.ndim != 6:
        raise ValueError("physical buffers must be int32 [E,2,Nt,K32,4,64] and BF16 [E,2,Nt,K128,64]")
    words, scales = restore_v1_tensors(repacked.words, repacked.scales)
    if (_digest(words) != metadata.get("canonical_words_sha256")
            or _digest(scales) != metadata.get("canonical_scales_sha256")):
        raise ValueError("restored v1 bit patterns do not match the canonical digests")
    return PackedGateUp(words, scales, deepcopy(metadata["canonical_v1_metadata"]))
