"""Offline W4G128 weight preparation; never called inside a forward.

Host-side mirror of the reference's ``moe_weight_quant`` (reference
moe_weight_quant.py:25-105): same ``PackedGateUp`` container, same format
(format_version 1): each signed INT4 ``q`` in [-7,7] is stored as the nibble
``q+8``, eight nibbles per int32 word with the lowest nibble holding the
earliest K, one BF16 scale per (expert, output channel, 128 consecutive K),
``scale = bf16(max|w|/7)`` (1 for an all-zero group), ``q`` rounded half-even
from ``w / float(scale)``. The device operand is ``bf16_rn(float(q)*float(scale))``.

Generalised from the reference's hard-wired (128,1536,2048) gate/up tensor to
any contiguous CPU BF16 ``[E, N, K]`` with ``K % 128 == 0``, so that the same
format also packs the down projection (``[E, H, I]``, K = I).
"""
from dataclasses import dataclass
import hashlib
import math

import torch

GROUP = 128
SHAPE = (128, 1536, 2048)  # the gate/up shape the reference's packer is fixed to


def _digest(tensor):
    tensor = tensor.detach().cpu().contiguous()
    digest = hashlib.sha256(str((str(tensor.dtype), tuple(tensor.shape))).encode())
    digest.update(tensor.view(torch.uint8).numpy().tobytes())
    return digest.hexdigest()


@dataclass(frozen=True)
class PackedGateUp:
    """Packed words (int32 storage of the uint32 bit pattern), BF16 scales, metadata."""
    words: torch.Tensor
    scales: torch.Tensor
    metadata: dict

    def to(self, device):
        return PackedGateUp(self.words.to(device), self.scales.to(device), self.metadata)


PackedWeight = PackedGateUp  # the same container holds a packed down projection


def _check_packed(packed):
    if not isinstance(packed, PackedGateUp):
        raise TypeError("PackedGateUp required")
    words, scales = packed.words, packed.scales
    if words.dtype != torch.int32 or scales.dtype != torch.bfloat16:
        raise ValueError("int32 bit-pattern words / BF16 scales required")
    if (words.ndim != 3 or scales.ndim != 3 or words.shape[:2] != scales.shape[:2]
            or words.shape[2] * 8 != scales.shape[2] * GROUP):
        raise ValueError("unsupported packed shapes")
    if not words.is_contiguous() or not scales.is_contiguous() or words.device != scales.device:
        raise ValueError("same-device contiguous packed buffers required")


def _unpack_nibbles(words):
    """int32 words [..., W] -> int64 nibbles [..., W*8], earliest K first."""
    unsigned = words.to(torch.int64) & 0xFFFFFFFF
    place = 16 ** torch.arange(8, dtype=torch.int64, device=words.device)
    return ((unsigned.unsqueeze(-1) // place) % 16).flatten(-2)


def dequantize_gate_up_reference(packed):
    """Materialise BF16 weights for offline oracle / audit use only, never on the hot path."""
    _check_packed(packed)
    experts, rows, word_count = packed.words.shape
    output = torch.empty((experts, rows, word_count * 8), dtype=torch.bfloat16, device=packed.words.device)
    for expert in range(experts):  # one expert at a time bounds the int64 temporaries
        q = (_unpack_nibbles(packed.words[expert]) - 8).to(torch.float32)
        scale = packed.scales[expert].to(torch.float32).repeat_interleave(GROUP, dim=1)
        output[expert] = (q * scale).to(torch.bfloat16)
    return output


def _quantize_rows(rows_fp32):
    """[N, K] FP32 -> (q int64 [N,K] in [-7,7], scale BF16 [N, K/128])."""
    n, k = rows_fp32.shape
    grouped = rows_fp32.view(n, k // GROUP, GROUP)
    peak = grouped.abs().amax(dim=2)
    scale = (peak / 7).masked_fill(peak == 0, 1.0).to(torch.bfloat16)
    q = torch.round(grouped / scale.to(torch.float32).unsqueeze(2)).clamp_(-7, 7).to(torch.int64)
    return q.view(n, k), scale


def quantize_gate_up(weight):
    """Pack one finite, contiguous CPU BF16 ``[E, N, K]`` weight tensor (K % 128 == 0)."""
    if weight.device.type != "cpu" or weight.dtype != torch.bfloat16:
        raise ValueError("offline packing requires CPU BF16 weights")
    if weight.ndim != 3 or weight.shape[2] % GROUP or not weight.is_contiguous():
        raise ValueError("expected contiguous [E,N,K] weights with K a multiple of 128")
    if not torch.isfinite(weight).all().item():
        raise ValueError("nonfinite source weights")
    experts, rows, k = weight.shape
    words = torch.empty((experts, rows, k // 8), dtype=torch.int32)
    scales = torch.empty((experts, rows, k // GROUP), dtype=torch.bfloat16)
    place = 16 ** torch.arange(8, dtype=torch.int64)
    squared_error = squared_norm = worst = largest = 0.0
    for expert in range(experts):
        source = weight[expert].to(torch.float32)
        q, scale = _quantize_rows(source)
        if not bool((torch.isfinite(scale) & (scale > 0)).all()):
            raise ValueError("scale is not representable as finite positive BF16")
        packed_word = ((q + 8).view(rows, k // 8, 8) * place).sum(dim=2)       # < 2**32
        words[expert] = torch.where(packed_word >= 2**31, packed_word - 2**32, packed_word).to(torch.int32)
        scales[expert] = scale
        decoded = (q.to(torch.float32) * scale.to(torch.float32).repeat_interleave(GROUP, dim=1)).to(torch.bfloat16)
        delta = decoded.double() - source.double()
        squared_error += float(delta.square().sum())
        squared_norm += float(source.double().square().sum())
        worst = max(worst, float(delta.abs().max()))
        largest = max(largest, float(source.abs().max()))
    metadata = dict(
        format_version=1, logical_shape=list(weight.shape), group_size=GROUP,
        encoding="q+8, q in [-7,7], low nibble is earliest K",
        word_storage="int32 storage of uint32 bit pattern", scale_dtype="bfloat16",
        activation_dtype="bfloat16", accumulator_dtype="float32",
        source_sha256=_digest(weight), words_sha256=_digest(words), scales_sha256=_digest(scales),
        source_weight_bytes=weight.numel() * weight.element_size(),
        packed_weight_bytes=words.numel() * words.element_size(),
        scale_bytes=scales.numel() * scales.element_size(),
        weight_format_error=dict(
            relative_rms=math.sqrt(squared_error / squared_norm) if squared_norm else 0.0,
            normalized_max=worst / largest if largest else 0.0, max_abs=worst),
        interpretation="format loss only; not kernel implementation error or model task quality")
    return PackedGateUp(words, scales, metadata)


quantize_down = quantize_gate_up  # same algorithm with K = I
