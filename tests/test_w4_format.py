"""The shipped W4G128 packer / re-layout against the reference-made golden vectors (no GPU)."""
import json

import pytest
import torch

from llm_gpu_kernels_b200.moe_weight_layout import RepackedGateUp, repack_gate_up, restore_v1_layout
from llm_gpu_kernels_b200.moe_weight_quant import (PackedGateUp, dequantize_gate_up_reference, quantize_down,
                                                    quantize_gate_up)
from oracle import moe_oracle as O
from tests.util import digest


def test_packer_matches_reference_slice(golden_dir):
    g = torch.load(golden_dir / "w4_slice.pt")
    packed = quantize_gate_up(g["source"][None].contiguous())
    assert torch.equal(packed.words[0], g["words"]) and torch.equal(packed.scales[0], g["scales"])
    assert torch.equal(dequantize_gate_up_reference(packed)[0], g["dequant"])
    assert packed.metadata["format_version"] == 1 and packed.metadata["group_size"] == 128


def test_packer_full_reference_shape_digests(golden_dir):
    meta = json.loads((golden_dir / "golden_meta.json").read_text())["w4"]
    g = torch.Generator().manual_seed(meta["seed"])
    w = torch.empty(128, 1536, 2048, dtype=torch.bfloat16)
    for e in range(128):
        w[e] = (0.02 * torch.randn(1536, 2048, generator=g)).bfloat16()
    w[5, 17, 256:384] = 0
    packed = quantize_gate_up(w)
    assert packed.metadata["words_sha256"] == meta["words_sha256"]
    assert packed.metadata["scales_sha256"] == meta["scales_sha256"]
    assert packed.metadata["packed_weight_bytes"] == 192 * 2**20 and packed.metadata["scale_bytes"] == 6 * 2**20
    assert abs(packed.metadata["weight_format_error"]["relative_rms"] - meta["format_error"]["relative_rms"]) < 1e-9
    repacked = repack_gate_up(packed)
    assert digest(repacked.words) == meta["v2_words_sha256"] and digest(repacked.scales) == meta["v2_scales_sha256"]
    back = restore_v1_layout(repacked)
    assert torch.equal(back.words, packed.words) and torch.equal(back.scales, packed.scales)


def test_down_projection_shape_and_oracle_agreement():
    g = torch.Generator().manual_seed(4)
    w = (0.02 * torch.randn(3, 64, 768, generator=g)).bfloat16()
    packed = quantize_down(w)
    words, scales = O.quantize_w4g128(w)
    assert torch.equal(packed.words, words) and torch.equal(packed.scales, scales)
    assert tuple(packed.words.shape) == (3, 64, 96) and tuple(packed.scales.shape) == (3, 64, 6)
    assert torch.equal(dequantize_gate_up_reference(packed), O.dequantize_w4g128(words, scales))


def test_validation_errors():
    with pytest.raises(ValueError):
        quantize_gate_up(torch.zeros(1, 4, 100, dtype=torch.bfloat16))        # K not a multiple of 128
    with pytest.raises(ValueError):
        quantize_gate_up(torch.zeros(1, 4, 128))                              # not BF16
    bad = torch.zeros(1, 4, 128, dtype=torch.bfloat16)
    bad[0, 0, 0] = float("inf")
    with pytest.raises(ValueError):
        quantize_gate_up(bad)
    with pytest.raises(TypeError):
        dequantize_gate_up_reference("nope")
    packed = quantize_gate_up(torch.ones(1, 128, 128, dtype=torch.bfloat16))
    tampered = RepackedGateUp(*(t.clone() for t in (repack_gate_up(packed).words, repack_gate_up(packed).scales)),
                              repack_gate_up(packed).metadata)
    tampered.words[0, 0, 0, 0, 0, 0] ^= 1
    with pytest.raises(ValueError):
        restore_v1_layout(tampered)
    assert isinstance(packed.to("cpu"), PackedGateUp)
