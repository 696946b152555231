"""The CPU oracle against the golden vectors produced by the reference itself
(tests/golden/make_golden.py). No GPU, no reference checkout needed."""
import json

import pytest
import torch

from oracle import moe_oracle as O
from tests.util import digest, seeded_layer


def test_mini_fixed_route_matches_reference(golden_dir):
    g = torch.load(golden_dir / "mini_fixed_route.pt")
    out = O.moe_oracle(g["x"], g["gate_up"], g["down"], g["ids"], g["rw"])
    assert O.error_metrics(out, g["out"])["relative_rms"] < 1e-6
    assert torch.allclose(out, g["out"], rtol=1e-5, atol=1e-4)


def test_three_token_hand_case(golden_dir):
    g = torch.load(golden_dir / "three_token.pt")
    args = (g["x"], g["gate_up"], g["down"], g["ids"], g["rw"])
    assert torch.allclose(O.moe_oracle(*args), g["out"], rtol=1e-5, atol=1e-5)
    assert torch.allclose(O.per_route_oracle(*args), g["per_route"], rtol=1e-5, atol=1e-5)
    assert O.error_metrics(O.moe_oracle(*args), O.per_route_oracle(*args))["passed"]


def test_tiny_layer_seed0(golden_dir):
    g = torch.load(golden_dir / "tiny_layer_seed0.pt")
    wr, gate_up, down, x = seeded_layer(0, 64, 256, 128, 8)
    got = {"router_weight": digest(wr), "gate_up": digest(gate_up), "down": digest(down), "x": digest(x)}
    assert got == g["digests"], "seeded CPU generator no longer reproduces the fixture inputs"
    ids, rw, _ = O.router_oracle(x, wr, 2)
    assert torch.equal(ids, g["ids"])
    assert torch.allclose(rw, g["rw"], rtol=0, atol=1e-7)
    out, ids2, rw2 = O.moe_layer_oracle(x, wr, gate_up, down, 2)
    assert torch.equal(ids2, ids)
    assert torch.allclose(out, g["out"], rtol=1e-5, atol=1e-6)
    assert tuple(out.shape) == (64, 256) and out.dtype == torch.float32


def test_dispatch_cases(golden_dir):
    for case in torch.load(golden_dir / "dispatch_cases.pt"):
        counts, offsets, ranks, mapping = O.dispatch_oracle(case["ids"], case["experts"])
        assert torch.equal(counts, case["counts"]) and torch.equal(offsets, case["offsets"])
        assert torch.equal(ranks, case["ranks"]) and torch.equal(mapping, case["mapping"])
        flat = case["ids"].reshape(-1)
        assert torch.equal(counts.long(), torch.bincount(flat, minlength=case["experts"]))
        assert sorted(mapping.tolist()) == list(range(flat.numel()))
        order = torch.argsort(flat, stable=True)
        assert torch.equal(mapping[order].long(), torch.arange(flat.numel()))


def test_dispatch_invalid_ids_and_status():
    ids = torch.tensor([[0, 5], [-1, 2], [2, 2]])
    counts, offsets, ranks, mapping = O.dispatch_oracle(ids, 4)
    assert counts.tolist() == [1, 0, 3, 0] and offsets.tolist() == [0, 1, 1, 4]
    assert mapping.tolist() == [0, -1, -1, 1, 2, 3] and ranks.tolist() == [0, -1, -1, 0, 1, 2]
    assert O.status_oracle(ids, torch.ones(3, 2), 4) == 1
    assert O.status_oracle(torch.zeros(1, 1, dtype=torch.long), torch.tensor([[float("nan")]]), 4) == 2
    assert O.status_oracle(ids, torch.tensor([[1.0, float("inf")]] * 3), 4) == 3


def test_w4_slice(golden_dir):
    g = torch.load(golden_dir / "w4_slice.pt")
    words, scales = O.quantize_w4g128(g["source"][None])
    assert torch.equal(words[0], g["words"]) and torch.equal(scales[0], g["scales"])
    assert torch.equal(O.dequantize_w4g128(words, scales)[0], g["dequant"])
    assert scales[0, 1, 2].item() == 1.0  # the all-zero group of the fixture
    nib = (words.long()[..., None] >> (torch.arange(8) * 4)) & 15
    assert int(nib.min()) >= 1 and int(nib.max()) <= 15


def test_w4_full_shape_digests(golden_dir):
    meta = json.loads((golden_dir / "golden_meta.json").read_text())["w4"]
    g = torch.Generator().manual_seed(meta["seed"])
    w = torch.empty(128, 1536, 2048, dtype=torch.bfloat16)
    for e in range(128):
        w[e] = (0.02 * torch.randn(1536, 2048, generator=g)).bfloat16()
    w[5, 17, 256:384] = 0
    assert digest(w) == meta["source_sha256"]
    words, scales = O.quantize_w4g128(w)
    assert digest(words) == meta["words_sha256"] and digest(scales) == meta["scales_sha256"]
    assert words.numel() * 4 == 192 * 2**20 and scales.numel() * 2 == 6 * 2**20  # the byte ledger
    assert digest(O.dequantize_w4g128(words, scales)) == meta["dequant_sha256"]
    w2, s2 = O.repack_v2(words, scales, 768)
    assert tuple(w2.shape) == (128, 2, 12, 64, 4, 64) and tuple(s2.shape) == (128, 2, 12, 16, 64)
    assert digest(w2) == meta["v2_words_sha256"] and digest(s2) == meta["v2_scales_sha256"]
    w1, s1 = O.restore_v1(w2, s2)
    assert torch.equal(w1, words) and torch.equal(s1, scales)


def test_w4_generalised_shape_roundtrip():
    g = torch.Generator().manual_seed(3)
    w = (0.02 * torch.randn(3, 40, 768, generator=g)).bfloat16()  # a down-projection-like K = 768
    words, scales = O.quantize_w4g128(w)
    assert tuple(words.shape) == (3, 40, 96) and tuple(scales.shape) == (3, 40, 6)
    deq = O.dequantize_w4g128(words, scales)
    err = O.error_metrics(deq, w)
    assert 0.05 < err["relative_rms"] < 0.2  # 4-bit format loss, same order as the reference reports
    # idempotence: quantising the dequantised weight reproduces the same integers
    words2, _ = O.quantize_w4g128(deq)
    assert torch.equal(O.dequantize_w4g128(words2, _), deq)


def test_router_properties():
    g = torch.Generator().manual_seed(9)
    x = torch.randn(33, 64, generator=g).bfloat16()
    wr = torch.randn(16, 64, generator=g).bfloat16()
    ids, rw, probs = O.router_oracle(x, wr, 4)
    assert ids.dtype == torch.int32 and rw.dtype == torch.float32
    assert torch.allclose(rw.sum(1), torch.ones(33), atol=1e-6) and (rw >= 0).all()
    assert (ids.sort(1).values[:, 1:] != ids.sort(1).values[:, :-1]).all()
    ok, msg = O.router_agrees(ids, rw, probs, 4)
    assert ok, msg
    bad = ids.clone()
    bad[0, 0] = probs[0].argmin()
    assert not O.router_agrees(bad, rw, probs, 4)[0]


def test_error_metrics_limits():
    a = torch.ones(4, 4)
    assert O.error_metrics(a, a)["passed"]
    assert not O.error_metrics(a * 1.02, a)["passed"]
    assert O.error_metrics(torch.empty(0, 4), torch.empty(0, 4))["empty"]
    with pytest.raises(ValueError):
        O.error_metrics(a, torch.ones(2, 2))
