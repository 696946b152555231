"""Real-trace bundle format and the file-backed tile policy (host logic, no GPU)."""
import json

import pytest
import torch

from llm_gpu_kernels_b200.gemm import GemmConfig
from llm_gpu_kernels_b200.moe_full_policy import FrozenMoEPolicy
from llm_gpu_kernels_b200.moe_real_trace import (tensor_sha256, validate_real_moe_trace, validate_trace_tensors,
                                                  write_real_moe_trace)

DIMS = dict(experts=8, hidden=64, intermediate=32, topk=2)


def small_trace(tokens=5):
    g = torch.Generator().manual_seed(0)
    x = torch.randn(tokens, 64, generator=g).bfloat16()
    ids = torch.stack([torch.randperm(8, generator=g)[:2] for _ in range(tokens)]).to(torch.int32)
    rw = torch.rand(tokens, 2, generator=g).bfloat16().float()
    gu = torch.randn(8, 64, 64, generator=g).bfloat16()
    dn = torch.randn(8, 64, 32, generator=g).bfloat16()
    return x, ids, rw, gu, dn


def test_trace_round_trip(tmp_path):
    x, ids, rw, gu, dn = small_trace()
    manifest = write_real_moe_trace(tmp_path, x, ids, rw, gu, dn, dims=DIMS)
    trace = validate_real_moe_trace(manifest, load_weights=True)
    assert torch.equal(trace.tensors["x"], x) and torch.equal(trace.tensors["expert_ids"], ids)
    assert torch.equal(trace.weights["down"], dn)
    assert trace.manifest["trace"]["tensors"]["x"]["sha256"] == tensor_sha256(x)
    assert validate_real_moe_trace(manifest, load_trace=False).tensors is None


def test_bundle_written_by_the_reference_is_accepted(golden_dir, tmp_path):
    """tests/golden/ref_trace holds a manifest and a trace bundle written by the reference's own
    write_real_moe_trace (see make_golden.py); the 1.8 GB weight bundle it points to is not committed."""
    import shutil
    for name in ("trace.json", "trace.pt"):
        shutil.copy(golden_dir / "ref_trace" / name, tmp_path / name)
    manifest = tmp_path / "trace.json"
    trace = validate_real_moe_trace(manifest, check_weight_files=False)
    assert tuple(trace.tensors["x"].shape) == (6, 2048) and tuple(trace.tensors["expert_ids"].shape) == (6, 8)
    assert trace.manifest["model"]["num_experts"] == 128 and trace.manifest["status"] == "passed"
    assert trace.manifest["trace"]["tensors"]["route_weights"]["sha256"] == tensor_sha256(trace.tensors["route_weights"])
    with pytest.raises(ValueError, match="existing file"):
        validate_real_moe_trace(manifest)                       # the weight bundle is required by default
    with pytest.raises(ValueError, match="expected"):
        validate_real_moe_trace(manifest, check_weight_files=False, dims=DIMS)
    # every manifest rule of the reference's validator is enforced here too
    good = json.loads(manifest.read_text())
    for mutate, message in (
            (lambda m: m.update(status="failed"), "not marked passed"),
            (lambda m: m["routing_contract"].update(renormalization="topk"), "routing contract"),
            (lambda m: m.pop("capture"), "capture metadata"),
            (lambda m: m["trace"].update(format="pickle"), "weights-only tensor dictionary"),
            (lambda m: m["weights"]["down"].update(format="pickle"), "weights-only torch bundle"),
            (lambda m: m["weights"]["down"].update(source_manifest_sha256="1" * 64), "same layer-extraction"),
            (lambda m: m["weights"]["gate_up"].update(shape=[128, 1536, 1024]), "shape/dtype"),
            (lambda m: m["trace"]["tensors"]["x"].update(dtype="float32"), "dtype must be"),
            (lambda m: m["model"].update(top_k=0), "model block")):
        bad = json.loads(json.dumps(good))
        mutate(bad)
        manifest.write_text(json.dumps(bad))
        with pytest.raises(ValueError, match=message):
            validate_real_moe_trace(manifest, check_weight_files=False)


def test_trace_tampering_is_detected(tmp_path):
    x, ids, rw, gu, dn = small_trace()
    manifest = write_real_moe_trace(tmp_path, x, ids, rw, gu, dn, dims=DIMS)
    payload = torch.load(tmp_path / "trace.pt", weights_only=True)
    payload["x"][0, 0] += 1
    torch.save(payload, tmp_path / "trace.pt")
    with pytest.raises(ValueError, match="SHA256 mismatch"):
        validate_real_moe_trace(manifest)
    with pytest.raises(ValueError, match="content hash"):
        validate_real_moe_trace(manifest, verify_hashes=False)
    data = json.loads(manifest.read_text())
    data["trace"]["path"] = "https://example.invalid/trace.pt"
    manifest.write_text(json.dumps(data))
    with pytest.raises(ValueError, match="local path"):
        validate_real_moe_trace(manifest)


def test_trace_tensor_rules():
    x, ids, rw, _, _ = small_trace()
    validate_trace_tensors(x, ids, rw, dims=DIMS)
    dup = ids.clone(); dup[0] = 3
    with pytest.raises(ValueError, match="unique"):
        validate_trace_tensors(x, dup, rw, dims=DIMS)
    with pytest.raises(ValueError, match="promotions"):
        validate_trace_tensors(x, ids, rw + 1e-4, dims=DIMS)
    with pytest.raises(TypeError):
        validate_trace_tensors(x.float(), ids, rw, dims=DIMS)
    with pytest.raises(ValueError):
        validate_trace_tensors(x, ids, -rw - 1, dims=DIMS)


def test_policy_file():
    policy = FrozenMoEPolicy.load()
    assert policy.select(17, 128, 8, 2048, 768) == (GemmConfig(block_m=16), "small")
    assert policy.select(1024, 128, 8, 2048, 768) == (GemmConfig(block_m=128), "medium")
    assert policy.select(32768, 8, 2, 4096, 14336) == (GemmConfig(block_m=256), "large")
    assert policy.select(9, 3, 2, 67, 33) == (policy.fallback, "shape_fallback")
    assert policy.verify_provenance()["sha256"] == policy.sha256
    with pytest.raises(ValueError):
        policy.select(-1, 128, 8, 2048, 768)
