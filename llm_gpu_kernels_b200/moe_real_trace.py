"""Loader for captured real-model MoE traces in the reference's bundle format.

Reads what the reference's ``write_real_moe_trace`` writes and its
``validate_real_moe_trace`` accepts (reference moe_real_trace.py:267-523): a JSON
manifest next to local ``.pt`` bundles, everything hashed with SHA-256.

* ``manifest["trace"]``: ``path`` / ``sha256`` of a weights-only ``.pt`` dict holding exactly
  ``x`` [T,H] BF16, ``expert_ids`` [T,K] int32/int64 (unique per token) and ``route_weights`` [T,K]
  FP32 that are exact promotions of BF16 router outputs; ``tensors[name]`` = shape, dtype, content hash.
* ``manifest["weights"]["gate_up" | "down"]``: ``path`` / ``sha256`` / ``tensor_name`` of ONE shared
  bundle holding ``gate_up`` [E,2I,H] and ``down`` [E,H,I] BF16.

The tensors of the reference's Qwen3-30B-A3B layer-0 capture are not distributed with it, so
this module ships the reader, the validation rules and a writer that produces the same layout
(used by the tests and by anyone who captures a trace); the dimensions default to that model
and can be overridden for other captures. ``prepare_trace_moe`` binds a loaded trace to the
prepared layer. Nothing here runs on the GPU or inside a forward.
"""
from __future__ import annotations

import hashlib
import json
import os
from dataclasses import dataclass
from pathlib import Path
from urllib.parse import urlsplit

import torch

SCHEMA = "llm_gpu_kernels.moe_real_trace"
SCHEMA_VERSION = 1
TRACE_TENSOR_NAMES = ("x", "expert_ids", "route_weights")
QWEN3_30B_A3B = dict(experts=128, hidden=2048, intermediate=768, topk=8)
# identity of the capture the reference pins (reference moe_real_trace.py:22-23); other captures pass their own
MODEL_REPO_ID = "Qwen/Qwen3-30B-A3B"
MODEL_REVISION = "ad44e777bcd18fa416d9da3bd8f70d33ebb85d39"
# what a stored route weight means (reference moe_real_trace.py:377-383): the model's BF16 router output,
# promoted exactly to FP32, not renormalised, ids unique per token
ROUTING_CONTRACT = {"source_dtype": "bfloat16", "stored_dtype": "float32",
                    "conversion": "exact_bfloat16_to_float32_promotion", "renormalization": "none",
                    "unique_expert_ids_per_token": True}
TRACE_FORMAT = "torch_weights_only_tensor_dict"
WEIGHTS_FORMAT = "torch_weights_only_bundle"


def _model_block(dims, repo_id, revision):
    return {"repo_id": repo_id, "revision": revision, "num_experts": dims["experts"], "hidden_size": dims["hidden"],
            "intermediate_size": dims["intermediate"], "top_k": dims["topk"]}


def _dims_of(model):
    keys = ("num_experts", "hidden_size", "intermediate_size", "top_k")
    if (not isinstance(model, dict) or not isinstance(model.get("repo_id"), str)
            or not isinstance(model.get("revision"), str)
            or any(type(model.get(k)) is not int or model[k] <= 0 for k in keys)):
        raise ValueError("manifest model block must name repo_id, revision and positive integer dimensions")
    return dict(experts=model["num_experts"], hidden=model["hidden_size"],
                intermediate=model["intermediate_size"], topk=model["top_k"])


@dataclass(frozen=True)
class RealMoETrace:
    """A validated manifest and, when asked for, its CPU tensors."""
    manifest_path: Path
    manifest: dict
    tensors: dict | None
    weights: dict | None


def sha256_file(path) -> str:
    digest = hashlib.sha256()
    with Path(path).open("rb") as stream:
        for block in iter(lambda: stream.read(8 << 20), b""):
            digest.update(block)
    return digest.hexdigest()


def tensor_sha256(tensor: torch.Tensor) -> str:
    """Content hash as the reference computes it: JSON descriptor of dtype and shape, a NUL, the bytes."""
    if tensor.device.type != "cpu":
        raise ValueError("artifact tensor hashing requires a CPU tensor")
    value = tensor.detach().contiguous()
    digest = hashlib.sha256()
    digest.update(json.dumps({"dtype": str(value.dtype), "shape": list(value.shape)}, sort_keys=True,
                             separators=(",", ":")).encode("utf-8"))
    digest.update(b"\0")
    digest.update(value.view(torch.uint8).numpy().tobytes())
    return digest.hexdigest()


def _sha(value, label):
    if not isinstance(value, str) or len(value) != 64 or any(c not in "0123456789abcdef" for c in value.lower()):
        raise ValueError(f"{label} must be a 64-character SHA256 hex digest")
    return value.lower()


def _local_path(value, base_dir: Path, label: str, must_exist: bool = True) -> Path:
    if not isinstance(value, (str, os.PathLike)):
        raise TypeError(f"{label} must be a local filesystem path")
    text = os.fspath(value)
    if urlsplit(text).scheme not in ("", "file") or "://" in text:
        raise ValueError(f"{label} must be a local path, not a URL")
    path = Path(text)
    path = (base_dir / path if not path.is_absolute() else path).resolve()
    if must_exist and not path.is_file():
        raise ValueError(f"{label} does not name an existing file: {path}")
    if path.suffix.lower() != ".pt":
        raise ValueError(f"{label} must be a local .pt weights-only bundle")
    return path


def validate_trace_tensors(x, expert_ids, route_weights, *, dims=QWEN3_30B_A3B):
    """The reference's rules for a captured trace (moe_real_trace.py:88-138); returns contiguous copies."""
    for name, t in (("x", x), ("expert_ids", expert_ids), ("route_weights", route_weights)):
        if not isinstance(t, torch.Tensor):
            raise TypeError(f"{name} must be a torch.Tensor")
        if t.device.type != "cpu":
            raise ValueError(f"{name} must be copied to CPU before artifact validation")
    if x.ndim != 2 or x.shape[0] <= 0 or x.shape[1] != dims["hidden"]:
        raise ValueError(f"x must have shape [T,{dims['hidden']}] with T > 0")
    if x.dtype != torch.bfloat16:
        raise TypeError("x must use bfloat16")
    if not torch.isfinite(x).all():
        raise ValueError("x contains nonfinite values")
    routes = (x.shape[0], dims["topk"])
    if tuple(expert_ids.shape) != routes or tuple(route_weights.shape) != routes:
        raise ValueError(f"expert_ids and route_weights must have shape {routes}")
    if expert_ids.dtype not in (torch.int32, torch.int64):
        raise TypeError("expert_ids must use int32 or int64")
    if torch.any((expert_ids < 0) | (expert_ids >= dims["experts"])):
        raise ValueError(f"expert_ids must lie in [0,{dims['experts']})")
    ordered = expert_ids.sort(dim=1).values
    if torch.any(ordered[:, 1:] == ordered[:, :-1]):
        raise ValueError("top-k expert IDs must be unique within each token")
    if route_weights.dtype != torch.float32:
        raise TypeError("route_weights must be stored as float32")
    if not torch.isfinite(route_weights).all() or torch.any(route_weights < 0):
        raise ValueError("route_weights must be finite and nonnegative")
    if not torch.equal(route_weights.to(torch.bfloat16).to(torch.float32), route_weights):
        raise ValueError("route_weights must be exact FP32 promotions of BF16 router outputs")
    return {"x": x.detach().contiguous().clone(), "expert_ids": expert_ids.detach().contiguous().clone(),
            "route_weights": route_weights.detach().contiguous().clone()}


def validate_weight_tensors(weights, *, dims=QWEN3_30B_A3B):
    shapes = {"gate_up": (dims["experts"], 2 * dims["intermediate"], dims["hidden"]),
              "down": (dims["experts"], dims["hidden"], dims["intermediate"])}
    if not isinstance(weights, dict) or set(weights) != set(shapes):
        raise ValueError("weights must contain exactly 'gate_up' and 'down'")
    for name, shape in shapes.items():
        t = weights[name]
        if not isinstance(t, torch.Tensor) or t.device.type != "cpu" or tuple(t.shape) != shape:
            raise ValueError(f"{name} must be a CPU tensor of shape {shape}")
        if t.dtype != torch.bfloat16:
            raise TypeError(f"{name} must use bfloat16")
        if not torch.isfinite(t).all():
            raise ValueError(f"{name} contains nonfinite values")
    return dict(weights)


def write_real_moe_trace(directory, x, expert_ids, route_weights, gate_up, down, *, name="trace",
                         dims=QWEN3_30B_A3B, provenance=None, repo_id=MODEL_REPO_ID, revision=MODEL_REVISION,
                         source_manifest_sha256=None) -> Path:
    """Write a trace bundle, a shared weight bundle and the manifest; returns the manifest path.

    The manifest has the fields of the reference's writer (moe_real_trace.py:314-352): ``status``, the ``model``
    block, the routing contract, per-tensor records, weight records with ``format`` / ``tensor_name`` /
    ``source_manifest_sha256``, and ``capture`` (``provenance``, any JSON mapping). With the default dimensions
    and model identity the reference's own ``validate_real_moe_trace`` accepts it."""
    if provenance is not None and not isinstance(provenance, dict):
        raise TypeError("provenance must be a JSON-safe mapping")
    capture = json.loads(json.dumps(dict(provenance or {}), allow_nan=False))
    directory = Path(directory)
    directory.mkdir(parents=True, exist_ok=True)
    tensors = validate_trace_tensors(x, expert_ids, route_weights, dims=dims)
    weights = validate_weight_tensors({"gate_up": gate_up, "down": down}, dims=dims)
    trace_path, weight_path = directory / f"{name}.pt", directory / f"{name}-weights.pt"
    torch.save(tensors, trace_path)
    torch.save({k: v.contiguous() for k, v in weights.items()}, weight_path)
    weight_sha = sha256_file(weight_path)
    source_sha = _sha(source_manifest_sha256 or weight_sha, "source_manifest_sha256")
    manifest = {
        "schema": SCHEMA, "schema_version": SCHEMA_VERSION, "status": "passed",
        "model": _model_block(dims, repo_id, revision), "routing_contract": dict(ROUTING_CONTRACT),
        "trace": {"path": trace_path.name, "sha256": sha256_file(trace_path), "format": TRACE_FORMAT,
                  "tensors": {k: {"shape": list(v.shape), "dtype": str(v.dtype).removeprefix("torch."),
                                  "sha256": tensor_sha256(v)} for k, v in tensors.items()}},
        "weights": {k: {"path": weight_path.name, "sha256": weight_sha, "format": WEIGHTS_FORMAT, "tensor_name": k,
                        "shape": list(v.shape), "dtype": "bfloat16", "source_manifest_sha256": source_sha}
                    for k, v in weights.items()},
        "capture": capture,
    }
    manifest_path = directory / f"{name}.json"
    partial = manifest_path.with_suffix(".json.partial")
    partial.write_text(json.dumps(manifest, indent=2, sort_keys=True, allow_nan=False) + "\n", encoding="utf-8")
    os.replace(partial, manifest_path)   # never a half-written manifest
    return manifest_path


def _validate_manifest(manifest, dims):
    """The manifest rules of the reference (moe_real_trace.py:357-445), with the dimensions taken from the
    manifest's own ``model`` block instead of being fixed to one model. Returns the dimensions."""
    if not isinstance(manifest, dict) or manifest.get("schema") != SCHEMA or manifest.get("schema_version") != 1:
        raise ValueError("not a moe_real_trace manifest of schema version 1")
    if manifest.get("status") != "passed":
        raise ValueError("real-MoE trace manifest is not marked passed")
    found = _dims_of(manifest.get("model"))
    if dims is not None and dict(dims) != found:
        raise ValueError(f"manifest describes {found}, expected {dict(dims)}")
    dims = found
    if manifest.get("routing_contract") != ROUTING_CONTRACT:
        raise ValueError("manifest routing contract differs from the fixed trace contract")
    if not isinstance(manifest.get("capture"), dict):
        raise ValueError("manifest capture metadata must be a JSON object")
    trace, weights = manifest.get("trace"), manifest.get("weights")
    if not isinstance(trace, dict) or not isinstance(weights, dict) or set(weights) != {"gate_up", "down"}:
        raise ValueError("manifest needs a trace record and gate_up / down weight records")
    if trace.get("format") != TRACE_FORMAT:
        raise ValueError("trace bundle format must be weights-only tensor dictionary")
    _sha(trace.get("sha256"), "trace.sha256")
    tensors = trace.get("tensors")
    if not isinstance(tensors, dict) or set(tensors) != set(TRACE_TENSOR_NAMES):
        raise ValueError("trace record must describe x, expert_ids and route_weights")
    token_counts = set()
    for name, rec in tensors.items():
        shape = rec.get("shape") if isinstance(rec, dict) else None
        if not isinstance(shape, list) or len(shape) != 2 or any(type(v) is not int for v in shape) or shape[0] <= 0:
            raise ValueError(f"trace.tensors.{name}.shape must be [T, n] with T > 0")
        _sha(rec.get("sha256"), f"trace.tensors.{name}.sha256")
        if shape[1] != (dims["hidden"] if name == "x" else dims["topk"]):
            raise ValueError(f"manifest {name} shape is incompatible with the model dimensions")
        allowed = {"x": ("bfloat16",), "expert_ids": ("int32", "int64"), "route_weights": ("float32",)}[name]
        if rec.get("dtype") not in allowed:
            raise ValueError(f"manifest {name} dtype must be one of {allowed}")
        token_counts.add(shape[0])
    if len(token_counts) != 1:
        raise ValueError("all manifest trace tensors must have the same token count T")
    shapes = {"gate_up": [dims["experts"], 2 * dims["intermediate"], dims["hidden"]],
              "down": [dims["experts"], dims["hidden"], dims["intermediate"]]}
    sources = set()
    for name, rec in weights.items():
        if not isinstance(rec, dict) or rec.get("format") != WEIGHTS_FORMAT or rec.get("tensor_name") != name:
            raise ValueError(f"manifest weights.{name} must declare a weights-only torch bundle holding {name!r}")
        if rec.get("shape") != shapes[name] or rec.get("dtype") != "bfloat16":
            raise ValueError(f"manifest weights.{name} shape/dtype violate the model dimensions")
        sources.add(_sha(rec.get("source_manifest_sha256"), f"weights.{name}.source_manifest_sha256"))
        _sha(rec.get("sha256"), f"weights.{name}.sha256")
    if len(sources) != 1:
        raise ValueError("gate_up and down must cite the same layer-extraction manifest")
    if (weights["gate_up"].get("path") != weights["down"].get("path")
            or weights["gate_up"].get("sha256") != weights["down"].get("sha256")):
        raise ValueError("gate_up and down must reference the same shared weight bundle")
    return dims


def validate_real_moe_trace(manifest_path, *, verify_hashes=True, load_trace=True, load_weights=False,
                            dims=None, check_weight_files=True) -> RealMoETrace:
    """Validate a manifest and optionally load its CPU tensors (``weights_only=True`` loads only).

    ``check_weight_files=False`` validates the weight records as written but does not require the (large)
    weight bundle to be present: for looking at a trace whose weights live elsewhere."""
    target = Path(manifest_path).expanduser().resolve(strict=True)
    manifest = json.loads(target.read_text(encoding="utf-8"))
    dims = _validate_manifest(manifest, dims)
    trace, weights = manifest["trace"], manifest["weights"]
    if load_weights and not check_weight_files:
        raise ValueError("load_weights needs the weight bundle: check_weight_files must stay True")
    base = target.parent
    records = {"trace": trace}
    if check_weight_files:
        records.update({"weights.gate_up": weights["gate_up"], "weights.down": weights["down"]})
    else:
        for key in ("gate_up", "down"):
            _local_path(weights[key].get("path"), base, f"weights.{key}.path", must_exist=False)
    paths = {key: _local_path(rec.get("path"), base, f"{key}.path") for key, rec in records.items()}
    if verify_hashes:
        cache = {}
        for key, rec in records.items():
            digest = cache.setdefault(paths[key], sha256_file(paths[key]))
            if digest != _sha(rec.get("sha256"), f"{key}.sha256"):
                raise ValueError(f"SHA256 mismatch for {key} artifact: {paths[key]}")
    tensors = loaded = None
    if load_trace:
        payload = torch.load(paths["trace"], map_location="cpu", weights_only=True)
        if not isinstance(payload, dict) or set(payload) != set(TRACE_TENSOR_NAMES):
            raise ValueError("trace .pt must contain only x, expert_ids, and route_weights tensors")
        tensors = validate_trace_tensors(payload["x"], payload["expert_ids"], payload["route_weights"], dims=dims)
        for name, tensor in tensors.items():
            rec = trace["tensors"][name]
            if list(tensor.shape) != rec["shape"] or str(tensor.dtype).removeprefix("torch.") != rec["dtype"]:
                raise ValueError(f"loaded trace tensor {name} disagrees with manifest metadata")
            if tensor_sha256(tensor) != rec["sha256"]:
                raise ValueError(f"tensor content hash mismatch for trace tensor {name}")
    if load_weights:
        bundle = torch.load(paths["weights.gate_up"], map_location="cpu", weights_only=True)
        if not isinstance(bundle, dict) or set(bundle) != {"gate_up", "down"}:
            raise ValueError("weight bundle must contain only gate_up and down")
        loaded = validate_weight_tensors({k: bundle[weights[k]["tensor_name"]] for k in ("gate_up", "down")},
                                         dims=dims)
    return RealMoETrace(manifest_path=target, manifest=manifest, tensors=tensors, weights=loaded)


def prepare_trace_moe(trace: RealMoETrace, device, **kwargs):
    """Bind a loaded trace (tensors and weights) to the prepared fixed-route layer on ``device``."""
    from .moe_ranked import prepare_ranked_moe_launcher
    if trace.tensors is None or trace.weights is None:
        raise ValueError("load the trace with load_trace=True and load_weights=True first")
    t, w = trace.tensors, trace.weights
    return prepare_ranked_moe_launcher(t["x"].to(device), w["gate_up"].to(device), w["down"].to(device),
                                       t["expert_ids"].to(device), t["route_weights"].to(device), **kwargs)
