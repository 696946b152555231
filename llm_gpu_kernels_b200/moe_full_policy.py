"""Shape-only schedule choice.

The reference freezes a tile policy keyed on ``mu = T*K/E`` with thresholds 8
and 64 (reference moe_full_policy.py:132-152, results/m7-policy.json) so that a
captured graph stays valid when routes change: nothing about the choice may
depend on ids or counts. The same rule holds here. ``select`` returns the
``GemmConfig`` whose ``block_m`` is the token tile the library would pick for
the shape, and the bucket name.
"""
import hashlib
import json
from dataclasses import dataclass
from pathlib import Path

from .gemm import GemmConfig

DEFAULT_POLICY = Path(__file__).resolve().parent / "policy" / "b200-policy.json"

BUCKET_NAMES = ("small", "medium", "large")
THRESHOLDS_MU = (8.0, 64.0)


def token_tile_for(tokens: int, experts: int, topk: int) -> int:
    """Twice the mean rows per expert as a power of two in [16,128]; 256 from 1024 rows per expert
    (the rule in csrc/abi.cu)."""
    routes = tokens * topk
    twice_mu = -(-2 * routes // experts)
    if twice_mu >= 2048:
        return 256
    tile = 16
    while tile < 128 and tile < twice_mu:
        tile <<= 1
    return tile


def select(T, E, topk, H, I):
    """Return ``(GemmConfig, bucket)`` from dimensions only; T may be zero."""
    tokens, experts, routed = int(T), int(E), int(topk)
    if tokens < 0:
        raise ValueError("T must be nonnegative")
    mu = tokens * routed / experts
    index = 0 if mu <= THRESHOLDS_MU[0] else 1 if mu <= THRESHOLDS_MU[1] else 2
    return GemmConfig(block_m=token_tile_for(tokens, experts, routed)), BUCKET_NAMES[index]


@dataclass(frozen=True)
class FrozenMoEPolicy:
    """File-backed form of the rule, with the reference's ``load`` / ``select`` surface
    (reference moe_full_policy.py:88-152). The file records the rule, the bucket thresholds and the
    B200 measurements behind it; ``sha256`` lets a caller pin the exact file it selected with."""
    path: str
    sha256: str
    thresholds: tuple
    fallback: GemmConfig

    @classmethod
    def load(cls, path=DEFAULT_POLICY):
        content = Path(path).read_bytes()
        data = json.loads(content)
        thresholds = tuple(float(v) for v in data["thresholds_mu"])
        if data.get("schema") != 1 or len(thresholds) != 2 or not thresholds[0] < thresholds[1]:
            raise ValueError("unsupported policy file")
        return cls(path=str(path), sha256=hashlib.sha256(content).hexdigest(), thresholds=thresholds,
                   fallback=GemmConfig(**data["fallback"]))

    def select(self, T, E, topk, H, I):
        """``(GemmConfig, bucket)`` from dimensions only. Shapes the tensor-core schedule cannot take
        (H or I not multiples of 8, or below 64) get the fallback config and ``"shape_fallback"``."""
        if int(T) < 0:
            raise ValueError("T must be nonnegative")
        if int(H) % 8 or int(I) % 8 or int(H) < 64 or int(I) < 64:
            return self.fallback, "shape_fallback"
        mu = int(T) * int(topk) / int(E)
        index = 0 if mu <= self.thresholds[0] else 1 if mu <= self.thresholds[1] else 2
        return GemmConfig(block_m=token_tile_for(int(T), int(E), int(topk))), BUCKET_NAMES[index]

    def verify_provenance(self, repository_root=None):
        """Re-hash the policy file; raises if it changed since it was loaded."""
        if hashlib.sha256(Path(self.path).read_bytes()).hexdigest() != self.sha256:
            raise ValueError("policy file changed since it was loaded")
        return {"path": self.path, "sha256": self.sha256}
