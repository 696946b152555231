"""CPU restatement of the reference MoE-layer forward. TEST INFRASTRUCTURE ONLY.

Every function here restates, in plain PyTorch CPU ops, one piece of the
reference project (llm-gpu-kernels); the citation beside each function is the
reference file and line range it follows. The reference's own arithmetic on
this path is PyTorch FP32 (``@``, ``silu``, ``index_add_``, ``softmax``,
``topk``), so the restatement uses the same ops on CPU tensors.

Parity pin: ``tests/golden/`` holds vectors produced by importing the
reference's ``moe_reference`` / ``quantize_gate_up`` / ``repack_gate_up`` /
``validate_dispatch`` (see ``tests/golden/make_golden.py``); the CPU test
suite checks this file against them.  Two pieces have no counterpart in the
reference operator and are pinned only transitively: the router (the
reference holds its formula only inside an offline capture script) and the
W4 packing of the *down* projection (the reference packs gate/up only).

The shipped package never imports this module.
"""
from __future__ import annotations

import math

import torch
from torch.nn import functional as F

GROUP = 128  # W4 scale-group length along K (src/llm_gpu_kernels/moe_weight_quant.py:14)
LIMITS = {"relative_rms": 0.008, "normalized_max": 0.008}  # src/llm_gpu_kernels/benchmark.py:20


# --------------------------------------------------------------------------- router
def router_oracle(x, router_weight, topk, *, renormalize=True, bf16_logits=False,
                  bf16_weights=False):
    """Top-k softmax router with renormalisation.

    Follows scripts/capture_qwen3_moe_layer0.py:583-587: FP32 softmax over the
    router logits, ``topk``, then divide by the row sum. ``bf16_logits`` rounds
    the logits to BF16 first (what the captured model does); ``bf16_weights``
    rounds the final weights through BF16 (``:587-588``). Both default off: the
    operator under test keeps FP32 end to end.

    Returns (ids int32 [T,K], weights float32 [T,K], probs float32 [T,E]).
    """
    logits = x.float() @ router_weight.float().T
    if bf16_logits:
        logits = logits.to(torch.bfloat16).float()
    probs = torch.softmax(logits, dim=1, dtype=torch.float32)
    weights, ids = torch.topk(probs, topk, dim=-1)
    if renormalize:
        weights = weights / weights.sum(dim=-1, keepdim=True)
    if bf16_weights:
        weights = weights.to(torch.bfloat16).float()
    return ids.to(torch.int32), weights.float(), probs


def router_agrees(ids_gpu, weights_gpu, probs, topk, *, renormalize=True, tie_tol=2e-6,
                  weight_tol=2e-6):
    """Tie-aware comparison of a device router result with oracle probabilities.

    Two FP32 summation orders may legitimately pick different experts when two
    probabilities differ by less than ``tie_tol``. A row passes when every
    expert the device chose has a probability >= (k-th largest oracle
    probability - tie_tol), the ids are unique, and the weights equal the
    renormalised oracle probabilities of the *chosen* ids within ``weight_tol``.
    Returns (ok, message).
    """
    ids_gpu = ids_gpu.long()
    t, k = ids_gpu.shape
    if k != topk:
        return False, "topk mismatch"
    if t == 0:
        return True, "empty"
    if ((ids_gpu < 0) | (ids_gpu >= probs.shape[1])).any():
        return False, "id out of range"
    sorted_ids = ids_gpu.sort(dim=1).values
    if k > 1 and (sorted_ids[:, 1:] == sorted_ids[:, :-1]).any():
        return False, "duplicate expert in a row"
    kth = torch.topk(probs, topk, dim=-1).values[:, -1:]
    chosen = probs.gather(1, ids_gpu)
    if (chosen < kth - tie_tol).any():
        bad = int((chosen < kth - tie_tol).any(dim=1).nonzero()[0])
        return False, f"row {bad}: chose an expert below the top-k threshold"
    # descending order of the chosen probabilities (torch.topk order), ties aside
    if k > 1 and (chosen[:, 1:] > chosen[:, :-1] + tie_tol).any():
        return False, "chosen experts not in descending probability order"
    expect = chosen / chosen.sum(dim=-1, keepdim=True) if renormalize else chosen
    err = (weights_gpu.float() - expect).abs().max().item()
    if err > weight_tol:
        return False, f"routing weight error {err:.3e}"
    return True, f"max weight error {err:.3e}"


# --------------------------------------------------------------------------- dispatch
def dispatch_oracle(ids, experts):
    """Canonical ranked dispatch: counts, offsets, ranks, mapping.

    ``counts`` = bincount, ``offsets`` = exclusive prefix sum (the checks of
    src/llm_gpu_kernels/moe_benchmark.py:139-160). The reference assigns the
    rank of a route inside its expert by atomic arrival order
    (src/llm_gpu_kernels/moe_ranked.py:34-37) and validates only the
    invariants (ranked_moe_benchmark.py:120-167); the canonical order used
    here is the stable one, by flat route index ``q = token*K + slot``, which
    equals ``argsort(ids.flatten(), stable=True)`` - the host grouping the
    reference itself uses (optimization_benchmark.py:30).
    ``mapping[q] = offsets[id[q]] + ranks[q]`` (moe_ranked.py:52-59).
    Invalid ids get rank -1 / mapping -1 and are not counted.
    """
    flat = ids.reshape(-1).to(torch.int64)
    valid = (flat >= 0) & (flat < experts)
    safe = torch.where(valid, flat, torch.zeros_like(flat))
    counts = torch.bincount(safe[valid], minlength=experts).to(torch.int64)
    offsets = torch.cumsum(counts, 0) - counts
    ranks = torch.full_like(flat, -1)
    order = torch.argsort(torch.where(valid, flat, torch.full_like(flat, experts)), stable=True)
    nvalid = int(valid.sum())
    sorted_ids = flat[order[:nvalid]]
    position = torch.arange(nvalid, dtype=torch.int64)
    ranks[order[:nvalid]] = position - offsets[sorted_ids]
    mapping = torch.where(valid, offsets[safe] + ranks, torch.full_like(flat, -1))
    return (counts.to(torch.int32), offsets.to(torch.int32), ranks.to(torch.int32),
            mapping.to(torch.int32))


def status_oracle(ids, routing_weights, experts):
    """Device status word: 1 = id outside [0,E), 2 = non-finite routing weight.

    src/llm_gpu_kernels/moe.py:21-30, docs/MOE_USAGE.md:110-113.
    """
    flat = ids.reshape(-1).to(torch.int64)
    bad_id = bool(((flat < 0) | (flat >= experts)).any())
    bad_w = bool((~torch.isfinite(routing_weights)).any())
    return int(bad_id) | (int(bad_w) << 1)


def grouped_input_oracle(x, mapping, topk):
    """``grouped_input[mapping[q], :] = x[q // K, :]`` (moe_ranked.py:61-65)."""
    rows = mapping.numel()
    out = torch.zeros((rows, x.shape[1]), dtype=x.dtype)
    q = torch.arange(rows)
    ok = mapping >= 0
    out[mapping[ok].long()] = x[(q // topk)[ok]]
    return out


# --------------------------------------------------------------------------- experts
def moe_oracle(x, gate_up, down, expert_ids, routing_weights):
    """FP32 expert-loop MoE forward for fixed routing.

    Follows src/llm_gpu_kernels/reference.py:17-45: for every expert, gather
    its routes, ``projected = x @ gate_up[e].T`` in FP32, split into gate | up,
    ``silu(gate) * up``, project with ``down[e]``, scale by the route's weight
    and ``index_add_`` into the token's row. Duplicate expert ids in one token
    contribute separately; no renormalisation.
    gate_up is [E, 2I, H] (gate rows then up rows); down is [E, H, I].
    """
    if x.ndim != 2 or gate_up.ndim != 3 or down.ndim != 3:
        raise ValueError("invalid ranks")
    e, h, inter = down.shape
    if (tuple(gate_up.shape) != (e, 2 * inter, h) or x.shape[1] != h or expert_ids.ndim != 2
            or expert_ids.shape != routing_weights.shape or expert_ids.shape[0] != x.shape[0]
            or expert_ids.shape[1] == 0):
        raise ValueError("incompatible MoE shapes")
    if expert_ids.dtype not in (torch.int32, torch.int64):
        raise ValueError("integer expert IDs required")
    if bool(((expert_ids < 0) | (expert_ids >= e)).any()) or not bool(torch.isfinite(routing_weights).all()):
        raise ValueError("invalid expert IDs or nonfinite routing weights")
    out = torch.zeros(x.shape, dtype=torch.float32)
    for expert in range(e):
        tokens, slots = torch.where(expert_ids == expert)
        if tokens.numel() == 0:
            continue
        projected = x[tokens].float() @ gate_up[expert].float().T
        gate, up = projected[:, :inter], projected[:, inter:]
        value = (F.silu(gate) * up) @ down[expert].float().T
        out.index_add_(0, tokens, value * routing_weights[tokens, slots, None].float())
    return out


def per_route_oracle(x, gate_up, down, expert_ids, routing_weights):
    """Independent token-by-token, slot-by-slot statement of the same semantics.

    src/llm_gpu_kernels/benchmark.py:152-163 (the reference's cross-check of
    its own oracle, including duplicate ids). Pure-Python loops: small cases only.
    """
    out = torch.zeros(x.shape, dtype=torch.float32)
    for token in range(x.shape[0]):
        for slot in range(expert_ids.shape[1]):
            e = int(expert_ids[token, slot])
            g, u = (gate_up[e].float() @ x[token].float()).chunk(2)
            out[token] += routing_weights[token, slot] * (down[e].float() @ (F.silu(g) * u))
    return out


def error_metrics(actual, oracle):
    """rel-RMS and max-normalised error (src/llm_gpu_kernels/benchmark.py:28-38;
    empty-T handling of moe_benchmark.py:114-121)."""
    if tuple(actual.shape) != tuple(oracle.shape):
        raise ValueError(f"output shape mismatch: {tuple(actual.shape)} != {tuple(oracle.shape)}")
    if actual.numel() == 0:
        return {"passed": True, "empty": True, "finite": True, "relative_rms": 0.0,
                "normalized_max": 0.0, "max_abs": 0.0}
    actual, oracle = actual.float(), oracle.float()
    delta = actual - oracle
    rel = (delta.square().mean().sqrt() / oracle.square().mean().sqrt().clamp_min(1e-12)).item()
    nmax = (delta.abs().max() / oracle.abs().max().clamp_min(1e-12)).item()
    metrics = {"relative_rms": rel, "normalized_max": nmax, "max_abs": delta.abs().max().item(),
               "finite": bool(torch.isfinite(actual).all())}
    metrics["passed"] = metrics["finite"] and all(metrics[k] <= v for k, v in LIMITS.items())
    return metrics


# --------------------------------------------------------------------------- W4G128 format
def quantize_w4g128(weight):
    """Pack a BF16 ``[E, N, K]`` weight (K % 128 == 0) into W4G128.

    Follows src/llm_gpu_kernels/moe_weight_quant.py:55-84, generalised from the
    reference's hard-wired (128,1536,2048) to any shape: per (expert, output
    channel, group of 128 along K) ``scale = bf16(max|w| / 7)`` (1 when the
    group is all zero); ``q = clamp(round_half_even(w / float(scale)), -7, 7)``;
    nibble = q + 8; eight nibbles per int32 word, lowest nibble = earliest K.
    Returns (words int32 [E,N,K/8], scales bf16 [E,N,K/128]).
    """
    if weight.dtype != torch.bfloat16 or weight.ndim != 3 or weight.shape[2] % GROUP:
        raise ValueError("BF16 [E,N,K] with K % 128 == 0 required")
    e, n, k = weight.shape
    words = torch.empty((e, n, k // 8), dtype=torch.int32)
    scales = torch.empty((e, n, k // GROUP), dtype=torch.bfloat16)
    shifts = torch.arange(8, dtype=torch.int64) * 4
    for expert in range(e):
        w = weight[expert].float().reshape(n, k // GROUP, GROUP)
        max_abs = w.abs().amax(-1)
        scale = torch.where(max_abs == 0, torch.ones_like(max_abs), max_abs / 7).to(torch.bfloat16)
        q = torch.round(w / scale.float()[..., None]).clamp(-7, 7).long()
        word = ((q.reshape(n, k // 8, 8) + 8) << shifts).sum(-1)
        # values above 2**31 wrap into the int32 bit pattern of the uint32 word
        words[expert] = ((word + 2**31) % 2**32 - 2**31).to(torch.int32)
        scales[expert] = scale
    return words, scales


def dequantize_w4g128(words, scales):
    """``bf16_rn(float(q) * float(scale))`` (moe_weight_quant.py:35-52; the device
    contract of cuda_w4_gate_up.cu:36-41). Returns BF16 [E,N,K]."""
    e, n, kw = words.shape
    k = kw * 8
    out = torch.empty((e, n, k), dtype=torch.bfloat16)
    shifts = torch.arange(8, dtype=torch.int64) * 4
    for expert in range(e):
        nibble = (words[expert].long()[..., None] >> shifts) & 15
        q = (nibble.reshape(n, k // GROUP, GROUP) - 8).float()
        out[expert] = (q * scales[expert].float()[..., None]).reshape(n, k).to(torch.bfloat16)
    return out


def repack_v2(words, scales, intermediate):
    """Bit-preserving v1 -> v2 permutation of packed gate/up.

    src/llm_gpu_kernels/moe_weight_layout.py:85-88:
    ``words_v2[e,p,nt,kt,w,nl] = words_v1[e, p*I + nt*64 + nl, kt*4 + w]`` and
    ``scales_v2[e,p,nt,kg,nl] = scales_v1[e, p*I + nt*64 + nl, kg]``.
    """
    e, n2, kw = words.shape
    nt, kt = intermediate // 64, kw // 4
    w2 = words.reshape(e, 2, nt, 64, kt, 4).permute(0, 1, 2, 4, 5, 3).contiguous()
    s2 = scales.reshape(e, 2, nt, 64, scales.shape[2]).permute(0, 1, 2, 4, 3).contiguous()
    return w2, s2


def restore_v1(words_v2, scales_v2):
    """Inverse of :func:`repack_v2` (moe_weight_layout.py:158-161)."""
    e, _, nt, kt, _, _ = words_v2.shape
    w1 = words_v2.permute(0, 1, 2, 5, 3, 4).contiguous().reshape(e, 2 * nt * 64, kt * 4)
    s1 = scales_v2.permute(0, 1, 2, 4, 3).contiguous().reshape(e, 2 * nt * 64, scales_v2.shape[3])
    return w1, s1


# --------------------------------------------------------------------------- whole layer
def moe_layer_oracle(x, router_weight, gate_up, down, topk):
    """Router followed by the expert forward; returns (out fp32, ids, weights)."""
    ids, weights, _ = router_oracle(x, router_weight, topk)
    return moe_oracle(x, gate_up, down, ids, weights), ids, weights


def algorithmic_work(tokens, experts, topk, hidden, intermediate, active_experts, w4=False):
    """(flops, bytes) one forward must do: 6*R*H*I + 2*T*H*E flops; each active
    expert's weights once, the router weight, x in, output out, ids+weights."""
    r = tokens * topk
    flops = 6 * r * hidden * intermediate + 2 * tokens * hidden * experts
    per_expert = 3 * hidden * intermediate * (0.5 if w4 else 2)
    if w4:
        per_expert += (2 * intermediate * hidden // GROUP + hidden * intermediate // GROUP) * 2
    nbytes = active_experts * per_expert + experts * hidden * 2 + 2 * tokens * hidden * 2 + tokens * topk * 8
    return flops, int(nbytes)


def cpu_threads():
    return torch.get_num_threads()


def _selfcheck():  # pragma: no cover - manual sanity
    g = torch.Generator().manual_seed(0)
    x = torch.randn(5, 16, generator=g).bfloat16()
    gu = torch.randn(3, 8, 16, generator=g).bfloat16()
    dn = torch.randn(3, 16, 4, generator=g).bfloat16()
    ids = torch.tensor([[0, 0], [2, 1], [1, 2], [0, 1], [2, 2]])
    rw = torch.rand(5, 2, generator=g)
    a, b = moe_oracle(x, gu, dn, ids, rw), per_route_oracle(x, gu, dn, ids, rw)
    assert error_metrics(a, b)["relative_rms"] < 1e-6
    assert math.isfinite(a.sum().item())


if __name__ == "__main__":
    _selfcheck()
    print("ok")
