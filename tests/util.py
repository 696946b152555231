"""Seeded input generators shared by the tests (CPU generator, then moved).

Route patterns restate reference moe_benchmark.py:43-64 (random / duplicate /
all_hot / hot); tensors follow moe_benchmark.py:67-82 (FP32 draws cast to
BF16, un-normalised uniform routing weights) with an optional weight scale.
"""
import hashlib

import torch


def digest(t):
    t = t.detach().cpu().contiguous()
    h = hashlib.sha256(str((str(t.dtype), tuple(t.shape))).encode())
    h.update(t.view(torch.uint8).numpy().tobytes())
    return h.hexdigest()


def make_ids(tokens, experts, topk, pattern, generator):
    if tokens == 0:
        return torch.empty((0, topk), dtype=torch.int64)
    if pattern == "duplicate":
        base = torch.arange(tokens)[:, None] % experts
        slots = torch.arange(topk)[None, :]
        return (base + slots // 2) % experts
    if pattern == "all_hot":
        return torch.zeros((tokens, topk), dtype=torch.int64)
    if pattern == "last_hot":
        return torch.full((tokens, topk), experts - 1, dtype=torch.int64)
    if pattern == "hot":
        hot = min(experts, max(topk, experts // 8))
        chosen = torch.randperm(experts, generator=generator)[:hot]
        return chosen[torch.rand((tokens, hot), generator=generator).topk(topk, dim=1).indices]
    if pattern == "balanced":
        return (torch.arange(tokens * topk).reshape(tokens, topk)) % experts
    if pattern == "random":
        return torch.rand((tokens, experts), generator=generator).topk(topk, dim=1).indices
    raise ValueError(pattern)


def make_inputs(tokens, experts, topk, hidden, inter, *, pattern="random", seed=0, id_dtype=torch.int32,
                wscale=1.0, signed=False, device="cpu"):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((tokens, hidden), generator=g).bfloat16()
    gate_up = (wscale * torch.randn((experts, 2 * inter, hidden), generator=g)).bfloat16()
    down = (wscale * torch.randn((experts, hidden, inter), generator=g)).bfloat16()
    ids = make_ids(tokens, experts, topk, pattern, g).to(id_dtype)
    rw = torch.rand((tokens, topk), generator=g)
    if signed:
        rw = rw * 2 - 1
    return tuple(t.to(device) for t in (x, gate_up, down, ids, rw))


def seeded_layer(seed, tokens, hidden, inter, experts, wscale=0.02, device="cpu"):
    """Draw order: router weight, gate_up, down, x (FP32 draws cast to BF16)."""
    g = torch.Generator().manual_seed(seed)
    wr = (wscale * torch.randn(experts, hidden, generator=g)).bfloat16()
    gate_up = (wscale * torch.randn(experts, 2 * inter, hidden, generator=g)).bfloat16()
    down = (wscale * torch.randn(experts, hidden, inter, generator=g)).bfloat16()
    x = torch.randn(tokens, hidden, generator=g).bfloat16()
    return tuple(t.to(device) for t in (wr, gate_up, down, x))


def zipf_bias(experts, s, seed=0):
    """log pmf of a Zipf(s) popularity over a seeded random permutation of the experts."""
    g = torch.Generator().manual_seed(seed)
    pmf = torch.arange(1, experts + 1, dtype=torch.float64) ** (-s)
    pmf = (pmf / pmf.sum())[torch.randperm(experts, generator=g)]
    return pmf.log().float()


def zipf_routes(x, router_weight, topk, s, seed=0):
    """Skewed routing stress: softmax top-k with renormalisation over router logits plus a Zipf(s)
    popularity prior (computed on the host: the device router has no bias input). Returns (ids int32, weights)."""
    logits = x.float() @ router_weight.float().T + zipf_bias(router_weight.shape[0], s, seed)
    weights, ids = torch.topk(torch.softmax(logits, dim=1), topk, dim=-1)
    return ids.to(torch.int32), (weights / weights.sum(-1, keepdim=True)).float()


def seeded_layer_per_expert(seed, hidden, inter, experts, wscale=0.02):
    """Router weight, gate_up, down with one FP32 draw per expert (the draw order of bench.py and of the
    golden real-trace bundle); bounds the FP32 temporaries at the Qwen shape."""
    g = torch.Generator().manual_seed(seed)
    wr = (wscale * torch.randn(experts, hidden, generator=g)).bfloat16()
    gate_up = torch.empty(experts, 2 * inter, hidden, dtype=torch.bfloat16)
    down = torch.empty(experts, hidden, inter, dtype=torch.bfloat16)
    for e in range(experts):
        gate_up[e] = (wscale * torch.randn(2 * inter, hidden, generator=g)).bfloat16()
    for e in range(experts):
        down[e] = (wscale * torch.randn(hidden, inter, generator=g)).bfloat16()
    return wr, gate_up, down
