"""Parity at the sizes the tensor-bound schedule serves: the reference's own performance matrix
(mature_moe_benchmark.py:319-342: T in {1, 17, 193, 1024, 2049} random, hot16 at T in {193, 1024}), T = 4096 and
8192 on the Qwen3-30B-A3B layer shape, the skewed-routing stress (Zipf(1.2) popularity prior, some experts with
more than ten times the mean load and some with none), the same case through W4A16, and the Mixtral-8x7B layer
shape with the 256-row token tile.

Bars as everywhere: dispatch bit-exact, BF16 output within relative RMS 5e-3 (max-normalised 8e-3) of the FP32
oracle, W4A16 within 1e-2 of the oracle evaluated on the dequantised weights. Where the full oracle would take
minutes on host cores (Mixtral shape) it runs on a seeded token subsample plus strided rows; the dispatch check
always covers every route.
"""
import pytest
import torch

from oracle import moe_oracle as O
from tests.util import make_ids, seeded_layer, zipf_routes

pytestmark = pytest.mark.gpu

QWEN = dict(hidden=2048, inter=768, experts=128, topk=8)


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "these tests need a GPU"
    assert torch.cuda.get_device_capability(0)[0] == 10, "sm_100 (B200) required"
    return torch.device("cuda:0")


@pytest.fixture(scope="module")
def qwen(dev):
    wr, gate_up, down, _ = seeded_layer(0, 1, QWEN["hidden"], QWEN["inter"], QWEN["experts"])
    return {"cpu": (wr, gate_up, down), "gpu": (wr.to(dev), gate_up.to(dev), down.to(dev))}


def tokens_for(t, hidden, seed):
    return torch.randn(t, hidden, generator=torch.Generator().manual_seed(seed)).bfloat16()


def check_dispatch(base, x_cpu, ids_cpu, experts):
    counts, offsets, ranks, mapping = O.dispatch_oracle(ids_cpu, experts)
    assert torch.equal(base.counts.cpu(), counts), "counts"
    assert torch.equal(base.offsets.cpu(), offsets), "offsets"
    assert torch.equal(base.ranks.cpu(), ranks), "ranks"
    assert torch.equal(base.mapping.cpu(), mapping), "mapping"
    topk = ids_cpu.shape[1]
    if base.gathers:   # no expert-contiguous copy: source_rows is the inverse permutation the gate/up kernel reads
        q = torch.arange(mapping.numel())
        assert torch.equal(base.source_rows.cpu()[mapping.long()], (q // topk).to(torch.int32)), "source_rows"
    else:
        gathered = base.grouped_input.cpu()[mapping.long()]
        assert torch.equal(gathered, x_cpu.repeat_interleave(topk, 0)), "grouped_input"
    return counts


def check_rows(out, rows, x, gate_up, down, ids, rw, limit, norm_limit):
    """FP32 oracle on the token rows `rows` only (each output row depends on its own token only)."""
    ref = O.moe_oracle(x[rows], gate_up, down, ids[rows], rw[rows])
    m = O.error_metrics(out.float().cpu()[rows], ref)
    assert m["finite"] and m["relative_rms"] <= limit and m["normalized_max"] <= norm_limit, m
    return m


@pytest.mark.parametrize("tokens", [1, 2049, 4096])
def test_qwen_router_layer_large_and_single_token(dev, qwen, tokens):
    from llm_gpu_kernels_b200.moe_ranked import prepare_ranked_moe_launcher
    wr, gate_up, down = qwen["cpu"]
    x = tokens_for(tokens, QWEN["hidden"], 100 + tokens)
    ids = torch.zeros(tokens, 8, dtype=torch.int32, device=dev)
    rw = torch.zeros(tokens, 8, dtype=torch.float32, device=dev)
    wr_d, gate_up_d, down_d = qwen["gpu"]
    p = prepare_ranked_moe_launcher(x.to(dev), gate_up_d, down_d, ids, rw, router_weight=wr_d)
    out = p.run()
    torch.cuda.synchronize()
    p.check_inputs()
    ids_cpu, rw_cpu = ids.cpu(), rw.cpu()
    _, _, probs = O.router_oracle(x, wr, 8)
    ok, msg = O.router_agrees(ids_cpu, rw_cpu, probs, 8)
    assert ok, msg
    check_dispatch(p.base, x, ids_cpu, 128)
    m = check_rows(out, torch.arange(tokens), x, gate_up, down, ids_cpu, rw_cpu, 5e-3, 8e-3)
    print(f"T={tokens} tile={p.base.token_tile} rel_rms={m['relative_rms']:.2e}")
    assert torch.equal(p.run(), out)


@pytest.mark.parametrize("tokens", [193, 1024])
def test_qwen_hot16_fixed_routes(dev, qwen, tokens):
    """The reference's hot16 pattern: every token picks its 8 experts among 16 hot ones (64 rows per expert
    at T=128 ... 512 at T=1024), so each expert has several token tiles under the shape-only tile."""
    from llm_gpu_kernels_b200.moe_ranked import prepare_ranked_moe_launcher
    _, gate_up, down = qwen["cpu"]
    g = torch.Generator().manual_seed(7 + tokens)
    x = tokens_for(tokens, QWEN["hidden"], 200 + tokens)
    ids = make_ids(tokens, 128, 8, "hot", g).to(torch.int32)
    rw = torch.rand(tokens, 8, generator=g) * 2 - 1
    _, gate_up_d, down_d = qwen["gpu"]
    p = prepare_ranked_moe_launcher(x.to(dev), gate_up_d, down_d, ids.to(dev), rw.to(dev))
    out = p.run()
    torch.cuda.synchronize()
    p.check_inputs()
    counts = check_dispatch(p.base, x, ids, 128)
    assert int((counts > 0).sum()) == 16
    check_rows(out, torch.arange(tokens), x, gate_up, down, ids, rw, 5e-3, 8e-3)


@pytest.fixture(scope="module")
def skew_case():
    """Qwen shape, T = 8192, Zipf(1.2) expert popularity added to the router logits (seed 0)."""
    wr, _, _, _ = seeded_layer(0, 1, QWEN["hidden"], QWEN["inter"], QWEN["experts"])
    x = tokens_for(8192, QWEN["hidden"], 4)
    ids, rw = zipf_routes(x, wr, 8, 1.2, seed=0)
    return x, ids, rw


def test_qwen_skewed_routing_8192(dev, qwen, skew_case):
    from llm_gpu_kernels_b200.moe_ranked import prepare_ranked_moe_launcher
    _, gate_up, down = qwen["cpu"]
    _, gate_up_d, down_d = qwen["gpu"]
    x, ids, rw = skew_case
    p = prepare_ranked_moe_launcher(x.to(dev), gate_up_d, down_d, ids.to(dev), rw.to(dev), keep_grouped_input="never")
    assert p.base.token_tile == 128 and p.base.gathers
    out = p.run()
    torch.cuda.synchronize()
    p.check_inputs()
    counts = check_dispatch(p.base, x, ids, 128)
    mean = 8192 * 8 / 128
    assert int(counts.max()) > 10 * mean and int((counts == 0).sum()) > 0, "the stress must be skewed"
    m = check_rows(out, torch.arange(8192), x, gate_up, down, ids, rw, 5e-3, 8e-3)
    print(f"zipf T=8192 max/mean rows {int(counts.max()) / mean:.1f} empty {int((counts == 0).sum())} "
          f"rel_rms={m['relative_rms']:.2e}")
    assert torch.equal(p.run(), out)
    # the reference's materialised dispatch gives the same bits
    kept = prepare_ranked_moe_launcher(x.to(dev), gate_up_d, down_d, ids.to(dev), rw.to(dev), keep_grouped_input=True)
    assert not kept.base.gathers and torch.equal(kept.run(), out)
    check_dispatch(kept.base, x, ids, 128)
    # at this size (512 rows per expert on average) the shape-only choice is the materialised dispatch
    auto = prepare_ranked_moe_launcher(x.to(dev), gate_up_d, down_d, ids.to(dev), rw.to(dev))
    assert not auto.base.gathers and torch.equal(auto.run(), out)


def test_qwen_skewed_routing_8192_w4(dev, qwen, skew_case):
    from llm_gpu_kernels_b200.moe_w4_cuda import prepare_w4_moe
    from llm_gpu_kernels_b200.moe_weight_quant import dequantize_gate_up_reference, quantize_down, quantize_gate_up
    _, gate_up, down = qwen["cpu"]
    x, ids, rw = skew_case
    pg, pd = quantize_gate_up(gate_up), quantize_down(down)
    p = prepare_w4_moe(x.to(dev), pg.to(dev), None, ids.to(dev), rw.to(dev), packed_down=pd.to(dev))
    out = p.run()
    torch.cuda.synchronize()
    p.check_inputs()
    check_dispatch(p.base, x, ids, 128)
    rows = torch.arange(0, 8192, 4)   # a quarter of the tokens, strided: every expert's segment is sampled
    check_rows(out, rows, x, dequantize_gate_up_reference(pg), dequantize_gate_up_reference(pd), ids, rw, 1e-2, 1e-2)


@pytest.mark.parametrize("tile", [256, 128])
def test_mixtral_shape_prefill_tile(dev, tile):
    """Mixtral-8x7B layer shape (E8 H4096 I14336 top-2), T = 2048: 512 rows per expert on average, the
    large-prefill schedule. Oracle on a seeded 256-token subsample plus every 61st token."""
    from llm_gpu_kernels_b200.moe_ranked import prepare_ranked_moe_launcher
    e, h, i, k, t = 8, 4096, 14336, 2, 2048
    g = torch.Generator().manual_seed(0)
    wr = (0.02 * torch.randn(e, h, generator=g)).bfloat16()
    gate_up = torch.empty(e, 2 * i, h, dtype=torch.bfloat16)
    down = torch.empty(e, h, i, dtype=torch.bfloat16)
    for j in range(e):
        gate_up[j] = (0.02 * torch.randn(2 * i, h, generator=g)).bfloat16()
    for j in range(e):
        down[j] = (0.02 * torch.randn(h, i, generator=g)).bfloat16()
    x = torch.randn(t, h, generator=g).bfloat16()
    ids = torch.zeros(t, k, dtype=torch.int32, device=dev)
    rw = torch.zeros(t, k, dtype=torch.float32, device=dev)
    p = prepare_ranked_moe_launcher(x.to(dev), gate_up.to(dev), down.to(dev), ids, rw, router_weight=wr.to(dev),
                                    token_tile=tile)
    assert p.base.token_tile == tile
    out = p.run()
    torch.cuda.synchronize()
    p.check_inputs()
    ids_cpu, rw_cpu = ids.cpu(), rw.cpu()
    _, _, probs = O.router_oracle(x, wr, k)
    ok, msg = O.router_agrees(ids_cpu, rw_cpu, probs, k)
    assert ok, msg
    check_dispatch(p.base, x, ids_cpu, e)
    sample = torch.randperm(t, generator=torch.Generator().manual_seed(1))[:256]
    rows = torch.unique(torch.cat([sample, torch.arange(0, t, 61)]))
    m = check_rows(out, rows, x, gate_up, down, ids_cpu, rw_cpu, 5e-3, 8e-3)
    print(f"mixtral T={t} tile={tile} rows checked {rows.numel()} rel_rms={m['relative_rms']:.2e}")
    assert torch.equal(p.run(), out)


def test_reference_written_trace_replays(dev, golden_dir, tmp_path):
    """The committed bundle written by the reference's write_real_moe_trace, its weight bundle regenerated from
    the seed (content hashes pinned in golden_meta.json), through prepare_trace_moe: the output must match the
    reference's own moe_reference output stored beside the bundle."""
    import json
    import shutil
    from llm_gpu_kernels_b200.moe_real_trace import prepare_trace_moe, tensor_sha256, validate_real_moe_trace
    from tests.util import seeded_layer_per_expert
    meta = json.loads((golden_dir / "golden_meta.json").read_text())["real_trace"]
    _, gate_up, down = seeded_layer_per_expert(0, 2048, 768, 128)
    assert tensor_sha256(gate_up) == meta["gate_up_tensor_sha256"] and tensor_sha256(down) == meta["down_tensor_sha256"]
    for name in ("trace.json", "trace.pt"):
        shutil.copy(golden_dir / "ref_trace" / name, tmp_path / name)
    torch.save({"gate_up": gate_up, "down": down}, tmp_path / "weights.pt")
    trace = validate_real_moe_trace(tmp_path / "trace.json", verify_hashes=False, load_weights=True)
    prepared = prepare_trace_moe(trace, dev)
    out = prepared.run()
    torch.cuda.synchronize()
    prepared.check_inputs()
    want = torch.load(golden_dir / "ref_trace" / "reference_output.pt")["out"]
    m = O.error_metrics(out.float().cpu(), want)
    assert m["finite"] and m["relative_rms"] <= 5e-3 and m["normalized_max"] <= 8e-3, m
    check_dispatch(prepared.base, trace.tensors["x"], trace.tensors["expert_ids"], 128)
