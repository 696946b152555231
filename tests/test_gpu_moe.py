"""Parity of the CUDA path (through the C ABI) with the CPU oracle on a B200.

Bars: dispatch counts / offsets / ranks / mapping / grouped_input bit-exact;
BF16 outputs within relative RMS 5e-3 of the FP32 oracle (and within the
reference's own 8e-3 max-normalised gate, reference benchmark.py:20).
"""
import pytest
import torch

from oracle import moe_oracle as O
from tests.util import make_inputs, seeded_layer

pytestmark = pytest.mark.gpu

REL_RMS_BF16 = 5e-3   # the stated tolerance for BF16 outputs
NORM_MAX = 8e-3       # reference gate on max|delta| / max|ref|


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "these tests need a GPU"
    assert torch.cuda.get_device_capability(0)[0] == 10, "sm_100 (B200) required"
    return torch.device("cuda:0")


def prep(entry="ranked", **kw):
    from llm_gpu_kernels_b200.moe import prepare_moe
    from llm_gpu_kernels_b200.moe_ranked import prepare_ranked_moe_launcher
    return {"ranked": prepare_ranked_moe_launcher, "base": prepare_moe}[entry]


def check_output(out, cpu_args, limit=REL_RMS_BF16):
    ref = O.moe_oracle(*cpu_args)
    m = O.error_metrics(out.float().cpu(), ref)
    assert m["finite"], m
    assert m["relative_rms"] <= limit and m["normalized_max"] <= NORM_MAX, m
    return m


def check_dispatch(base, x_cpu, ids_cpu, experts):
    counts, offsets, ranks, mapping = O.dispatch_oracle(ids_cpu, experts)
    assert torch.equal(base.counts.cpu(), counts), "counts"
    assert torch.equal(base.offsets.cpu(), offsets), "offsets"
    assert torch.equal(base.ranks.cpu(), ranks), "ranks"
    assert torch.equal(base.mapping.cpu(), mapping), "mapping"
    topk = ids_cpu.shape[1]
    if base.gathers:   # no expert-contiguous copy: source_rows is the inverse permutation the gate/up kernel reads
        assert base.grouped_input.numel() == 0
        valid = mapping >= 0
        q = torch.arange(mapping.numel())[valid]
        assert torch.equal(base.source_rows.cpu()[mapping[valid].long()], (q // topk).to(torch.int32)), "source_rows"
    elif mapping.numel() and (mapping >= 0).all():
        gathered = base.grouped_input.cpu()[mapping.long()]
        assert torch.equal(gathered, x_cpu.repeat_interleave(topk, 0)), "grouped_input"


# --- the reference's odd-shape functional matrix (moe_benchmark.py:356-376), CUDA-core schedule
ODD = [
    (5, 1, 1, 31, 17, torch.int32, "random", False),
    (7, 3, 2, 33, 19, torch.int64, "random", True),
    (9, 8, 4, 47, 25, torch.int32, "duplicate", False),
    (17, 16, 8, 64, 32, torch.int64, "random", True),
    (19, 16, 4, 67, 33, torch.int32, "all_hot", False),
    (33, 8, 2, 40, 24, torch.int32, "duplicate", True),
    (31, 3, 2, 131, 67, torch.int32, "random", False),   # moe_full_holdout.py:52-56
    (1, 4, 1, 17, 9, torch.int32, "random", False),
]


@pytest.mark.parametrize("t,e,k,h,i,dt,pattern,signed", ODD)
def test_odd_shapes_generic(dev, t, e, k, h, i, dt, pattern, signed):
    cpu = make_inputs(t, e, k, h, i, pattern=pattern, seed=11 + t, id_dtype=dt, signed=signed)
    gpu = tuple(a.to(dev) for a in cpu)
    p = prep()(*gpu)
    assert p.base.schedule == "generic"
    out = p.run()
    torch.cuda.synchronize()
    p.check_inputs()
    assert out.dtype == torch.bfloat16 and tuple(out.shape) == (t, h)
    check_dispatch(p.base, cpu[0], cpu[3], e)
    check_output(out, cpu)


# --- tensor-core schedule: small aligned shapes incl. ragged K tails and many token tiles
TC = [
    (64, 8, 2, 256, 128, "random", 0),       # the tiny benchmark shape, fixed routes
    (17, 16, 4, 128, 64, "random", 16),
    (33, 4, 2, 192, 96, "duplicate", 16),    # K tails: 192 = 3x64, 96 = 64 + 32
    (40, 8, 8, 72, 200, "random", 32),       # H, I not multiples of 64 / 128
    (300, 4, 2, 256, 128, "all_hot", 64),    # one expert owns 600 rows: 10 token tiles
    (257, 3, 4, 128, 384, "last_hot", 256),  # token tile 256 (single TMEM buffer)
    (129, 16, 4, 320, 136, "hot", 128),
]


@pytest.mark.parametrize("keep", [False, True])
@pytest.mark.parametrize("t,e,k,h,i,pattern,tile", TC)
def test_tcgen05_small_shapes(dev, t, e, k, h, i, pattern, tile, keep):
    """keep=False: the gate/up kernel gathers the token rows itself (no grouped_input); keep=True: the dispatch
    materialises grouped_input as the reference does. Same bits either way."""
    cpu = make_inputs(t, e, k, h, i, pattern=pattern, seed=100 + t, wscale=0.1, signed=True)
    gpu = tuple(a.to(dev) for a in cpu)
    p = prep()(*gpu, schedule="tcgen05", token_tile=tile, keep_grouped_input=keep)
    assert p.base.schedule == "tcgen05" and p.base.gathers == (not keep)
    out = p.run()
    torch.cuda.synchronize()
    p.check_inputs()
    check_dispatch(p.base, cpu[0], cpu[3], e)
    check_output(out, cpu)
    if not keep:   # gathered and materialised rows give the same bits
        assert torch.equal(prep()(*gpu, schedule="tcgen05", token_tile=tile, keep_grouped_input=True).run(), out)
    # same inputs through the CUDA-core schedule agree as well (two independent kernels)
    q = prep()(*gpu, schedule="generic")
    m = O.error_metrics(out.float().cpu(), q.run().float().cpu())
    assert m["relative_rms"] <= REL_RMS_BF16, m


@pytest.mark.parametrize("t,e,k,h,i,pattern,tile", [c for c in TC if 0 < c[6] <= 128])
def test_down_pair_tiles(dev, t, e, k, h, i, pattern, tile):
    """The down projection over 256-channel pair tiles (one MMA issuer per 128 channels, no partial sums) at every
    token tile it serves, including H that is not a multiple of 256 (the second weight box runs past the expert)."""
    cpu = make_inputs(t, e, k, h, i, pattern=pattern, seed=100 + t, wscale=0.1, signed=True)
    gpu = tuple(a.to(dev) for a in cpu)
    p = prep()(*gpu, schedule="tcgen05", token_tile=tile, down_pair=True)
    assert p.base.down_pair and p.base.token_tile == tile
    out = p.run()
    torch.cuda.synchronize()
    p.check_inputs()
    check_output(out, cpu)
    split = prep()(*gpu, schedule="tcgen05", token_tile=tile, down_pair=False)
    assert not split.base.down_pair
    m = O.error_metrics(out.float().cpu(), split.run().float().cpu())
    assert m["relative_rms"] <= REL_RMS_BF16, m


@pytest.mark.parametrize("t,e,k,h,i,pattern", [(129, 16, 4, 320, 136, "hot"), (300, 4, 2, 256, 128, "all_hot"),
                                               (700, 8, 2, 192, 200, "random"), (64, 8, 2, 256, 128, "random")])
@pytest.mark.parametrize("keep", [False, True])
def test_down_wide_tiles(dev, t, e, k, h, i, pattern, keep):
    """down_tiles = 3: gate/up and the `tasks` prefix keep token tile 128, the down kernel re-tiles every expert at
    256 rows from the counts (experts of 600 rows = 256 + 256 + 88, of 30 rows, of none)."""
    cpu = make_inputs(t, e, k, h, i, pattern=pattern, seed=300 + t, wscale=0.1, signed=True)
    gpu = tuple(a.to(dev) for a in cpu)
    p = prep()(*gpu, schedule="tcgen05", token_tile=128, down_tiles=3, keep_grouped_input=keep)
    assert p.base.down_tiles == 3 and not p.base.down_pair and p.base.token_tile == 128
    out = p.run()
    torch.cuda.synchronize()
    p.check_inputs()
    check_dispatch(p.base, cpu[0], cpu[3], e)
    check_output(out, cpu)
    assert torch.equal(p.run(), out)
    pair = prep()(*gpu, schedule="tcgen05", token_tile=128, down_tiles=1, keep_grouped_input=keep)
    assert pair.base.down_tiles == 1
    m = O.error_metrics(out.float().cpu(), pair.run().float().cpu())
    assert m["relative_rms"] <= REL_RMS_BF16, m
    with pytest.raises(ValueError):
        prep()(*gpu, schedule="tcgen05", token_tile=64, down_tiles=3)


@pytest.mark.parametrize("tokens", [17, 193, 1024])
def test_qwen_shape_full_layer(dev, tokens):
    """benchmark configuration 2: router + experts, Qwen3-30B-A3B layer shape, seeded synthetic weights."""
    from llm_gpu_kernels_b200.moe_ranked import prepare_ranked_moe_launcher
    wr, gate_up, down, x = seeded_layer(0, tokens, 2048, 768, 128)
    ids = torch.zeros(tokens, 8, dtype=torch.int32, device=dev)
    rw = torch.zeros(tokens, 8, dtype=torch.float32, device=dev)
    p = prepare_ranked_moe_launcher(x.to(dev), gate_up.to(dev), down.to(dev), ids, rw, router_weight=wr.to(dev))
    assert p.names == ("router", "dispatch", "gate_up_swiglu", "down", "combine")
    assert p.base.schedule == "tcgen05"
    out = p.run()
    torch.cuda.synchronize()
    p.check_inputs()
    ids_cpu, rw_cpu = ids.cpu(), rw.cpu()
    _, _, probs = O.router_oracle(x, wr, 8)
    ok, msg = O.router_agrees(ids_cpu, rw_cpu, probs, 8)
    assert ok, msg
    check_dispatch(p.base, x, ids_cpu, 128)
    # experts are compared on the routes the device chose (ties between FP32 orders are legal)
    m = check_output(out, (x, gate_up, down, ids_cpu, rw_cpu))
    print(f"T={tokens} rel_rms={m['relative_rms']:.2e} norm_max={m['normalized_max']:.2e}")
    # determinism: three runs, identical bits
    first = out.clone()
    for _ in range(2):
        assert torch.equal(p.run(), first)


ROUTER = [
    (64, 8, 2, 256, 128, None),       # tensor-core router, E padded to 16 columns
    (300, 20, 5, 192, 64, None),      # three token tiles, E = 20 -> 32 columns, ragged last tile
    (130, 256, 32, 128, 64, None),    # widest supported: E = 256, K = 32
    (40, 16, 4, 128, 64, "generic"),  # CUDA-core router on an aligned shape
    (9, 3, 3, 67, 33, None),          # odd H: CUDA-core router and GEMMs
    (5, 130, 8, 96, 72, None),
]


@pytest.mark.parametrize("t,e,k,h,i,schedule", ROUTER)
def test_router_shapes(dev, t, e, k, h, i, schedule):
    from llm_gpu_kernels_b200.moe_ranked import prepare_ranked_moe_launcher
    wr, gate_up, down, x = seeded_layer(3 + t, t, h, i, e, wscale=0.05)
    for id_dtype in (torch.int32, torch.int64):
        ids = torch.zeros(t, k, dtype=id_dtype, device=dev)
        rw = torch.zeros(t, k, dtype=torch.float32, device=dev)
        p = prepare_ranked_moe_launcher(x.to(dev), gate_up.to(dev), down.to(dev), ids, rw,
                                        router_weight=wr.to(dev), schedule=schedule)
        out = p.run()
        torch.cuda.synchronize()
        p.check_inputs()
        _, _, probs = O.router_oracle(x, wr, k)
        ok, msg = O.router_agrees(ids.cpu(), rw.cpu(), probs, k)
        assert ok, msg
        check_dispatch(p.base, x, ids.cpu(), e)
        check_output(out, (x, gate_up, down, ids.cpu(), rw.cpu()))


@pytest.mark.parametrize("pattern", ["random", "hot", "all_hot"])
def test_large_route_count_multi_block_dispatch(dev, pattern):
    """R = 20000 routes takes the multi-block count / scan / permute path."""
    cpu = make_inputs(2500, 64, 8, 64, 64, pattern=pattern, seed=77, wscale=0.2, signed=True)
    gpu = tuple(a.to(dev) for a in cpu)
    p = prep()(*gpu)
    out = p.run()
    torch.cuda.synchronize()
    p.check_inputs()
    check_dispatch(p.base, cpu[0], cpu[3], 64)
    check_output(out, cpu)


@pytest.mark.parametrize("tokens,dt", [(300, torch.int32), (1000, torch.int64), (2040, torch.int32), (2048, torch.int32)])
@pytest.mark.parametrize("pattern", ["random", "hot", "all_hot"])
def test_cluster_dispatch(dev, tokens, dt, pattern):
    """2049..16384 routes: the one-kernel dispatch as a thread-block cluster of 2 / 4 / 8 blocks that exchange their
    per-expert totals through distributed shared memory. Same stable order, bit-exact; a bad id and a non-finite
    weight in the LAST block's routes reach the status word that block 0 writes."""
    cpu = make_inputs(tokens, 64, 8, 64, 64, pattern=pattern, seed=78, wscale=0.2, signed=True, id_dtype=dt)
    gpu = tuple(a.to(dev) for a in cpu)
    p = prep()(*gpu)
    out = p.run()
    torch.cuda.synchronize()
    p.check_inputs()
    check_dispatch(p.base, cpu[0], cpu[3], 64)
    check_output(out, cpu)
    ids, rw = gpu[3], gpu[4]
    ids[tokens - 1, 7] = 64
    rw[tokens - 2, 3] = float("inf")
    p.run()
    assert int(p.base.status.item()) == 3
    assert int(p.base.mapping[-1]) == -1 and int(p.base.ranks[-1]) == -1


@pytest.mark.parametrize("schedule", [None, "generic"])
def test_router_bf16_rounded_weights(dev, schedule):
    """The captured model's convention: weights rounded through BF16, then promoted (capture script :587-588)."""
    from llm_gpu_kernels_b200.moe_ranked import prepare_ranked_moe_launcher
    wr, gate_up, down, x = seeded_layer(8, 70, 256, 128, 16, wscale=0.05)
    ids = torch.zeros(70, 4, dtype=torch.int32, device=dev)
    rw = torch.zeros(70, 4, dtype=torch.float32, device=dev)
    p = prepare_ranked_moe_launcher(x.to(dev), gate_up.to(dev), down.to(dev), ids, rw, router_weight=wr.to(dev),
                                    schedule=schedule, router_bf16_weights=True)
    out = p.run()
    torch.cuda.synchronize()
    got = rw.cpu()
    assert torch.equal(got.bfloat16().float(), got)                 # exact promotions of BF16 values
    ref_ids, ref_w, _ = O.router_oracle(x, wr, 4, bf16_weights=True)
    same = ids.cpu() == ref_ids
    assert same.float().mean() > 0.99
    assert (got[same] - ref_w[same]).abs().max() <= 2.0 ** -8       # at most one BF16 step apart
    check_output(out, (x, gate_up, down, ids.cpu(), got))


@pytest.mark.parametrize("schedule,h", [(None, 256), ("generic", 100)])
def test_residual_added_in_combine(dev, schedule, h):
    """output = bf16(residual + bf16(layer)): bit-identical to the plain layer followed by a BF16 add."""
    from llm_gpu_kernels_b200.moe_ranked import prepare_ranked_moe_launcher
    args = make_inputs(45, 8, 3, h, 128 if h == 256 else 72, seed=13, wscale=0.1, device=dev)
    plain = prepare_ranked_moe_launcher(*args, schedule=schedule).run().clone()
    residual = torch.randn(45, h, generator=torch.Generator().manual_seed(4)).bfloat16().to(dev)
    fused = prepare_ranked_moe_launcher(*args, schedule=schedule, residual=residual)
    want = (residual.float() + plain.float()).bfloat16()
    assert torch.equal(fused.run(), want)
    residual.mul_(-2.0)                      # read every forward, not captured at prepare time
    assert torch.equal(fused.run(), (residual.float() + plain.float()).bfloat16())
    with pytest.raises(ValueError):
        prepare_ranked_moe_launcher(*args, residual=residual.float())


def test_tiny_layer_golden(dev, golden_dir):
    """benchmark configuration 1 against the reference's own output on the same seeded inputs."""
    from llm_gpu_kernels_b200.moe_ranked import prepare_ranked_moe_launcher
    g = torch.load(golden_dir / "tiny_layer_seed0.pt")
    wr, gate_up, down, x = seeded_layer(0, 64, 256, 128, 8)
    ids = torch.zeros(64, 2, dtype=torch.int32, device=dev)
    rw = torch.zeros(64, 2, dtype=torch.float32, device=dev)
    p = prepare_ranked_moe_launcher(x.to(dev), gate_up.to(dev), down.to(dev), ids, rw, router_weight=wr.to(dev))
    out = p.run()
    torch.cuda.synchronize()
    assert torch.equal(ids.cpu(), g["ids"])
    assert torch.allclose(rw.cpu(), g["rw"], atol=2e-6, rtol=0)
    m = O.error_metrics(out.float().cpu(), g["out"])
    assert m["relative_rms"] <= REL_RMS_BF16 and m["normalized_max"] <= NORM_MAX, m


def test_mini_fixed_route_golden(dev, golden_dir):
    g = torch.load(golden_dir / "mini_fixed_route.pt")
    args = [g[k].to(dev) for k in ("x", "gate_up", "down", "ids", "rw")]
    p = prep()(*args)
    out = p.run()
    torch.cuda.synchronize()
    m = O.error_metrics(out.float().cpu(), g["out"])
    assert m["relative_rms"] <= REL_RMS_BF16 and m["normalized_max"] <= NORM_MAX, m
    check_dispatch(p.base, g["x"], g["ids"], 4)


def test_status_flags(dev):
    """reference moe_benchmark.py:209-240: bad id -> 1, NaN weight -> 2, check_inputs raises."""
    from llm_gpu_kernels_b200.moe import prepare_moe
    for kind, expected in (("id", 1), ("weight", 2), ("both", 3)):
        x, gu, dn, ids, rw = make_inputs(3, 4, 2, 64, 64, seed=101, device=dev)
        if kind in ("id", "both"):
            ids[0, 0] = 4
        if kind in ("weight", "both"):
            rw[1, 1] = float("nan")
        p = prepare_moe(x, gu, dn, ids, rw)
        with pytest.raises(ValueError, match=f"status={expected}"):
            p.check_inputs()
        assert int(p.status.item()) == expected
        if kind == "id":
            assert int(p.mapping[0]) == -1 and int(p.ranks[0]) == -1
            # repairing the id in place clears the status on the next forward
            ids[0, 0] = 3
            p.run()
            p.check_inputs()
    x, gu, dn, ids, rw = make_inputs(3, 4, 2, 64, 64, seed=5, device=dev)
    rw[2, 0] = float("-inf")
    ids[1, 1] = -7
    assert int(prepare_moe(x, gu, dn, ids, rw).status.item()) == 3


def test_empty_tokens(dev):
    x, gu, dn, ids, rw = make_inputs(0, 4, 2, 128, 64, device=dev)
    p = prep()(x, gu, dn, ids, rw)
    out = p.run()
    assert p.launches == () and tuple(out.shape) == (0, 128) and out.dtype == torch.bfloat16
    p.check_inputs()


def test_workspace_contract(dev):
    """Buffers are distinct storages, owned by the plan (reference moe_benchmark.py:193-206)."""
    args = make_inputs(9, 8, 2, 128, 64, device=dev)
    p = prep()(*args, keep_grouped_input=True)
    b = p.base
    names = ("output", "counts", "offsets", "cursors", "tasks", "mapping", "grouped_input", "projected",
             "activated", "down_output", "status")
    ws = [getattr(b, n).untyped_storage()._cdata for n in names]
    user = {t.untyped_storage()._cdata for t in args}
    assert len(set(ws)) == len(ws) and not (set(ws) & user)
    assert p.workspace_bytes == b.workspace_bytes + 9 * 2 * 4
    assert tuple(b.grouped_input.shape) == (18, 128) and tuple(b.activated.shape) == (18, 64)
    assert b.tasks.numel() == 9 and int(b.cursors.abs().sum()) == 0
    total_tiles = int(b.tasks[-1])
    assert total_tiles == int(((b.counts + b.token_tile - 1) // b.token_tile).sum())


def test_stage_calls_equal_run(dev):
    args = make_inputs(50, 8, 4, 256, 128, seed=3, wscale=0.1, device=dev)
    p = prep()(*args)
    whole = p.run().clone()
    p.base.output.zero_()
    p.base.activated.zero_()
    for launch in p.launches:
        launch.run()
    torch.cuda.synchronize()
    assert torch.equal(p.base.output, whole)
    b = p.base
    b.output.zero_()
    b.dispatch(); b.project(); b.activate(); b.down_project(); b.combine()
    assert torch.equal(b.output, whole)


def test_graph_replay_with_in_place_updates(dev):
    """reference moe_benchmark.py:290-321: capture, copy_ new x / ids / signed weights into the same
    addresses, replay, verify; all-to-one-expert stress under the same graph (moe_cuda_audit.py:102-105)."""
    t, e, k, h, i = 96, 16, 4, 256, 128
    cpu = make_inputs(t, e, k, h, i, seed=21, wscale=0.1)
    gpu = tuple(a.to(dev) for a in cpu)
    p = prep()(*gpu)
    for _ in range(3):
        p.run()
    torch.cuda.synchronize()
    stream = torch.cuda.Stream(device=dev)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        for _ in range(2):
            out = p.run()
    graph.replay()
    torch.cuda.synchronize()
    check_output(out, cpu)
    for seed, pattern in ((22, "random"), (23, "all_hot"), (24, "last_hot"), (25, "duplicate")):
        new = make_inputs(t, e, k, h, i, seed=seed, pattern=pattern, wscale=0.1, signed=True)
        gpu[0].copy_(new[0]); gpu[3].copy_(new[3]); gpu[4].copy_(new[4])
        graph.replay()
        torch.cuda.synchronize()
        p.check_inputs()
        fresh = (new[0], cpu[1], cpu[2], new[3], new[4])
        check_output(out, fresh)
        check_dispatch(p.base, new[0], new[3], e)


def test_side_stream(dev):
    """Update and run on a non-default stream (reference moe_cuda_audit.py:106-122)."""
    cpu = make_inputs(40, 8, 2, 128, 128, seed=31, wscale=0.1)
    gpu = tuple(a.to(dev) for a in cpu)
    p = prep()(*gpu)
    new = make_inputs(40, 8, 2, 128, 128, seed=32, wscale=0.1)
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        gpu[0].copy_(new[0].to(dev), non_blocking=True)
        gpu[3].copy_(new[3].to(dev), non_blocking=True)
        out = p.run()
    side.synchronize()
    check_output(out, (new[0], cpu[1], cpu[2], new[3], cpu[4]))


def test_configured_and_cuda_entry_points(dev):
    from llm_gpu_kernels_b200.gemm import GemmConfig
    from llm_gpu_kernels_b200.moe_configured import prepare_configured_moe
    from llm_gpu_kernels_b200.moe_cuda import prepare_cuda_moe
    cpu = make_inputs(70, 8, 2, 256, 128, seed=41, wscale=0.1)
    gpu = tuple(a.to(dev) for a in cpu)
    outs = []
    for tile in (16, 64):
        p = prepare_configured_moe(*gpu, GemmConfig(block_m=tile))
        assert p.base.token_tile == tile and p.base.config.block_m == tile
        outs.append(p.run().clone())
        check_output(outs[-1], cpu)
    c = prepare_cuda_moe(*gpu, variant="async_skip")
    check_output(c.run(), cpu)
    with pytest.raises(ValueError):
        prepare_cuda_moe(*gpu, variant="bogus")
    with pytest.raises(TypeError):
        prepare_configured_moe(*gpu, {"block_m": 32})


def test_bind_rejects_bad_arguments(dev):
    from llm_gpu_kernels_b200.moe import prepare_moe
    x, gu, dn, ids, rw = make_inputs(4, 4, 2, 128, 64, device=dev)
    with pytest.raises(ValueError):
        prepare_moe(x, gu, dn[:, :, :32], ids, rw)             # non-contiguous / wrong I
    with pytest.raises(ValueError):
        prepare_moe(x, gu, dn, ids.float(), rw)                # ids dtype
    with pytest.raises(ValueError):
        prepare_moe(x, gu, dn, ids, rw.double())               # weights dtype
    with pytest.raises(ValueError):
        prepare_moe(x.float(), gu, dn, ids, rw)                # x dtype
    with pytest.raises(ValueError):
        prepare_moe(x, gu, dn, ids, rw, router_weight=torch.zeros(3, 128, device=dev, dtype=torch.bfloat16))
    with pytest.raises(RuntimeError):
        prepare_moe(*make_inputs(4, 4, 2, 67, 33, device=dev), schedule="tcgen05")


def test_registered_operator_graph_capture_and_compile(dev):
    """``run()`` goes through ``torch.ops.b200moe.forward``: the op passes PyTorch's schema / fake-tensor checks,
    is captured by ``torch.cuda.graph`` and traces under ``torch.compile(fullgraph=True)`` without a graph break."""
    import llm_gpu_kernels_b200._ops  # noqa: F401  (registers the op)
    cpu = make_inputs(48, 8, 2, 256, 128, seed=61, wscale=0.1)
    gpu = tuple(a.to(dev) for a in cpu)
    p = prep()(*gpu)
    base = p.base
    want = p.run().clone()
    check_output(want, cpu)
    args = base._op_args
    assert args is not None and args[0] == base._plan.value
    torch.library.opcheck(torch.ops.b200moe.forward.default, args, test_utils=("test_schema", "test_faketensor"))
    base.output.zero_()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=torch.cuda.Stream(device=dev)):
        torch.ops.b200moe.forward(*args)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(base.output, want)

    def layer(scale):
        torch.ops.b200moe.forward(*args)
        return base.output.float() * scale

    base.output.zero_()
    compiled = torch.compile(layer, fullgraph=True, backend="aot_eager")
    got = compiled(torch.tensor(2.0, device=dev))
    torch.cuda.synchronize()
    assert torch.equal(got, want.float() * 2.0)
