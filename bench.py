"""Benchmark of the MoE-layer forward (router -> ranked dispatch -> gate/up +
SwiGLU -> down -> weighted combine) on the Qwen3-30B-A3B layer shape.

    python bench.py --gpus 1 --steps K --warmup W            # this implementation
    python bench.py --impl reference --steps K --warmup W    # FP32 CPU oracle on the host cores

One "step" is one forward of the layer over one batch of T synthetic tokens
(seeded N(0,1) activations, N(0,0.02) weights; no checkpoint or trace is
read). The headline line is T=1024; T=17 and T=193 are reported in ``by_tokens``.
The device-timed value is a CUDA-graph replay of the forward with all inputs
resident in HBM; the 1.2 GB of expert weights exceed the 126 MB L2, so every
step streams them from HBM again. ``e2e`` goes through the public prepared-MoE
API with host buffers: pinned-host activations are copied in and the BF16
result is copied back inside the timed region. Rank 0 prints ONE JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

QWEN = dict(experts=128, hidden=2048, intermediate=768, topk=8)
SHAPES = {"qwen": QWEN, "mixtral": dict(experts=8, hidden=4096, intermediate=14336, topk=2)}
TOKENS = (17, 193, 1024)
METRIC = "moe_layer_tokens_per_s"
UNIT = "tokens/s"


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        data = json.loads(path.read_text())
        return {"hbm_gbs": float(data["hbm_gbs"]), "bf16_tflops": float(data["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def seeded_weights(seed=0, wscale=0.02, **shape):
    shape.pop("topk", None)
    e, h, i = shape["experts"], shape["hidden"], shape["intermediate"]
    g = torch.Generator().manual_seed(seed)
    wr = (wscale * torch.randn(e, h, generator=g)).bfloat16()
    gate_up = torch.empty(e, 2 * i, h, dtype=torch.bfloat16)
    down = torch.empty(e, h, i, dtype=torch.bfloat16)
    for k in range(e):  # per-expert draws bound the FP32 temporaries
        gate_up[k] = (wscale * torch.randn(2 * i, h, generator=g)).bfloat16()
    for k in range(e):
        down[k] = (wscale * torch.randn(h, i, generator=g)).bfloat16()
    return wr, gate_up, down, g


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed regions run."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nvml = None

    def _loop(self):
        n = self._nvml
        names = {"hw_slowdown": n.nvmlClocksEventReasonHwSlowdown if hasattr(n, "nvmlClocksEventReasonHwSlowdown")
                 else n.nvmlClocksThrottleReasonHwSlowdown,
                 "hw_thermal_slowdown": getattr(n, "nvmlClocksEventReasonHwThermalSlowdown",
                                                getattr(n, "nvmlClocksThrottleReasonHwThermalSlowdown", 0)),
                 "sw_thermal_slowdown": getattr(n, "nvmlClocksEventReasonSwThermalSlowdown",
                                                getattr(n, "nvmlClocksThrottleReasonSwThermalSlowdown", 0)),
                 "sw_power_cap": getattr(n, "nvmlClocksEventReasonSwPowerCap",
                                         getattr(n, "nvmlClocksThrottleReasonSwPowerCap", 0))}
        while not self._stop.is_set():
            try:
                self.samples.append(n.nvmlDeviceGetClockInfo(self._handle, n.NVML_CLOCK_SM))
                try:
                    mask = n.nvmlDeviceGetCurrentClocksEventReasons(self._handle)
                except Exception:
                    mask = n.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle)
                self.reasons.update(k for k, bit in names.items() if bit and mask & bit)
            except Exception:
                pass
            time.sleep(0.002)

    def __enter__(self):
        if self._nvml:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["unavailable"]}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def event_ms(fn, steps, stream):
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record(stream)
    for _ in range(steps):
        fn()
    end.record(stream)
    end.synchronize()
    return start.elapsed_time(end) / steps


def zipf_bias(experts, s, seed=0):
    """log pmf of a Zipf(s) popularity over a seeded random permutation of the experts."""
    g = torch.Generator().manual_seed(seed)
    pmf = torch.arange(1, experts + 1, dtype=torch.float64) ** (-s)
    pmf = (pmf / pmf.sum())[torch.randperm(experts, generator=g)]
    return pmf.log().float()


def bench_tokens(tokens, weights, dev, steps, warmup, peaks, dist_ctx, packed=None, shape=QWEN, token_tile=0,
                 zipf=0.0):
    """Prepare one layer at T tokens and time it: graph replay, eager, gate/up stage, end to end.
    `packed` = (PackedGateUp gate/up, PackedGateUp down) on the device selects the W4A16 path."""
    from llm_gpu_kernels_b200.moe_ranked import prepare_ranked_moe_launcher
    from llm_gpu_kernels_b200.moe_w4_cuda import prepare_w4_moe
    from oracle.moe_oracle import algorithmic_work
    wr, gate_up, down, x_host = weights
    e, h, i, k = shape["experts"], shape["hidden"], shape["intermediate"], shape["topk"]
    x = x_host.to(dev)
    ids = torch.zeros(tokens, k, dtype=torch.int32, device=dev)
    rw = torch.zeros(tokens, k, dtype=torch.float32, device=dev)
    def build(x_, ids_, rw_):
        if zipf > 0:
            return prepare_ranked_moe_launcher(x_, gate_up, down, ids_, rw_, token_tile=token_tile)
        if packed is not None:
            return prepare_w4_moe(x_, packed[0], None, ids_, rw_, packed_down=packed[1], router_weight=wr)
        return prepare_ranked_moe_launcher(x_, gate_up, down, ids_, rw_, router_weight=wr, token_tile=token_tile)

    if zipf > 0:
        # skewed routing: the popularity prior is added to the router logits on the host (the device router has
        # no bias input), so this case runs the fixed-route path: dispatch + experts + combine
        logits = x_host.float() @ wr.float().cpu().T + zipf_bias(e, zipf)
        p = torch.softmax(logits, dim=1)
        w_top, id_top = torch.topk(p, k, dim=-1)
        ids.copy_(id_top.to(torch.int32))
        rw.copy_(w_top / w_top.sum(-1, keepdim=True))
    prepared = build(x, ids, rw)
    base = prepared.base
    stream = torch.cuda.current_stream(dev)
    for _ in range(max(3, warmup)):
        prepared.run()
    torch.cuda.synchronize(dev)
    prepared.check_inputs()
    active = int((base.counts > 0).sum())
    max_rows = int(base.counts.max())

    graph = torch.cuda.CUDAGraph()
    capture = torch.cuda.Stream(device=dev)
    with torch.cuda.graph(graph, stream=capture):
        prepared.run()
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize(dev)

    def barrier():
        if dist_ctx is not None:
            torch.distributed.barrier()
        torch.cuda.synchronize(dev)

    barrier()
    graph_ms = event_ms(graph.replay, steps, stream)
    barrier()
    eager_ms = event_ms(prepared.run, steps, stream)

    # dominant kernel (gate/up + SwiGLU): events around that stage alone, inside a full forward
    launches = {l.name: l for l in prepared.launches}
    stage_ms = {name: 0.0 for name in launches}
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in launches]
    reps = min(steps, 50)
    for _ in range(reps):
        prepared.run()  # untimed: keeps the GPU busy while the timed launches queue up behind it
        for (a, b), launch in zip(evs, prepared.launches):
            a.record(stream)
            launch.run()
            b.record(stream)
        torch.cuda.synchronize(dev)
        for (a, b), launch in zip(evs, prepared.launches):
            stage_ms[launch.name] += a.elapsed_time(b) / reps
    # the dominant kernel once more as the average of back-to-back launches: an event pair around a single
    # launch also times the gap in front of it, which for a 100 us kernel is several per cent
    burst = 10
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    gate_up_ms = 0.0
    for _ in range(max(1, reps // burst)):
        prepared.run()
        a.record(stream)
        for _ in range(burst):
            launches["gate_up_swiglu"].run()
        b.record(stream)
        torch.cuda.synchronize(dev)
        gate_up_ms += a.elapsed_time(b) / burst / max(1, reps // burst)

    # end to end through the public API with host buffers
    x_pinned = x_host.clone().pin_memory()
    out_pinned = torch.empty(tokens, h, dtype=torch.bfloat16).pin_memory()

    def e2e_step():
        x.copy_(x_pinned, non_blocking=True)
        out_pinned.copy_(prepared.run(), non_blocking=True)

    for _ in range(3):
        e2e_step()
    barrier()
    e2e_serial_ms = event_ms(e2e_step, steps, stream)
    torch.cuda.synchronize(dev)

    # the same with several forwards in flight: further prepared layers (own activations and workspace, same
    # weights) on a second stream, so one step's copies overlap the other step's kernels. Every step still
    # copies its input from pinned host memory and its result back.
    slots = [{"x": x, "prepared": prepared, "graph": graph, "x_pinned": x_pinned, "out_pinned": out_pinned,
              "stream": torch.cuda.Stream(device=dev)}]
    for _ in range(2):   # two more slots: three forwards in flight cover the two copy directions and the kernels
        x2, ids2, rw2 = x.clone(), ids.clone(), rw.clone()
        prepared2 = build(x2, ids2, rw2)
        graph2 = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph2, stream=torch.cuda.Stream(device=dev)):
            prepared2.run()
        slots.append({"x": x2, "prepared": prepared2, "graph": graph2, "x_pinned": x_host.clone().pin_memory(),
                      "out_pinned": torch.empty(tokens, h, dtype=torch.bfloat16).pin_memory(),
                      "stream": torch.cuda.Stream(device=dev)})

    def e2e_pipelined(count):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(stream)
        for slot in slots:
            slot["stream"].wait_event(start)
        for i in range(count):
            slot = slots[i % len(slots)]
            with torch.cuda.stream(slot["stream"]):
                slot["x"].copy_(slot["x_pinned"], non_blocking=True)
                slot["graph"].replay()
                slot["out_pinned"].copy_(slot["prepared"].base.output, non_blocking=True)
        for slot in slots:
            stream.wait_stream(slot["stream"])
        end.record(stream)
        end.synchronize()
        return start.elapsed_time(end) / count

    e2e_pipelined(6)
    barrier()
    e2e_ms = e2e_pipelined(steps)
    torch.cuda.synchronize(dev)
    assert all(torch.equal(slot["out_pinned"], out_pinned) for slot in slots[1:]), "the pipeline slots disagree"

    w4 = packed is not None
    flops, nbytes = algorithmic_work(tokens, e, k, h, i, active, w4=w4)
    t_roof_ms = max(nbytes / (peaks["hbm_gbs"] * 1e9), flops / (peaks["bf16_tflops"] * 1e12)) * 1e3
    gate_up_weight_bytes = 2 * i * h * 2 if not w4 else 2 * i * h // 2 + 2 * i * (h // 128) * 2
    gate_up_bytes = active * gate_up_weight_bytes + tokens * k * h * 2 + tokens * k * i * 2
    gate_up_gbs = gate_up_bytes / (gate_up_ms * 1e-3) / 1e9
    return {
        "tokens": tokens, "ms_graph": graph_ms, "ms_eager": eager_ms, "ms_e2e": e2e_ms, "ms_e2e_serial": e2e_serial_ms,
        "tokens_per_s": tokens / (graph_ms * 1e-3), "tokens_per_s_e2e": tokens / (e2e_ms * 1e-3),
        "active_experts": active, "max_rows_per_expert": max_rows, "token_tile": base.token_tile,
        "tflops": flops / (graph_ms * 1e-3) / 1e12, "tensor_frac": flops / (graph_ms * 1e-3) / 1e12 / peaks["bf16_tflops"],
        "schedule": base.schedule, "alg_flops": flops, "alg_bytes": nbytes,
        "layer_hbm_gbs": nbytes / (graph_ms * 1e-3) / 1e9, "layer_roofline_frac": t_roof_ms / graph_ms,
        "stage_ms": stage_ms, "gate_up_ms": gate_up_ms, "gate_up_alg_bytes": gate_up_bytes, "gate_up_gbs": gate_up_gbs,
        "h2d_bytes": tokens * h * 2, "d2h_bytes": tokens * h * 2, "launches": base.kernel_launches,
    }


def bench_ep(tokens, weights_cpu, x_host, dev, steps, warmup, rank, world, mode):
    """Expert-parallel layer: this rank owns E/world experts and `tokens` tokens; NCCL all-to-all between ranks."""
    from llm_gpu_kernels_b200.moe_ep import expert_range, prepare_ep_moe, prepare_peer_ep_moe
    wr, gate_up, down = weights_cpu
    e, h, k = QWEN["experts"], QWEN["hidden"], QWEN["topk"]
    lo, hi = expert_range(rank, world, e)
    x = x_host.to(dev)
    ids = torch.zeros(tokens, k, dtype=torch.int32, device=dev)
    rw = torch.zeros(tokens, k, dtype=torch.float32, device=dev)
    prepare = prepare_ep_moe if mode == "nccl" else prepare_peer_ep_moe
    ep = prepare(x, gate_up[lo:hi].contiguous().to(dev), down[lo:hi].contiguous().to(dev), ids, rw,
                 experts=e, router_weight=wr.to(dev))
    stream = torch.cuda.current_stream(dev)
    for _ in range(max(3, warmup)):
        ep.run()
    torch.cuda.synchronize(dev)
    ep.check_inputs()

    def barrier():
        torch.distributed.barrier()
        torch.cuda.synchronize(dev)

    step, timing = ep.run, "eager forwards"
    if mode == "peer":  # the whole forward is kernel launches on one stream: replay it as a CUDA graph
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=torch.cuda.Stream(device=dev)):
            ep.run()
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize(dev)
        ep.check_inputs()
        step, timing = graph.replay, "CUDA-graph replay of one forward per step"
    barrier()
    ms = event_ms(step, steps, stream)
    barrier()
    eager_ms = event_ms(ep.run, steps, stream)
    x_pinned = x_host.clone().pin_memory()
    out_pinned = torch.empty(tokens, h, dtype=torch.bfloat16).pin_memory()

    def e2e_step():
        x.copy_(x_pinned, non_blocking=True)
        out_pinned.copy_(ep.run(), non_blocking=True)

    for _ in range(3):
        e2e_step()
    barrier()
    e2e_ms = event_ms(e2e_step, steps, stream)
    torch.cuda.synchronize(dev)
    extra = []
    if mode == "peer":
        # The same with three forwards in flight per rank, as at N=1: two more layers (own activations, workspace
        # and peer buffers, same weights), each captured as a graph and replayed on a stream of its own. Every rank
        # issues the three in the same order; the only kernels that wait for other GPUs are one-block barriers, so
        # forwards of different slots cannot block each other's progress.
        slots = [{"x": x, "graph": graph, "out": ep.token_plan.output, "x_pinned": x_pinned, "out_pinned": out_pinned,
                  "stream": torch.cuda.Stream(device=dev)}]
        weights_dev = (ep.expert_plan.gate_up, ep.expert_plan.down)
        for _ in range(2):
            x2, ids2, rw2 = x.clone(), ids.clone(), rw.clone()
            ep2 = prepare(x2, weights_dev[0], weights_dev[1], ids2, rw2, experts=e, router_weight=wr.to(dev))
            for _ in range(3):
                ep2.run()
            torch.cuda.synchronize(dev)
            graph2 = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph2, stream=torch.cuda.Stream(device=dev)):
                ep2.run()
            extra.append(ep2)
            slots.append({"x": x2, "graph": graph2, "out": ep2.token_plan.output,
                          "x_pinned": x_host.clone().pin_memory(),
                          "out_pinned": torch.empty(tokens, h, dtype=torch.bfloat16).pin_memory(),
                          "stream": torch.cuda.Stream(device=dev)})

        def e2e_pipelined(count):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record(stream)
            for slot in slots:
                slot["stream"].wait_event(start)
            for i in range(count):
                slot = slots[i % len(slots)]
                with torch.cuda.stream(slot["stream"]):
                    slot["x"].copy_(slot["x_pinned"], non_blocking=True)
                    slot["graph"].replay()
                    slot["out_pinned"].copy_(slot["out"], non_blocking=True)
            for slot in slots:
                stream.wait_stream(slot["stream"])
            end.record(stream)
            end.synchronize()
            return start.elapsed_time(end) / count

        e2e_pipelined(6)
        barrier()
        e2e_serial_ms, e2e_ms = e2e_ms, e2e_pipelined(steps)
        torch.cuda.synchronize(dev)
        assert all(torch.equal(slot["out_pinned"], out_pinned) for slot in slots[1:]), "the pipeline slots disagree"
        for status_of in (ep, *extra):
            status_of.check_inputs()
    if mode == "nccl":
        launches = ep.backend.token_plan.kernel_launches + 1 + ep.backend.expert_plan.kernel_launches
        rows, tile = ep.stats.rows_received, ep.backend.expert_plan.token_tile
    else:  # router + dispatch meta, counts, send + barrier, gate_up, down, return + barrier, combine
        launches = ep.token_plan.kernel_launches + 1 + 1 + 2 + 2 + 2
        rows, tile = ep.rows_received, ep.expert_plan.token_tile
        torch.distributed.barrier()
        for layer in (*extra, ep):
            layer.close()
    return {"ms": ms, "ms_eager": eager_ms, "ms_e2e": e2e_ms, "ms_e2e_serial": e2e_serial_ms if extra else e2e_ms,
            "in_flight": 1 + len(extra), "rows_received": rows, "launches": launches, "token_tile": tile,
            "timing": timing}


def cpu_baseline(tokens, weights_cpu, x_cpu, repeats):
    """Oracle port (router + FP32 expert loop) on the host cores; best of `repeats` after one warm-up."""
    from oracle import moe_oracle as O
    torch.set_num_threads(os.cpu_count() or 1)
    wr, gate_up, down = weights_cpu
    O.moe_layer_oracle(x_cpu, wr, gate_up, down, QWEN["topk"])
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        O.moe_layer_oracle(x_cpu, wr, gate_up, down, QWEN["topk"])
        best = min(best, time.perf_counter() - t0)
    return {"value": tokens / best, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"router_oracle + moe_oracle, one forward of T={tokens} tokens (full workload), "
                      f"best of {repeats} after 1 warm-up, {best * 1e3:.1f} ms"}


def run_reference(args, rank):
    if rank != 0:
        return
    tokens = args.tokens
    wr, gate_up, down, g = seeded_weights(**QWEN)
    x = torch.randn(tokens, QWEN["hidden"], generator=g).bfloat16()
    from oracle import moe_oracle as O
    torch.set_num_threads(os.cpu_count() or 1)
    for _ in range(max(1, min(args.warmup, 3))):
        O.moe_layer_oracle(x, wr, gate_up, down, QWEN["topk"])
    steps = max(1, min(args.steps, 20))
    t0 = time.perf_counter()
    for _ in range(steps):
        O.moe_layer_oracle(x, wr, gate_up, down, QWEN["topk"])
    ms = (time.perf_counter() - t0) / steps * 1e3
    value = tokens / (ms * 1e-3)
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"Qwen3-30B-A3B MoE layer forward, T={tokens}, E128 H2048 I768 top-8, "
                                   "FP32 CPU oracle (port of the reference's moe_reference + router formula)"},
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                             "sample": f"{steps} forwards of T={tokens} tokens on the host cores"},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="b200", choices=("b200", "reference"))
    ap.add_argument("--tokens", type=int, default=1024, help="headline batch size")
    ap.add_argument("--weights", default="bf16", choices=("bf16", "w4"),
                    help="w4: gate/up and down packed W4G128 (int4 + BF16 group scales), BF16 activations")
    ap.add_argument("--shape", default="qwen", choices=tuple(SHAPES), help="layer shape (qwen is the headline)")
    ap.add_argument("--token-tile", type=int, default=0, help="rows of one expert per tile (0 = shape-only rule)")
    ap.add_argument("--zipf", type=float, default=0.0, help="skewed routing: Zipf exponent of the expert popularity prior")
    ap.add_argument("--ep-mode", default="peer", choices=("peer", "nccl"),
                    help="N>1: exchange rows by peer stores inside the kernels (default) or by NCCL all-to-all")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--only-headline", action="store_true", help="time only --tokens (short profiling runs)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, rank)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a GPU (there is no CPU fallback); use --impl reference for the CPU oracle")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    dist_ctx = None
    if world > 1:
        torch.distributed.init_process_group("nccl", device_id=dev)
        dist_ctx = True
    peaks = measured_peaks()

    shape = SHAPES[args.shape]
    wr, gate_up, down, g = seeded_weights(**{k: v for k, v in shape.items() if k != "topk"})
    weights_cpu = (wr, gate_up, down)
    xs = {t: torch.randn(t, shape["hidden"], generator=g).bfloat16() for t in (TOKENS if args.shape == "qwen" else ())}
    if args.only_headline or args.zipf > 0 or args.token_tile:
        xs = {t: v for t, v in xs.items() if t == args.tokens}
    if args.tokens not in xs:
        xs[args.tokens] = torch.randn(args.tokens, shape["hidden"], generator=g).bfloat16()
    packed = None
    if args.weights == "w4":
        from llm_gpu_kernels_b200.moe_weight_quant import (dequantize_gate_up_reference, quantize_down,
                                                            quantize_gate_up)
        pg, pd = quantize_gate_up(gate_up), quantize_down(down)
        packed = (pg.to(dev), pd.to(dev))
        # the CPU baseline evaluates the FP32 oracle on the dequantised weights
        weights_cpu = (wr, dequantize_gate_up_reference(pg), dequantize_gate_up_reference(pd))
        wr_d, gate_up_d, down_d = wr.to(dev), None, None
    else:
        wr_d, gate_up_d, down_d = (t.to(dev) for t in weights_cpu)

    results = {}
    ep = None
    with ClockSampler(local_rank) as clocks:
        if world > 1:
            # weak scaling: every rank brings `--tokens` tokens of its own and owns E/world experts
            gx = torch.Generator().manual_seed(1000 + rank)
            x_rank = torch.randn(args.tokens, QWEN["hidden"], generator=gx).bfloat16()
            ep = bench_ep(args.tokens, weights_cpu, x_rank, dev, args.steps, args.warmup, rank, world, args.ep_mode)
        else:
            for tokens in sorted(xs):
                results[tokens] = bench_tokens(tokens, (wr_d, gate_up_d, down_d, xs[tokens]), dev, args.steps,
                                               args.warmup, peaks, dist_ctx, packed=packed, shape=shape,
                                               token_tile=args.token_tile, zipf=args.zipf)
    if world > 1:
        t = torch.tensor([ep["ms"], ep["ms_e2e"], float(ep["rows_received"])], device=dev, dtype=torch.float64)
        tmax, tsum = t.clone(), t.clone()
        torch.distributed.all_reduce(tmax, op=torch.distributed.ReduceOp.MAX)
        torch.distributed.all_reduce(tsum, op=torch.distributed.ReduceOp.SUM)
        if rank == 0:
            ms, e2e_ms, max_rows = tmax.tolist()
            mean_rows = tsum.tolist()[2] / world
            line = {
                "metric": METRIC, "value": world * args.tokens / (ms * 1e-3), "unit": UNIT, "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": f"Qwen3-30B-A3B MoE layer forward, expert-parallel: {args.tokens} tokens per GPU, "
                                       f"E128 split {128 // world} experts per GPU, H2048 I768 top-8, BF16",
                           "timing": ep["timing"] + (", rows exchanged by NVLink peer stores inside the dispatch / "
                                                     "return kernels, no host read" if args.ep_mode == "peer" else
                                                     ", NCCL all-to-all, one host read of the split sizes per step")
                                     + ", CUDA events, max over ranks",
                           "ms_eager_rank0": ep["ms_eager"],
                           "l2": "inputs larger than L2: each rank streams its experts' weights "
                                 f"({1.2 / world:.2f} GB) per step",
                           "parallelism": f"ep{world}", "ep_mode": args.ep_mode, "token_tile": ep["token_tile"],
                           "rows_received_max": max_rows, "rows_received_mean": mean_rows},
                "e2e": {"value": world * args.tokens / (e2e_ms * 1e-3), "unit": UNIT,
                        "h2d_bytes_per_step": args.tokens * QWEN["hidden"] * 2,
                        "d2h_bytes_per_step": args.tokens * QWEN["hidden"] * 2, "ms_per_step": e2e_ms,
                        "ms_per_step_one_in_flight_rank0": ep["ms_e2e_serial"],
                        "mode": f"{ep['in_flight']} forward(s) in flight per rank, each step copies its input from pinned "
                                "host memory and its BF16 result back; max over ranks"},
                "gpu_launches": args.steps * ep["launches"],
                "clocks": clocks.summary(),
                "roofline": {"bound": "hbm", "achieved": None, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": None,
                             "traffic": None, "note": "per-kernel roofline is reported by the 1-GPU run"},
            }
            print(json.dumps(line), flush=True)
        torch.distributed.destroy_process_group()
        return
    head = results[args.tokens]
    ms, e2e_ms = head["ms_graph"], head["ms_e2e"]

    cpu = None
    if not args.no_cpu_baseline and args.shape == "qwen" and args.tokens <= 2048:
        cpu = cpu_baseline(args.tokens, weights_cpu, xs[args.tokens], repeats=3)

    line = {
        "metric": METRIC, "value": world * args.tokens / (ms * 1e-3), "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"{'Qwen3-30B-A3B' if args.shape == 'qwen' else 'Mixtral-8x7B'} MoE layer forward "
                               f"(router+dispatch+gate/up SwiGLU+down+combine), T={args.tokens} tokens per GPU, "
                               f"E{shape['experts']} H{shape['hidden']} I{shape['intermediate']} top-{shape['topk']}, "
                               + (f"Zipf({args.zipf}) expert popularity, fixed routes from the host router, " if args.zipf else "")
                               + ("BF16" if packed is None else "W4A16 (W4G128 gate/up and down, BF16 activations)"),
                   "timing": "CUDA-graph replay of one forward per step, CUDA events",
                   "l2": "inputs larger than L2: %s of expert weights streamed per step" % (
                       "1.2 GB" if packed is None else "0.31 GB"),
                   "parallelism": "single GPU" if world == 1 else f"{world} independent replicas",
                   "token_tile": head["token_tile"], "schedule": head["schedule"],
                   "active_experts": head["active_experts"]},
        "roofline": {"bound": "hbm", "achieved": head["gate_up_gbs"], "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": head["gate_up_gbs"] / peaks["hbm_gbs"],
                     # dram__bytes_read + write of one gate/up launch from the ncu capture summarised in
                     # profiles/moe_layer_subsystems_qwen_bf16.md (BF16, Qwen shape)
                     "traffic": {17: 583.1e6, 1024: 843.4e6}.get(args.tokens) if (
                         packed is None and args.shape == "qwen" and not args.zipf) else None,
                     "tensor": {"achieved_tflops": head["tflops"], "peak_tflops": peaks["bf16_tflops"],
                                "frac": head["tensor_frac"]},
                     "kernel": "grouped_gemm_tc_kernel<gate_up>" if packed is None else "grouped_gemm_w4_kernel<gate_up>", "peak_source": peaks["source"],
                     "alg_bytes_per_launch": head["gate_up_alg_bytes"],
                     "ms_per_launch": head["gate_up_ms"],
                     "ms_per_launch_method": "CUDA events around 10 back-to-back launches of the stage, behind an "
                                             "untimed forward; event pair around a single launch inside a forward: "
                                             "%.4f ms" % head["stage_ms"]["gate_up_swiglu"],
                     "layer": {"alg_bytes": head["alg_bytes"], "alg_flops": head["alg_flops"],
                               "achieved_gbs": head["layer_hbm_gbs"], "frac": head["layer_roofline_frac"]}},
        "e2e": {"value": world * args.tokens / (e2e_ms * 1e-3), "unit": UNIT,
                "h2d_bytes_per_step": head["h2d_bytes"], "d2h_bytes_per_step": head["d2h_bytes"],
                "ms_per_step": e2e_ms, "ms_per_step_one_in_flight": head["ms_e2e_serial"],
                "mode": "prepared.run() captured once and replayed; three forwards in flight on three streams "
                        "(triple-buffered activations and workspace), each step copies its input from pinned host "
                        "memory and its BF16 result back; it can exceed `value` (one forward at a time) because the "
                        "latency-bound router / dispatch of one forward overlaps the weight streaming of another"},
        "gpu_launches": args.steps * head["launches"],
        "clocks": clocks.summary(),
        "by_tokens": {str(t): {k: v for k, v in r.items() if k not in ("tokens",)} for t, r in results.items()},
    }
    if cpu is not None:
        line["cpu_baseline"] = cpu
    print(json.dumps(line), flush=True)
    if world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
