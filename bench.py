"""Benchmark of the MoE-layer forward (router -> ranked dispatch -> gate/up +
SwiGLU -> down -> weighted combine) on the Qwen3-30B-A3B layer shape.

    python bench.py --gpus 1 --steps K --warmup W            # this implementation
    python bench.py --impl reference --steps K --warmup W    # FP32 CPU oracle on the host cores
    torchrun --nproc-per-node N bench.py --gpus N ...        # expert parallel, one rank per GPU

One "step" is one forward of the layer over one batch of T synthetic tokens
(seeded N(0,1) activations, N(0,0.02) weights; no checkpoint or trace is
read). The headline line is T=1024 with BF16 weights; T=17 and T=193 are in
``by_tokens``, the W4A16 weights at the same three sizes in ``by_tokens_w4`` and
the tensor-bound sizes (T=8192, uniform and Zipf-skewed routing) in ``large_t``.
The device-timed value is a CUDA-graph replay of the forward with all inputs
resident in HBM; the 1.2 GB of expert weights exceed the 126 MB L2, so every
step streams them from HBM again. A timing window is exactly ``--steps``
forwards between two CUDA events; windows are repeated until a quarter of a
second of device time has been timed and the median window is reported.
``e2e`` goes through the public prepared-MoE API with host buffers:
pinned-host activations are copied in and the BF16 result is copied back inside
the timed region. With N > 1 ranks every rank owns E/N experts and its own
tokens; before anything is timed every rank checks its expert-parallel output
against the single-GPU plan (bit for bit) and against the FP32 CPU oracle.
Rank 0 prints ONE JSON line.
"""
from __future__ import annotations

import argparse
import json
import math
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
MIXTRAL = dict(experts=8, hidden=4096, intermediate=14336, topk=2)
SHAPES = {"qwen": QWEN, "mixtral": MIXTRAL}
TOKENS = (17, 193, 1024)
METRIC = "moe_layer_tokens_per_s"
UNIT = "tokens/s"
NVLINK_GBS = 770.0       # measured peer-copy bandwidth per direction per GPU on this pool (nominal 900)
MIN_TIMED_MS = 250.0     # device time every reported figure is the median over
REL_RMS_BF16 = 5e-3


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        data = json.loads(path.read_text())
        return {"hbm_gbs": float(data["hbm_gbs"]), "bf16_tflops": float(data["bf16_tflops"]),
                "bf16_tflops_sustained": float(data.get("bf16_tflops_sustained", data["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def traffic_table():
    """DRAM bytes per launch of the gate/up kernel from the committed ncu captures (profiles/traffic.json)."""
    path = ROOT / "profiles" / "traffic.json"
    return json.loads(path.read_text()) if path.is_file() else {}


def algorithmic_work(tokens, experts, topk, hidden, intermediate, active_experts, w4=False, routes=None):
    """(flops, bytes) one forward must do: 6*R*H*I + 2*T*H*E flops; each active expert's weights (and W4
    group scales) once, the router weight, x in, output out, ids + routing weights."""
    r = tokens * topk if routes is None else routes
    flops = 6 * r * hidden * intermediate + 2 * tokens * hidden * experts
    per_expert = 3 * hidden * intermediate * (0.5 if w4 else 2)
    if w4:
        per_expert += (2 * intermediate * hidden // 128 + hidden * intermediate // 128) * 2
    nbytes = active_experts * per_expert + experts * hidden * 2 + 2 * tokens * hidden * 2 + tokens * topk * 8
    return flops, int(nbytes)


def seeded_weights(seed=0, wscale=0.02, only_expert=None, **shape):
    """Router weight, gate/up, down (FP32 draws cast to BF16). `only_expert` draws the router weight from the
    layer seed and ONE expert's weights from a seed of its own (expert-parallel ranks that own a single expert)."""
    e, h, i = shape["experts"], shape["hidden"], shape["intermediate"]
    g = torch.Generator().manual_seed(seed)
    wr = (wscale * torch.randn(e, h, generator=g)).bfloat16()
    if only_expert is not None:
        ge = torch.Generator().manual_seed(seed * 1000 + 17 + only_expert)
        gate_up = (wscale * torch.randn(1, 2 * i, h, generator=ge)).bfloat16()
        down = (wscale * torch.randn(1, h, i, generator=ge)).bfloat16()
        return wr, gate_up, down, g
    gate_up = torch.empty(e, 2 * i, h, dtype=torch.bfloat16)
    down = torch.empty(e, h, i, dtype=torch.bfloat16)
    for k in range(e):  # per-expert draws bound the FP32 temporaries
        gate_up[k] = (wscale * torch.randn(2 * i, h, generator=g)).bfloat16()
    for k in range(e):
        down[k] = (wscale * torch.randn(h, i, generator=g)).bfloat16()
    return wr, gate_up, down, g


def zipf_bias(experts, s, seed=0):
    """log pmf of a Zipf(s) popularity over a seeded random permutation of the experts."""
    g = torch.Generator().manual_seed(seed)
    pmf = torch.arange(1, experts + 1, dtype=torch.float64) ** (-s)
    pmf = (pmf / pmf.sum())[torch.randperm(experts, generator=g)]
    return pmf.log().float()


def host_routes(x, wr, topk, zipf):
    """Softmax top-k with renormalisation on the host, a Zipf(s) popularity prior added to the logits: the skewed
    routing stress runs the fixed-route path (the device router has no bias input)."""
    logits = x.float() @ wr.float().T + zipf_bias(wr.shape[0], zipf)
    w_top, id_top = torch.topk(torch.softmax(logits, dim=1), topk, dim=-1)
    return id_top.to(torch.int32), (w_top / w_top.sum(-1, keepdim=True)).float()


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed regions run."""

    def __init__(self, index, interval_s=0.01, enabled=True):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        self._interval = interval_s
        self._nvml = None
        if not enabled:
            return
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
            time.sleep(self._interval)

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


class Timer:
    """Windows of exactly `steps` calls between two CUDA events, each bracketed by a barrier and a device
    synchronise, repeated until MIN_TIMED_MS of device time is covered; reports the median window (ms per step).
    With several ranks every rank times the same number of windows (the forwards contain cross-rank barriers) and
    each window counts with its maximum over the ranks."""

    def __init__(self, dev, steps, world=1):
        self.dev, self.steps, self.world = dev, max(1, steps), world
        self.stream = torch.cuda.current_stream(dev)
        self.launch_windows = 0

    def barrier(self):
        if self.world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize(self.dev)

    def _max_over_ranks(self, values):
        if self.world == 1:
            return list(values)
        t = torch.tensor(list(values), device=self.dev, dtype=torch.float64)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        return t.tolist()

    def median_ms(self, fn, count_windows=False):
        self.barrier()
        first = self._max_over_ranks([event_ms(fn, self.steps, self.stream)])[0]
        windows = int(min(200, max(1, math.ceil(MIN_TIMED_MS / max(first * self.steps, 1e-3)))))
        times = []
        for _ in range(windows):
            self.barrier()
            times.append(event_ms(fn, self.steps, self.stream))
        self.barrier()
        times = self._max_over_ranks(times)
        if count_windows:
            self.launch_windows = windows
        return statistics.median(times), windows


def capture(run, dev):
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=torch.cuda.Stream(device=dev)):
        run()
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize(dev)
    return graph


def pipelined_e2e(slots, stream, count):
    """`count` steps round-robin over the slots, each on its own stream: copy in, replay, copy out."""
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


# --------------------------------------------------------------------------------------- one GPU
def bench_tokens(tokens, weights, dev, steps, warmup, peaks, packed=None, shape=QWEN, token_tile=0, zipf=0.0,
                 e2e=True, headline=False):
    """Prepare one layer at T tokens and time it: graph replay, eager, the stages, end to end.
    `packed` = (PackedGateUp gate/up, PackedGateUp down) on the device selects the W4A16 path."""
    from llm_gpu_kernels_b200.moe_ranked import prepare_ranked_moe_launcher
    from llm_gpu_kernels_b200.moe_w4_cuda import prepare_w4_moe
    wr, gate_up, down, x_host = weights
    e, h, i, k = shape["experts"], shape["hidden"], shape["intermediate"], shape["topk"]
    x = x_host.to(dev)
    ids = torch.zeros(tokens, k, dtype=torch.int32, device=dev)
    rw = torch.zeros(tokens, k, dtype=torch.float32, device=dev)
    router = None if zipf > 0 else wr

    def build(x_, ids_, rw_):
        if packed is not None:
            from llm_gpu_kernels_b200.gemm import GemmConfig
            return prepare_w4_moe(x_, packed[0], None, ids_, rw_, packed_down=packed[1], router_weight=router,
                                  down_config=GemmConfig(block_m=token_tile) if token_tile else None)
        return prepare_ranked_moe_launcher(x_, gate_up, down, ids_, rw_, router_weight=router, token_tile=token_tile)

    if zipf > 0:
        id_top, w_top = host_routes(x_host, wr.cpu(), k, zipf)
        ids.copy_(id_top)
        rw.copy_(w_top)
    prepared = build(x, ids, rw)
    base = prepared.base
    timer = Timer(dev, steps)
    stream = timer.stream
    for _ in range(max(3, warmup)):
        prepared.run()
    torch.cuda.synchronize(dev)
    prepared.check_inputs()
    active = int((base.counts > 0).sum())
    max_rows = int(base.counts.max())

    graph = capture(prepared.run, dev)
    graph_ms, windows = timer.median_ms(graph.replay, count_windows=headline)
    eager_ms, _ = timer.median_ms(prepared.run)

    # every stage alone: an event pair around a single launch, behind an untimed forward that keeps the GPU
    # busy while the timed launches queue up. This is the figure the roofline fraction of a kernel uses.
    stage_samples = {l.name: [] for l in prepared.launches}
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in prepared.launches]
    reps = max(10, min(60, int(MIN_TIMED_MS / max(graph_ms, 1e-3) / 8)))
    for _ in range(reps):
        prepared.run()
        for (a, b), launch in zip(evs, prepared.launches):
            a.record(stream)
            launch.run()
            b.record(stream)
        torch.cuda.synchronize(dev)
        for (a, b), launch in zip(evs, prepared.launches):
            stage_samples[launch.name].append(a.elapsed_time(b))
    stage_ms = {name: statistics.median(v) for name, v in stage_samples.items()}
    # the gate/up stage once more as the average of back-to-back launches (secondary figure: with programmatic
    # dependent launch a train of launches overlaps each prologue with its predecessor's tail)
    launches = {l.name: l for l in prepared.launches}
    burst, bursts = 10, []
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(max(3, reps // burst)):
        prepared.run()
        a.record(stream)
        for _ in range(burst):
            launches["gate_up_swiglu"].run()
        b.record(stream)
        torch.cuda.synchronize(dev)
        bursts.append(a.elapsed_time(b) / burst)
    gate_up_burst_ms = statistics.median(bursts)

    w4 = packed is not None
    flops, nbytes = algorithmic_work(tokens, e, k, h, i, active, w4=w4)
    t_hbm_ms = nbytes / (peaks["hbm_gbs"] * 1e9) * 1e3
    t_tensor_ms = flops / (peaks["bf16_tflops_sustained"] * 1e12) * 1e3
    gate_up_weight_bytes = 2 * i * h * 2 if not w4 else 2 * i * h // 2 + 2 * i * (h // 128) * 2
    gate_up_bytes = active * gate_up_weight_bytes + tokens * k * h * 2 + tokens * k * i * 2
    gate_up_ms = stage_ms["gate_up_swiglu"]
    result = {
        "tokens": tokens, "ms_graph": graph_ms, "windows": windows, "ms_eager": eager_ms,
        "tokens_per_s": tokens / (graph_ms * 1e-3),
        "active_experts": active, "max_rows_per_expert": max_rows,
        "max_over_mean_rows": max_rows / (tokens * k / e), "token_tile": base.token_tile,
        "tflops": flops / (graph_ms * 1e-3) / 1e12,
        "tensor_frac_burst_peak": flops / (graph_ms * 1e-3) / 1e12 / peaks["bf16_tflops"],
        "tensor_frac_sustained_peak": t_tensor_ms / graph_ms,
        "schedule": base.schedule, "alg_flops": flops, "alg_bytes": nbytes,
        "layer_hbm_gbs": nbytes / (graph_ms * 1e-3) / 1e9, "layer_hbm_frac": t_hbm_ms / graph_ms,
        "layer_roofline_frac": max(t_hbm_ms, t_tensor_ms) / graph_ms,
        "bound": "hbm" if t_hbm_ms >= t_tensor_ms else "tensor",
        "stage_ms": stage_ms, "gate_up_ms": gate_up_ms, "gate_up_burst_ms": gate_up_burst_ms,
        "gate_up_alg_bytes": gate_up_bytes, "gate_up_gbs": gate_up_bytes / (gate_up_ms * 1e-3) / 1e9,
        "gate_up_hbm_frac": gate_up_bytes / (gate_up_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
        "gate_up_tflops": 4 * tokens * k * h * i / (gate_up_ms * 1e-3) / 1e12,
        "launches": base.kernel_launches,
    }
    if not e2e:
        return result

    # end to end through the public API with host buffers, one forward in flight
    x_pinned = x_host.clone().pin_memory()
    out_pinned = torch.empty(tokens, h, dtype=torch.bfloat16).pin_memory()

    def e2e_step():
        x.copy_(x_pinned, non_blocking=True)
        out_pinned.copy_(prepared.run(), non_blocking=True)

    for _ in range(3):
        e2e_step()
    e2e_serial_ms, _ = timer.median_ms(e2e_step)
    # the same with three forwards in flight: further prepared layers (own activations and workspace, same
    # weights) on streams of their own, so one step's copies overlap another step's kernels. Every step still
    # copies its input from pinned host memory and its result back.
    slots = [{"x": x, "out": base.output, "graph": graph, "x_pinned": x_pinned, "out_pinned": out_pinned,
              "stream": torch.cuda.Stream(device=dev)}]
    keep = []
    for _ in range(2):
        x2, ids2, rw2 = x.clone(), ids.clone(), rw.clone()
        prepared2 = build(x2, ids2, rw2)
        keep.append(prepared2)
        slots.append({"x": x2, "out": prepared2.base.output, "graph": capture(prepared2.run, dev),
                      "x_pinned": x_host.clone().pin_memory(),
                      "out_pinned": torch.empty(tokens, h, dtype=torch.bfloat16).pin_memory(),
                      "stream": torch.cuda.Stream(device=dev)})
    pipelined_e2e(slots, stream, 6)
    count = max(steps, 3 * int(math.ceil(MIN_TIMED_MS / max(graph_ms, 1e-3) / 3)))
    e2e_windows = [pipelined_e2e(slots, stream, count) for _ in range(3)]
    torch.cuda.synchronize(dev)
    assert all(torch.equal(slot["out_pinned"], out_pinned) for slot in slots[1:]), "the pipeline slots disagree"
    e2e_ms = statistics.median(e2e_windows)
    result.update({"ms_e2e": e2e_ms, "ms_e2e_serial": e2e_serial_ms, "tokens_per_s_e2e": tokens / (e2e_ms * 1e-3),
                   "h2d_bytes": tokens * h * 2, "d2h_bytes": tokens * h * 2})
    return result


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


def roofline_block(r, peaks, traffic, kernel):
    """The `roofline` object of one measured case: the gate/up kernel, timed as a single launch."""
    tensor_bound = r["bound"] == "tensor"
    block = {
        "bound": r["bound"], "kernel": kernel, "peak_source": peaks["source"],
        "achieved": r["gate_up_tflops"] if tensor_bound else r["gate_up_gbs"],
        "peak": peaks["bf16_tflops"] if tensor_bound else peaks["hbm_gbs"],
        "unit": "TFLOP/s" if tensor_bound else "GB/s",
        "traffic": traffic,
        "alg_bytes_per_launch": r["gate_up_alg_bytes"], "ms_per_launch": r["gate_up_ms"],
        "ms_per_launch_method": "median of CUDA-event pairs around a single launch of the stage, queued behind an "
                                "untimed forward",
        "ms_per_launch_back_to_back": r["gate_up_burst_ms"],
        "hbm_frac": r["gate_up_hbm_frac"], "tensor_frac_burst_peak": r["gate_up_tflops"] / peaks["bf16_tflops"],
        "layer": {"alg_bytes": r["alg_bytes"], "alg_flops": r["alg_flops"], "achieved_gbs": r["layer_hbm_gbs"],
                  "hbm_frac": r["layer_hbm_frac"], "tensor_frac_sustained_peak": r["tensor_frac_sustained_peak"],
                  "frac": r["layer_roofline_frac"], "ms": r["ms_graph"]},
    }
    block["frac"] = block["achieved"] / block["peak"]
    return block


def main_single(args, dev, peaks, clocks_enabled=True):
    shape = SHAPES[args.shape]
    e, h, i, k = shape["experts"], shape["hidden"], shape["intermediate"], shape["topk"]
    wr, gate_up, down, g = seeded_weights(**shape)
    weights_cpu = (wr, gate_up, down)
    xs = {t: torch.randn(t, h, generator=g).bfloat16() for t in (TOKENS if args.shape == "qwen" else ())}
    full = args.shape == "qwen" and not (args.only_headline or args.zipf > 0 or args.token_tile)
    if not full:
        xs = {t: v for t, v in xs.items() if t == args.tokens}
    if args.tokens not in xs:
        xs[args.tokens] = torch.randn(args.tokens, h, generator=g).bfloat16()
    x_large = torch.randn(8192, h, generator=g).bfloat16() if full else None
    want_w4 = args.weights == "w4" or (full and not args.no_w4)
    packed, deq = None, None
    if want_w4:
        from llm_gpu_kernels_b200.moe_weight_quant import (dequantize_gate_up_reference, quantize_down,
                                                            quantize_gate_up)
        pg, pd = quantize_gate_up(gate_up), quantize_down(down)
        packed = (pg.to(dev), pd.to(dev))
        if args.weights == "w4":   # the CPU baseline then evaluates the FP32 oracle on the dequantised weights
            deq = (wr, dequantize_gate_up_reference(pg), dequantize_gate_up_reference(pd))
    wr_d = wr.to(dev)
    gate_up_d, down_d = (None, None) if args.weights == "w4" else (gate_up.to(dev), down.to(dev))
    traffic = traffic_table()

    results, results_w4, large = {}, {}, {}
    with ClockSampler(dev.index, enabled=clocks_enabled) as clocks:
        for tokens in sorted(xs):
            results[tokens] = bench_tokens(tokens, (wr_d, gate_up_d, down_d, xs[tokens]), dev, args.steps,
                                           args.warmup, peaks, packed=packed if args.weights == "w4" else None,
                                           shape=shape, token_tile=args.token_tile, zipf=args.zipf,
                                           headline=tokens == args.tokens)
        if full and args.weights == "bf16":
            if packed is not None:
                for tokens in sorted(xs):
                    results_w4[tokens] = bench_tokens(tokens, (wr_d, None, None, xs[tokens]), dev, args.steps,
                                                      args.warmup, peaks, packed=packed, e2e=tokens == args.tokens)
            for name, zipf in (("qwen_T8192_uniform", 0.0), ("qwen_T8192_zipf1.2", 1.2)):
                large[name] = bench_tokens(8192, (wr_d, gate_up_d, down_d, x_large), dev, args.steps, args.warmup,
                                           peaks, zipf=zipf, e2e=False)
    head = results[args.tokens]
    w4 = args.weights == "w4"
    cpu = None
    if not args.no_cpu_baseline and args.shape == "qwen" and args.tokens <= 2048:
        cpu = cpu_baseline(args.tokens, deq if deq is not None else weights_cpu, xs[args.tokens], repeats=3)

    def traffic_for(kind, tokens):
        if args.shape != "qwen" or args.zipf or args.token_tile:
            return None
        return traffic.get(kind, {}).get(str(tokens))

    kernel_bf16, kernel_w4 = "grouped_gemm_tc_kernel<gate_up>", "grouped_gemm_w4t_kernel / grouped_gemm_w4_kernel <gate_up>"
    line = {
        "metric": METRIC, "value": args.tokens / (head["ms_graph"] * 1e-3), "unit": UNIT, "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": head["ms_graph"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"{'Qwen3-30B-A3B' if args.shape == 'qwen' else 'Mixtral-8x7B'} MoE layer forward "
                               f"(router+dispatch+gate/up SwiGLU+down+combine), T={args.tokens} tokens per GPU, "
                               f"E{e} H{h} I{i} top-{k}, "
                               + (f"Zipf({args.zipf}) expert popularity, fixed routes from the host router, " if args.zipf else "")
                               + ("W4A16 (W4G128 gate/up and down, BF16 activations)" if w4 else "BF16"),
                   "timing": f"CUDA-graph replay of one forward per step; windows of exactly {args.steps} steps "
                             f"between CUDA events, median of {head['windows']} windows (>= {MIN_TIMED_MS:.0f} ms "
                             "of device time)",
                   "l2": "inputs larger than L2: %s of expert weights streamed per step" % ("0.31 GB" if w4 else "1.2 GB"),
                   "parallelism": "single GPU", "token_tile": head["token_tile"], "schedule": head["schedule"],
                   "active_experts": head["active_experts"]},
        "roofline": roofline_block(head, peaks, traffic_for("w4" if w4 else "bf16", args.tokens),
                                   kernel_w4 if w4 else kernel_bf16),
        "e2e": {"value": args.tokens / (head["ms_e2e"] * 1e-3), "unit": UNIT,
                "h2d_bytes_per_step": head["h2d_bytes"], "d2h_bytes_per_step": head["d2h_bytes"],
                "ms_per_step": head["ms_e2e"], "ms_per_step_one_in_flight": head["ms_e2e_serial"],
                "mode": "prepared.run() captured once and replayed; three forwards in flight on three streams "
                        "(triple-buffered activations and workspace), each step copies its input from pinned host "
                        "memory and its BF16 result back; it can exceed `value` (one forward at a time) because the "
                        "latency-bound router / dispatch of one forward overlaps the weight streaming of another"},
        "gpu_launches": args.steps * head["windows"] * head["launches"],
        "clocks": clocks.summary(),
        "by_tokens": {str(t): {kk: v for kk, v in r.items() if kk != "tokens"} for t, r in results.items()},
    }
    if results_w4:
        line["by_tokens_w4"] = {
            str(t): dict({kk: v for kk, v in r.items() if kk != "tokens"},
                         roofline=roofline_block(r, peaks, traffic_for("w4", t), kernel_w4))
            for t, r in results_w4.items()}
    if large:
        line["large_t"] = {
            name: dict({kk: v for kk, v in r.items() if kk != "tokens"},
                       roofline=roofline_block(r, peaks, None, kernel_bf16)) for name, r in large.items()}
    if cpu is not None:
        line["cpu_baseline"] = cpu
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------- expert parallel
def ep_case(name, shape, tokens, x_host, local_weights, wr, routes, dev, timer, rank, world, mode, peaks,
            full_weights=None, oracle_rows=64, do_e2e=False, warmup=3):
    """One expert-parallel configuration on this rank: build, check, time. `routes` = (ids, rw) host tensors for
    the fixed-route path or None for the device router. `full_weights` = all experts' (gate_up, down) on this
    device for the bit-exact comparison with the single-GPU plan."""
    from llm_gpu_kernels_b200.moe_ep import expert_range, prepare_ep_moe, prepare_peer_ep_moe
    from llm_gpu_kernels_b200.moe_ranked import prepare_ranked_moe_launcher
    dist = torch.distributed
    e, h, i, k = shape["experts"], shape["hidden"], shape["intermediate"], shape["topk"]
    x = x_host.to(dev)
    ids = torch.zeros(tokens, k, dtype=torch.int32, device=dev)
    rw = torch.zeros(tokens, k, dtype=torch.float32, device=dev)
    if routes is not None:
        ids.copy_(routes[0])
        rw.copy_(routes[1])
    wr_d = None if routes is not None else wr.to(dev)
    prepare = prepare_ep_moe if mode == "nccl" else prepare_peer_ep_moe
    ep = prepare(x, local_weights[0], local_weights[1], ids, rw, experts=e, router_weight=wr_d)
    stream = timer.stream
    for _ in range(max(3, warmup)):
        out = ep.run()
    torch.cuda.synchronize(dev)
    ep.check_inputs()
    token_plan = ep.token_plan if mode == "peer" else ep.backend.token_plan
    expert_plan = ep.expert_plan if mode == "peer" else ep.backend.expert_plan
    rows = ep.rows_received if mode == "peer" else ep.stats.rows_received

    # ---- parity, before anything is timed (the checker leg: the oracle is imported here only)
    parity = {}
    ids_cpu, rw_cpu = ids.cpu(), rw.cpu()
    total = token_plan.counts.clone()
    dist.all_reduce(total)
    gathered = [torch.empty_like(ids) for _ in range(world)]
    dist.all_gather(gathered, ids)
    expect = torch.bincount(torch.cat(gathered).reshape(-1).long().cpu(), minlength=e)
    ok_counts = torch.equal(total.cpu().long(), expect)
    parity["counts"] = "exact" if ok_counts else "MISMATCH"
    ok_single = True
    if full_weights is not None:
        # the single-GPU twin on the same tile schedule (the two down schedules sum over K in a different order)
        single = prepare_ranked_moe_launcher(x.clone(), full_weights[0], full_weights[1], ids.clone(), rw.clone(),
                                             token_tile=expert_plan.token_tile, down_tiles=expert_plan.down_tiles)
        ok_single = torch.equal(single.run(), out)
        torch.cuda.synchronize(dev)
        del single
        parity["vs_single_gpu"] = "bit-exact" if ok_single else "MISMATCH"
    rel_rms = None
    if oracle_rows:
        from oracle import moe_oracle as O
        pick = torch.randperm(tokens, generator=torch.Generator().manual_seed(5 + rank))[:oracle_rows]
        gate_up_cpu, down_cpu = full_weights[2], full_weights[3]
        ref = O.moe_oracle(x_host[pick], gate_up_cpu, down_cpu, ids_cpu[pick], rw_cpu[pick])
        rel_rms = O.error_metrics(out.float().cpu()[pick], ref)["relative_rms"]
    flags = torch.tensor([float(ok_counts and ok_single), -(rel_rms or 0.0)], device=dev, dtype=torch.float64)
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    all_ok, worst_rms = bool(flags[0].item()), -flags[1].item()
    parity["rel_rms_max_over_ranks"] = worst_rms if oracle_rows else None
    parity["oracle_rows_per_rank"] = oracle_rows
    if not all_ok or (oracle_rows and worst_rms > REL_RMS_BF16):
        raise SystemExit(f"expert-parallel parity FAILED in {name} on rank {rank}: {parity}")

    # ---- timing
    step, timing = ep.run, "eager forwards (NCCL all-to-all with one host read of the split sizes per step)"
    graph = None
    if mode == "peer":  # the whole forward is kernel launches on one stream: replay it as a CUDA graph
        graph = capture(ep.run, dev)
        ep.check_inputs()
        step, timing = graph.replay, "CUDA-graph replay of one forward per step"
    ms, windows = timer.median_ms(step, count_windows=name == "headline")
    stats = torch.tensor([float(rows), float(int((expert_plan.counts > 0).sum()))], device=dev, dtype=torch.float64)
    smax, ssum = stats.clone(), stats.clone()
    dist.all_reduce(smax, op=dist.ReduceOp.MAX)
    dist.all_reduce(ssum, op=dist.ReduceOp.SUM)
    rows_max, active_max = smax.tolist()
    rows_mean = ssum.tolist()[0] / world
    # roofline of the slowest rank: its own weight streaming or tensor work, plus its rows over NVLink both ways
    el = e // world
    bytes_rank = active_max * 3 * h * i * 2 + e * h * 2 + 2 * tokens * h * 2 + tokens * k * 8
    flops_rank = 6 * rows_max * h * i + 2 * tokens * h * e
    t_hbm = bytes_rank / (peaks["hbm_gbs"] * 1e9) * 1e3
    t_tensor = flops_rank / (peaks["bf16_tflops_sustained"] * 1e12) * 1e3
    t_link = 2 * rows_max * h * 2 * (world - 1) / world / (NVLINK_GBS * 1e9) * 1e3
    t_roof = max(t_hbm, t_tensor) + t_link
    status = int(token_plan.status.item()) | int(expert_plan.status.item())
    result = {"ms": ms, "windows": windows, "timing": timing, "tokens_per_rank": tokens,
              "tokens_per_s": world * tokens / (ms * 1e-3), "rows_received_max": rows_max,
              "rows_received_mean": rows_mean, "rows_max_over_mean": rows_max / max(rows_mean, 1.0),
              "status": status, "token_tile": expert_plan.token_tile, "experts_per_rank": el, "parity": parity,
              "roofline": {"bound": "tensor+nvlink" if t_tensor >= t_hbm else "hbm+nvlink",
                           "t_hbm_ms": t_hbm, "t_tensor_ms": t_tensor, "t_nvlink_ms": t_link, "t_roof_ms": t_roof,
                           "frac": t_roof / ms, "nvlink_gbs_used": NVLINK_GBS,
                           "peak_tflops_used": peaks["bf16_tflops_sustained"], "peak_hbm_gbs_used": peaks["hbm_gbs"],
                           "note": "slowest rank: max(weights + activations over HBM, 6*rows*H*I over the "
                                   "sustained BF16 peak) + 2*rows*H*2*(N-1)/N bytes over one NVLink direction"}}
    if mode == "peer":
        # router + dispatch, count exchange, send + barrier, gate/up, down, (return copy unless the down epilogue
        # returns the rows), closing barrier, combine
        result["launches"] = token_plan.kernel_launches + 1 + 2 + 2 + (0 if expert_plan.fused_return else 1) + 1 + 1
    else:
        result["launches"] = token_plan.kernel_launches + 1 + expert_plan.kernel_launches

    if do_e2e:
        x_pinned = x_host.clone().pin_memory()
        out_pinned = torch.empty(tokens, h, dtype=torch.bfloat16).pin_memory()

        def e2e_step():
            x.copy_(x_pinned, non_blocking=True)
            graph.replay()
            out_pinned.copy_(token_plan.output, non_blocking=True)

        for _ in range(3):
            e2e_step()
        serial_ms, _ = timer.median_ms(e2e_step)
        # three forwards in flight per rank, as on one GPU: two more layers (own activations, workspace and peer
        # buffers, same weights), each captured as a graph and replayed on a stream of its own. Every rank issues
        # them in the same order; the kernels that wait for other GPUs are one-block barriers, so forwards of
        # different slots cannot block each other's progress.
        slots = [{"x": x, "graph": graph, "out": token_plan.output, "x_pinned": x_pinned, "out_pinned": out_pinned,
                  "stream": torch.cuda.Stream(device=dev)}]
        extra = []
        for _ in range(2):
            x2, ids2, rw2 = x.clone(), ids.clone(), rw.clone()
            ep2 = prepare(x2, local_weights[0], local_weights[1], ids2, rw2, experts=e, router_weight=wr_d)
            for _ in range(3):
                ep2.run()
            torch.cuda.synchronize(dev)
            extra.append(ep2)
            slots.append({"x": x2, "graph": capture(ep2.run, dev), "out": ep2.token_plan.output,
                          "x_pinned": x_host.clone().pin_memory(),
                          "out_pinned": torch.empty(tokens, h, dtype=torch.bfloat16).pin_memory(),
                          "stream": torch.cuda.Stream(device=dev)})
        pipelined_e2e(slots, stream, 6)
        count = 3 * int(math.ceil(max(timer.steps, MIN_TIMED_MS / max(ms, 1e-3)) / 3))
        e2e_times = []
        for _ in range(3):
            timer.barrier()
            e2e_times.append(pipelined_e2e(slots, stream, count))
        timer.barrier()
        e2e_times = timer._max_over_ranks(e2e_times)
        assert all(torch.equal(slot["out_pinned"], out_pinned) for slot in slots[1:]), "the pipeline slots disagree"
        for layer in (ep, *extra):
            layer.check_inputs()
        result.update({"ms_e2e": statistics.median(e2e_times), "ms_e2e_serial": serial_ms, "in_flight": 3})
        dist.barrier()
        for layer in extra:
            layer.close()
    dist.barrier()
    torch.cuda.synchronize(dev)
    if mode == "peer":
        ep.close()
    return result


def copy_probe(dev, timer, nbytes, rank, world):
    """Pinned host <-> device copy rate of this rank alone and with every rank copying at once (GB/s): what the
    end-to-end leg can at best get from the host side of an N-GPU box."""
    host = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    device = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    stream = timer.stream

    def both():
        device.copy_(host, non_blocking=True)
        host.copy_(device, non_blocking=True)

    both()
    torch.cuda.synchronize(dev)
    timer.barrier()
    together = event_ms(both, 50, stream)
    alone = None
    for r in range(world):   # one rank at a time
        timer.barrier()
        if r == rank:
            alone = event_ms(both, 50, stream)
    timer.barrier()
    t = torch.tensor([together, alone], device=dev, dtype=torch.float64)
    torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    together, alone = t.tolist()
    return {"bytes_each_way": nbytes, "gbs_alone_min_over_ranks": 2 * nbytes / (alone * 1e-3) / 1e9,
            "gbs_all_ranks_min_over_ranks": 2 * nbytes / (together * 1e-3) / 1e9}


def main_ep(args, dev, peaks, rank, world):
    from llm_gpu_kernels_b200.moe_ep import expert_range
    dist = torch.distributed
    e, h, k = QWEN["experts"], QWEN["hidden"], QWEN["topk"]
    lo, hi = expert_range(rank, world, e)
    wr, gate_up, down, _ = seeded_weights(**QWEN)
    full = (gate_up.to(dev), down.to(dev), gate_up, down)
    local = (full[0][lo:hi].contiguous(), full[1][lo:hi].contiguous())
    timer = Timer(dev, args.steps, world)
    configs = {}
    with ClockSampler(dev.index, interval_s=0.05, enabled=rank == 0) as clocks:
        # headline: weak scaling, every rank brings `--tokens` tokens of its own and owns E/world experts
        gx = torch.Generator().manual_seed(1000 + rank)
        x_rank = torch.randn(args.tokens, h, generator=gx).bfloat16()
        head = ep_case("headline", QWEN, args.tokens, x_rank, local, wr, None, dev, timer, rank, world,
                       args.ep_mode, peaks, full_weights=full, do_e2e=args.ep_mode == "peer", warmup=args.warmup)
        if not args.only_headline:
            # the transport the single-GPU reference would reach for first, beside the peer-store number
            other = "nccl" if args.ep_mode == "peer" else "peer"
            alt = ep_case(f"headline_{other}", QWEN, args.tokens, x_rank, local, wr, None, dev, timer, rank, world,
                          other, peaks, full_weights=full, oracle_rows=0, warmup=args.warmup)
            configs[f"headline_{other}"] = {kk: alt[kk] for kk in ("ms", "tokens_per_s", "timing", "parity")}
            # benchmark configuration 4: T=8192 over all ranks, Zipf(1.2) popularity prior, fixed routes from the host
            t_all = 8192
            gz = torch.Generator().manual_seed(4)
            x_all = torch.randn(t_all, h, generator=gz).bfloat16()
            ids_all, rw_all = host_routes(x_all, wr, k, 1.2)
            mine = slice(rank * t_all // world, (rank + 1) * t_all // world)
            configs["skew_T8192"] = ep_case("skew_T8192", QWEN, t_all // world, x_all[mine].contiguous(), local, wr,
                                            (ids_all[mine], rw_all[mine]), dev, timer, rank, world, args.ep_mode,
                                            peaks, full_weights=full, warmup=args.warmup)
            configs["skew_T8192"]["workload"] = (f"Qwen shape, T=8192 split {t_all // world} tokens per rank, "
                                                 "Zipf(1.2) expert popularity (fixed routes from the host router)")
            configs["copy_probe"] = copy_probe(dev, timer, args.tokens * h * 2, rank, world)
        del full, local
        torch.cuda.empty_cache()
        if MIXTRAL["experts"] % world == 0 and not args.only_headline:
            # benchmark configuration 5: Mixtral-8x7B layer shape, T=32768 over all ranks, 8/N experts per GPU (one expert per
            # GPU at N=8). Every rank draws only its own experts' weights, each from a seed of its own; rank 0
            # redraws the experts its sampled tokens use for the oracle check.
            m = MIXTRAL
            mlo, mhi = expert_range(rank, world, m["experts"])
            drawn = [seeded_weights(only_expert=expert, **m) for expert in range(mlo, mhi)]
            wr_m = drawn[0][0]
            gu_m = torch.cat([d[1] for d in drawn]).to(dev)
            dn_m = torch.cat([d[2] for d in drawn]).to(dev)
            del drawn
            t_rank = 32768 // world
            x_m = torch.randn(t_rank, m["hidden"], generator=torch.Generator().manual_seed(2000 + rank)).bfloat16()
            configs["mixtral_T32768"] = mixtral_case(m, t_rank, x_m, (gu_m, dn_m), wr_m, dev, timer, rank, world, peaks)
    if rank == 0:
        ms = head["ms"]
        line = {
            "metric": METRIC, "value": world * args.tokens / (ms * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"Qwen3-30B-A3B MoE layer forward, expert-parallel: {args.tokens} tokens per GPU, "
                                   f"E128 split {128 // world} experts per GPU, H2048 I768 top-8, BF16",
                       "timing": head["timing"] + (", rows exchanged by NVLink peer stores inside the kernels, no "
                                                   "host read" if args.ep_mode == "peer" else "")
                                 + f"; windows of exactly {args.steps} steps between CUDA events, each the max "
                                   f"over ranks, median of {head['windows']} windows",
                       "l2": f"inputs larger than L2: each rank streams its experts' weights ({1.2 / world:.2f} GB) per step",
                       "parallelism": f"ep{world}", "ep_mode": args.ep_mode, "token_tile": head["token_tile"],
                       "rows_received_max": head["rows_received_max"], "rows_received_mean": head["rows_received_mean"],
                       "nccl_ms": configs.get("headline_nccl", {}).get("ms")},
            "parity": head["parity"],
            "roofline": dict(head["roofline"], achieved=head["roofline"]["t_roof_ms"], peak=ms, unit="ms (roofline time / measured time)",
                             traffic=None),
            "gpu_launches": args.steps * head["windows"] * head["launches"],
            "clocks": clocks.summary(),
            "configs": configs,
        }
        if "ms_e2e" in head:
            line["e2e"] = {"value": world * args.tokens / (head["ms_e2e"] * 1e-3), "unit": UNIT,
                           "h2d_bytes_per_step": args.tokens * h * 2, "d2h_bytes_per_step": args.tokens * h * 2,
                           "ms_per_step": head["ms_e2e"], "ms_per_step_one_in_flight": head["ms_e2e_serial"],
                           "mode": "3 forwards in flight per rank, each step copies its input from pinned host "
                                   "memory and its BF16 result back; max over ranks"}
        else:
            line["e2e"] = {"value": world * args.tokens / (ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": 0,
                           "d2h_bytes_per_step": 0, "mode": "not measured in nccl mode"}
        print(json.dumps(line), flush=True)


def mixtral_case(m, tokens, x_host, local_weights, wr, dev, timer, rank, world, peaks):
    """8/N experts per GPU at the Mixtral shape. No rank holds all experts, so the check is the FP32 oracle on a
    few sampled tokens of rank 0, whose experts' weights rank 0 redraws from their seeds on the host."""
    from llm_gpu_kernels_b200.moe_ep import prepare_peer_ep_moe
    dist = torch.distributed
    e, h, i, k = m["experts"], m["hidden"], m["intermediate"], m["topk"]
    x = x_host.to(dev)
    ids = torch.zeros(tokens, k, dtype=torch.int32, device=dev)
    rw = torch.zeros(tokens, k, dtype=torch.float32, device=dev)
    ep = prepare_peer_ep_moe(x, local_weights[0], local_weights[1], ids, rw, experts=e, router_weight=wr.to(dev))
    for _ in range(3):
        out = ep.run()
    torch.cuda.synchronize(dev)
    ep.check_inputs()
    parity = {}
    total = ep.token_plan.counts.clone()
    dist.all_reduce(total)
    gathered = [torch.empty_like(ids) for _ in range(world)]
    dist.all_gather(gathered, ids)
    ok = torch.equal(total.cpu().long(), torch.bincount(torch.cat(gathered).reshape(-1).long().cpu(), minlength=e))
    parity["counts"] = "exact" if ok else "MISMATCH"
    rel = 0.0
    if rank == 0:
        from oracle import moe_oracle as O
        pick = torch.arange(0, tokens, tokens // 4)[:4]
        ids_cpu, rw_cpu = ids.cpu(), rw.cpu()
        gate_up = torch.zeros(e, 2 * i, h, dtype=torch.bfloat16)
        down = torch.zeros(e, h, i, dtype=torch.bfloat16)
        for expert in sorted(set(ids_cpu[pick].reshape(-1).tolist())):
            _, gu1, dn1, _ = seeded_weights(only_expert=expert, **m)
            gate_up[expert], down[expert] = gu1[0], dn1[0]
        ref = O.moe_oracle(x_host[pick], gate_up, down, ids_cpu[pick], rw_cpu[pick])
        rel = O.error_metrics(out.float().cpu()[pick], ref)["relative_rms"]
        del gate_up, down
    flags = torch.tensor([float(ok), -rel], device=dev, dtype=torch.float64)
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    parity["rel_rms_rank0"] = -flags[1].item()
    parity["oracle_rows"] = 4
    if not bool(flags[0].item()) or -flags[1].item() > REL_RMS_BF16:
        raise SystemExit(f"expert-parallel parity FAILED in mixtral_T32768: {parity}")
    graph = capture(ep.run, dev)
    ms, windows = timer.median_ms(graph.replay)
    rows = torch.tensor([float(ep.rows_received)], device=dev, dtype=torch.float64)
    rmax, rsum = rows.clone(), rows.clone()
    dist.all_reduce(rmax, op=dist.ReduceOp.MAX)
    dist.all_reduce(rsum, op=dist.ReduceOp.SUM)
    rows_max, rows_mean = rmax.item(), rsum.item() / world
    t_tensor = 6 * rows_max * h * i / (peaks["bf16_tflops_sustained"] * 1e12) * 1e3
    t_link = 2 * rows_max * h * 2 * (world - 1) / world / (NVLINK_GBS * 1e9) * 1e3
    status = int(ep.token_plan.status.item()) | int(ep.expert_plan.status.item())
    dist.barrier()
    ep.close()
    return {"workload": f"Mixtral-8x7B layer shape E8 H4096 I14336 top-2, T=32768 over {world} GPUs ({tokens} tokens and "
                        f"{e // world} expert(s) per GPU), device router", "ms": ms, "windows": windows,
            "tokens_per_s": world * tokens / (ms * 1e-3), "rows_received_max": rows_max, "rows_received_mean": rows_mean,
            "rows_max_over_mean": rows_max / max(rows_mean, 1.0), "status": status,
            "token_tile": ep.expert_plan.token_tile, "parity": parity,
            "tflops_per_gpu_slowest": 6 * rows_max * h * i / (ms * 1e-3) / 1e12,
            "roofline": {"bound": "tensor+nvlink", "t_tensor_ms": t_tensor, "t_nvlink_ms": t_link,
                         "t_roof_ms": t_tensor + t_link, "frac": (t_tensor + t_link) / ms,
                         "peak_tflops_used": peaks["bf16_tflops_sustained"], "nvlink_gbs_used": NVLINK_GBS}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=("b200", "reference"))
    ap.add_argument("--tokens", type=int, default=1024, help="headline batch size (per GPU)")
    ap.add_argument("--weights", default="bf16", choices=("bf16", "w4"),
                    help="w4: the headline itself runs gate/up and down packed W4G128 (int4 + BF16 group scales)")
    ap.add_argument("--shape", default="qwen", choices=tuple(SHAPES), help="layer shape (qwen is the headline)")
    ap.add_argument("--token-tile", type=int, default=0, help="rows of one expert per tile (0 = shape-only rule)")
    ap.add_argument("--zipf", type=float, default=0.0, help="skewed routing: Zipf exponent of the expert popularity prior")
    ap.add_argument("--ep-mode", default="peer", choices=("peer", "nccl"),
                    help="N>1: exchange rows by peer stores inside the kernels (default) or by NCCL all-to-all")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-w4", action="store_true", help="skip the W4A16 cases of the default run")
    ap.add_argument("--only-headline", action="store_true", help="time only --tokens (short profiling runs)")
    ap.add_argument("--min-timed-ms", type=float, default=MIN_TIMED_MS,
                    help="device time every figure is the median over (profiling runs under ncu pass a small value)")
    args = ap.parse_args()
    globals()["MIN_TIMED_MS"] = float(args.min_timed_ms)
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
    peaks = measured_peaks()
    if world > 1:
        torch.distributed.init_process_group("nccl", device_id=dev)
        try:
            main_ep(args, dev, peaks, rank, world)
        finally:
            torch.distributed.destroy_process_group()
        return
    main_single(args, dev, peaks)


if __name__ == "__main__":
    main()
