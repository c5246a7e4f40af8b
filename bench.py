"""Benchmark of the OrbitQuant quantized-linear forward on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload dit_block|single_layer|mixed_bit|video_dit|vit_decode]

Default workload (``dit_block``): the four W4A4 projections of one DiT double-stream block
-- fused QKV 3072->9216, out-proj 3072->3072, MLP 3072->12288 and 12288->3072 -- on
M = 4096 image + 512 text = 4608 bf16 tokens with 0.5 % outlier channels (x20), weights
~N(0, 0.02), RPBH block "paper", seed 1; synthetic data, random-init weights.  A step is
one OrbitLinear forward (rotate-and-quantize prologue + packed-weight GEMM) of each of the
projections on inputs already resident in HBM.  ``value`` is the algorithmic 2*M*K*N flop
of the step divided by its device time.

The one-GPU default run also carries the other half of the metric and the other
configurations in the same JSON line: ``decode`` (ViT-base W4A6, M = 1 / 4 / 16, twelve
blocks in one CUDA graph, HBM GB/s with the weights cold in L2) and ``configs`` (single
layer M=1024, the mixed-bit 8-block stack, the video-DiT shapes).

With ``--gpus N`` (launched under torchrun, one rank per GPU) every projection is sharded
along its output features; out-proj / MLP outputs are reassembled because their consumers
need full rows, the QKV output stays head-sharded.  Total work is fixed, so the scaling is
"strong".

``--impl reference`` times the reference's own CPU kernels (``oracle/_ref``, compiled from
the reference sources) on a bounded row sample of the same workload, on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from collections import namedtuple
from pathlib import Path

import torch

REPO = Path(__file__).resolve().parent
if str(REPO) not in sys.path:
    sys.path.insert(0, str(REPO))

Layer = namedtuple("Layer", "name k n gather w_bits a_bits")

CPU_SAMPLE_ROWS = 512
MIN_SUSTAINED_SECONDS = 1.0

# (rows, [(layer name, K, N, gather_output)], weight std, seed, w_bits, a_bits): the uniform
# workloads; `workload_spec` expands them and builds the two non-uniform ones.
WORKLOADS = {
    "dit_block": (4608, [("qkv", 3072, 9216, False), ("out", 3072, 3072, True),
                         ("fc1", 3072, 12288, True), ("fc2", 12288, 3072, True)], 0.02, 1, 4, 4),
    "video_dit": (32760, [("qkv", 5120, 15360, False), ("out", 5120, 5120, True),
                          ("fc1", 5120, 13824, True), ("fc2", 13824, 5120, True)], 0.015, 3, 4, 4),
    "vit_decode": (16, [("qkv", 768, 2304, False), ("out", 768, 768, True),
                        ("fc1", 768, 3072, True), ("fc2", 3072, 768, True)], 0.02, 4, 4, 6),
}
WORKLOAD_NAMES = ("dit_block", "single_layer", "mixed_bit", "video_dit", "vit_decode")

# DRAM bytes (read + write) per launch of the dominant kernel from an ncu capture of the
# one-GPU run, keyed by workload (None until captured).
NCU_TRAFFIC_BYTES = {"dit_block": 100.8e6}


def mixed_bit_assignment(blocks: int = 8, protected_blocks: int = 4):
    """Per-block bit widths of the mixed-bit configuration, following the reference's rule
    (``src/orbitquant/policies/lowbit_protection.py:100-104``): the number of boundary blocks
    kept at W4 is ``min(protected_blocks, (blocks - 1) // 2)`` at either end -- 3 for an
    8-block stack, i.e. blocks 0-2 and 5-7 are W4A4 and blocks 3-4 are mixed (the other
    reading of "first/last four" would protect all eight and leave nothing mixed).  In a mixed
    block the separate Q and K projections are W2A4 (``:23-36``) and the rest W3A3."""
    keep = protected_blocks if blocks <= 2 else min(protected_blocks, (blocks - 1) // 2)
    plan = []
    for b in range(blocks):
        boundary = b < keep or b > blocks - 1 - keep
        plan.append({name: (4, 4) if boundary else ((2, 4) if name in ("q", "k") else (3, 3))
                     for name in ("q", "k", "v", "out", "fc1", "fc2")})
    return plan


def workload_spec(name: str) -> dict:
    if name in WORKLOADS:
        rows, specs, std, seed, w_bits, a_bits = WORKLOADS[name]
        layers = [Layer(n_, k, n, g, w_bits, a_bits) for n_, k, n, g in specs]
        return {"rows": rows, "layers": layers, "std": std, "seed": seed, "block_size": "paper",
                "outliers": "random"}
    if name == "single_layer":
        return {"rows": 1024, "layers": [Layer("linear", 3072, 3072, True, 4, 4)], "std": 0.02,
                "seed": 0, "block_size": 256, "outliers": "first8"}
    if name == "mixed_bit":
        shapes = {"q": (3072, 3072, False), "k": (3072, 3072, False), "v": (3072, 3072, False),
                  "out": (3072, 3072, True), "fc1": (3072, 12288, True), "fc2": (12288, 3072, True)}
        layers = []
        for b, bits in enumerate(mixed_bit_assignment()):
            for lname, (k, n, gather) in shapes.items():
                layers.append(Layer(f"b{b}.{lname}", k, n, gather, *bits[lname]))
        return {"rows": 4096, "layers": layers, "std": 0.02, "seed": 2, "block_size": "paper",
                "outliers": "random"}
    raise KeyError(name)


def describe(name: str, spec: dict, rows: int) -> str:
    layers = spec["layers"]
    if name == "mixed_bit":
        return (f"mixed_bit: 8 DiT blocks x (q, k, v, out 3072->3072, fc1 3072->12288, fc2 12288->3072), "
                f"blocks 0-2 and 5-7 W4A4, blocks 3-4 q/k W2A4 and the rest W3A3, bf16, M={rows}")
    bits = f"W{layers[0].w_bits}A{layers[0].a_bits}"
    return (f"{name}: OrbitLinear {bits} bf16, M={rows}, "
            + ", ".join(f"{l.name} {l.k}->{l.n}" for l in layers))


def measured_peaks():
    path = REPO / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return {"hbm_gbs": float(data["hbm_gbs"]), "tflops_burst": float(data["bf16_tflops"]),
                "tflops_sustained": float(data["bf16_tflops_sustained"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops_burst": 1590.0, "tflops_sustained": 1400.0,
            "source": "fallback"}


def layer_flops(rows, k, n):
    return 2.0 * rows * k * n


def layer_bytes(rows, k, n, w_bits, a_bits):
    """Algorithmic bytes of one OrbitLinear call: x read, packed W, row norms, bias, y write,
    constants (perm, signs, codebooks); intermediates are not counted."""
    const = 4 * k + k + 4 * (2 ** a_bits - 1) + 4 * 2 ** a_bits + 4 * 2 ** w_bits
    return rows * k * 2 + (n * k * w_bits + 7) // 8 + 2 * n + 2 * n + rows * n * 2 + const


def synth_weight_payload(k, n, w_bits, std, seed, device=None):
    """Packed indices / row norms with the statistics OrbitQuant produces for W ~ N(0, std):
    rotated unit rows are near-Gaussian with variance 1/K, so indices follow the codebook's
    cell probabilities and row norms concentrate at std*sqrt(K).  Drawing them directly
    (instead of quantising an N x K fp32 matrix on the CPU) keeps start-up short; parity
    tests quantise real matrices.  With a CUDA `device` the draw and the packing happen
    there (another random stream, the same distribution)."""
    from orbitquant_b200 import get_codebook, native, pack_lowbit

    cb = get_codebook(k, w_bits)
    if device is not None and torch.device(device).type == "cuda":
        g = torch.Generator(device=device).manual_seed(seed)
        parts = []
        rows_per_chunk = max(1, (1 << 26) // k)
        for lo in range(0, n, rows_per_chunk):
            hi = min(n, lo + rows_per_chunk)
            unit = torch.randn(hi - lo, k, generator=g, device=device) / (k ** 0.5)
            parts.append(native.pack_lowbit(cb.quantize_indices(unit), w_bits, validate=False))
        packed = torch.cat(parts)
        norms = (std * (k ** 0.5) * (1 + 0.02 * torch.randn(n, generator=g, device=device))).to(torch.bfloat16)
        bias = (torch.randn(n, generator=g, device=device) * 0.02).to(torch.bfloat16)
        return packed, norms, bias
    g = torch.Generator().manual_seed(seed)
    packed_parts = []
    rows_per_chunk = max(1, (1 << 24) // k)
    for lo in range(0, n, rows_per_chunk):
        hi = min(n, lo + rows_per_chunk)
        unit = torch.randn(hi - lo, k, generator=g) / (k ** 0.5)
        packed_parts.append(pack_lowbit(cb.quantize_indices(unit), w_bits, validate=False))
    packed = torch.cat(packed_parts)
    norms = (std * (k ** 0.5) * (1 + 0.02 * torch.randn(n, generator=g))).to(torch.bfloat16)
    bias = (torch.randn(n, generator=g) * 0.02).to(torch.bfloat16)
    return packed, norms, bias


def synth_activations(rows, k, seed, outliers="random", device=None):
    if device is not None and torch.device(device).type == "cuda":
        g = torch.Generator(device=device).manual_seed(seed)
        x = torch.randn(rows, k, generator=g, device=device)
    else:
        g = torch.Generator().manual_seed(seed)
        x = torch.randn(rows, k, generator=g)
    if outliers == "first8":
        x[:, :8] *= 20.0
    else:
        cpu_g = torch.Generator().manual_seed(seed + 1)
        columns = torch.randperm(k, generator=cpu_g)[: max(1, round(0.005 * k))].to(x.device)
        x[:, columns] *= 20.0
    return x.to(torch.bfloat16)


def build_layers(workload, device, rank=0, world=1, rows_override=0, on_device=False, weight_mode=None):
    """[(Layer, module on `device`)] of a workload; column shards when world > 1.  `weight_mode`
    selects another formulation of the same layers ("int8_surrogate": the integer route)."""
    from orbitquant_b200 import OrbitQuantConfig, OrbitQuantLinear
    from orbitquant_b200.sharding import shard_linear

    spec = workload_spec(workload)
    cache = {}
    layers = []
    for i, layer in enumerate(spec["layers"]):
        cfg = OrbitQuantConfig(weight_bits=layer.w_bits, activation_bits=layer.a_bits,
                               rotation_seed=spec["seed"], block_size=spec["block_size"])
        key = (layer.k, layer.n, layer.w_bits)
        if key not in cache:   # stacked blocks reuse one payload per shape and width
            cache[key] = synth_weight_payload(layer.k, layer.n, layer.w_bits, spec["std"],
                                              spec["seed"] * 100 + len(cache),
                                              device if on_device else None)
        packed, norms, bias = cache[key]
        module = OrbitQuantLinear(in_features=layer.k, out_features=layer.n, config=cfg,
                                  module_name=layer.name, source_weight_layout="out_in",
                                  bias=bias.clone(), packed_weight_indices=packed.clone(),
                                  row_norms=norms.clone(), debug_weight=None)
        if world > 1:
            module = shard_linear(module, rank, world, config=cfg)
        if weight_mode is not None:
            module.weight_mode = weight_mode
        layers.append((layer, module.to(device)))
    return (rows_override or spec["rows"]), layers, spec


class ClockSampler:
    """Samples SM clocks / throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.lines: list[str] = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, sm_max, power, reasons = [], [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                sm_max.append(float(parts[1]))
                power.append(float(parts[2]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[3:7]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        # the median over the samples taken under load (the GPU idles while the host prepares)
        loaded = sorted(s for s, p in zip(sm, power) if p >= 0.5 * max(power)) or sorted(sm)
        return {"sm_mhz": loaded[len(loaded) // 2], "sm_max_mhz": max(sm_max), "reasons": sorted(reasons),
                "samples": len(sm), "samples_under_load": len(loaded), "power_w_max": max(power)}


def host_physical_cores() -> int:
    """Physical cores in this process's affinity mask, at most 64: the reference's own default
    thread count (``orbitquant_packed_matmul_cpu/cpu_threads.cpp:39-101``)."""
    try:
        cpus = sorted(os.sched_getaffinity(0))
    except AttributeError:
        return min(64, os.cpu_count() or 1)
    cores = set()
    for cpu in cpus:
        try:
            base = Path(f"/sys/devices/system/cpu/cpu{cpu}/topology")
            cores.add((int((base / "physical_package_id").read_text()), int((base / "core_id").read_text())))
        except (OSError, ValueError):
            pass
    return min(64, len(cores) if cores else len(cpus))


def time_reference_cpu(workload, passes, warmup, sample_rows):
    """The reference's compiled CPU kernels on `sample_rows` rows of every layer, with all the
    host's physical cores (stated explicitly: a launcher's OMP_NUM_THREADS=1 must not apply)."""
    from oracle import ref_cpu
    from orbitquant_b200 import get_codebook, get_rpbh_rotation

    threads = host_physical_cores()
    os.environ["ORBITQUANT_CPU_THREADS"] = str(threads)
    spec = workload_spec(workload)
    m = min(spec["rows"], sample_rows)
    cache = {}
    prepared = []
    for i, layer in enumerate(spec["layers"]):
        key = (layer.k, layer.n, layer.w_bits)
        if key not in cache:
            cache[key] = synth_weight_payload(layer.k, layer.n, layer.w_bits, spec["std"],
                                              spec["seed"] * 100 + len(cache))
        packed, norms, bias = cache[key]
        rot = get_rpbh_rotation(layer.k, spec["seed"], spec["block_size"])
        prepared.append((layer, packed, norms, bias.float(), rot, get_codebook(layer.k, layer.a_bits),
                         get_codebook(layer.k, layer.w_bits),
                         synth_activations(m, layer.k, spec["seed"] * 1000 + i % 6, spec["outliers"])))

    def one_pass():
        for layer, packed, norms, bias, rot, acb, wcb, x in prepared:
            ref_cpu.linear_forward(
                x, packed, norms, bias, permutation=rot.permutation, signs=rot.signs,
                act_centroids=acb.centroids, act_boundaries=acb.boundaries,
                w_centroids=wcb.centroids, w_bits=layer.w_bits, out_features=layer.n, eps=1e-10,
                block_size=rot.block_size)

    for _ in range(max(1, warmup)):
        one_pass()
    t0 = time.perf_counter()
    for _ in range(passes):
        one_pass()
    seconds = (time.perf_counter() - t0) / passes
    flops = sum(layer_flops(m, l.k, l.n) for l in spec["layers"])
    report = ref_cpu.host_isa_report()
    return {
        "value": flops / seconds / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "reference",
        "sample": (f"{m} of {spec['rows']} rows of each of the {len(spec['layers'])} projections, "
                   f"{passes} timed pass(es); reference CPU kernels oracle/_ref with "
                   f"ORBITQUANT_CPU_THREADS={threads}, ORBITQUANT_CPU_ISA={report['isa_env']}, "
                   f"avx512_bf16={report['avx512_bf16']}"),
        "ms_per_step": seconds * 1e3, "rows": m,
    }


def cpu_sample_note(workload: str) -> str:
    rows = workload_spec(workload)["rows"]
    return (f"the CPU reference arm runs {min(rows, CPU_SAMPLE_ROWS)} of the {rows} rows (a rate, "
            f"so comparable)")


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import ref_cpu

    spec = workload_spec(args.workload)
    if not ref_cpu.available():
        print(json.dumps({"impl": "reference",
                          "unavailable": "oracle/_ref (reference CPU kernels) was not built"}))
        return
    # each "step" is one pass over the bounded row sample; at most 5 so the run stays short
    passes = max(3, min(args.steps, 5))
    warm = max(1, min(args.warmup, 2))
    cpu = time_reference_cpu(args.workload, passes, warm, CPU_SAMPLE_ROWS)
    line = {
        "impl": "reference", "metric": "orbitlinear_tflops", "value": cpu["value"], "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": passes, "warmup": warm, "ms_per_step": cpu["ms_per_step"],
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": describe(args.workload, spec, spec["rows"]),
                   "cpu_sample": cpu_sample_note(args.workload)},
        "cpu_baseline": {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": cpu["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ---- decode (rows <= 16): HBM GB/s -----------------------------------------------------------

def measure_decode(workload, rows, device, steps, warmup, with_e2e=True):
    """Decode-sized batches: the forward is weight streaming, so the figure of merit is HBM
    GB/s.  One pass = 12 transformer blocks x 4 projections, captured in a CUDA graph (launch
    overhead would otherwise dominate layers this small).  Two graphs: `warm` replays one
    12-block weight set that fits the 126 MB L2; `cold` walks enough distinct weight sets
    (> 2x L2) that every weight byte comes from HBM."""
    from orbitquant_b200 import OrbitQuantConfig, OrbitQuantLinear, native

    spec = workload_spec(workload)
    specs = spec["layers"]
    w_bits, a_bits = specs[0].w_bits, specs[0].a_bits
    blocks = 12
    cfg = OrbitQuantConfig(weight_bits=w_bits, activation_bits=a_bits, rotation_seed=spec["seed"])
    set_bytes = blocks * sum((l.n * l.k * w_bits + 7) // 8 for l in specs)
    sets = max(2, -(-300_000_000 // set_bytes))
    payloads = [synth_weight_payload(l.k, l.n, w_bits, spec["std"], spec["seed"] * 100 + i)
                for i, l in enumerate(specs)]
    modules = []
    for s_idx in range(sets):
        for b in range(blocks):
            for i, l in enumerate(specs):
                packed, norms, bias = payloads[i]
                # distinct device copies: same statistics, different addresses
                modules.append(OrbitQuantLinear(
                    in_features=l.k, out_features=l.n, config=cfg, module_name=f"s{s_idx}.b{b}.{l.name}",
                    source_weight_layout="out_in", bias=bias.clone(), packed_weight_indices=packed.clone(),
                    row_norms=norms.clone(), debug_weight=None).to(device))
    per_set = blocks * len(specs)
    inputs = [synth_activations(rows, l.k, spec["seed"] * 1000 + i).to(device) for i, l in enumerate(specs)]

    def run_set(s_idx):
        for j in range(per_set):
            modules[s_idx * per_set + j](inputs[j % len(specs)])

    def capture(fn):
        fn()  # builds device constants, warms the allocator
        torch.cuda.synchronize()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn()
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            fn()
        return graph

    def time_graph(graph, replays):
        for _ in range(max(3, warmup)):
            graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(replays):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / replays

    launches0 = native.launch_count()
    warm_graph = capture(lambda: run_set(0))
    launches_per_pass = (native.launch_count() - launches0) // 3
    warm_ms = time_graph(warm_graph, steps)

    def all_sets():
        for s_idx in range(sets):
            run_set(s_idx)

    cold_graph = capture(all_sets)
    cold_ms = time_graph(cold_graph, max(3, steps // sets)) / sets

    pass_bytes = blocks * sum(layer_bytes(rows, l.k, l.n, w_bits, a_bits) for l in specs)
    pass_flops = blocks * sum(layer_flops(rows, l.k, l.n) for l in specs)
    peaks = measured_peaks()
    cold_gbs = pass_bytes / (cold_ms * 1e-3) / 1e9
    # A layer of these sizes is one launch whose duration is set by launch latency, not by
    # bytes: the floor per layer is the back-to-back launch interval inside a graph.
    result = {
        "workload": (f"{workload}: {blocks} blocks x ({', '.join(f'{l.name} {l.k}->{l.n}' for l in specs)}) "
                     f"OrbitLinear W{w_bits}A{a_bits} bf16, M={rows}, one CUDA graph per pass"),
        "rows": rows, "value": cold_gbs, "unit": "GB/s", "ms_per_pass": cold_ms,
        "frac_of_hbm": cold_gbs / peaks["hbm_gbs"], "hbm_peak": peaks["hbm_gbs"],
        "peak_source": peaks["source"],
        "l2": f"cold: {sets} distinct weight sets ({sets * set_bytes / 1e6:.0f} MB > 2x L2) walked per replay",
        "l2_warm": {"value": pass_bytes / (warm_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_pass": warm_ms,
                    "note": f"one {set_bytes / 1e6:.1f} MB weight set replayed; it fits the L2"},
        "algorithmic_bytes_per_pass": pass_bytes, "us_per_layer": cold_ms * 1e3 / per_set,
        "launches_per_layer": launches_per_pass / per_set, "tflops": pass_flops / (cold_ms * 1e-3) / 1e12,
        "kernels": decode_kernel_names(specs, rows, w_bits),
    }
    if with_e2e:
        # end to end through the module API, eager, pinned host input and output
        host_x = synth_activations(rows, specs[0].k, 7).pin_memory()
        host_y = torch.empty((rows, specs[-1].n), dtype=torch.bfloat16).pin_memory()

        def e2e_pass():
            h = host_x.to(device, non_blocking=True)
            for b in range(blocks):
                qkv = modules[4 * b](h)
                a = modules[4 * b + 1](qkv[:, :specs[1].k].contiguous())
                u = torch.nn.functional.gelu(modules[4 * b + 2](a))
                h = modules[4 * b + 3](u)
            host_y.copy_(h, non_blocking=True)

        for _ in range(3):
            e2e_pass()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e2e_steps = max(3, steps // 4)
        e0.record()
        for _ in range(e2e_steps):
            e2e_pass()
        e1.record()
        torch.cuda.synchronize()
        e2e_ms = e0.elapsed_time(e1) / e2e_steps
        result["e2e"] = {"value": pass_bytes / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s",
                         "h2d_bytes_per_step": host_x.numel() * 2, "d2h_bytes_per_step": host_y.numel() * 2,
                         "ms_per_step": e2e_ms,
                         "what": "12 blocks chained eagerly through OrbitQuantLinear (QKV, out, MLP up, GELU, MLP down)"}
    result["gpu_launches_per_pass"] = int(launches_per_pass)
    del modules, warm_graph, cold_graph
    torch.cuda.empty_cache()
    return result


def decode_kernel_names(specs, rows, w_bits):
    from orbitquant_b200 import get_rpbh_rotation, native

    names = set()
    for l in specs:
        block = get_rpbh_rotation(l.k, 0, "paper").block_size
        names.add(native.forward_kernel_name(rows, l.k, l.n, w_bits, l.a_bits, block))
    return sorted(names)


def run_decode(args, device, rank):
    rows = args.rows or min(workload_spec(args.workload)["rows"], 16)
    from orbitquant_b200 import native

    sampler = ClockSampler(device.index or 0)
    sampler.start()
    res = measure_decode(args.workload, rows, device, args.steps, args.warmup)
    clocks = sampler.stop()
    line = {
        "metric": "orbitlinear_decode_hbm_gbs", "value": res["value"], "unit": "GB/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": res["ms_per_pass"],
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": res["workload"], "l2": res["l2"],
                   "algorithmic_bytes_per_pass": res["algorithmic_bytes_per_pass"]},
        "l2_warm": res["l2_warm"], "us_per_layer": res["us_per_layer"], "tflops": res["tflops"],
        "roofline": {"bound": "hbm", "achieved": res["value"], "peak": res["hbm_peak"], "unit": "GB/s",
                     "frac": res["frac_of_hbm"], "traffic": None, "peak_source": res["peak_source"],
                     "kernel": " / ".join(res["kernels"]),
                     "avg_launch_us": res["us_per_layer"] / max(1.0, res["launches_per_layer"])},
        "e2e": res.get("e2e"), "gpu_launches": res["gpu_launches_per_pass"] * args.steps,
        "clocks": clocks, "gemm_device_status": native.gemm_device_status(),
    }
    if not args.no_cpu_baseline:
        try:
            from oracle import ref_cpu
            if ref_cpu.available():
                cpu = time_reference_cpu(args.workload, 3, 1, rows)
                seconds = cpu["ms_per_step"] * 1e-3 * 12
                line["cpu_baseline"] = {"value": res["algorithmic_bytes_per_pass"] / seconds / 1e9,
                                        "unit": "GB/s", "cores": cpu["cores"], "kind": "reference",
                                        "sample": cpu["sample"]}
        except Exception as exc:
            line["cpu_baseline"] = {"error": str(exc)}
    if rank == 0:
        print(json.dumps(line))


# ---- large row counts: TFLOP/s ------------------------------------------------------------------

def time_steps(step, steps, barrier):
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    start.record()
    for _ in range(steps):
        step()
    stop.record()
    barrier()
    return start.elapsed_time(stop)


def kernel_alone(layers, inputs, steps, peaks):
    """The dominant kernel timed alone: one CUDA-event pair around every launch of the
    packed-weight GEMM on a prepared operand.  Launches timed one by one run in isolation (the
    GPU idles between them), so the denominator is the BURST cuBLAS figure."""
    from orbitquant_b200 import native

    prepared = []
    for (layer, module), x in zip(layers, inputs):
        xq = native.quantize_activations(
            x, module._rotation_permutation, module._rotation_signs,
            module._activation_codebook_centroids, module._activation_codebook_boundaries,
            eps=module.activation_eps, block_size=module.rotation.block_size)
        prepared.append(native.rows_to_f16_operand(xq, module._weight_codebook_centroids))
    torch.cuda.synchronize()
    events = []
    for it in range(steps + 2):
        for (layer, module), (operand, scale, table) in zip(layers, prepared):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            native.gemm_tcgen05_f16(operand, scale, module.packed_weight_indices, module.row_norms,
                                    module._weight_codebook_centroids, out_features=module.out_features,
                                    bits=layer.w_bits, bias=module.bias, table_scale=table)
            e1.record()
            if it >= 2:
                events.append((e0, e1))
    torch.cuda.synchronize()
    kernel_ms = sum(e0.elapsed_time(e1) for e0, e1 in events)
    rows = inputs[0].shape[0]
    names = sorted({native.forward_kernel_name(rows, l.k, m.out_features, l.w_bits, l.a_bits,
                                               m.rotation.block_size).split(" + ")[-1]
                    for l, m in layers})
    flops = sum(layer_flops(rows, l.k, m.out_features) for l, m in layers)
    achieved = flops * steps / (kernel_ms * 1e-3) / 1e12
    return {"bound": "tensor", "achieved": achieved, "peak": peaks["tflops_burst"], "unit": "TFLOP/s",
            "frac": achieved / peaks["tflops_burst"],
            "peak_sustained": peaks["tflops_sustained"],
            "frac_of_sustained": achieved / peaks["tflops_sustained"],
            "peak_source": peaks["source"], "kernel": " / ".join(names),
            "timed": "every launch alone between its own CUDA events",
            "avg_launch_us": kernel_ms * 1e3 / max(1, len(events)), "launches_timed": len(events)}


def measure_single_gpu(workload, device, steps, warmup, rows_override=0, on_device=False,
                       with_kernel=True, sustained=True, weight_mode=None, graph=False):
    """value / ms_per_step of a large-row workload on one GPU, resident inputs.  With `graph` the
    step is captured once in a CUDA graph and replayed (for routes whose host-side call is long
    next to their kernels)."""
    from orbitquant_b200 import native

    rows, layers, spec = build_layers(workload, device, rows_override=rows_override, on_device=on_device,
                                      weight_mode=weight_mode)
    # stacked blocks share the input tensors of their (up to six) distinct projections
    distinct = [synth_activations(rows, l.k, spec["seed"] * 1000 + i, spec["outliers"],
                                  device if on_device else None).to(device)
                for i, (l, _m) in enumerate(layers[:6])]
    inputs = [distinct[i % 6] for i in range(len(layers))]

    def step():
        for (layer, module), x in zip(layers, inputs):
            module(x)

    def barrier():
        torch.cuda.synchronize()

    for _ in range(max(3, warmup)):
        step()
    if graph:
        eager_step = step
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            eager_step()
        torch.cuda.current_stream().wait_stream(side)
        captured = torch.cuda.CUDAGraph()
        launches0 = native.launch_count()
        with torch.cuda.graph(captured):
            eager_step()
        per_step = native.launch_count() - launches0
        step = captured.replay
        for _ in range(3):
            step()
        elapsed_ms = time_steps(step, steps, barrier)
        launches = per_step * steps
    else:
        launches0 = native.launch_count()
        elapsed_ms = time_steps(step, steps, barrier)
        launches = native.launch_count() - launches0
    ms_per_step = elapsed_ms / steps
    flops = sum(layer_flops(rows, l.k, l.n) for l, _m in layers)
    result = {"workload": describe(workload, spec, rows), "value": flops / (ms_per_step * 1e-3) / 1e12,
              "unit": "TFLOP/s", "ms_per_step": ms_per_step, "steps": steps,
              "us_per_layer": ms_per_step * 1e3 / len(layers), "gpu_launches": int(launches)}
    peaks = measured_peaks()
    result["frac_of_burst"] = result["value"] / peaks["tflops_burst"]
    result["frac_of_sustained"] = result["value"] / peaks["tflops_sustained"]
    if sustained:
        # the same step repeated for at least a second, under the power cap
        repeats = max(steps, int(MIN_SUSTAINED_SECONDS * 1e3 / ms_per_step) + 1)
        sampler = ClockSampler(device.index or 0)
        sampler.start()
        long_ms = time_steps(step, repeats, barrier)
        clocks = sampler.stop()
        per = long_ms / repeats
        result["sustained"] = {"value": flops / (per * 1e-3) / 1e12, "unit": "TFLOP/s", "steps": repeats,
                               "seconds": long_ms * 1e-3, "ms_per_step": per, "clocks": clocks,
                               "ms_x_sm_mhz": (per * clocks["sm_mhz"]) if clocks.get("sm_mhz") else None,
                               "frac_of_sustained_peak": flops / (per * 1e-3) / 1e12 / peaks["tflops_sustained"]}
    if with_kernel:
        result["roofline"] = kernel_alone(layers, inputs, steps, peaks)
    return result, layers, inputs, spec


def block_chain(layers, forward):
    """Data flow of the stacked blocks for the end-to-end pass: the block input feeds q/k/v (or
    the fused qkv); the first K columns of the first of them stand in for the attention
    output -> out-proj -> MLP up -> GELU -> MLP down -> next block.  A single layer is just
    y = layer(x)."""
    def run(x):
        h = x
        i = 0
        while i < len(layers):
            names = [layers[j][0].name.split(".")[-1] for j in range(i, min(i + 6, len(layers)))]
            if names[0] in ("q", "qkv"):
                heads = 3 if names[0] == "q" else 1
                outs = [forward(i + j, h, False) for j in range(heads)]
                a = outs[0][:, :layers[i + heads][0].k]
                a = forward(i + heads, a if a.is_contiguous() else a.contiguous(), True)
                u = torch.nn.functional.gelu(forward(i + heads + 1, a, True))
                h = forward(i + heads + 2, u, True)
                i += heads + 3
            else:
                h = forward(i, h, True)
                i += 1
        return h
    return run


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--workload", default="dit_block", choices=WORKLOAD_NAMES)
    parser.add_argument("--weight-mode", default="auto", choices=["auto", "int8_surrogate"],
                        help="one GPU, large batches: int8_surrogate runs the workload through the "
                             "integer route (approximate by construction; T-op/s, no kernel-alone pass)")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-extras", action="store_true",
                        help="one GPU: skip the decode and other-configuration measurements")
    parser.add_argument("--gather", default="epilogue", choices=["epilogue", "dma", "nccl"],
                        help="multi-GPU: how column shards are reassembled")
    parser.add_argument("--shard", default="n", choices=["n", "m"],
                        help="multi-GPU: n = output features sharded (the default; outputs gathered), "
                             "m = tokens sharded (every rank holds all weights, no collective)")
    parser.add_argument("--rows", type=int, default=0,
                        help="override the workload's token count (profiling on a smaller case)")
    args = parser.parse_args()

    if args.impl == "reference":
        run_reference_arm(args)
        return

    from orbitquant_b200 import native

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path to benchmark)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        run_multi_gpu(args, device, rank, world, local_rank)
        return
    if (args.rows or workload_spec(args.workload)["rows"]) <= 16:
        run_decode(args, device, rank)
        return

    warmup = max(3, args.warmup)
    sampler = ClockSampler(local_rank)
    sampler.start()
    integer_route = args.weight_mode == "int8_surrogate"
    result, layers, inputs, spec = measure_single_gpu(args.workload, device, args.steps, warmup,
                                                      rows_override=args.rows,
                                                      with_kernel=not integer_route,
                                                      weight_mode="int8_surrogate" if integer_route else None,
                                                      graph=integer_route)
    clocks = sampler.stop()
    rows = inputs[0].shape[0]

    # ---- end to end through the module API with host buffers ----
    host_x = synth_activations(rows, layers[0][0].k, 7, spec["outliers"]).pin_memory()
    host_y = torch.empty((rows, layers[-1][0].n), dtype=torch.bfloat16).pin_memory()
    chain = block_chain(layers, lambda i, x, _full: layers[i][1](x))
    e2e_ms, e2e_steps, e2e_mode = time_e2e(chain, host_x, host_y, device, args.steps,
                                           lambda: torch.cuda.synchronize(), use_graph=True)
    total_flops = sum(layer_flops(rows, l.k, l.n) for l, _m in layers)

    roofline = result.get("roofline")
    if roofline is not None:
        roofline["traffic"] = NCU_TRAFFIC_BYTES.get(args.workload) if not args.rows else None
    line = {
        "metric": "orbitlinear_tflops", "value": result["value"],
        "unit": "T-op/s" if integer_route else "TFLOP/s", "n_gpus": 1,
        "steps": args.steps, "warmup": warmup, "ms_per_step": result["ms_per_step"],
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "int8 (int32 accumulation)" if integer_route else "bf16",
        "data": "synthetic",
        "config": {
            "workload": result["workload"],
            "l2": "per-step working set (inputs+weights+outputs) exceeds the 126 MB L2; no flush",
            "parallelism": "single", "gather": None,
            "weight_mode": ("int8_surrogate (INT8 code operands on tcgen05.mma kind::i8; approximate by "
                            "construction; the step replayed from a CUDA graph)" if integer_route else
                            "centroid (f16 centroid operand, row norm in the epilogue)"),
            "cpu_sample": cpu_sample_note(args.workload),
        },
        "roofline": roofline,
        # fractions of the bf16 peaks say nothing about integer operations
        "forward": None if integer_route else {
            "frac_of_burst": result["frac_of_burst"], "frac_of_sustained": result["frac_of_sustained"],
            "what": "value / measured cuBLAS bf16 peak: prologue + GEMM of every projection"},
        "sustained": result.get("sustained"),
        "e2e": {"value": total_flops / (e2e_ms / e2e_steps * 1e-3) / 1e12, "unit": "TFLOP/s",
                "h2d_bytes_per_step": host_x.numel() * 2, "d2h_bytes_per_step": host_y.numel() * 2,
                "ms_per_step": e2e_ms / e2e_steps,
                "what": "OrbitQuantLinear modules chained as DiT block(s) (QKV, out, MLP up, GELU, "
                        "MLP down); pinned host input and output, copies on side streams "
                        "overlapping the neighbouring steps",
                "launch": ("sixteen steps per CUDA graph replay, host copies inside the graph"
                           if e2e_mode == "graph" else "eager, one C call per layer")},
        "gpu_launches": result["gpu_launches"], "clocks": clocks,
        "us_per_layer": result["us_per_layer"],
    }
    del layers, inputs, chain
    torch.cuda.empty_cache()

    if integer_route and line["sustained"]:
        line["sustained"]["unit"] = "T-op/s"
        line["sustained"].pop("frac_of_sustained_peak", None)
    if not args.no_extras and args.workload == "dit_block" and not args.rows and not integer_route:
        extras_steps = max(5, min(args.steps, 10))
        decode = {}
        for m in (1, 4, 16):
            try:
                decode[f"M={m}"] = measure_decode("vit_decode", m, device, 20, 3, with_e2e=False)
            except Exception as exc:  # the headline stands on its own
                decode[f"M={m}"] = {"error": f"{type(exc).__name__}: {exc}"}
        try:
            # the same pass on the DiT block's own layers at one token: the CUDA-core GEMV
            decode["dit_block M=1"] = measure_decode("dit_block", 1, device, 10, 3, with_e2e=False)
        except Exception as exc:
            decode["dit_block M=1"] = {"error": f"{type(exc).__name__}: {exc}"}
        line["decode"] = {"metric": "orbitlinear_decode_hbm_gbs", "unit": "GB/s",
                          "what": "ViT-base W4A6 (and, last case, the DiT block's W4A4 layers), 12 blocks x 4 "
                                  "projections in one CUDA graph, weights cold in L2 (several weight sets "
                                  "> 2x L2 walked per replay)",
                          "cases": decode}
        others = {}
        for name in ("single_layer", "mixed_bit", "video_dit"):
            try:
                res, l_, i_, _s = measure_single_gpu(name, device, extras_steps, 3, on_device=True,
                                                     sustained=False)
                del l_, i_
                torch.cuda.empty_cache()
                others[name] = res
            except Exception as exc:
                others[name] = {"error": f"{type(exc).__name__}: {exc}"}
        try:
            # the same four projections through the integer route of the reference's INT8
            # surrogate: INT8 code operands on the INT8 tensor-core instructions; approximate by
            # construction, so it is reported beside the headline, never as it
            res, l_, i_, _s = measure_single_gpu("dit_block", device, extras_steps, 3, on_device=True,
                                                 sustained=False, with_kernel=False,
                                                 weight_mode="int8_surrogate", graph=True)
            backends = sorted({m.last_activation_kernel_backend for _l, m in l_})
            del l_, i_
            torch.cuda.empty_cache()
            res["unit"] = "T-op/s"
            res["what"] = ("weight_mode int8_surrogate: rotate + quantise to INT8 codes, "
                           "tcgen05.mma kind::i8 with int32 accumulation; 2*M*K*N operations per layer; "
                           "the step captured in a CUDA graph and replayed")
            res["backends"] = backends
            res.pop("frac_of_burst", None)
            res.pop("frac_of_sustained", None)
            others["dit_block_int8_surrogate"] = res
        except Exception as exc:
            others["dit_block_int8_surrogate"] = {"error": f"{type(exc).__name__}: {exc}"}
        line["configs"] = others
    line["gemm_device_status"] = native.gemm_device_status()

    if not args.no_cpu_baseline:
        try:
            from oracle import ref_cpu
            if ref_cpu.available():
                cpu = time_reference_cpu(args.workload, 3, 1, CPU_SAMPLE_ROWS)
                line["cpu_baseline"] = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")}
            else:
                line["cpu_baseline"] = None
        except Exception as exc:  # the GPU numbers stand on their own
            line["cpu_baseline"] = {"error": str(exc)}
    print(json.dumps(line))


def time_e2e(chain, host_x, host_y, device, steps, barrier, use_graph=False):
    """Every step copies its input from pinned host memory and its result back; the copies of
    neighbouring steps run on two side streams so that PCIe transfers overlap the kernels
    (double-buffered device input, as a serving loop would do).  With `use_graph` sixteen such steps
    are also captured in one CUDA graph (copies included) and replayed, which takes the host's
    launch overhead out of the measurement; the faster of the two ways is returned.
    Returns (milliseconds, steps, "graph" | "eager")."""
    copy_in, copy_out = torch.cuda.Stream(), torch.cuda.Stream()
    dev_x = [torch.empty_like(host_x, device=device) for _ in range(2)]
    x_ready = [torch.cuda.Event() for _ in range(2)]
    x_free = [torch.cuda.Event() for _ in range(2)]
    main_stream = torch.cuda.current_stream()
    for ev in x_free:
        ev.record(main_stream)

    def e2e_step(i):
        b = i & 1
        with torch.cuda.stream(copy_in):
            copy_in.wait_event(x_free[b])
            dev_x[b].copy_(host_x, non_blocking=True)
            x_ready[b].record(copy_in)
        main_stream.wait_event(x_ready[b])
        h = chain(dev_x[b])
        x_free[b].record(main_stream)
        done = torch.cuda.Event()
        done.record(main_stream)
        with torch.cuda.stream(copy_out):
            copy_out.wait_event(done)
            host_y.copy_(h, non_blocking=True)
        h.record_stream(copy_out)

    for i in range(4):
        e2e_step(i)
    main_stream.wait_stream(copy_out)
    barrier()

    graph = None
    steps_per_replay = 16   # a replay starts and ends with an exposed copy: amortise them
    if use_graph:
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                cap = torch.cuda.current_stream()
                fork = torch.cuda.Event()
                fork.record(cap)
                copy_in.wait_event(fork)       # the side streams join the capture
                copy_out.wait_event(fork)
                free = [None, None]
                for i in range(steps_per_replay):
                    b = i & 1
                    with torch.cuda.stream(copy_in):
                        if free[b] is not None:
                            copy_in.wait_event(free[b])
                        dev_x[b].copy_(host_x, non_blocking=True)
                        ready = torch.cuda.Event()
                        ready.record(copy_in)
                    cap.wait_event(ready)
                    h = chain(dev_x[b])
                    free[b] = torch.cuda.Event()
                    free[b].record(cap)
                    with torch.cuda.stream(copy_out):
                        copy_out.wait_event(free[b])
                        host_y.copy_(h, non_blocking=True)
                cap.wait_stream(copy_in)
                cap.wait_stream(copy_out)
            for _ in range(2):
                graph.replay()
            torch.cuda.synchronize()
        except Exception as exc:  # eager timing below
            print(f"[bench] end-to-end graph capture failed ({type(exc).__name__}: {exc}); timing eagerly",
                  file=sys.stderr)
            graph = None
            torch.cuda.synchronize()

    # Both ways of driving the same calls are timed and the faster one is reported: the eager loop
    # overlaps the copies of ALL neighbouring steps but depends on the host keeping up with one C
    # call per layer; the graph needs no host work but exposes one copy at each end of a replay.
    e_start, e_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2e_steps = max(4, steps // 2 * 2)
    e_start.record()
    for i in range(e2e_steps):
        e2e_step(i)
    main_stream.wait_stream(copy_out)
    main_stream.wait_stream(copy_in)
    e_stop.record()
    barrier()
    best = (e_start.elapsed_time(e_stop), e2e_steps, "eager")
    if graph is not None:
        replays = max(1, (steps + steps_per_replay - 1) // steps_per_replay)
        g_start, g_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g_start.record()
        for _ in range(replays):
            graph.replay()
        g_stop.record()
        barrier()
        graph_ms = g_start.elapsed_time(g_stop)
        if graph_ms / (replays * steps_per_replay) < best[0] / best[1]:
            best = (graph_ms, replays * steps_per_replay, "graph")
    return best


def run_multi_gpu(args, device, rank, world, local_rank):
    import torch.distributed as dist

    from orbitquant_b200 import native
    from orbitquant_b200.sharding import gather_columns

    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=device)
    warmup = max(3, args.warmup)
    token_sharded = args.shard == "m"
    rows, layers, spec = build_layers(args.workload, device, rank, 1 if token_sharded else world, args.rows)
    global_rows = rows
    if token_sharded:
        rows = global_rows // world + (1 if rank < global_rows % world else 0)
    distinct = [synth_activations(rows, l.k, spec["seed"] * 1000 + i, spec["outliers"]).to(device)
                for i, (l, _m) in enumerate(layers[:6])]
    inputs = [distinct[i % 6] for i in range(len(layers))]

    # Column shards are reassembled either by the GEMM epilogue itself (each finished tile is
    # stored into every rank's full-width buffer over NVLink; one inter-rank barrier follows)
    # or, with --gather nccl, by an all-gather collective after the kernel.
    fused_gather = not token_sharded and args.gather in ("epilogue", "dma") and rows > 128
    dma_gather = fused_gather and args.gather == "dma"
    copy_stream = torch.cuda.Stream() if dma_gather else None
    peers = {}
    gather_note = None
    if fused_gather:
        from orbitquant_b200.sharding import PeerOutput
        ok = 1
        try:
            for i, (layer, _m) in enumerate(layers):
                if layer.gather:
                    peers[i] = PeerOutput(rows, layer.n, device)
        except Exception as exc:  # symmetric memory unavailable on this box: all ranks fall back together
            ok = 0
            gather_note = f"symmetric memory unavailable ({type(exc).__name__}); NCCL all-gather used"
        flag = torch.tensor([ok], device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) == 0:
            fused_gather = False
            peers = {}
            gather_note = gather_note or "a peer could not map symmetric memory; NCCL all-gather used"

    def sharded_forward(i, x, want_full, defer_wait=False):
        layer, module = layers[i]
        if not want_full or token_sharded:
            return module(x)
        if dma_gather:
            peers[i].scatter_dma(module, x, copy_stream)
            if not defer_wait:
                peers[i].wait()
            return peers[i].tensor
        if fused_gather:
            peers[i].scatter(module, x)
            if defer_wait:
                return None
            peers[i].wait()
            return peers[i].tensor
        return gather_columns(module(x), layer.n)

    # Before anything is timed: one gathered layer computed both ways must agree bit for bit
    # on every rank (peer-stored full-width buffer against the NCCL all-gather of the shards).
    gather_check = "not applicable (no output is gathered)"
    check_layer = next((i for i, (l, _m) in enumerate(layers) if l.gather), None)
    if check_layer is not None and not token_sharded:
        layer, module = layers[check_layer]
        full = sharded_forward(check_layer, inputs[check_layer], True).clone()
        expect = gather_columns(module(inputs[check_layer]), layer.n)
        same = torch.tensor([1 if torch.equal(full, expect) else 0], device=device)
        dist.all_reduce(same, op=dist.ReduceOp.MIN)
        gather_check = "bit-equal" if int(same.item()) == 1 else "MISMATCH"

    def step():
        # the projections are independent here, so each layer's transfers (peer stores issued by
        # the GEMM epilogue, or copy-engine copies) may still be landing while the next layer
        # computes; the inter-rank barriers that complete them are joined at the end of the step
        outs = [sharded_forward(i, x, layers[i][0].gather, defer_wait=True) for i, x in enumerate(inputs)]
        if dma_gather or fused_gather:
            for i, (layer, _m) in enumerate(layers):
                if layer.gather:
                    peers[i].wait()
                    outs[i] = peers[i].tensor
        return outs

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        step()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = native.launch_count()
    elapsed_ms = time_steps(step, args.steps, barrier)
    launches = native.launch_count() - launches0
    t = torch.tensor([elapsed_ms], device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_per_step = float(t.item()) / args.steps
    total_flops = sum(layer_flops(global_rows, l.k, l.n) for l, _m in layers)
    value = total_flops / (ms_per_step * 1e-3) / 1e12

    peaks = measured_peaks()
    roofline = kernel_alone(layers, inputs, args.steps, peaks)
    roofline["traffic"] = None  # the one-GPU ncu capture does not describe a shard's launch
    roofline["what"] = "this rank's shard GEMMs (rank 0)"

    # ---- end to end through the module API with host buffers ----
    host_x = synth_activations(rows, layers[0][0].k, 7, spec["outliers"]).pin_memory()
    host_y = torch.empty((rows, layers[-1][0].n), dtype=torch.bfloat16).pin_memory()

    def e2e_forward(i, x, want_full):
        if want_full or token_sharded:
            return sharded_forward(i, x, True)
        # head-sharded QKV: the rank keeps its columns; what stands in for its attention output
        # (its share of the first K columns) is all-gathered for the out-proj, as the heads'
        # outputs would be
        layer, module = layers[i]
        local = module(x)
        k_next = layers[i + 1][0].k if i + 1 < len(layers) else layer.n
        share = local[:, :k_next // world].contiguous()
        return gather_columns(share, k_next)

    chain = block_chain(layers, e2e_forward)
    e2e_ms, e2e_steps, _e2e_mode = time_e2e(chain, host_x, host_y, device, args.steps, barrier)
    t = torch.tensor([e2e_ms], device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t.item())
    clocks = sampler.stop() if rank == 0 else None

    if rank == 0:
        if dma_gather:
            gather = ("copy engines (cudaMemcpy2DAsync into every rank's buffer) under the next "
                      "layer's kernels, barriers at the end of the step")
        elif fused_gather:
            gather = ("gemm epilogue stores into every rank's buffer (peer memory); one barrier per "
                      "gathered layer, joined at the end of the step (the projections are independent)")
        elif token_sharded:
            gather = "none (token-sharded)"
        else:
            gather = gather_note or "nccl all_gather_into_tensor"
        line = {
            "metric": "orbitlinear_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {
                "workload": describe(args.workload, spec, global_rows),
                "l2": "per-step working set (inputs+weights+outputs) exceeds the 126 MB L2; no flush",
                "parallelism": f"m_shard{world}" if token_sharded else f"n_shard{world}",
                "gather": gather,
                "weight_mode": "centroid (f16 centroid operand, row norm in the epilogue)",
                "cpu_sample": cpu_sample_note(args.workload),
            },
            "gather_check": gather_check,
            "roofline": roofline,
            "e2e": {"value": total_flops / (e2e_ms / e2e_steps * 1e-3) / 1e12, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": host_x.numel() * 2, "d2h_bytes_per_step": host_y.numel() * 2,
                    "ms_per_step": e2e_ms / e2e_steps,
                    "what": "OrbitQuantLinear column shards chained as a DiT block; QKV stays "
                            "head-sharded (its attention stand-in is all-gathered), out-proj and "
                            "MLP outputs are reassembled; pinned host input and output"},
            "gpu_launches": int(launches), "clocks": clocks,
            "us_per_layer": ms_per_step * 1e3 / len(layers),
            "gemm_device_status": native.gemm_device_status(),
        }
        print(json.dumps(line))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
