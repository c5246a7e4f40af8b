"""Benchmark of the OrbitQuant quantized-linear forward on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload dit_block|video_dit|vit_decode]

Default workload (``dit_block``): the four W4A4 projections of one DiT double-stream block
-- fused QKV 3072->9216, out-proj 3072->3072, MLP 3072->12288 and 12288->3072 -- on
M = 4096 image + 512 text = 4608 bf16 tokens with 0.5 % outlier channels (x20), weights
~N(0, 0.02), RPBH block "paper", seed 1; synthetic data, random-init weights.  A step is
one OrbitLinear forward (rotate-and-quantize prologue + packed-weight GEMM) of each of the
four projections on inputs already resident in HBM.  ``value`` is the algorithmic
2*M*K*N flop of the step divided by its device time.

With ``--gpus N`` (launched under torchrun, one rank per GPU) every projection is sharded
along its output features; out-proj / MLP outputs are all-gathered over NCCL because their
consumers need full rows, the QKV output stays head-sharded.  Total work is fixed, so the
scaling is "strong".

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
from pathlib import Path

import torch

REPO = Path(__file__).resolve().parent
if str(REPO) not in sys.path:
    sys.path.insert(0, str(REPO))

WORKLOADS = {
    # name: (rows, [(layer name, K, N, gather_output)], weight std, seed, w_bits, a_bits)
    "dit_block": (4608, [("qkv", 3072, 9216, False), ("out", 3072, 3072, True),
                         ("fc1", 3072, 12288, True), ("fc2", 12288, 3072, True)], 0.02, 1, 4, 4),
    "video_dit": (32760, [("qkv", 5120, 15360, False), ("out", 5120, 5120, True),
                          ("fc1", 5120, 13824, True), ("fc2", 13824, 5120, True)], 0.015, 3, 4, 4),
    "vit_decode": (16, [("qkv", 768, 2304, False), ("out", 768, 768, True),
                        ("fc1", 768, 3072, True), ("fc2", 3072, 768, True)], 0.02, 4, 4, 6),
}

# DRAM bytes (read + write) per launch of the dominant kernel from an ncu capture, keyed by
# workload; filled from the summaries under profiles/ (None until captured).
NCU_TRAFFIC_BYTES = {
    # profiles/gemm_w4_tcgen05_dit_block_traffic.md: mean over the four projections
    "dit_block": 97.5e6,
    "video_dit": None,
    "vit_decode": None,
}

CPU_SAMPLE_ROWS = 512


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


def synth_weight_payload(k, n, w_bits, std, seed):
    """Packed indices / row norms with the statistics OrbitQuant produces for W ~ N(0, std):
    rotated unit rows are near-Gaussian with variance 1/K, so indices follow the codebook's
    cell probabilities and row norms concentrate at std*sqrt(K).  Drawing them directly
    (instead of quantising an N x K fp32 matrix on the CPU) keeps start-up short; parity
    tests quantise real matrices."""
    from orbitquant_b200 import get_codebook, pack_lowbit

    g = torch.Generator().manual_seed(seed)
    cb = get_codebook(k, w_bits)
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


def synth_activations(rows, k, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, k, generator=g)
    outliers = torch.randperm(k, generator=g)[: max(1, round(0.005 * k))]
    x[:, outliers] *= 20.0
    return x.to(torch.bfloat16)


def build_layers(workload, device, rank=0, world=1, rows_override=0):
    from orbitquant_b200 import OrbitQuantConfig, OrbitQuantLinear
    from orbitquant_b200.sharding import shard_linear

    rows, specs, std, seed, w_bits, a_bits = WORKLOADS[workload]
    cfg = OrbitQuantConfig(weight_bits=w_bits, activation_bits=a_bits, rotation_seed=seed)
    layers = []
    for i, (name, k, n, gather) in enumerate(specs):
        packed, norms, bias = synth_weight_payload(k, n, w_bits, std, seed * 100 + i)
        module = OrbitQuantLinear(in_features=k, out_features=n, config=cfg, module_name=name,
                                  source_weight_layout="out_in", bias=bias,
                                  packed_weight_indices=packed, row_norms=norms, debug_weight=None)
        if world > 1:
            module = shard_linear(module, rank, world, config=cfg)
        layers.append((name, k, n, gather, module.to(device)))
    return (rows_override or rows), layers, w_bits, a_bits


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
        sm, sm_max, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                sm_max.append(float(parts[1]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[3:7]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(sm_max), "reasons": sorted(reasons),
                "samples": len(sm)}


def time_reference_cpu(workload, steps, warmup, sample_rows):
    """The reference's compiled CPU kernels on `sample_rows` rows of every layer."""
    from oracle import ref_cpu
    from orbitquant_b200 import get_codebook, get_rpbh_rotation

    rows, specs, std, seed, w_bits, a_bits = WORKLOADS[workload]
    m = min(rows, sample_rows)
    prepared = []
    for i, (name, k, n, _g) in enumerate(specs):
        packed, norms, bias = synth_weight_payload(k, n, w_bits, std, seed * 100 + i)
        rot = get_rpbh_rotation(k, seed, "paper")
        prepared.append((k, n, packed, norms, bias.float(), rot, get_codebook(k, a_bits),
                         get_codebook(k, w_bits), synth_activations(m, k, seed * 1000 + i)))

    def one_pass():
        for k, n, packed, norms, bias, rot, acb, wcb, x in prepared:
            ref_cpu.linear_forward(
                x, packed, norms, bias, permutation=rot.permutation, signs=rot.signs,
                act_centroids=acb.centroids, act_boundaries=acb.boundaries,
                w_centroids=wcb.centroids, w_bits=w_bits, out_features=n, eps=1e-10,
                block_size=rot.block_size)

    for _ in range(max(1, warmup)):
        one_pass()
    t0 = time.perf_counter()
    for _ in range(steps):
        one_pass()
    seconds = (time.perf_counter() - t0) / steps
    flops = sum(layer_flops(m, k, n) for _n, k, n, _g in specs)
    threads = int(os.environ.get("ORBITQUANT_CPU_THREADS") or os.environ.get("OMP_NUM_THREADS") or 0)
    if threads <= 0:
        try:
            threads = min(64, len(os.sched_getaffinity(0)))
        except AttributeError:
            threads = os.cpu_count() or 1
    report = ref_cpu.host_isa_report()
    return {
        "value": flops / seconds / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "reference",
        "sample": (f"{m} of {rows} rows of each of the {len(specs)} projections, "
                   f"{steps} timed pass(es); reference CPU kernels oracle/_ref, "
                   f"ORBITQUANT_CPU_ISA={report['isa_env']}, avx512_bf16={report['avx512_bf16']}"),
        "ms_per_step": seconds * 1e3,
    }


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import ref_cpu

    rows, specs, _std, _seed, w_bits, a_bits = WORKLOADS[args.workload]
    base = {"impl": "reference", "metric": "orbitlinear_tflops", "unit": "TFLOP/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "higher_is_better": True}
    if not ref_cpu.available():
        print(json.dumps({"impl": "reference",
                          "unavailable": "oracle/_ref (reference CPU kernels) was not built"}))
        return
    steps = max(1, min(args.steps, 3))
    cpu = time_reference_cpu(args.workload, steps, min(args.warmup, 1), CPU_SAMPLE_ROWS)
    line = dict(base)
    line.update({
        "value": cpu["value"], "ms_per_step": cpu["ms_per_step"], "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"{args.workload} W{w_bits}A{a_bits} bf16, rows sample "
                               f"{min(rows, CPU_SAMPLE_ROWS)}/{rows}",
                   "layers": [[n_, k, n] for n_, k, n, _g in specs]},
        "cpu_baseline": {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": cpu["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    })
    print(json.dumps(line))


def run_decode(args, device, rank):
    """Decode-sized batches (rows <= 16): the forward is weight streaming, so the figure of
    merit is HBM GB/s.  One pass = 12 transformer blocks x 4 projections, captured in a
    CUDA graph (launch overhead would otherwise dominate layers this small).  Two graphs:
    `warm` replays one 12-block weight set that fits the 126 MB L2; `cold` walks enough
    distinct weight sets (> 2x L2) that every weight byte comes from HBM."""
    from orbitquant_b200 import OrbitQuantConfig, OrbitQuantLinear, native

    rows_default, specs, std, seed, w_bits, a_bits = WORKLOADS[args.workload]
    rows = args.rows or min(rows_default, 16)
    blocks = 12
    cfg = OrbitQuantConfig(weight_bits=w_bits, activation_bits=a_bits, rotation_seed=seed)
    set_bytes = blocks * sum((n * k * w_bits + 7) // 8 for _n, k, n, _g in specs)
    sets = max(2, -(-300_000_000 // set_bytes))
    payloads = [synth_weight_payload(k, n, w_bits, std, seed * 100 + i) for i, (_n, k, n, _g) in enumerate(specs)]
    modules = []
    for s_idx in range(sets):
        for b in range(blocks):
            for i, (name, k, n, _g) in enumerate(specs):
                packed, norms, bias = payloads[i]
                # distinct device copies: same statistics, different addresses
                modules.append(OrbitQuantLinear(
                    in_features=k, out_features=n, config=cfg, module_name=f"s{s_idx}.b{b}.{name}",
                    source_weight_layout="out_in", bias=bias.clone(), packed_weight_indices=packed.clone(),
                    row_norms=norms.clone(), debug_weight=None).to(device))
    per_set = blocks * len(specs)
    inputs = [synth_activations(rows, k, seed * 1000 + i).to(device) for i, (_n, k, _N, _g) in enumerate(specs)]

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
        for _ in range(max(3, args.warmup)):
            graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(replays):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / replays

    sampler = ClockSampler(device.index or 0)
    sampler.start()
    launches0 = native.launch_count()
    warm_graph = capture(lambda: run_set(0))
    launches_per_pass = (native.launch_count() - launches0) // 3
    warm_ms = time_graph(warm_graph, args.steps)

    def all_sets():
        for s_idx in range(sets):
            run_set(s_idx)

    cold_graph = capture(all_sets)
    cold_ms = time_graph(cold_graph, max(3, args.steps // sets)) / sets

    # the matmul kernel alone, cold, on pre-quantised activations
    xqs = []
    for j, (name, k, n, _g) in enumerate(specs):
        m = modules[j]
        xqs.append(native.quantize_activations(
            inputs[j], m._rotation_permutation, m._rotation_signs, m._activation_codebook_centroids,
            m._activation_codebook_boundaries, eps=m.activation_eps, block_size=m.rotation.block_size))

    def matmul_only():
        for idx, m in enumerate(modules):
            native.matmul_packed_weight(xqs[idx % len(specs)], m.packed_weight_indices, m.row_norms,
                                        m._weight_codebook_centroids, bits=w_bits,
                                        out_features=m.out_features, in_features=m.in_features,
                                        bias=m.bias)

    # layers of 3 MB and more take the few-token tcgen05 kernel (preceded here by the kernel
    # that converts the caller's activations to its f16 operand), smaller ones the
    # single-launch small-rows kernel
    big = [n * k * w_bits // 8 >= 3 << 20 for _n, k, n, _g in specs]
    decode_kernel_name = ("rows_to_f16_kernel + skinny_tcgen05_kernel" if all(big) else
                          "small_rows_w4_kernel" if not any(big) else
                          "small_rows_w4_kernel / rows_to_f16_kernel + skinny_tcgen05_kernel by layer size")
    kernel_graph = capture(matmul_only)
    kernel_ms = time_graph(kernel_graph, max(3, args.steps // sets)) / sets
    clocks = sampler.stop()

    pass_bytes = blocks * sum(layer_bytes(rows, k, n, w_bits, a_bits) for _n, k, n, _g in specs)
    pass_flops = blocks * sum(layer_flops(rows, k, n) for _n, k, n, _g in specs)
    peaks = measured_peaks()
    cold_gbs = pass_bytes / (cold_ms * 1e-3) / 1e9
    kernel_gbs = pass_bytes / (kernel_ms * 1e-3) / 1e9

    # end to end through the module API, eager, pinned host input and output
    host_x = synth_activations(rows, specs[0][1], 7).pin_memory()
    host_y = torch.empty((rows, specs[-1][2]), dtype=torch.bfloat16).pin_memory()

    def e2e_pass():
        h = host_x.to(device, non_blocking=True)
        for b in range(blocks):
            qkv = modules[4 * b](h)
            a = modules[4 * b + 1](qkv[:, :specs[1][1]].contiguous())
            u = torch.nn.functional.gelu(modules[4 * b + 2](a))
            h = modules[4 * b + 3](u)
        host_y.copy_(h, non_blocking=True)

    for _ in range(3):
        e2e_pass()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2e_steps = max(3, args.steps // 4)
    e0.record()
    for _ in range(e2e_steps):
        e2e_pass()
    e1.record()
    torch.cuda.synchronize()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps

    line = {
        "metric": "orbitlinear_decode_hbm_gbs", "value": cold_gbs, "unit": "GB/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": cold_ms,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {
            "workload": (f"{args.workload}: {blocks} blocks x ({', '.join(f'{n_} {k}->{n}' for n_, k, n, _g in specs)}) "
                         f"OrbitLinear W{w_bits}A{a_bits} bf16, M={rows}, one CUDA graph per pass"),
            "l2": f"cold: {sets} distinct weight sets ({sets * set_bytes / 1e6:.0f} MB > 2x L2) walked per replay",
            "algorithmic_bytes_per_pass": pass_bytes,
        },
        "l2_warm": {"value": pass_bytes / (warm_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_pass": warm_ms,
                    "note": f"one {set_bytes / 1e6:.1f} MB weight set replayed; it fits the L2"},
        "us_per_layer": cold_ms * 1e3 / per_set,
        "tflops": pass_flops / (cold_ms * 1e-3) / 1e12,
        "roofline": {"bound": "hbm", "achieved": kernel_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": kernel_gbs / peaks["hbm_gbs"], "traffic": NCU_TRAFFIC_BYTES.get(args.workload),
                     "peak_source": peaks["source"], "kernel": decode_kernel_name,
                     "avg_launch_us": kernel_ms * 1e3 / per_set, "launches_timed": per_set * sets},
        "e2e": {"value": pass_bytes / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s",
                "h2d_bytes_per_step": host_x.numel() * 2, "d2h_bytes_per_step": host_y.numel() * 2,
                "ms_per_step": e2e_ms,
                "what": "12 blocks chained eagerly through OrbitQuantLinear (QKV, out, MLP up, GELU, MLP down)"},
        "gpu_launches": int(launches_per_pass * args.steps), "clocks": clocks,
        "gemm_device_status": native.gemm_device_status(),
    }
    if not args.no_cpu_baseline:
        try:
            from oracle import ref_cpu
            if ref_cpu.available():
                cpu = time_reference_cpu(args.workload, 3, 1, rows)
                seconds = cpu["ms_per_step"] * 1e-3 * blocks
                line["cpu_baseline"] = {"value": pass_bytes / seconds / 1e9, "unit": "GB/s",
                                        "cores": cpu["cores"], "kind": "reference", "sample": cpu["sample"]}
        except Exception as exc:
            line["cpu_baseline"] = {"error": str(exc)}
    if rank == 0:
        print(json.dumps(line))


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--workload", default="dit_block", choices=sorted(WORKLOADS))
    parser.add_argument("--no-cpu-baseline", action="store_true")
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

    import torch.distributed as dist

    from orbitquant_b200 import native
    from orbitquant_b200.sharding import gather_columns

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path to benchmark)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    distributed = world > 1
    if distributed:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)

    if not distributed and (args.rows or WORKLOADS[args.workload][0]) <= 16:
        run_decode(args, device, rank)
        return

    warmup = max(3, args.warmup)
    token_sharded = distributed and args.shard == "m"
    rows, layers, w_bits, a_bits = build_layers(args.workload, device, rank, 1 if token_sharded else world,
                                                args.rows)
    global_rows = rows
    if token_sharded:
        rows = global_rows // world + (1 if rank < global_rows % world else 0)
    inputs = [synth_activations(rows, k, WORKLOADS[args.workload][3] * 1000 + i).to(device)
              for i, (_n, k, _N, _g, _m) in enumerate(layers)]

    # Column shards are reassembled either by the GEMM epilogue itself (each finished tile is
    # stored into every rank's full-width buffer over NVLink; one inter-rank barrier follows)
    # or, with --gather nccl, by an all-gather collective after the kernel.
    fused_gather = distributed and not token_sharded and args.gather in ("epilogue", "dma") and rows > 128
    dma_gather = fused_gather and args.gather == "dma"
    copy_stream = torch.cuda.Stream() if dma_gather else None
    peers = {}
    gather_note = None
    if fused_gather:
        from orbitquant_b200.sharding import PeerOutput
        ok = 1
        try:
            for i, (_name, _k, n, _g, _m) in enumerate(layers):
                peers[i] = PeerOutput(rows, n, device)
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
        _name, _k, n, _g, module = layers[i]
        if not (distributed and want_full) or token_sharded:
            return module(x)
        if dma_gather:
            peers[i].scatter_dma(module, x, copy_stream)
            if not defer_wait:
                peers[i].wait()
            return peers[i].tensor
        if fused_gather:
            peers[i].scatter(module, x)
            peers[i].wait()
            return peers[i].tensor
        return gather_columns(module(x), n)

    def step():
        # the four projections are independent here, so with the copy-engine gather each
        # layer's transfers run under the next layer's kernels and are joined at the end
        outs = [sharded_forward(i, x, layers[i][3], defer_wait=True) for i, x in enumerate(inputs)]
        if dma_gather:
            for i, layer in enumerate(layers):
                if layer[3]:
                    peers[i].wait()
        return outs

    def barrier():
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = native.launch_count()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        step()
    stop.record()
    barrier()
    launches = native.launch_count() - launches0
    elapsed_ms = start.elapsed_time(stop)
    if distributed:
        t = torch.tensor([elapsed_ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    ms_per_step = elapsed_ms / args.steps
    total_flops = sum(layer_flops(global_rows, k, n) for _n, k, n, _g, _m in layers)
    value = total_flops / (ms_per_step * 1e-3) / 1e12

    # ---- dominant kernel alone: the packed-weight GEMM on pre-quantised activations ----
    peaks = measured_peaks()
    kernel_ms = 0.0
    kernel_launches = 0
    small = rows <= 16
    prepared = []
    for (name, k, n, gather, module), x in zip(layers, inputs):
        xq = native.quantize_activations(
            x, module._rotation_permutation, module._rotation_signs,
            module._activation_codebook_centroids, module._activation_codebook_boundaries,
            eps=module.activation_eps, block_size=module.rotation.block_size)
        if small:
            prepared.append((xq, None, None))
        else:
            prepared.append(native.rows_to_f16_operand(xq, module._weight_codebook_centroids))
    torch.cuda.synchronize()
    events = []
    for it in range(args.steps + 2):
        for (name, k, n, gather, module), (operand, scale, table) in zip(layers, prepared):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            if small:
                native.matmul_packed_weight(operand, module.packed_weight_indices, module.row_norms,
                                            module._weight_codebook_centroids, bits=w_bits,
                                            out_features=module.out_features, in_features=k,
                                            bias=module.bias)
            else:
                native.gemm_tcgen05_f16(operand, scale, module.packed_weight_indices,
                                        module.row_norms, module._weight_codebook_centroids,
                                        out_features=module.out_features, bias=module.bias,
                                        table_scale=table)
            e1.record()
            if it >= 2:
                events.append((e0, e1))
    torch.cuda.synchronize()
    for e0, e1 in events:
        kernel_ms += e0.elapsed_time(e1)
        kernel_launches += 1
    local_flops = sum(layer_flops(rows, k, m.out_features) for _n, k, _N, _g, m in layers)
    if small:
        algo_bytes = sum(layer_bytes(rows, k, m.out_features, w_bits, a_bits) for _n, k, _N, _g, m in layers)
        achieved = algo_bytes * args.steps / (kernel_ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": achieved / peaks["hbm_gbs"]}
    else:
        achieved = local_flops * args.steps / (kernel_ms * 1e-3) / 1e12
        roofline = {"bound": "tensor", "achieved": achieved, "peak": peaks["tflops_sustained"],
                    "unit": "TFLOP/s", "frac": achieved / peaks["tflops_sustained"],
                    "peak_burst": peaks["tflops_burst"], "frac_of_burst": achieved / peaks["tflops_burst"]}
    roofline.update({"traffic": NCU_TRAFFIC_BYTES.get(args.workload), "peak_source": peaks["source"],
                     "kernel": "small_rows_w4_kernel" if small else "gemm_w4_tcgen05_kernel",
                     "avg_launch_us": kernel_ms * 1e3 / max(1, kernel_launches),
                     "launches_timed": kernel_launches})

    # ---- end to end through the module API with host buffers ----
    name0, k0, n0, _g0, first = layers[0]
    host_x = synth_activations(rows, k0, 7).pin_memory()
    last_n = layers[-1][2]
    host_y = torch.empty((rows, last_n), dtype=torch.bfloat16).pin_memory()

    # Every step copies its input from pinned host memory and its result back; the copies of
    # neighbouring steps run on two side streams so that PCIe transfers overlap the kernels
    # (double-buffered device input, as a serving loop would do).
    copy_in, copy_out = torch.cuda.Stream(), torch.cuda.Stream()
    dev_x = [torch.empty_like(host_x, device=device) for _ in range(2)]
    x_ready = [torch.cuda.Event() for _ in range(2)]
    x_free = [torch.cuda.Event() for _ in range(2)]
    main = torch.cuda.current_stream()
    for ev in x_free:
        ev.record(main)

    def e2e_step(i):
        # DiT block data flow: x -> QKV; the q slice stands in for the attention output;
        # -> out-proj -> MLP up -> GELU -> MLP down; only x and the block output cross PCIe.
        b = i & 1
        with torch.cuda.stream(copy_in):
            copy_in.wait_event(x_free[b])
            dev_x[b].copy_(host_x, non_blocking=True)
            x_ready[b].record(copy_in)
        main.wait_event(x_ready[b])
        qkv = sharded_forward(0, dev_x[b], True)
        x_free[b].record(main)
        h = qkv[:, :layers[1][1]].contiguous()
        h = sharded_forward(1, h, True)
        h = sharded_forward(2, h, True)
        h = torch.nn.functional.gelu(h)
        h = sharded_forward(3, h, True)
        done = torch.cuda.Event()
        done.record(main)
        with torch.cuda.stream(copy_out):
            copy_out.wait_event(done)
            host_y.copy_(h, non_blocking=True)
        h.record_stream(copy_out)

    for i in range(4):
        e2e_step(i)
    main.wait_stream(copy_out)
    barrier()
    e_start, e_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2e_steps = max(4, args.steps // 2 * 2)
    e_start.record()
    for i in range(e2e_steps):
        e2e_step(i)
    main.wait_stream(copy_out)
    main.wait_stream(copy_in)
    e_stop.record()
    barrier()
    e2e_ms = e_start.elapsed_time(e_stop)
    if distributed:
        t = torch.tensor([e2e_ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_value = total_flops / (e2e_ms / e2e_steps * 1e-3) / 1e12
    clocks = sampler.stop() if rank == 0 else None

    if rank == 0:
        line = {
            "metric": "orbitlinear_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {
                "workload": (f"{args.workload}: OrbitLinear W{w_bits}A{a_bits} bf16, M={global_rows}, "
                             + ", ".join(f"{n_} {k}->{n}" for n_, k, n, _g, _m in layers)),
                "l2": "per-step working set (inputs+weights+outputs) exceeds the 126 MB L2; no flush",
                "parallelism": (f"m_shard{world}" if token_sharded else f"n_shard{world}") if distributed else "single",
                "gather": (("copy engines (cudaMemcpy2DAsync into every rank's buffer) under the next layer's kernels, barriers at the end of the step"
                            if dma_gather else "gemm epilogue stores into every rank's buffer (peer memory), one barrier")
                           if fused_gather else ("none (token-sharded)" if token_sharded else
                                                 (gather_note or "nccl all_gather_into_tensor"))) if distributed else None,
                "weight_mode": "centroid (f16 centroid operand, row norm in the epilogue)",
            },
            "roofline": roofline,
            "e2e": {"value": e2e_value, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": host_x.numel() * 2, "d2h_bytes_per_step": host_y.numel() * 2,
                    "ms_per_step": e2e_ms / e2e_steps,
                    "what": "OrbitQuantLinear modules chained as a DiT block (QKV, out, MLP up, "
                            "GELU, MLP down); pinned host input and output, copies on side "
                            "streams overlapping the neighbouring steps"},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "us_per_layer": ms_per_step * 1e3 / len(layers),
            "gemm_device_status": native.gemm_device_status(),
        }
        if not args.no_cpu_baseline and not distributed:
            try:
                from oracle import ref_cpu
                if ref_cpu.available():
                    cpu = time_reference_cpu(args.workload, 1, 1, CPU_SAMPLE_ROWS)
                    line["cpu_baseline"] = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")}
                else:
                    line["cpu_baseline"] = None
            except Exception as exc:  # the GPU numbers stand on their own
                line["cpu_baseline"] = {"error": str(exc)}
        print(json.dumps(line))
    if distributed:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
