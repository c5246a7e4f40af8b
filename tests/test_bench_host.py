"""Host-side pieces of bench.py that need no GPU: the workload tables (shapes and bit widths of
the benchmark configurations), the byte / flop accounting behind the roofline figures, and the
reference arm (the reference's CPU kernels timed on a row sample), which must print one JSON
line with the contract's keys."""
from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import bench

REPO = Path(__file__).resolve().parent.parent


def test_mixed_bit_assignment_follows_the_boundary_rule():
    plan = bench.mixed_bit_assignment()
    assert len(plan) == 8
    for b in (0, 1, 2, 5, 6, 7):
        assert set(plan[b].values()) == {(4, 4)}
    for b in (3, 4):
        assert plan[b]["q"] == plan[b]["k"] == (2, 4)
        assert plan[b]["v"] == plan[b]["out"] == plan[b]["fc1"] == plan[b]["fc2"] == (3, 3)
    # two blocks: min(4, (2 - 1) // 2) = 0 would protect nothing; short stacks keep the full count
    assert all(set(block.values()) == {(4, 4)} for block in bench.mixed_bit_assignment(blocks=2))


def test_workload_tables():
    counts = {"dit_block": 4, "single_layer": 1, "mixed_bit": 48, "video_dit": 4, "vit_decode": 4}
    for name in bench.WORKLOAD_NAMES:
        spec = bench.workload_spec(name)
        assert len(spec["layers"]) == counts[name]
        for layer in spec["layers"]:
            assert layer.k % 64 == 0 and layer.n % 8 == 0
            assert layer.w_bits in (2, 3, 4) and layer.a_bits in (3, 4, 6)
        assert bench.describe(name, spec, spec["rows"]).startswith(name)
    dit = bench.workload_spec("dit_block")
    assert dit["rows"] == 4608
    assert [(l.k, l.n) for l in dit["layers"]] == [(3072, 9216), (3072, 3072), (3072, 12288), (12288, 3072)]
    assert bench.workload_spec("single_layer")["block_size"] == 256


def test_flop_and_byte_accounting():
    assert bench.layer_flops(4608, 3072, 9216) == 2.0 * 4608 * 3072 * 9216
    k, n, rows = 3072, 3072, 16
    weights = n * k // 2
    total = bench.layer_bytes(rows, k, n, 4, 4)
    # packed weights dominate a decode-sized call; activations in and out, norms and bias follow
    assert weights < total < weights + rows * k * 2 + rows * n * 2 + 4 * n + 6 * k + 1024
    # three-bit rows are 3/8 of a byte per weight, rounded up once per layer
    assert bench.layer_bytes(1, 64, 8, 3, 3) - bench.layer_bytes(1, 64, 8, 4, 3) == (8 * 64 * 3 + 7) // 8 - 8 * 64 // 2 - 32


def test_reference_arm_prints_the_contract_line():
    done = subprocess.run([sys.executable, str(REPO / "bench.py"), "--impl", "reference", "--steps", "1",
                           "--warmup", "1"], capture_output=True, text=True, timeout=600, cwd=REPO)
    assert done.returncode == 0, done.stderr[-2000:]
    lines = [l for l in done.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference"
    if "unavailable" in line:
        assert isinstance(line["unavailable"], str) and line["unavailable"]
        return
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better",
                "config", "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["metric"] == "orbitlinear_tflops" and line["value"] > 0
    assert line["cpu_baseline"]["kind"] == "reference" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
