"""N-sharding host logic on two gloo ranks (CPU): shard bounds, byte ranges, the column
all-gather -- with the CPU oracle standing in for the GPU kernels."""
from __future__ import annotations

import os
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

REPO = Path(__file__).resolve().parent.parent

from orbitquant_b200 import OrbitQuantConfig, OrbitQuantLinear
from orbitquant_b200.sharding import gather_columns, shard_bounds, shard_byte_range, shard_linear


def test_shard_bounds_cover_and_align():
    for n, world in ((9216, 8), (3072, 8), (13824, 8), (100, 3), (8, 4), (1, 2), (2304, 2)):
        covered = []
        for r in range(world):
            lo, hi = shard_bounds(n, world, r)
            assert 0 <= lo <= hi <= n
            assert lo % 8 == 0 or lo == n
            covered.append((lo, hi))
        assert covered[0][0] == 0 and covered[-1][1] == n
        for (a, b), (c, d) in zip(covered, covered[1:]):
            assert b == c
    assert shard_bounds(9216, 8, 3) == (3456, 4608)
    assert shard_byte_range(8, 16, 768, 3) == (8 * 288, 16 * 288)
    with pytest.raises(ValueError):
        shard_byte_range(0, 8, 5, 3)
    with pytest.raises(ValueError):
        shard_bounds(8, 2, 2)


def test_shard_linear_views_the_byte_stream():
    cfg = OrbitQuantConfig(weight_bits=3, activation_bits=3, rotation_seed=2)
    full = OrbitQuantLinear.from_linear(torch.nn.Linear(256, 40), config=cfg, module_name="p")
    parts = [shard_linear(full, r, 3) for r in range(3)]
    assert sum(p.out_features for p in parts) == 40
    assert torch.equal(torch.cat([p.packed_weight_indices for p in parts]), full.packed_weight_indices)
    assert torch.equal(torch.cat([p.row_norms for p in parts]), full.row_norms)
    assert torch.equal(torch.cat([p.bias for p in parts]), full.bias)
    assert parts[1].shard_rows == shard_bounds(40, 3, 1)
    assert torch.equal(parts[0].rotation.permutation, full.rotation.permutation)
    assert parts[0].rotation.block_size == full.rotation.block_size


def _worker(rank: int, world: int, port: int, out_path: str):
    sys.path.insert(0, str(REPO))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import oracle
        torch.manual_seed(0)
        cfg = OrbitQuantConfig(weight_bits=4, activation_bits=4, rotation_seed=1)
        full = OrbitQuantLinear.from_linear(torch.nn.Linear(256, 52), config=cfg, module_name="p")
        x = torch.randn(7, 256).to(torch.bfloat16)

        def run(module):
            y, _ = oracle.linear_forward(
                x, module.packed_weight_indices.detach(), module.row_norms.detach(),
                None if module.bias is None else module.bias.detach(),
                perm=module.rotation.permutation, signs=module.rotation.signs,
                block=module.rotation.block_size,
                act_boundaries=module.activation_codebook.boundaries,
                act_centroids=module.activation_codebook.centroids,
                w_centroids=module.weight_codebook.centroids, w_bits=4,
                out_features=module.out_features)
            return y

        mine = run(shard_linear(full, rank, world))
        gathered = gather_columns(mine, full.out_features)
        expect = run(full)
        ok = torch.equal(gathered.view(torch.int16), expect.view(torch.int16))
        # equal-width path as well
        even = gather_columns(torch.full((3, 8), float(rank)), 8 * world)
        ok = ok and torch.equal(even[:, 8 * rank:8 * rank + 8], torch.full((3, 8), float(rank)))
        flags = [None] * world
        dist.all_gather_object(flags, bool(ok))
        if rank == 0:
            Path(out_path).write_text("ok" if all(flags) else "mismatch")
    finally:
        dist.destroy_process_group()


def test_two_rank_column_shards_gather_to_the_full_result(tmp_path):
    out = tmp_path / "result.txt"
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, str(out)), nprocs=2, join=True)
    assert out.read_text() == "ok"
