"""Forward of a column shard with the all-gather folded into the GEMM epilogue: the result
tile is stored into several full-width buffers (own + peers).  One-GPU part: several
destinations on the same device.  Two-GPU part (skipped on a single GPU): two ranks over
symmetric memory, compared bit for bit with the NCCL all-gather of the same shards."""
from __future__ import annotations

import os
import socket

import pytest
import torch

from orbitquant_b200 import OrbitQuantConfig, OrbitQuantLinear, native
from orbitquant_b200.sharding import shard_linear
from test_gpu_parity import _dev

pytestmark = pytest.mark.gpu


def _module(k, n, seed=0):
    torch.manual_seed(seed)
    lin = torch.nn.Linear(k, n, bias=True)
    cfg = OrbitQuantConfig(weight_bits=4, activation_bits=4, rotation_seed=seed)
    return OrbitQuantLinear.from_linear(lin, config=cfg, module_name=f"scatter.{k}.{n}")


def test_scatter_into_several_buffers_on_one_device():
    dev = _dev()
    native.gemm_clear_device_status()
    k, n, rows, ld, col = 512, 264, 300, 1024, 408
    q = _module(k, n).to(dev)
    x = (torch.randn(rows, k) * 0.7).to(torch.bfloat16).to(dev)
    expect = q(x)
    bufs = [torch.full((rows, ld), -7.0, dtype=torch.bfloat16, device=dev) for _ in range(3)]
    q.forward_scatter(x, [b.data_ptr() for b in bufs], ld, col)
    torch.cuda.synchronize()
    assert native.gemm_device_status() == 0
    for b in bufs:
        assert torch.equal(b[:, col:col + n], expect)
        assert torch.all(b[:, :col] == -7.0) and torch.all(b[:, col + n:] == -7.0)


def test_scatter_argument_errors():
    dev = _dev()
    q = _module(256, 64).to(dev)
    x = torch.zeros(300, 256, dtype=torch.bfloat16, device=dev)
    out = torch.zeros(300, 64, dtype=torch.bfloat16, device=dev)
    with pytest.raises(ValueError):       # column range outside the leading dimension
        q.forward_scatter(x, [out.data_ptr()], 64, 8)
    with pytest.raises(ValueError):       # nine destinations
        q.forward_scatter(x, [out.data_ptr()] * 9, 64, 0)
    few = torch.zeros(16, 256, dtype=torch.bfloat16, device=dev)
    with pytest.raises(RuntimeError):     # the few-token kernel has no multi-destination epilogue
        q.forward_scatter(few, [out.data_ptr()], 64, 0)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _two_rank_worker(rank, world, port, result):
    import torch.distributed as dist
    from orbitquant_b200.sharding import PeerOutput, gather_columns

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        k, n, rows = 1024, 1536, 520
        full = _module(k, n, seed=5)
        shard = shard_linear(full, rank, world).to(dev)
        x = (torch.randn(rows, k, generator=torch.Generator().manual_seed(9)) * 0.8).to(torch.bfloat16).to(dev)
        gathered = gather_columns(shard(x), n)
        peer = PeerOutput(rows, n, dev)
        peer.tensor.fill_(-3.0)
        peer.wait()
        peer.scatter(shard, x)
        peer.wait()
        torch.cuda.synchronize()
        fused_ok = bool(torch.equal(peer.tensor, gathered))
        # the same gather by the copy engines
        peer.tensor.fill_(-3.0)
        peer.wait()
        peer.scatter_dma(shard, x, torch.cuda.Stream())
        peer.wait()
        torch.cuda.synchronize()
        dma_ok = bool(torch.equal(peer.tensor, gathered))
        # Reuse: three rounds back to back into one PeerOutput while rank 1 reads slowly.  A
        # round's result must still be intact when its (delayed) reader runs, although the
        # fast rank has by then started storing the next round.
        reuse_ok = True
        xs = [(torch.randn(rows, k, generator=torch.Generator().manual_seed(20 + i)) * 0.8)
              .to(torch.bfloat16).to(dev) for i in range(3)]
        expected = [gather_columns(shard(xi), n) for xi in xs]
        kept = []
        for i, xi in enumerate(xs):
            peer.scatter(shard, xi)
            peer.wait()
            if rank == 1:
                torch.cuda._sleep(200_000_000)   # ~0.1 s: the reader lags behind its peer
            kept.append(peer.tensor.clone())
        torch.cuda.synchronize()
        for got, want in zip(kept, expected):
            reuse_ok = reuse_ok and bool(torch.equal(got, want))
        result[rank] = fused_ok and dma_ok and reuse_ok and native.gemm_device_status() == 0
    finally:
        dist.destroy_process_group()


def test_scatter_two_ranks_matches_all_gather():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    manager = mp.Manager()
    result = manager.dict()
    mp.spawn(_two_rank_worker, args=(2, _free_port(), result), nprocs=2, join=True)
    assert result.get(0) is True and result.get(1) is True
