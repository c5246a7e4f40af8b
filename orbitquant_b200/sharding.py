"""Output-feature (N) sharding of an ``OrbitQuantLinear`` across the GPUs of one box.

Every output column of ``y = x_q W^T + b`` depends on one packed weight row, one row norm,
one bias element and the WHOLE quantised activation row; the token norm and the global
RPBH permutation span all of K.  So the path shards along N and only along N: rank r keeps
a contiguous run of rows of the row-major bit stream (a contiguous byte range because
``K*bits`` is a multiple of 8), the matching ``row_norms`` / ``bias`` slices, and replicates
the (cheap) rotate-and-quantize prologue.  No collective is needed to compute a shard; an
all-gather of the ``[M, N/R]`` slices runs only when the consumer needs full rows
(``gather_columns``).  The reference has no multi-GPU code; this module has no counterpart
there.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .config import OrbitQuantConfig
from .layers import OrbitQuantLinear

# Shard boundaries fall on multiples of this many rows, so every shard's byte offset is
# 16-byte aligned for any K*bits that is a multiple of 16 (TMA and vector loads need it).
ROW_ALIGN = 8


def shard_bounds(out_features: int, world_size: int, rank: int, align: int = ROW_ALIGN):
    """Contiguous ``[lo, hi)`` rows of rank ``rank``; sizes differ by at most ``align``."""
    if world_size <= 0 or not 0 <= rank < world_size:
        raise ValueError("rank must be in [0, world_size)")
    units = (out_features + align - 1) // align
    base, extra = divmod(units, world_size)
    lo_units = rank * base + min(rank, extra)
    hi_units = lo_units + base + (1 if rank < extra else 0)
    return min(lo_units * align, out_features), min(hi_units * align, out_features)


def shard_byte_range(lo: int, hi: int, in_features: int, bits: int):
    if (in_features * bits) % 8 != 0:
        raise ValueError("rows must end on byte boundaries to shard the packed stream "
                         "(in_features * bits must be a multiple of 8)")
    row_bytes = in_features * bits // 8
    return lo * row_bytes, hi * row_bytes


def shard_linear(module: OrbitQuantLinear, rank: int, world_size: int,
                 config: OrbitQuantConfig | None = None) -> OrbitQuantLinear:
    """The rank's column shard as a stand-alone ``OrbitQuantLinear`` (views, no copies)."""
    lo, hi = shard_bounds(module.out_features, world_size, rank)
    b0, b1 = shard_byte_range(lo, hi, module.in_features, module.weight_bits)
    if config is None:
        config = OrbitQuantConfig(
            weight_bits=module.weight_bits, activation_bits=module.activation_bits,
            rotation_seed=module.rotation.seed, block_size=module.rotation.block_size,
            activation_eps=module.activation_eps,
            codebook_version=module.weight_codebook.algorithm_version)
    shard = OrbitQuantLinear(
        in_features=module.in_features, out_features=hi - lo, config=config,
        module_name=f"{module.module_name}[{lo}:{hi}]",
        source_weight_layout=module.source_weight_layout,
        bias=None if module.bias is None else module.bias.detach()[lo:hi],
        packed_weight_indices=module.packed_weight_indices.detach()[b0:b1],
        row_norms=module.row_norms.detach()[lo:hi], debug_weight=None)
    shard.weight_mode = module.weight_mode
    shard.kernel = module.kernel
    shard.shard_rows = (lo, hi)
    return shard


def gather_columns(y_local: torch.Tensor, out_features: int, group=None) -> torch.Tensor:
    """All-gather ``[..., n_r]`` column slices (rank order) into ``[..., out_features]``.

    Shards may be ragged (``shard_bounds``); slices are padded to the widest shard for the
    collective and trimmed afterwards.  One ``all_gather`` over NCCL (NVLink/NVSwitch) on
    GPUs, gloo on CPU."""
    world = dist.get_world_size(group)
    if world == 1:
        return y_local
    widths = [hi - lo for lo, hi in (shard_bounds(out_features, world, r) for r in range(world))]
    widest = max(widths)
    lead = y_local.shape[:-1]
    flat = y_local.reshape(-1, y_local.shape[-1])
    if flat.shape[-1] != widest:
        flat = torch.nn.functional.pad(flat, (0, widest - flat.shape[-1]))
    flat = flat.contiguous()
    # The collective concatenates along dim 0 (gloo accepts only that shape).
    stacked = torch.empty((world * flat.shape[0], widest), dtype=flat.dtype, device=flat.device)
    dist.all_gather_into_tensor(stacked, flat, group=group)
    gathered = stacked.view(world, flat.shape[0], widest)
    if all(w == widest for w in widths):
        full = gathered.permute(1, 0, 2).reshape(flat.shape[0], world * widest)
    else:
        full = torch.cat([gathered[r, :, :widths[r]] for r in range(world)], dim=-1)
    return full.reshape(*lead, out_features)


class PeerOutput:
    """Full-width ``[rows, out_features]`` bf16 output of a column-sharded layer, allocated in
    symmetric memory so that every rank holds the peer-mapped address of every other rank's
    copy.  ``scatter(module, x)`` runs the rank's shard with the all-gather folded into the
    GEMM epilogue (each finished tile is stored into all ranks' copies over NVLink);
    ``wait()`` is the inter-rank barrier after which ``tensor`` holds every shard.

    Reuse rule.  The object owns TWO buffers and alternates between them: round ``i`` (one
    ``scatter`` + ``wait``) fills buffer ``i % 2``, and ``tensor`` is the buffer of the last
    completed round.  A peer may start round ``i + 2`` -- which overwrites the buffer of
    round ``i`` on THIS rank -- only after it has passed the barrier of round ``i + 1``,
    i.e. after this rank's stream has reached its own ``wait()`` of round ``i + 1``.  So the
    result of a round stays valid, on every rank, until that rank calls ``wait()`` for the
    next round, provided its reads were enqueued on the same stream before that call (a
    consumer on another stream must be joined first).  With a single buffer a fast rank's
    next epilogue could overwrite a slow peer's copy while that peer still reads it.

    Plain peer stores only: no multicast object is created, so a rank that dies does not
    take the others' NVLink down with it."""

    def __init__(self, rows: int, out_features: int, device, group=None):
        import os

        # peer loads/stores only; no NVLink multicast object is bound to the buffer
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.out_features = out_features
        self.buffers = symm_mem.empty((2, rows, out_features), dtype=torch.bfloat16, device=device)
        self.handle = symm_mem.rendezvous(self.buffers, self.group)
        # own copy first (the next layer reads it soonest), then the peers starting from the
        # next rank, so that at any moment the ranks store into different destinations
        order = [(self.rank + i) % self.world for i in range(self.world)]
        half = rows * out_features * 2
        self.ptrs = [[int(self.handle.buffer_ptrs[r]) + b * half for r in order] for b in range(2)]
        self.lo, self.hi = shard_bounds(out_features, self.world, self.rank)
        self.round = 0          # rounds started
        self.tensor = self.buffers[0]

    def scatter(self, module, x: torch.Tensor) -> None:
        if module.out_features != self.hi - self.lo:
            raise ValueError("module is not this rank's column shard of the output")
        slot = self.round % 2
        self.round += 1
        self._filling = slot
        module.forward_scatter(x, self.ptrs[slot], self.out_features, self.lo)

    def scatter_dma(self, module, x: torch.Tensor, copy_stream: "torch.cuda.Stream") -> None:
        """The rank's shard computed by the ordinary forward, then copied into every rank's
        buffer by the copy engines (one strided ``cudaMemcpy2DAsync`` per destination on
        ``copy_stream``): the transfers use no SM and run under whatever the compute stream does
        next.  ``wait()`` joins them."""
        from cuda.bindings import runtime as cudart

        if module.out_features != self.hi - self.lo:
            raise ValueError("module is not this rank's column shard of the output")
        y = module(x).reshape(-1, module.out_features)
        slot = self.round % 2
        self.round += 1
        self._filling = slot
        ready = torch.cuda.Event()
        ready.record()
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(ready)
            width = y.shape[1] * 2
            for ptr in self.ptrs[slot]:
                (err,) = cudart.cudaMemcpy2DAsync(
                    ptr + self.lo * 2, self.out_features * 2, y.data_ptr(), width, width, y.shape[0],
                    cudart.cudaMemcpyKind.cudaMemcpyDeviceToDevice, copy_stream.cuda_stream)
                if err != cudart.cudaError_t.cudaSuccess:
                    raise RuntimeError(f"cudaMemcpy2DAsync failed: {err}")
            self._copied = torch.cuda.Event()
            self._copied.record(copy_stream)
        y.record_stream(copy_stream)

    def wait(self) -> None:
        """Every rank's stores into this rank's copy have landed (and this rank's into theirs)."""
        copied = getattr(self, "_copied", None)
        if copied is not None:
            torch.cuda.current_stream().wait_event(copied)
            self._copied = None
        self.handle.barrier()
        filling = getattr(self, "_filling", None)
        if filling is not None:
            self.tensor = self.buffers[filling]
            self._filling = None
