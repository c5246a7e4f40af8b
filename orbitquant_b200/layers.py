"""``OrbitQuantLinear`` and the ``orbitquant::packed_linear_forward`` custom op.

Drop-in for the reference module (``src/orbitquant/layers.py:302-1455``) on B200:

* same constructor keywords and classmethods (``from_linear``, ``from_weight``,
  ``empty_from_linear``);
* same parameters and **state-dict keys** ``{packed_weight_indices, row_norms, bias}``:
  flat ``uint8`` little-endian bit stream of ``ceil(N*K*bits/8)`` bytes, ``bfloat16`` row
  norms (``layers.py:159-222``), so a reference ``model.safetensors`` loads unchanged;
* same non-persistent constant buffers (``_rotation_permutation`` int32,
  ``_rotation_signs`` int8, codebook tables fp32), rebuilt after ``.to()`` /
  meta-initialisation (``layers.py:557-561, 625-649``);
* same custom op name, schema and fake implementation (``layers.py:59-72``), so the module
  traces as one opaque node under ``torch.compile(fullgraph=True)``; the integer handle
  is resolved through a weakref-cleaned registry and a stale handle raises
  ``RuntimeError`` (``layers.py:38-56``).

What differs is below the op: the reference's Python dispatch tree over Triton / native /
dequantised paths collapses into ONE call into ``liborbit_b200.so``
(``oq_linear_forward``), which picks the streaming small-rows kernel, the tcgen05 kernel
or the general tiled kernel by shape.  There is no CPU path: CPU inputs raise.
"""
from __future__ import annotations

import weakref
from math import gcd

import torch
from torch import nn

from . import native
from .codebooks import get_codebook
from .config import OrbitQuantConfig
from .packing import pack_lowbit, packed_length
from .rotations import RPBHRotation, get_rpbh_rotation

_COMPILE_REGISTRY: dict[int, "weakref.ref"] = {}


def _registry_lookup(handle: int):
    ref = _COMPILE_REGISTRY.get(handle)
    module = None if ref is None else ref()
    if module is None:
        raise RuntimeError(
            "orbitquant compiled-forward handle is stale; rebuild the module before calling "
            "the compiled graph")
    return module


def _registry_register(module) -> int:
    handle = id(module)
    if handle not in _COMPILE_REGISTRY:
        # A weak reference: the registry must not keep a replaced module (and its packed
        # weights) alive; the finalizer drops the entry when the module dies.
        _COMPILE_REGISTRY[handle] = weakref.ref(module)
        weakref.finalize(module, _COMPILE_REGISTRY.pop, handle, None)
    return handle


@torch.library.custom_op("orbitquant::packed_linear_forward", mutates_args=())
def _packed_linear_forward_op(
    x: torch.Tensor, handle: int, out_features: int, bf16_output: bool
) -> torch.Tensor:
    return _registry_lookup(handle)._forward_impl(x)


@_packed_linear_forward_op.register_fake
def _packed_linear_forward_fake(
    x: torch.Tensor, handle: int, out_features: int, bf16_output: bool
) -> torch.Tensor:
    dtype = torch.bfloat16 if bf16_output else x.dtype
    return x.new_empty((*x.shape[:-1], out_features), dtype=dtype)


def iter_aligned_row_tiles(row_count: int, values_per_row: int, bits: int, max_rows: int):
    """Row tiles whose packed payloads (except the last) end on a byte boundary
    (``src/orbitquant/streaming.py:8-28``), so tiles can be packed independently and
    concatenated."""
    if row_count < 0 or values_per_row <= 0 or not 0 < bits <= 8 or max_rows <= 0:
        raise ValueError("invalid row tiling arguments")
    align = 8 // gcd(8, values_per_row * bits)
    step = max(align, max_rows - max_rows % align)
    for start in range(0, row_count, step):
        yield start, min(start + step, row_count)


def quantize_weight(weight: torch.Tensor, *, rotation: RPBHRotation, codebook, bits: int,
                    eps: float, row_tile_size: int = 256) -> tuple[torch.Tensor, torch.Tensor]:
    """Offline weight quantisation: ``W [N,K]`` -> (packed uint8 stream, bf16 row norms).

    Per row: fp32 L2 norm of the un-rotated row, rotate by R, divide by
    ``max(norm, eps)``, bucketize against the codebook, bit-pack.  Runs on the CPU with
    the same torch ops, in the same order, as the reference
    (``layers.py:102-222``), which makes indices and norms bit-identical to it; results
    are returned on ``weight.device``."""
    if weight.ndim != 2:
        raise ValueError("weight must be a matrix")
    n, k = weight.shape
    device = weight.device
    packed = torch.empty(packed_length(n * k, bits), dtype=torch.uint8)
    norms_out = torch.empty(n, dtype=torch.bfloat16)
    offset = 0
    for lo, hi in iter_aligned_row_tiles(n, k, bits, row_tile_size):
        tile = weight[lo:hi].detach().to(device="cpu", dtype=torch.float32)
        norms = tile.norm(dim=-1)
        unit = rotation.apply_to_weight(tile) / norms.clamp_min(eps)[:, None]
        chunk = pack_lowbit(codebook.quantize_indices(unit), bits, validate=False)
        packed[offset:offset + chunk.numel()] = chunk
        norms_out[lo:hi] = norms.to(torch.bfloat16)
        offset += chunk.numel()
    if offset != packed.numel():
        raise RuntimeError(f"row-tiled packing wrote {offset} bytes, expected {packed.numel()}")
    return packed.to(device), norms_out.to(device)


def quantize_weight_gpu(weight: torch.Tensor, *, rotation: RPBHRotation, codebook, bits: int,
                        eps: float, row_norms: torch.Tensor | None = None
                        ) -> tuple[torch.Tensor, torch.Tensor]:
    """``quantize_weight`` on the GPU (``oq_quantize_weight``): same arithmetic per element
    (rotate, ``* 1/sqrt(block)``, divide by ``max(norm, eps)``, bucketize, pack).  Given the
    same fp32 ``row_norms`` the packed stream is bit-identical to the CPU path; without them
    the norms are computed on the device with double accumulation, which can differ from
    torch's CPU reduction in the last bit of a norm (and then flip an index that sits within
    one ulp of a boundary)."""
    return native.quantize_weight_packed(
        weight, permutation=rotation.permutation, signs=rotation.signs,
        block_size=rotation.block_size, boundaries=codebook.boundaries, centroids=codebook.centroids,
        bits=bits, eps=eps, row_norms=row_norms)


def _linear_spec(layer: nn.Module) -> tuple[int, int]:
    weight = getattr(layer, "weight", None)
    if not isinstance(layer, nn.Linear) or not isinstance(weight, torch.Tensor) or weight.ndim != 2:
        raise TypeError(f"no OrbitQuant linear adapter registered for {type(layer).__name__}")
    return int(layer.in_features), int(layer.out_features)


def _first_device(*tensors):
    for t in tensors:
        if t is not None and t.device.type != "meta":
            return t.device
    return None


class OrbitQuantLinear(nn.Module):
    """Linear layer with OrbitQuant-packed rotated weights, computed by the sm_100a kernels."""

    def __init__(self, *, in_features: int, out_features: int, config: OrbitQuantConfig,
                 module_name: str, source_weight_layout: str, bias: torch.Tensor | None,
                 packed_weight_indices: torch.Tensor | None, row_norms: torch.Tensor | None,
                 debug_weight: torch.Tensor | None = None) -> None:
        super().__init__()
        if debug_weight is not None or config.runtime_mode in {"debug_no_quant",
                                                               "debug_no_activation_quant"}:
            raise ValueError("the debug runtime modes keep an unquantised weight and are not "
                             "part of the B200 quantized-linear path")
        self.in_features = in_features
        self.out_features = out_features
        self.weight_bits = config.weight_bits
        self.activation_bits = config.activation_bits
        self.runtime_mode = config.runtime_mode
        self.activation_kernel_backend = config.activation_kernel_backend
        self.packed_matmul_block_m = config.packed_matmul_block_m
        self.packed_matmul_block_n = config.packed_matmul_block_n
        self.packed_matmul_block_k = config.packed_matmul_block_k
        self.packed_matmul_num_warps = config.packed_matmul_num_warps
        self.module_name = module_name
        self.source_weight_layout = source_weight_layout
        self.activation_eps = config.activation_eps
        self.rotation = get_rpbh_rotation(dim=in_features, seed=config.rotation_seed,
                                          block_size=config.block_size)
        self.weight_codebook = get_codebook(in_features, config.weight_bits, config.codebook_version)
        self.activation_codebook = get_codebook(in_features, config.activation_bits,
                                                config.codebook_version)
        device = _first_device(packed_weight_indices, row_norms, bias)
        for name, source, dtype in self._constant_sources():
            value = source.detach().clone().to(dtype)
            self.register_buffer(name, value if device is None else value.to(device),
                                 persistent=False)
        if bias is None:
            self.register_parameter("bias", None)
        else:
            self.bias = nn.Parameter(bias.detach().clone(), requires_grad=False)
        self.packed_weight_indices = (None if packed_weight_indices is None else
                                      nn.Parameter(packed_weight_indices, requires_grad=False))
        self.row_norms = None if row_norms is None else nn.Parameter(row_norms, requires_grad=False)
        self.debug_weight = None
        # Kernel selection knobs of this implementation (names from include/orbit_b200.h).
        self.weight_mode = "auto"
        self.kernel = "auto"
        self._bias_cache: tuple[tuple[str, torch.dtype], torch.Tensor] | None = None
        self._norms_cache: tuple[str, torch.Tensor] | None = None
        self._compile_handle = _registry_register(self)
        self.last_effective_runtime_mode: str | None = None
        self.last_activation_kernel_backend: str | None = None
        self.last_forward_device_type: str | None = None
        self._derived_constants_valid = True

    def _constant_sources(self):
        return (
            ("_rotation_permutation", self.rotation.permutation, torch.int32),
            ("_rotation_signs", self.rotation.signs, torch.int8),
            ("_activation_codebook_centroids", self.activation_codebook.centroids, torch.float32),
            ("_activation_codebook_boundaries", self.activation_codebook.boundaries, torch.float32),
            ("_weight_codebook_centroids", self.weight_codebook.centroids, torch.float32),
        )

    # ---- construction -------------------------------------------------------------------

    @classmethod
    def from_linear(cls, layer: nn.Module, *, config: OrbitQuantConfig, module_name: str,
                    quantization_device: torch.device | None = None) -> "OrbitQuantLinear":
        in_features, out_features = _linear_spec(layer)
        bias = None if layer.bias is None else layer.bias.detach()
        return cls.from_weight(layer.weight.detach(), bias=bias, in_features=in_features,
                               out_features=out_features, source_weight_layout="out_in",
                               config=config, module_name=module_name,
                               quantization_device=quantization_device)

    @classmethod
    def from_weight(cls, weight: torch.Tensor, *, bias: torch.Tensor | None, in_features: int,
                    out_features: int, source_weight_layout: str, config: OrbitQuantConfig,
                    module_name: str, quantization_device: torch.device | None = None
                    ) -> "OrbitQuantLinear":
        if tuple(weight.shape) != (out_features, in_features):
            raise ValueError(f"expected canonical weight shape {(out_features, in_features)}, "
                             f"got {tuple(weight.shape)}")
        rotation = get_rpbh_rotation(dim=in_features, seed=config.rotation_seed,
                                     block_size=config.block_size)
        codebook = get_codebook(in_features, config.weight_bits, config.codebook_version)
        on_gpu = (quantization_device is not None and torch.device(quantization_device).type == "cuda")
        if on_gpu:
            # the library's quantise-and-pack kernels (norm, RPBH, bucketize, bit stream)
            packed, row_norms = quantize_weight_gpu(
                weight.detach().to(quantization_device), rotation=rotation, codebook=codebook,
                bits=config.weight_bits, eps=config.activation_eps)
            packed, row_norms = packed.to(weight.device), row_norms.to(weight.device)
        else:
            packed, row_norms = quantize_weight(
                weight, rotation=rotation, codebook=codebook, bits=config.weight_bits,
                eps=config.activation_eps, row_tile_size=config.weight_row_tile_size)
        return cls(in_features=in_features, out_features=out_features, config=config,
                   module_name=module_name, source_weight_layout=source_weight_layout, bias=bias,
                   packed_weight_indices=packed, row_norms=row_norms, debug_weight=None)

    @classmethod
    def empty_from_linear(cls, layer: nn.Module, *, config: OrbitQuantConfig,
                          module_name: str) -> "OrbitQuantLinear":
        in_features, out_features = _linear_spec(layer)
        device = layer.weight.device
        bias = None
        if layer.bias is not None:
            bias = torch.zeros(out_features, dtype=layer.bias.dtype, device=layer.bias.device)
        packed = torch.empty(packed_length(out_features * in_features, config.weight_bits),
                             dtype=torch.uint8, device=device)
        row_norms = torch.empty(out_features, dtype=torch.bfloat16, device=device)
        empty = cls(in_features=in_features, out_features=out_features, config=config,
                    module_name=module_name, source_weight_layout="out_in", bias=bias,
                    packed_weight_indices=packed, row_norms=row_norms, debug_weight=None)
        # Loaders may replace non-persistent buffers while materialising a meta skeleton;
        # rebuild the deterministic constants on the first real forward.
        empty._derived_constants_valid = False
        return empty

    # ---- cached device constants ----------------------------------------------------------

    def _apply(self, fn, recurse: bool = True):
        result = super()._apply(fn, recurse=recurse)
        self._derived_constants_valid = False
        self._bias_cache = None
        self._norms_cache = None
        self._int8_surrogate_cache = None
        self._pair_lut_cache = None
        return result

    def _ensure_derived_constants(self, device: torch.device) -> None:
        if self._derived_constants_valid and self._rotation_permutation.device == device:
            return
        for name, source, dtype in self._constant_sources():
            setattr(self, name, source.to(device=device, dtype=dtype).clone())
        self._derived_constants_valid = True

    def _bias_for(self, device: torch.device) -> torch.Tensor | None:
        """The bias in its own floating dtype: the kernels add it in fp32 before the final
        cast (as the reference's CPU kernels do with their fp32 bias), so nothing is gained
        by rounding it to the activation dtype first."""
        if self.bias is None:
            return None
        dtype = self.bias.dtype if self.bias.dtype in native.DTYPE_CODES else torch.float32
        if self.bias.device == device and self.bias.dtype == dtype and self.bias.is_contiguous():
            return self.bias
        key = (str(device), dtype)
        if self._bias_cache is None or self._bias_cache[0] != key:
            self._bias_cache = (key, self.bias.to(device=device, dtype=dtype).contiguous())
        return self._bias_cache[1]

    def _row_norms_for(self, device: torch.device) -> torch.Tensor:
        norms = self.row_norms
        if norms.device == device and norms.dtype == torch.bfloat16 and norms.is_contiguous():
            return norms
        key = str(device)
        if self._norms_cache is None or self._norms_cache[0] != key:
            self._norms_cache = (key, norms.to(device=device, dtype=torch.bfloat16).contiguous())
        return self._norms_cache[1]

    # ---- forward ------------------------------------------------------------------------

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if torch.compiler.is_compiling():
            return torch.ops.orbitquant.packed_linear_forward(
                x, self._compile_handle, self.out_features, False)
        return self._forward_impl(x)

    def _forward_impl(self, x: torch.Tensor) -> torch.Tensor:
        if x.device.type != "cuda":
            raise RuntimeError(
                "OrbitQuantLinear (orbitquant_b200) requires CUDA input tensors on an sm_100 "
                f"device; got {x.device.type}. There is no CPU path in this package.")
        if x.shape[-1] != self.in_features:
            raise ValueError(f"expected last dimension {self.in_features}, got {x.shape[-1]}")
        if self.packed_weight_indices is None or self.row_norms is None:
            raise RuntimeError("OrbitQuantLinear is missing quantized weight buffers")
        device = x.device
        self._ensure_derived_constants(device)
        packed = self.packed_weight_indices
        if packed.device != device or packed.dtype != torch.uint8 or not packed.is_contiguous():
            raise RuntimeError("packed_weight_indices must be a contiguous uint8 tensor on the "
                               "input's device; move the module with .to(device)")
        self.last_effective_runtime_mode = "native_packed_matmul"
        self.last_activation_kernel_backend = "orbit_b200"
        self.last_forward_device_type = "cuda"
        if self.weight_mode == "int8_surrogate":
            return self._forward_int8_surrogate(x)
        if self.weight_mode == "pair_lut":
            return self._forward_pair_lut(x)
        return native.linear_forward(
            x, packed, self._row_norms_for(device), self._bias_for(device),
            permutation=self._rotation_permutation, signs=self._rotation_signs,
            block_size=self.rotation.block_size,
            act_boundaries=self._activation_codebook_boundaries,
            act_centroids=self._activation_codebook_centroids,
            weight_centroids=self._weight_codebook_centroids,
            weight_bits=self.weight_bits, out_features=self.out_features,
            eps=self.activation_eps,
            weight_mode=native.WEIGHT_MODE_NAMES[self.weight_mode],
            kernel=native.KERNEL_NAMES[self.kernel])

    def _int8_surrogate_constants(self, device: torch.device):
        """INT8 code tables and scales of both codebooks (reference ``layers.py:811-835``)."""
        cache = getattr(self, "_int8_surrogate_cache", None)
        if cache is None or cache[0] != str(device):
            from .int8_surrogate import fit_int8_centroid_surrogate
            a_codes, a_scale = fit_int8_centroid_surrogate(self.activation_codebook.centroids)
            w_codes, w_scale = fit_int8_centroid_surrogate(self.weight_codebook.centroids)
            cache = (str(device), a_codes.to(device), a_scale, w_codes.to(device), w_scale)
            self._int8_surrogate_cache = cache
        return cache[1:]

    def _forward_int8_surrogate(self, x: torch.Tensor) -> torch.Tensor:
        """The reference's integer path for W4A4 / W2A4 (``layers.py:1097-1352``): packed 4-bit
        activation codes, INT8 code tables, integer contraction, rescale.  Approximate (the
        codes are rounded centroids); selected with ``module.weight_mode = "int8_surrogate"``."""
        if self.activation_bits != 4 or self.weight_bits not in (2, 3, 4, 6):
            raise ValueError("the INT8 surrogate path takes 4-bit activations and 2/3/4/6-bit weights")
        device = x.device
        a_codes, a_scale, w_codes, w_scale = self._int8_surrogate_constants(device)
        if native.linear_w4a4_int8_supported(x, self.in_features, self.out_features,
                                             self.rotation.block_size, self.weight_bits):
            self.last_activation_kernel_backend = "orbit_b200_int8_surrogate_fused"
            y = native.linear_w4a4_int8(
                x, self.packed_weight_indices, self._row_norms_for(device), self._bias_for(device),
                permutation=self._rotation_permutation, signs=self._rotation_signs,
                block_size=self.rotation.block_size,
                act_boundaries=self._activation_codebook_boundaries,
                act_centroids=self._activation_codebook_centroids, act_codes=a_codes,
                weight_codes=w_codes, act_scale=a_scale, weight_scale=w_scale,
                out_features=self.out_features, eps=self.activation_eps)
            return y if y.dtype == x.dtype else y.to(x.dtype)
        packed_x, token_norms = native.quantize_activations_packed_w4(
            x, self._rotation_permutation, self._rotation_signs, self._activation_codebook_centroids,
            self._activation_codebook_boundaries, eps=self.activation_eps,
            block_size=self.rotation.block_size)
        self.last_activation_kernel_backend = "orbit_b200_int8_surrogate"
        y = native.matmul_packed_w4a4_int8(
            packed_x, self.packed_weight_indices, token_norms, self._row_norms_for(device), a_codes,
            w_codes, act_scale=a_scale, weight_scale=w_scale, out_features=self.out_features,
            in_features=self.in_features, weight_bits=self.weight_bits, bias=self._bias_for(device))
        return y if y.dtype == x.dtype else y.to(x.dtype)

    def _forward_pair_lut(self, x: torch.Tensor) -> torch.Tensor:
        """Exact W4A4 through the 256-entry pair-product table
        (``src/orbitquant/kernels/executorch_vulkan.py:15-61``); ``weight_mode = "pair_lut"``."""
        if self.activation_bits != 4 or self.weight_bits != 4:
            raise ValueError("the pair-product table exists for W4A4 only")
        device = x.device
        lut = getattr(self, "_pair_lut_cache", None)
        if lut is None or lut.device != device:
            lut = (self.activation_codebook.centroids.float()[:, None]
                   * self.weight_codebook.centroids.float()[None, :]).flatten().contiguous().to(device)
            self._pair_lut_cache = lut
        return native.linear_w4a4_pair_lut(
            x, self.packed_weight_indices, self._row_norms_for(device), self._bias_for(device),
            permutation=self._rotation_permutation, signs=self._rotation_signs,
            block_size=self.rotation.block_size,
            act_boundaries=self._activation_codebook_boundaries,
            act_centroids=self._activation_codebook_centroids, pair_lut=lut,
            out_features=self.out_features, eps=self.activation_eps)

    def forward_scatter(self, x: torch.Tensor, out_ptrs, out_ld: int, out_col: int) -> None:
        """Forward of a column shard whose result goes straight into every buffer of
        ``out_ptrs`` (device addresses of row-major bf16 ``[rows, out_ld]`` buffers, this
        rank's and its peers') at columns ``out_col .. out_col + out_features``.  See
        ``orbitquant_b200.sharding.PeerOutput``."""
        if x.device.type != "cuda":
            raise RuntimeError("OrbitQuantLinear (orbitquant_b200) requires CUDA input tensors")
        if x.shape[-1] != self.in_features:
            raise ValueError(f"expected last dimension {self.in_features}, got {x.shape[-1]}")
        device = x.device
        self._ensure_derived_constants(device)
        packed = self.packed_weight_indices
        if packed.device != device or packed.dtype != torch.uint8 or not packed.is_contiguous():
            raise RuntimeError("move the module to the input's device first")
        native.linear_forward_scatter(
            x, packed, self._row_norms_for(device), self._bias_for(device),
            out_ptrs=out_ptrs, out_ld=out_ld, out_col=out_col,
            permutation=self._rotation_permutation, signs=self._rotation_signs,
            block_size=self.rotation.block_size,
            act_boundaries=self._activation_codebook_boundaries,
            act_centroids=self._activation_codebook_centroids,
            weight_centroids=self._weight_codebook_centroids,
            weight_bits=self.weight_bits, out_features=self.out_features,
            eps=self.activation_eps)

    def dequantize_weight(self, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        """Dense ``row_norm[n] * centroid[idx[n,k]]`` in the ROTATED basis
        (``layers.py:1060-1070``)."""
        return native.dequantize_packed_weight(
            self.packed_weight_indices, self.row_norms, self.weight_codebook.centroids,
            bits=self.weight_bits, out_features=self.out_features, in_features=self.in_features,
            dtype=dtype)

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, "
                f"W{self.weight_bits}A{self.activation_bits}, block={self.rotation.block_size}")
