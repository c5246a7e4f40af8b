"""ctypes binding of ``liborbit_b200.so`` -- the only way this package computes.

The functions here mirror the reference's thin wrappers around its native kernel package
(``src/orbitquant/kernels/native_packed_matmul.py:99-330`` and
``native-kernels/orbitquant-packed-matmul/torch-ext/orbitquant_packed_matmul/__init__.py``):
they make inputs contiguous, allocate outputs with torch, and call one C entry point on
the current CUDA stream.  There is no fallback: a missing library, a CPU tensor or a
non-sm_100 device raises.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

import torch

_LIB_PATH = Path(__file__).resolve().parent / "liborbit_b200.so"
_lib = None

DTYPE_CODES = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}
WEIGHT_AUTO, WEIGHT_CENTROID, WEIGHT_BF16_SCALED = 0, 1, 2
KERNEL_AUTO, KERNEL_SMALL_ROWS, KERNEL_TILED, KERNEL_TCGEN05 = 0, 1, 2, 3
KERNEL_NAMES = {"auto": 0, "small_rows": 1, "tiled": 2, "tcgen05": 3}
WEIGHT_MODE_NAMES = {"auto": 0, "centroid": 1, "bf16_scaled": 2}

_i64, _int, _vp, _f32, _sz = (ctypes.c_int64, ctypes.c_int, ctypes.c_void_p, ctypes.c_float,
                              ctypes.c_size_t)

_SIGNATURES = {
    "oq_abi_version": (ctypes.c_int, []),
    "oq_last_error": (ctypes.c_char_p, []),
    "oq_launch_count": (ctypes.c_uint64, []),
    "oq_set_tunable": (_int, [ctypes.c_char_p, _int]),
    "oq_unpack_lowbit": (_int, [_vp, _int, _i64, _vp, _vp]),
    "oq_pack_lowbit": (_int, [_vp, _int, _i64, _vp, _vp]),
    "oq_dequantize_weight": (_int, [_vp, _int, _i64, _i64, _vp, _vp, _vp, _int, _vp]),
    "oq_quantize_activations": (_int, [_vp, _int, _i64, _i64, _vp, _vp, _i64, _vp, _vp, _int,
                                       _f32, _vp, _vp, _vp, _vp]),
    "oq_quantize_activations_packed_w4_workspace_bytes": (_sz, [_i64, _i64]),
    "oq_quantize_activations_packed_w4": (_int, [_vp, _int, _i64, _i64, _vp, _vp, _i64, _vp, _vp, _f32,
                                                 _vp, _vp, _vp, _sz, _vp]),
    "oq_quantize_activations_int8": (_int, [_vp, _int, _i64, _i64, _vp, _vp, _i64, _vp, _vp, _int, _vp,
                                            _f32, _vp, _vp, _vp]),
    "oq_matmul_packed_w4a4_int8_workspace_bytes": (_sz, [_i64, _i64]),
    "oq_linear_w4a4_int8_supported": (_int, [_int, _i64, _i64, _i64, _i64]),
    "oq_linear_w4a4_int8_workspace_bytes": (_sz, [_i64, _i64]),
    "oq_linear_w4a4_int8": (_int, [_vp, _vp, _int, _i64, _i64, _i64, _vp, _i64, _vp, _vp, _int, _vp, _vp, _i64,
                                   _vp, _vp, _vp, _vp, _f32, _f32, _f32, _vp, _sz, _vp]),
    "oq_matmul_packed_w4a4_int8": (_int, [_vp, _vp, _vp, _i64, _int, _vp, _vp, _vp, _vp, _vp, _int, _f32,
                                          _f32, _i64, _i64, _i64, _vp, _sz, _vp]),
    "oq_linear_w4a4_pair_lut_workspace_bytes": (_sz, [_i64, _i64]),
    "oq_linear_w4a4_pair_lut": (_int, [_vp, _vp, _int, _i64, _i64, _i64, _vp, _i64, _vp, _vp, _int, _vp,
                                       _vp, _i64, _vp, _vp, _vp, _f32, _vp, _sz, _vp]),
    "oq_matmul_packed_weight": (_int, [_vp, _vp, _int, _i64, _i64, _i64, _vp, _i64, _int, _vp,
                                       _vp, _vp, _int, _int, _int, _vp, _sz, _vp]),
    "oq_matmul_workspace_bytes": (_sz, [_i64, _i64, _i64, _int, _int, _int, _int]),
    "oq_gemm_tcgen05_supported": (_int, [_i64, _i64, _i64, _int, _int, _int]),
    "oq_gemm_tcgen05_f16": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _i64, _int, _vp, _vp, _vp,
                                   _int, _vp]),
    "oq_rows_to_f16_operand": (_int, [_vp, _int, _i64, _i64, _vp, _vp, _vp, _int, _vp, _vp]),
    "oq_linear_forward": (_int, [_vp, _vp, _int, _i64, _i64, _i64, _vp, _i64, _int, _vp, _vp,
                                 _vp, _int, _vp, _vp, _i64, _vp, _vp, _int, _f32, _int, _int,
                                 _vp, _sz, _vp]),
    "oq_linear_forward_static": (_int, [_vp, _vp, _int, _i64, _i64, _i64, _vp, _i64, _int, _vp, _vp,
                                        _vp, _int, _vp, _vp, _i64, _vp, _vp, _int, _f32, _int, _int,
                                        _vp]),
    "oq_linear_forward_scatter": (_int, [_vp, _int, _i64, _i64, _vp, _int, _i64, _i64, _i64, _vp, _i64,
                                         _int, _vp, _vp, _vp, _int, _vp, _vp, _i64, _vp, _vp, _int,
                                         _f32, _vp, _sz, _vp]),
    "oq_quantize_weight": (_int, [_vp, _int, _i64, _i64, _vp, _vp, _i64, _vp, _vp, _int, _f32, _vp, _vp,
                                  _vp, _vp, _sz, _vp]),
    "oq_quantize_weight_workspace_bytes": (_sz, [_i64, _i64]),
    "oq_rtn_int4_linear_forward": (_int, [_vp, _vp, _i64, _i64, _i64, _vp, _i64, _vp, _int, _vp, _int,
                                          _vp, _sz, _vp]),
    "oq_rtn_int4_workspace_bytes": (_sz, [_i64, _i64, _i64]),
    "oq_static_scratch_bytes": (_sz, []),
    "oq_linear_workspace_bytes": (_sz, [_i64, _i64, _i64, _int, _int, _int, _int]),
    "oq_linear_kernel_name": (ctypes.c_char_p, [_i64, _i64, _i64, _int, _int, _i64, _int, _int, _int]),
    "oq_gemm_device_status": (_int, [ctypes.POINTER(ctypes.c_int)]),
    "oq_gemm_clear_device_status": (_int, []),
}


def library_path() -> Path:
    return _LIB_PATH


def exported_symbols() -> tuple[str, ...]:
    return tuple(_SIGNATURES)


def load():
    """dlopen the library (no CUDA call is made) and declare the signatures."""
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise RuntimeError(
                f"{_LIB_PATH} is missing; build it with `python -m orbitquant_b200.build` "
                "(there is no CPU or Triton fallback)")
        lib = ctypes.CDLL(str(_LIB_PATH))
        for name, (restype, argtypes) in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = restype
            fn.argtypes = argtypes
        if lib.oq_abi_version() != 1:
            raise RuntimeError("liborbit_b200.so has an unexpected ABI version; rebuild it")
        _lib = lib
    return _lib


def _raise(status: int) -> None:
    message = load().oq_last_error().decode("utf-8", "replace")
    if status == -1:
        raise ValueError(message)
    raise RuntimeError(f"orbit_b200 error {status}: {message}")


def _check(status: int) -> None:
    if status != 0:
        _raise(status)


def _require_cuda(name: str, tensor: torch.Tensor) -> None:
    if tensor.device.type != "cuda":
        raise RuntimeError(
            f"{name} must be a CUDA tensor (got {tensor.device.type}); orbitquant_b200 has no "
            "CPU path")


def _ptr(tensor: torch.Tensor | None):
    return None if tensor is None else ctypes.c_void_p(tensor.data_ptr())


def _stream(device: torch.device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def launch_count() -> int:
    return int(load().oq_launch_count())


def set_tunable(name: str, value: int | None) -> None:
    """Pin (or, with ``None``, release) one of the library's tuning switches; see
    ``oq_set_tunable`` in ``include/orbit_b200.h``.  For tests and profiling."""
    _check(load().oq_set_tunable(name.encode(), -1 if value is None else int(value)))


def forward_kernel_name(rows: int, in_features: int, out_features: int, weight_bits: int,
                        act_bits: int, block_size: int, *, dtype=torch.bfloat16,
                        weight_mode=WEIGHT_AUTO, kernel=KERNEL_AUTO) -> str:
    """Which kernels ``linear_forward`` launches for this problem (``oq_linear_kernel_name``)."""
    return load().oq_linear_kernel_name(rows, in_features, out_features, weight_bits, act_bits,
                                        int(block_size), DTYPE_CODES[dtype], weight_mode, kernel).decode()


def gemm_device_status() -> int:
    value = ctypes.c_int(0)
    _check(load().oq_gemm_device_status(ctypes.byref(value)))
    return int(value.value)


def gemm_clear_device_status() -> None:
    _check(load().oq_gemm_clear_device_status())


def unpack_lowbit(packed: torch.Tensor, bits: int, length: int) -> torch.Tensor:
    if bits <= 0 or bits > 8:
        raise ValueError("bits must be in [1, 8]")
    if length < 0:
        raise ValueError("length must be non-negative")
    _require_cuda("packed", packed)
    packed = packed.to(torch.uint8).contiguous().flatten()
    if packed.numel() * 8 < length * bits:
        raise ValueError("packed tensor is too short for the requested length")
    out = torch.empty(length, dtype=torch.uint8, device=packed.device)
    with torch.cuda.device(packed.device):
        _check(load().oq_unpack_lowbit(_ptr(packed), bits, length, _ptr(out), _stream(packed.device)))
    return out


def pack_lowbit(values: torch.Tensor, bits: int, *, validate: bool = True) -> torch.Tensor:
    if bits <= 0 or bits > 8:
        raise ValueError("bits must be in [1, 8]")
    _require_cuda("values", values)
    flat = values.flatten()
    if validate and flat.numel() and (int(flat.min()) < 0 or int(flat.max()) > (1 << bits) - 1):
        raise ValueError(f"all values must fit in {bits} bits")
    flat = flat.to(torch.uint8).contiguous()
    out = torch.empty((flat.numel() * bits + 7) // 8, dtype=torch.uint8, device=flat.device)
    with torch.cuda.device(flat.device):
        _check(load().oq_pack_lowbit(_ptr(flat), bits, flat.numel(), _ptr(out), _stream(flat.device)))
    return out


def dequantize_packed_weight(packed, row_norms, centroids, *, bits, out_features, in_features,
                             dtype=torch.bfloat16) -> torch.Tensor:
    _require_cuda("packed_weight_indices", packed)
    device = packed.device
    packed = packed.to(torch.uint8).contiguous()
    if packed.numel() < (out_features * in_features * bits + 7) // 8:
        raise ValueError("packed weights are too short")
    norms = row_norms.to(device=device, dtype=torch.bfloat16).contiguous()
    cent = centroids.to(device=device, dtype=torch.float32).contiguous()
    out = torch.empty((out_features, in_features), dtype=dtype, device=device)
    with torch.cuda.device(device):
        _check(load().oq_dequantize_weight(_ptr(packed), bits, out_features, in_features,
                                           _ptr(norms), _ptr(cent), _ptr(out), DTYPE_CODES[dtype],
                                           _stream(device)))
    return out


def quantize_activations(x, permutation, signs, centroids, boundaries, *, eps, block_size,
                         return_codes=False, return_norms=False):
    """RPBH rotate + online quantise; returns ``x_q`` (and optionally codes / norms)."""
    _require_cuda("x", x)
    if x.dtype not in DTYPE_CODES:
        raise ValueError("x must be float32, float16, or bfloat16")
    if block_size <= 0 or block_size & (block_size - 1):
        raise ValueError("block_size must be a positive power of two")
    dim = x.shape[-1]
    if dim % block_size != 0:
        raise ValueError("block_size must divide the input dimension")
    device = x.device
    values = x.contiguous().reshape(-1, dim)
    rows = values.shape[0]
    bits = int(centroids.numel()).bit_length() - 1
    if centroids.numel() != 1 << bits or boundaries.numel() != (1 << bits) - 1:
        raise ValueError("centroids must have 2^bits entries and boundaries 2^bits - 1")
    perm = permutation.to(device=device, dtype=torch.int32).contiguous()
    sgn = signs.to(device=device, dtype=torch.int8).contiguous()
    cent = centroids.to(device=device, dtype=torch.float32).contiguous()
    bnd = boundaries.to(device=device, dtype=torch.float32).contiguous()
    out = torch.empty_like(values)
    codes = torch.empty((rows, dim), dtype=torch.uint8, device=device) if return_codes else None
    norms = torch.empty((rows,), dtype=torch.float32, device=device) if return_norms else None
    with torch.cuda.device(device):
        _check(load().oq_quantize_activations(
            _ptr(values), DTYPE_CODES[x.dtype], rows, dim, _ptr(perm), _ptr(sgn), int(block_size),
            _ptr(bnd), _ptr(cent), bits, float(eps), _ptr(out), _ptr(codes), _ptr(norms),
            _stream(device)))
    result = [out.reshape(x.shape)]
    if return_codes:
        result.append(codes.reshape(x.shape))
    if return_norms:
        result.append(norms.reshape(x.shape[:-1]))
    return result[0] if len(result) == 1 else tuple(result)


def matmul_packed_weight(x, packed_weight_indices, row_norms, centroids, *, bits, out_features,
                         in_features, bias=None, weight_mode=WEIGHT_AUTO, kernel=KERNEL_AUTO,
                         block_m=64, block_n=64, block_k=128):
    """``x @ W^T + bias`` with W decoded from the packed stream.  ``block_*`` are accepted
    for signature compatibility and ignored, as the reference's CUDA kernels ignore them."""
    if bits <= 0 or bits > 8:
        raise ValueError("bits must be in [1, 8]")
    if x.shape[-1] != in_features:
        raise ValueError(f"expected input last dimension {in_features}, got {x.shape[-1]}")
    if block_m <= 0 or block_n <= 0 or block_k <= 0:
        raise ValueError("packed matmul tile sizes must be positive")
    _require_cuda("x", x)
    if x.dtype not in DTYPE_CODES:
        raise ValueError("x must be float32, float16, or bfloat16")
    device = x.device
    x2 = x.contiguous().reshape(-1, in_features)
    rows = x2.shape[0]
    out = torch.empty((rows, out_features), dtype=x.dtype, device=device)
    packed = packed_weight_indices.to(device=device, dtype=torch.uint8).contiguous()
    norms = row_norms.to(device=device, dtype=torch.bfloat16).contiguous()
    cent = centroids.to(device=device, dtype=torch.float32).contiguous()
    bias_t = None if bias is None else bias.to(device=device).contiguous()
    if bias_t is not None and bias_t.dtype not in DTYPE_CODES:
        bias_t = bias_t.to(torch.float32)
    bias_code = 0 if bias_t is None else DTYPE_CODES[bias_t.dtype]
    lib = load()
    ws_bytes = lib.oq_matmul_workspace_bytes(rows, in_features, out_features, bits,
                                             DTYPE_CODES[x.dtype], weight_mode, kernel)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=device) if ws_bytes else None
    with torch.cuda.device(device):
        _check(lib.oq_matmul_packed_weight(
            _ptr(out), _ptr(x2), DTYPE_CODES[x.dtype], rows, in_features, out_features,
            _ptr(packed), packed.numel(), bits, _ptr(norms), _ptr(cent), _ptr(bias_t), bias_code,
            weight_mode, kernel, _ptr(ws), ws_bytes, _stream(device)))
    return out.reshape(*x.shape[:-1], out_features)


def rows_to_f16_operand(x, centroids=None):
    """``x`` (bf16/f16 ``[rows, K]``) -> (f16 operand, per-token power-of-two factors, table
    scale).  The table scale (a 1-element f32 tensor) is searched for ``centroids`` when
    given, else ``None``."""
    _require_cuda("x", x)
    x2 = x.contiguous().reshape(-1, x.shape[-1])
    out = torch.empty(x2.shape, dtype=torch.float16, device=x.device)
    scale = torch.empty(x2.shape[0], dtype=torch.float32, device=x.device)
    table = None
    bits = 0
    if centroids is not None:
        centroids = centroids.to(device=x.device, dtype=torch.float32).contiguous()
        bits = int(centroids.numel()).bit_length() - 1
        table = torch.empty(1, dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _check(load().oq_rows_to_f16_operand(_ptr(x2), DTYPE_CODES[x.dtype], x2.shape[0], x2.shape[1],
                                             _ptr(out), _ptr(scale), _ptr(centroids), bits,
                                             _ptr(table), _stream(x.device)))
    return out, scale, table


def gemm_tcgen05_f16(x_f16, row_scale, packed, row_norms, centroids, *, out_features, bits=4,
                     bias=None, out=None, table_scale=None):
    """The tcgen05 GEMM alone on a prepared f16 operand; all tensors already on the device
    with their final dtypes (uint8 / bf16 / f32), nothing is converted here."""
    _require_cuda("x_f16", x_f16)
    rows, k = x_f16.shape
    if out is None:
        out = torch.empty((rows, out_features), dtype=torch.bfloat16, device=x_f16.device)
    bias_code = 0 if bias is None else DTYPE_CODES[bias.dtype]
    with torch.cuda.device(x_f16.device):
        _check(load().oq_gemm_tcgen05_f16(
            _ptr(out), _ptr(x_f16), _ptr(row_scale), _ptr(table_scale), rows, k, out_features,
            _ptr(packed), packed.numel(), int(bits), _ptr(row_norms), _ptr(centroids), _ptr(bias),
            bias_code, _stream(x_f16.device)))
    return out


def linear_forward(x, packed, row_norms, bias, *, permutation, signs, block_size,
                   act_boundaries, act_centroids, weight_centroids, weight_bits, out_features,
                   eps, weight_mode=WEIGHT_AUTO, kernel=KERNEL_AUTO, out_dtype=None):
    """The whole forward in one C call (prologue + packed matmul).  All constant tensors
    must already live on ``x.device`` with the dtypes the C ABI expects; the caller (the
    module) caches them, so nothing is converted or copied here."""
    _require_cuda("x", x)
    if x.dtype not in DTYPE_CODES:
        raise ValueError("x must be float32, float16, or bfloat16")
    in_features = x.shape[-1]
    device = x.device
    x2 = x.contiguous().reshape(-1, in_features)
    rows = x2.shape[0]
    out = torch.empty((rows, out_features), dtype=x.dtype, device=device)
    act_bits = int(act_centroids.numel()).bit_length() - 1
    code = DTYPE_CODES[x.dtype]
    lib = load()
    ws_bytes = lib.oq_linear_workspace_bytes(rows, in_features, out_features, weight_bits, code,
                                             weight_mode, kernel)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=device)
    bias_code = 0 if bias is None else DTYPE_CODES[bias.dtype]
    with torch.cuda.device(device):
        _check(lib.oq_linear_forward(
            _ptr(out), _ptr(x2), code, rows, in_features, out_features, _ptr(packed),
            packed.numel(), weight_bits, _ptr(row_norms), _ptr(weight_centroids), _ptr(bias),
            bias_code, _ptr(permutation), _ptr(signs), int(block_size), _ptr(act_boundaries),
            _ptr(act_centroids), act_bits, float(eps), weight_mode, kernel, _ptr(ws), ws_bytes,
            _stream(device)))
    result = out.reshape(*x.shape[:-1], out_features)
    if out_dtype is not None and out_dtype != result.dtype:
        result = result.to(out_dtype)
    return result


def linear_forward_scatter(x, packed, row_norms, bias, *, out_ptrs, out_ld, out_col, permutation,
                           signs, block_size, act_boundaries, act_centroids, weight_centroids,
                           weight_bits, out_features, eps):
    """The whole forward of a column shard, its result stored into every buffer of
    ``out_ptrs`` (device addresses of row-major bf16 ``[rows, out_ld]`` buffers: this rank's
    and its peers' mapped copies) at columns ``out_col ..``.  Nothing is returned; the caller
    synchronises the ranks before reading.  Raises RuntimeError where the large-row
    tcgen05 kernel does not apply."""
    _require_cuda("x", x)
    if x.dtype not in DTYPE_CODES:
        raise ValueError("x must be float32, float16, or bfloat16")
    in_features = x.shape[-1]
    device = x.device
    x2 = x.contiguous().reshape(-1, in_features)
    rows = x2.shape[0]
    act_bits = int(act_centroids.numel()).bit_length() - 1
    code = DTYPE_CODES[x.dtype]
    lib = load()
    ws_bytes = lib.oq_linear_workspace_bytes(rows, in_features, out_features, weight_bits, code,
                                             WEIGHT_AUTO, KERNEL_TCGEN05)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=device)
    bias_code = 0 if bias is None else DTYPE_CODES[bias.dtype]
    ptr_array = (ctypes.c_void_p * len(out_ptrs))(*[int(p) for p in out_ptrs])
    with torch.cuda.device(device):
        _check(lib.oq_linear_forward_scatter(
            ptr_array, len(out_ptrs), int(out_ld), int(out_col), _ptr(x2), code, rows, in_features,
            out_features, _ptr(packed), packed.numel(), weight_bits, _ptr(row_norms),
            _ptr(weight_centroids), _ptr(bias), bias_code, _ptr(permutation), _ptr(signs),
            int(block_size), _ptr(act_boundaries), _ptr(act_centroids), act_bits, float(eps),
            _ptr(ws), ws_bytes, _stream(device)))


def quantize_weight_packed(weight, *, permutation, signs, block_size, boundaries, centroids, bits,
                           eps, row_norms=None):
    """Offline weight quantisation on the GPU: ``weight [N, K]`` (CUDA) -> (packed uint8 stream,
    bf16 row norms).  ``row_norms`` (f32 ``[N]``) pins the norms, e.g. to the ones a CPU
    reference computed; otherwise they are computed on the device."""
    _require_cuda("weight", weight)
    if weight.ndim != 2:
        raise ValueError("weight must be a matrix")
    if weight.dtype not in DTYPE_CODES:
        raise ValueError("weight must be float32, float16, or bfloat16")
    device = weight.device
    w = weight.contiguous()
    n, k = w.shape
    perm = permutation.to(device=device, dtype=torch.int32).contiguous()
    sg = signs.to(device=device, dtype=torch.int8).contiguous()
    bnd = boundaries.to(device=device, dtype=torch.float32).contiguous()
    cent = centroids.to(device=device, dtype=torch.float32).contiguous()
    norms_in = None if row_norms is None else row_norms.to(device=device, dtype=torch.float32).contiguous()
    packed = torch.empty((n * k * bits + 7) // 8, dtype=torch.uint8, device=device)
    norms_out = torch.empty(n, dtype=torch.bfloat16, device=device)
    lib = load()
    ws_bytes = lib.oq_quantize_weight_workspace_bytes(n, k)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=device)
    with torch.cuda.device(device):
        _check(lib.oq_quantize_weight(
            _ptr(w), DTYPE_CODES[w.dtype], n, k, _ptr(perm), _ptr(sg), int(block_size), _ptr(bnd),
            _ptr(cent), int(bits), float(eps), _ptr(norms_in), _ptr(norms_out), _ptr(packed),
            _ptr(ws), ws_bytes, _stream(device)))
    return packed, norms_out


def rtn_int4_linear_forward(x, packed, scales, bias, *, out_features, group_size=64):
    """``x @ W^T + bias`` with ``W[n, k] = bf16((code - 8) * scale[n, k // 64])`` decoded from
    the packed 4-bit codes; bf16 in, bf16 out (the AdaLN modulation layers)."""
    _require_cuda("x", x)
    in_features = x.shape[-1]
    device = x.device
    x2 = x.to(torch.bfloat16).contiguous().reshape(-1, in_features)
    rows = x2.shape[0]
    out = torch.empty((rows, out_features), dtype=torch.bfloat16, device=device)
    lib = load()
    ws_bytes = lib.oq_rtn_int4_workspace_bytes(rows, in_features, out_features)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=device)
    bias_code = 0 if bias is None else DTYPE_CODES[bias.dtype]
    with torch.cuda.device(device):
        _check(lib.oq_rtn_int4_linear_forward(
            _ptr(out), _ptr(x2), rows, in_features, out_features, _ptr(packed), packed.numel(),
            _ptr(scales), int(group_size), _ptr(bias), bias_code, _ptr(ws), ws_bytes, _stream(device)))
    return out.reshape(*x.shape[:-1], out_features)


def _activation_constants(x, permutation, signs, centroids, boundaries):
    device = x.device
    return (permutation.to(device=device, dtype=torch.int32).contiguous(),
            signs.to(device=device, dtype=torch.int8).contiguous(),
            centroids.to(device=device, dtype=torch.float32).contiguous(),
            boundaries.to(device=device, dtype=torch.float32).contiguous())


def quantize_activations_packed_w4(x, permutation, signs, centroids, boundaries, *, eps, block_size):
    """4-bit activation indices packed two per byte ``[..., K/2]`` (low nibble = even k) and the
    fp32 token norms -- the activation stream of the integer matmuls
    (reference wrapper ``orbitquant_packed_matmul/__init__.py``: ``quantize_activations_packed_w4``)."""
    _require_cuda("x", x)
    if x.dtype not in DTYPE_CODES:
        raise ValueError("x must be float32, float16, or bfloat16")
    if centroids.numel() != 16 or boundaries.numel() != 15:
        raise ValueError("the packed 4-bit output needs a 4-bit activation codebook")
    dim = x.shape[-1]
    values = x.contiguous().reshape(-1, dim)
    rows = values.shape[0]
    device = x.device
    perm, sgn, cent, bnd = _activation_constants(x, permutation, signs, centroids, boundaries)
    packed = torch.empty((rows, dim // 2), dtype=torch.uint8, device=device)
    norms = torch.empty((rows,), dtype=torch.float32, device=device)
    lib = load()
    ws_bytes = lib.oq_quantize_activations_packed_w4_workspace_bytes(rows, dim)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=device)
    with torch.cuda.device(device):
        _check(lib.oq_quantize_activations_packed_w4(
            _ptr(values), DTYPE_CODES[x.dtype], rows, dim, _ptr(perm), _ptr(sgn), int(block_size),
            _ptr(bnd), _ptr(cent), float(eps), _ptr(packed), _ptr(norms), _ptr(ws), ws_bytes,
            _stream(device)))
    return packed.reshape(*x.shape[:-1], dim // 2), norms.reshape(x.shape[:-1])


def quantize_activations_int8(x, permutation, signs, centroids, boundaries, act_codes, *, eps, block_size):
    """``act_codes[index]`` as int8 ``[..., K]`` and the fp32 token norms (reference wrapper
    ``quantize_activations_int8``)."""
    _require_cuda("x", x)
    if x.dtype not in DTYPE_CODES:
        raise ValueError("x must be float32, float16, or bfloat16")
    dim = x.shape[-1]
    values = x.contiguous().reshape(-1, dim)
    rows = values.shape[0]
    device = x.device
    bits = int(centroids.numel()).bit_length() - 1
    perm, sgn, cent, bnd = _activation_constants(x, permutation, signs, centroids, boundaries)
    table = act_codes.to(device=device, dtype=torch.int8).contiguous()
    if table.numel() < 1 << bits:
        raise ValueError("act_codes must hold 2^bits entries")
    codes = torch.empty((rows, dim), dtype=torch.int8, device=device)
    norms = torch.empty((rows,), dtype=torch.float32, device=device)
    with torch.cuda.device(device):
        _check(load().oq_quantize_activations_int8(
            _ptr(values), DTYPE_CODES[x.dtype], rows, dim, _ptr(perm), _ptr(sgn), int(block_size),
            _ptr(bnd), _ptr(cent), bits, _ptr(table), float(eps), _ptr(codes), _ptr(norms),
            _stream(device)))
    return codes.reshape(x.shape), norms.reshape(x.shape[:-1])


def matmul_packed_w4a4_int8(packed_act, packed_weight, token_norms, row_norms, act_codes, weight_codes, *,
                            act_scale, weight_scale, out_features, in_features, weight_bits=4, bias=None):
    """The INT8-surrogate matmul on packed 4-bit activations (reference wrapper
    ``matmul_packed_w4a4_int8``); bf16 output."""
    _require_cuda("packed_act", packed_act)
    device = packed_act.device
    pa = packed_act.to(torch.uint8).contiguous().reshape(-1, in_features // 2)
    rows = pa.shape[0]
    pw = packed_weight.to(device=device, dtype=torch.uint8).contiguous()
    tn = token_norms.to(device=device, dtype=torch.float32).contiguous().reshape(-1)
    rn = row_norms.to(device=device, dtype=torch.bfloat16).contiguous()
    ac = act_codes.to(device=device, dtype=torch.int8).contiguous()
    wc = weight_codes.to(device=device, dtype=torch.int8).contiguous()
    bias_t = None if bias is None else bias.to(device=device).contiguous()
    if bias_t is not None and bias_t.dtype not in DTYPE_CODES:
        bias_t = bias_t.to(torch.float32)
    out = torch.empty((rows, out_features), dtype=torch.bfloat16, device=device)
    lib = load()
    ws_bytes = lib.oq_matmul_packed_w4a4_int8_workspace_bytes(rows, in_features)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=device)
    with torch.cuda.device(device):
        _check(lib.oq_matmul_packed_w4a4_int8(
            _ptr(out), _ptr(pa), _ptr(pw), pw.numel(), int(weight_bits), _ptr(tn), _ptr(rn), _ptr(ac),
            _ptr(wc), _ptr(bias_t), 0 if bias_t is None else DTYPE_CODES[bias_t.dtype],
            float(act_scale), float(weight_scale), rows, in_features, out_features, _ptr(ws), ws_bytes,
            _stream(device)))
    return out.reshape(*packed_act.shape[:-1], out_features)


def linear_w4a4_int8_supported(x, in_features, out_features, block_size, weight_bits=4):
    """Whether ``linear_w4a4_int8`` takes this problem (bf16 rows, more than 128 of them, 4-bit
    weights, ``in_features % 256 == 0``, rotation block 256 .. 4096)."""
    if weight_bits != 4 or x.dtype not in DTYPE_CODES or not x.is_cuda:
        return False
    rows = x.numel() // max(in_features, 1)
    return bool(load().oq_linear_w4a4_int8_supported(
        DTYPE_CODES[x.dtype], rows, int(in_features), int(out_features), int(block_size)))


def linear_w4a4_int8(x, packed_weight, row_norms, bias, *, permutation, signs, block_size, act_boundaries,
                     act_centroids, act_codes, weight_codes, act_scale, weight_scale, out_features, eps):
    """The INT8-surrogate W4A4 linear in one call: rotate + quantise straight to the INT8 operand,
    INT8 tensor-core matmul (the reference module's fused INT8 route, ``layers.py:1097-1352``);
    bf16 output equal to ``quantize_activations_packed_w4`` + ``matmul_packed_w4a4_int8``."""
    _require_cuda("x", x)
    in_features = x.shape[-1]
    device = x.device
    values = x.contiguous().reshape(-1, in_features)
    rows = values.shape[0]
    perm, sgn, cent, bnd = _activation_constants(x, permutation, signs, act_centroids, act_boundaries)
    pw = packed_weight.to(device=device, dtype=torch.uint8).contiguous()
    rn = row_norms.to(device=device, dtype=torch.bfloat16).contiguous()
    ac = act_codes.to(device=device, dtype=torch.int8).contiguous()
    wc = weight_codes.to(device=device, dtype=torch.int8).contiguous()
    bias_t = None if bias is None else bias.to(device=device).contiguous()
    if bias_t is not None and bias_t.dtype not in DTYPE_CODES:
        bias_t = bias_t.to(torch.float32)
    out = torch.empty((rows, out_features), dtype=torch.bfloat16, device=device)
    lib = load()
    ws_bytes = lib.oq_linear_w4a4_int8_workspace_bytes(rows, in_features)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=device)
    with torch.cuda.device(device):
        _check(lib.oq_linear_w4a4_int8(
            _ptr(out), _ptr(values), DTYPE_CODES[x.dtype], rows, in_features, out_features, _ptr(pw),
            pw.numel(), _ptr(rn), _ptr(bias_t), 0 if bias_t is None else DTYPE_CODES[bias_t.dtype],
            _ptr(perm), _ptr(sgn), int(block_size), _ptr(bnd), _ptr(cent), _ptr(ac), _ptr(wc),
            float(act_scale), float(weight_scale), float(eps), _ptr(ws), ws_bytes, _stream(device)))
    return out.reshape(*x.shape[:-1], out_features)


def linear_w4a4_pair_lut(x, packed, row_norms, bias, *, permutation, signs, block_size, act_boundaries,
                         act_centroids, pair_lut, out_features, eps):
    """The exact W4A4 linear through the 256-entry pair-product table (the arithmetic of the
    reference's ``orbitquant_vulkan::linear_w4a4_exact``); output in ``x``'s dtype."""
    _require_cuda("x", x)
    if x.dtype not in DTYPE_CODES:
        raise ValueError("x must be float32, float16, or bfloat16")
    in_features = x.shape[-1]
    device = x.device
    x2 = x.contiguous().reshape(-1, in_features)
    rows = x2.shape[0]
    perm, sgn, cent, bnd = _activation_constants(x, permutation, signs, act_centroids, act_boundaries)
    lut = pair_lut.to(device=device, dtype=torch.float32).contiguous()
    if lut.numel() != 256:
        raise ValueError("pair_lut must hold 256 entries")
    pw = packed.to(device=device, dtype=torch.uint8).contiguous()
    rn = row_norms.to(device=device, dtype=torch.bfloat16).contiguous()
    bias_t = None if bias is None else bias.to(device=device).contiguous()
    if bias_t is not None and bias_t.dtype not in DTYPE_CODES:
        bias_t = bias_t.to(torch.float32)
    out = torch.empty((rows, out_features), dtype=x.dtype, device=device)
    lib = load()
    ws_bytes = lib.oq_linear_w4a4_pair_lut_workspace_bytes(rows, in_features)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=device)
    with torch.cuda.device(device):
        _check(lib.oq_linear_w4a4_pair_lut(
            _ptr(out), _ptr(x2), DTYPE_CODES[x.dtype], rows, in_features, out_features, _ptr(pw),
            pw.numel(), _ptr(rn), _ptr(bias_t), 0 if bias_t is None else DTYPE_CODES[bias_t.dtype],
            _ptr(perm), _ptr(sgn), int(block_size), _ptr(bnd), _ptr(cent), _ptr(lut), float(eps),
            _ptr(ws), ws_bytes, _stream(device)))
    return out.reshape(*x.shape[:-1], out_features)
