"""ctypes front end of ``oracle/orbit_oracle.c`` (the CPU parity oracle).

TEST INFRASTRUCTURE ONLY -- imported by ``tests/``, ``__graft_entry__.smoke()`` and the
CPU-baseline leg of ``bench.py``; never by the product package.

All tensors are CPU torch tensors; bf16 travels as raw 16-bit patterns.
"""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
_SRC = HERE / "orbit_oracle.c"
_LIB = HERE / "liborbit_oracle.so"

NORM_SCALAR, NORM_AVX512, NORM_AVX2 = 0, 1, 2
MM_FP32_CENTROIDS, MM_BF16_LUT = 0, 1
_DTYPES = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}

_lib = None


def build(force: bool = False) -> Path:
    if force or not _LIB.exists() or _LIB.stat().st_mtime < _SRC.stat().st_mtime:
        cc = "/usr/bin/gcc" if Path("/usr/bin/gcc").exists() else "gcc"
        subprocess.run(
            [cc, "-O2", "-ffp-contract=off", "-fopenmp", "-fPIC", "-shared",
             "-o", str(_LIB), str(_SRC), "-lm"], check=True)
    return _LIB


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(str(_LIB))
        _lib.oqo_quantize_activations.restype = ctypes.c_int
        _lib.oqo_quantize_activations.argtypes = [
            ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_int64,
            ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64,
            ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
            ctypes.c_float, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
        _lib.oqo_matmul_packed.restype = ctypes.c_int
        _lib.oqo_matmul_packed.argtypes = [
            ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
            ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
            ctypes.c_int, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p]
        _lib.oqo_unpack.restype = None
        _lib.oqo_unpack.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_void_p]
        _lib.oqo_pack.restype = None
        _lib.oqo_pack.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_void_p]
        _lib.oqo_fwht.restype = None
        _lib.oqo_fwht.argtypes = [ctypes.c_void_p, ctypes.c_int64]
    return _lib


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def unpack(packed: torch.Tensor, bits: int, count: int) -> torch.Tensor:
    packed = packed.contiguous()
    out = torch.empty(count, dtype=torch.uint8)
    lib().oqo_unpack(_ptr(packed), bits, count, _ptr(out))
    return out


def pack(values: torch.Tensor, bits: int) -> torch.Tensor:
    values = values.to(torch.uint8).contiguous().flatten()
    out = torch.empty((values.numel() * bits + 7) // 8, dtype=torch.uint8)
    lib().oqo_pack(_ptr(values), bits, values.numel(), _ptr(out))
    return out


def fwht(values: torch.Tensor) -> torch.Tensor:
    out = values.to(torch.float32).contiguous().clone()
    n = out.shape[-1]
    flat = out.reshape(-1, n)
    for row in range(flat.shape[0]):
        lib().oqo_fwht(ctypes.c_void_p(flat[row].data_ptr()), n)
    return out


def quantize_activations(x, perm, signs, block, boundaries, centroids, *, eps=1e-10,
                         norm_order=NORM_AVX512):
    """Returns ``(x_q [same dtype/shape as x], codes u8, norms f32)``."""
    dim = x.shape[-1]
    x2 = x.contiguous().reshape(-1, dim)
    rows = x2.shape[0]
    perm = perm.to(torch.int32).contiguous()
    signs = signs.to(torch.int8).contiguous()
    boundaries = boundaries.to(torch.float32).contiguous()
    centroids = centroids.to(torch.float32).contiguous()
    bits = int(centroids.numel()).bit_length() - 1
    out = torch.empty_like(x2)
    codes = torch.empty((rows, dim), dtype=torch.uint8)
    norms = torch.empty(rows, dtype=torch.float32)
    rc = lib().oqo_quantize_activations(
        _ptr(x2), _DTYPES[x.dtype], rows, dim, _ptr(perm), _ptr(signs), int(block),
        _ptr(boundaries), _ptr(centroids), bits, float(eps), int(norm_order),
        _ptr(out), _ptr(codes), _ptr(norms))
    if rc != 0:
        raise ValueError(f"oracle quantize_activations failed ({rc})")
    return out.reshape(x.shape), codes.reshape(x.shape), norms


def matmul_packed(x_q, packed, row_norms, centroids, *, bits, out_features, bias=None,
                  mode=MM_FP32_CENTROIDS, n_begin=0, n_end=None):
    """Returns ``(y [x dtype], y_f32)`` for output columns ``[n_begin, n_end)``; the other
    columns are left zero."""
    k = x_q.shape[-1]
    x2 = x_q.contiguous().reshape(-1, k)
    rows = x2.shape[0]
    n_end = out_features if n_end is None else n_end
    packed = packed.to(torch.uint8).contiguous()
    row_norms = row_norms.to(torch.float32).contiguous()
    centroids = centroids.to(torch.float32).contiguous()
    bias_f = None if bias is None else bias.to(torch.float32).contiguous()
    out = torch.zeros((rows, out_features), dtype=x_q.dtype)
    out_f32 = torch.zeros((rows, out_features), dtype=torch.float32)
    rc = lib().oqo_matmul_packed(
        _ptr(x2), _DTYPES[x_q.dtype], rows, k, out_features, _ptr(packed), int(bits),
        _ptr(row_norms), _ptr(centroids), _ptr(bias_f), int(mode), int(n_begin), int(n_end),
        _ptr(out), _ptr(out_f32))
    if rc != 0:
        raise ValueError(f"oracle matmul_packed failed ({rc})")
    shape = (*x_q.shape[:-1], out_features)
    return out.reshape(shape), out_f32.reshape(shape)


def linear_forward(x, packed, row_norms, bias, *, perm, signs, block, act_boundaries,
                   act_centroids, w_centroids, w_bits, out_features, eps=1e-10,
                   norm_order=NORM_AVX512, mode=MM_FP32_CENTROIDS):
    x_q, _, _ = quantize_activations(x, perm, signs, block, act_boundaries, act_centroids,
                                     eps=eps, norm_order=norm_order)
    return matmul_packed(x_q, packed, row_norms, w_centroids, bits=w_bits,
                         out_features=out_features, bias=bias, mode=mode)


def rtn_int4_matmul(x, packed, scales, *, out_features, in_features, group_size=64, bias=None):
    """RTN-INT4 group linear as the reference's scalar CPU kernel defines it
    (``orbitquant_packed_matmul_cpu/packed_adaln_cpu.cpp:54-100``): weight value
    ``bf16((code - 8) * scale)``, fp32 products accumulated over k in ascending order in fp32,
    ``+ bias``, rounded to bf16.  numpy restatement (test infrastructure; small sizes)."""
    import numpy as np

    groups = (in_features + group_size - 1) // group_size
    padded = groups * group_size
    raw = packed.cpu().numpy().astype(np.uint8)
    codes = np.empty(raw.size * 2, dtype=np.int32)
    codes[0::2] = raw & 15
    codes[1::2] = raw >> 4
    codes = codes[: out_features * padded].reshape(out_features, padded) - 8
    scale = scales.cpu().to(torch.float32).numpy().reshape(out_features, groups)
    dense = (codes.astype(np.float32).reshape(out_features, groups, group_size) * scale[..., None]).astype(np.float32)
    weight = torch.from_numpy(dense.reshape(out_features, padded)[:, :in_features].copy()).to(torch.bfloat16).to(torch.float32).numpy()
    x2 = x.to(torch.bfloat16).to(torch.float32).reshape(-1, in_features).cpu().numpy()
    acc = np.zeros((x2.shape[0], out_features), dtype=np.float32)
    for k in range(in_features):   # ascending k, one fp32 rounding per product and per add
        acc += (x2[:, k:k + 1] * weight[None, :, k]).astype(np.float32)
    if bias is not None:
        acc += bias.cpu().to(torch.float32).numpy()[None, :]
    out = torch.from_numpy(acc).to(torch.bfloat16)
    return out.reshape(*x.shape[:-1], out_features)


def pair_lut_linear(x, packed, row_norms, bias, *, perm, signs, block, act_boundaries, act_centroids,
                    pair_lut, out_features, eps=1e-10, norm_order=NORM_AVX512):
    """Exact W4A4 linear through the 256-entry pair-product table, the arithmetic of the
    reference's ``_linear_w4a4_exact_reference`` (``src/orbitquant/kernels/executorch_vulkan.py:
    15-61``): ``(sum_k lut[16 a + w]) * token_norm * row_norm + bias`` in fp32, rounded to
    ``x``'s dtype.  The table entries are added one by one in ascending k (the reference sums
    with ``torch.sum``, whose order is unspecified; the difference is fp32 summation noise).
    Activation indices and token norms come from ``quantize_activations`` above (the native CPU
    pipeline's order) rather than from the reference's torch expressions.  numpy; small sizes."""
    import numpy as np

    k = x.shape[-1]
    x2 = x.contiguous().reshape(-1, k)
    _, codes, norms = quantize_activations(x2, perm, signs, block, act_boundaries, act_centroids,
                                           eps=eps, norm_order=norm_order)
    a = codes.numpy().astype(np.int64)
    w = unpack(packed, 4, out_features * k).numpy().astype(np.int64).reshape(out_features, k)
    lut = pair_lut.to(torch.float32).numpy()
    acc = np.zeros((a.shape[0], out_features), dtype=np.float32)
    for kk in range(k):
        acc += lut[a[:, kk][:, None] * 16 + w[:, kk][None, :]]
    rn = row_norms.to(torch.float32).numpy()
    out = (acc * norms.numpy()[:, None]).astype(np.float32) * rn[None, :]
    if bias is not None:
        out = out + bias.to(torch.float32).numpy()[None, :]
    y32 = torch.from_numpy(out.astype(np.float32))
    return y32.to(x.dtype).reshape(*x.shape[:-1], out_features), y32.reshape(*x.shape[:-1], out_features)


def int8_surrogate_linear(x, packed, row_norms, bias, *, perm, signs, block, act_boundaries,
                          act_centroids, act_codes, act_scale, w_codes, w_scale, w_bits, out_features,
                          eps=1e-10, norm_order=NORM_AVX512):
    """The reference's integer matmul (``packed_matmul.cu:744-1009``, epilogue ``:976-1007``):
    ``(sum_k act_codes[a] * w_codes[w]) * token_norm * row_norm * (s_a * s_w) + bias`` with an
    int32 sum, rounded to bf16.  numpy; small sizes."""
    import numpy as np

    k = x.shape[-1]
    x2 = x.contiguous().reshape(-1, k)
    _, codes, norms = quantize_activations(x2, perm, signs, block, act_boundaries, act_centroids,
                                           eps=eps, norm_order=norm_order)
    a = act_codes.numpy().astype(np.int64)[codes.numpy().astype(np.int64)]
    w_idx = unpack(packed, w_bits, out_features * k).numpy().astype(np.int64).reshape(out_features, k)
    w = w_codes.numpy().astype(np.int64)[w_idx]
    acc = (a @ w.T).astype(np.float32)                      # exact: |sum| < 2^24 for these sizes
    scale = np.float32(np.float32(act_scale) * np.float32(w_scale))
    rn = row_norms.to(torch.float32).numpy()
    out = acc * (norms.numpy() * scale)[:, None].astype(np.float32) * rn[None, :]
    if bias is not None:
        out = out + bias.to(torch.float32).numpy()[None, :]
    y32 = torch.from_numpy(out.astype(np.float32))
    return y32.to(torch.bfloat16).reshape(*x.shape[:-1], out_features), y32.reshape(*x.shape[:-1], out_features)
