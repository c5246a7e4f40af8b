// General packed-weight matmul on CUDA cores, plus the bit-stream utilities.
//
// This is the kernel for shapes the specialised kernels do not take (in_features not a
// multiple of 64, bit widths other than the tensor-core kernel's, fp32 activations).  It
// decodes any 1..8-bit little-endian stream field by field, so it doubles as the in-library
// cross-check for the fast kernels.  Tile 64x64x32 (or 16x64x32 for <= 16 rows), 256
// threads, 4 output columns per thread, fp32 accumulation in k order.
#include "common.cuh"

namespace oq {
namespace {

constexpr int kThreads = 256;
constexpr int kBN = 64;
constexpr int kBK = 32;

struct TiledParams {
  void *out;
  const void *x;
  const uint8_t *packed;
  const __nv_bfloat16 *row_norms;
  const float *centroids;
  const void *bias;
  int64_t rows;
  int64_t in_features;
  int64_t out_features;
  int bits;
  int bias_dtype;  // -1 = none
  int scaled_bf16; // 1: operand is bf16(centroid*row_norm); 0: centroid, row_norm afterwards
};

__device__ __forceinline__ float load_bias(const void *bias, int dtype, int64_t n) {
  switch (dtype) {
    case OQ_DTYPE_F32: return Scalar<OQ_DTYPE_F32>::load(bias, n);
    case OQ_DTYPE_F16: return Scalar<OQ_DTYPE_F16>::load(bias, n);
    default: return Scalar<OQ_DTYPE_BF16>::load(bias, n);
  }
}

template <int DTYPE, int BM>
__global__ void __launch_bounds__(kThreads) tiled_matmul_kernel(const TiledParams p) {
  constexpr int TM = BM / 16;
  __shared__ float xs[kBK][BM + 1];
  __shared__ float ws[kBK][kBN + 1];
  __shared__ float s_cent[256];
  const int tx = threadIdx.x & 15;
  const int ty = threadIdx.x >> 4;
  const int64_t m0 = static_cast<int64_t>(blockIdx.y) * BM;
  const int64_t n0 = static_cast<int64_t>(blockIdx.x) * kBN;
  for (int i = threadIdx.x; i < (1 << p.bits); i += kThreads) {
    s_cent[i] = p.centroids[i];
  }
  __syncthreads();

  float acc[TM][4];
#pragma unroll
  for (int i = 0; i < TM; ++i) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      acc[i][j] = 0.0f;
    }
  }

  for (int64_t k0 = 0; k0 < p.in_features; k0 += kBK) {
    for (int i = threadIdx.x; i < BM * kBK; i += kThreads) {
      const int m = i / kBK;
      const int k = i % kBK;
      float v = 0.0f;
      if (m0 + m < p.rows && k0 + k < p.in_features) {
        v = Scalar<DTYPE>::load(p.x, (m0 + m) * p.in_features + k0 + k);
      }
      xs[k][m] = v;
    }
    for (int i = threadIdx.x; i < kBN * kBK; i += kThreads) {
      const int n = i / kBK;
      const int k = i % kBK;
      float w = 0.0f;
      if (n0 + n < p.out_features && k0 + k < p.in_features) {
        const uint32_t idx = unpack_field(p.packed, (n0 + n) * p.in_features + k0 + k, p.bits);
        w = s_cent[idx];
        if (p.scaled_bf16) {
          const float rn = __bfloat162float(p.row_norms[n0 + n]);
          w = __bfloat162float(__float2bfloat16_rn(__fmul_rn(w, rn)));
        }
      }
      ws[k][n] = w;
    }
    __syncthreads();
#pragma unroll 8
    for (int k = 0; k < kBK; ++k) {
      float a[TM];
      float b[4];
#pragma unroll
      for (int i = 0; i < TM; ++i) {
        a[i] = xs[k][ty * TM + i];
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        b[j] = ws[k][tx * 4 + j];
      }
#pragma unroll
      for (int i = 0; i < TM; ++i) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
      }
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int64_t m = m0 + ty * TM + i;
    if (m >= p.rows) {
      continue;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t n = n0 + tx * 4 + j;
      if (n >= p.out_features) {
        continue;
      }
      float v = acc[i][j];
      if (!p.scaled_bf16) {
        v *= __bfloat162float(p.row_norms[n]);
      }
      if (p.bias_dtype >= 0) {
        v += load_bias(p.bias, p.bias_dtype, n);
      }
      Scalar<DTYPE>::store(p.out, m * p.out_features + n, v);
    }
  }
}

__global__ void unpack_kernel(const uint8_t *packed, int bits, int64_t count, uint8_t *values) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < count;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    values[i] = static_cast<uint8_t>(unpack_field(packed, i, bits));
  }
}

// One thread per output byte: gathers the (at most 8) fields that touch it.
__global__ void pack_kernel(const uint8_t *values, int bits, int64_t count, int64_t bytes,
                            uint8_t *packed) {
  const uint32_t mask = (1u << bits) - 1u;
  for (int64_t b = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; b < bytes;
       b += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t bit_lo = b * 8;
    int64_t first = bit_lo / bits;
    uint32_t byte = 0;
    for (int64_t i = first; i < count && i * bits < bit_lo + 8; ++i) {
      const int64_t shift = i * bits - bit_lo;  // may be negative for a straddling field
      const uint32_t field = static_cast<uint32_t>(values[i]) & mask;
      byte |= shift >= 0 ? (field << shift) : (field >> (-shift));
    }
    packed[b] = static_cast<uint8_t>(byte & 0xffu);
  }
}

template <int DTYPE>
__global__ void dequantize_kernel(const uint8_t *packed, int bits, int64_t out_features,
                                  int64_t in_features, const __nv_bfloat16 *row_norms,
                                  const float *centroids, void *out) {
  const int64_t total = out_features * in_features;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t n = i / in_features;
    const float w = __fmul_rn(__bfloat162float(row_norms[n]), centroids[unpack_field(packed, i, bits)]);
    Scalar<DTYPE>::store(out, i, w);
  }
}

int grid_for(int64_t work, int threads) {
  const int64_t blocks = (work + threads - 1) / threads;
  return static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(blocks, 148 * 32)));
}

}  // namespace

int launch_tiled_matmul(void *out, const void *x, int dtype, int64_t rows, int64_t in_features,
                        int64_t out_features, const uint8_t *packed, int bits,
                        const void *row_norms_bf16, const float *centroids, const void *bias,
                        int bias_dtype, int weight_mode, cudaStream_t stream) {
  TiledParams p{};
  p.out = out;
  p.x = x;
  p.packed = packed;
  p.row_norms = static_cast<const __nv_bfloat16 *>(row_norms_bf16);
  p.centroids = centroids;
  p.bias = bias;
  p.rows = rows;
  p.in_features = in_features;
  p.out_features = out_features;
  p.bits = bits;
  p.bias_dtype = bias == nullptr ? -1 : bias_dtype;
  p.scaled_bf16 = weight_mode == OQ_WEIGHT_BF16_SCALED ? 1 : 0;
  const bool small = rows <= 16;
  const int bm = small ? 16 : 64;
  dim3 grid(static_cast<unsigned>((out_features + kBN - 1) / kBN),
            static_cast<unsigned>((rows + bm - 1) / bm));
  OQ_CHECK_ARG(grid.y <= 65535u, "rows above %d are not supported by the tiled kernel", 65535 * 64);
#define OQ_LAUNCH_TILED(DT)                                                        \
  do {                                                                             \
    if (small) {                                                                   \
      tiled_matmul_kernel<DT, 16><<<grid, kThreads, 0, stream>>>(p);               \
    } else {                                                                       \
      tiled_matmul_kernel<DT, 64><<<grid, kThreads, 0, stream>>>(p);               \
    }                                                                              \
  } while (0)
  switch (dtype) {
    case OQ_DTYPE_F32: OQ_LAUNCH_TILED(OQ_DTYPE_F32); break;
    case OQ_DTYPE_F16: OQ_LAUNCH_TILED(OQ_DTYPE_F16); break;
    default: OQ_LAUNCH_TILED(OQ_DTYPE_BF16); break;
  }
#undef OQ_LAUNCH_TILED
  OQ_CHECK_CUDA(cudaGetLastError());
  count_launch();
  return OQ_OK;
}

int launch_unpack(const uint8_t *packed, int bits, int64_t count, uint8_t *values,
                  cudaStream_t stream) {
  unpack_kernel<<<grid_for(count, 256), 256, 0, stream>>>(packed, bits, count, values);
  OQ_CHECK_CUDA(cudaGetLastError());
  count_launch();
  return OQ_OK;
}

int launch_pack(const uint8_t *values, int bits, int64_t count, uint8_t *packed,
                cudaStream_t stream) {
  const int64_t bytes = (count * bits + 7) / 8;
  pack_kernel<<<grid_for(bytes, 256), 256, 0, stream>>>(values, bits, count, bytes, packed);
  OQ_CHECK_CUDA(cudaGetLastError());
  count_launch();
  return OQ_OK;
}

int launch_dequantize(const uint8_t *packed, int bits, int64_t out_features, int64_t in_features,
                      const void *row_norms_bf16, const float *centroids, void *out,
                      int out_dtype, cudaStream_t stream) {
  const int grid = grid_for(out_features * in_features, 256);
  const auto *rn = static_cast<const __nv_bfloat16 *>(row_norms_bf16);
  switch (out_dtype) {
    case OQ_DTYPE_F32:
      dequantize_kernel<OQ_DTYPE_F32><<<grid, 256, 0, stream>>>(packed, bits, out_features, in_features, rn, centroids, out);
      break;
    case OQ_DTYPE_F16:
      dequantize_kernel<OQ_DTYPE_F16><<<grid, 256, 0, stream>>>(packed, bits, out_features, in_features, rn, centroids, out);
      break;
    default:
      dequantize_kernel<OQ_DTYPE_BF16><<<grid, 256, 0, stream>>>(packed, bits, out_features, in_features, rn, centroids, out);
      break;
  }
  OQ_CHECK_CUDA(cudaGetLastError());
  count_launch();
  return OQ_OK;
}

}  // namespace oq
