// The two integer-index formulations of the W4A4 linear that the reference carries beside its
// exact centroid kernels:
//
//  * INT8-surrogate matmul (reference: orbitquant_packed_matmul_cuda/packed_matmul.cu:744-1009,
//    src/orbitquant/kernels/triton_cuda.py:1861-2099): both code streams are mapped through
//    small INT8 code tables fitted to the centroids, the contraction is an integer dot
//    product, and the epilogue multiplies by token_norm[m] * row_norm[n] * s_a * s_w.  Here the
//    packed activation nibbles are expanded to the f16 operand of the tensor-core GEMM
//    (INT8 codes are exact in f16, their products and sums exact in the fp32 accumulator up to
//    2^24), and the GEMM runs with the weight code table in place of the centroids.
//
//  * exact pair-product table (reference: src/orbitquant/kernels/executorch_vulkan.py:15-61,
//    the CPU restatement of its Vulkan shader): out[m, n] = (sum_k LUT[16 a[m,k] + w[n,k]])
//    * token_norm[m] * row_norm[n] + bias[n] with LUT[16 i + j] = c_a[i] * c_w[j] in fp32.
//    One thread owns an output element and adds the table entries in ascending k, so the
//    result does not depend on the launch shape.
#include <algorithm>

#include "common.cuh"

namespace oq {
namespace {

constexpr int kExpandThreads = 256;

// The weight code table as floats and the table scale 1.0, where the GEMM expects its codebook
// and table scale.  A launch of its own, one kernel EARLIER than the operand expansion: the GEMM
// starts under programmatic stream serialization and reads its codebook before it waits for
// the kernel directly ahead of it.
__global__ void write_code_table_kernel(const int8_t *w_codes, int w_levels, float *table_scale,
                                        float *w_code_floats) {
  for (int i = threadIdx.x; i < 256; i += blockDim.x) {
    w_code_floats[i] = i < w_levels ? static_cast<float>(w_codes[i]) : 0.0f;
  }
  if (threadIdx.x == 0) {
    *table_scale = 1.0f;
  }
}

// packed_act [rows, dim/2] (low nibble = even k) -> out [rows, dim] f16(code table entry);
// row_scale[m] = token_norms[m] * scale.
__global__ void __launch_bounds__(kExpandThreads)
expand_packed_a4_kernel(const uint8_t *packed_act, const float *token_norms, const int8_t *act_codes,
                        float scale, int64_t rows, int64_t dim, __half *out, float *row_scale) {
  __shared__ uint32_t s_pair[256];   // byte -> the two f16 values of its nibbles
  for (int i = threadIdx.x; i < 256; i += kExpandThreads) {
    const __half lo = __float2half_rn(static_cast<float>(act_codes[i & 15]));
    const __half hi = __float2half_rn(static_cast<float>(act_codes[i >> 4]));
    s_pair[i] = static_cast<uint32_t>(__half_as_ushort(lo)) | (static_cast<uint32_t>(__half_as_ushort(hi)) << 16);
  }
  __syncthreads();
  const int64_t row_bytes = dim / 2;
  const int64_t vectors = rows * row_bytes / 8;   // 8 packed bytes -> 16 values
  for (int64_t v = blockIdx.x * static_cast<int64_t>(kExpandThreads) + threadIdx.x; v < vectors;
       v += static_cast<int64_t>(gridDim.x) * kExpandThreads) {
    const uint2 in = __ldg(reinterpret_cast<const uint2 *>(packed_act) + v);
    const uint32_t w[2] = {in.x, in.y};
    uint32_t o[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      o[q] = s_pair[(w[q >> 2] >> (8 * (q & 3))) & 0xffu];
    }
    uint4 *dst = reinterpret_cast<uint4 *>(out) + 2 * v;
    dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
    dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
  }
  for (int64_t m = blockIdx.x * static_cast<int64_t>(kExpandThreads) + threadIdx.x; m < rows;
       m += static_cast<int64_t>(gridDim.x) * kExpandThreads) {
    row_scale[m] = __fmul_rn(token_norms[m], scale);
  }
}

// packed_act [rows, dim/2] (low nibble = even k) -> out [rows, dim] INT8 code table entries (the
// operand of the kind::i8 tensor-core GEMM); row_scale[m] = token_norms[m] * scale.
__global__ void __launch_bounds__(kExpandThreads)
expand_packed_a4_int8_kernel(const uint8_t *packed_act, const float *token_norms, const int8_t *act_codes,
                             float scale, int64_t rows, int64_t dim, int8_t *out, float *row_scale) {
  __shared__ uint16_t s_pair[256];   // byte -> the two code-table bytes of its nibbles
  for (int i = threadIdx.x; i < 256; i += kExpandThreads) {
    s_pair[i] = static_cast<uint16_t>(static_cast<uint8_t>(act_codes[i & 15])) |
                static_cast<uint16_t>(static_cast<uint16_t>(static_cast<uint8_t>(act_codes[i >> 4])) << 8);
  }
  __syncthreads();
  const int64_t vectors = rows * (dim / 2) / 8;   // 8 packed bytes -> 16 values
  for (int64_t v = blockIdx.x * static_cast<int64_t>(kExpandThreads) + threadIdx.x; v < vectors;
       v += static_cast<int64_t>(gridDim.x) * kExpandThreads) {
    const uint2 in = __ldg(reinterpret_cast<const uint2 *>(packed_act) + v);
    const uint32_t w[2] = {in.x, in.y};
    uint32_t o[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const uint32_t lo = s_pair[(w[q >> 1] >> (16 * (q & 1))) & 0xffu];
      const uint32_t hi = s_pair[(w[q >> 1] >> (16 * (q & 1) + 8)) & 0xffu];
      o[q] = lo | (hi << 16);
    }
    reinterpret_cast<uint4 *>(out)[v] = make_uint4(o[0], o[1], o[2], o[3]);
  }
  for (int64_t m = blockIdx.x * static_cast<int64_t>(kExpandThreads) + threadIdx.x; m < rows;
       m += static_cast<int64_t>(gridDim.x) * kExpandThreads) {
    row_scale[m] = __fmul_rn(token_norms[m], scale);
  }
}

// ---- exact pair-product table ----
constexpr int kLutThreads = 256;
constexpr int kLutCols = 64;      // output features per CTA
constexpr int kLutRows = 16;      // tokens per CTA (4 per thread)
constexpr int kLutChunk = 128;    // k values staged per step

struct PairLutParams {
  void *out;
  int out_dtype;
  const uint8_t *codes;       // [rows, dim] activation indices
  const float *token_norms;   // [rows]
  const uint8_t *packed;      // 4-bit weight stream
  const __nv_bfloat16 *row_norms;
  const float *pair_lut;      // [256]
  const void *bias;
  int bias_dtype;             // -1 none
  int64_t rows;
  int64_t in_features;
  int64_t out_features;
};

__device__ __forceinline__ float lut_load_bias(const void *bias, int dtype, int64_t n) {
  switch (dtype) {
    case OQ_DTYPE_F32: return Scalar<OQ_DTYPE_F32>::load(bias, n);
    case OQ_DTYPE_F16: return Scalar<OQ_DTYPE_F16>::load(bias, n);
    default: return Scalar<OQ_DTYPE_BF16>::load(bias, n);
  }
}

__global__ void __launch_bounds__(kLutThreads) pair_lut_w4a4_kernel(const PairLutParams p) {
  __shared__ float s_lut[256];
  __shared__ uint8_t s_codes[kLutRows][kLutChunk];
  const int col = threadIdx.x & (kLutCols - 1);
  const int rg = threadIdx.x >> 6;                 // row group: tokens 4 rg .. 4 rg + 3
  const int64_t n = static_cast<int64_t>(blockIdx.x) * kLutCols + col;
  const int64_t m0 = static_cast<int64_t>(blockIdx.y) * kLutRows;
  for (int i = threadIdx.x; i < 256; i += kLutThreads) {
    s_lut[i] = p.pair_lut[i];
  }
  const bool col_ok = n < p.out_features;
  const uint8_t *wrow = p.packed + (col_ok ? n : 0) * (p.in_features / 2);
  float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  for (int64_t k0 = 0; k0 < p.in_features; k0 += kLutChunk) {
    const int span = static_cast<int>(min(static_cast<int64_t>(kLutChunk), p.in_features - k0));
    __syncthreads();
    for (int i = threadIdx.x; i < kLutRows * kLutChunk; i += kLutThreads) {
      const int r = i / kLutChunk;
      const int k = i - r * kLutChunk;
      s_codes[r][k] = (m0 + r < p.rows && k < span) ? p.codes[(m0 + r) * p.in_features + k0 + k] : 0;
    }
    __syncthreads();
    if (col_ok) {
      for (int k = 0; k < span; k += 2) {
        const uint32_t byte = wrow[(k0 + k) >> 1];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          if (k + half < span) {
            const uint32_t w = half == 0 ? (byte & 15u) : (byte >> 4);
#pragma unroll
            for (int r = 0; r < 4; ++r) {
              acc[r] = __fadd_rn(acc[r], s_lut[s_codes[4 * rg + r][k + half] * 16u + w]);
            }
          }
        }
      }
    }
  }
  if (!col_ok) {
    return;
  }
  const float rn = __bfloat162float(p.row_norms[n]);
  const float b = p.bias_dtype >= 0 ? lut_load_bias(p.bias, p.bias_dtype, n) : 0.0f;
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int64_t m = m0 + 4 * rg + r;
    if (m < p.rows) {
      float value = __fmul_rn(__fmul_rn(acc[r], p.token_norms[m]), rn);
      if (p.bias_dtype >= 0) {
        value = __fadd_rn(value, b);
      }
      switch (p.out_dtype) {
        case OQ_DTYPE_F32: Scalar<OQ_DTYPE_F32>::store(p.out, m * p.out_features + n, value); break;
        case OQ_DTYPE_F16: Scalar<OQ_DTYPE_F16>::store(p.out, m * p.out_features + n, value); break;
        default: Scalar<OQ_DTYPE_BF16>::store(p.out, m * p.out_features + n, value); break;
      }
    }
  }
}

}  // namespace

int launch_expand_packed_a4(const uint8_t *packed_act, const float *token_norms, const int8_t *act_codes,
                            const int8_t *w_codes, int w_levels, float scale, int64_t rows, int64_t dim,
                            void *out_f16, float *row_scale, float *table_scale, float *w_code_floats,
                            cudaStream_t stream) {
  OQ_CHECK_ARG(dim % 16 == 0, "in_features must be a multiple of 16");
  OQ_CHECK_ARG(aligned16(out_f16) && (reinterpret_cast<uintptr_t>(packed_act) & 7u) == 0,
               "packed activations must be 8-byte aligned, the operand 16-byte aligned");
  const int64_t vectors = rows * dim / 16;
  const unsigned grid = static_cast<unsigned>(std::min<int64_t>((vectors + kExpandThreads - 1) / kExpandThreads, 148 * 16));
  write_code_table_kernel<<<1, 256, 0, stream>>>(w_codes, w_levels, table_scale, w_code_floats);
  OQ_CHECK_CUDA(cudaGetLastError());
  expand_packed_a4_kernel<<<grid > 0 ? grid : 1, kExpandThreads, 0, stream>>>(
      packed_act, token_norms, act_codes, scale, rows, dim, static_cast<__half *>(out_f16), row_scale);
  OQ_CHECK_CUDA(cudaGetLastError());
  count_launch(2);
  return OQ_OK;
}

// As launch_expand_packed_a4, with an INT8 operand [rows, dim] for the kind::i8 GEMM.
// The weight code table as floats (what the GEMM's operand expansion reads) and a table scale
// of 1, for callers that produce the INT8 activation operand themselves.
int launch_write_code_table(const int8_t *w_codes, int w_levels, float *table_scale, float *w_code_floats,
                            cudaStream_t stream) {
  write_code_table_kernel<<<1, 256, 0, stream>>>(w_codes, w_levels, table_scale, w_code_floats);
  OQ_CHECK_CUDA(cudaGetLastError());
  count_launch();
  return OQ_OK;
}

int launch_expand_packed_a4_int8(const uint8_t *packed_act, const float *token_norms, const int8_t *act_codes,
                                 const int8_t *w_codes, int w_levels, float scale, int64_t rows, int64_t dim,
                                 void *out_int8, float *row_scale, float *table_scale, float *w_code_floats,
                                 cudaStream_t stream) {
  OQ_CHECK_ARG(dim % 16 == 0, "in_features must be a multiple of 16");
  OQ_CHECK_ARG(aligned16(out_int8) && (reinterpret_cast<uintptr_t>(packed_act) & 7u) == 0,
               "packed activations must be 8-byte aligned, the operand 16-byte aligned");
  const int64_t vectors = rows * dim / 16;
  const unsigned grid = static_cast<unsigned>(std::min<int64_t>((vectors + kExpandThreads - 1) / kExpandThreads, 148 * 16));
  write_code_table_kernel<<<1, 256, 0, stream>>>(w_codes, w_levels, table_scale, w_code_floats);
  OQ_CHECK_CUDA(cudaGetLastError());
  expand_packed_a4_int8_kernel<<<grid > 0 ? grid : 1, kExpandThreads, 0, stream>>>(
      packed_act, token_norms, act_codes, scale, rows, dim, static_cast<int8_t *>(out_int8), row_scale);
  OQ_CHECK_CUDA(cudaGetLastError());
  count_launch(2);
  return OQ_OK;
}

int launch_pair_lut(void *out, int out_dtype, const uint8_t *codes, const float *token_norms,
                    const uint8_t *packed, const void *row_norms_bf16, const float *pair_lut,
                    const void *bias, int bias_dtype, int64_t rows, int64_t in_features,
                    int64_t out_features, cudaStream_t stream) {
  PairLutParams p{};
  p.out = out;
  p.out_dtype = out_dtype;
  p.codes = codes;
  p.token_norms = token_norms;
  p.packed = packed;
  p.row_norms = static_cast<const __nv_bfloat16 *>(row_norms_bf16);
  p.pair_lut = pair_lut;
  p.bias = bias;
  p.bias_dtype = bias == nullptr ? -1 : bias_dtype;
  p.rows = rows;
  p.in_features = in_features;
  p.out_features = out_features;
  const dim3 grid(static_cast<unsigned>((out_features + kLutCols - 1) / kLutCols),
                  static_cast<unsigned>((rows + kLutRows - 1) / kLutRows));
  OQ_CHECK_ARG(grid.y <= 65535u, "too many rows for the pair-product kernel (at most 1048560)");
  pair_lut_w4a4_kernel<<<grid, kLutThreads, 0, stream>>>(p);
  OQ_CHECK_CUDA(cudaGetLastError());
  count_launch();
  return OQ_OK;
}

}  // namespace oq
