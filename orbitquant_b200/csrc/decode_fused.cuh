// The whole forward of a decode-sized batch in ONE launch: rotate-and-quantize + packed 4-bit
// weight matmul, for rows <= 16 and rows * in_features <= 4096 (one token of up to 4096
// features, four of 1024, ...): beyond that the rotation, which every CTA repeats, costs more
// than the second launch it saves (measured on 768-wide layers: 11.4 against 9.5 us at 4 tokens,
// 17.2 against 10.3 at 16).
//
// At these sizes a layer is a megabyte of weights and the forward is bound by launch and
// dependency latency, not by bytes: two dependent kernels per layer cost more than the
// streaming itself.  Here every CTA owns 8 * nb output features and
//
//   0. asks the L2 for its slice of the packed weights (prefetch; they do not depend on x) and
//      lets the next kernel in the stream start (griddepcontrol.launch_dependents), so that
//      layer i+1's prefetch and table build run under layer i's tail;
//   1. builds the weight table (byte -> two bf16 centroid pairs, high and low part);
//   2. waits for the kernel before it (griddepcontrol.wait: x may be its output);
//   3. rotates and quantises ALL tokens itself -- the same code, order and bits as
//      rotate_quantize_fast_kernel (every CTA repeats this small computation; nothing is
//      exchanged between CTAs and no second launch is needed);
//   4. multiplies: the loop of small_rows_w4_kernel (mma.sync.m16n8k16, tokens as the 16-row
//      operand, bf16 high + low split of the centroid, fp32 accumulation) with the activations
//      read from shared memory;
//   5. reduces across its warps, applies row norm and bias, rounds to bf16.
#pragma once

namespace oq {
namespace {

constexpr int kDfMaxNB = 4;
constexpr int kDfLutRep = 16;
constexpr int kDfKStep = 128;
constexpr float kDfCentroidScale = 256.0f;
constexpr int64_t kDfMaxElements = 4096;    // rows * in_features one CTA rotates by itself

struct DecodeFusedParams {
  PrologueParams pro;
  void *out;
  const uint8_t *packed;
  const __nv_bfloat16 *row_norms;
  const float *w_centroids;
  const void *bias;
  int bias_dtype;   // -1 none
  int64_t out_features;
  int k_steps;
  int nb;           // blocks of 8 output features per CTA
};

__device__ __forceinline__ void df_mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                            uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
      "{%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t df_pack_bf16x2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t *>(&v);
}

__device__ __forceinline__ float df_load_bias(const void *bias, int dtype, int64_t n) {
  switch (dtype) {
    case OQ_DTYPE_F32: return Scalar<OQ_DTYPE_F32>::load(bias, n);
    case OQ_DTYPE_F16: return Scalar<OQ_DTYPE_F16>::load(bias, n);
    default: return Scalar<OQ_DTYPE_BF16>::load(bias, n);
  }
}

__host__ __device__ inline size_t df_prologue_bytes(int dim, int rows, int bits) {
  return static_cast<size_t>(rows) * dim * 6 + (2u << bits) * 4 + 3 * 16 * 4 +
         ((static_cast<size_t>(rows) << bits) * 2 + 15) / 16 * 16 +
         static_cast<size_t>(dim) * 5;   // shared-memory copy of the permutation and the signs
}

inline size_t df_smem_bytes(int dim, int rows, int bits, int nb, bool scaled) {
  return df_prologue_bytes(dim, rows, bits) + (scaled ? 64 : 256 * kDfLutRep * 8) +
         static_cast<size_t>(kFastWarps) * nb * 128 * 4 + 16;
}

template <int BITS, bool SCALED>
__global__ void __launch_bounds__(kFastThreads) decode_fused_kernel(const DecodeFusedParams p) {
  extern __shared__ __align__(16) unsigned char smem[];
  constexpr int kLevels = 1 << BITS;
  const PrologueParams &pp = p.pro;
  const int dim = pp.dim;
  const int rows = static_cast<int>(pp.rows);
  float *rot = reinterpret_cast<float *>(smem);                                        // [rows][dim]
  uint16_t *xin = reinterpret_cast<uint16_t *>(rot + static_cast<size_t>(rows) * dim);  // [rows][dim]
  float *s_bnd = reinterpret_cast<float *>(xin + static_cast<size_t>(rows) * dim);
  float *s_cent = s_bnd + kLevels;
  float *s_norm = s_cent + kLevels;   // [16]
  float *s_inv = s_norm + 16;         // [16]
  float *s_opscale = s_inv + 16;      // [16]
  uint16_t *s_outtab = reinterpret_cast<uint16_t *>(s_opscale + 16);                    // [rows][levels]
  int32_t *s_perm = reinterpret_cast<int32_t *>(
      reinterpret_cast<unsigned char *>(s_outtab) + (((static_cast<size_t>(rows) << BITS) * 2 + 15) / 16 * 16));
  int8_t *s_signs = reinterpret_cast<int8_t *>(s_perm + dim);
  unsigned char *after = smem + ((df_prologue_bytes(dim, rows, BITS) + 15) & ~static_cast<size_t>(15));
  uint2 *s_lut = reinterpret_cast<uint2 *>(after);
  float *s_wcent = reinterpret_cast<float *>(after);
  float *s_red = reinterpret_cast<float *>(after + (SCALED ? 64 : 256 * kDfLutRep * 8));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2;
  const int t = lane & 3;
  const int64_t n0 = static_cast<int64_t>(blockIdx.x) * 8 * p.nb;
  const int64_t row_bytes = static_cast<int64_t>(dim) / 2;

  // 0. this CTA's weight rows on their way into the L2; the next kernel may start
  {
    const int64_t n_end = min(p.out_features, n0 + 8 * p.nb);
    const unsigned char *first = p.packed + n0 * row_bytes;
    const int64_t bytes = n_end > n0 ? (n_end - n0) * row_bytes : 0;
    for (int64_t off = static_cast<int64_t>(threadIdx.x) * 128; off < bytes; off += kFastThreads * 128) {
      asm volatile("prefetch.global.L2 [%0];" ::"l"(first + off));
    }
  }
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // the weights of each warp's first step, loaded while everything else is set up
  uint4 first_wv[kDfMaxNB];
#pragma unroll
  for (int b = 0; b < kDfMaxNB; ++b) {
    const int64_t n = n0 + 8 * b + g;
    first_wv[b] = make_uint4(0, 0, 0, 0);
    if (b < p.nb && n < p.out_features && warp < p.k_steps) {
      first_wv[b] = __ldg(reinterpret_cast<const uint4 *>(p.packed + n * row_bytes + (warp * kDfKStep + 32 * t) / 2));
    }
  }
  // permutation and signs: constants too, copied next to the rows they will index
  for (int i = threadIdx.x; i < dim / 4; i += kFastThreads) {
    reinterpret_cast<int4 *>(s_perm)[i] = __ldg(reinterpret_cast<const int4 *>(pp.perm) + i);
    reinterpret_cast<int32_t *>(s_signs)[i] = __ldg(reinterpret_cast<const int32_t *>(pp.signs) + i);
  }

  // 1. codebooks and the weight table
  for (int i = threadIdx.x; i < kLevels; i += kFastThreads) {
    s_cent[i] = pp.centroids[i];
    s_bnd[i] = i < kLevels - 1 ? pp.boundaries[i] : 0.0f;
  }
  if (SCALED) {
    if (threadIdx.x < 16) {
      s_wcent[threadIdx.x] = p.w_centroids[threadIdx.x];
    }
  } else {
    for (int v = threadIdx.x; v < 256; v += kFastThreads) {
      const float c0 = p.w_centroids[v & 15] * kDfCentroidScale;
      const float c1 = p.w_centroids[v >> 4] * kDfCentroidScale;
      const float h0 = __bfloat162float(__float2bfloat16_rn(c0));
      const float h1 = __bfloat162float(__float2bfloat16_rn(c1));
      const uint2 e = make_uint2(df_pack_bf16x2(h0, h1), df_pack_bf16x2(c0 - h0, c1 - h1));
#pragma unroll
      for (int r = 0; r < kDfLutRep; ++r) {
        s_lut[v * kDfLutRep + r] = e;
      }
    }
  }
  // 2. everything below may read what the kernel before this one wrote
  asm volatile("griddepcontrol.wait;" ::: "memory");
  __syncthreads();

  // 3. rotate and quantise every token (results: bf16 x_q rows in `stage`)
  const bool wide = pp.block > 256;
  uint16_t *stage = wide ? xin : reinterpret_cast<uint16_t *>(rot);
  PrologueParams local = pp;
  local.perm = s_perm;
  local.signs = s_signs;
  fast_rotate_rows<BITS, false>(local, rot, xin, s_cent, reinterpret_cast<const unsigned char *>(s_bnd), s_norm,
                                s_inv, s_opscale, s_outtab, stage, 0, rows, 0, dim >> 8, 1);

  // 4. packed-weight matmul, activations from shared memory
  float acc[kDfMaxNB][4];
#pragma unroll
  for (int b = 0; b < kDfMaxNB; ++b) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      acc[b][i] = 0.0f;
    }
  }
  float rn[kDfMaxNB];
#pragma unroll
  for (int b = 0; b < kDfMaxNB; ++b) {
    const int64_t n = n0 + 8 * b + g;
    rn[b] = (SCALED && b < p.nb && n < p.out_features) ? __bfloat162float(p.row_norms[n]) : 0.0f;
  }
  const uint2 *lut = s_lut + (lane & (kDfLutRep - 1));
  for (int j = warp; j < p.k_steps; j += kFastWarps) {
    const int k0 = j * kDfKStep + 32 * t;
    uint4 xa[4];
    uint4 xb[4];
    {
      const uint4 zero = make_uint4(0, 0, 0, 0);
      const uint4 *ra = reinterpret_cast<const uint4 *>(stage + g * dim + k0);
      const uint4 *rb = reinterpret_cast<const uint4 *>(stage + (g + 8) * dim + k0);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        xa[q] = g < rows ? ra[q] : zero;
        xb[q] = g + 8 < rows ? rb[q] : zero;
      }
    }
#pragma unroll
    for (int b = 0; b < kDfMaxNB; ++b) {
      if (b < p.nb) {
        const int64_t n = n0 + 8 * b + g;
        uint4 wv = first_wv[b];
        if (j != warp) {
          wv = make_uint4(0, 0, 0, 0);
          if (n < p.out_features) {
            wv = __ldg(reinterpret_cast<const uint4 *>(p.packed + n * row_bytes + k0 / 2));
          }
        }
        const uint32_t words[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const uint32_t pair = (words[i >> 1] >> ((i & 1) * 16)) & 0xffffu;  // bytes 2i, 2i+1
          const uint4 a_lo = xa[i >> 1];
          const uint4 a_hi = xb[i >> 1];
          const uint32_t a0 = (i & 1) ? a_lo.z : a_lo.x;
          const uint32_t a2 = (i & 1) ? a_lo.w : a_lo.y;
          const uint32_t a1 = (i & 1) ? a_hi.z : a_hi.x;
          const uint32_t a3 = (i & 1) ? a_hi.w : a_hi.y;
          if (SCALED) {
            const float w0 = __fmul_rn(s_wcent[pair & 15u], rn[b]);
            const float w1 = __fmul_rn(s_wcent[(pair >> 4) & 15u], rn[b]);
            const float w2 = __fmul_rn(s_wcent[(pair >> 8) & 15u], rn[b]);
            const float w3 = __fmul_rn(s_wcent[pair >> 12], rn[b]);
            df_mma_bf16(acc[b], a0, a1, a2, a3, df_pack_bf16x2(w0, w1), df_pack_bf16x2(w2, w3));
          } else {
            const uint2 e0 = lut[(pair & 0xffu) * kDfLutRep];
            const uint2 e1 = lut[(pair >> 8) * kDfLutRep];
            df_mma_bf16(acc[b], a0, a1, a2, a3, e0.x, e1.x);
            df_mma_bf16(acc[b], a0, a1, a2, a3, e0.y, e1.y);
          }
        }
      }
    }
  }

  // 5. cross-warp reduction: s_red[warp][nb][row 0..15][col 0..7]
#pragma unroll
  for (int b = 0; b < kDfMaxNB; ++b) {
    if (b < p.nb) {
      float *dst = s_red + ((warp * p.nb + b) * 16) * 8;
      dst[g * 8 + 2 * t] = acc[b][0];
      dst[g * 8 + 2 * t + 1] = acc[b][1];
      dst[(g + 8) * 8 + 2 * t] = acc[b][2];
      dst[(g + 8) * 8 + 2 * t + 1] = acc[b][3];
    }
  }
  __syncthreads();
  const int outputs = p.nb * 128;
  for (int o = threadIdx.x; o < outputs; o += kFastThreads) {
    const int b = o >> 7;
    const int row = (o >> 3) & 15;
    const int col = o & 7;
    const int64_t n = n0 + 8 * b + col;
    if (row >= rows || n >= p.out_features) {
      continue;
    }
    float sum = 0.0f;
    for (int w = 0; w < kFastWarps; ++w) {
      sum += s_red[((w * p.nb + b) * 16 + row) * 8 + col];
    }
    if (!SCALED) {
      sum *= __bfloat162float(p.row_norms[n]) * (1.0f / kDfCentroidScale);
    }
    if (p.bias_dtype >= 0) {
      sum += df_load_bias(p.bias, p.bias_dtype, n);
    }
    static_cast<__nv_bfloat16 *>(p.out)[static_cast<int64_t>(row) * p.out_features + n] = __float2bfloat16_rn(sum);
  }
}

template <bool SCALED>
void (*decode_fused_for(int bits))(DecodeFusedParams) {
  switch (bits) {
    case 2: return decode_fused_kernel<2, SCALED>;
    case 3: return decode_fused_kernel<3, SCALED>;
    case 4: return decode_fused_kernel<4, SCALED>;
    case 6: return decode_fused_kernel<6, SCALED>;
    case 8: return decode_fused_kernel<8, SCALED>;
    default: return nullptr;
  }
}

}  // namespace

bool decode_fused_supported(int64_t rows, int64_t in_features, int64_t out_features, int weight_bits,
                            int act_bits, int dtype, int64_t block) {
  const bool bits_ok = act_bits == 2 || act_bits == 3 || act_bits == 4 || act_bits == 6 || act_bits == 8;
  return rows >= 1 && rows <= 16 && weight_bits == 4 && bits_ok && dtype == OQ_DTYPE_BF16 &&
         out_features >= 1 && in_features % 256 == 0 && block >= 256 && (block & (block - 1)) == 0 &&
         in_features % block == 0 && rows * in_features <= kDfMaxElements;
}

int launch_decode_fused(void *out, const void *x, int64_t rows, int64_t in_features, int64_t out_features,
                        const uint8_t *packed, const void *row_norms_bf16, const float *w_centroids,
                        const void *bias, int bias_dtype, const int32_t *perm, const int8_t *signs,
                        int64_t block, const float *act_boundaries, const float *act_centroids,
                        int act_bits, float eps, int weight_mode, cudaStream_t stream) {
  OQ_CHECK_ARG(aligned16(x) && aligned16(packed) && aligned16(perm) &&
                   (reinterpret_cast<uintptr_t>(signs) & 7u) == 0,
               "x, packed weights and perm must be 16-byte aligned, signs 8-byte aligned");
  OQ_CHECK_ARG(eps >= 0.0f, "eps must be non-negative");
  int device = 0;
  int sm_count = 0;
  int max_smem = 0;
  OQ_CHECK_CUDA(cudaGetDevice(&device));
  OQ_CHECK_CUDA(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device));
  OQ_CHECK_CUDA(cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, device));
  DecodeFusedParams p{};
  p.pro.x = x;
  p.pro.perm = perm;
  p.pro.signs = signs;
  p.pro.boundaries = act_boundaries;
  p.pro.centroids = act_centroids;
  p.pro.rows = rows;
  p.pro.dim = static_cast<int>(in_features);
  p.pro.block = static_cast<int>(block);
  p.pro.bits = act_bits;
  p.pro.rows_per_cta = static_cast<int>(rows);
  p.pro.eps = eps;
  p.pro.inv_sqrt_block = static_cast<float>(1.0 / sqrt(static_cast<double>(block)));
  p.pro.slices = 1;
  p.out = out;
  p.packed = packed;
  p.row_norms = static_cast<const __nv_bfloat16 *>(row_norms_bf16);
  p.w_centroids = w_centroids;
  p.bias = bias;
  p.bias_dtype = bias == nullptr ? -1 : bias_dtype;
  p.out_features = out_features;
  p.k_steps = static_cast<int>(in_features / kDfKStep);
  // output features per CTA: the fewest that keep the grid within two CTAs per SM (every CTA
  // repeats the rotation, so more CTAs than that only add work)
  int nb = 1;
  while (nb < kDfMaxNB && (out_features + 8 * nb - 1) / (8 * nb) > 2 * static_cast<int64_t>(sm_count)) {
    nb *= 2;
  }
  p.nb = nb;
  const bool scaled = weight_mode == OQ_WEIGHT_BF16_SCALED;
  const size_t smem = df_smem_bytes(p.pro.dim, static_cast<int>(rows), act_bits, nb, scaled);
  OQ_CHECK_ARG(smem <= static_cast<size_t>(max_smem), "the fused decode kernel needs %zu bytes of shared memory", smem);
  void (*kernel)(DecodeFusedParams) = scaled ? decode_fused_for<true>(act_bits) : decode_fused_for<false>(act_bits);
  OQ_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(static_cast<unsigned>((out_features + 8 * nb - 1) / (8 * nb)));
  config.blockDim = dim3(kFastThreads);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attr;
  config.numAttrs = 1;
  OQ_CHECK_CUDA(cudaLaunchKernelEx(&config, kernel, p));
  count_launch();
  return OQ_OK;
}

}  // namespace oq
