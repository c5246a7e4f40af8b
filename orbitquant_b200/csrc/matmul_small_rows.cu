// Packed 4-bit weight matmul for decode-sized batches (rows <= 16): weight streaming.
//
// Every packed weight byte is read from HBM exactly once; the activations (at most
// 16 x in_features bf16) stay in L1/L2.  A CTA owns 8*NB consecutive output features and
// its warps split the reduction dimension in interleaved 128-wide steps, so even a
// 768 -> 2304 layer spreads over hundreds of CTAs.  Per step a lane loads 16 packed bytes
// of "its" weight row (lanes 4g..4g+3 cover 64 contiguous bytes of row g), expands them
// through a shared-memory table and feeds mma.sync.m16n8k16 with the 16 (zero-padded)
// activation rows as the A operand.  The MMA's k slots are a free permutation of the
// reduction index, chosen here so that a lane's 4 slots are 4 consecutive k -- exactly
// what one packed 16-bit pair of bytes and one 8-byte activation load provide.
//
// Weight arithmetic:
//   centroid mode: centroid*2^8 is split into bf16 hi + bf16 lo (two MMAs, 16 mantissa
//                  bits), the sum is scaled by row_norm*2^-8 afterwards;
//   scaled mode:   the operand is bf16(centroid*row_norm), one MMA.
// The per-warp partial sums meet in shared memory; the epilogue adds the bias and rounds.
#include "common.cuh"

namespace oq {
namespace {

constexpr int kMaxWarps = 8;
constexpr int kKStep = 128;
constexpr int kLutRep = 16;
constexpr int kMaxNB = 4;
constexpr float kCentroidScale = 256.0f;

struct SmallRowsParams {
  void *out;
  const __nv_bfloat16 *x;
  const uint8_t *packed;
  const __nv_bfloat16 *row_norms;
  const float *centroids;
  const void *bias;
  int bias_dtype;
  int rows;
  int64_t in_features;
  int64_t out_features;
  int k_steps;
  int nb;  // n-blocks of 8 output features per CTA
};

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
      "{%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t *>(&v);
}

__device__ __forceinline__ float load_bias(const void *bias, int dtype, int64_t n) {
  switch (dtype) {
    case OQ_DTYPE_F32: return Scalar<OQ_DTYPE_F32>::load(bias, n);
    case OQ_DTYPE_F16: return Scalar<OQ_DTYPE_F16>::load(bias, n);
    default: return Scalar<OQ_DTYPE_BF16>::load(bias, n);
  }
}

template <bool SCALED>
__global__ void __launch_bounds__(kMaxWarps * 32) small_rows_w4_kernel(const SmallRowsParams p) {
  // centroid mode: byte -> {hi pair, lo pair} as uint2, replicated kLutRep times (32 KB);
  // scaled mode:   16 fp32 centroids.
  extern __shared__ __align__(16) unsigned char smem[];
  uint2 *s_lut = reinterpret_cast<uint2 *>(smem);
  float *s_cent = reinterpret_cast<float *>(smem);
  float *s_red = reinterpret_cast<float *>(smem + (SCALED ? 64 : 256 * kLutRep * 8));

  const int warps = blockDim.x >> 5;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2;
  const int t = lane & 3;
  const int64_t n0 = static_cast<int64_t>(blockIdx.x) * 8 * p.nb;

  // This CTA's weight rows on their way into the L2 (they do not depend on the kernel before
  // this one, whose tail this kernel's start overlaps): with the weights cold in HBM their
  // latency would otherwise sit between the dependency wait and the first MMA.
  {
    const int64_t prefetch_row_bytes = p.in_features / 2;
    const int64_t n_end = min(p.out_features, n0 + 8 * static_cast<int64_t>(p.nb));
    const unsigned char *first = reinterpret_cast<const unsigned char *>(p.packed) + n0 * prefetch_row_bytes;
    const int64_t bytes = n_end > n0 ? (n_end - n0) * prefetch_row_bytes : 0;
    for (int64_t off = static_cast<int64_t>(threadIdx.x) * 128; off < bytes;
         off += static_cast<int64_t>(blockDim.x) * 128) {
      asm volatile("prefetch.global.L2 [%0];" ::"l"(first + off));
    }
    // the epilogue's per-column operands likewise (one line each covers this CTA's columns)
    if (threadIdx.x == 0 && n0 < p.out_features) {
      asm volatile("prefetch.global.L2 [%0];" ::"l"(p.row_norms + n0));
      if (p.bias_dtype >= 0) {
        asm volatile("prefetch.global.L2 [%0];" ::"l"(static_cast<const unsigned char *>(p.bias) +
                                                       n0 * (p.bias_dtype == OQ_DTYPE_F32 ? 4 : 2)));
      }
    }
  }

  // the next kernel in the stream (the next layer's prologue) may start its own prefetches
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (SCALED) {
    if (threadIdx.x < 16) {
      s_cent[threadIdx.x] = p.centroids[threadIdx.x];
    }
  } else {
    for (int v = threadIdx.x; v < 256; v += blockDim.x) {
      const float c0 = p.centroids[v & 15] * kCentroidScale;
      const float c1 = p.centroids[v >> 4] * kCentroidScale;
      const float h0 = __bfloat162float(__float2bfloat16_rn(c0));
      const float h1 = __bfloat162float(__float2bfloat16_rn(c1));
      const uint2 e = make_uint2(pack_bf16x2(h0, h1), pack_bf16x2(c0 - h0, c1 - h1));
#pragma unroll
      for (int r = 0; r < kLutRep; ++r) {
        s_lut[v * kLutRep + r] = e;
      }
    }
  }
  __syncthreads();
  // Launched with programmatic stream serialization: the table above was built while the
  // kernel that produces the activations was still running; its output is read from here on.
  asm volatile("griddepcontrol.wait;" ::: "memory");

  float acc[kMaxNB][4];
#pragma unroll
  for (int b = 0; b < kMaxNB; ++b) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      acc[b][i] = 0.0f;
    }
  }
  float rn[kMaxNB];
#pragma unroll
  for (int b = 0; b < kMaxNB; ++b) {
    const int64_t n = n0 + 8 * b + g;
    rn[b] = (SCALED && b < p.nb && n < p.out_features) ? __bfloat162float(p.row_norms[n]) : 0.0f;
  }

  const int64_t row_bytes = p.in_features / 2;
  const uint2 *lut = s_lut + (lane & (kLutRep - 1));
  for (int j = warp; j < p.k_steps; j += warps) {
    const int64_t k0 = static_cast<int64_t>(j) * kKStep + 32 * t;
    // A fragments: activation rows g and g+8, 32 consecutive k each.
    uint4 xa[4];
    uint4 xb[4];
    {
      const uint4 zero = make_uint4(0, 0, 0, 0);
      const uint4 *ra = reinterpret_cast<const uint4 *>(p.x + static_cast<int64_t>(g) * p.in_features + k0);
      const uint4 *rb = reinterpret_cast<const uint4 *>(p.x + static_cast<int64_t>(g + 8) * p.in_features + k0);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        xa[q] = g < p.rows ? __ldg(ra + q) : zero;
        xb[q] = g + 8 < p.rows ? __ldg(rb + q) : zero;
      }
    }
#pragma unroll
    for (int b = 0; b < kMaxNB; ++b) {
      if (b < p.nb) {
        const int64_t n = n0 + 8 * b + g;
        uint4 wv = make_uint4(0, 0, 0, 0);
        if (n < p.out_features) {
          wv = __ldg(reinterpret_cast<const uint4 *>(p.packed + n * row_bytes + k0 / 2));
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
            const float w0 = __fmul_rn(s_cent[pair & 15u], rn[b]);
            const float w1 = __fmul_rn(s_cent[(pair >> 4) & 15u], rn[b]);
            const float w2 = __fmul_rn(s_cent[(pair >> 8) & 15u], rn[b]);
            const float w3 = __fmul_rn(s_cent[pair >> 12], rn[b]);
            mma_bf16(acc[b], a0, a1, a2, a3, pack_bf16x2(w0, w1), pack_bf16x2(w2, w3));
          } else {
            const uint2 e0 = lut[(pair & 0xffu) * kLutRep];
            const uint2 e1 = lut[(pair >> 8) * kLutRep];
            mma_bf16(acc[b], a0, a1, a2, a3, e0.x, e1.x);
            mma_bf16(acc[b], a0, a1, a2, a3, e0.y, e1.y);
          }
        }
      }
    }
  }

  // Cross-warp reduction: s_red[warp][nb][row 0..15][col 0..7].
#pragma unroll
  for (int b = 0; b < kMaxNB; ++b) {
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
  for (int o = threadIdx.x; o < outputs; o += blockDim.x) {
    const int b = o >> 7;
    const int row = (o >> 3) & 15;
    const int col = o & 7;
    const int64_t n = n0 + 8 * b + col;
    if (row >= p.rows || n >= p.out_features) {
      continue;
    }
    float sum = 0.0f;
    for (int w = 0; w < warps; ++w) {
      sum += s_red[((w * p.nb + b) * 16 + row) * 8 + col];
    }
    if (!SCALED) {
      sum *= __bfloat162float(p.row_norms[n]) * (1.0f / kCentroidScale);
    }
    if (p.bias_dtype >= 0) {
      sum += load_bias(p.bias, p.bias_dtype, n);
    }
    static_cast<__nv_bfloat16 *>(p.out)[static_cast<int64_t>(row) * p.out_features + n] =
        __float2bfloat16_rn(sum);
  }
}

}  // namespace

bool small_rows_supported(int64_t rows, int64_t in_features, int64_t out_features, int bits,
                          int dtype, int weight_mode) {
  (void)weight_mode;
  return rows >= 1 && rows <= 16 && bits == 4 && dtype == OQ_DTYPE_BF16 && out_features >= 1 &&
         in_features >= kKStep && in_features % kKStep == 0;
}

int launch_small_rows(void *out, const void *x, int dtype, int64_t rows, int64_t in_features,
                      int64_t out_features, const uint8_t *packed, int bits,
                      const void *row_norms_bf16, const float *centroids, const void *bias,
                      int bias_dtype, int weight_mode, cudaStream_t stream) {
  (void)dtype;
  (void)bits;
  OQ_CHECK_ARG(aligned16(x) && aligned16(packed),
               "x and packed weights must be 16-byte aligned for the small-rows kernel");
  int device = 0;
  int sm_count = 0;
  OQ_CHECK_CUDA(cudaGetDevice(&device));
  OQ_CHECK_CUDA(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device));

  SmallRowsParams p{};
  p.out = out;
  p.x = static_cast<const __nv_bfloat16 *>(x);
  p.packed = packed;
  p.row_norms = static_cast<const __nv_bfloat16 *>(row_norms_bf16);
  p.centroids = centroids;
  p.bias = bias;
  p.bias_dtype = bias == nullptr ? -1 : bias_dtype;
  p.rows = static_cast<int>(rows);
  p.in_features = in_features;
  p.out_features = out_features;
  p.k_steps = static_cast<int>(in_features / kKStep);
  // Output features per CTA: as many as keep at least ~2 CTAs per SM in flight.
  int nb = 1;
  while (nb < kMaxNB && (out_features + 8 * (2 * nb) - 1) / (8 * (2 * nb)) >= 2 * sm_count) {
    nb *= 2;
  }
  p.nb = nb;
  const int warps = std::min(kMaxWarps, p.k_steps);
  const int grid = static_cast<int>((out_features + 8 * nb - 1) / (8 * nb));
  const bool scaled = weight_mode == OQ_WEIGHT_BF16_SCALED;
  const size_t smem = (scaled ? 64 : 256 * kLutRep * 8) + static_cast<size_t>(warps) * nb * 128 * 4;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(grid);
  config.blockDim = dim3(warps * 32);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attr;
  config.numAttrs = 1;
  if (scaled) {
    OQ_CHECK_CUDA(cudaLaunchKernelEx(&config, small_rows_w4_kernel<true>, p));
  } else {
    OQ_CHECK_CUDA(cudaLaunchKernelEx(&config, small_rows_w4_kernel<false>, p));
  }
  OQ_CHECK_CUDA(cudaGetLastError());
  count_launch();
  return OQ_OK;
}

}  // namespace oq
