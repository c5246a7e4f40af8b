// Packed 4-bit weight matmul for decode-sized batches (rows <= 16) on LARGE layers: a
// persistent weight-streaming kernel.
//
// The small-rows kernel in matmul_small_rows.cu gives every CTA one short dependent chain,
// which is right for layers of a megabyte (launch latency dominates) and wrong for layers of
// tens of megabytes: HBM only delivers its bandwidth with tens of kilobytes in flight per SM.
// Here one CTA per SM stays resident and
//   * stages the activations of its current k range ONCE in shared memory (laid out so that
//     an MMA A-fragment is one conflict-free 16-byte read), instead of every CTA re-reading
//     them from L2 for every 8 weight rows;
//   * gives each warp whole units -- 8 weight rows x one k range -- and keeps kDepth 16-byte
//     weight loads per lane in flight ahead of the MMAs (a register ring), so that the 8
//     warps of an SM hold ~40 KB of HBM reads outstanding;
//   * decodes through the same lane-replicated byte table and feeds mma.sync.m16n8k16 with
//     the k slots permuted so that a lane's four slots are four consecutive k.
// When the layer has too few 8-row units to occupy the machine (or K exceeds the staging
// buffer) the reduction dimension is split; each split writes fp32 partial sums to the
// caller's workspace and a second small kernel adds them in a fixed order, scales, adds the
// bias and rounds -- deterministic, no atomics.
#include <algorithm>
#include <mutex>

#include "common.cuh"

namespace oq {
namespace {

constexpr int kThreads = 512;
constexpr int kWarps = 16;
constexpr int kKStep = 128;
constexpr int kLutRep = 16;
constexpr int kDepth = 8;             // weight loads in flight per lane
constexpr int kMaxChunk = 4096;       // k range staged at once (16 x 4096 bf16 = 128 KB)
constexpr float kCentroidScale = 256.0f;

struct StreamParams {
  void *out;
  float *partial;  // [splits][16][out_features] when splits > 1
  const __nv_bfloat16 *x;
  const uint8_t *packed;
  const __nv_bfloat16 *row_norms;
  const float *centroids;
  const void *bias;
  int bias_dtype;
  int rows;
  int64_t in_features;
  int64_t out_features;
  int n_blocks;     // ceil(out_features / 8)
  int splits;       // k ranges
  int chunk;        // length of a k range (multiple of 128), the last one may be shorter
  int scaled;       // 1: operand bf16(centroid * row_norm)
};

__device__ __forceinline__ uint4 ld_stream(const uint4 *ptr) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(ptr));
  return v;
}

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
__global__ void __launch_bounds__(kThreads, 1) stream_rows_w4_kernel(const StreamParams p) {
  extern __shared__ __align__(16) unsigned char smem[];
  uint2 *s_lut = reinterpret_cast<uint2 *>(smem);                       // [256][kLutRep]
  float *s_cent = reinterpret_cast<float *>(smem + 256 * kLutRep * 8);  // [16]
  // activations of the current k range: [k step][q 0..3][row 0..15][t 0..3] 16-byte pieces,
  // piece (j, q, row, t) = x[row][k0 + 128 j + 32 t + 8 q .. + 8)
  uint4 *s_act = reinterpret_cast<uint4 *>(smem + 256 * kLutRep * 8 + 64);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2;
  const int t = lane & 3;

  if (threadIdx.x < 16) {
    s_cent[threadIdx.x] = p.centroids[threadIdx.x];
  }
  for (int v = threadIdx.x; v < 256; v += kThreads) {
    const float c0 = p.centroids[v & 15] * kCentroidScale;
    const float c1 = p.centroids[v >> 4] * kCentroidScale;
    const float h0 = __bfloat162float(__float2bfloat16_rn(c0));
    const float h1 = __bfloat162float(__float2bfloat16_rn(c1));
    const uint2 e = make_uint2(pack_bf16x2(h0, h1), pack_bf16x2(c0 - h0, c1 - h1));
    const uint4 e2 = make_uint4(e.x, e.y, e.x, e.y);
    uint4 *dst = reinterpret_cast<uint4 *>(s_lut + v * kLutRep);
#pragma unroll
    for (int r = 0; r < kLutRep / 2; ++r) {
      dst[r] = e2;
    }
  }

  // Units are (k range, 8-row block), k range major; every CTA takes a contiguous share.
  const int64_t total = static_cast<int64_t>(p.splits) * p.n_blocks;
  const int64_t u_begin = total * blockIdx.x / gridDim.x;
  const int64_t u_end = total * (blockIdx.x + 1) / gridDim.x;
  const int64_t row_bytes = p.in_features / 2;
  const uint2 *lut = s_lut + (lane & (kLutRep - 1));

  int64_t u = u_begin;
  while (u < u_end) {
    const int split = static_cast<int>(u / p.n_blocks);
    const int64_t split_end = std::min<int64_t>(u_end, static_cast<int64_t>(split + 1) * p.n_blocks);
    const int64_t k_begin = static_cast<int64_t>(split) * p.chunk;
    const int k_len = static_cast<int>(std::min<int64_t>(p.chunk, p.in_features - k_begin));
    const int steps = k_len / kKStep;

    __syncthreads();  // everyone is done with the previous k range (and the tables are built)
    for (int i = threadIdx.x; i < 16 * (k_len / 8); i += kThreads) {
      const int row = i / (k_len / 8);
      const int piece = i - row * (k_len / 8);  // 8-value piece index inside the k range
      const int j = piece >> 4;
      const int tt = (piece >> 2) & 3;
      const int q = piece & 3;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (row < p.rows) {
        v = __ldg(reinterpret_cast<const uint4 *>(p.x + static_cast<int64_t>(row) * p.in_features + k_begin) + piece);
      }
      s_act[((j * 4 + q) * 16 + row) * 4 + tt] = v;
    }
    __syncthreads();

    for (int64_t unit = u + warp; unit < split_end; unit += kWarps) {
      const int nb = static_cast<int>(unit - static_cast<int64_t>(split) * p.n_blocks);
      const int64_t n = static_cast<int64_t>(nb) * 8 + g;  // this lane's weight row
      const bool n_ok = n < p.out_features;
      const uint4 *wptr = reinterpret_cast<const uint4 *>(p.packed + (n_ok ? n : 0) * row_bytes + k_begin / 2) + t;
      const float rn = (SCALED && n_ok) ? __bfloat162float(p.row_norms[n]) : 0.0f;
      // four independent accumulation chains (an mma.sync on the accumulator it just wrote
      // waits out the whole pipeline latency); summed in a fixed order at the end
      float acc4[4][4] = {};
      uint4 ring[kDepth];
#pragma unroll
      for (int d = 0; d < kDepth; ++d) {
        ring[d] = (n_ok && d < steps) ? ld_stream(wptr + 4 * d) : make_uint4(0, 0, 0, 0);
      }
      for (int j0 = 0; j0 < steps; j0 += kDepth) {
#pragma unroll
        for (int d = 0; d < kDepth; ++d) {
          const int j = j0 + d;
          if (j < steps) {
            const uint4 wv = ring[d];
            if (n_ok && j + kDepth < steps) {
              ring[d] = ld_stream(wptr + 4 * (j + kDepth));
            }
            const uint4 *frag = s_act + (j * 4 * 16 + g) * 4 + t;
            const uint32_t words[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const uint4 a_lo = frag[q * 64];        // row g
              const uint4 a_hi = frag[q * 64 + 32];   // row g + 8
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                const uint32_t pair = (words[q] >> (16 * h)) & 0xffffu;  // bytes 2i, 2i+1 (i = 2q+h)
                const uint32_t a0 = h ? a_lo.z : a_lo.x;
                const uint32_t a2 = h ? a_lo.w : a_lo.y;
                const uint32_t a1 = h ? a_hi.z : a_hi.x;
                const uint32_t a3 = h ? a_hi.w : a_hi.y;
                if (SCALED) {
                  const float w0 = __fmul_rn(s_cent[pair & 15u], rn);
                  const float w1 = __fmul_rn(s_cent[(pair >> 4) & 15u], rn);
                  const float w2 = __fmul_rn(s_cent[(pair >> 8) & 15u], rn);
                  const float w3 = __fmul_rn(s_cent[pair >> 12], rn);
                  mma_bf16(acc4[2 * (q & 1) + h], a0, a1, a2, a3, pack_bf16x2(w0, w1), pack_bf16x2(w2, w3));
                } else {
                  const uint2 e0 = lut[(pair & 0xffu) * kLutRep];
                  const uint2 e1 = lut[(pair >> 8) * kLutRep];
                  mma_bf16(acc4[h], a0, a1, a2, a3, e0.x, e1.x);
                  mma_bf16(acc4[2 + h], a0, a1, a2, a3, e0.y, e1.y);
                }
              }
            }
          }
        }
      }
      float acc[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        acc[e] = (acc4[0][e] + acc4[1][e]) + (acc4[2][e] + acc4[3][e]);
      }
      // acc[0..1]: token g, features 2t, 2t+1 of the block; acc[2..3]: token g + 8.
      const int64_t col = static_cast<int64_t>(nb) * 8 + 2 * t;
      if (p.splits > 1) {
        float *dst = p.partial + (static_cast<int64_t>(split) * 16) * p.out_features;
        if (col < p.out_features) {
          dst[static_cast<int64_t>(g) * p.out_features + col] = acc[0];
          dst[static_cast<int64_t>(g + 8) * p.out_features + col] = acc[2];
        }
        if (col + 1 < p.out_features) {
          dst[static_cast<int64_t>(g) * p.out_features + col + 1] = acc[1];
          dst[static_cast<int64_t>(g + 8) * p.out_features + col + 1] = acc[3];
        }
      } else {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int64_t c = col + e;
          if (c < p.out_features) {
            const float scale = SCALED ? 1.0f : __bfloat162float(p.row_norms[c]) * (1.0f / kCentroidScale);
            const float b = p.bias_dtype >= 0 ? load_bias(p.bias, p.bias_dtype, c) : 0.0f;
            __nv_bfloat16 *o = static_cast<__nv_bfloat16 *>(p.out);
            if (g < p.rows) {
              o[static_cast<int64_t>(g) * p.out_features + c] = __float2bfloat16_rn(fmaf(acc[e], scale, b));
            }
            if (g + 8 < p.rows) {
              o[static_cast<int64_t>(g + 8) * p.out_features + c] = __float2bfloat16_rn(fmaf(acc[2 + e], scale, b));
            }
          }
        }
      }
    }
    u = split_end;
  }
}

// Adds the per-range partial sums in range order, scales, adds the bias, rounds.
template <bool SCALED>
__global__ void stream_rows_finish_kernel(const StreamParams p) {
  const int64_t total = static_cast<int64_t>(p.rows) * p.out_features;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t row = i / p.out_features;
    const int64_t c = i - row * p.out_features;
    float sum = 0.0f;
    for (int s = 0; s < p.splits; ++s) {
      sum += p.partial[(static_cast<int64_t>(s) * 16 + row) * p.out_features + c];
    }
    const float scale = SCALED ? 1.0f : __bfloat162float(p.row_norms[c]) * (1.0f / kCentroidScale);
    const float b = p.bias_dtype >= 0 ? load_bias(p.bias, p.bias_dtype, c) : 0.0f;
    static_cast<__nv_bfloat16 *>(p.out)[i] = __float2bfloat16_rn(fmaf(sum, scale, b));
  }
}

struct Plan {
  int splits;
  int chunk;
};

Plan plan_for(int64_t in_features, int64_t out_features, int sm_count) {
  const int steps = static_cast<int>(in_features / kKStep);
  const int n_blocks = static_cast<int>((out_features + 7) / 8);
  int splits = (static_cast<int>(in_features) + kMaxChunk - 1) / kMaxChunk;
  // enough units for every warp of the machine to get at least one
  const int wanted = sm_count * kWarps;
  while (splits * n_blocks < wanted && splits * 2 <= steps) {
    splits *= 2;
  }
  int chunk_steps = (steps + splits - 1) / splits;
  Plan plan;
  plan.chunk = chunk_steps * kKStep;
  plan.splits = (steps + chunk_steps - 1) / chunk_steps;
  return plan;
}

int sm_count_of_current_device(int *count) {
  int device = 0;
  OQ_CHECK_CUDA(cudaGetDevice(&device));
  OQ_CHECK_CUDA(cudaDeviceGetAttribute(count, cudaDevAttrMultiProcessorCount, device));
  return OQ_OK;
}

}  // namespace

// Worth it once the packed weights are a few megabytes; below that the single-launch
// small-rows kernel has the lower latency.
bool stream_rows_preferred(int64_t rows, int64_t in_features, int64_t out_features, int bits, int dtype) {
  return rows >= 1 && rows <= 16 && bits == 4 && dtype == OQ_DTYPE_BF16 && in_features % kKStep == 0 &&
         in_features >= kKStep && out_features * in_features / 2 >= (int64_t(3) << 20);
}

size_t stream_rows_workspace_bytes(int64_t in_features, int64_t out_features) {
  // Sized for the B200's 148 SMs or fewer: the plan only splits further on larger parts.
  const Plan plan = plan_for(in_features, out_features, 148);
  const Plan wide = plan_for(in_features, out_features, 512);
  const int splits = std::max(plan.splits, wide.splits);
  return splits > 1 ? static_cast<size_t>(splits) * 16 * out_features * sizeof(float) : 0;
}

int launch_stream_rows(void *out, const void *x, int64_t rows, int64_t in_features,
                       int64_t out_features, const uint8_t *packed, const void *row_norms_bf16,
                       const float *centroids, const void *bias, int bias_dtype, int weight_mode,
                       void *workspace, size_t workspace_bytes, cudaStream_t stream) {
  OQ_CHECK_ARG(aligned16(x) && aligned16(packed),
               "x and packed weights must be 16-byte aligned for the streaming kernel");
  int sm_count = 0;
  if (int rc = sm_count_of_current_device(&sm_count)) {
    return rc;
  }
  const Plan plan = plan_for(in_features, out_features, sm_count);
  StreamParams p{};
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
  p.n_blocks = static_cast<int>((out_features + 7) / 8);
  p.splits = plan.splits;
  p.chunk = plan.chunk;
  p.scaled = weight_mode == OQ_WEIGHT_BF16_SCALED ? 1 : 0;
  if (plan.splits > 1) {
    const size_t need = static_cast<size_t>(plan.splits) * 16 * out_features * sizeof(float);
    if (workspace == nullptr || workspace_bytes < need) {
      return fail(OQ_ERR_WORKSPACE, "workspace of %zu bytes given, %zu needed", workspace_bytes, need);
    }
    OQ_CHECK_ARG(aligned16(workspace), "workspace must be 16-byte aligned");
    p.partial = static_cast<float *>(workspace);
  }
  const size_t smem = 256 * kLutRep * 8 + 64 + static_cast<size_t>(16) * plan.chunk * 2;
  const bool scaled = p.scaled != 0;
  auto kernel = scaled ? stream_rows_w4_kernel<true> : stream_rows_w4_kernel<false>;
  static std::once_flag once[2];
  static cudaError_t status[2] = {cudaSuccess, cudaSuccess};
  std::call_once(once[scaled ? 1 : 0], [&] {
    status[scaled ? 1 : 0] = cudaFuncSetAttribute(
        kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
        static_cast<int>(256 * kLutRep * 8 + 64 + 16 * kMaxChunk * 2));
  });
  OQ_CHECK_CUDA(status[scaled ? 1 : 0]);
  const int64_t total = static_cast<int64_t>(p.splits) * p.n_blocks;
  const int grid = static_cast<int>(std::min<int64_t>(sm_count, (total + kWarps - 1) / kWarps));
  kernel<<<grid, kThreads, smem, stream>>>(p);
  OQ_CHECK_CUDA(cudaGetLastError());
  count_launch();
  if (plan.splits > 1) {
    const int threads = 256;
    const int blocks = static_cast<int>(std::min<int64_t>((rows * out_features + threads - 1) / threads, 4 * sm_count));
    if (scaled) {
      stream_rows_finish_kernel<true><<<blocks, threads, 0, stream>>>(p);
    } else {
      stream_rows_finish_kernel<false><<<blocks, threads, 0, stream>>>(p);
    }
    OQ_CHECK_CUDA(cudaGetLastError());
    count_launch();
  }
  return OQ_OK;
}

}  // namespace oq
