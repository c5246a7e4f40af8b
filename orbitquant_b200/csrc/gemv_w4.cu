// Packed 4-bit weight matmul for one to four tokens on large layers: a CUDA-core GEMV in fp32.
//
// At one to four tokens a tensor-core tile is almost empty and the cost of a layer is the decode
// of its weight indices, so this kernel spends as few instructions per weight as the arithmetic
// allows: a warp owns 8 weight rows and a slice of the reduction dimension; each lane keeps its
// KS activations of every token in registers as fp32, loads KS/2 packed bytes of each of the 8
// rows, turns every byte into its two fp32 centroids with ONE 8-byte shared-memory read (a
// 256-entry table with a copy per lane, so that the lanes of a half-warp never share a bank;
// the table address is one byte permute of the packed word) and issues two fused multiply-adds
// per token: (2 + 2 M) / 2 instructions per weight.
//
// The grid is persistent (one CTA of 16 or 24 warps per SM walks the row blocks; the table is
// built once per CTA and the next step's packed words are loaded under the current step's
// arithmetic).  The rows are finished inside the CTA: the 8 x M per-lane sums are reduced across the warp by a
// transposing butterfly (9 shuffles per token instead of 40), the warps that split the reduction
// dimension meet in shared memory and are added in slice order, so the result does not depend
// on scheduling.  Every packed byte is read once; a CTA asks the L2 for its whole slab of
// weights at its first instruction, before it waits for the kernel that produces the
// activations (the launch is programmatic), so the stream from HBM runs ahead of the arithmetic.
//
// Arithmetic: out[m, n] = (sum_k x[m, k] * centroid[w[n, k]]) * row_norm[n] + bias[n] with fp32
// centroids and fp32 accumulation (reference: the fp32-centroid kernels of
// orbitquant_packed_matmul_cpu/packed_matmul_cpu.cpp:115-201 and the single-launch CUDA GEMV
// orbitquant_packed_matmul_cuda/packed_matmul.cu:1202-1259).
#include "common.cuh"

namespace oq {
namespace {

constexpr int kGvRows = 8;        // weight rows a warp carries at a time
constexpr int kGvLutRep = 32;     // copies of the byte table: one per lane
constexpr int kGvLutBytes = 256 * kGvLutRep * 8;   // 64 KB, entry v of lane l at v * 256 + l * 8
// The table starts on a 64 KB boundary of the shared address space, so that "byte 1 of the
// address" IS the packed byte and one byte permute builds a table address; the dynamic shared
// memory is sized so that such a window exists wherever the allocation starts.
constexpr int kGvSmemBytes = 2 * kGvLutBytes;
constexpr int kGvPartBytes = 8 * 1024;             // two buffers of per-warp sums, beside the table
// One CTA per SM: 24 warps for one and two tokens (85 registers), 16 for three and four (128).
constexpr int gv_cta_warps(int rows) { return rows <= 2 ? 24 : 16; }

struct GemvParams {
  void *out;
  const __nv_bfloat16 *x;
  const uint8_t *packed;
  const __nv_bfloat16 *row_norms;
  const float *centroids;
  const void *bias;
  int bias_dtype;
  int64_t in_features;
  int64_t out_features;
  int slices;           // slices of 32 * KS reduction indices
  int ksplit;           // warps that share a row group along the reduction dimension
  int slices_per_warp;
  int groups;           // row groups (of 8 rows) per CTA
  int64_t row_blocks;   // blocks of groups * 8 rows; a CTA walks them with the grid's stride
};

__device__ __forceinline__ float gv_bias(const void *bias, int dtype, int64_t n) {
  switch (dtype) {
    case OQ_DTYPE_F32: return Scalar<OQ_DTYPE_F32>::load(bias, n);
    case OQ_DTYPE_F16: return Scalar<OQ_DTYPE_F16>::load(bias, n);
    default: return Scalar<OQ_DTYPE_BF16>::load(bias, n);
  }
}

// KS / 8 words of packed indices (KS weights) of one row.
template <int KS>
struct GvWords {
  uint32_t w[KS / 8];
};

template <int KS>
__device__ __forceinline__ GvWords<KS> gv_load_words(const uint8_t *src) {
  GvWords<KS> r;
  if constexpr (KS == 32) {
    const uint4 v = __ldg(reinterpret_cast<const uint4 *>(src));
    r.w[0] = v.x;
    r.w[1] = v.y;
    r.w[2] = v.z;
    r.w[3] = v.w;
  } else if constexpr (KS == 16) {
    const uint2 v = __ldg(reinterpret_cast<const uint2 *>(src));
    r.w[0] = v.x;
    r.w[1] = v.y;
  } else {
    r.w[0] = __ldg(reinterpret_cast<const uint32_t *>(src));
  }
  return r;
}

// This lane's KS activations of every token as fp32.
template <int M, int KS>
__device__ __forceinline__ void gv_load_x(float (&xr)[M][KS], const GemvParams &p, int64_t k0, bool active) {
#pragma unroll
  for (int m = 0; m < M; ++m) {
#pragma unroll
    for (int q = 0; q < KS / 8; ++q) {
      uint4 v = make_uint4(0, 0, 0, 0);
      if (active) {
        v = __ldg(reinterpret_cast<const uint4 *>(p.x + static_cast<int64_t>(m) * p.in_features + k0) + q);
      }
      const uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        xr[m][8 * q + 2 * i] = __uint_as_float(words[i] << 16);
        xr[m][8 * q + 2 * i + 1] = __uint_as_float(words[i] & 0xffff0000u);
      }
    }
  }
}

__device__ __forceinline__ float2 gv_lds_f32x2(uint32_t addr) {
  float2 v;
  asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr));
  return v;
}

template <int M, int KS>
__global__ void __launch_bounds__(gv_cta_warps(M) * 32, 1) gemv_w4_kernel(const GemvParams p) {
  extern __shared__ __align__(16) unsigned char smem[];
  const uint32_t smem_addr = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  const uint32_t lut_addr = (smem_addr + 0xffffu) & ~0xffffu;
  unsigned char *lut_ptr = smem + (lut_addr - smem_addr);
  float2 *s_lut = reinterpret_cast<float2 *>(lut_ptr);              // [256][kGvLutRep]
  // [2][groups][ksplit][8][M] sums: before the table where the window leaves room, else after it
  float *s_part = reinterpret_cast<float *>(lut_addr - smem_addr >= kGvPartBytes ? smem : lut_ptr + kGvLutBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int group = warp / p.ksplit;
  const int kw = warp - group * p.ksplit;
  const int64_t row_bytes = p.in_features / 2;
  const int64_t block_rows = static_cast<int64_t>(p.groups) * kGvRows;

  // The packed weights of every row block this CTA will walk, on their way into the L2: they do
  // not depend on the kernel before this one, whose tail this kernel's start overlaps.
  for (int64_t b = blockIdx.x; b < p.row_blocks; b += gridDim.x) {
    const int64_t first_row = b * block_rows;
    const int64_t end_row = min(p.out_features, first_row + block_rows);
    const unsigned char *first = reinterpret_cast<const unsigned char *>(p.packed) + first_row * row_bytes;
    const int64_t bytes = (end_row - first_row) * row_bytes;
    for (int64_t off = static_cast<int64_t>(threadIdx.x) * 128; off < bytes;
         off += static_cast<int64_t>(blockDim.x) * 128) {
      asm volatile("prefetch.global.L2 [%0];" ::"l"(first + off));
    }
    if (threadIdx.x == 0) {
      asm volatile("prefetch.global.L2 [%0];" ::"l"(p.row_norms + first_row));
      if (p.bias_dtype >= 0) {
        asm volatile("prefetch.global.L2 [%0];" ::"l"(static_cast<const unsigned char *>(p.bias) +
                                                       first_row * (p.bias_dtype == OQ_DTYPE_F32 ? 4 : 2)));
      }
    }
  }
  // the next kernel in the stream (the next layer's prologue) may start its own prefetches
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  for (int i = threadIdx.x; i < 256 * kGvLutRep; i += blockDim.x) {
    const int v = i / kGvLutRep;
    s_lut[i] = make_float2(p.centroids[v & 15], p.centroids[v >> 4]);
  }

  // this warp's slices of the reduction dimension and the row blocks of its CTA
  const int s_begin = kw * p.slices_per_warp;
  const int my_slices = min(p.slices, s_begin + p.slices_per_warp) - s_begin;   // >= 1 by construction
  const int my_blocks = blockIdx.x < p.row_blocks
                            ? static_cast<int>((p.row_blocks - blockIdx.x + gridDim.x - 1) / gridDim.x)
                            : 0;
  const int steps = my_blocks * my_slices;
  const int features = static_cast<int>(p.in_features);
  const int rows_total = static_cast<int>(p.out_features);
  const int block_rows_i = p.groups * kGvRows;

  // Where a step's packed words are: every address stays inside the weights -- rows past the end
  // repeat the last row and lanes past the end of the reduction dimension read its start (their
  // activations are zero, the rows' results are never stored) -- so the loads need no predicates.
  // Byte offset of this lane's indices within a row, for slice `sl` of this warp:
  auto lane_bytes = [&](int sl) -> int {
    const int k0 = ((s_begin + sl) * 32 + lane) * KS;
    return k0 < features ? k0 / 2 : 0;
  };
  // The 8 rows of block `b` (a multiple of the grid's stride from this CTA's first block).
  auto load_step = [&](GvWords<KS> (&w)[kGvRows], int b, int sl) {
    const int n0 = b * block_rows_i + group * kGvRows;
    const int first = min(n0, rows_total - 1);
    const uint8_t *ptr = p.packed + static_cast<int64_t>(first) * row_bytes + lane_bytes(sl);
    const int valid = rows_total - first;   // rows from `first` to the end, >= 1
    if (valid >= kGvRows) {
#pragma unroll
      for (int r = 0; r < kGvRows; ++r) {
        w[r] = gv_load_words<KS>(ptr);
        ptr += row_bytes;
      }
    } else {
#pragma unroll
      for (int r = 0; r < kGvRows; ++r) {
        w[r] = gv_load_words<KS>(ptr);
        ptr += r + 1 < valid ? row_bytes : 0;
      }
    }
  };

  // the first step's weights are on their way while the table is finished
  GvWords<KS> w_a[kGvRows];
  GvWords<KS> w_b[kGvRows];
  if (steps > 0) {
    load_step(w_a, static_cast<int>(blockIdx.x), 0);
  }
  __syncthreads();
  // the activations are read from here on
  asm volatile("griddepcontrol.wait;" ::: "memory");

  float acc[kGvRows][M];
#pragma unroll
  for (int r = 0; r < kGvRows; ++r) {
#pragma unroll
    for (int m = 0; m < M; ++m) {
      acc[r][m] = 0.0f;
    }
  }
  float xr[M][KS];
  auto load_x = [&](int sl) {
    const int k0 = ((s_begin + sl) * 32 + lane) * KS;
    gv_load_x<M, KS>(xr, p, k0, k0 < features);
  };
  if (my_slices == 1) {   // one slice per warp: its activations never change
    load_x(0);
  }

  // entry v of this lane's copy of the table: byte 1 of this address replaced by v
  const uint32_t lane_base = lut_addr + static_cast<uint32_t>(lane) * 8u;
  const bool b16 = (lane & 16) != 0;
  const bool b8 = (lane & 8) != 0;
  const bool b4 = (lane & 4) != 0;
  const int my_row = (b16 ? 4 : 0) + (b8 ? 2 : 0) + (b4 ? 1 : 0);
  const int part_floats = p.groups * p.ksplit * kGvRows * M;
  const int outputs = p.groups * kGvRows * M;

  // The thread that finishes output (row, token) of a block: its place, and the row norm and
  // bias of the first block (they depend on nothing this kernel waits for).
  const int out_g = threadIdx.x / (kGvRows * M);
  const int out_r = (threadIdx.x - out_g * (kGvRows * M)) / M;
  const int out_m = threadIdx.x - out_g * (kGvRows * M) - out_r * M;
  const int out_row = out_g * kGvRows + out_r;
  float out_norm = 0.0f;
  float out_bias = 0.0f;
  if (threadIdx.x < outputs) {
    const int n = static_cast<int>(blockIdx.x) * block_rows_i + out_row;
    if (n < rows_total) {
      out_norm = __bfloat162float(p.row_norms[n]);
      out_bias = p.bias_dtype >= 0 ? gv_bias(p.bias, p.bias_dtype, n) : 0.0f;
    }
  }

  int blk = static_cast<int>(blockIdx.x);
  int sl = 0;
  int parity = 0;
  // One step: the next step's packed words first, so that they arrive under this step's
  // arithmetic, then 8 rows x KS indices of this step.
  auto step = [&](GvWords<KS> (&cur)[kGvRows], GvWords<KS> (&nxt)[kGvRows], bool more) {
    int next_sl = sl + 1;
    int next_blk = blk;
    if (next_sl == my_slices) {
      next_sl = 0;
      next_blk += static_cast<int>(gridDim.x);
    }
    if (more) {
      load_step(nxt, next_blk, next_sl);
    }
    if (my_slices > 1) {
      load_x(sl);
    }

    // byte by byte, the 8 rows interleaved: 8 * M independent accumulation chains
#pragma unroll
    for (int q = 0; q < KS / 8; ++q) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int r = 0; r < kGvRows; ++r) {
          // one byte permute: bytes 0, 2, 3 of the lane's base address, byte 1 = packed byte j
          const float2 e = gv_lds_f32x2(__byte_perm(lane_base, cur[r].w[q], 0x3240 + 0x10 * j));
#pragma unroll
          for (int m = 0; m < M; ++m) {
            acc[r][m] = fmaf(e.x, xr[m][8 * q + 2 * j], acc[r][m]);
            acc[r][m] = fmaf(e.y, xr[m][8 * q + 2 * j + 1], acc[r][m]);
          }
        }
      }
    }

    if (sl == my_slices - 1) {
      // Transposing butterfly across the warp: afterwards every lane holds the warp's sum for
      // row 4 * bit4 + 2 * bit3 + bit2 of its lane number.
      float *part = s_part + parity * part_floats;
#pragma unroll
      for (int m = 0; m < M; ++m) {
        float v4[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const float keep = b16 ? acc[r + 4][m] : acc[r][m];
          const float send = b16 ? acc[r][m] : acc[r + 4][m];
          v4[r] = __fadd_rn(keep, __shfl_xor_sync(0xffffffffu, send, 16));
        }
        float v2[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const float keep = b8 ? v4[r + 2] : v4[r];
          const float send = b8 ? v4[r] : v4[r + 2];
          v2[r] = __fadd_rn(keep, __shfl_xor_sync(0xffffffffu, send, 8));
        }
        const float keep = b4 ? v2[1] : v2[0];
        const float send = b4 ? v2[0] : v2[1];
        float v1 = __fadd_rn(keep, __shfl_xor_sync(0xffffffffu, send, 4));
        v1 = __fadd_rn(v1, __shfl_xor_sync(0xffffffffu, v1, 2));
        v1 = __fadd_rn(v1, __shfl_xor_sync(0xffffffffu, v1, 1));
        if ((lane & 3) == 0) {
          part[((group * p.ksplit + kw) * kGvRows + my_row) * M + m] = v1;
        }
      }
#pragma unroll
      for (int r = 0; r < kGvRows; ++r) {
#pragma unroll
        for (int m = 0; m < M; ++m) {
          acc[r][m] = 0.0f;
        }
      }
      // Every warp of the CTA ends a row block once per block, so the barrier counts agree even
      // where the warps' slice counts differ.  The sums alternate between two buffers: a buffer
      // is rewritten only after the barrier of the block in between.
      __syncthreads();
      // the slices of a row in slice order, then row norm and bias
      if (threadIdx.x < outputs) {
        const int n = blk * block_rows_i + out_row;
        if (n < rows_total) {
          float sum = 0.0f;
          for (int k = 0; k < p.ksplit; ++k) {
            sum = __fadd_rn(sum, part[((out_g * p.ksplit + k) * kGvRows + out_r) * M + out_m]);
          }
          sum = __fadd_rn(__fmul_rn(sum, out_norm), out_bias);
          static_cast<__nv_bfloat16 *>(p.out)[static_cast<int64_t>(out_m) * p.out_features + n] =
              __float2bfloat16_rn(sum);
        }
        // the next block's row norm and bias, long before they are needed
        const int next_n = (blk + static_cast<int>(gridDim.x)) * block_rows_i + out_row;
        if (next_n < rows_total) {
          out_norm = __bfloat162float(p.row_norms[next_n]);
          out_bias = p.bias_dtype >= 0 ? gv_bias(p.bias, p.bias_dtype, next_n) : 0.0f;
        }
      }
      parity ^= 1;
    }
    sl = next_sl;
    blk = next_blk;
  };
  // two steps per trip: the two sets of packed words swap roles without being copied
  for (int t = 0; t < steps; t += 2) {
    step(w_a, w_b, t + 1 < steps);
    if (t + 1 < steps) {
      step(w_b, w_a, t + 2 < steps);
    }
  }
}

// Reduction indices per lane and slice: 8 keep the kernel within its register budget at every
// token count (activations of M tokens + two sets of packed words of 8 rows + 8 * M sums); one
// token has room for 16, which halves the steps and measures faster up to K = 8192 (9.1 against
// 10.1 us on 3072 -> 9216; beyond, 8 is faster: 10.4 against 11.7 us on 12288 -> 3072).
template <int M, int KS>
int launch_gemv_rows(GemvParams p, cudaStream_t stream) {
  constexpr int kWarps = gv_cta_warps(M);
  static_assert(2 * kWarps * kGvRows * M * sizeof(float) <= kGvPartBytes, "per-warp sums fit beside the table");
  int device = 0;
  int sm_count = 0;
  OQ_CHECK_CUDA(cudaGetDevice(&device));
  OQ_CHECK_CUDA(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device));
  const int64_t chunks = (p.out_features + kGvRows - 1) / kGvRows;
  p.slices = static_cast<int>((p.in_features + 32 * KS - 1) / (32 * KS));
  // How many warps share a row group along the reduction dimension (a divisor of the CTA's
  // warps) and how many row groups a CTA carries: the split that wastes the least of a
  // persistent grid of one CTA per SM -- whole passes over the row blocks, equal slice counts,
  // every SM and warp busy.  One slice per warp keeps its activations in registers for the
  // whole kernel, a small bonus.
  double best = -1.0;
  int best_grid = 1;
  for (int d = 1; d <= kWarps; ++d) {
    if (kWarps % d != 0 || d > p.slices) {
      continue;
    }
    const int spw = (p.slices + d - 1) / d;
    if (static_cast<int64_t>(d - 1) * spw >= p.slices) {
      continue;   // a warp without a slice
    }
    const int groups = kWarps / d;
    const int64_t row_blocks = (chunks + groups - 1) / groups;
    const int64_t grid = std::min<int64_t>(row_blocks, sm_count);
    const int64_t passes = (row_blocks + grid - 1) / grid;
    const double rows_eff = static_cast<double>(chunks) / static_cast<double>(passes * grid * groups);
    const double k_eff = static_cast<double>(p.slices) / (static_cast<double>(d) * spw);
    const double fill = static_cast<double>(grid) / sm_count;
    const double score = rows_eff * k_eff * fill * (spw == 1 ? 1.03 : 1.0);
    if (score > best * 1.001) {
      best = score;
      p.ksplit = d;
      p.slices_per_warp = spw;
      p.groups = groups;
      p.row_blocks = row_blocks;
      best_grid = static_cast<int>(grid);
    }
  }
  if (best < 0.0) {
    return fail(OQ_ERR_UNSUPPORTED, "the GEMV kernel found no split for this problem");
  }
  // per device and cheap: set at every launch, like the other kernels' attributes
  OQ_CHECK_CUDA(cudaFuncSetAttribute(gemv_w4_kernel<M, KS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     kGvSmemBytes));
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(static_cast<unsigned>(best_grid));
  config.blockDim = dim3(static_cast<unsigned>(kWarps * 32));
  config.dynamicSmemBytes = kGvSmemBytes;
  config.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attr;
  config.numAttrs = 1;
  OQ_CHECK_CUDA(cudaLaunchKernelEx(&config, gemv_w4_kernel<M, KS>, p));
  count_launch();
  return OQ_OK;
}

}  // namespace

// One to four bf16 tokens, 4-bit weights, centroid arithmetic, in_features a multiple of 256.
bool gemv_w4_supported(int64_t rows, int64_t in_features, int64_t out_features, int bits, int dtype,
                       int weight_mode) {
  return rows >= 1 && rows <= 4 && bits == 4 && dtype == OQ_DTYPE_BF16 && weight_mode != OQ_WEIGHT_BF16_SCALED &&
         out_features >= 1 && out_features <= (1 << 28) && in_features >= 256 && in_features % 256 == 0 &&
         in_features <= (1 << 24);   // row and feature numbers are 32-bit inside the kernel
}

int launch_gemv_w4(void *out, const void *x, int64_t rows, int64_t in_features, int64_t out_features,
                   const uint8_t *packed, const void *row_norms_bf16, const float *centroids,
                   const void *bias, int bias_dtype, cudaStream_t stream) {
  OQ_CHECK_ARG(aligned16(x) && aligned16(packed), "x and packed weights must be 16-byte aligned for the GEMV kernel");
  GemvParams p{};
  p.out = out;
  p.x = static_cast<const __nv_bfloat16 *>(x);
  p.packed = packed;
  p.row_norms = static_cast<const __nv_bfloat16 *>(row_norms_bf16);
  p.centroids = centroids;
  p.bias = bias;
  p.bias_dtype = bias == nullptr ? -1 : bias_dtype;
  p.in_features = in_features;
  p.out_features = out_features;
  switch (rows) {
    case 1:
      return in_features < 8192 ? launch_gemv_rows<1, 16>(p, stream) : launch_gemv_rows<1, 8>(p, stream);
    case 2: return launch_gemv_rows<2, 8>(p, stream);
    case 3: return launch_gemv_rows<3, 8>(p, stream);
    case 4: return launch_gemv_rows<4, 8>(p, stream);
    default: return fail(OQ_ERR_UNSUPPORTED, "the GEMV kernel takes one to four tokens");
  }
}

}  // namespace oq
