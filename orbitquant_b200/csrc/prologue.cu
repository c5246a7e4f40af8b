// Fused RPBH rotate-and-quantize prologue (online activation quantisation).
//
// One CTA owns `rows_per_cta` tokens at a time and keeps them in shared memory from the
// first load to the last store, so a token is read from HBM once and written once:
//
//   1. the raw rows arrive by 16-byte vector loads;
//   2. per-token sum of squares in the reference's AVX-512 order: 16 fused-multiply-add
//      lanes striding the row, folded 8/4/2/1 by xor-shuffles (commutative adds, so the
//      tree equals _mm512_reduce_add_ps);
//   3. each warp takes 256-element chunks: lane l gathers x[perm[i]]*sign[i]*(1/(n+eps))
//      for its 8 consecutive i, runs butterfly widths 1,2,4 in registers and 8..128 as
//      warp-shuffle butterflies -- a complete 256-point Walsh-Hadamard per warp;
//   4. blocks wider than 256 finish in a second pass where one thread owns the
//      block/256 values 256 apart and runs the remaining widths 256,512,... in registers;
//   5. branch-free bucketize against the Lloyd-Max boundaries, centroid*norm, round to the
//      activation dtype, and the row leaves by 16-byte vector stores.
//
// Butterfly widths run in increasing order and every pair computes (l + r, l - r) with l
// the lower index, which keeps the fp32 result bit-identical to the reference's kernels.
#include <cstdlib>

#include "common.cuh"
#include "table_scale.cuh"

namespace oq {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kChunk = 256;  // elements one warp transforms at a time (8 per lane)

struct PrologueParams {
  const void *x;
  void *xq;
  uint8_t *codes;
  float *norms;
  const int32_t *perm;
  const int8_t *signs;
  const float *boundaries;
  const float *centroids;
  int64_t rows;
  int dim;
  int block;
  int bits;
  int rows_per_cta;
  float eps;
  float inv_sqrt_block;
  // f16 operand mode (16-bit activations only): instead of x_q in x's dtype the kernel
  // writes half(x_q * 2^(14 - E_row)) with E_row = exponent of the token norm, and the
  // exact inverse factor 2^(E_row - 14) to row_scale.  x_q is already rounded to x's dtype
  // (8 or 11 mantissa bits) and |x_q| < norm, so the scaled value is exact in f16 down to
  // 2^-28 of the norm.  This is the A operand of the tcgen05 kernel, whose MMA needs both
  // operands in one 16-bit format.
  int f16_operand;
  float *row_scale;
  // When set, CTA 0 also picks the scale of the GEMM's f16 weight table (table_scale.cuh).
  const float *w_centroids;
  int w_bits;
  float *table_scale_out;
  int *zero_words;   // cleared by CTA 0 (slice counters of the kernel that follows)
  int zero_count;
  // Weight mode (offline quantise-and-pack, reference layers.py:102-121): the row norm is
  // GIVEN, nothing is pre-scaled, and the direction is (fwht * 1/sqrt(block)) / max(norm, eps)
  // -- a true division, after the transform, as the reference's torch expression has it.
  const float *given_norms;
  // When set, the code output holds code_map[index] instead of the index: the INT8 surrogate
  // codes of the reference's integer matmul (orbitquant_rpbh_quantize_int8_kernel,
  // packed_matmul.cu:659-742).  General kernel only.
  const int8_t *code_map;
  // Few rows (decode): a row is split over `slices` CTAs along whole rotation blocks.  Every
  // CTA still loads the row and computes its norm (both are needed everywhere and cheap), but
  // transforms, quantises and stores only its own blocks.  1 = no split.  Fast kernel only.
  int slices;
};

// Number of boundaries strictly below `v` (sorted ascending, count = 2^bits - 1), as a
// branch-free binary search.  `!(v <= b)` keeps the reference's treatment of NaN (counts
// as above every boundary).
template <int BITS>
__device__ __forceinline__ int bucketize_fixed(float v, const float *bnd) {
  int pos = 0;
#pragma unroll
  for (int step = 1 << (BITS - 1); step >= 1; step >>= 1) {
    pos += !(v <= bnd[pos + step - 1]) ? step : 0;
  }
  return pos;
}

__device__ __forceinline__ int bucketize(float v, const float *bnd, int bits) {
  switch (bits) {  // uniform across the grid
    case 4: return bucketize_fixed<4>(v, bnd);
    case 3: return bucketize_fixed<3>(v, bnd);
    case 6: return bucketize_fixed<6>(v, bnd);
    case 2: return bucketize_fixed<2>(v, bnd);
    case 8: return bucketize_fixed<8>(v, bnd);
    default: break;
  }
  int pos = 0;
#pragma unroll 1
  for (int step = 1 << (bits - 1); step >= 1; step >>= 1) {
    pos += !(v <= bnd[pos + step - 1]) ? step : 0;
  }
  return pos;
}

template <int DTYPE>
__device__ __forceinline__ void emit(const PrologueParams &p, void *stage_row, uint8_t *codes_row,
                                     const float *s_bnd, const float *s_cent, int i, float v,
                                     float norm, float opscale) {
  float direction = __fmul_rn(v, p.inv_sqrt_block);
  if (p.given_norms != nullptr) {
    direction = __fdiv_rn(direction, norm);
  }
  const int idx = bucketize(direction, s_bnd, p.bits);
  const float q = __fmul_rn(s_cent[idx], norm);
  if (p.f16_operand) {
    const float rounded = static_cast<float>(static_cast<typename Scalar<DTYPE>::type>(q));
    static_cast<__half *>(stage_row)[i] = __float2half_rn(__fmul_rn(rounded, opscale));
  } else {
    Scalar<DTYPE>::store(stage_row, i, q);
  }
  if (codes_row != nullptr) {
    codes_row[i] = p.code_map != nullptr ? static_cast<uint8_t>(p.code_map[idx]) : static_cast<uint8_t>(idx);
  }
}

// Remaining butterfly widths 256, 512, ... for one group of S values 256 apart.
template <int S>
__device__ __forceinline__ void strided_butterflies(float (&v)[S]) {
#pragma unroll
  for (int h = 1; h < S; h <<= 1) {
#pragma unroll
    for (int a = 0; a < S; ++a) {
      if ((a & h) == 0) {
        const float l = v[a];
        const float r = v[a | h];
        v[a] = __fadd_rn(l, r);
        v[a | h] = __fsub_rn(l, r);
      }
    }
  }
}

// One pass over butterfly widths stride, 2*stride, ..., stride*S/2: a thread owns the S values
// `stride` apart of one group.  With LAST the results are quantised and staged, otherwise
// they return to `rot` for the next pass (the caller synchronises in between).
template <int DTYPE, int S, bool LAST>
__device__ __forceinline__ void strided_pass(const PrologueParams &p, float *rot, void *stage,
                                             const float *s_bnd, const float *s_cent,
                                             const float *s_norm, const float *s_opscale,
                                             int64_t row_base, int nrows, int stride) {
  // A row splits into dim/(stride*S) super-groups of stride*S contiguous values; inside one,
  // column j in [0, stride) and s in [0, S) address value j + stride*s.  stride is a
  // multiple of 256 and a power of two, so thread t owns the columns congruent to t mod 256
  // and the index arithmetic is shifts and masks.
  const int sq_log2 = __ffs(stride / kChunk) - 1;
  const int sq_mask = (stride / kChunk) - 1;
  const int cols = p.dim / (S * kChunk);
  constexpr int kElem = static_cast<int>(sizeof(typename Scalar<DTYPE>::type));
  for (int r = 0; r < nrows; ++r) {
    float *row = rot + r * p.dim;
    void *stage_row = static_cast<unsigned char *>(stage) + static_cast<size_t>(r) * p.dim * kElem;
    uint8_t *codes_row = p.codes == nullptr ? nullptr : p.codes + (row_base + r) * p.dim;
    const float norm = s_norm[r];
    const float opscale = s_opscale[r];
    for (int c = 0; c < cols; ++c) {
      const int base = (c >> sq_log2) * (stride * S) + (c & sq_mask) * kChunk + static_cast<int>(threadIdx.x);
      float *src = row + base;
      float v[S];
#pragma unroll
      for (int s = 0; s < S; ++s) {
        v[s] = src[s * stride];
      }
      strided_butterflies<S>(v);
      if (LAST) {
#pragma unroll
        for (int s = 0; s < S; ++s) {
          emit<DTYPE>(p, stage_row, codes_row, s_bnd, s_cent, base + s * stride, v[s], norm, opscale);
        }
      } else {
#pragma unroll
        for (int s = 0; s < S; ++s) {
          src[s * stride] = v[s];
        }
      }
    }
  }
}

template <int DTYPE, bool LAST>
__device__ __forceinline__ void strided_pass_any(const PrologueParams &p, float *rot, void *stage,
                                                 const float *s_bnd, const float *s_cent,
                                                 const float *s_norm, const float *s_opscale,
                                                 int64_t row_base, int nrows, int stride, int radix) {
  switch (radix) {
    case 2: strided_pass<DTYPE, 2, LAST>(p, rot, stage, s_bnd, s_cent, s_norm, s_opscale, row_base, nrows, stride); break;
    case 4: strided_pass<DTYPE, 4, LAST>(p, rot, stage, s_bnd, s_cent, s_norm, s_opscale, row_base, nrows, stride); break;
    case 8: strided_pass<DTYPE, 8, LAST>(p, rot, stage, s_bnd, s_cent, s_norm, s_opscale, row_base, nrows, stride); break;
    default: strided_pass<DTYPE, 16, LAST>(p, rot, stage, s_bnd, s_cent, s_norm, s_opscale, row_base, nrows, stride); break;
  }
}

template <int DTYPE>
__global__ void __launch_bounds__(kThreads, 3)
rotate_quantize_kernel(const PrologueParams p) {
  using elem_t = typename Scalar<DTYPE>::type;
  extern __shared__ __align__(16) unsigned char smem[];
  const int dim = p.dim;
  const int R = p.rows_per_cta;
  float *rot = reinterpret_cast<float *>(smem);                       // [R][dim] fp32
  elem_t *xin = reinterpret_cast<elem_t *>(rot + static_cast<size_t>(R) * dim);  // [R][dim]
  const size_t tables_offset =
      (static_cast<size_t>(R) * dim * (sizeof(float) + sizeof(elem_t)) + 15) & ~static_cast<size_t>(15);
  float *s_bnd = reinterpret_cast<float *>(smem + tables_offset);
  float *s_cent = s_bnd + 256;
  float *s_norm = s_cent + 256;  // [R] norms
  float *s_inv = s_norm + 8;     // [R] 1/(norm+eps)
  float *s_opscale = s_inv + 8;  // [R] 2^(14 - E) in f16 operand mode

  // A kernel launched with programmatic stream serialization may start its own set-up now;
  // it still waits (griddepcontrol.wait) for this grid to finish before it reads our output.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // The last CTA of the grid does nothing but the table-scale search and the counter clearing,
  // so that with few rows (decode) they are not on any token's critical path.
  const int workers = static_cast<int>(gridDim.x) - (p.table_scale_out != nullptr ? 1 : 0);
  if (static_cast<int>(blockIdx.x) == workers) {
    clear_words(p.zero_words, p.zero_count);
    search_table_scale(p.w_centroids, p.w_bits, p.table_scale_out, s_bnd);
    return;
  }
  const int levels = 1 << p.bits;
  for (int i = threadIdx.x; i < levels; i += kThreads) {
    s_cent[i] = p.centroids[i];
    if (i < levels - 1) {
      s_bnd[i] = p.boundaries[i];
    }
  }

  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const bool wide = p.block > kChunk;
  // Quantised rows are staged in whichever buffer is idle while they are produced.
  void *stage = wide ? static_cast<void *>(xin) : static_cast<void *>(rot);
  const int chunks = (dim + kChunk - 1) / kChunk;
  constexpr int kVec = 16 / static_cast<int>(sizeof(elem_t));
  const bool vec_ok = (dim % kVec) == 0;

  for (int64_t row_base = static_cast<int64_t>(blockIdx.x) * R; row_base < p.rows;
       row_base += static_cast<int64_t>(workers) * R) {
    const int nrows = static_cast<int>(min(static_cast<int64_t>(R), p.rows - row_base));
    __syncthreads();  // previous iteration's stores are done with the staging buffer

    // 1. load
    const elem_t *src = static_cast<const elem_t *>(p.x) + row_base * dim;
    const int total = nrows * dim;
    if (vec_ok) {
      const uint4 *src4 = reinterpret_cast<const uint4 *>(src);
      uint4 *dst4 = reinterpret_cast<uint4 *>(xin);
      for (int i = threadIdx.x; i < total / kVec; i += kThreads) {
        dst4[i] = __ldg(src4 + i);
      }
    } else {
      for (int i = threadIdx.x; i < total; i += kThreads) {
        xin[i] = src[i];
      }
    }
    __syncthreads();

    // 2. norms: thread t -> row t/16, lane-of-16 t%16
    if (threadIdx.x < ((16 * nrows + 31) & ~31)) {
      const int r = threadIdx.x >> 4;
      const int j = threadIdx.x & 15;
      float acc = 0.0f;
      if (r < nrows) {
        const elem_t *xr = xin + static_cast<size_t>(r) * dim;
        const int full = dim & ~15;
        int i = j;
        for (; i + 7 * 16 < full; i += 8 * 16) {
          float v[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            v[u] = static_cast<float>(xr[i + 16 * u]);
          }
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            acc = __fmaf_rn(v[u], v[u], acc);
          }
        }
        for (; i < full; i += 16) {
          const float v = static_cast<float>(xr[i]);
          acc = __fmaf_rn(v, v, acc);
        }
      }
      acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 8));
      acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 4));
      acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 2));
      acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 1));
      if (r < nrows && j == 0) {
        const elem_t *xr = xin + static_cast<size_t>(r) * dim;
        for (int i = dim & ~15; i < dim; ++i) {
          const float v = static_cast<float>(xr[i]);
          acc = __fadd_rn(acc, __fmul_rn(v, v));
        }
        float norm = __fsqrt_rn(acc);
        float inv = __fdiv_rn(1.0f, __fadd_rn(norm, p.eps));
        if (p.given_norms != nullptr) {
          norm = fmaxf(p.given_norms[row_base + r], p.eps);  // clamp_min(eps); the divisor
          inv = 1.0f;                                        // x * 1 is exact: no pre-scaling
        }
        s_norm[r] = norm;
        s_inv[r] = inv;
        if (p.norms != nullptr) {
          p.norms[row_base + r] = norm;
        }
        if (p.f16_operand) {
          float mult = 1.0f;
          float back = 1.0f;
          if (norm > 0.0f && norm < __int_as_float(0x7f800000)) {
            const int e = max(ilogbf(norm) + 1, -100);
            mult = ldexpf(1.0f, 14 - e);
            back = ldexpf(1.0f, e - 14);
          }
          s_opscale[r] = mult;
          p.row_scale[row_base + r] = back;
        }
      }
    }
    __syncthreads();

    // 3. gather + 256-point transform per (row, chunk)
    const int items = nrows * chunks;
    for (int item = warp; item < items; item += kWarps) {
      const int r = item / chunks;
      const int c = item - r * chunks;
      const int i0 = c * kChunk + lane * 8;
      const elem_t *xr = xin + static_cast<size_t>(r) * dim;
      const float inv = s_inv[r];
      float v[8];
      if (i0 + 8 <= dim) {
        const int4 pa = __ldg(reinterpret_cast<const int4 *>(p.perm + i0));
        const int4 pb = __ldg(reinterpret_cast<const int4 *>(p.perm + i0 + 4));
        const int2 sg = __ldg(reinterpret_cast<const int2 *>(p.signs + i0));
        const int pi[8] = {pa.x, pa.y, pa.z, pa.w, pb.x, pb.y, pb.z, pb.w};
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          // x * (+-1) is exact: flip the sign bit where the sign byte is negative
          const uint32_t word = static_cast<uint32_t>(e < 4 ? sg.x : sg.y);
          const uint32_t flip = (word << (24 - 8 * (e & 3))) & 0x80000000u;
          const float signed_x = __uint_as_float(__float_as_uint(static_cast<float>(xr[pi[e]])) ^ flip);
          v[e] = __fmul_rn(signed_x, inv);
        }
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int i = i0 + e;
          v[e] = 0.0f;
          if (i < dim) {
            const float sign = static_cast<float>(p.signs[i]);
            v[e] = __fmul_rn(__fmul_rn(static_cast<float>(xr[p.perm[i]]), sign), inv);
          }
        }
      }
      // widths 1, 2, 4 in registers
#pragma unroll
      for (int h = 1; h < 8; h <<= 1) {
        if (h < p.block) {
#pragma unroll
          for (int a = 0; a < 8; ++a) {
            if ((a & h) == 0) {
              const float l = v[a];
              const float rr = v[a | h];
              v[a] = __fadd_rn(l, rr);
              v[a | h] = __fsub_rn(l, rr);
            }
          }
        }
      }
      // widths 8 .. 128 across lanes
#pragma unroll
      for (int m = 1; m < 32; m <<= 1) {
        if (m * 8 < p.block) {
          // lower lane: v + other; upper lane: other - v.  (+-1)*v is exact, so one fused
          // multiply-add rounds exactly like the add / subtract it replaces.
          const float sgn = (lane & m) != 0 ? -1.0f : 1.0f;
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float other = __shfl_xor_sync(0xffffffffu, v[e], m);
            v[e] = __fmaf_rn(sgn, v[e], other);
          }
        }
      }
      if (wide) {
        if (i0 + 8 <= dim) {
          float4 *dst = reinterpret_cast<float4 *>(rot + static_cast<size_t>(r) * dim + i0);
          dst[0] = make_float4(v[0], v[1], v[2], v[3]);
          dst[1] = make_float4(v[4], v[5], v[6], v[7]);
        }
      } else {
        const float norm = s_norm[r];
        const float opscale = s_opscale[r];
        void *stage_row = static_cast<unsigned char *>(stage) + static_cast<size_t>(r) * dim * sizeof(elem_t);
        uint8_t *codes_row = p.codes == nullptr ? nullptr : p.codes + (row_base + r) * dim;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          if (i0 + e < dim) {
            emit<DTYPE>(p, stage_row, codes_row, s_bnd, s_cent, i0 + e, v[e], norm, opscale);
          }
        }
      }
    }
    __syncthreads();

    // 4. widths >= 256: radix-16 passes in registers, the last one quantises
    if (wide) {
      int stride = kChunk;
      while (p.block / stride > 16) {
        strided_pass_any<DTYPE, false>(p, rot, stage, s_bnd, s_cent, s_norm, s_opscale, row_base,
                                       nrows, stride, 16);
        stride *= 16;
        __syncthreads();
      }
      strided_pass_any<DTYPE, true>(p, rot, stage, s_bnd, s_cent, s_norm, s_opscale, row_base, nrows,
                                    stride, p.block / stride);
      __syncthreads();
    }

    // 5. store
    if (p.xq != nullptr) {
      elem_t *dst = static_cast<elem_t *>(p.xq) + row_base * dim;
      if (vec_ok) {
        const uint4 *s4 = reinterpret_cast<const uint4 *>(stage);
        uint4 *d4 = reinterpret_cast<uint4 *>(dst);
        for (int i = threadIdx.x; i < total / kVec; i += kThreads) {
          d4[i] = s4[i];
        }
      } else {
        const elem_t *s = static_cast<const elem_t *>(stage);
        for (int i = threadIdx.x; i < total; i += kThreads) {
          dst[i] = s[i];
        }
      }
    }
  }
}

}  // namespace
}  // namespace oq

#include "prologue_fast.cuh"
#include "prologue_warp.cuh"
#include "decode_fused.cuh"

namespace oq {
namespace {

template <bool F16OP, int TW>
void (*warp_kernel_for(int bits))(WarpPrologueParams) {
  switch (bits) {
    case 2: return rotate_quantize_warp_kernel<2, F16OP, TW>;
    case 3: return rotate_quantize_warp_kernel<3, F16OP, TW>;
    case 4: return rotate_quantize_warp_kernel<4, F16OP, TW>;
    case 6: return rotate_quantize_warp_kernel<6, F16OP, TW>;
    case 8: return rotate_quantize_warp_kernel<8, F16OP, TW>;
    default: return nullptr;
  }
}

// Tokens per batch, copy slots and CTAs per SM of the warp-per-block kernel: two CTAs per SM
// where the shared memory allows it (latency hiding across CTAs), at least three slots (copies
// must run ahead of the norm warps, which run ahead of the transform warps), then as many
// tokens per batch as fit.
bool plan_warp_prologue(int dim, int block, int bits, int64_t rows, int max_smem, int *batch_rows,
                        int *slots, int *ctas_per_sm, int *smem, int *transform_warps) {
  const int shared_per_sm = 228 * 1024;
  // Blocks of 4096 are shared by teams of four warps and their rows leave room for one CTA per
  // SM only: sixteen transform warps (four teams) keep that SM busy where eight leave it half
  // idle.
  if (block == 4 * kPwChunk) {
    static const int kWide[][2] = {{1, 3}, {1, 2}};
    for (const auto &choice : kWide) {
      const int total = pw_layout(dim, block, choice[0], choice[1], bits, kPwWideWarps).total;
      if (total <= max_smem && total + 1024 <= shared_per_sm) {
        *batch_rows = choice[0];
        *slots = choice[1];
        *ctas_per_sm = 1;
        *smem = total;
        *transform_warps = kPwWideWarps;
        return true;
      }
    }
  }
  *transform_warps = kPwWarps;
  static const int kChoices[][2] = {{4, 3}, {2, 4}, {2, 3}, {1, 4}, {1, 3}, {1, 2}};
  for (int per_sm = 2; per_sm >= 1; --per_sm) {
    for (const auto &choice : kChoices) {
      if (choice[0] > rows) {
        continue;
      }
      const int total = pw_layout(dim, block, choice[0], choice[1], bits).total;
      if (total <= max_smem && per_sm * (total + 1024) <= shared_per_sm) {
        *batch_rows = choice[0];
        *slots = choice[1];
        *ctas_per_sm = per_sm;
        *smem = total;
        return true;
      }
    }
  }
  return false;
}

template <bool F16OP>
void (*fast_kernel_for(int bits))(PrologueParams) {
  switch (bits) {
    case 2: return rotate_quantize_fast_kernel<2, F16OP>;
    case 3: return rotate_quantize_fast_kernel<3, F16OP>;
    case 4: return rotate_quantize_fast_kernel<4, F16OP>;
    case 6: return rotate_quantize_fast_kernel<6, F16OP>;
    case 8: return rotate_quantize_fast_kernel<8, F16OP>;
    default: return nullptr;
  }
}

size_t prologue_smem_bytes(int dim, int rows_per_cta, int dtype) {
  return ((static_cast<size_t>(rows_per_cta) * dim * (4 + dtype_size(dtype)) + 15) & ~static_cast<size_t>(15)) +
         (256 + 256 + 24) * 4;
}

}  // namespace

// Blocks of any power of two up to the dim limit: 256 (warp) x 16 per register pass.
constexpr int64_t kMaxBlock = 1 << 20;

bool int8_operand_prologue_supported(int x_dtype, int64_t dim, int64_t block) {
  return block > 0 && dim % block == 0 && warp_prologue_supported(x_dtype, dim, block, 4);
}

// The INT8 activation operand of the INT8 tensor-core GEMM in one pass: out[m, k] =
// code_map[level of element k of token m] (one byte), row_scale[m] = token norm * out_scale.  The
// warp-per-block kernel only (bf16 rows, dim % 256 == 0, block 256 .. 4096); OQ_ERR_UNSUPPORTED
// otherwise, and the caller takes the general kernel's code output instead.
int launch_rotate_quantize_int8_operand(const void *x, int x_dtype, int64_t rows, int64_t dim,
                                        const int32_t *perm, const int8_t *signs, int64_t block,
                                        const float *boundaries, const float *centroids, int bits, float eps,
                                        const int8_t *code_map, float out_scale, int8_t *out,
                                        float *row_scale, cudaStream_t stream) {
  if (!(bits == 4 && rows > 0 && int8_operand_prologue_supported(x_dtype, dim, block))) {
    return OQ_ERR_UNSUPPORTED;
  }
  OQ_CHECK_ARG(x != nullptr && perm != nullptr && signs != nullptr && boundaries != nullptr &&
                   centroids != nullptr && code_map != nullptr && out != nullptr && row_scale != nullptr,
               "null device pointer");
  OQ_CHECK_ARG(aligned16(x) && aligned16(out) && aligned16(perm) &&
                   (reinterpret_cast<uintptr_t>(signs) & 7u) == 0,
               "x, the operand and perm must be 16-byte aligned, signs 8-byte aligned");
  int device = 0;
  int sm_count = 0;
  int max_smem = 0;
  OQ_CHECK_CUDA(cudaGetDevice(&device));
  OQ_CHECK_CUDA(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device));
  OQ_CHECK_CUDA(cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, device));
  int batch_rows = 0;
  int slots = 0;
  int ctas_per_sm = 0;
  int smem_bytes = 0;
  int transform_warps = kPwWarps;
  if (!plan_warp_prologue(static_cast<int>(dim), static_cast<int>(block), bits, rows, max_smem, &batch_rows,
                          &slots, &ctas_per_sm, &smem_bytes, &transform_warps)) {
    return OQ_ERR_UNSUPPORTED;
  }
  WarpPrologueParams wp{};
  wp.x = static_cast<const uint16_t *>(x);
  wp.xq = reinterpret_cast<uint16_t *>(out);
  wp.row_scale = row_scale;
  wp.code_map = code_map;
  wp.out_scale = out_scale;
  wp.perm = perm;
  wp.signs = signs;
  wp.boundaries = boundaries;
  wp.centroids = centroids;
  wp.rows = rows;
  wp.dim = static_cast<int>(dim);
  wp.log2_block = 0;
  while ((int64_t(1) << wp.log2_block) < block) {
    ++wp.log2_block;
  }
  wp.batch_rows = batch_rows;
  wp.slots = slots;
  wp.eps = eps;
  wp.inv_sqrt_block = static_cast<float>(1.0 / sqrt(static_cast<double>(block)));
  void (*wkernel)(WarpPrologueParams) =
      transform_warps == kPwWideWarps ? rotate_quantize_warp_kernel<4, false, kPwWideWarps, true>
                                      : rotate_quantize_warp_kernel<4, false, kPwWarps, true>;
  OQ_CHECK_CUDA(cudaFuncSetAttribute(wkernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
  const int64_t batches = (rows + batch_rows - 1) / batch_rows;
  const int wgrid = static_cast<int>(std::min<int64_t>(batches, static_cast<int64_t>(sm_count) * ctas_per_sm));
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(static_cast<unsigned>(wgrid));
  config.blockDim = dim3(static_cast<unsigned>(pw_threads(transform_warps)));
  config.dynamicSmemBytes = static_cast<size_t>(smem_bytes);
  config.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attr;
  config.numAttrs = 1;
  OQ_CHECK_CUDA(cudaLaunchKernelEx(&config, wkernel, wp));
  count_launch();
  return OQ_OK;
}

int launch_rotate_quantize(const void *x, int x_dtype, int64_t rows, int64_t dim,
                           const int32_t *perm, const int8_t *signs, int64_t block,
                           const float *boundaries, const float *centroids, int bits, float eps,
                           void *x_q, uint8_t *codes, float *norms, float *f16_row_scale,
                           const float *w_centroids, int w_bits, float *table_scale_out,
                           int *zero_words, int zero_count, cudaStream_t stream,
                           const float *given_norms, const int8_t *code_map) {
  OQ_CHECK_ARG(table_scale_out == nullptr || (w_centroids != nullptr && w_bits >= 1 && w_bits <= 8),
               "the table scale search needs the weight codebook");
  OQ_CHECK_ARG(f16_row_scale == nullptr || (x_dtype != OQ_DTYPE_F32 && x_q != nullptr),
               "the f16 operand output needs 16-bit activations and an output buffer");
  OQ_CHECK_ARG(valid_dtype(x_dtype), "x must be float32, float16, or bfloat16");
  OQ_CHECK_ARG(rows >= 0 && dim > 0, "rows must be >= 0 and dim positive");
  OQ_CHECK_ARG(block > 0 && (block & (block - 1)) == 0, "block_size must be a positive power of two");
  OQ_CHECK_ARG(dim % block == 0, "block_size must divide the input dimension");
  OQ_CHECK_ARG(block <= kMaxBlock, "block_size above %lld is not supported", (long long)kMaxBlock);
  OQ_CHECK_ARG(bits >= 1 && bits <= 8, "bits must be in [1, 8]");
  OQ_CHECK_ARG(eps >= 0.0f, "eps must be non-negative");
  OQ_CHECK_ARG(dim <= (1 << 20), "dim above 2^20 is not supported");
  if (rows == 0) {
    return OQ_OK;
  }
  OQ_CHECK_ARG(x != nullptr && perm != nullptr && signs != nullptr && boundaries != nullptr &&
                   centroids != nullptr, "null device pointer");
  OQ_CHECK_ARG(aligned16(x) && (x_q == nullptr || aligned16(x_q)) && aligned16(perm) &&
                   (reinterpret_cast<uintptr_t>(signs) & 7u) == 0,
               "x, x_q and perm must be 16-byte aligned, signs 8-byte aligned");

  int device = 0;
  OQ_CHECK_CUDA(cudaGetDevice(&device));
  int sm_count = 0;
  int max_smem = 0;
  OQ_CHECK_CUDA(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device));
  OQ_CHECK_CUDA(cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, device));

  // Kernel choice.  The prologue_kernel tunable pins it: 0 = general, 1 = multi-token CTA,
  // 2 = warp-per-block; otherwise 2048 tokens and more take the warp-per-block kernel (measured
  // cross-over at 3072 features: 14.2 against 13.5 us at 1184 tokens, 20.6 against 24.5 at 2368).
  const int forced = tunable(OQ_TUNE_PROLOGUE_KERNEL);
  const bool plain_output = codes == nullptr && norms == nullptr && x_q != nullptr && given_norms == nullptr;
  if (plain_output && warp_prologue_supported(x_dtype, dim, block, bits) &&
      (forced == 2 || (forced < 0 && rows >= 2048))) {
    int batch_rows = 0;
    int slots = 0;
    int ctas_per_sm = 0;
    int smem_bytes = 0;
    int transform_warps = kPwWarps;
    if (plan_warp_prologue(static_cast<int>(dim), static_cast<int>(block), bits, rows, max_smem,
                           &batch_rows, &slots, &ctas_per_sm, &smem_bytes, &transform_warps)) {
      WarpPrologueParams wp{};
      wp.x = static_cast<const uint16_t *>(x);
      wp.xq = static_cast<uint16_t *>(x_q);
      wp.row_scale = f16_row_scale;
      wp.perm = perm;
      wp.signs = signs;
      wp.boundaries = boundaries;
      wp.centroids = centroids;
      wp.rows = rows;
      wp.dim = static_cast<int>(dim);
      wp.log2_block = 0;
      while ((int64_t(1) << wp.log2_block) < block) {
        ++wp.log2_block;
      }
      wp.batch_rows = batch_rows;
      wp.slots = slots;
      wp.eps = eps;
      wp.inv_sqrt_block = static_cast<float>(1.0 / sqrt(static_cast<double>(block)));
      wp.w_centroids = w_centroids;
      wp.w_bits = w_bits;
      wp.table_scale_out = table_scale_out;
      wp.zero_words = zero_words;
      wp.zero_count = zero_words != nullptr ? zero_count : 0;
      const bool wide = transform_warps == kPwWideWarps;
      void (*wkernel)(WarpPrologueParams) =
          f16_row_scale != nullptr
              ? (wide ? warp_kernel_for<true, kPwWideWarps>(bits) : warp_kernel_for<true, kPwWarps>(bits))
              : (wide ? warp_kernel_for<false, kPwWideWarps>(bits) : warp_kernel_for<false, kPwWarps>(bits));
      OQ_CHECK_CUDA(cudaFuncSetAttribute(wkernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
      const int64_t batches = (rows + batch_rows - 1) / batch_rows;
      const int wgrid = static_cast<int>(std::min<int64_t>(batches, static_cast<int64_t>(sm_count) * ctas_per_sm)) +
                        (table_scale_out != nullptr ? 1 : 0);
      // Programmatic stream serialization: the CTAs may become resident, and build their
      // permutation and cell tables, while the kernel before this one in the stream drains its
      // last wave; griddepcontrol.wait inside the kernel precedes every access to x, to the
      // outputs and to the workspace.
      cudaLaunchConfig_t config = {};
      config.gridDim = dim3(static_cast<unsigned>(wgrid));
      config.blockDim = dim3(static_cast<unsigned>(pw_threads(transform_warps)));
      config.dynamicSmemBytes = static_cast<size_t>(smem_bytes);
      config.stream = stream;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[0].val.programmaticStreamSerializationAllowed = 1;
      config.attrs = attr;
      config.numAttrs = 1;
      OQ_CHECK_CUDA(cudaLaunchKernelEx(&config, wkernel, wp));
      count_launch();
      return OQ_OK;
    }
  }

  void (*fast)(PrologueParams) = nullptr;
  if (forced != 0 && x_dtype == OQ_DTYPE_BF16 && dim % 256 == 0 && block >= 256 && codes == nullptr &&
      norms == nullptr && x_q != nullptr) {
    fast = f16_row_scale != nullptr ? fast_kernel_for<true>(bits) : fast_kernel_for<false>(bits);
  }

  // Rows per CTA: enough (row, chunk) items to fill the 8 warps evenly, within ~96 KB so
  // two CTAs share an SM, and never more than the problem offers per SM.
  const int chunks = static_cast<int>((dim + kChunk - 1) / kChunk);
  int rows_per_cta = 1;
  for (int r = 1; r <= 8; r *= 2) {
    if (prologue_smem_bytes(static_cast<int>(dim), r, x_dtype) > (fast != nullptr ? 52 : 72) * 1024 ||
        static_cast<int64_t>(r) * sm_count > rows) {
      break;
    }
    rows_per_cta = r;
    if ((r * chunks) % kWarps == 0) {
      break;
    }
  }
  {
    const int value = tunable(OQ_TUNE_PROLOGUE_ROWS);  // profiling only
    if (value >= 1 && value <= 8 && value <= rows) {
      rows_per_cta = value;
    }
  }
  const size_t smem = fast != nullptr ? fast_smem_bytes(static_cast<int>(dim), rows_per_cta, bits)
                                      : prologue_smem_bytes(static_cast<int>(dim), rows_per_cta, x_dtype);
  OQ_CHECK_ARG(smem <= static_cast<size_t>(max_smem),
               "dim %lld needs %zu bytes of shared memory per token (limit %d)", (long long)dim,
               smem, max_smem);

  PrologueParams p{};
  p.x = x;
  p.xq = x_q;
  p.codes = codes;
  p.norms = norms;
  p.perm = perm;
  p.signs = signs;
  p.boundaries = boundaries;
  p.centroids = centroids;
  p.rows = rows;
  p.dim = static_cast<int>(dim);
  p.block = static_cast<int>(block);
  p.bits = bits;
  p.rows_per_cta = rows_per_cta;
  p.eps = eps;
  p.inv_sqrt_block = static_cast<float>(1.0 / sqrt(static_cast<double>(block)));
  p.f16_operand = f16_row_scale != nullptr ? 1 : 0;
  p.row_scale = f16_row_scale;
  p.w_centroids = w_centroids;
  p.w_bits = w_bits;
  p.table_scale_out = table_scale_out;
  p.zero_words = zero_words;
  p.zero_count = zero_words != nullptr ? zero_count : 0;
  p.given_norms = given_norms;
  p.code_map = code_map;
  p.slices = 1;

  if (fast != nullptr && rows * 2 <= sm_count) {
    // largest divisor of the number of rotation blocks that keeps the grid within the machine
    const int blocks_per_row = static_cast<int>(dim / block);
    for (int cand = blocks_per_row; cand >= 2; --cand) {
      if (blocks_per_row % cand == 0 && rows * cand <= 2 * sm_count) {
        p.slices = cand;
        break;
      }
    }
    if (p.slices > 1) {
      p.rows_per_cta = 1;
    }
  }
  const int64_t ctas_needed = p.slices > 1 ? rows * p.slices : (rows + rows_per_cta - 1) / rows_per_cta;
  const int grid = static_cast<int>(std::min<int64_t>(ctas_needed, static_cast<int64_t>(sm_count) * 8)) +
                   (table_scale_out != nullptr ? 1 : 0);  // + the search CTA
  void (*kernel)(PrologueParams) = nullptr;
  switch (x_dtype) {
    case OQ_DTYPE_F32: kernel = rotate_quantize_kernel<OQ_DTYPE_F32>; break;
    case OQ_DTYPE_F16: kernel = rotate_quantize_kernel<OQ_DTYPE_F16>; break;
    default: kernel = rotate_quantize_kernel<OQ_DTYPE_BF16>; break;
  }
  if (fast != nullptr) {
    kernel = fast;
  }
  if (smem > 48 * 1024) {
    OQ_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(smem)));
  }
  if (fast != nullptr) {
    // programmatic stream serialization: the kernel prefetches its constants and then waits
    // for the kernel before it (griddepcontrol.wait at its top)
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(static_cast<unsigned>(grid));
    config.blockDim = dim3(kThreads);
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attr;
    config.numAttrs = 1;
    OQ_CHECK_CUDA(cudaLaunchKernelEx(&config, kernel, p));
  } else {
    kernel<<<grid, kThreads, smem, stream>>>(p);
    OQ_CHECK_CUDA(cudaGetLastError());
  }
  count_launch();
  return OQ_OK;
}

namespace {

// L2 norm of every weight row, accumulated in double (one warp per row, fixed order) and
// rounded once to fp32: at least as accurate as any fp32 reduction order, and deterministic.
template <int DTYPE>
__global__ void __launch_bounds__(256) weight_row_norms_kernel(const void *w, int64_t rows, int64_t dim,
                                                               float *norms_f32,
                                                               __nv_bfloat16 *norms_bf16) {
  const int lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (row >= rows) {
    return;
  }
  double acc = 0.0;
  for (int64_t i = lane; i < dim; i += 32) {
    const double v = static_cast<double>(Scalar<DTYPE>::load(w, row * dim + i));
    acc = fma(v, v, acc);
  }
#pragma unroll
  for (int m = 16; m >= 1; m >>= 1) {
    acc += __shfl_xor_sync(0xffffffffu, acc, m);
  }
  if (lane == 0) {
    const float norm = static_cast<float>(sqrt(acc));
    norms_f32[row] = norm;
    if (norms_bf16 != nullptr) {
      norms_bf16[row] = __float2bfloat16_rn(norm);
    }
  }
}

__global__ void norms_to_bf16_kernel(const float *norms, int64_t rows, __nv_bfloat16 *out) {
  const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (i < rows) {
    out[i] = __float2bfloat16_rn(norms[i]);
  }
}

}  // namespace

int launch_weight_row_norms(const void *w, int dtype, int64_t rows, int64_t dim, float *norms_f32,
                            void *norms_bf16, cudaStream_t stream) {
  const unsigned grid = static_cast<unsigned>((rows + 7) / 8);
  __nv_bfloat16 *bf = static_cast<__nv_bfloat16 *>(norms_bf16);
  switch (dtype) {
    case OQ_DTYPE_F32: weight_row_norms_kernel<OQ_DTYPE_F32><<<grid, 256, 0, stream>>>(w, rows, dim, norms_f32, bf); break;
    case OQ_DTYPE_F16: weight_row_norms_kernel<OQ_DTYPE_F16><<<grid, 256, 0, stream>>>(w, rows, dim, norms_f32, bf); break;
    default: weight_row_norms_kernel<OQ_DTYPE_BF16><<<grid, 256, 0, stream>>>(w, rows, dim, norms_f32, bf); break;
  }
  OQ_CHECK_CUDA(cudaGetLastError());
  count_launch();
  return OQ_OK;
}

int read_prologue_status(int *status) {
  OQ_CHECK_CUDA(cudaMemcpyFromSymbol(status, g_prologue_status, sizeof(int)));
  return OQ_OK;
}

int clear_prologue_status() {
  const int zero = 0;
  OQ_CHECK_CUDA(cudaMemcpyToSymbol(g_prologue_status, &zero, sizeof(int)));
  return OQ_OK;
}

int launch_norms_to_bf16(const float *norms, int64_t rows, void *out, cudaStream_t stream) {
  norms_to_bf16_kernel<<<static_cast<unsigned>((rows + 255) / 256), 256, 0, stream>>>(
      norms, rows, static_cast<__nv_bfloat16 *>(out));
  OQ_CHECK_CUDA(cudaGetLastError());
  count_launch();
  return OQ_OK;
}

}  // namespace oq
