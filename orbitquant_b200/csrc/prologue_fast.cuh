// Specialised rotate-and-quantize kernel for the shapes the benchmark layers use:
// bf16 activations, dim a multiple of 256, block >= 256, no code / norm side outputs.
// Same arithmetic, same operation order and therefore the same bits as the general kernel
// in prologue.cu; everything that is uniform across the grid (bit width, output format,
// butterfly widths below 256) is a template parameter instead of a run-time branch, and
// the per-token output values -- only 2^BITS distinct ones exist: round(centroid * norm),
// optionally rescaled to the f16 operand -- are tabulated once per token so that the inner
// loop is: scale, binary search, one 16-bit table read, one 16-bit store.
#pragma once

namespace oq {
namespace {

constexpr int kFastThreads = 256;
constexpr int kFastWarps = 8;

template <int BITS>
__device__ __forceinline__ uint32_t search_offset(float d, const unsigned char *bnd_bytes) {
  // byte offset (4 * index) of the bucket: index = #{boundaries < d}
  uint32_t off = 0;
#pragma unroll
  for (int step = 1 << (BITS - 1); step >= 1; step >>= 1) {
    const float b = *reinterpret_cast<const float *>(bnd_bytes + off + 4 * (step - 1));
    off += !(d <= b) ? 4u * step : 0u;
  }
  return off;
}

template <int S>
__device__ __forceinline__ void radix_butterflies(float (&v)[S]) {
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

// One pass over butterfly widths stride .. stride*S/2.  U column groups are processed
// together so that U*S independent boundary searches are in flight per thread: the search
// is a chain of dependent shared-memory reads, and without that much instruction-level
// parallelism its latency, not any throughput limit, sets the pace of the whole kernel.
template <int BITS, int S, int U, bool LAST>
__device__ __forceinline__ void fast_strided_pass(float *rot, uint16_t *stage, const unsigned char *bnd,
                                                  const uint16_t *outtab, int dim, int nrows,
                                                  int stride, float inv_sqrt_block) {
  const int sq_log2 = __ffs(stride >> 8) - 1;
  const int sq_mask = (stride >> 8) - 1;
  const int cols = dim / (S * 256);
  for (int r = 0; r < nrows; ++r) {
    float *row = rot + r * dim;
    uint16_t *stage_row = stage + r * dim;
    const unsigned char *tab = reinterpret_cast<const unsigned char *>(outtab + (r << BITS));
    for (int c0 = 0; c0 < cols; c0 += U) {
      int base[U];
      float v[U][S];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int c = c0 + u;
        base[u] = (c >> sq_log2) * (stride * S) + (c & sq_mask) * 256 + static_cast<int>(threadIdx.x);
#pragma unroll
        for (int s = 0; s < S; ++s) {
          v[u][s] = row[base[u] + s * stride];
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        radix_butterflies<S>(v[u]);
      }
      if (LAST) {
        uint32_t off[U][S];
#pragma unroll
        for (int u = 0; u < U; ++u) {
#pragma unroll
          for (int s = 0; s < S; ++s) {
            off[u][s] = search_offset<BITS>(__fmul_rn(v[u][s], inv_sqrt_block), bnd);
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
#pragma unroll
          for (int s = 0; s < S; ++s) {
            stage_row[base[u] + s * stride] = *reinterpret_cast<const uint16_t *>(tab + (off[u][s] >> 1));
          }
        }
      } else {
#pragma unroll
        for (int u = 0; u < U; ++u) {
#pragma unroll
          for (int s = 0; s < S; ++s) {
            row[base[u] + s * stride] = v[u][s];
          }
        }
      }
    }
  }
}

template <int BITS, int S, bool LAST>
__device__ __forceinline__ void fast_strided_unroll(float *rot, uint16_t *stage, const unsigned char *bnd,
                                                    const uint16_t *outtab, int dim, int nrows, int stride,
                                                    float isb) {
  const int cols = dim / (S * 256);
  if (S <= 4 && cols % 3 == 0) {
    fast_strided_pass<BITS, S, 3, LAST>(rot, stage, bnd, outtab, dim, nrows, stride, isb);
  } else if (S <= 8 && cols % 2 == 0) {
    fast_strided_pass<BITS, S, 2, LAST>(rot, stage, bnd, outtab, dim, nrows, stride, isb);
  } else {
    fast_strided_pass<BITS, S, 1, LAST>(rot, stage, bnd, outtab, dim, nrows, stride, isb);
  }
}

template <int BITS, bool LAST>
__device__ __forceinline__ void fast_strided_any(float *rot, uint16_t *stage, const unsigned char *bnd,
                                                 const uint16_t *outtab, int dim, int nrows, int stride,
                                                 int radix, float isb) {
  switch (radix) {
    case 2: fast_strided_unroll<BITS, 2, LAST>(rot, stage, bnd, outtab, dim, nrows, stride, isb); break;
    case 4: fast_strided_unroll<BITS, 4, LAST>(rot, stage, bnd, outtab, dim, nrows, stride, isb); break;
    case 8: fast_strided_unroll<BITS, 8, LAST>(rot, stage, bnd, outtab, dim, nrows, stride, isb); break;
    default: fast_strided_unroll<BITS, 16, LAST>(rot, stage, bnd, outtab, dim, nrows, stride, isb); break;
  }
}

// Steps 1 - 4 for the tokens row_base .. row_base + nrows (rotation blocks c_lo .. c_hi in units
// of 256 elements): load, norms, per-token output table, gather + 256-point transforms, wider
// butterfly passes with the quantisation.  Called by all 256 threads; on return (after a
// barrier) the results of token r sit at stage[r * dim + first ...].
template <int BITS, bool F16OP>
__device__ __forceinline__ void fast_rotate_rows(const PrologueParams &p, float *rot, uint16_t *xin,
                                                 const float *s_cent, const unsigned char *bnd_bytes,
                                                 float *s_norm, float *s_inv, float *s_opscale,
                                                 uint16_t *s_outtab, uint16_t *stage, int64_t row_base,
                                                 int nrows, int c_lo, int c_hi, int slices) {
  constexpr int kLevels = 1 << BITS;
  const int dim = p.dim;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const bool wide = p.block > 256;
  const float isb = p.inv_sqrt_block;

  // 1. load
  {
    const uint4 *src4 = reinterpret_cast<const uint4 *>(static_cast<const uint16_t *>(p.x) + row_base * dim);
    uint4 *dst4 = reinterpret_cast<uint4 *>(xin);
    const int vecs = nrows * dim / 8;
    for (int i = threadIdx.x; i < vecs; i += kFastThreads) {
      dst4[i] = __ldg(src4 + i);
    }
  }
  __syncthreads();

  // 2. norms in AVX-512 order (16 fused-multiply-add lanes per token, 8/4/2/1 fold)
  if (threadIdx.x < ((16 * nrows + 31) & ~31)) {
    const int r = threadIdx.x >> 4;
    const int j = threadIdx.x & 15;
    float acc = 0.0f;
    if (r < nrows) {
      const uint16_t *xr = xin + r * dim;
      int i = j;
      for (; i + 7 * 16 < dim; i += 8 * 16) {
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          v[u] = bf16_bits_to_float(xr[i + 16 * u]);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          acc = __fmaf_rn(v[u], v[u], acc);
        }
      }
      for (; i < dim; i += 16) {
        const float v = bf16_bits_to_float(xr[i]);
        acc = __fmaf_rn(v, v, acc);
      }
    }
    acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 8));
    acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 4));
    acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 2));
    acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 1));
    if (r < nrows && j == 0) {
      const float norm = __fsqrt_rn(acc);
      s_norm[r] = norm;
      s_inv[r] = __fdiv_rn(1.0f, __fadd_rn(norm, p.eps));
      float mult = 1.0f;
      if (F16OP) {
        float back = 1.0f;
        if (norm > 0.0f && norm < __int_as_float(0x7f800000)) {
          const int e = max(ilogbf(norm) + 1, -100);
          mult = ldexpf(1.0f, 14 - e);
          back = ldexpf(1.0f, e - 14);
        }
        if (c_lo == 0) {
          p.row_scale[row_base + r] = back;
        }
      }
      s_opscale[r] = mult;
    }
  }
  __syncthreads();

  // 2b. the 2^BITS possible outputs of every token
  for (int t = threadIdx.x; t < (nrows << BITS); t += kFastThreads) {
    const int r = t >> BITS;
    const float q = __fmul_rn(s_cent[t & (kLevels - 1)], s_norm[r]);
    const __nv_bfloat16 qb = __float2bfloat16_rn(q);
    uint16_t bits;
    if (F16OP) {
      bits = __half_as_ushort(__float2half_rn(__fmul_rn(__bfloat162float(qb), s_opscale[r])));
    } else {
      bits = __bfloat16_as_ushort(qb);
    }
    s_outtab[t] = bits;
  }
  __syncthreads();

  // 3. gather + complete 256-point transform per (token, chunk)
  const int my_chunks = c_hi - c_lo;
  const int items = nrows * my_chunks;
  for (int item = warp; item < items; item += kFastWarps) {
    const int r = item / my_chunks;
    const int c = c_lo + (item - r * my_chunks);
    const int i0 = (c << 8) + lane * 8;
    const uint16_t *xr = xin + r * dim;
    const float inv = s_inv[r];
    // plain loads: the permutation may sit in global memory or in a shared-memory copy
    const int4 pa = *reinterpret_cast<const int4 *>(p.perm + i0);
    const int4 pb = *reinterpret_cast<const int4 *>(p.perm + i0 + 4);
    const int2 sg = *reinterpret_cast<const int2 *>(p.signs + i0);
    const int pi[8] = {pa.x, pa.y, pa.z, pa.w, pb.x, pb.y, pb.z, pb.w};
    float v[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const uint32_t word = static_cast<uint32_t>(e < 4 ? sg.x : sg.y);
      const uint32_t flip = (word << (24 - 8 * (e & 3))) & 0x80000000u;
      const uint32_t xbits = (static_cast<uint32_t>(xr[pi[e]]) << 16) ^ flip;
      v[e] = __fmul_rn(__uint_as_float(xbits), inv);
    }
    radix_butterflies<8>(v);
#pragma unroll
    for (int m = 1; m < 32; m <<= 1) {
      const float sgn = (lane & m) != 0 ? -1.0f : 1.0f;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float other = __shfl_xor_sync(0xffffffffu, v[e], m);
        v[e] = __fmaf_rn(sgn, v[e], other);
      }
    }
    if (wide) {
      float4 *dst = reinterpret_cast<float4 *>(rot + r * dim + i0);
      dst[0] = make_float4(v[0], v[1], v[2], v[3]);
      dst[1] = make_float4(v[4], v[5], v[6], v[7]);
    } else {
      const unsigned char *tab = reinterpret_cast<const unsigned char *>(s_outtab + (r << BITS));
      uint32_t packed[4];
#pragma unroll
      for (int e = 0; e < 8; e += 2) {
        const uint32_t o0 = search_offset<BITS>(__fmul_rn(v[e], isb), bnd_bytes);
        const uint32_t o1 = search_offset<BITS>(__fmul_rn(v[e + 1], isb), bnd_bytes);
        packed[e >> 1] = static_cast<uint32_t>(*reinterpret_cast<const uint16_t *>(tab + (o0 >> 1))) |
                         (static_cast<uint32_t>(*reinterpret_cast<const uint16_t *>(tab + (o1 >> 1))) << 16);
      }
      *reinterpret_cast<uint4 *>(stage + r * dim + i0) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    }
  }
  __syncthreads();

  // 4. widths >= 256
  // A slice is a run of whole blocks, so the strided passes see it as a shorter row (with
  // one row per CTA the row pitch does not matter).
  const int span = slices > 1 ? my_chunks << 8 : dim;
  const int first = c_lo << 8;
  if (wide) {
    int stride = 256;
    while (p.block / stride > 16) {
      fast_strided_any<BITS, false>(rot + first, stage + first, bnd_bytes, s_outtab, span, nrows, stride, 16, isb);
      stride *= 16;
      __syncthreads();
    }
    fast_strided_any<BITS, true>(rot + first, stage + first, bnd_bytes, s_outtab, span, nrows, stride,
                                 p.block / stride, isb);
    __syncthreads();
  }
}

template <int BITS, bool F16OP>
__global__ void __launch_bounds__(kFastThreads, 4)
rotate_quantize_fast_kernel(const PrologueParams p) {
  extern __shared__ __align__(16) unsigned char smem[];
  const int dim = p.dim;
  const int R = p.rows_per_cta;
  constexpr int kLevels = 1 << BITS;
  float *rot = reinterpret_cast<float *>(smem);                                    // [R][dim]
  uint16_t *xin = reinterpret_cast<uint16_t *>(rot + static_cast<size_t>(R) * dim);  // [R][dim]
  float *s_bnd = reinterpret_cast<float *>(xin + static_cast<size_t>(R) * dim);     // [kLevels]
  float *s_cent = s_bnd + kLevels;                                                  // [kLevels]
  float *s_norm = s_cent + kLevels;                                                 // [8]
  float *s_inv = s_norm + 8;                                                        // [8]
  float *s_opscale = s_inv + 8;                                                     // [8]
  uint16_t *s_outtab = reinterpret_cast<uint16_t *>(s_opscale + 8);                 // [R][kLevels]

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // see rotate_quantize_kernel
  // Launched with programmatic stream serialization: while the kernel before this one drains,
  // the constants of THIS layer (its own permutation, signs and codebook: cold in a chain of
  // layers) are already on their way into the L2.  x, the outputs and the workspace are touched
  // after the wait only.
  {
    const unsigned char *perm_bytes = reinterpret_cast<const unsigned char *>(p.perm);
    const unsigned char *sign_bytes = reinterpret_cast<const unsigned char *>(p.signs);
    for (int off = threadIdx.x * 128; off < dim * 4; off += kFastThreads * 128) {
      asm volatile("prefetch.global.L2 [%0];" ::"l"(perm_bytes + off));
    }
    for (int off = threadIdx.x * 128; off < dim; off += kFastThreads * 128) {
      asm volatile("prefetch.global.L2 [%0];" ::"l"(sign_bytes + off));
    }
    if (threadIdx.x == 0) {
      asm volatile("prefetch.global.L2 [%0];" ::"l"(p.centroids));
      asm volatile("prefetch.global.L2 [%0];" ::"l"(p.boundaries));
    }
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");
  // The last CTA of the grid does nothing but the table-scale search and the counter clearing,
  // so that with few rows (decode) they are not on any token's critical path.
  const int workers = static_cast<int>(gridDim.x) - (p.table_scale_out != nullptr ? 1 : 0);
  if (static_cast<int>(blockIdx.x) == workers) {
    clear_words(p.zero_words, p.zero_count);
    search_table_scale(p.w_centroids, p.w_bits, p.table_scale_out, rot);
    return;
  }
  for (int i = threadIdx.x; i < kLevels; i += kFastThreads) {
    s_cent[i] = p.centroids[i];
    s_bnd[i] = i < kLevels - 1 ? p.boundaries[i] : 0.0f;
  }
  const bool wide = p.block > 256;
  uint16_t *stage = wide ? xin : reinterpret_cast<uint16_t *>(rot);
  const int chunks = dim >> 8;
  const unsigned char *bnd_bytes = reinterpret_cast<const unsigned char *>(s_bnd);

  // Work items: groups of R rows, or (row, slice of whole rotation blocks) when rows are few.
  const int slices = p.slices;
  const int slice_chunks = chunks / slices;
  const int64_t items_total = slices > 1 ? p.rows * slices : (p.rows + R - 1) / R;
  for (int64_t work = blockIdx.x; work < items_total; work += workers) {
    const int64_t row_base = slices > 1 ? work / slices : work * R;
    const int c_lo = slices > 1 ? static_cast<int>(work % slices) * slice_chunks : 0;
    const int c_hi = slices > 1 ? c_lo + slice_chunks : chunks;
    const int nrows = static_cast<int>(min(static_cast<int64_t>(R), p.rows - row_base));
    __syncthreads();
    fast_rotate_rows<BITS, F16OP>(p, rot, xin, s_cent, bnd_bytes, s_norm, s_inv, s_opscale, s_outtab,
                                  stage, row_base, nrows, c_lo, c_hi, slices);

    // 5. store
    {
      const int my_chunks = c_hi - c_lo;
      const int span = slices > 1 ? my_chunks << 8 : dim;
      const int first = c_lo << 8;
      const uint4 *s4 = reinterpret_cast<const uint4 *>(stage + first);
      uint4 *d4 = reinterpret_cast<uint4 *>(static_cast<uint16_t *>(p.xq) + row_base * dim + first);
      const int vecs = slices > 1 ? span / 8 : nrows * dim / 8;
      for (int i = threadIdx.x; i < vecs; i += kFastThreads) {
        d4[i] = s4[i];
      }
    }
  }
}

inline size_t fast_smem_bytes(int dim, int rows_per_cta, int bits) {
  return static_cast<size_t>(rows_per_cta) * dim * 6 + (2u << bits) * 4 + 24 * 4 +
         (static_cast<size_t>(rows_per_cta) << bits) * 2 + 16;
}

}  // namespace
}  // namespace oq
