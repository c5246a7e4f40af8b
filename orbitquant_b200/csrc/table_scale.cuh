// Choice of the scale of the tensor-core kernel's f16 weight table.
//
// The f16 operand is f16(centroid * scale).  Rounding a centroid to f16 costs up to 2^-12
// relative, but the scale is free (the GEMM epilogue divides it out in fp32), so one CTA of
// the kernel that runs right before the GEMM (the rotate-and-quantize prologue, or the
// operand conversion) picks, from 1024 candidates in [2^8, 2^9), the scale whose rounded
// table is closest to the exact centroids (sum of squared relative errors) and leaves it
// in the workspace.  With 2^bits <= 16 distinct values this buys 1.3 to 5 bits of accuracy.
#pragma once

#include <cuda_fp16.h>
#include <stdint.h>

namespace oq {

constexpr float kTableScaleBase = 256.0f;

// The same CTA clears the few-token kernel's slice counters (one int per weight tile), which
// live in the caller's workspace and so hold arbitrary bytes on entry.
__device__ __forceinline__ void clear_words(int *words, int count) {
  for (int i = threadIdx.x; i < count; i += blockDim.x) {
    words[i] = 0;
  }
}

// Barrier among the 256 searching threads (a named barrier, so that a CTA with more threads
// than that can leave the others out).
__device__ __forceinline__ void search_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

// Called by threads 0 .. 255 of one CTA.  `scratch` holds at least 272 floats of shared memory.
__device__ __forceinline__ void search_table_scale(const float *centroids, int bits, float *out,
                                                   float *scratch) {
  float *s_cent = scratch;
  unsigned long long *s_best = reinterpret_cast<unsigned long long *>(scratch + 256);  // [8]
  const int levels = 1 << bits;
  for (int i = threadIdx.x; i < levels; i += 256) {
    s_cent[i] = centroids[i];
  }
  search_sync();
  const int candidates = bits == 8 ? 256 : 1024;
  const int per_thread = candidates / 256;
  const float step = 1.0f / static_cast<float>(candidates);
  unsigned long long best = ~0ull;
#pragma unroll 1
  for (int u = 0; u < per_thread; ++u) {
    const int cand = static_cast<int>(threadIdx.x) * per_thread + u;
    const float scale = kTableScaleBase * (1.0f + static_cast<float>(cand) * step);
    float cost = 0.0f;
#pragma unroll 1
    for (int i = 0; i < levels; ++i) {
      const float exact = s_cent[i] * scale;
      const float rounded = __half2float(__float2half_rn(exact));
      const float rel = exact != 0.0f ? __fdividef(rounded - exact, exact) : 0.0f;
      cost = fmaf(rel, rel, cost);
    }
    const unsigned long long key =
        (static_cast<unsigned long long>(__float_as_uint(cost)) << 32) | static_cast<unsigned>(cand);
    best = key < best ? key : best;
  }
#pragma unroll
  for (int m = 16; m >= 1; m >>= 1) {
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, m);
    best = other < best ? other : best;
  }
  if ((threadIdx.x & 31) == 0) {
    s_best[threadIdx.x >> 5] = best;
  }
  search_sync();
  if (threadIdx.x == 0) {
    unsigned long long total = s_best[0];
    for (int w = 1; w < 8; ++w) {
      total = s_best[w] < total ? s_best[w] : total;
    }
    const int cand = static_cast<int>(total & 0xffffffffu);
    *out = kTableScaleBase * (1.0f + static_cast<float>(cand) * step);
  }
  search_sync();
}

}  // namespace oq
