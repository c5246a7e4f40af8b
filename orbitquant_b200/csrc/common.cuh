// Shared host/device helpers of the orbit_b200 library.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>

#include "../../include/orbit_b200.h"

namespace oq {

// ---- host-side status plumbing ---------------------------------------------------------

extern thread_local char g_last_error[512];
extern std::atomic<uint64_t> g_launch_count;

int fail(int status, const char *format, ...);

inline void count_launch(uint64_t n = 1) { g_launch_count.fetch_add(n, std::memory_order_relaxed); }

// Tuning switches for tests and profiling.  Process-wide; each starts from the environment
// variable ORBIT_B200_<NAME> (read once, when the first switch is looked up) and can be
// changed afterwards with oq_set_tunable().  -1 = not set: the library decides by shape.
enum {
  OQ_TUNE_TILE_N = 0,            // large-row tcgen05 kernel: output tile width 128 | 192 | 256
  OQ_TUNE_TILE_ORDER,            // 1 = column tiles fastest, 0 = row tiles fastest
  OQ_TUNE_SKINNY,                // 0 = rows <= 128 stay on the large-row tcgen05 kernel
  OQ_TUNE_STREAM_ROWS,           // 0 / 1 = never / always the persistent small-rows kernel
  OQ_TUNE_PROLOGUE_ROWS,         // tokens per CTA of the general rotate-and-quantize kernel
  OQ_TUNE_SKINNY_UNITS_PER_SM,   // few-token kernel: work units per SM
  OQ_TUNE_SKINNY_MIN_ITERS,      // few-token kernel: fewest k steps per reduction slice
  OQ_TUNE_FUSED_DECODE,          // 0 = rows <= 16 never take the single-launch fused kernel
  OQ_TUNE_PROLOGUE_KERNEL,       // 0 = general, 1 = multi-token CTA, 2 = warp-per-block kernel
  OQ_TUNE_PAIR,                  // large-row tcgen05 kernel: 0 / 1 = never / always the CTA-pair variant
  OQ_TUNE_INT8_MMA,              // INT8-surrogate matmul: 0 = INT8 codes as f16 on the f16 kernel, never kind::i8
  OQ_TUNE_GEMV,                  // 0 / 1 = never / always the CUDA-core GEMV at one to four tokens
  OQ_TUNE_COUNT
};
int tunable(int which);

// OQ_OK when the current device is an sm_100 part, OQ_ERR_DEVICE otherwise.
int check_device();

#define OQ_CHECK_ARG(cond, ...)                         \
  do {                                                  \
    if (!(cond)) {                                      \
      return ::oq::fail(OQ_ERR_INVALID, __VA_ARGS__);   \
    }                                                   \
  } while (0)

#define OQ_CHECK_CUDA(expr)                                                              \
  do {                                                                                   \
    cudaError_t oq_err__ = (expr);                                                       \
    if (oq_err__ != cudaSuccess) {                                                       \
      return ::oq::fail(OQ_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(oq_err__)); \
    }                                                                                    \
  } while (0)

inline bool valid_dtype(int dtype) {
  return dtype == OQ_DTYPE_F32 || dtype == OQ_DTYPE_F16 || dtype == OQ_DTYPE_BF16;
}

inline size_t dtype_size(int dtype) { return dtype == OQ_DTYPE_F32 ? 4 : 2; }

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---- device-side scalar access -----------------------------------------------------------

template <int DTYPE>
struct Scalar;
template <>
struct Scalar<OQ_DTYPE_F32> {
  using type = float;
  static __device__ __forceinline__ float load(const void *p, int64_t i) {
    return static_cast<const float *>(p)[i];
  }
  static __device__ __forceinline__ void store(void *p, int64_t i, float v) {
    static_cast<float *>(p)[i] = v;
  }
};
template <>
struct Scalar<OQ_DTYPE_F16> {
  using type = __half;
  static __device__ __forceinline__ float load(const void *p, int64_t i) {
    return __half2float(static_cast<const __half *>(p)[i]);
  }
  static __device__ __forceinline__ void store(void *p, int64_t i, float v) {
    static_cast<__half *>(p)[i] = __float2half_rn(v);
  }
};
template <>
struct Scalar<OQ_DTYPE_BF16> {
  using type = __nv_bfloat16;
  static __device__ __forceinline__ float load(const void *p, int64_t i) {
    return __bfloat162float(static_cast<const __nv_bfloat16 *>(p)[i]);
  }
  static __device__ __forceinline__ void store(void *p, int64_t i, float v) {
    static_cast<__nv_bfloat16 *>(p)[i] = __float2bfloat16_rn(v);
  }
};

__device__ __forceinline__ float bf16_bits_to_float(uint16_t bits) {
  return __uint_as_float(static_cast<uint32_t>(bits) << 16);
}

// Field `index` of the little-endian `bits`-wide stream (1 <= bits <= 8).
__device__ __forceinline__ uint32_t unpack_field(const uint8_t *packed, int64_t index, int bits) {
  const int64_t bit_start = index * bits;
  const int64_t byte_index = bit_start >> 3;
  const uint32_t shift = static_cast<uint32_t>(bit_start & 7);
  uint32_t raw = packed[byte_index];
  if (shift + static_cast<uint32_t>(bits) > 8u) {
    raw |= static_cast<uint32_t>(packed[byte_index + 1]) << 8;
  }
  return (raw >> shift) & ((1u << bits) - 1u);
}

}  // namespace oq
