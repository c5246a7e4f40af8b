/*
 * orbit_b200 -- C ABI of the B200 (sm_100a) OrbitQuant quantized-linear forward.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream
 * (a cudaStream_t passed as void*; NULL = the legacy default stream).  All pointers are
 * DEVICE pointers owned by the caller and must stay alive until the stream has run the
 * work.  Unless an entry point's comment says otherwise the library allocates nothing and
 * never synchronises the host with the device, so every call may be captured into a CUDA
 * graph.  Its only device state is the status word of the tensor-core kernels' bounded
 * waits (oq_gemm_device_status) and the fixed scratch array of the no-allocation variant.
 *
 * Return value: 0 on success, a negative oq_status otherwise; oq_last_error() then holds
 * a message for the calling thread.  The host binding turns OQ_ERR_INVALID into the
 * ValueError / RuntimeError the reference raises for the same misuse.
 *
 * Citations name the reference interface each entry point replaces, as path:line inside
 * the reference project (iamwavecut/OrbitQuant v0.9.0).
 */
#ifndef ORBIT_B200_H_
#define ORBIT_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define OQ_ABI_VERSION 1

/* Element types of activations / outputs / bias. */
#define OQ_DTYPE_F32 0
#define OQ_DTYPE_F16 1
#define OQ_DTYPE_BF16 2

typedef enum oq_status {
  OQ_OK = 0,
  OQ_ERR_INVALID = -1,     /* bad argument (shape, dtype, bits, alignment, null pointer)   */
  OQ_ERR_UNSUPPORTED = -2, /* valid request this build has no kernel for                   */
  OQ_ERR_CUDA = -3,        /* a CUDA runtime / driver call failed                          */
  OQ_ERR_WORKSPACE = -4,   /* caller's workspace is smaller than oq_*_workspace_bytes says */
  OQ_ERR_DEVICE = -5       /* not an sm_100 device                                         */
} oq_status;

/* Arithmetic of the weight operand.
 *   OQ_WEIGHT_CENTROID  : the contraction uses the codebook centroid itself (fp32 on the
 *                         CUDA-core kernels, fp16(centroid * 2^8) on the tensor-core
 *                         kernel) and multiplies the sum by row_norm[n] afterwards -- the
 *                         arithmetic of the reference's fp32-centroid CPU kernels
 *                         (packed_matmul_scalar.cpp:46-74, packed_matmul_x86.cpp,
 *                         packed_matmul_x86_avx512.cpp:200-546).
 *   OQ_WEIGHT_BF16_SCALED: the contraction uses bf16(centroid * row_norm[n]) -- the
 *                         arithmetic of the reference's AVX512-BF16 W4 kernel
 *                         (packed_matmul_x86_avx512.cpp:548-699) and of its CUDA wmma
 *                         kernels (packed_matmul.cu:86-125).
 *   OQ_WEIGHT_AUTO      : OQ_WEIGHT_CENTROID. */
#define OQ_WEIGHT_AUTO 0
#define OQ_WEIGHT_CENTROID 1
#define OQ_WEIGHT_BF16_SCALED 2

/* Kernel selection for oq_matmul_packed_weight / oq_linear_forward.  AUTO picks by shape:
 * rows <= 16 -> the streaming small-rows kernel; otherwise the tcgen05 kernel when the
 * shape qualifies (see oq_gemm_tcgen05_supported), else the general tiled kernel. */
#define OQ_KERNEL_AUTO 0
#define OQ_KERNEL_SMALL_ROWS 1
#define OQ_KERNEL_TILED 2
#define OQ_KERNEL_TCGEN05 3

int oq_abi_version(void);
const char *oq_last_error(void);

/* Number of kernels this library has launched from the calling process since load
 * (monotonic; used by the benchmark to report its own launch count). */
uint64_t oq_launch_count(void);

/* Tuning switches for tests and profiling (no counterpart in the reference, whose kernels
 * read ORBITQUANT_MMA64_{DISABLE,FORCE}_PIPELINE from the environment at every launch,
 * packed_matmul.cu:22-38).  Each switch starts from the environment variable
 * ORBIT_B200_<NAME>, read once per process, and is changed afterwards only through this
 * call; value -1 returns the decision to the library.  Names (case-insensitive): tile_n
 * (128|192|256), tile_order (0|1), skinny (0|1), stream_rows (0|1), prologue_rows (1..8),
 * skinny_units_per_sm, skinny_min_iters, fused_decode (0|1), prologue_kernel (0|1|2),
 * pair (0 = never the CTA-pair kernel, 1 = always, 192|256 = always with that tile width),
 * int8_mma (0 = the INT8-surrogate matmul never uses INT8 tensor-core instructions),
 * gemv (0 = one to four tokens never take the CUDA-core GEMV, 1 = wherever it is supported).
 * Process-wide and not synchronised with launches in flight on other threads. */
int oq_set_tunable(const char *name, int value);

/* ---- bit stream --------------------------------------------------------------------- */

/* Unpack `count` little-endian `bits`-wide fields of `packed` into one byte each.
 * Replaces unpack_lowbit on CUDA tensors (src/orbitquant/packing/bitpack.py:63-97,
 * src/orbitquant/kernels/triton_cuda.py:879-923).  Bit-exact. */
int oq_unpack_lowbit(const uint8_t *packed, int bits, int64_t count, uint8_t *values,
                     void *stream);

/* Inverse of oq_unpack_lowbit; writes ceil(count*bits/8) bytes.  Replaces pack_lowbit on
 * CUDA tensors (bitpack.py:49-60).  Bit-exact. */
int oq_pack_lowbit(const uint8_t *values, int bits, int64_t count, uint8_t *packed,
                   void *stream);

/* Dense weight W[n,k] = f32(row_norm[n]) * centroid[idx[n,k]], written as `out_dtype`.
 * Replaces OrbitQuantLinear._dequantize_weight on CUDA
 * (src/orbitquant/layers.py:1001-1070, triton_cuda.py:524-547). */
int oq_dequantize_weight(const uint8_t *packed, int bits, int64_t out_features,
                         int64_t in_features, const void *row_norms_bf16,
                         const float *centroids, void *out, int out_dtype, void *stream);

/* ---- online activation quantisation ------------------------------------------------- */

/* Fused RPBH rotate-and-quantize of `rows` tokens of width `dim`:
 *   n = ||x||_2 (fp32), s = x[perm]*sign/(n+eps), per-`block` Walsh-Hadamard, /sqrt(block),
 *   idx = #{boundaries < s}, x_q = centroid[idx]*n rounded to x's dtype.
 * The fp32 operation order (16-lane fused-multiply-add sum of squares folded 8/4/2/1,
 * multiply by the reciprocal, radix-2 stages h=1,2,4,...) is the one of the reference's
 * AVX-512 CPU kernel, so x_q is bit-identical to it.
 * Replaces quantize_activations_cpu
 * (native-kernels/orbitquant-packed-matmul/orbitquant_packed_matmul_cpu/
 *  quantize_activations_cpu.cpp:633-664,731-867; op schema torch-ext/torch_binding.cpp:12-15)
 * and the CUDA/Triton prologues (orbitquant_packed_matmul_cuda/packed_matmul.cu:581-742,
 * src/orbitquant/kernels/triton_cuda.py:221-357).
 *   x, x_q   : [rows, dim] contiguous, dtype x_dtype (x_q may be NULL)
 *   perm     : int32[dim]; signs: int8[dim] (+1/-1)
 *   block    : power of two dividing dim
 *   boundaries: f32[2^bits-1] ascending; centroids: f32[2^bits]
 *   codes    : optional u8[rows, dim] (the indices); norms: optional f32[rows] */
int oq_quantize_activations(const void *x, int x_dtype, int64_t rows, int64_t dim,
                            const int32_t *perm, const int8_t *signs, int64_t block,
                            const float *boundaries, const float *centroids, int bits,
                            float eps, void *x_q, uint8_t *codes, float *norms, void *stream);

/* The same pipeline with the output forms the reference's integer matmul consumes
 * (op schemas torch-ext/torch_binding.cpp:32-62):
 *
 * oq_quantize_activations_packed_w4: 4-bit activation indices packed two per byte (low
 * nibble = even k) into packed_out[rows, dim/2] plus the token norms f32[rows].  Replaces
 * quantize_activations_packed_w4 (orbitquant_packed_matmul_cuda/packed_matmul.cu:581-657,
 * host :1894-2023; src/orbitquant/kernels/triton_cuda.py:290-357); any block dividing dim is
 * accepted, not only block == dim.  The indices are the ones of oq_quantize_activations
 * (reference CPU AVX-512 order).  The workspace holds the unpacked indices.
 *
 * oq_quantize_activations_int8: codes_out[rows, dim] = act_codes[index] (int8) plus the
 * token norms -- the INT8 surrogate activation stream.  Replaces quantize_activations_int8
 * (packed_matmul.cu:659-742, host :2025-2164). */
size_t oq_quantize_activations_packed_w4_workspace_bytes(int64_t rows, int64_t dim);
int oq_quantize_activations_packed_w4(const void *x, int x_dtype, int64_t rows, int64_t dim,
                                      const int32_t *perm, const int8_t *signs, int64_t block,
                                      const float *boundaries, const float *centroids, float eps,
                                      uint8_t *packed_out, float *norms_out, void *workspace,
                                      size_t workspace_bytes, void *stream);
int oq_quantize_activations_int8(const void *x, int x_dtype, int64_t rows, int64_t dim,
                                 const int32_t *perm, const int8_t *signs, int64_t block,
                                 const float *boundaries, const float *centroids, int bits,
                                 const int8_t *act_codes, float eps, int8_t *codes_out,
                                 float *norms_out, void *stream);

/* ---- packed-weight matmul ----------------------------------------------------------- */

/* out[m,n] = sum_k x[m,k] * W[n,k] (+ bias[n]),  W decoded on the fly from the packed
 * `bits`-wide codebook indices (row-major [out_features, in_features] bit stream).
 * Replaces the native op matmul_packed_weight
 * (schema torch-ext/torch_binding.cpp:9-11; CUDA host packed_matmul.cu:1335-1713;
 *  CPU packed_matmul_cpu.cpp:115-201; Python wrapper
 *  torch-ext/orbitquant_packed_matmul/__init__.py:109-160).
 *   x        : [rows, in_features] contiguous, dtype `dtype` (the quantised activations)
 *   packed   : u8, at least ceil(out_features*in_features*bits/8) bytes (packed_bytes is
 *              checked, as the reference checks numel)
 *   row_norms: bf16[out_features]; centroids: f32[2^bits]
 *   bias     : NULL or [out_features] of dtype `bias_dtype`
 *   out      : [rows, out_features] contiguous, dtype `dtype`
 *   workspace: see oq_matmul_workspace_bytes (may be NULL when that returns 0) */
int oq_matmul_packed_weight(void *out, const void *x, int dtype, int64_t rows,
                            int64_t in_features, int64_t out_features, const uint8_t *packed,
                            int64_t packed_bytes, int bits, const void *row_norms_bf16,
                            const float *centroids, const void *bias, int bias_dtype,
                            int weight_mode, int kernel, void *workspace,
                            size_t workspace_bytes, void *stream);

size_t oq_matmul_workspace_bytes(int64_t rows, int64_t in_features, int64_t out_features,
                                 int bits, int dtype, int weight_mode, int kernel);

/* 1 when the tcgen05/TMEM kernel can run this problem (bf16 activations, 2/3/4/6/8-bit
 * weights, in_features % 64 == 0, centroid weight mode), else 0. */
int oq_gemm_tcgen05_supported(int64_t rows, int64_t in_features, int64_t out_features,
                              int bits, int dtype, int weight_mode);

/* The tcgen05 kernel alone, on an activation operand that is already in its f16 form:
 * x_f16[m,k] = f16(x[m,k] / row_scale[m]) with row_scale[m] an exact power of two (what
 * oq_linear_forward's prologue writes into the workspace, and what oq_matmul_packed_weight
 * derives from a caller-supplied x).  table_scale points at the scale of the kernel's f16
 * weight table f16(centroid * scale), chosen by oq_rows_to_f16_operand (NULL: 2^8).
 * out is bf16.  Same reference counterpart as oq_matmul_packed_weight; exposed so that
 * tests and the benchmark can time and check the GEMM kernel in isolation.  Requires
 * oq_gemm_tcgen05_supported(...) == 1. */
int oq_gemm_tcgen05_f16(void *out, const void *x_f16, const float *row_scale,
                        const float *table_scale, int64_t rows, int64_t in_features,
                        int64_t out_features, const uint8_t *packed, int64_t packed_bytes, int bits,
                        const void *row_norms_bf16, const float *centroids, const void *bias,
                        int bias_dtype, void *stream);

/* x (bf16 or f16, [rows, dim]) -> the f16 operand and per-token factors used above.  When
 * table_scale is not NULL the kernel also searches the weight-table scale for the codebook
 * `centroids` (f32[2^bits]) and writes it there (one float). */
int oq_rows_to_f16_operand(const void *x, int dtype, int64_t rows, int64_t dim, void *x_f16,
                           float *row_scale, const float *centroids, int bits,
                           float *table_scale, void *stream);

/* ---- integer-index formulations --------------------------------------------------- */

/* INT8-surrogate matmul: out[m, n] = (sum_k act_codes[a[m,k]] * weight_codes[w[n,k]])
 *   * token_norms[m] * row_norm[n] * act_scale * weight_scale + bias[n], bf16 output.
 * packed_act is the nibble stream of oq_quantize_activations_packed_w4; the weights are the
 * ordinary packed stream (2, 3, 4 or 6 bits); the code tables and scales come from the
 * reference's fit_int8_centroid_surrogate (src/orbitquant/kernels/triton_cuda.py:1826-1857).
 * Replaces matmul_packed_w4a4_int8 (packed_matmul.cu:744-1009, host :1715-1892) and the
 * fused Triton kernels (triton_cuda.py:1861-2099).  Approximate by construction (the codes
 * are rounded centroids); the integer contraction itself is exact: above 128 rows of a 4-bit
 * layer with in_features % 128 == 0 it runs on the INT8 tensor-core instructions with int32
 * accumulators (tunable int8_mma = 0 switches that off), otherwise on the f16 tensor cores,
 * where INT8 codes, their products and sums below 2^24 are exact.
 * Three launches (code table, operand expansion, GEMM); in_features % 64 == 0. */
size_t oq_matmul_packed_w4a4_int8_workspace_bytes(int64_t rows, int64_t in_features);
int oq_matmul_packed_w4a4_int8(void *out, const uint8_t *packed_act, const uint8_t *packed_weight,
                               int64_t packed_weight_bytes, int weight_bits, const float *token_norms,
                               const void *row_norms_bf16, const int8_t *act_codes,
                               const int8_t *weight_codes, const void *bias, int bias_dtype,
                               float act_scale, float weight_scale, int64_t rows, int64_t in_features,
                               int64_t out_features, void *workspace, size_t workspace_bytes,
                               void *stream);

/* The whole INT8-surrogate W4A4 linear in three launches (code table, rotate + quantise
 * straight to the INT8 operand, INT8 tensor-core GEMM): out = the result of
 * oq_quantize_activations_packed_w4 followed by oq_matmul_packed_w4a4_int8, without the packed
 * intermediate.  Replaces the reference module's fused INT8 route
 * (src/orbitquant/layers.py:1097-1352 calling quantize_activations_int8 and the fused kernels of
 * src/orbitquant/kernels/triton_cuda.py:1861-2099).  bf16 output.  oq_linear_w4a4_int8_supported
 * returns 1 for the problems it takes: bf16 x, rows > 128, in_features % 256 == 0, a rotation
 * block of 256 .. 4096 dividing in_features, 4-bit weights; other problems go through the two
 * calls above. */
int oq_linear_w4a4_int8_supported(int dtype, int64_t rows, int64_t in_features, int64_t out_features,
                                  int64_t block);
size_t oq_linear_w4a4_int8_workspace_bytes(int64_t rows, int64_t in_features);
int oq_linear_w4a4_int8(void *out, const void *x, int dtype, int64_t rows, int64_t in_features,
                        int64_t out_features, const uint8_t *packed_weight, int64_t packed_weight_bytes,
                        const void *row_norms_bf16, const void *bias, int bias_dtype, const int32_t *perm,
                        const int8_t *signs, int64_t block, const float *act_boundaries,
                        const float *act_centroids, const int8_t *act_codes, const int8_t *weight_codes,
                        float act_scale, float weight_scale, float eps, void *workspace,
                        size_t workspace_bytes, void *stream);

/* Exact W4A4 linear through the 256-entry pair-product table:
 *   out[m, n] = (sum_k pair_lut[16 * a[m,k] + w[n,k]]) * token_norm[m] * row_norm[n] + bias[n]
 * in fp32, rounded to x's dtype, pair_lut[16 i + j] = act_centroid[i] * weight_centroid[j].
 * Replaces orbitquant_vulkan::linear_w4a4_exact, i.e. the arithmetic of
 * _linear_w4a4_exact_reference (src/orbitquant/kernels/executorch_vulkan.py:15-61; the shader
 * native-kernels/orbitquant-vulkan/glsl/orbitquant_w4a4_lut_tiled.glsl computes the same).
 * The table entries are added in ascending k by one thread per output element; the
 * activation indices are those of oq_quantize_activations. */
size_t oq_linear_w4a4_pair_lut_workspace_bytes(int64_t rows, int64_t in_features);
int oq_linear_w4a4_pair_lut(void *out, const void *x, int dtype, int64_t rows, int64_t in_features,
                            int64_t out_features, const uint8_t *packed, int64_t packed_bytes,
                            const void *row_norms_bf16, const void *bias, int bias_dtype,
                            const int32_t *perm, const int8_t *signs, int64_t block,
                            const float *act_boundaries, const float *act_centroids,
                            const float *pair_lut, float eps, void *workspace, size_t workspace_bytes,
                            void *stream);

/* ---- the whole quantized-linear forward --------------------------------------------- */

/* Names of the kernels oq_linear_forward launches for a problem (static string; "a + b" =
 * two launches).  The reference reports the same decision after the fact through
 * OrbitQuantLinear.last_effective_runtime_mode / last_activation_kernel_backend
 * (src/orbitquant/layers.py:1079-1455); here it can be asked up front. */
const char *oq_linear_kernel_name(int64_t rows, int64_t in_features, int64_t out_features,
                                  int weight_bits, int act_bits, int64_t block, int dtype,
                                  int weight_mode, int kernel);

/* y = OrbitQuantLinear(x): oq_quantize_activations into workspace, then
 * oq_matmul_packed_weight.  Replaces OrbitQuantLinear._forward_impl on CUDA
 * (src/orbitquant/layers.py:1079-1455), i.e. the body of the custom op
 * orbitquant::packed_linear_forward (layers.py:59-72).
 * The workspace (oq_linear_workspace_bytes) holds the quantised activations
 * [rows, in_features] of x's dtype plus whatever the chosen matmul kernel needs. */
int oq_linear_forward(void *out, const void *x, int dtype, int64_t rows, int64_t in_features,
                      int64_t out_features, const uint8_t *packed, int64_t packed_bytes,
                      int weight_bits, const void *row_norms_bf16, const float *weight_centroids,
                      const void *bias, int bias_dtype, const int32_t *perm,
                      const int8_t *signs, int64_t block, const float *act_boundaries,
                      const float *act_centroids, int act_bits, float eps, int weight_mode,
                      int kernel, void *workspace, size_t workspace_bytes, void *stream);

size_t oq_linear_workspace_bytes(int64_t rows, int64_t in_features, int64_t out_features,
                                 int weight_bits, int dtype, int weight_mode, int kernel);

/* ---- offline weight quantise-and-pack --------------------------------------------------- */

/* W [out_features, in_features] (row-major, any of the three dtypes) -> the packed index
 * stream and the bf16 row norms a layer stores.  Replaces the reference's weight path
 * (src/orbitquant/layers.py:102-222; on CUDA its Triton kernels, triton_cuda.py:2849-2935):
 * index = bucketize( (fwht(W[n, perm] * signs) * 1/sqrt(block)) / max(norm_n, eps) ), packed
 * little-endian.  With `row_norms_in` (f32 [out_features]) the indices are bit-identical to
 * the reference's torch CPU expression evaluated with those norms; with NULL the norms are
 * computed here (double accumulation, rounded once to f32), which may differ from a given
 * fp32 reduction order in the last bit.  `centroids` is the codebook's table (unused by the
 * indices; kept for a uniform interface).  Workspace: oq_quantize_weight_workspace_bytes
 * (one byte per weight + the f32 norms). */
int oq_quantize_weight(const void *weight, int dtype, int64_t out_features, int64_t in_features,
                       const int32_t *perm, const int8_t *signs, int64_t block,
                       const float *boundaries, const float *centroids, int bits, float eps,
                       const float *row_norms_in, void *row_norms_bf16_out, uint8_t *packed_out,
                       void *workspace, size_t workspace_bytes, void *stream);

size_t oq_quantize_weight_workspace_bytes(int64_t out_features, int64_t in_features);

/* ---- RTN-INT4 linear (AdaLN modulation layers) ------------------------------------------- */

/* out[m, n] = bf16( sum_k x[m, k] * bf16((code[n, k] - 8) * scale[n, k / 64]) + bias[n] ),
 * fp32 accumulation: the reference's RTNInt4Linear forward (src/orbitquant/adaln.py:294-430)
 * in the arithmetic of its CPU kernel (orbitquant_packed_matmul_cpu/packed_adaln_cpu.cpp:54-100).
 * x, out: bf16 row-major; packed: 4-bit codes, two per byte (low nibble = even k), every row
 * padded to ceil(in_features / 64) * 64 values; scales_bf16: [out_features, ceil(K / 64)];
 * group_size must be 64; in_features a multiple of 8.  Runs on the few-token tensor-core
 * kernel (bf16 x bf16), 128 rows per launch. */
int oq_rtn_int4_linear_forward(void *out, const void *x_bf16, int64_t rows, int64_t in_features,
                               int64_t out_features, const uint8_t *packed, int64_t packed_bytes,
                               const void *scales_bf16, int group_size, const void *bias,
                               int bias_dtype, void *workspace, size_t workspace_bytes, void *stream);

size_t oq_rtn_int4_workspace_bytes(int64_t rows, int64_t in_features, int64_t out_features);

/* ---- column-sharded layers: forward with the all-gather in the epilogue ----------------- */

/* oq_linear_forward whose result tile is stored into EVERY one of `n_outs` (1..8) row-major
 * bf16 buffers, each [rows, out_ld] with this call's columns starting at `out_col`.  A layer
 * sharded along its output features over several GPUs passes its own full-width buffer and
 * the peer-mapped address of the same buffer on every other GPU (symmetric memory / CUDA
 * IPC): the kernel's epilogue stores each finished tile over NVLink while the next tiles are
 * still being computed, and no all-gather collective follows.  The caller synchronises the
 * ranks afterwards (every peer's stores must have landed before a rank reads its buffer).
 * The reference has no multi-GPU path for this operator; its closest counterpart is the
 * torch.distributed all-gather a caller would run on the column shards
 * (orbitquant_b200/sharding.py: gather_columns).  Exists in the large-row tcgen05 kernel
 * only: bf16, rows > 128, in_features % 64 == 0, centroid weight arithmetic; other
 * problems return OQ_ERR_UNSUPPORTED.  out_ld, out_col and out_features multiples of 8
 * keep the stores 16 bytes wide.  Workspace: oq_linear_workspace_bytes(..., OQ_KERNEL_TCGEN05). */
int oq_linear_forward_scatter(void *const *outs, int n_outs, int64_t out_ld, int64_t out_col,
                              const void *x, int dtype, int64_t rows, int64_t in_features,
                              int64_t out_features, const uint8_t *packed, int64_t packed_bytes,
                              int weight_bits, const void *row_norms_bf16,
                              const float *weight_centroids, const void *bias, int bias_dtype,
                              const int32_t *perm, const int8_t *signs, int64_t block,
                              const float *act_boundaries, const float *act_centroids,
                              int act_bits, float eps, void *workspace, size_t workspace_bytes,
                              void *stream);

/* ---- no-allocation variant ------------------------------------------------------------ */

/* oq_linear_forward for callers that cannot allocate device memory at all -- plugin code
 * running inside another runtime's enqueue callback, programs that gave all GPU memory to
 * one pool at start-up.  Same arguments as oq_linear_forward without the workspace: the
 * scratch for the quantised activations is a fixed 4 MiB device array inside the library
 * image (oq_static_scratch_bytes()), so the call performs no cudaMalloc / cudaFree and uses
 * no allocating library routine.  This entry point has no counterpart in the reference.
 *
 *  - Limit: oq_linear_workspace_bytes(...) for the problem must not exceed
 *    oq_static_scratch_bytes() (about rows * in_features * 2 <= 4 MiB, e.g. 128 tokens of
 *    16384 features); larger problems return OQ_ERR_WORKSPACE with a message and run nothing.
 *  - Cost: every GPU on which the library is loaded holds the 4 MiB until the process exits.
 *  - The first call on each device looks the array's device address up
 *    (cudaGetSymbolAddress, with that device current) and caches it.  That lookup may load
 *    the library's device code on that device and allocate inside the driver, so make one
 *    warm-up call per device at start-up: outside the region that must not allocate and
 *    before any stream capture begins.
 *  - The cached address does not survive cudaDeviceReset or any other re-creation of the
 *    device's primary context; do not use this entry point in a process after that.
 *  - All calls on a device share the one array, which keeps the previous call's contents.
 *    Nothing in it needs clearing between calls (each call overwrites all it reads), but two
 *    calls that overlap on the GPU (different streams, or concurrent graph branches) race
 *    on it: serialise them. */
size_t oq_static_scratch_bytes(void);
int oq_linear_forward_static(void *out, const void *x, int dtype, int64_t rows,
                             int64_t in_features, int64_t out_features, const uint8_t *packed,
                             int64_t packed_bytes, int weight_bits, const void *row_norms_bf16,
                             const float *weight_centroids, const void *bias, int bias_dtype,
                             const int32_t *perm, const int8_t *signs, int64_t block,
                             const float *act_boundaries, const float *act_centroids,
                             int act_bits, float eps, int weight_mode, int kernel, void *stream);

/* ---- device status ------------------------------------------------------------------- */

/* Every wait inside the tcgen05 kernel (on an mbarrier) is bounded; a wait that gives up
 * records a non-zero code in a per-device status word, releases its tensor memory and
 * returns instead of hanging.  *status receives that word (0 = every wait completed).
 * This call copies from the device and therefore synchronises; it is meant for tests and
 * debugging, not for the forward path.  No counterpart in the reference (its kernels have
 * no device-side waits). */
int oq_gemm_device_status(int *status);
int oq_gemm_clear_device_status(void);

#ifdef __cplusplus
}
#endif
#endif /* ORBIT_B200_H_ */
