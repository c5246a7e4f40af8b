// extern "C" surface of liborbit_b200.so: argument validation, kernel choice, status.
#include <cstdlib>
#include <cstring>
#include <strings.h>
#include <mutex>

#include "common.cuh"

namespace oq {

thread_local char g_last_error[512] = "";
std::atomic<uint64_t> g_launch_count{0};

namespace {
const char *const kTunableNames[OQ_TUNE_COUNT] = {
    "TILE_N", "TILE_ORDER", "SKINNY", "STREAM_ROWS", "PROLOGUE_ROWS", "SKINNY_UNITS_PER_SM",
    "SKINNY_MIN_ITERS", "FUSED_DECODE", "PROLOGUE_KERNEL", "PAIR", "INT8_MMA", "GEMV"};
std::atomic<int> g_tunables[OQ_TUNE_COUNT];
std::once_flag g_tunables_once;

void init_tunables() {
  std::call_once(g_tunables_once, [] {
    for (int i = 0; i < OQ_TUNE_COUNT; ++i) {
      char name[64];
      snprintf(name, sizeof(name), "ORBIT_B200_%s", kTunableNames[i]);
      const char *env = std::getenv(name);
      g_tunables[i].store(env == nullptr ? -1 : std::atoi(env), std::memory_order_relaxed);
    }
  });
}
}  // namespace

int tunable(int which) {
  init_tunables();
  return g_tunables[which].load(std::memory_order_relaxed);
}

int fail(int status, const char *format, ...) {
  va_list args;
  va_start(args, format);
  vsnprintf(g_last_error, sizeof(g_last_error), format, args);
  va_end(args);
  return status;
}

int launch_rotate_quantize(const void *x, int x_dtype, int64_t rows, int64_t dim,
                           const int32_t *perm, const int8_t *signs, int64_t block,
                           const float *boundaries, const float *centroids, int bits, float eps,
                           void *x_q, uint8_t *codes, float *norms, float *f16_row_scale,
                           const float *w_centroids, int w_bits, float *table_scale_out,
                           int *zero_words, int zero_count, cudaStream_t stream,
                           const float *given_norms = nullptr, const int8_t *code_map = nullptr);
bool tcgen05_i8_supported(int64_t rows, int64_t in_features, int64_t out_features, int bits);
int launch_tcgen05_gemm_i8(void *out, const void *a_int8, const float *row_scale, const float *table_scale,
                           int64_t rows, int64_t in_features, int64_t out_features, const uint8_t *packed,
                           const void *row_norms_bf16, const float *code_floats, const void *bias,
                           int bias_dtype, cudaStream_t stream);
int launch_expand_packed_a4_int8(const uint8_t *packed_act, const float *token_norms, const int8_t *act_codes,
                                 const int8_t *w_codes, int w_levels, float scale, int64_t rows, int64_t dim,
                                 void *out_int8, float *row_scale, float *table_scale, float *w_code_floats,
                                 cudaStream_t stream);
int launch_write_code_table(const int8_t *w_codes, int w_levels, float *table_scale, float *w_code_floats,
                            cudaStream_t stream);
bool int8_operand_prologue_supported(int x_dtype, int64_t dim, int64_t block);
int launch_rotate_quantize_int8_operand(const void *x, int x_dtype, int64_t rows, int64_t dim,
                                        const int32_t *perm, const int8_t *signs, int64_t block,
                                        const float *boundaries, const float *centroids, int bits, float eps,
                                        const int8_t *code_map, float out_scale, int8_t *out,
                                        float *row_scale, cudaStream_t stream);
int launch_expand_packed_a4(const uint8_t *packed_act, const float *token_norms, const int8_t *act_codes,
                            const int8_t *w_codes, int w_levels, float scale, int64_t rows, int64_t dim,
                            void *out_f16, float *row_scale, float *table_scale, float *w_code_floats,
                            cudaStream_t stream);
int launch_pair_lut(void *out, int out_dtype, const uint8_t *codes, const float *token_norms,
                    const uint8_t *packed, const void *row_norms_bf16, const float *pair_lut,
                    const void *bias, int bias_dtype, int64_t rows, int64_t in_features,
                    int64_t out_features, cudaStream_t stream);
int launch_weight_row_norms(const void *w, int dtype, int64_t rows, int64_t dim, float *norms_f32,
                            void *norms_bf16, cudaStream_t stream);
int launch_norms_to_bf16(const float *norms, int64_t rows, void *out, cudaStream_t stream);
int launch_tiled_matmul(void *out, const void *x, int dtype, int64_t rows, int64_t in_features,
                        int64_t out_features, const uint8_t *packed, int bits,
                        const void *row_norms_bf16, const float *centroids, const void *bias,
                        int bias_dtype, int weight_mode, cudaStream_t stream);
int launch_small_rows(void *out, const void *x, int dtype, int64_t rows, int64_t in_features,
                      int64_t out_features, const uint8_t *packed, int bits,
                      const void *row_norms_bf16, const float *centroids, const void *bias,
                      int bias_dtype, int weight_mode, cudaStream_t stream);
bool small_rows_supported(int64_t rows, int64_t in_features, int64_t out_features, int bits,
                          int dtype, int weight_mode);
bool stream_rows_preferred(int64_t rows, int64_t in_features, int64_t out_features, int bits,
                           int dtype);
size_t stream_rows_workspace_bytes(int64_t in_features, int64_t out_features);
int launch_stream_rows(void *out, const void *x, int64_t rows, int64_t in_features,
                       int64_t out_features, const uint8_t *packed, const void *row_norms_bf16,
                       const float *centroids, const void *bias, int bias_dtype, int weight_mode,
                       void *workspace, size_t workspace_bytes, cudaStream_t stream);
int launch_unpack(const uint8_t *packed, int bits, int64_t count, uint8_t *values,
                  cudaStream_t stream);
int launch_pack(const uint8_t *values, int bits, int64_t count, uint8_t *packed,
                cudaStream_t stream);
int launch_dequantize(const uint8_t *packed, int bits, int64_t out_features, int64_t in_features,
                      const void *row_norms_bf16, const float *centroids, void *out,
                      int out_dtype, cudaStream_t stream);
bool tcgen05_gemm_supported(int64_t rows, int64_t in_features, int64_t out_features, int bits,
                            int dtype, int weight_mode);
const char *tcgen05_gemm_kernel_name(int64_t rows, int64_t out_features, int bits);
int launch_rows_to_f16(const void *x, int dtype, int64_t rows, int64_t dim, void *out_f16,
                       float *row_scale, const float *centroids, int bits, float *table_scale_out,
                       int *zero_words, int zero_count, cudaStream_t stream);
int launch_tcgen05_gemm(void *out, const void *x_f16, const float *row_scale,
                        const float *table_scale, int64_t rows, int64_t in_features, int64_t out_features, const uint8_t *packed, int bits,
                        const void *row_norms_bf16, const float *centroids, const void *bias,
                        int bias_dtype, cudaStream_t stream, bool scaled = false);
bool tcgen05_skinny_supported(int64_t rows, int64_t in_features, int64_t out_features, int bits,
                              int dtype, int weight_mode);
size_t tcgen05_skinny_workspace_bytes(int64_t rows, int64_t in_features, int64_t out_features);
int tcgen05_skinny_counter_words(int64_t rows, int64_t in_features, int64_t out_features);
int launch_tcgen05_skinny(void *out, const void *x_f16, const float *row_scale,
                          const float *table_scale, int64_t rows, int64_t in_features,
                          int64_t out_features, const uint8_t *packed, int bits,
                          const void *row_norms_bf16, const float *centroids, const void *bias,
                          int bias_dtype, void *workspace, size_t workspace_bytes,
                          cudaStream_t stream);
int launch_tcgen05_gemm_scatter(void *const *outs, int n_outs, int64_t out_ld, int64_t out_col,
                                const void *x_f16, const float *row_scale, const float *table_scale,
                                int64_t rows, int64_t in_features, int64_t out_features,
                                const uint8_t *packed, int bits, const void *row_norms_bf16,
                                const float *centroids, const void *bias, int bias_dtype,
                                cudaStream_t stream, bool scaled = false);
size_t tcgen05_rtn_workspace_bytes(int64_t rows, int64_t in_features, int64_t out_features);
int launch_tcgen05_rtn_int4(void *out, const void *x_bf16, int64_t rows, int64_t in_features,
                            int64_t out_features, const uint8_t *packed, const void *scales_bf16,
                            const void *bias, int bias_dtype, void *workspace,
                            size_t workspace_bytes, cudaStream_t stream);
bool gemv_w4_supported(int64_t rows, int64_t in_features, int64_t out_features, int bits, int dtype,
                       int weight_mode);
int launch_gemv_w4(void *out, const void *x, int64_t rows, int64_t in_features, int64_t out_features,
                   const uint8_t *packed, const void *row_norms_bf16, const float *centroids,
                   const void *bias, int bias_dtype, cudaStream_t stream);
bool decode_fused_supported(int64_t rows, int64_t in_features, int64_t out_features, int weight_bits,
                            int act_bits, int dtype, int64_t block);
int launch_decode_fused(void *out, const void *x, int64_t rows, int64_t in_features, int64_t out_features,
                        const uint8_t *packed, const void *row_norms_bf16, const float *w_centroids,
                        const void *bias, int bias_dtype, const int32_t *perm, const int8_t *signs,
                        int64_t block, const float *act_boundaries, const float *act_centroids,
                        int act_bits, float eps, int weight_mode, cudaStream_t stream);
int read_gemm_status(int *status);
int clear_gemm_status();
int read_prologue_status(int *status);
int clear_prologue_status();

// The kernels are built for sm_100a only; refuse anything else before a launch fails with
// "no kernel image".
int check_device() {
  static thread_local int checked_device = -1;
  int device = 0;
  OQ_CHECK_CUDA(cudaGetDevice(&device));
  if (device == checked_device) {
    return OQ_OK;
  }
  int major = 0;
  OQ_CHECK_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
  if (major != 10) {
    return fail(OQ_ERR_DEVICE, "orbit_b200 kernels are built for sm_100a; device %d is sm_%d", device,
                major * 10);
  }
  checked_device = device;
  return OQ_OK;
}

namespace {

int resolve_weight_mode(int weight_mode) {
  return weight_mode == OQ_WEIGHT_AUTO ? OQ_WEIGHT_CENTROID : weight_mode;
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Within the tcgen05 family: up to 128 rows go to the operand-swapped few-token kernel.
// The skinny tunable set to 0 keeps them on the large-row kernel (for A/B timing).
bool use_skinny(int64_t rows, int64_t in_features, int64_t out_features, int bits, int dtype, int mode) {
  return tunable(OQ_TUNE_SKINNY) != 0 &&
         tcgen05_skinny_supported(rows, in_features, out_features, bits, dtype, mode);
}

// Within the small-rows family: one to four tokens on a layer of megabytes go to the CUDA-core
// GEMV, whose cost per weight is the lowest there.  The gemv tunable set to 0 / 1 forces never /
// wherever it is supported (for A/B timing).
bool use_gemv(int64_t rows, int64_t in_features, int64_t out_features, int bits, int dtype, int mode) {
  const int forced = tunable(OQ_TUNE_GEMV);
  if (forced == 0 || !gemv_w4_supported(rows, in_features, out_features, bits, dtype, mode)) {
    return false;
  }
  return forced > 0 || out_features * in_features / 2 >= (int64_t(3) << 20);
}

// Kernel for a problem: the caller's explicit choice, or by shape.
int choose_kernel(int kernel, int64_t rows, int64_t in_features, int64_t out_features, int bits,
                  int dtype, int mode) {
  if (kernel != OQ_KERNEL_AUTO) {
    return kernel;
  }
  if (use_gemv(rows, in_features, out_features, bits, dtype, mode)) {
    return OQ_KERNEL_SMALL_ROWS;
  }
  const int64_t weight_bytes = out_features * in_features * bits / 8;
  const bool skinny = use_skinny(rows, in_features, out_features, bits, dtype, mode);
  if (rows <= 16 && small_rows_supported(rows, in_features, out_features, bits, dtype, mode) &&
      (!skinny || weight_bytes < (int64_t(3) << 20))) {
    // one launch, lowest latency; large layers in this mode stream through the persistent variant
    return OQ_KERNEL_SMALL_ROWS;
  }
  // few tokens on the tensor cores: any bit width, layers of a megabyte and more (below that
  // the set-up of a tcgen05 kernel costs more than the general kernel's whole run)
  if (skinny && (rows > 16 || weight_bytes >= (int64_t(1) << 20))) {
    return OQ_KERNEL_TCGEN05;
  }
  if (rows > 16 && tcgen05_gemm_supported(rows, in_features, out_features, bits, dtype, mode)) {
    return OQ_KERNEL_TCGEN05;
  }
  return OQ_KERNEL_TILED;
}

// Within the small-rows family: large layers go to the persistent streaming kernel.
// The stream_rows tunable set to 0 / 1 forces one or the other (for A/B timing).
bool use_stream_rows(int64_t rows, int64_t in_features, int64_t out_features, int bits, int dtype) {
  const int forced = tunable(OQ_TUNE_STREAM_ROWS);
  if (forced == 0) {
    return false;
  }
  const bool fits = stream_rows_preferred(rows, in_features, out_features, bits, dtype);
  if (forced > 0) {
    return rows >= 1 && rows <= 16 && bits == 4 && dtype == OQ_DTYPE_BF16 && in_features % 128 == 0;
  }
  return fits;
}

// Decode-sized batches on small layers: the whole forward in one launch (decode_fused.cuh).
// The fused_decode tunable set to 0 keeps the two-kernel path (for A/B timing).
bool use_fused_decode(int kernel, int64_t rows, int64_t in_features, int64_t out_features, int weight_bits,
                      int act_bits, int dtype, int64_t block) {
  return kernel == OQ_KERNEL_AUTO && tunable(OQ_TUNE_FUSED_DECODE) != 0 &&
         decode_fused_supported(rows, in_features, out_features, weight_bits, act_bits, dtype, block);
}

// Bytes of the f16 operand [rows, K] (256-aligned); the per-token factors follow it.
size_t f16_operand_bytes(int64_t rows, int64_t in_features) {
  return align_up(static_cast<size_t>(rows) * in_features * 2, 256);
}

// Workspace of the tcgen05 family: f16 operand | per-token factors + table scale | partial
// sums of the few-token kernel's reduction slices.
size_t tcgen05_head_bytes(int64_t rows, int64_t in_features) {
  return f16_operand_bytes(rows, in_features) + align_up(static_cast<size_t>(rows + 1) * 4, 256);
}

size_t tcgen05_workspace_bytes(int64_t rows, int64_t in_features, int64_t out_features, int bits,
                               int dtype, int mode) {
  size_t bytes = tcgen05_head_bytes(rows, in_features);
  if (use_skinny(rows, in_features, out_features, bits, dtype, mode)) {
    bytes += tcgen05_skinny_workspace_bytes(rows, in_features, out_features);
  }
  return bytes;
}

// The few-token kernel's slice counters (head of its part of the workspace) have to be
// cleared by the kernel that prepares the operand; NULL / 0 when there are none.
int *tcgen05_counters(void *workspace, int64_t rows, int64_t in_features, int64_t out_features,
                      int bits, int dtype, int mode, int *count) {
  *count = 0;
  if (!use_skinny(rows, in_features, out_features, bits, dtype, mode) ||
      tcgen05_skinny_workspace_bytes(rows, in_features, out_features) == 0) {
    return nullptr;
  }
  *count = tcgen05_skinny_counter_words(rows, in_features, out_features);
  return reinterpret_cast<int *>(static_cast<unsigned char *>(workspace) +
                                 tcgen05_head_bytes(rows, in_features));
}

// GEMM on the prepared operand at the head of `workspace`.
int tcgen05_matmul(void *out, void *workspace, size_t workspace_bytes, int64_t rows,
                   int64_t in_features, int64_t out_features, const uint8_t *packed, int bits,
                   int dtype, int mode, const void *row_norms_bf16, const float *centroids,
                   const void *bias, int bias_dtype, cudaStream_t s) {
  float *row_scale = reinterpret_cast<float *>(static_cast<unsigned char *>(workspace) +
                                               f16_operand_bytes(rows, in_features));
  float *table_scale = row_scale + rows;  // one float after the per-token factors
  if (use_skinny(rows, in_features, out_features, bits, dtype, mode)) {
    const size_t head = tcgen05_head_bytes(rows, in_features);
    return launch_tcgen05_skinny(out, workspace, row_scale, table_scale, rows, in_features,
                                 out_features, packed, bits, row_norms_bf16, centroids, bias,
                                 bias_dtype, static_cast<unsigned char *>(workspace) + head,
                                 workspace_bytes - head, s);
  }
  // bf16_scaled: the operand at the head of the workspace is x_q itself (bf16, not rescaled)
  return launch_tcgen05_gemm(out, workspace, row_scale, table_scale, rows, in_features,
                             out_features, packed, bits, row_norms_bf16, centroids, bias,
                             bias_dtype, s, mode == OQ_WEIGHT_BF16_SCALED);
}

}  // namespace
}  // namespace oq

using namespace oq;

extern "C" {

int oq_abi_version(void) { return OQ_ABI_VERSION; }

const char *oq_last_error(void) { return g_last_error; }

uint64_t oq_launch_count(void) { return g_launch_count.load(std::memory_order_relaxed); }

int oq_set_tunable(const char *name, int value) {
  OQ_CHECK_ARG(name != nullptr, "null tunable name");
  init_tunables();
  for (int i = 0; i < OQ_TUNE_COUNT; ++i) {
    if (strcasecmp(name, kTunableNames[i]) == 0) {
      g_tunables[i].store(value, std::memory_order_relaxed);
      return OQ_OK;
    }
  }
  return fail(OQ_ERR_INVALID, "unknown tunable '%s'", name);
}

int oq_unpack_lowbit(const uint8_t *packed, int bits, int64_t count, uint8_t *values, void *stream) {
  OQ_CHECK_ARG(bits >= 1 && bits <= 8, "bits must be in [1, 8]");
  OQ_CHECK_ARG(count >= 0, "length must be non-negative");
  if (count == 0) {
    return OQ_OK;
  }
  OQ_CHECK_ARG(packed != nullptr && values != nullptr, "null device pointer");
  if (int rc = check_device()) {
    return rc;
  }
  return launch_unpack(packed, bits, count, values, static_cast<cudaStream_t>(stream));
}

int oq_pack_lowbit(const uint8_t *values, int bits, int64_t count, uint8_t *packed, void *stream) {
  OQ_CHECK_ARG(bits >= 1 && bits <= 8, "bits must be in [1, 8]");
  OQ_CHECK_ARG(count >= 0, "length must be non-negative");
  if (count == 0) {
    return OQ_OK;
  }
  OQ_CHECK_ARG(packed != nullptr && values != nullptr, "null device pointer");
  if (int rc = check_device()) {
    return rc;
  }
  return launch_pack(values, bits, count, packed, static_cast<cudaStream_t>(stream));
}

int oq_dequantize_weight(const uint8_t *packed, int bits, int64_t out_features, int64_t in_features,
                         const void *row_norms_bf16, const float *centroids, void *out,
                         int out_dtype, void *stream) {
  OQ_CHECK_ARG(bits >= 1 && bits <= 8, "bits must be in [1, 8]");
  OQ_CHECK_ARG(valid_dtype(out_dtype), "out must be float32, float16, or bfloat16");
  OQ_CHECK_ARG(out_features >= 0 && in_features >= 0, "negative shape");
  if (out_features == 0 || in_features == 0) {
    return OQ_OK;
  }
  OQ_CHECK_ARG(packed && row_norms_bf16 && centroids && out, "null device pointer");
  if (int rc = check_device()) {
    return rc;
  }
  return launch_dequantize(packed, bits, out_features, in_features, row_norms_bf16, centroids, out,
                           out_dtype, static_cast<cudaStream_t>(stream));
}

int oq_quantize_activations(const void *x, int x_dtype, int64_t rows, int64_t dim,
                            const int32_t *perm, const int8_t *signs, int64_t block,
                            const float *boundaries, const float *centroids, int bits, float eps,
                            void *x_q, uint8_t *codes, float *norms, void *stream) {
  if (int rc = check_device()) {
    return rc;
  }
  return launch_rotate_quantize(x, x_dtype, rows, dim, perm, signs, block, boundaries, centroids,
                                bits, eps, x_q, codes, norms, nullptr, nullptr, 0, nullptr, nullptr, 0,
                                static_cast<cudaStream_t>(stream));
}

size_t oq_quantize_activations_packed_w4_workspace_bytes(int64_t rows, int64_t dim) {
  return rows <= 0 || dim <= 0 ? 0 : align_up(static_cast<size_t>(rows) * dim, 256);
}

int oq_quantize_activations_packed_w4(const void *x, int x_dtype, int64_t rows, int64_t dim,
                                      const int32_t *perm, const int8_t *signs, int64_t block,
                                      const float *boundaries, const float *centroids, float eps,
                                      uint8_t *packed_out, float *norms_out, void *workspace,
                                      size_t workspace_bytes, void *stream) {
  OQ_CHECK_ARG(dim % 2 == 0, "the packed 4-bit output needs an even in_features");
  if (rows == 0) {
    return OQ_OK;
  }
  OQ_CHECK_ARG(packed_out != nullptr && norms_out != nullptr, "null device pointer");
  const size_t need = oq_quantize_activations_packed_w4_workspace_bytes(rows, dim);
  if (workspace == nullptr || workspace_bytes < need) {
    return fail(OQ_ERR_WORKSPACE, "workspace of %zu bytes given, %zu needed", workspace_bytes, need);
  }
  if (int rc = check_device()) {
    return rc;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint8_t *codes = static_cast<uint8_t *>(workspace);
  if (int rc = launch_rotate_quantize(x, x_dtype, rows, dim, perm, signs, block, boundaries, centroids,
                                      4, eps, nullptr, codes, norms_out, nullptr, nullptr, 0, nullptr,
                                      nullptr, 0, s)) {
    return rc;
  }
  return launch_pack(codes, 4, rows * dim, packed_out, s);
}

int oq_quantize_activations_int8(const void *x, int x_dtype, int64_t rows, int64_t dim,
                                 const int32_t *perm, const int8_t *signs, int64_t block,
                                 const float *boundaries, const float *centroids, int bits,
                                 const int8_t *act_codes, float eps, int8_t *codes_out,
                                 float *norms_out, void *stream) {
  if (rows == 0) {
    return OQ_OK;
  }
  OQ_CHECK_ARG(act_codes != nullptr && codes_out != nullptr && norms_out != nullptr, "null device pointer");
  if (int rc = check_device()) {
    return rc;
  }
  return launch_rotate_quantize(x, x_dtype, rows, dim, perm, signs, block, boundaries, centroids, bits,
                                eps, nullptr, reinterpret_cast<uint8_t *>(codes_out), norms_out, nullptr,
                                nullptr, 0, nullptr, nullptr, 0, static_cast<cudaStream_t>(stream),
                                nullptr, act_codes);
}

size_t oq_matmul_packed_w4a4_int8_workspace_bytes(int64_t rows, int64_t in_features) {
  if (rows <= 0 || in_features <= 0) {
    return 0;
  }
  return tcgen05_head_bytes(rows, in_features) + 256 * sizeof(float);
}

int oq_matmul_packed_w4a4_int8(void *out, const uint8_t *packed_act, const uint8_t *packed_weight,
                               int64_t packed_weight_bytes, int weight_bits, const float *token_norms,
                               const void *row_norms_bf16, const int8_t *act_codes,
                               const int8_t *weight_codes, const void *bias, int bias_dtype,
                               float act_scale, float weight_scale, int64_t rows, int64_t in_features,
                               int64_t out_features, void *workspace, size_t workspace_bytes,
                               void *stream) {
  OQ_CHECK_ARG(rows >= 0 && in_features > 0 && out_features >= 0, "negative or empty shape");
  OQ_CHECK_ARG(weight_bits == 2 || weight_bits == 3 || weight_bits == 4 || weight_bits == 6,
               "the INT8 surrogate exists for 2-, 3-, 4- and 6-bit weights");
  OQ_CHECK_ARG(bias == nullptr || valid_dtype(bias_dtype), "bias must be float32, float16, or bfloat16");
  OQ_CHECK_ARG(packed_weight_bytes >= (out_features * in_features * weight_bits + 7) / 8,
               "packed weights are too short");
  if (rows == 0 || out_features == 0) {
    return OQ_OK;
  }
  OQ_CHECK_ARG(out && packed_act && packed_weight && token_norms && row_norms_bf16 && act_codes && weight_codes,
               "null device pointer");
  if (!tcgen05_gemm_supported(rows, in_features, out_features, weight_bits, OQ_DTYPE_BF16, OQ_WEIGHT_CENTROID)) {
    return fail(OQ_ERR_UNSUPPORTED, "the INT8-surrogate matmul needs in_features %% 64 == 0");
  }
  const size_t need = oq_matmul_packed_w4a4_int8_workspace_bytes(rows, in_features);
  if (workspace == nullptr || workspace_bytes < need) {
    return fail(OQ_ERR_WORKSPACE, "workspace of %zu bytes given, %zu needed", workspace_bytes, need);
  }
  OQ_CHECK_ARG(aligned16(workspace), "workspace must be 16-byte aligned");
  if (int rc = check_device()) {
    return rc;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  unsigned char *ws = static_cast<unsigned char *>(workspace);
  float *row_scale = reinterpret_cast<float *>(ws + f16_operand_bytes(rows, in_features));
  float *table_scale = row_scale + rows;
  float *code_floats = reinterpret_cast<float *>(ws + tcgen05_head_bytes(rows, in_features));
  // Large batches of a W4 layer: INT8 operands on the tensor cores (kind::i8), the integer
  // contraction the reference's kernels perform (packed_matmul.cu:744-1009), exact in int32.
  if (tcgen05_i8_supported(rows, in_features, out_features, weight_bits) && tunable(OQ_TUNE_INT8_MMA) != 0) {
    if (int rc = launch_expand_packed_a4_int8(packed_act, token_norms, act_codes, weight_codes,
                                              1 << weight_bits, act_scale * weight_scale, rows, in_features,
                                              workspace, row_scale, table_scale, code_floats, s)) {
      return rc;
    }
    return launch_tcgen05_gemm_i8(out, workspace, row_scale, table_scale, rows, in_features, out_features,
                                  packed_weight, row_norms_bf16, code_floats, bias, bias_dtype, s);
  }
  if (int rc = launch_expand_packed_a4(packed_act, token_norms, act_codes, weight_codes, 1 << weight_bits,
                                       act_scale * weight_scale, rows, in_features, workspace, row_scale,
                                       table_scale, code_floats, s)) {
    return rc;
  }
  // integer codes are exact in f16; the table scale is 1 and the per-token factor carries
  // token_norm * s_a * s_w, so the ordinary epilogue computes the surrogate's
  return launch_tcgen05_gemm(out, workspace, row_scale, table_scale, rows, in_features, out_features,
                             packed_weight, weight_bits, row_norms_bf16, code_floats, bias, bias_dtype, s);
}

int oq_linear_w4a4_int8_supported(int dtype, int64_t rows, int64_t in_features, int64_t out_features,
                                  int64_t block) {
  return tcgen05_i8_supported(rows, in_features, out_features, 4) &&
                 int8_operand_prologue_supported(dtype, in_features, block) && tunable(OQ_TUNE_INT8_MMA) != 0
             ? 1
             : 0;
}

size_t oq_linear_w4a4_int8_workspace_bytes(int64_t rows, int64_t in_features) {
  return oq_matmul_packed_w4a4_int8_workspace_bytes(rows, in_features);
}

int oq_linear_w4a4_int8(void *out, const void *x, int dtype, int64_t rows, int64_t in_features,
                        int64_t out_features, const uint8_t *packed_weight, int64_t packed_weight_bytes,
                        const void *row_norms_bf16, const void *bias, int bias_dtype, const int32_t *perm,
                        const int8_t *signs, int64_t block, const float *act_boundaries,
                        const float *act_centroids, const int8_t *act_codes, const int8_t *weight_codes,
                        float act_scale, float weight_scale, float eps, void *workspace,
                        size_t workspace_bytes, void *stream) {
  OQ_CHECK_ARG(rows >= 0 && in_features > 0 && out_features >= 0, "negative or empty shape");
  OQ_CHECK_ARG(bias == nullptr || valid_dtype(bias_dtype), "bias must be float32, float16, or bfloat16");
  OQ_CHECK_ARG(packed_weight_bytes >= (out_features * in_features * 4 + 7) / 8, "packed weights are too short");
  if (rows == 0 || out_features == 0) {
    return OQ_OK;
  }
  OQ_CHECK_ARG(out && x && packed_weight && row_norms_bf16 && act_codes && weight_codes, "null device pointer");
  if (!oq_linear_w4a4_int8_supported(dtype, rows, in_features, out_features, block)) {
    return fail(OQ_ERR_UNSUPPORTED,
                "the fused INT8-surrogate linear takes bf16 rows, more than 128 of them, in_features %% 256 == 0 "
                "and a rotation block of 256 .. 4096");
  }
  const size_t need = oq_linear_w4a4_int8_workspace_bytes(rows, in_features);
  if (workspace == nullptr || workspace_bytes < need) {
    return fail(OQ_ERR_WORKSPACE, "workspace of %zu bytes given, %zu needed", workspace_bytes, need);
  }
  OQ_CHECK_ARG(aligned16(workspace), "workspace must be 16-byte aligned");
  if (int rc = check_device()) {
    return rc;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  unsigned char *ws = static_cast<unsigned char *>(workspace);
  float *row_scale = reinterpret_cast<float *>(ws + f16_operand_bytes(rows, in_features));
  float *table_scale = row_scale + rows;
  float *code_floats = reinterpret_cast<float *>(ws + tcgen05_head_bytes(rows, in_features));
  if (int rc = launch_write_code_table(weight_codes, 16, table_scale, code_floats, s)) {
    return rc;
  }
  if (int rc = launch_rotate_quantize_int8_operand(x, dtype, rows, in_features, perm, signs, block,
                                                   act_boundaries, act_centroids, 4, eps, act_codes,
                                                   act_scale * weight_scale, reinterpret_cast<int8_t *>(ws),
                                                   row_scale, s)) {
    return rc == OQ_ERR_UNSUPPORTED ? fail(rc, "the INT8-operand prologue does not take this problem") : rc;
  }
  return launch_tcgen05_gemm_i8(out, workspace, row_scale, table_scale, rows, in_features, out_features,
                                packed_weight, row_norms_bf16, code_floats, bias, bias_dtype, s);
}

size_t oq_linear_w4a4_pair_lut_workspace_bytes(int64_t rows, int64_t in_features) {
  if (rows <= 0 || in_features <= 0) {
    return 0;
  }
  return align_up(static_cast<size_t>(rows) * in_features, 256) + align_up(static_cast<size_t>(rows) * 4, 256);
}

int oq_linear_w4a4_pair_lut(void *out, const void *x, int dtype, int64_t rows, int64_t in_features,
                            int64_t out_features, const uint8_t *packed, int64_t packed_bytes,
                            const void *row_norms_bf16, const void *bias, int bias_dtype,
                            const int32_t *perm, const int8_t *signs, int64_t block,
                            const float *act_boundaries, const float *act_centroids,
                            const float *pair_lut, float eps, void *workspace, size_t workspace_bytes,
                            void *stream) {
  OQ_CHECK_ARG(valid_dtype(dtype), "x must be float32, float16, or bfloat16");
  OQ_CHECK_ARG(rows >= 0 && in_features > 0 && out_features >= 0, "negative or empty shape");
  OQ_CHECK_ARG(in_features % 2 == 0, "in_features must be even");
  OQ_CHECK_ARG(bias == nullptr || valid_dtype(bias_dtype), "bias must be float32, float16, or bfloat16");
  OQ_CHECK_ARG(packed_bytes >= out_features * in_features / 2, "packed weights are too short");
  if (rows == 0 || out_features == 0) {
    return OQ_OK;
  }
  OQ_CHECK_ARG(out && x && packed && row_norms_bf16 && pair_lut, "null device pointer");
  const size_t need = oq_linear_w4a4_pair_lut_workspace_bytes(rows, in_features);
  if (workspace == nullptr || workspace_bytes < need) {
    return fail(OQ_ERR_WORKSPACE, "workspace of %zu bytes given, %zu needed", workspace_bytes, need);
  }
  if (int rc = check_device()) {
    return rc;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint8_t *codes = static_cast<uint8_t *>(workspace);
  float *norms = reinterpret_cast<float *>(static_cast<unsigned char *>(workspace) +
                                           align_up(static_cast<size_t>(rows) * in_features, 256));
  if (int rc = launch_rotate_quantize(x, dtype, rows, in_features, perm, signs, block, act_boundaries,
                                      act_centroids, 4, eps, nullptr, codes, norms, nullptr, nullptr, 0,
                                      nullptr, nullptr, 0, s)) {
    return rc;
  }
  return launch_pair_lut(out, dtype, codes, norms, packed, row_norms_bf16, pair_lut, bias, bias_dtype,
                         rows, in_features, out_features, s);
}

int oq_gemm_tcgen05_supported(int64_t rows, int64_t in_features, int64_t out_features, int bits,
                              int dtype, int weight_mode) {
  return tcgen05_gemm_supported(rows, in_features, out_features, bits, dtype,
                                resolve_weight_mode(weight_mode))
             ? 1
             : 0;
}

size_t oq_matmul_workspace_bytes(int64_t rows, int64_t in_features, int64_t out_features, int bits,
                                 int dtype, int weight_mode, int kernel) {
  if (rows <= 0 || in_features <= 0 || out_features <= 0) {
    return 0;
  }
  const int mode = resolve_weight_mode(weight_mode);
  const int chosen = choose_kernel(kernel, rows, in_features, out_features, bits, dtype, mode);
  if (chosen == OQ_KERNEL_SMALL_ROWS && use_stream_rows(rows, in_features, out_features, bits, dtype)) {
    return stream_rows_workspace_bytes(in_features, out_features);
  }
  if (chosen != OQ_KERNEL_TCGEN05) {
    return 0;
  }
  return tcgen05_workspace_bytes(rows, in_features, out_features, bits, dtype, mode);
}

int oq_matmul_packed_weight(void *out, const void *x, int dtype, int64_t rows, int64_t in_features,
                            int64_t out_features, const uint8_t *packed, int64_t packed_bytes,
                            int bits, const void *row_norms_bf16, const float *centroids,
                            const void *bias, int bias_dtype, int weight_mode, int kernel,
                            void *workspace, size_t workspace_bytes, void *stream) {
  OQ_CHECK_ARG(bits >= 1 && bits <= 8, "bits must be in [1, 8]");
  OQ_CHECK_ARG(valid_dtype(dtype), "x must be float32, float16, or bfloat16");
  OQ_CHECK_ARG(rows >= 0 && in_features > 0 && out_features >= 0, "negative or empty shape");
  OQ_CHECK_ARG(weight_mode >= OQ_WEIGHT_AUTO && weight_mode <= OQ_WEIGHT_BF16_SCALED,
               "unknown weight_mode %d", weight_mode);
  OQ_CHECK_ARG(kernel >= OQ_KERNEL_AUTO && kernel <= OQ_KERNEL_TCGEN05, "unknown kernel %d", kernel);
  OQ_CHECK_ARG(bias == nullptr || valid_dtype(bias_dtype), "bias must be float32, float16, or bfloat16");
  const int64_t needed = (out_features * in_features * bits + 7) / 8;
  OQ_CHECK_ARG(packed_bytes >= needed, "packed weights are too short");
  if (rows == 0 || out_features == 0) {
    return OQ_OK;
  }
  OQ_CHECK_ARG(out && x && packed && row_norms_bf16 && centroids, "null device pointer");
  if (int rc = check_device()) {
    return rc;
  }
  const int mode = resolve_weight_mode(weight_mode);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int chosen = choose_kernel(kernel, rows, in_features, out_features, bits, dtype, mode);
  switch (chosen) {
    case OQ_KERNEL_SMALL_ROWS:
      if (!small_rows_supported(rows, in_features, out_features, bits, dtype, mode)) {
        return fail(OQ_ERR_UNSUPPORTED, "the small-rows kernel does not take this problem");
      }
      if (use_gemv(rows, in_features, out_features, bits, dtype, mode)) {
        return launch_gemv_w4(out, x, rows, in_features, out_features, packed, row_norms_bf16, centroids,
                              bias, bias_dtype, s);
      }
      if (use_stream_rows(rows, in_features, out_features, bits, dtype)) {
        return launch_stream_rows(out, x, rows, in_features, out_features, packed, row_norms_bf16,
                                  centroids, bias, bias_dtype, mode, workspace, workspace_bytes, s);
      }
      return launch_small_rows(out, x, dtype, rows, in_features, out_features, packed, bits,
                               row_norms_bf16, centroids, bias, bias_dtype, mode, s);
    case OQ_KERNEL_TCGEN05:
      if (!tcgen05_gemm_supported(rows, in_features, out_features, bits, dtype, mode)) {
        return fail(OQ_ERR_UNSUPPORTED,
                    "the tcgen05 kernel takes bf16 activations, in_features %% 64 == 0 and "
                    "2/3/4/6/8-bit weights (2/3/4-bit in the bf16_scaled weight mode)");
      }
      if (mode == OQ_WEIGHT_BF16_SCALED) {
        // both operands bf16: the caller's activations are the A operand as they are
        OQ_CHECK_ARG(aligned16(x), "x must be 16-byte aligned");
        return launch_tcgen05_gemm(out, x, nullptr, nullptr, rows, in_features, out_features, packed,
                                   bits, row_norms_bf16, centroids, bias, bias_dtype, s, true);
      }
      {
        const size_t need = oq_matmul_workspace_bytes(rows, in_features, out_features, bits, dtype,
                                                      mode, OQ_KERNEL_TCGEN05);
        if (workspace == nullptr || workspace_bytes < need) {
          return fail(OQ_ERR_WORKSPACE, "workspace of %zu bytes given, %zu needed", workspace_bytes, need);
        }
        OQ_CHECK_ARG(aligned16(workspace), "workspace must be 16-byte aligned");
        float *row_scale = reinterpret_cast<float *>(static_cast<unsigned char *>(workspace) +
                                                     f16_operand_bytes(rows, in_features));
        float *table_scale = row_scale + rows;  // one float after the per-token factors
        int zero_count = 0;
        int *zero_words = tcgen05_counters(workspace, rows, in_features, out_features, bits, dtype,
                                           mode, &zero_count);
        if (int rc = launch_rows_to_f16(x, dtype, rows, in_features, workspace, row_scale, centroids,
                                        bits, table_scale, zero_words, zero_count, s)) {
          return rc;
        }
        return tcgen05_matmul(out, workspace, workspace_bytes, rows, in_features, out_features,
                              packed, bits, dtype, mode, row_norms_bf16, centroids, bias, bias_dtype, s);
      }
    default:
      return launch_tiled_matmul(out, x, dtype, rows, in_features, out_features, packed, bits,
                                 row_norms_bf16, centroids, bias, bias_dtype, mode, s);
  }
}

int oq_gemm_tcgen05_f16(void *out, const void *x_f16, const float *row_scale,
                        const float *table_scale, int64_t rows,
                        int64_t in_features, int64_t out_features, const uint8_t *packed,
                        int64_t packed_bytes, int bits, const void *row_norms_bf16,
                        const float *centroids, const void *bias, int bias_dtype, void *stream) {
  OQ_CHECK_ARG(rows >= 0 && in_features > 0 && out_features >= 0, "negative or empty shape");
  OQ_CHECK_ARG(bits >= 1 && bits <= 8, "bits must be in [1, 8]");
  OQ_CHECK_ARG(bias == nullptr || valid_dtype(bias_dtype), "bias must be float32, float16, or bfloat16");
  OQ_CHECK_ARG(packed_bytes >= (out_features * in_features * bits + 7) / 8, "packed weights are too short");
  if (rows == 0 || out_features == 0) {
    return OQ_OK;
  }
  OQ_CHECK_ARG(out && x_f16 && row_scale && packed && row_norms_bf16 && centroids, "null device pointer");
  if (!tcgen05_gemm_supported(rows, in_features, out_features, bits, OQ_DTYPE_BF16, OQ_WEIGHT_CENTROID)) {
    return fail(OQ_ERR_UNSUPPORTED, "the tcgen05 kernel needs 2/3/4/6/8-bit weights and in_features %% 64 == 0");
  }
  if (int rc = check_device()) {
    return rc;
  }
  return launch_tcgen05_gemm(out, x_f16, row_scale, table_scale, rows, in_features, out_features,
                             packed, bits,
                             row_norms_bf16, centroids, bias, bias_dtype,
                             static_cast<cudaStream_t>(stream));
}

int oq_rows_to_f16_operand(const void *x, int dtype, int64_t rows, int64_t dim, void *x_f16,
                           float *row_scale, const float *centroids, int bits,
                           float *table_scale, void *stream) {
  OQ_CHECK_ARG(rows >= 0 && dim > 0, "negative or empty shape");
  if (rows == 0) {
    return OQ_OK;
  }
  OQ_CHECK_ARG(x && x_f16 && row_scale, "null device pointer");
  if (int rc = check_device()) {
    return rc;
  }
  return launch_rows_to_f16(x, dtype, rows, dim, x_f16, row_scale, centroids, bits, table_scale,
                            nullptr, 0, static_cast<cudaStream_t>(stream));
}

size_t oq_linear_workspace_bytes(int64_t rows, int64_t in_features, int64_t out_features,
                                 int weight_bits, int dtype, int weight_mode, int kernel) {
  if (rows <= 0 || in_features <= 0 || out_features <= 0) {
    return 0;
  }
  const int mode = resolve_weight_mode(weight_mode);
  if (choose_kernel(kernel, rows, in_features, out_features, weight_bits, dtype, mode) ==
      OQ_KERNEL_TCGEN05) {
    // the prologue writes the f16 operand and its per-token factors straight into it
    return tcgen05_workspace_bytes(rows, in_features, out_features, weight_bits, dtype, mode);
  }
  // quantised activations, then whatever the matmul kernel wants for itself
  return align_up(static_cast<size_t>(rows) * in_features * dtype_size(dtype), 256) +
         oq_matmul_workspace_bytes(rows, in_features, out_features, weight_bits, dtype, weight_mode,
                                   kernel == OQ_KERNEL_AUTO ? OQ_KERNEL_AUTO : kernel);
}

const char *oq_linear_kernel_name(int64_t rows, int64_t in_features, int64_t out_features,
                                  int weight_bits, int act_bits, int64_t block, int dtype,
                                  int weight_mode, int kernel) {
  if (rows <= 0 || in_features <= 0 || out_features <= 0) {
    return "none";
  }
  const int mode = resolve_weight_mode(weight_mode);
  switch (choose_kernel(kernel, rows, in_features, out_features, weight_bits, dtype, mode)) {
    case OQ_KERNEL_SMALL_ROWS:
      if (use_gemv(rows, in_features, out_features, weight_bits, dtype, mode)) {
        return "rotate_quantize + gemv_w4_kernel";
      }
      if (use_fused_decode(kernel, rows, in_features, out_features, weight_bits, act_bits, dtype, block)) {
        return "decode_fused_kernel";
      }
      return use_stream_rows(rows, in_features, out_features, weight_bits, dtype)
                 ? "rotate_quantize + stream_rows_w4_kernel"
                 : "rotate_quantize + small_rows_w4_kernel";
    case OQ_KERNEL_TCGEN05:
      if (use_skinny(rows, in_features, out_features, weight_bits, dtype, mode)) {
        return "rotate_quantize + skinny_tcgen05_kernel";
      }
      return tcgen05_gemm_kernel_name(rows, out_features, weight_bits)[5] == 'p'
                 ? "rotate_quantize + gemm_pair_tcgen05_kernel"
                 : "rotate_quantize + gemm_w4_tcgen05_kernel";
    default:
      return "rotate_quantize + tiled_matmul_kernel";
  }
}

int oq_linear_forward(void *out, const void *x, int dtype, int64_t rows, int64_t in_features,
                      int64_t out_features, const uint8_t *packed, int64_t packed_bytes,
                      int weight_bits, const void *row_norms_bf16, const float *weight_centroids,
                      const void *bias, int bias_dtype, const int32_t *perm, const int8_t *signs,
                      int64_t block, const float *act_boundaries, const float *act_centroids,
                      int act_bits, float eps, int weight_mode, int kernel, void *workspace,
                      size_t workspace_bytes, void *stream) {
  OQ_CHECK_ARG(valid_dtype(dtype), "x must be float32, float16, or bfloat16");
  OQ_CHECK_ARG(rows >= 0 && in_features > 0 && out_features >= 0, "negative or empty shape");
  OQ_CHECK_ARG(weight_bits >= 1 && weight_bits <= 8, "bits must be in [1, 8]");
  OQ_CHECK_ARG(weight_mode >= OQ_WEIGHT_AUTO && weight_mode <= OQ_WEIGHT_BF16_SCALED,
               "unknown weight_mode %d", weight_mode);
  OQ_CHECK_ARG(kernel >= OQ_KERNEL_AUTO && kernel <= OQ_KERNEL_TCGEN05, "unknown kernel %d", kernel);
  OQ_CHECK_ARG(bias == nullptr || valid_dtype(bias_dtype), "bias must be float32, float16, or bfloat16");
  const int64_t needed = (out_features * in_features * weight_bits + 7) / 8;
  OQ_CHECK_ARG(packed_bytes >= needed, "packed weights are too short");
  if (rows == 0 || out_features == 0) {
    return OQ_OK;
  }
  const size_t need = oq_linear_workspace_bytes(rows, in_features, out_features, weight_bits, dtype,
                                                weight_mode, kernel);
  if (workspace == nullptr || workspace_bytes < need) {
    return fail(OQ_ERR_WORKSPACE, "workspace of %zu bytes given, %zu needed", workspace_bytes, need);
  }
  OQ_CHECK_ARG(aligned16(workspace), "workspace must be 16-byte aligned");
  if (int rc = check_device()) {
    return rc;
  }
  const int mode = resolve_weight_mode(weight_mode);
  const int chosen = choose_kernel(kernel, rows, in_features, out_features, weight_bits, dtype, mode);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (chosen == OQ_KERNEL_TCGEN05) {
    if (!tcgen05_gemm_supported(rows, in_features, out_features, weight_bits, dtype, mode)) {
      return fail(OQ_ERR_UNSUPPORTED, "the tcgen05 kernel does not take this problem");
    }
    OQ_CHECK_ARG(out && packed && row_norms_bf16 && weight_centroids, "null device pointer");
    float *row_scale = reinterpret_cast<float *>(static_cast<unsigned char *>(workspace) +
                                                 f16_operand_bytes(rows, in_features));
    float *table_scale = row_scale + rows;  // one float after the per-token factors
    int zero_count = 0;
    int *zero_words = tcgen05_counters(workspace, rows, in_features, out_features, weight_bits,
                                       dtype, mode, &zero_count);
    if (mode == OQ_WEIGHT_BF16_SCALED) {
      // x_q in bf16 is the operand; no rescaling, no table scale
      if (int rc = launch_rotate_quantize(x, dtype, rows, in_features, perm, signs, block,
                                          act_boundaries, act_centroids, act_bits, eps, workspace,
                                          nullptr, nullptr, nullptr, nullptr, 0, nullptr, nullptr, 0, s)) {
        return rc;
      }
    } else if (int rc = launch_rotate_quantize(x, dtype, rows, in_features, perm, signs, block,
                                               act_boundaries, act_centroids, act_bits, eps, workspace,
                                               nullptr, nullptr, row_scale, weight_centroids, weight_bits,
                                               table_scale, zero_words, zero_count, s)) {
      return rc;
    }
    return tcgen05_matmul(out, workspace, workspace_bytes, rows, in_features, out_features, packed,
                          weight_bits, dtype, mode, row_norms_bf16, weight_centroids, bias,
                          bias_dtype, s);
  }
  if (chosen == OQ_KERNEL_SMALL_ROWS && !use_gemv(rows, in_features, out_features, weight_bits, dtype, mode) &&
      use_fused_decode(kernel, rows, in_features, out_features, weight_bits, act_bits, dtype, block)) {
    OQ_CHECK_ARG(out && x && packed && row_norms_bf16 && weight_centroids && perm && signs &&
                     act_boundaries && act_centroids, "null device pointer");
    return launch_decode_fused(out, x, rows, in_features, out_features, packed, row_norms_bf16,
                               weight_centroids, bias, bias_dtype, perm, signs, block, act_boundaries,
                               act_centroids, act_bits, eps, mode, s);
  }
  if (int rc = launch_rotate_quantize(x, dtype, rows, in_features, perm, signs, block, act_boundaries,
                                      act_centroids, act_bits, eps, workspace, nullptr, nullptr,
                                      nullptr, nullptr, 0, nullptr, nullptr, 0, s)) {
    return rc;
  }
  const size_t xq_bytes = align_up(static_cast<size_t>(rows) * in_features * dtype_size(dtype), 256);
  return oq_matmul_packed_weight(out, workspace, dtype, rows, in_features, out_features, packed,
                                 packed_bytes, weight_bits, row_norms_bf16, weight_centroids, bias,
                                 bias_dtype, weight_mode, chosen,
                                 static_cast<unsigned char *>(workspace) + xq_bytes,
                                 workspace_bytes - xq_bytes, stream);
}

int oq_linear_forward_scatter(void *const *outs, int n_outs, int64_t out_ld, int64_t out_col,
                              const void *x, int dtype, int64_t rows, int64_t in_features,
                              int64_t out_features, const uint8_t *packed, int64_t packed_bytes,
                              int weight_bits, const void *row_norms_bf16,
                              const float *weight_centroids, const void *bias, int bias_dtype,
                              const int32_t *perm, const int8_t *signs, int64_t block,
                              const float *act_boundaries, const float *act_centroids,
                              int act_bits, float eps, void *workspace, size_t workspace_bytes,
                              void *stream) {
  OQ_CHECK_ARG(outs != nullptr, "null output list");
  OQ_CHECK_ARG(valid_dtype(dtype), "x must be float32, float16, or bfloat16");
  OQ_CHECK_ARG(bias == nullptr || valid_dtype(bias_dtype), "bias must be float32, float16, or bfloat16");
  OQ_CHECK_ARG(rows >= 0 && in_features > 0 && out_features >= 0, "negative or empty shape");
  OQ_CHECK_ARG(weight_bits >= 1 && weight_bits <= 8, "bits must be in [1, 8]");
  const int64_t needed = (out_features * in_features * weight_bits + 7) / 8;
  OQ_CHECK_ARG(packed_bytes >= needed, "packed weights are too short");
  if (rows == 0 || out_features == 0) {
    return OQ_OK;
  }
  if (int rc = check_device()) {
    return rc;
  }
  const int mode = OQ_WEIGHT_CENTROID;
  if (!tcgen05_gemm_supported(rows, in_features, out_features, weight_bits, dtype, mode) ||
      use_skinny(rows, in_features, out_features, weight_bits, dtype, mode)) {
    return fail(OQ_ERR_UNSUPPORTED,
                "the multi-destination epilogue exists in the large-row tcgen05 kernel only "
                "(bf16, more than 128 rows, in_features %% 64 == 0)");
  }
  const size_t need = tcgen05_head_bytes(rows, in_features);
  if (workspace == nullptr || workspace_bytes < need) {
    return fail(OQ_ERR_WORKSPACE, "workspace of %zu bytes given, %zu needed", workspace_bytes, need);
  }
  OQ_CHECK_ARG(aligned16(workspace), "workspace must be 16-byte aligned");
  OQ_CHECK_ARG(packed && row_norms_bf16 && weight_centroids, "null device pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  float *row_scale = reinterpret_cast<float *>(static_cast<unsigned char *>(workspace) +
                                               f16_operand_bytes(rows, in_features));
  float *table_scale = row_scale + rows;
  if (int rc = launch_rotate_quantize(x, dtype, rows, in_features, perm, signs, block, act_boundaries,
                                      act_centroids, act_bits, eps, workspace, nullptr, nullptr,
                                      row_scale, weight_centroids, weight_bits, table_scale, nullptr,
                                      0, s)) {
    return rc;
  }
  return launch_tcgen05_gemm_scatter(outs, n_outs, out_ld, out_col, workspace, row_scale, table_scale,
                                     rows, in_features, out_features, packed, weight_bits,
                                     row_norms_bf16, weight_centroids, bias, bias_dtype, s);
}

size_t oq_quantize_weight_workspace_bytes(int64_t out_features, int64_t in_features) {
  if (out_features <= 0 || in_features <= 0) {
    return 0;
  }
  return align_up(static_cast<size_t>(out_features) * in_features, 256) +
         align_up(static_cast<size_t>(out_features) * 4, 256);
}

int oq_quantize_weight(const void *weight, int dtype, int64_t out_features, int64_t in_features,
                       const int32_t *perm, const int8_t *signs, int64_t block,
                       const float *boundaries, const float *centroids, int bits, float eps,
                       const float *row_norms_in, void *row_norms_bf16_out, uint8_t *packed_out,
                       void *workspace, size_t workspace_bytes, void *stream) {
  OQ_CHECK_ARG(bits >= 1 && bits <= 8, "bits must be in [1, 8]");
  OQ_CHECK_ARG(valid_dtype(dtype), "weight must be float32, float16, or bfloat16");
  OQ_CHECK_ARG(out_features >= 0 && in_features > 0, "negative or empty shape");
  if (out_features == 0) {
    return OQ_OK;
  }
  OQ_CHECK_ARG(weight && row_norms_bf16_out && packed_out, "null device pointer");
  const size_t need = oq_quantize_weight_workspace_bytes(out_features, in_features);
  if (workspace == nullptr || workspace_bytes < need) {
    return fail(OQ_ERR_WORKSPACE, "workspace of %zu bytes given, %zu needed", workspace_bytes, need);
  }
  OQ_CHECK_ARG(aligned16(workspace), "workspace must be 16-byte aligned");
  if (int rc = check_device()) {
    return rc;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint8_t *codes = static_cast<uint8_t *>(workspace);
  float *norms = reinterpret_cast<float *>(static_cast<unsigned char *>(workspace) +
                                           align_up(static_cast<size_t>(out_features) * in_features, 256));
  const float *use_norms = row_norms_in;
  if (row_norms_in == nullptr) {
    if (int rc = launch_weight_row_norms(weight, dtype, out_features, in_features, norms,
                                         row_norms_bf16_out, s)) {
      return rc;
    }
    use_norms = norms;
  } else if (int rc = launch_norms_to_bf16(row_norms_in, out_features, row_norms_bf16_out, s)) {
    return rc;
  }
  if (int rc = launch_rotate_quantize(weight, dtype, out_features, in_features, perm, signs, block,
                                      boundaries, centroids, bits, eps, nullptr, codes, nullptr,
                                      nullptr, nullptr, 0, nullptr, nullptr, 0, s, use_norms)) {
    return rc;
  }
  return launch_pack(codes, bits, out_features * in_features, packed_out, s);
}

size_t oq_rtn_int4_workspace_bytes(int64_t rows, int64_t in_features, int64_t out_features) {
  if (rows <= 0 || in_features <= 0 || out_features <= 0) {
    return 0;
  }
  return tcgen05_rtn_workspace_bytes(rows > 128 ? 128 : rows, in_features, out_features);
}

int oq_rtn_int4_linear_forward(void *out, const void *x_bf16, int64_t rows, int64_t in_features,
                               int64_t out_features, const uint8_t *packed, int64_t packed_bytes,
                               const void *scales_bf16, int group_size, const void *bias,
                               int bias_dtype, void *workspace, size_t workspace_bytes, void *stream) {
  OQ_CHECK_ARG(rows >= 0 && in_features > 0 && out_features >= 0, "negative or empty shape");
  OQ_CHECK_ARG(group_size == 64, "only the group size 64 is implemented");
  OQ_CHECK_ARG(bias == nullptr || valid_dtype(bias_dtype), "bias must be float32, float16, or bfloat16");
  const int64_t groups = (in_features + 63) / 64;
  OQ_CHECK_ARG(packed_bytes >= out_features * groups * 32, "packed weights are too short");
  if (rows == 0 || out_features == 0) {
    return OQ_OK;
  }
  OQ_CHECK_ARG(out && x_bf16 && packed && scales_bf16, "null device pointer");
  if (int rc = check_device()) {
    return rc;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // more than 128 rows: one launch per 128-row slab (these layers see the batch, not the tokens)
  for (int64_t first = 0; first < rows; first += 128) {
    const int64_t slab = rows - first < 128 ? rows - first : 128;
    if (int rc = launch_tcgen05_rtn_int4(static_cast<unsigned char *>(out) + first * out_features * 2,
                                         static_cast<const unsigned char *>(x_bf16) + first * in_features * 2,
                                         slab, in_features, out_features, packed, scales_bf16, bias,
                                         bias_dtype, workspace, workspace_bytes, s)) {
      return rc;
    }
  }
  return OQ_OK;
}

// Status word of the tcgen05 kernel's bounded waits (0 = every wait completed).  Reading
// it synchronises the host with the device; it is meant for tests and debugging.
int oq_gemm_device_status(int *status) {
  OQ_CHECK_ARG(status != nullptr, "null pointer");
  if (int rc = read_gemm_status(status)) {
    return rc;
  }
  if (*status == 0) {  // the rotate-and-quantize kernel's waits report as 100 + code
    int prologue = 0;
    if (int rc = read_prologue_status(&prologue)) {
      return rc;
    }
    *status = prologue != 0 ? 100 + prologue : 0;
  }
  return OQ_OK;
}

int oq_gemm_clear_device_status(void) {
  if (int rc = clear_gemm_status()) {
    return rc;
  }
  return clear_prologue_status();
}

}  // extern "C"
