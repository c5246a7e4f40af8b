// oq_linear_forward_static: the quantized-linear forward for callers that cannot allocate.
//
// oq_linear_forward needs a caller-provided workspace for the quantised activations that
// travel from the rotate-and-quantize kernel to the matmul kernel.  Some callers have no
// way to provide one: code that runs inside another runtime's enqueue method (an
// inference-engine plugin), where cudaMalloc and every allocating library routine are off
// limits, and C programs that hand the GPU's whole memory to one pool at start-up and have
// no allocator left on the hot path.  For them this file holds the workspace itself, as a
// fixed-size device array that is part of the loaded library image.
//
// The first call on a device looks the array's address up (cudaGetSymbolAddress), which may
// load the library's device code on that device and so may allocate inside the driver: make
// one warm-up call per device at start-up, outside the region that must not allocate and
// before any stream capture.  The address is cached per device index for the life of the
// process; after cudaDeviceReset (or any re-creation of the device's primary context) the
// cached address is stale and this entry point must not be used again in that process.
#include <mutex>

#include "common.cuh"

namespace oq {
namespace {

// The scratch area.  Fixed size, so every GPU on which this library is loaded carries these
// 4 MiB from load to process exit, used or not.
constexpr size_t kStaticScratchBytes = size_t(4) << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_scratch_mutex;
void *g_scratch_address[kMaxDevices] = {};

// In host code `g_static_scratch` is only a handle for the runtime, not a device address;
// the address a kernel can use comes from cudaGetSymbolAddress, asked once per device with
// that device current.
int static_scratch_for_current_device(void **address) {
  int device = 0;
  OQ_CHECK_CUDA(cudaGetDevice(&device));
  if (device < 0 || device >= kMaxDevices) {
    return fail(OQ_ERR_UNSUPPORTED, "device index %d is outside the supported range", device);
  }
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_address[device] == nullptr) {
    void *ptr = nullptr;
    OQ_CHECK_CUDA(cudaGetSymbolAddress(&ptr, g_static_scratch));
    if (ptr == nullptr) {
      return fail(OQ_ERR_CUDA, "cudaGetSymbolAddress returned a null address for the static scratch");
    }
    g_scratch_address[device] = ptr;
  }
  *address = g_scratch_address[device];
  return OQ_OK;
}

}  // namespace
}  // namespace oq

using namespace oq;

extern "C" {

size_t oq_static_scratch_bytes(void) { return kStaticScratchBytes; }

int oq_linear_forward_static(void *out, const void *x, int dtype, int64_t rows, int64_t in_features,
                             int64_t out_features, const uint8_t *packed, int64_t packed_bytes,
                             int weight_bits, const void *row_norms_bf16,
                             const float *weight_centroids, const void *bias, int bias_dtype,
                             const int32_t *perm, const int8_t *signs, int64_t block,
                             const float *act_boundaries, const float *act_centroids, int act_bits,
                             float eps, int weight_mode, int kernel, void *stream) {
  OQ_CHECK_ARG(valid_dtype(dtype), "x must be float32, float16, or bfloat16");
  OQ_CHECK_ARG(rows >= 0 && in_features > 0 && out_features >= 0, "negative or empty shape");
  const size_t need = oq_linear_workspace_bytes(rows, in_features, out_features, weight_bits, dtype,
                                                weight_mode, kernel);
  if (need > kStaticScratchBytes) {
    return fail(OQ_ERR_WORKSPACE,
                "this problem needs %zu bytes of scratch but the built-in scratch holds %zu "
                "(rows * in_features * 2 must stay below about 4 MiB); use oq_linear_forward "
                "with a caller-provided workspace instead",
                need, kStaticScratchBytes);
  }
  if (int rc = check_device()) {  // before the symbol lookup: a foreign device gets OQ_ERR_DEVICE
    return rc;
  }
  void *scratch = nullptr;
  if (int rc = static_scratch_for_current_device(&scratch)) {
    return rc;
  }
  // Nothing in the scratch has to start at zero on entry: the first kernel overwrites every
  // byte the second one reads (activations and per-token factors of exactly `rows` tokens)
  // and clears the reduction-slice counters the few-token kernel keeps there.
  return oq_linear_forward(out, x, dtype, rows, in_features, out_features, packed, packed_bytes,
                           weight_bits, row_norms_bf16, weight_centroids, bias, bias_dtype, perm,
                           signs, block, act_boundaries, act_centroids, act_bits, eps, weight_mode,
                           kernel, scratch, kStaticScratchBytes, stream);
}

}  // extern "C"
