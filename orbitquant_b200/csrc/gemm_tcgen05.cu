// Codebook-decode GEMM for large row counts on the 5th-generation tensor cores.
//
//   out[m, n] = (sum_k a[m, k] * f16(centroid[idx[n, k]] * 2^8)) * row_scale[m] * row_norm[n] * 2^-8
//               + bias[n],        a[m, k] = f16(xq[m, k] / row_scale[m])
//
// tcgen05.mma kind::f16 takes both operands in ONE 16-bit format, and bf16 cannot hold a
// centroid to better than 2^-9, so both operands are f16: the activations arrive rescaled
// per token by an exact power of two (written by the rotate-and-quantize prologue in its
// f16 operand mode, or by rows_to_f16_kernel below for a caller-supplied x) and the factor
// returns in the epilogue.
//
// One CTA computes a 256 x BN output tile (two 128 x BN fp32 accumulators in tensor
// memory that share every expanded weight tile).  Warp roles:
//
//   warp 8 (one lane)  TMA producer: per 64-wide k step, one bulk tensor copy of the
//                      256 x 64 f16 activation tile (128-byte swizzle) and one of the
//                      BN x 32-byte packed 4-bit weight tile, both signalling `full[s]`.
//   warps 0..7         expanders: read the packed tile from shared memory, turn every 4-bit
//                      index into its f16 centroid with byte-permute lookups in a
//                      register-resident table (16 entries x 2 bytes = 8 registers; no
//                      shared-memory table, so no bank conflicts and no LSU traffic for the
//                      lookup) and write the BN x 64 f16 operand tile in the
//                      128-byte-swizzled K-major layout the MMA descriptor expects; then
//                      `bready[s]`.  After the last k step the same warps run the epilogue.
//   warp 9 (one lane)  MMA issuer: 2 x 4 tcgen05.mma (128 x BN x 16, f16 x f16 -> f32)
//                      per k step, tcgen05.commit to `empty[s]`; the last commit signals
//                      `acc_full`.
//   epilogue           tcgen05.ld of 32 columns at a time, scale by row_norm[n] * 2^-8,
//                      add bias, round to bf16, 16-byte stores.
//
// SCALED variant (2-, 3-, 4-bit): the reference's other weight arithmetic, operand
// bf16(centroid * row_norm[n]) against the bf16 activations themselves (its AVX512-BF16 CPU
// kernel and its CUDA kernels).  Every expander thread owns one weight row for the whole k loop,
// so its register table is simply built from that row's norm; both operands are bf16, nothing
// is rescaled and the epilogue only adds the bias.
//
// Every mbarrier wait is bounded: when a wait gives up it raises the CTA's abort flag
// and the device status word, every role leaves its loop, in-flight bulk copies are
// drained (bounded again), tensor memory is released and the kernel returns.
#include <cuda.h>

#include <algorithm>
#include <cstdlib>
#include <mutex>

#include "common.cuh"
#include "table_scale.cuh"

namespace oq {

__device__ int g_gemm_status = 0;  // 0 = ok; otherwise the code of the first wait that gave up

namespace {

constexpr int kBM = 256;
constexpr int kBK = 64;
constexpr int kEpilogueWarps = 8;  // two accumulators x four TMEM lane quarters
constexpr float kCentroidScale = kTableScaleBase;  // table scale when none was searched
constexpr uint32_t kSpinLimit = 1u << 22;
// rates of the CTA-pair kernel relative to the 256-wide single-CTA tile
constexpr double kPairRate256 = 1.10;
constexpr double kPairRate192 = 0.98;

template <int BN, int BITS>
struct Tile {

  static constexpr bool kI8 = false;                   // 16-bit operands
  static constexpr int kStepElems = kBK;               // k values per pipeline step
  static constexpr int kABytes = kBM * kBK * 2;        // 32 KB
  static constexpr int kBBytes = BN * kBK * 2;         // expanded f16 tile
  static constexpr int kRowBytes = kBK * BITS / 8;     // packed bytes of one weight row per k step
  // 3-bit rows advance by 24 bytes per k step, which no bulk tensor copy can address
  // (16-byte rule); those tiles are read from global memory by the expanders instead.
  // (Reading 4-bit tiles the same way -- skipping the shared-memory round trip of the packed
  // bytes -- measured +1.4 % at 4608 rows with 3072-wide layers and -1.5 % at K = 12288; not
  // worth a second code path.)
  static constexpr bool kPackedByTma = BITS > 4 || (BN == 256 && BITS != 3);
  static constexpr int kPBytes = kPackedByTma ? BN * kRowBytes : 0;  // packed tile
  static constexpr int kLutBytes = BITS == 6 ? 64 * 32 * 2 : (BITS == 8 ? 256 * 8 * 2 : 0);
  // every stage starts 1024-byte aligned (the 128-byte swizzle pattern repeats every 1024 bytes)
  static constexpr int kStageBytes = (kABytes + kBBytes + kPBytes + 1023) / 1024 * 1024;
  static constexpr int kCentFloats = 1 << BITS;
  static constexpr int kHeaderBytes =
      256 /*barriers*/ + 2 * BN * 4 /*scale,bias*/ + kCentFloats * 4 /*centroids*/ + kLutBytes;
  // as many stages as fit in the 227 KB a CTA may use, at most 4
  static constexpr int kFit = (232448 - kHeaderBytes - 1024) / kStageBytes;
  static constexpr int kStages = kFit > 4 ? 4 : kFit;
  static_assert(kStages >= 2, "tile does not fit in shared memory");
  static constexpr int kSmemBytes = kHeaderBytes + 1024 /*alignment slack*/ + kStages * kStageBytes;
  static constexpr int kTmemCols = BN == 128 ? 256 : 512;  // power of two >= 2 * BN
  // expander threads per weight row: the decode of one k step has to finish well inside the
  // MMA time of that step, so rows are split over 2 (or 4) threads
  static constexpr int kTpr = BN == 128 ? (BITS == 3 ? 2 : 4) : 2;
  static constexpr int kExpanderWarps = BN * kTpr / 32;
  static constexpr int kProducerWarp = kExpanderWarps;
  static constexpr int kMmaWarp = kExpanderWarps + 1;
  static constexpr int kThreads = (kExpanderWarps + 2) * 32;
};

constexpr int kMaxOutputs = 8;

struct GemmParams {
  // The result tile is stored into every one of `n_outs` row-major buffers (leading dimension
  // `out_ld` elements, first column `out_col`): the caller's own buffer and, in a
  // column-sharded layer, the same buffer on each peer GPU -- the all-gather of the shards
  // happens in the epilogue, tile by tile, instead of in a collective afterwards.
  void *outs[kMaxOutputs];
  int n_outs;
  int64_t out_ld;
  int64_t out_col;
  const uint8_t *packed;   // the bit stream (read directly only by the 3-bit expanders)
  const float *row_scale;  // per token: factor the f16 activations were divided by
  const float *table_scale;  // scale of the f16 weight table (NULL: 2^8)
  const __nv_bfloat16 *row_norms;
  const float *centroids;
  const void *bias;
  int bias_dtype;  // -1 none
  int64_t rows;
  int64_t out_features;
  int k_iters;
  int m_tiles;
  int n_tiles;
  // Tile order.  0: consecutive CTAs walk the row tiles of one column tile (they share the
  // weight tile); 1: they walk the column tiles of one row tile (they share the activation
  // tile).  The second keeps DRAM traffic minimal when the activations do not fit in L2: every
  // activation row tile is then read once while the whole weight matrix stays L2-resident.
  int columns_fastest;
};

// ---- PTX wrappers ------------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}

// Non-blocking test (try_wait may suspend the thread for a while even when it then succeeds).
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}

// Bounded wait.  Returns false (after raising the abort flag) when the barrier did not
// flip within the spin limit or another role has already aborted.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag,
                                          int code) {
  if (mbar_test_wait(bar, parity)) {
    return true;
  }
  for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
    if (mbar_try_wait(bar, parity)) {
      return true;
    }
    if ((spin & 63u) == 63u && *abort_flag != 0) {
      return false;
    }
  }
  *abort_flag = code;
  atomicCAS(&g_gemm_status, 0, code);
  return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar,
                                            int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
               "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols)
               : "memory");
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                         uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}

__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
        "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
        "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes (64 16-bit
// values) with the 128-byte swizzle: 8-row groups are 1024 bytes apart (stride byte
// offset), the leading byte offset is unused for this layout, descriptor version 1.
__device__ __forceinline__ uint64_t smem_desc_k_sw128(uint32_t addr) {
  uint64_t desc = 0;
  desc |= static_cast<uint64_t>((addr & 0x3ffffu) >> 4);
  desc |= static_cast<uint64_t>(1) << 16;            // leading byte offset (ignored)
  desc |= static_cast<uint64_t>(1024 >> 4) << 32;    // stride byte offset
  desc |= static_cast<uint64_t>(1) << 46;            // descriptor version
  desc |= static_cast<uint64_t>(2) << 61;            // 128-byte swizzle
  return desc;
}

// Instruction descriptor: f32 accumulator, A = B = f16 (format code 0) or bf16 (1), K-major,
// M = 128.
__host__ __device__ constexpr uint32_t instr_desc(int n, bool bf16_operands = false) {
  return (1u << 4)                                   // D format f32
         | ((bf16_operands ? 1u : 0u) << 7)          // A format
         | ((bf16_operands ? 1u : 0u) << 10)         // B format
         | (static_cast<uint32_t>(n >> 3) << 17)
         | (static_cast<uint32_t>(128 >> 4) << 24);
}

__device__ __forceinline__ float load_bias(const void *bias, int dtype, int64_t n) {
  switch (dtype) {
    case OQ_DTYPE_F32: return Scalar<OQ_DTYPE_F32>::load(bias, n);
    case OQ_DTYPE_F16: return Scalar<OQ_DTYPE_F16>::load(bias, n);
    default: return Scalar<OQ_DTYPE_BF16>::load(bias, n);
  }
}

// ---- index -> f16 centroid decode ---------------------------------------------------------
//
// Every routine turns the 8*BITS bits of eight consecutive indices (lowest k first, held in
// `lo` / `hi`) into eight f16 table entries in k order.  Tables of up to 16 entries live in
// registers as separate high-byte / low-byte vectors and are read with prmt (byte permute,
// 3-bit selectors); 64- and 256-entry tables live in shared memory.

struct RegTable {
  uint32_t hi[4];  // high bytes of entries 4q .. 4q+3
  uint32_t lo[4];
};

__device__ __forceinline__ void pair_up(uint32_t lo, uint32_t hi, uint32_t &r0, uint32_t &r1) {
  r0 = __byte_perm(lo, hi, 0x5140u);  // entries 0, 1 as two f16
  r1 = __byte_perm(lo, hi, 0x7362u);  // entries 2, 3
}

// 4-bit: two 8-entry halves, bit 3 of the index picks the half through a byte mask.
__device__ __forceinline__ void decode8_w4(uint32_t w, const RegTable &t, uint4 &out) {
  const uint32_t low3 = w & 0x77777777u;
  const uint32_t bit3 = (w >> 3) & 0x11111111u;
  uint32_t r[4];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const uint32_t sel = low3 >> (16 * h);
    const uint32_t mask = __byte_perm(0x0000ff00u, 0u, bit3 >> (16 * h));
    const uint32_t hx = __byte_perm(t.hi[0], t.hi[1], sel);
    const uint32_t hy = __byte_perm(t.hi[2], t.hi[3], sel);
    const uint32_t lx = __byte_perm(t.lo[0], t.lo[1], sel);
    const uint32_t ly = __byte_perm(t.lo[2], t.lo[3], sel);
    pair_up((lx & ~mask) | (ly & mask), (hx & ~mask) | (hy & mask), r[2 * h], r[2 * h + 1]);
  }
  out = make_uint4(r[0], r[1], r[2], r[3]);
}

// 4-bit with a sign-symmetric table (entry 15 - i = -entry i, which holds for every Lloyd-Max
// codebook): only the upper half of the table (entries 8..15, the positive values in ascending
// order) is looked up.  Index i >= 8 selects entry i - 8 = its low three bits; index i < 8
// selects entry 7 - i = its low three bits inverted, and sets the sign bit.
__device__ __forceinline__ void decode8_w4_symmetric(uint32_t w, const RegTable &t, uint4 &out) {
  const uint32_t neg = ~(w >> 3) & 0x11111111u;      // 1 per nibble whose bit 3 is clear
  const uint32_t sel = (w ^ (neg * 7u)) & 0x77777777u;
  uint32_t r[4];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const uint32_t s = sel >> (16 * h);
    const uint32_t lo = __byte_perm(t.lo[2], t.lo[3], s);
    const uint32_t hi = __byte_perm(t.hi[2], t.hi[3], s) | __byte_perm(0x00008000u, 0u, neg >> (16 * h));
    pair_up(lo, hi, r[2 * h], r[2 * h + 1]);
  }
  out = make_uint4(r[0], r[1], r[2], r[3]);
}

// True when entry 15 - i of a 16-entry table is entry i with the sign bit flipped, for all i.
__device__ __forceinline__ bool table_is_symmetric(const RegTable &t) {
  return t.lo[0] == __byte_perm(t.lo[3], 0u, 0x0123u) && t.lo[1] == __byte_perm(t.lo[2], 0u, 0x0123u) &&
         t.hi[0] == (__byte_perm(t.hi[3], 0u, 0x0123u) ^ 0x80808080u) &&
         t.hi[1] == (__byte_perm(t.hi[2], 0u, 0x0123u) ^ 0x80808080u);
}

// INT8 code table (4-bit indices -> one signed byte each): sixteen entries in four registers,
// eight indices -> eight bytes.
__device__ __forceinline__ void decode8_w4_bytes(uint32_t w, const uint32_t (&tb)[4], uint32_t &r0, uint32_t &r1) {
  const uint32_t low3 = w & 0x77777777u;
  const uint32_t bit3 = (w >> 3) & 0x11111111u;
  uint32_t r[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const uint32_t sel = low3 >> (16 * h);
    const uint32_t mask = __byte_perm(0x0000ff00u, 0u, bit3 >> (16 * h));
    const uint32_t x = __byte_perm(tb[0], tb[1], sel);
    const uint32_t y = __byte_perm(tb[2], tb[3], sel);
    r[h] = (x & ~mask) | (y & mask);
  }
  r0 = r[0];
  r1 = r[1];
}

// 3-bit: 24 bits; spread each 3-bit field to its own selector nibble.
__device__ __forceinline__ void decode8_w3(uint32_t w, const RegTable &t, uint4 &out) {
  uint32_t r[4];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const uint32_t v = (w >> (12 * h)) & 0xfffu;                      // fields f0..f3
    const uint32_t a = (v & 0x03fu) | ((v & 0xfc0u) << 2);            // f0 f1 | f2 f3 per byte
    const uint32_t sel = (a & 0x0707u) | ((a & 0x3838u) << 1);        // one field per nibble
    pair_up(__byte_perm(t.lo[0], t.lo[1], sel), __byte_perm(t.hi[0], t.hi[1], sel), r[2 * h],
            r[2 * h + 1]);
  }
  out = make_uint4(r[0], r[1], r[2], r[3]);
}

// 2-bit: 16 bits; spread each 2-bit field to its own selector nibble.
__device__ __forceinline__ void decode8_w2(uint32_t w, const RegTable &t, uint4 &out) {
  uint32_t r[4];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const uint32_t v = (w >> (8 * h)) & 0xffu;
    const uint32_t a = (v | (v << 4)) & 0x0f0fu;
    const uint32_t sel = (a | (a << 2)) & 0x3333u;
    pair_up(__byte_perm(t.lo[0], 0u, sel), __byte_perm(t.hi[0], 0u, sel), r[2 * h], r[2 * h + 1]);
  }
  out = make_uint4(r[0], r[1], r[2], r[3]);
}

// 6- and 8-bit: one shared-memory read per index.  `lut` already points at this lane's copy;
// entry e sits kStride halfwords further.
template <int BITS, int kStride>
__device__ __forceinline__ void decode8_lut(uint32_t lo, uint32_t hi, const uint16_t *lut, uint4 &out) {
  const uint64_t v = (static_cast<uint64_t>(hi) << 32) | lo;
  uint32_t r[4];
#pragma unroll
  for (int e = 0; e < 8; e += 2) {
    const uint32_t i0 = static_cast<uint32_t>(v >> (BITS * e)) & ((1u << BITS) - 1u);
    const uint32_t i1 = static_cast<uint32_t>(v >> (BITS * (e + 1))) & ((1u << BITS) - 1u);
    r[e >> 1] = static_cast<uint32_t>(lut[i0 * kStride]) | (static_cast<uint32_t>(lut[i1 * kStride]) << 16);
  }
  out = make_uint4(r[0], r[1], r[2], r[3]);
}

// Bits [offset, offset + 8*BITS) of a word array, offset a compile-time constant after unrolling.
template <int BITS, int NWORDS>
__device__ __forceinline__ void group_bits(const uint32_t (&words)[NWORDS], int group, uint32_t &lo,
                                           uint32_t &hi) {
  const int offset = 8 * BITS * group;
  const int w = offset >> 5;
  const int sh = offset & 31;
  const uint32_t w0 = words[w];
  const uint32_t w1 = w + 1 < NWORDS ? words[w + 1] : 0u;
  const uint32_t w2 = w + 2 < NWORDS ? words[w + 2] : 0u;
  lo = __funnelshift_r(w0, w1, sh);
  hi = BITS > 4 ? __funnelshift_r(w1, w2, sh) : 0u;
}

// ---- expander warps ------------------------------------------------------------------------
// Thread `et` of the expander warps turns the packed indices of weight row `n_first + et / kTpr`
// into the 16-bit operand tile of every k step (T::kBBytes at offset T::kABytes of a stage).
// Returns false when a wait gave up.
template <class T, int BITS, bool SCALED>
__device__ __forceinline__ bool expand_weight_tiles(const GemmParams &p, int64_t n_first, uint32_t stage_base,
                                                    uint32_t bar_base, const float *s_cent,
                                                    const uint16_t *s_lut, float table_scale,
                                                    volatile int *s_abort, int warp, int lane) {
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (T::kStages + s); };
  auto bready_bar = [&](int s) { return bar_base + 8u * (2 * T::kStages + s); };
  const int64_t n0 = n_first;

  constexpr int kThreadsPerRow = T::kTpr;
  constexpr int kBytesPerThread = T::kRowBytes / kThreadsPerRow;
  constexpr int kWords = kBytesPerThread / 4;
  constexpr int kGroups = 8 / kThreadsPerRow;   // 16-byte chunks of the 128-byte output row per thread
  const int et = threadIdx.x;  // expander thread index (every expander warp owns rows)
  const int row = et / kThreadsPerRow;
  const int part = et % kThreadsPerRow;
  // Register table (2-, 3-, 4-bit): entry i = f16(centroid[i] * table scale), or, SCALED,
  // bf16(centroid[i] * row_norm) of the weight row this thread expands.
  const int64_t table_row = n0 + et / kThreadsPerRow;
  const float table_norm = (SCALED && table_row < p.out_features)
                               ? __bfloat162float(p.row_norms[table_row]) : 0.0f;
  RegTable table;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    uint32_t hi = 0;
    uint32_t lo = 0;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int idx = 4 * q + e;
      const float c = (BITS <= 4 && idx < (1 << BITS)) ? s_cent[idx] : 0.0f;
      const uint32_t bits =
          SCALED ? static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(__fmul_rn(c, table_norm))))
                 : static_cast<uint32_t>(__half_as_ushort(__float2half_rn(c * table_scale)));
      hi |= (bits >> 8) << (8 * e);
      lo |= (bits & 0xffu) << (8 * e);
    }
    table.hi[q] = hi;
    table.lo[q] = lo;
  }
  // INT8 operands: the codebook holds the (integer-valued) code table
  uint32_t byte_table[4] = {0u, 0u, 0u, 0u};
  if (T::kI8) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int code = __float2int_rn(s_cent[4 * q + e]);
        byte_table[q] |= (static_cast<uint32_t>(code) & 0xffu) << (8 * e);
      }
    }
  }
  const uint16_t *lane_lut = s_lut + (BITS == 6 ? lane : (lane & 7));
  // the symmetric decode is taken by the whole warp or not at all
  const bool symmetric = BITS == 4 && !T::kI8 && __all_sync(0xffffffffu, table_is_symmetric(table));
  const uint32_t row_off = (row >> 3) * 1024 + (row & 7) * 128;
  // Shared-memory addresses of this thread's packed bytes and of the 16-byte chunks it writes,
  // in stage 0.  The k loop below is unrolled over the stages, so a stage's offset is an
  // immediate in every load and store and nothing is recomputed per k step.
  const uint32_t src0 = stage_base + T::kABytes + T::kBBytes + row * T::kRowBytes + part * kBytesPerThread;
  uint32_t dst0[kGroups];
#pragma unroll
  for (int c = 0; c < kGroups; ++c) {
    dst0[c] = stage_base + T::kABytes + row_off + ((((part * kGroups + c) ^ (row & 7)) & 7) << 4);
  }
  // 3-bit rows come straight from global memory (8-byte loads, two k steps ahead).
  const int64_t n_global = n0 + row;
  const bool row_valid = n_global < p.out_features;
  const uint8_t *grow = p.packed + n_global * (static_cast<int64_t>(p.k_iters) * T::kRowBytes) +
                        part * kBytesPerThread;
  uint32_t words[kWords];
  auto load_global = [&](int it, uint32_t (&dst)[kWords]) {
    if (kWords % 4 == 0 && row_valid && it < p.k_iters) {
#pragma unroll
      for (int q = 0; q < kWords / 4; ++q) {
        const uint4 v = __ldg(reinterpret_cast<const uint4 *>(grow + static_cast<int64_t>(it) * T::kRowBytes) + q);
        dst[4 * q] = v.x;
        dst[4 * q + 1] = v.y;
        dst[4 * q + 2] = v.z;
        dst[4 * q + 3] = v.w;
      }
      return;
    }
    if (kWords % 2 == 0 && row_valid && it < p.k_iters) {
#pragma unroll
      for (int q = 0; q < kWords / 2; ++q) {
        const uint2 v = __ldg(reinterpret_cast<const uint2 *>(grow + static_cast<int64_t>(it) * T::kRowBytes) + q);
        dst[2 * q] = v.x;
        dst[2 * q + 1] = v.y;
      }
      return;
    }
#pragma unroll
    for (int q = 0; q < kWords; ++q) {
      dst[q] = (row_valid && it < p.k_iters)
                   ? __ldg(reinterpret_cast<const uint32_t *>(grow + static_cast<int64_t>(it) * T::kRowBytes) + q)
                   : 0u;
    }
  };
  bool ok = true;
  const int expand_iters = warp < T::kExpanderWarps ? p.k_iters : 0;
  uint32_t ahead_words[kWords];  // the k step after next: loads stay two steps ahead of their use
  if (!T::kPackedByTma && expand_iters > 0) {
    load_global(0, words);
    load_global(1, ahead_words);
  }
  uint32_t phase = 0;
  for (int it0 = 0; it0 < expand_iters && ok; it0 += T::kStages, phase ^= 1u) {
#pragma unroll
    for (int s = 0; s < T::kStages; ++s) {
      const int it = it0 + s;
      if (it >= expand_iters) {
        break;
      }
      uint32_t next_words[kWords];
      if (!T::kPackedByTma) {
#pragma unroll
        for (int q = 0; q < kWords; ++q) {
          next_words[q] = ahead_words[q];
        }
        load_global(it + 2, ahead_words);
      }
      // Packed bytes that came by TMA: wait for them.  Packed bytes in registers: the only
      // thing to wait for is the expanded tile of this stage being free again (the MMAs of
      // the k step kStages earlier have read it) -- the activation tile is the MMA's concern.
      if (!(T::kPackedByTma ? mbar_wait(full_bar(s), phase, s_abort, 4)
                            : mbar_wait(empty_bar(s), phase ^ 1u, s_abort, 4))) {
        ok = false;
        break;
      }
      if (T::kPackedByTma) {
        const uint32_t src = src0 + s * T::kStageBytes;
        if (kBytesPerThread % 16 == 0) {
#pragma unroll
          for (int q = 0; q < kWords / 4; ++q) {
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(words[4 * q]), "=r"(words[4 * q + 1]), "=r"(words[4 * q + 2]),
                           "=r"(words[4 * q + 3])
                         : "r"(src + 16 * q)
                         : "memory");
          }
        } else if (kBytesPerThread % 8 == 0) {
#pragma unroll
          for (int q = 0; q < kWords / 2; ++q) {
            asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];"
                         : "=r"(words[2 * q]), "=r"(words[2 * q + 1])
                         : "r"(src + 8 * q)
                         : "memory");
          }
        } else {
#pragma unroll
          for (int q = 0; q < kWords; ++q) {
            asm volatile("ld.shared.b32 %0, [%1];" : "=r"(words[q]) : "r"(src + 4 * q) : "memory");
          }
        }
      }
      // Decode every group first and store afterwards: the stores are volatile asm, which the
      // compiler keeps in program order, and a decode-store-decode-store sequence would chain
      // the (latency-bound) byte-permute sequences one after the other instead of overlapping
      // them.
      uint4 expanded[kGroups];
      if (T::kI8) {
        // sixteen 4-bit indices (two words) per 16-byte chunk
#pragma unroll
        for (int c = 0; c < kGroups; ++c) {
          decode8_w4_bytes(words[(2 * c) % kWords], byte_table, expanded[c].x, expanded[c].y);
          decode8_w4_bytes(words[(2 * c + 1) % kWords], byte_table, expanded[c].z, expanded[c].w);
        }
      } else if (symmetric) {
#pragma unroll
        for (int c = 0; c < kGroups; ++c) {
          uint32_t lo;
          uint32_t hi;
          group_bits<BITS, kWords>(words, c, lo, hi);
          decode8_w4_symmetric(lo, table, expanded[c]);
        }
      } else {
#pragma unroll
        for (int c = 0; c < kGroups; ++c) {
          uint32_t lo;
          uint32_t hi;
          group_bits<BITS, kWords>(words, c, lo, hi);
          if (BITS == 4) {
            decode8_w4(lo, table, expanded[c]);
          } else if (BITS == 3) {
            decode8_w3(lo, table, expanded[c]);
          } else if (BITS == 2) {
            decode8_w2(lo, table, expanded[c]);
          } else if (BITS == 6) {
            decode8_lut<6, 32>(lo, hi, lane_lut, expanded[c]);
          } else {
            decode8_lut<8, 8>(lo, hi, lane_lut, expanded[c]);
          }
        }
      }
#pragma unroll
      for (int c = 0; c < kGroups; ++c) {
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst0[c] + s * T::kStageBytes),
                     "r"(expanded[c].x), "r"(expanded[c].y), "r"(expanded[c].z), "r"(expanded[c].w)
                     : "memory");
      }
      if (!T::kPackedByTma) {
#pragma unroll
        for (int q = 0; q < kWords; ++q) {
          words[q] = next_words[q];
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(bready_bar(s));
      }
    }
  }
  return ok;
}

// ---- epilogue -------------------------------------------------------------------------------
// Warp w (0..7) reads accumulator w / 4, TMEM lanes 32 * (w % 4) .., of the CTA's 256 x BN tile
// whose first row is m0 and first column n0, and stores it to every destination buffer.
template <class T, int BN, bool SCALED>
__device__ __forceinline__ void store_output_tile(const GemmParams &p, int64_t m0, int64_t n0,
                                                  uint32_t tmem_base, unsigned char *stage_ptr,
                                                  uint32_t acc_full_bar, const float *s_scale,
                                                  const float *s_bias, volatile int *s_abort, bool ok,
                                                  int warp, int lane) {

  // A lane of tcgen05.ld holds one output ROW, so storing from registers would write 32
  // scattered 16-byte pieces per instruction.  The warp instead parks its 32 x BN bf16 tile
  // in the (now idle) pipeline stages and writes it out row by row: one instruction = one
  // contiguous run of BN*2 bytes, which is what both L2 and -- for a peer GPU's buffer --
  // NVLink want.  The row pitch is padded by 16 bytes so that the row-per-lane writes hit
  // all banks.
  constexpr int kPitch = BN * 2 + 16;
  static_assert(kEpilogueWarps * 32 * kPitch <= T::kStages * T::kStageBytes, "epilogue staging space");
  if (ok && warp < kEpilogueWarps && mbar_wait(acc_full_bar, 0, s_abort, 5)) {
    tc_fence_after();
    const int half = warp >> 2;
    const int quarter = warp & 3;
    const int64_t m_first = m0 + half * 128 + quarter * 32;
    const int64_t m = m_first + lane;
    const float row_scale = m < p.rows ? (SCALED ? 1.0f : p.row_scale[m]) : 0.0f;
    unsigned char *park = stage_ptr + warp * (32 * kPitch);
#pragma unroll 1
    for (int c0 = 0; c0 < BN; c0 += 32) {
      uint32_t v[32];
      tmem_ld_32x32b_x32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + half * BN + c0, v);
      tmem_ld_wait();
      uint4 *dst = reinterpret_cast<uint4 *>(park + lane * kPitch + c0 * 2);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint32_t w[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = 4 * q + e;
          // the accumulator holds fp32 sums, or, with INT8 operands, 32-bit integers
          const float acc_a = T::kI8 ? __int2float_rn(static_cast<int>(v[2 * j])) : __uint_as_float(v[2 * j]);
          const float acc_b =
              T::kI8 ? __int2float_rn(static_cast<int>(v[2 * j + 1])) : __uint_as_float(v[2 * j + 1]);
          const float a = fmaf(acc_a, row_scale * s_scale[c0 + 2 * j], s_bias[c0 + 2 * j]);
          const float b = fmaf(acc_b, row_scale * s_scale[c0 + 2 * j + 1], s_bias[c0 + 2 * j + 1]);
          const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
          w[e] = *reinterpret_cast<const uint32_t *>(&h);
        }
        dst[q] = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
    __syncwarp();
    // lane l carries columns 8l .. 8l+7 of every row
    const bool vec_ok = (p.out_features % 8) == 0 && (p.out_ld % 8) == 0 && (p.out_col % 8) == 0;
    const int64_t n = n0 + lane * 8;
    const bool lane_in_tile = lane * 8 < BN;
    const bool lane_full = lane_in_tile && n + 8 <= p.out_features;
    const int64_t rows_here = p.rows - m_first < 32 ? p.rows - m_first : 32;
    for (int d = 0; d < p.n_outs; ++d) {
      __nv_bfloat16 *out = static_cast<__nv_bfloat16 *>(p.outs[d]) + p.out_col + n;
#pragma unroll 4
      for (int r = 0; r < rows_here; ++r) {
        if (!lane_in_tile) {
          continue;
        }
        const uint4 val = *reinterpret_cast<const uint4 *>(park + r * kPitch + lane * 16);
        __nv_bfloat16 *dst = out + (m_first + r) * p.out_ld;
        if (vec_ok && lane_full) {
          *reinterpret_cast<uint4 *>(dst) = val;
        } else {
          const uint32_t w[4] = {val.x, val.y, val.z, val.w};
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            if (n + j < p.out_features) {
              reinterpret_cast<uint16_t *>(dst)[j] = static_cast<uint16_t>(w[j >> 1] >> ((j & 1) * 16));
            }
          }
        }
      }
    }
  }
}

template <int BN, int BITS, bool SCALED = false>
__global__ void __launch_bounds__((Tile<BN, BITS>::kThreads), 1)
gemm_w4_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a,
                       const __grid_constant__ CUtensorMap map_p, const GemmParams p) {
  using T = Tile<BN, BITS>;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  // header: barriers | scale[BN] | bias[BN]
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem_raw);
  uint32_t *s_tmem = reinterpret_cast<uint32_t *>(smem_raw + 192);
  volatile int *s_abort = reinterpret_cast<volatile int *>(smem_raw + 200);
  float *s_scale = reinterpret_cast<float *>(smem_raw + 256);
  float *s_bias = s_scale + BN;
  float *s_cent = s_bias + BN;                                   // [2^BITS] codebook
  uint16_t *s_lut = reinterpret_cast<uint16_t *>(s_cent + T::kCentFloats);  // 6- and 8-bit tables only
  const uint32_t header_end = smem_u32(smem_raw) + T::kHeaderBytes;
  const uint32_t stage_base = (header_end + 1023u) & ~1023u;
  unsigned char *stage_ptr = smem_raw + (stage_base - smem_u32(smem_raw));

  const uint32_t bar_base = smem_u32(bars);
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (T::kStages + s); };
  auto bready_bar = [&](int s) { return bar_base + 8u * (2 * T::kStages + s); };
  const uint32_t acc_full_bar = bar_base + 8u * (3 * T::kStages);

  auto a_addr = [&](int s) { return stage_base + s * T::kStageBytes; };
  auto b_addr = [&](int s) { return stage_base + s * T::kStageBytes + T::kABytes; };
  auto p_ptr = [&](int s) { return stage_ptr + s * T::kStageBytes + T::kABytes + T::kBBytes; };

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m_tile = p.columns_fastest ? blockIdx.x / p.n_tiles : blockIdx.x % p.m_tiles;
  const int n_tile = p.columns_fastest ? blockIdx.x % p.n_tiles : blockIdx.x / p.m_tiles;
  const int64_t m0 = static_cast<int64_t>(m_tile) * kBM;
  const int64_t n0 = static_cast<int64_t>(n_tile) * BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < T::kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
      mbar_init(bready_bar(s), T::kExpanderWarps);
    }
    mbar_init(acc_full_bar, 1);
    *s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == T::kMmaWarp) {
    tmem_alloc(smem_u32(s_tmem), T::kTmemCols);
  }
  if (warp == T::kProducerWarp && lane == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_p) : "memory");
  }
  for (int i = threadIdx.x; i < (1 << BITS); i += T::kThreads) {
    s_cent[i] = p.centroids[i];
  }
  __syncthreads();
  // The launch allows this grid to become resident while the kernel before it in the stream
  // (the prologue) is still running; everything below reads that kernel's output.  The kernel
  // after this one (the next layer's prologue, launched the same way) may in turn take over SMs
  // as this grid's last wave drains; it touches nothing of ours before its own wait.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  // The copies of the first stages leave before the tables below are built: their latency is
  // the longest item of the pipeline fill.
  int issued_early = 0;
  if (warp == T::kProducerWarp && lane == 0) {
    for (; issued_early < T::kStages && issued_early < p.k_iters; ++issued_early) {
      const int s = issued_early;
      mbar_arrive_expect_tx(full_bar(s), T::kABytes + (T::kPackedByTma ? T::kPBytes : 0));
      tma_load_2d(a_addr(s), &map_a, full_bar(s), s * kBK, static_cast<int>(m0));
      if (T::kPackedByTma) {
        tma_load_2d(smem_u32(p_ptr(s)), &map_p, full_bar(s), s * T::kRowBytes, static_cast<int>(n0));
      }
    }
  }
  // chosen by the kernel that ran just before this one (table_scale.cuh); 2^8 without it
  const float table_scale =
      SCALED ? 1.0f : (p.table_scale != nullptr ? __ldg(p.table_scale) : kCentroidScale);
  if (BITS == 6) {  // [entry][32 lane copies]
    for (int i = threadIdx.x; i < 64 * 32; i += T::kThreads) {
      s_lut[i] = __half_as_ushort(__float2half_rn(s_cent[i >> 5] * table_scale));
    }
  } else if (BITS == 8) {  // [entry][8 copies]
    for (int i = threadIdx.x; i < 256 * 8; i += T::kThreads) {
      s_lut[i] = __half_as_ushort(__float2half_rn(s_cent[i >> 3] * table_scale));
    }
  }
  for (int i = threadIdx.x; i < BN; i += T::kThreads) {
    const int64_t n = n0 + i;
    const bool ok = n < p.out_features;
    s_scale[i] = ok ? (SCALED ? 1.0f : __fdiv_rn(__bfloat162float(p.row_norms[n]), table_scale)) : 0.0f;
    s_bias[i] = (ok && p.bias_dtype >= 0) ? load_bias(p.bias, p.bias_dtype, n) : 0.0f;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *s_tmem;

  if (warp == T::kProducerWarp) {
    if (lane == 0) {
      int issued = issued_early;
      for (int it = issued_early; it < p.k_iters; ++it) {
        const int s = it % T::kStages;
        const uint32_t phase = (it / T::kStages) & 1u;
        if (!mbar_wait(empty_bar(s), phase ^ 1u, s_abort, 1)) {
          break;
        }
        mbar_arrive_expect_tx(full_bar(s), T::kABytes + (T::kPackedByTma ? T::kPBytes : 0));
        tma_load_2d(a_addr(s), &map_a, full_bar(s), it * kBK, static_cast<int>(m0));
        if (T::kPackedByTma) {
          tma_load_2d(smem_u32(p_ptr(s)), &map_p, full_bar(s), it * T::kRowBytes, static_cast<int>(n0));
        }
        issued = it + 1;
      }
      if (*s_abort != 0) {
        // Drain: the copies already issued must land before the CTA may exit.
        const int first = issued > T::kStages ? issued - T::kStages : 0;
        for (int it = first; it < issued; ++it) {
          const uint32_t bar = full_bar(it % T::kStages);
          const uint32_t phase = (it / T::kStages) & 1u;
          for (uint32_t spin = 0; spin < kSpinLimit && !mbar_try_wait(bar, phase); ++spin) {
          }
        }
      }
    }
  } else if (warp == T::kMmaWarp) {
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc(BN, SCALED);
      bool ok = true;
      for (int it = 0; it < p.k_iters && ok; ++it) {
        const int s = it % T::kStages;
        const uint32_t phase = (it / T::kStages) & 1u;
        ok = mbar_wait(full_bar(s), phase, s_abort, 2) && mbar_wait(bready_bar(s), phase, s_abort, 3);
        if (!ok) {
          break;
        }
        tc_fence_after();
#pragma unroll
        for (int half = 0; half < 2; ++half) {
#pragma unroll
          for (int j = 0; j < kBK / 16; ++j) {
            const uint64_t da = smem_desc_k_sw128(a_addr(s) + half * (128 * 128) + j * 32);
            const uint64_t db = smem_desc_k_sw128(b_addr(s) + j * 32);
            umma_f16(tmem_base + half * BN, da, db, idesc, (it > 0 || j > 0) ? 1u : 0u);
          }
        }
        umma_commit(empty_bar(s));
      }
      if (ok) {
        umma_commit(acc_full_bar);
      }
    }
  } else {
    // ---- expanders, then epilogue ----
    const bool ok = expand_weight_tiles<T, BITS, SCALED>(p, n0, stage_base, bar_base, s_cent, s_lut,
                                                         table_scale, s_abort, warp, lane);
    store_output_tile<T, BN, SCALED>(p, m0, n0, tmem_base, stage_ptr, acc_full_bar, s_scale, s_bias,
                                     s_abort, ok, warp, lane);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == T::kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, T::kTmemCols);
  }
}

// Caller-supplied 16-bit activations -> the f16 operand + per-token factor (one warp per
// token: absolute maximum, exponent, rescale).  bf16/f16 values times a power of two are
// exact in f16 unless they lie more than 2^28 below the token's maximum.
template <int DTYPE>
__global__ void __launch_bounds__(256) rows_to_f16_kernel(const void *x, int64_t rows, int64_t dim,
                                                          __half *out, float *row_scale,
                                                          const float *centroids, int bits,
                                                          float *table_scale_out, int *zero_words,
                                                          int zero_count) {
  __shared__ float s_search[272];
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (blockIdx.x == 0 && table_scale_out != nullptr) {
    clear_words(zero_words, zero_count);
    search_table_scale(centroids, bits, table_scale_out, s_search);
  }
  const int lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (row >= rows) {
    return;
  }
  const uint4 *src = reinterpret_cast<const uint4 *>(static_cast<const uint16_t *>(x) + row * dim);
  const int vecs = static_cast<int>(dim / 8);
  uint32_t top = 0;  // largest |x| as raw 15-bit magnitude pattern (monotonic for both formats)
  for (int i = lane; i < vecs; i += 32) {
    const uint4 v = __ldg(src + i);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      top = max(top, max(w[q] & 0x7fffu, (w[q] >> 16) & 0x7fffu));
    }
  }
#pragma unroll
  for (int m = 16; m >= 1; m >>= 1) {
    top = max(top, __shfl_xor_sync(0xffffffffu, top, m));
  }
  const float biggest = DTYPE == OQ_DTYPE_BF16 ? bf16_bits_to_float(static_cast<uint16_t>(top))
                                               : __half2float(__ushort_as_half(static_cast<uint16_t>(top)));
  float mult = 1.0f;
  float back = 1.0f;
  if (biggest > 0.0f && biggest < __int_as_float(0x7f800000)) {
    const int e = max(ilogbf(biggest) + 1, -100);
    mult = ldexpf(1.0f, 14 - e);
    back = ldexpf(1.0f, e - 14);
  }
  if (lane == 0) {
    row_scale[row] = back;
  }
  uint4 *dst = reinterpret_cast<uint4 *>(out + row * dim);
  for (int i = lane; i < vecs; i += 32) {
    const uint4 v = __ldg(src + i);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t o[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float lo;
      float hi;
      if (DTYPE == OQ_DTYPE_BF16) {
        lo = bf16_bits_to_float(static_cast<uint16_t>(w[q] & 0xffffu));
        hi = bf16_bits_to_float(static_cast<uint16_t>(w[q] >> 16));
      } else {
        lo = __half2float(__ushort_as_half(static_cast<uint16_t>(w[q] & 0xffffu)));
        hi = __half2float(__ushort_as_half(static_cast<uint16_t>(w[q] >> 16)));
      }
      const __half2 h = __floats2half2_rn(lo * mult, hi * mult);
      o[q] = *reinterpret_cast<const uint32_t *>(&h);
    }
    dst[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// ---- host side ---------------------------------------------------------------------------

using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                   const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                   const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *ptr = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) ==
            cudaSuccess &&
        result == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
  });
  return fn;
}

template <int BN, int BITS, bool SCALED = false>
int launch_bn(const CUtensorMap &map_a, const CUtensorMap &map_p, const GemmParams &p, int grid,
              cudaStream_t stream) {
  static std::once_flag once;
  static cudaError_t attr_status = cudaSuccess;
  std::call_once(once, [] {
    attr_status = cudaFuncSetAttribute(gemm_w4_tcgen05_kernel<BN, BITS, SCALED>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       Tile<BN, BITS>::kSmemBytes);
  });
  OQ_CHECK_CUDA(attr_status);
  // Programmatic stream serialization: CTAs may take over SMs as the prologue's last wave
  // drains (set-up, tensor-memory allocation); griddepcontrol.wait orders the dependent reads.
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(grid);
  config.blockDim = dim3(Tile<BN, BITS>::kThreads);
  config.dynamicSmemBytes = Tile<BN, BITS>::kSmemBytes;
  config.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attr;
  config.numAttrs = 1;
  OQ_CHECK_CUDA(cudaLaunchKernelEx(&config, gemm_w4_tcgen05_kernel<BN, BITS, SCALED>, map_a, map_p, p));
  count_launch();
  return OQ_OK;
}

#include "gemm_pair_tcgen05.cuh"
#include "skinny_tcgen05.cuh"

}  // namespace

bool tcgen05_gemm_supported(int64_t rows, int64_t in_features, int64_t out_features, int bits,
                            int dtype, int weight_mode) {
  // bf16(centroid * row_norm) operands need a per-row table: the register-table widths only
  const bool bits_ok = weight_mode == OQ_WEIGHT_BF16_SCALED
                           ? (bits == 2 || bits == 3 || bits == 4)
                           : (bits == 2 || bits == 3 || bits == 4 || bits == 6 || bits == 8);
  return rows > 0 && out_features > 0 && bits_ok && dtype == OQ_DTYPE_BF16 &&
         in_features >= kBK && in_features % kBK == 0 &&
         in_features <= (1 << 30) && rows < (1ll << 31) && out_features < (1ll << 31);
}

int launch_rows_to_f16(const void *x, int dtype, int64_t rows, int64_t dim, void *out_f16,
                       float *row_scale, const float *centroids, int bits, float *table_scale_out,
                       int *zero_words, int zero_count, cudaStream_t stream) {
  zero_count = zero_words != nullptr ? zero_count : 0;
  OQ_CHECK_ARG(table_scale_out == nullptr || (centroids != nullptr && bits >= 1 && bits <= 8),
               "the table scale search needs the weight codebook");
  OQ_CHECK_ARG(dtype == OQ_DTYPE_BF16 || dtype == OQ_DTYPE_F16, "16-bit activations expected");
  OQ_CHECK_ARG(dim % 8 == 0 && aligned16(x) && aligned16(out_f16), "rows must be 16-byte aligned");
  const unsigned grid = static_cast<unsigned>((rows + 7) / 8);
  if (dtype == OQ_DTYPE_BF16) {
    rows_to_f16_kernel<OQ_DTYPE_BF16><<<grid, 256, 0, stream>>>(x, rows, dim, static_cast<__half *>(out_f16), row_scale, centroids, bits, table_scale_out, zero_words, zero_count);
  } else {
    rows_to_f16_kernel<OQ_DTYPE_F16><<<grid, 256, 0, stream>>>(x, rows, dim, static_cast<__half *>(out_f16), row_scale, centroids, bits, table_scale_out, zero_words, zero_count);
  }
  OQ_CHECK_CUDA(cudaGetLastError());
  count_launch();
  return OQ_OK;
}

// `x` is the f16 operand [rows, in_features] and `row_scale` its per-token factor.
template <int BITS, bool SCALED = false>
int launch_bits(int bn, const CUtensorMap &map_a, const CUtensorMap &map_p, const GemmParams &p,
                int grid, cudaStream_t stream) {
  switch (bn) {
    case 256: return launch_bn<256, BITS, SCALED>(map_a, map_p, p, grid, stream);
    case 192: return launch_bn<192, BITS, SCALED>(map_a, map_p, p, grid, stream);
    default: return launch_bn<128, BITS, SCALED>(map_a, map_p, p, grid, stream);
  }
}

// Output tile of the large-row kernel for a problem: `*tile_n` = width of the single-CTA tile
// (256 | 192 | 128), `*pair_n` = width of the CTA-pair tile (256 | 192) or 0 when the single-CTA
// kernel runs.
void choose_tile(int64_t rows, int64_t out_features, int bits, int sm_count, int *tile_n, int *pair_n,
                 bool pair_only = false) {
  // Tile width.  Wider tiles move fewer shared-memory bytes per flop (the activation tile
  // is re-read once per MMA), narrower ones can fill the last wave better; pick the width
  // with the best product of the two.  The per-width rates are measured ratios.
  const int64_t m_tiles = (rows + kBM - 1) / kBM;
  auto score = [&](int width, double rate) {
    const int64_t tiles = m_tiles * ((out_features + width - 1) / width);
    const int64_t waves = (tiles + sm_count - 1) / sm_count;
    const double useful = static_cast<double>(out_features) /
                          static_cast<double>(((out_features + width - 1) / width) * width);
    return rate * useful * static_cast<double>(tiles) / static_cast<double>(waves * sm_count);
  };
  // 6- and 8-bit packed tiles leave room for only two 256-wide stages; start from 192 there.
  int bn = bits >= 6 ? 192 : 256;
  double best = bits >= 6 ? score(192, 0.93) : score(256, 1.0);
  if (score(192, 0.93) > best) {
    bn = 192;
    best = score(192, 0.93);
  }
  if (score(128, 0.76) > best) {
    bn = 128;
  }
  // the tile_n tunable (128 | 192 | 256) pins the width (tests and profiling)
  {
    const int value = tunable(OQ_TUNE_TILE_N);
    if (value == 128 || value == 192 || value == 256) {
      bn = value;
    }
  }
  // A pair of CTAs (cta_group::2) on a 512 x 256 (or 512 x 192) tile halves the decode work
  // and the shared-memory traffic per MMA; it wins when its grid fills the machine about as
  // well.  The pair tunable pins the choice: 0 = never, 1 = best pair width, 192 / 256 = that
  // pair width.
  const int64_t m_pairs = (rows + 2 * kBM - 1) / (2 * kBM);
  int pair_bn = 0;
  if (bits <= 4) {
    auto pair_score = [&](int width, double rate) {
      const int64_t n_tiles_w = (out_features + width - 1) / width;
      const int64_t ctas = 2 * m_pairs * n_tiles_w;
      const int64_t waves = (ctas + sm_count - 1) / sm_count;
      const double useful_n = static_cast<double>(out_features) / static_cast<double>(n_tiles_w * width);
      const double useful_m = static_cast<double>(rows) / static_cast<double>(m_pairs * 2 * kBM);
      return rate * useful_n * useful_m * static_cast<double>(ctas) / static_cast<double>(waves * sm_count);
    };
    const double single_useful_m = static_cast<double>(rows) / static_cast<double>(m_tiles * kBM);
    const double single_score =
        score(bn, bn == 256 ? 1.0 : (bn == 192 ? 0.93 : 0.76)) * single_useful_m;
    const double p256 = pair_score(256, kPairRate256);
    const double p192 = pair_score(192, kPairRate192);
    const int best_pair = p192 > p256 ? 192 : 256;
    if (std::max(p256, p192) > single_score || pair_only) {
      pair_bn = best_pair;
    }
    const int forced = tunable(OQ_TUNE_PAIR);
    if (forced == 0) {
      pair_bn = 0;
    } else if (forced == 192 || forced == 256) {
      pair_bn = forced;
    } else if (forced > 0) {
      pair_bn = best_pair;
    }
    if (pair_only && pair_bn == 0) {
      pair_bn = best_pair;
    }
  }
  *tile_n = bn;
  *pair_n = pair_bn;
}

int launch_tcgen05_gemm_scatter(void *const *outs, int n_outs, int64_t out_ld, int64_t out_col,
                                const void *x, const float *row_scale, const float *table_scale,
                                int64_t rows, int64_t in_features, int64_t out_features,
                                const uint8_t *packed, int bits, const void *row_norms_bf16,
                                const float *centroids, const void *bias, int bias_dtype,
                                cudaStream_t stream, bool scaled);

int launch_tcgen05_gemm(void *out, const void *x, const float *row_scale, const float *table_scale,
                        int64_t rows, int64_t in_features, int64_t out_features, const uint8_t *packed, int bits,
                        const void *row_norms_bf16, const float *centroids, const void *bias,
                        int bias_dtype, cudaStream_t stream, bool scaled) {
  void *outs[1] = {out};
  return launch_tcgen05_gemm_scatter(outs, 1, out_features, 0, x, row_scale, table_scale, rows,
                                     in_features, out_features, packed, bits, row_norms_bf16,
                                     centroids, bias, bias_dtype, stream, scaled);
}

int launch_tcgen05_gemm_scatter(void *const *outs, int n_outs, int64_t out_ld, int64_t out_col,
                                const void *x, const float *row_scale, const float *table_scale,
                                int64_t rows, int64_t in_features, int64_t out_features,
                                const uint8_t *packed, int bits, const void *row_norms_bf16,
                                const float *centroids, const void *bias, int bias_dtype,
                                cudaStream_t stream, bool scaled) {
  OQ_CHECK_ARG(n_outs >= 1 && n_outs <= kMaxOutputs, "1 to %d output buffers", kMaxOutputs);
  OQ_CHECK_ARG(!scaled || bits <= 4, "the bf16(centroid * row_norm) operand exists for 2-, 3- and 4-bit weights");
  OQ_CHECK_ARG(out_col >= 0 && out_ld >= out_col + out_features,
               "the column range does not fit the leading dimension");
  for (int d = 0; d < n_outs; ++d) {
    OQ_CHECK_ARG(outs[d] != nullptr && aligned16(outs[d]), "output buffers must be 16-byte aligned");
  }
  OQ_CHECK_ARG(aligned16(x) && aligned16(packed),
               "x and packed weights must be 16-byte aligned for the tcgen05 kernel");
  EncodeTiledFn encode = encode_tiled_fn();
  if (encode == nullptr) {
    return fail(OQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  }
  int device = 0;
  int sm_count = 0;
  OQ_CHECK_CUDA(cudaGetDevice(&device));
  OQ_CHECK_CUDA(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device));

  int bn = 0;
  int pair_bn = 0;
  choose_tile(rows, out_features, bits, sm_count, &bn, &pair_bn);
  const int64_t m_tiles = (rows + kBM - 1) / kBM;
  const int64_t m_pairs = (rows + 2 * kBM - 1) / (2 * kBM);
  const bool use_pair = pair_bn != 0;
  const int64_t pair_n_tiles = use_pair ? (out_features + pair_bn - 1) / pair_bn : 0;
  const int64_t pair_tiles = m_pairs * pair_n_tiles;
  if (use_pair) {
    bn = pair_bn / 2;  // the packed tensor map's box: the weight rows one CTA of the pair expands
  }
  const int64_t n_tiles = (out_features + bn - 1) / bn;
  OQ_CHECK_ARG(m_tiles * n_tiles < (1ll << 31) && pair_tiles < (1ll << 30), "too many output tiles");

  CUtensorMap map_a;
  CUtensorMap map_p;
  {
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(in_features), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(in_features) * 2};
    const cuuint32_t box[2] = {kBK, kBM};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult rc = encode(&map_a, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(x),
                               dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) {
      return fail(OQ_ERR_CUDA, "cuTensorMapEncodeTiled(activations) failed with code %d", (int)rc);
    }
  }
  {
    // 3-bit tiles are not fetched through this map (see Tile::kPackedByTma); it is still
    // encoded, over a 16-byte-aligned view, so that every kernel takes the same arguments.
    const int64_t row_bytes = in_features * bits / 8;
    const bool by_tma = bits != 3;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(by_tma ? row_bytes : 16),
                                static_cast<cuuint64_t>(by_tma ? out_features : 1)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(by_tma ? row_bytes : 16)};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(by_tma ? kBK * bits / 8 : 16),
                               static_cast<cuuint32_t>(by_tma ? bn : 1)};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult rc = encode(&map_p, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t *>(packed),
                               dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                               CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) {
      return fail(OQ_ERR_CUDA, "cuTensorMapEncodeTiled(packed weights) failed with code %d", (int)rc);
    }
  }

  GemmParams p{};
  for (int d = 0; d < n_outs; ++d) {
    p.outs[d] = outs[d];
  }
  p.n_outs = n_outs;
  p.out_ld = out_ld;
  p.out_col = out_col;
  p.packed = packed;
  p.row_scale = row_scale;
  p.table_scale = table_scale;
  p.row_norms = static_cast<const __nv_bfloat16 *>(row_norms_bf16);
  p.centroids = centroids;
  p.bias = bias;
  p.bias_dtype = bias == nullptr ? -1 : bias_dtype;
  p.rows = rows;
  p.out_features = out_features;
  p.k_iters = static_cast<int>(in_features / kBK);
  p.m_tiles = static_cast<int>(m_tiles);
  p.n_tiles = static_cast<int>(n_tiles);
  // Column tiles fastest unless it is the weight matrix that cannot stay in L2 and the
  // activations are the smaller operand.  Measured: 947 -> 1129 TFLOP/s on the 32760-row
  // video-DiT layers (activations of 335..906 MB), 1089 -> 1108 on the 4608-row DiT block.
  const int64_t act_bytes = rows * in_features * 2;
  const int64_t weight_bytes = out_features * in_features * bits / 8;
  p.columns_fastest = (weight_bytes > (int64_t(96) << 20) && act_bytes < weight_bytes) ? 0 : 1;
  if (tunable(OQ_TUNE_TILE_ORDER) >= 0) {  // 0 / 1 pins it (profiling)
    p.columns_fastest = tunable(OQ_TUNE_TILE_ORDER) != 0 ? 1 : 0;
  }
  if (use_pair) {
    p.m_tiles = static_cast<int>(m_pairs);
    p.n_tiles = static_cast<int>(pair_n_tiles);
    const int pairs = static_cast<int>(pair_tiles);
    if (scaled) {
      switch (bits) {
        case 2: return launch_pair_bits<2, true>(pair_bn, map_a, map_p, p, pairs, stream);
        case 3: return launch_pair_bits<3, true>(pair_bn, map_a, map_p, p, pairs, stream);
        default: return launch_pair_bits<4, true>(pair_bn, map_a, map_p, p, pairs, stream);
      }
    }
    switch (bits) {
      case 2: return launch_pair_bits<2, false>(pair_bn, map_a, map_p, p, pairs, stream);
      case 3: return launch_pair_bits<3, false>(pair_bn, map_a, map_p, p, pairs, stream);
      default: return launch_pair_bits<4, false>(pair_bn, map_a, map_p, p, pairs, stream);
    }
  }
  const int grid = static_cast<int>(m_tiles * n_tiles);
  if (scaled) {
    switch (bits) {
      case 2: return launch_bits<2, true>(bn, map_a, map_p, p, grid, stream);
      case 3: return launch_bits<3, true>(bn, map_a, map_p, p, grid, stream);
      default: return launch_bits<4, true>(bn, map_a, map_p, p, grid, stream);
    }
  }
  switch (bits) {
    case 2: return launch_bits<2>(bn, map_a, map_p, p, grid, stream);
    case 3: return launch_bits<3>(bn, map_a, map_p, p, grid, stream);
    case 4: return launch_bits<4>(bn, map_a, map_p, p, grid, stream);
    case 6: return launch_bits<6>(bn, map_a, map_p, p, grid, stream);
    default: return launch_bits<8>(bn, map_a, map_p, p, grid, stream);
  }
}

// The INT8 formulation on the tensor cores (kind::i8, 32-bit integer accumulation, CTA-pair
// kernel): `a_int8` is the [rows, in_features] INT8 activation operand, `code_floats` the
// (integer-valued) weight code table where the other kernels take their centroids.
bool tcgen05_i8_supported(int64_t rows, int64_t in_features, int64_t out_features, int bits) {
  return bits == 4 && rows > kSkMaxTokens && in_features % 128 == 0 && out_features > 0 &&
         in_features <= (1 << 30) && rows < (1ll << 31) && out_features < (1ll << 31);
}

int launch_tcgen05_gemm_i8(void *out, const void *a_int8, const float *row_scale, const float *table_scale,
                           int64_t rows, int64_t in_features, int64_t out_features, const uint8_t *packed,
                           const void *row_norms_bf16, const float *code_floats, const void *bias,
                           int bias_dtype, cudaStream_t stream) {
  OQ_CHECK_ARG(tcgen05_i8_supported(rows, in_features, out_features, 4),
               "the INT8 tensor-core kernel needs more than 128 rows and in_features %% 128 == 0");
  OQ_CHECK_ARG(out != nullptr && aligned16(out) && aligned16(a_int8) && aligned16(packed),
               "buffers must be 16-byte aligned for the tcgen05 kernel");
  EncodeTiledFn encode = encode_tiled_fn();
  if (encode == nullptr) {
    return fail(OQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  }
  int device = 0;
  int sm_count = 0;
  OQ_CHECK_CUDA(cudaGetDevice(&device));
  OQ_CHECK_CUDA(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device));
  int bn = 0;
  int pair_bn = 0;
  choose_tile(rows, out_features, 4, sm_count, &bn, &pair_bn, /*pair_only=*/true);
  const int64_t m_pairs = (rows + 2 * kBM - 1) / (2 * kBM);
  const int64_t pair_n_tiles = (out_features + pair_bn - 1) / pair_bn;
  OQ_CHECK_ARG(m_pairs * pair_n_tiles < (1ll << 30), "too many output tiles");
  constexpr int kStepBytes = 128;   // INT8 values per k step = operand row bytes
  CUtensorMap map_a;
  CUtensorMap map_p;
  {
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(in_features), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(in_features)};
    const cuuint32_t box[2] = {kStepBytes, kBM};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult rc = encode(&map_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(a_int8), dims,
                               strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) {
      return fail(OQ_ERR_CUDA, "cuTensorMapEncodeTiled(INT8 activations) failed with code %d", (int)rc);
    }
  }
  {
    const int64_t row_bytes = in_features / 2;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(row_bytes), static_cast<cuuint64_t>(out_features)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(row_bytes)};
    const cuuint32_t box[2] = {kStepBytes / 2, static_cast<cuuint32_t>(pair_bn / 2)};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult rc = encode(&map_p, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t *>(packed), dims,
                               strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) {
      return fail(OQ_ERR_CUDA, "cuTensorMapEncodeTiled(packed weights) failed with code %d", (int)rc);
    }
  }
  GemmParams p{};
  p.outs[0] = out;
  p.n_outs = 1;
  p.out_ld = out_features;
  p.out_col = 0;
  p.packed = packed;
  p.row_scale = row_scale;
  p.table_scale = table_scale;
  p.row_norms = static_cast<const __nv_bfloat16 *>(row_norms_bf16);
  p.centroids = code_floats;
  p.bias = bias;
  p.bias_dtype = bias == nullptr ? -1 : bias_dtype;
  p.rows = rows;
  p.out_features = out_features;
  p.k_iters = static_cast<int>(in_features / kStepBytes);
  p.m_tiles = static_cast<int>(m_pairs);
  p.n_tiles = static_cast<int>(pair_n_tiles);
  p.columns_fastest = 1;
  const int pairs = static_cast<int>(m_pairs * pair_n_tiles);
  return pair_bn == 256 ? launch_pair_bn<256, 4, false, true>(map_a, map_p, p, pairs, stream)
                        : launch_pair_bn<192, 4, false, true>(map_a, map_p, p, pairs, stream);
}

// Name of the large-row kernel this problem gets (for reports; launches nothing).
const char *tcgen05_gemm_kernel_name(int64_t rows, int64_t out_features, int bits) {
  int device = 0;
  int sm_count = 0;
  if (cudaGetDevice(&device) != cudaSuccess ||
      cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sm_count <= 0) {
    sm_count = 148;
  }
  int bn = 0;
  int pair_bn = 0;
  choose_tile(rows, out_features, bits, sm_count, &bn, &pair_bn);
  return pair_bn != 0 ? "gemm_pair_tcgen05_kernel" : "gemm_w4_tcgen05_kernel";
}

// Few tokens (rows <= 128): the operand-swapped kernel of skinny_tcgen05.cuh.
bool tcgen05_skinny_supported(int64_t rows, int64_t in_features, int64_t out_features, int bits,
                              int dtype, int weight_mode) {
  return rows <= kSkMaxTokens && weight_mode != OQ_WEIGHT_BF16_SCALED &&
         tcgen05_gemm_supported(rows, in_features, out_features, bits, dtype, weight_mode);
}

size_t tcgen05_skinny_workspace_bytes(int64_t rows, int64_t in_features, int64_t out_features) {
  // sized for the larger of two machine widths so that the figure does not depend on the
  // device that happens to be current when the caller asks
  const size_t a = skinny_partial_bytes(skinny_plan(rows, in_features, out_features, 148), out_features);
  const size_t b = skinny_partial_bytes(skinny_plan(rows, in_features, out_features, 256), out_features);
  return a > b ? a : b;
}

// Ints at the head of the few-token kernel's workspace that the preceding kernel must clear.
int tcgen05_skinny_counter_words(int64_t rows, int64_t in_features, int64_t out_features) {
  (void)rows;
  (void)in_features;
  return static_cast<int>((out_features + kSkRows - 1) / kSkRows) * 4;
}

int launch_tcgen05_skinny(void *out, const void *x, const float *row_scale, const float *table_scale,
                          int64_t rows, int64_t in_features, int64_t out_features,
                          const uint8_t *packed, int bits, const void *row_norms_bf16,
                          const float *centroids, const void *bias, int bias_dtype, void *workspace,
                          size_t workspace_bytes, cudaStream_t stream) {
  OQ_CHECK_ARG(aligned16(x) && aligned16(packed), "x and packed weights must be 16-byte aligned");
  OQ_CHECK_ARG(rows >= 1 && rows <= kSkMaxTokens, "the few-token kernel takes 1..128 rows");
  EncodeTiledFn encode = encode_tiled_fn();
  if (encode == nullptr) {
    return fail(OQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  }
  int device = 0;
  int sm_count = 0;
  OQ_CHECK_CUDA(cudaGetDevice(&device));
  OQ_CHECK_CUDA(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device));
  const SkinnyPlan plan = skinny_plan(rows, in_features, out_features, sm_count > 256 ? 256 : sm_count);

  CUtensorMap map_x;
  CUtensorMap map_p;
  {
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(in_features), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(in_features) * 2};
    const cuuint32_t box[2] = {kBK, static_cast<cuuint32_t>(plan.n_pad)};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult rc = encode(&map_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(x),
                               dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) {
      return fail(OQ_ERR_CUDA, "cuTensorMapEncodeTiled(activations) failed with code %d", (int)rc);
    }
  }
  {
    const int64_t row_bytes = in_features * bits / 8;
    const bool by_tma = bits != 3;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(by_tma ? row_bytes : 16),
                                static_cast<cuuint64_t>(by_tma ? out_features : 1)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(by_tma ? row_bytes : 16)};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(by_tma ? kBK * bits / 8 : 16),
                               static_cast<cuuint32_t>(by_tma ? kSkRows : 1)};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult rc = encode(&map_p, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t *>(packed),
                               dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                               CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) {
      return fail(OQ_ERR_CUDA, "cuTensorMapEncodeTiled(packed weights) failed with code %d", (int)rc);
    }
  }

  SkinnyParams p{};
  p.out = out;
  p.packed = packed;
  p.row_scale = row_scale;
  p.table_scale = table_scale;
  p.row_norms = static_cast<const __nv_bfloat16 *>(row_norms_bf16);
  p.centroids = centroids;
  p.bias = bias;
  p.bias_dtype = bias == nullptr ? -1 : bias_dtype;
  p.rows = static_cast<int>(rows);
  p.out_features = out_features;
  p.k_iters = static_cast<int>(in_features / kBK);
  p.n_pad = plan.n_pad;
  p.splits = plan.splits;
  p.chunk_iters = plan.chunk_iters;
  p.n_tiles = plan.n_tiles;
  if (plan.splits > 1) {
    const size_t need = skinny_partial_bytes(plan, out_features);
    if (workspace == nullptr || workspace_bytes < need) {
      return fail(OQ_ERR_WORKSPACE, "workspace of %zu bytes given, %zu needed", workspace_bytes, need);
    }
    OQ_CHECK_ARG(aligned16(workspace), "workspace must be 16-byte aligned");
    p.counters = static_cast<int *>(workspace);  // cleared by the kernel that ran just before
    p.partial = reinterpret_cast<float *>(static_cast<unsigned char *>(workspace) + skinny_counter_bytes(plan));
  }
  int rc = OQ_OK;
  switch (bits) {
    case 2: rc = launch_skinny_bits<2>(map_x, map_p, p, sm_count, stream); break;
    case 3: rc = launch_skinny_bits<3>(map_x, map_p, p, sm_count, stream); break;
    case 4: rc = launch_skinny_bits<4>(map_x, map_p, p, sm_count, stream); break;
    case 6: rc = launch_skinny_bits<6>(map_x, map_p, p, sm_count, stream); break;
    default: rc = launch_skinny_bits<8>(map_x, map_p, p, sm_count, stream); break;
  }
  return rc;
}

// RTN-INT4 group-64 weights (AdaLN modulation layers), 1..128 rows of bf16 activations.
size_t tcgen05_rtn_workspace_bytes(int64_t rows, int64_t in_features, int64_t out_features) {
  const int64_t padded = (in_features + kBK - 1) / kBK * kBK;
  return tcgen05_skinny_workspace_bytes(rows, padded, out_features);
}

int launch_tcgen05_rtn_int4(void *out, const void *x_bf16, int64_t rows, int64_t in_features,
                            int64_t out_features, const uint8_t *packed, const void *scales_bf16,
                            const void *bias, int bias_dtype, void *workspace,
                            size_t workspace_bytes, cudaStream_t stream) {
  OQ_CHECK_ARG(aligned16(x_bf16) && aligned16(packed), "x and packed weights must be 16-byte aligned");
  OQ_CHECK_ARG(rows >= 1 && rows <= kSkMaxTokens, "1..128 rows per launch");
  OQ_CHECK_ARG(in_features % 8 == 0, "in_features must be a multiple of 8 (16-byte activation rows)");
  EncodeTiledFn encode = encode_tiled_fn();
  if (encode == nullptr) {
    return fail(OQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  }
  int device = 0;
  int sm_count = 0;
  OQ_CHECK_CUDA(cudaGetDevice(&device));
  OQ_CHECK_CUDA(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device));
  const int64_t groups = (in_features + kBK - 1) / kBK;  // 64-wide groups = k steps; rows are padded to them
  const SkinnyPlan plan = skinny_plan(rows, groups * kBK, out_features, sm_count > 256 ? 256 : sm_count);

  CUtensorMap map_x;
  CUtensorMap map_p;
  {
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(in_features), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(in_features) * 2};
    const cuuint32_t box[2] = {kBK, static_cast<cuuint32_t>(plan.n_pad)};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult rc = encode(&map_x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(x_bf16),
                               dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) {
      return fail(OQ_ERR_CUDA, "cuTensorMapEncodeTiled(activations) failed with code %d", (int)rc);
    }
  }
  {
    const int64_t row_bytes = groups * 32;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(row_bytes), static_cast<cuuint64_t>(out_features)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(row_bytes)};
    const cuuint32_t box[2] = {32, static_cast<cuuint32_t>(kSkRows)};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult rc = encode(&map_p, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t *>(packed),
                               dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                               CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) {
      return fail(OQ_ERR_CUDA, "cuTensorMapEncodeTiled(packed weights) failed with code %d", (int)rc);
    }
  }
  SkinnyParams p{};
  p.out = out;
  p.packed = packed;
  p.rtn_scales = static_cast<const __nv_bfloat16 *>(scales_bf16);
  p.bias = bias;
  p.bias_dtype = bias == nullptr ? -1 : bias_dtype;
  p.rows = static_cast<int>(rows);
  p.out_features = out_features;
  p.k_iters = static_cast<int>(groups);
  p.n_pad = plan.n_pad;
  p.splits = plan.splits;
  p.chunk_iters = plan.chunk_iters;
  p.n_tiles = plan.n_tiles;
  if (plan.splits > 1) {
    const size_t need = skinny_partial_bytes(plan, out_features);
    if (workspace == nullptr || workspace_bytes < need) {
      return fail(OQ_ERR_WORKSPACE, "workspace of %zu bytes given, %zu needed", workspace_bytes, need);
    }
    OQ_CHECK_ARG(aligned16(workspace), "workspace must be 16-byte aligned");
    p.counters = static_cast<int *>(workspace);
    p.partial = reinterpret_cast<float *>(static_cast<unsigned char *>(workspace) + skinny_counter_bytes(plan));
    // no kernel of this library runs before this one: clear the slice counters with a memset node
    OQ_CHECK_CUDA(cudaMemsetAsync(workspace, 0, skinny_counter_bytes(plan), stream));
  }
  return launch_skinny_bits<4, true>(map_x, map_p, p, sm_count, stream);
}

int read_gemm_status(int *status) {
  OQ_CHECK_CUDA(cudaMemcpyFromSymbol(status, g_gemm_status, sizeof(int)));
  return OQ_OK;
}

int clear_gemm_status() {
  const int zero = 0;
  OQ_CHECK_CUDA(cudaMemcpyToSymbol(g_gemm_status, &zero, sizeof(int)));
  return OQ_OK;
}

}  // namespace oq
