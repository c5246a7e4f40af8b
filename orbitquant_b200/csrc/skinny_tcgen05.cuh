// Codebook-decode GEMM for FEW tokens (rows <= 128) on the 5th-generation tensor cores.
// This file is included by gemm_tcgen05.cu inside its anonymous namespace and uses that
// file's PTX wrappers, decode routines and status word.
//
// With few tokens the forward is weight streaming, and what limits it is how fast indices
// become f16 centroids, so the operands trade places: the WEIGHT tile is the MMA's M side
// (128 weight rows, expanded once into shared memory in the K-major 128-byte-swizzled
// layout) and the tokens are its N side (16 .. 128 columns, one small bulk tensor copy per
// k step).  An expanded weight value is then written once and read once, the accumulator is
// 128 lanes x n_pad columns of tensor memory, and the MMA time is negligible.
//
// A unit of work is 128 weight rows x one slice of the reduction dimension; slices exist so
// that small layers still fill the machine.  The kernel is PERSISTENT: up to two CTAs per SM
// walk the unit list, and the copy / expand / MMA pipeline runs straight through unit
// boundaries (the per-CTA set-up and the ~1 us it takes the first tile to arrive are paid
// once, not once per unit).  Two accumulators in tensor memory alternate, so the epilogue of
// one unit (four warps of their own) overlaps the main loop of the next.  With one slice
// the epilogue writes bf16 outputs; with several, fp32 partial sums go to the workspace, a
// per-tile counter (cleared by the preceding kernel) tells which CTA finished a tile's last
// slice, and that CTA adds all the slices in slice order -- so the result does not depend on
// which CTA it was, and no second kernel is needed.
//
// The kernel is launched with programmatic stream serialization: it may start while the
// kernel that produces the activations is still running, pulls its share of the packed
// weights into L2 meanwhile, and executes griddepcontrol.wait before it touches anything
// that kernel writes.
//
// Warps: 0..7 expand (2 threads per weight row), 8 issues the bulk copies, 9 the MMAs,
// 10..13 run the epilogue (warp w reads tensor-memory lanes 32*(w%4)..).  Every mbarrier
// wait is bounded, as in the large-row kernel.

constexpr int kSkRows = 128;          // weight rows per unit = MMA M
constexpr int kSkMaxCopyStages = 12;  // ring of packed + activation tiles (what is in flight)
constexpr int kSkMaxSlots = 4;        // ring of expanded weight tiles
constexpr int kSkBarrierBytes = 512;
constexpr int kSkExpanderWarps = 8;
constexpr int kSkProducerWarp = kSkExpanderWarps;
constexpr int kSkMmaWarp = kSkExpanderWarps + 1;
constexpr int kSkEpilogueWarp0 = kSkExpanderWarps + 2;
constexpr int kSkThreads = (kSkExpanderWarps + 2 + 4) * 32;
constexpr int kSkMaxTokens = 128;
constexpr int kSkMinItersPerSplit = 12;  // measured: 12 beats 8 and 16 on 3072-wide layers at 16 tokens

template <int BITS>
struct SkinnyTile {
  static constexpr int kRowBytes = kBK * BITS / 8;
  static constexpr int kPBytes = kSkRows * kRowBytes;
  static constexpr bool kPackedByTma = BITS != 3;
  static constexpr int kLutBytes = BITS == 6 ? 64 * 32 * 2 : (BITS == 8 ? 256 * 8 * 2 : 0);
  static constexpr int kWBytes = kSkRows * kBK * 2;  // expanded weight tile, 16 KB
  static constexpr int kHeaderBytes = kSkBarrierBytes + kSkMaxTokens * 4 /*token factors*/ +
                                      256 * 4 /*centroids*/ + kLutBytes;
  // one copy stage: activation tile (n_pad rows of 128 bytes, a multiple of 2 KB) + packed tile
  static int copy_stage_bytes(int n_pad) { return n_pad * 128 + (kPBytes + 1023) / 1024 * 1024; }
  // Up to 48 tokens two CTAs share an SM (113 KB each) with three expanded-tile slots;
  // above that one CTA has the SM to itself and takes four.
  static int slots(int n_pad) { return n_pad <= 48 ? 3 : kSkMaxSlots; }
  static int copy_stages(int n_pad) {
    const int budget = (n_pad <= 48 ? 113 : 226) * 1024 - kHeaderBytes - 1024 - slots(n_pad) * kWBytes;
    const int fit = budget / copy_stage_bytes(n_pad);
    return fit > kSkMaxCopyStages ? kSkMaxCopyStages : fit;
  }
  static int smem_bytes(int n_pad) {
    return kHeaderBytes + 1024 + slots(n_pad) * kWBytes + copy_stages(n_pad) * copy_stage_bytes(n_pad);
  }
};

struct SkinnyParams {
  void *out;
  float *partial;          // [splits][n_pad][out_features] when splits > 1
  int *counters;           // [n_tiles] slices finished per weight tile, zero on entry
  const uint8_t *packed;
  const float *row_scale;
  const float *table_scale;
  const __nv_bfloat16 *row_norms;
  const float *centroids;
  const void *bias;
  int bias_dtype;
  int rows;
  int64_t out_features;
  int k_iters;             // 64-wide k steps of the whole reduction
  int n_pad;               // tokens rounded up to a multiple of 16
  int splits;
  int chunk_iters;         // k steps per slice (the last slice may be shorter)
  int n_tiles;
  int units;               // n_tiles * splits
  int copy_stages;         // ring of packed + activation tiles
  int copy_stage_bytes;
  int slots;               // ring of expanded weight tiles
  // RTN-INT4 group-64 weights (the AdaLN modulation layers): value = bf16((code - 8) * scale),
  // one bf16 scale per weight row and 64-wide k step; both MMA operands are then bf16.
  const __nv_bfloat16 *rtn_scales;  // [out_features][k_iters]
};

__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}

// Bulk tensor prefetch into L2 (no shared-memory destination, no barrier).
__device__ __forceinline__ void tma_prefetch_l2_2d(const CUtensorMap *map, int x, int y) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global [%0, {%1, %2}];" ::"l"(map), "r"(x), "r"(y)
               : "memory");
}

// Instruction descriptor with a run-time N (tokens): f32 accumulator, f16 x f16, M = 128.
__device__ __forceinline__ uint32_t instr_desc_tokens(int n, bool bf16_operands) {
  const uint32_t format = bf16_operands ? 1u : 0u;  // A and B always share one format
  return (1u << 4) | (format << 7) | (format << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(128 >> 4) << 24);
}

// Position in a ring of `size` entries and the parity of its current pass.
struct SkinnyRing {
  int index = 0;
  uint32_t phase = 0;
  __device__ __forceinline__ void advance(int size) {
    if (++index == size) {
      index = 0;
      phase ^= 1u;
    }
  }
};

// Unit u -> (weight tile, reduction slice).  Slice-major, so that the CTAs running at the
// same time read neighbouring weight tiles.
struct SkinnyUnit {
  int n_tile;
  int split;
  int it_begin;
  int iters;
};

__device__ __forceinline__ SkinnyUnit skinny_unit(const SkinnyParams &p, int u) {
  SkinnyUnit unit;
  unit.split = u / p.n_tiles;
  unit.n_tile = u - unit.split * p.n_tiles;
  unit.it_begin = unit.split * p.chunk_iters;
  unit.iters = min(p.k_iters, unit.it_begin + p.chunk_iters) - unit.it_begin;
  return unit;
}


template <int BITS, bool RTN = false>
__global__ void __launch_bounds__(kSkThreads, 2)
skinny_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x,
                      const __grid_constant__ CUtensorMap map_p, const SkinnyParams p) {
  using T = SkinnyTile<BITS>;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem_raw);
  uint32_t *s_tmem = reinterpret_cast<uint32_t *>(smem_raw + kSkBarrierBytes - 16);
  volatile int *s_abort = reinterpret_cast<volatile int *>(smem_raw + kSkBarrierBytes - 8);
  float *s_tok = reinterpret_cast<float *>(smem_raw + kSkBarrierBytes);  // [128] per-token factors
  float *s_cent = s_tok + kSkMaxTokens;                          // [256] codebook
  uint16_t *s_lut = reinterpret_cast<uint16_t *>(s_cent + 256);  // 6- and 8-bit tables only
  const uint32_t header_end = smem_u32(smem_raw) + T::kHeaderBytes;
  const uint32_t stage_base = (header_end + 1023u) & ~1023u;
  unsigned char *stage_ptr = smem_raw + (stage_base - smem_u32(smem_raw));
  const int x_bytes = p.n_pad * 128;

  const uint32_t bar_base = smem_u32(bars);
  // copy ring: full (tiles landed) / empty (MMA done with them); slot ring: ready (expanded)
  // / free (MMA done with it); two accumulators: full / empty
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kSkMaxCopyStages + s); };
  auto ready_bar = [&](int w) { return bar_base + 8u * (2 * kSkMaxCopyStages + w); };
  auto free_bar = [&](int w) { return bar_base + 8u * (2 * kSkMaxCopyStages + kSkMaxSlots + w); };
  auto acc_full_bar = [&](int b) { return bar_base + 8u * (2 * kSkMaxCopyStages + 2 * kSkMaxSlots + b); };
  auto acc_empty_bar = [&](int b) { return bar_base + 8u * (2 * kSkMaxCopyStages + 2 * kSkMaxSlots + 2 + b); };
  static_assert(8 * (2 * kSkMaxCopyStages + 2 * kSkMaxSlots + 4) <= kSkBarrierBytes - 16, "barrier space");

  const uint32_t copy_base = stage_base + p.slots * T::kWBytes;
  auto w_addr = [&](int w) { return stage_base + w * T::kWBytes; };
  auto x_addr = [&](int s) { return copy_base + s * p.copy_stage_bytes; };
  auto p_ptr = [&](int s) {
    return stage_ptr + p.slots * T::kWBytes + s * p.copy_stage_bytes + x_bytes;
  };

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // tensor-memory columns come in powers of two, 32 at least; two accumulators
  const uint32_t acc_cols = p.n_pad <= 32 ? 32u : (p.n_pad <= 64 ? 64u : 128u);
  const uint32_t tmem_cols = 2u * acc_cols;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.copy_stages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int w = 0; w < p.slots; ++w) {
      mbar_init(ready_bar(w), kSkExpanderWarps);
      mbar_init(free_bar(w), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full_bar(b), 1);
      mbar_init(acc_empty_bar(b), 4);
    }
    *s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kSkMmaWarp) {
    tmem_alloc(smem_u32(s_tmem), tmem_cols);
  }
  if (warp == kSkProducerWarp && lane == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_p) : "memory");
  }
  for (int i = threadIdx.x; i < (1 << BITS); i += kSkThreads) {
    s_cent[i] = RTN ? 0.0f : p.centroids[i];
  }
  if (warp == kSkProducerWarp && lane == 0 && T::kPackedByTma) {
    // The packed tiles are fetched 32..64 bytes per row and k step, but L2 fills 256-byte
    // lines: asking for the first tile of every 256-byte group pulls a whole unit into L2.
    // Doing that for all of this CTA's units NOW -- the weights do not depend on the kernel
    // that is still producing the activations -- hides the weight stream behind it.
    constexpr int kPrefetchStep = T::kRowBytes >= 256 ? 1 : 256 / T::kRowBytes;
    for (int u = blockIdx.x; u < p.units; u += gridDim.x) {
      const SkinnyUnit ahead = skinny_unit(p, u);
      for (int it = 0; it < ahead.iters; it += kPrefetchStep) {
        tma_prefetch_l2_2d(&map_p, (ahead.it_begin + it) * T::kRowBytes, ahead.n_tile * kSkRows);
      }
    }
  }
  // Everything below reads what the preceding kernel wrote (activations, per-token factors,
  // table scale, cleared counters).  A no-op unless launched with programmatic serialization.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  for (int i = threadIdx.x; i < kSkMaxTokens; i += kSkThreads) {
    s_tok[i] = i < p.rows ? (RTN ? 1.0f : p.row_scale[i]) : 0.0f;
  }
  const float table_scale = RTN ? 1.0f : (p.table_scale != nullptr ? __ldg(p.table_scale) : kCentroidScale);
  __syncthreads();
  if (BITS == 6) {
    for (int i = threadIdx.x; i < 64 * 32; i += kSkThreads) {
      s_lut[i] = __half_as_ushort(__float2half_rn(s_cent[i >> 5] * table_scale));
    }
  } else if (BITS == 8) {
    for (int i = threadIdx.x; i < 256 * 8; i += kSkThreads) {
      s_lut[i] = __half_as_ushort(__float2half_rn(s_cent[i >> 3] * table_scale));
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *s_tmem;

  if (warp == kSkProducerWarp) {
    if (lane == 0) {
      SkinnyRing copy;
      int issued = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < p.units && ok; u += gridDim.x) {
        const SkinnyUnit unit = skinny_unit(p, u);
        for (int it = 0; it < unit.iters; ++it) {
          const int s = copy.index;
          if (!mbar_wait(empty_bar(s), copy.phase ^ 1u, s_abort, 11)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(full_bar(s), x_bytes + (T::kPackedByTma ? T::kPBytes : 0));
          tma_load_2d(x_addr(s), &map_x, full_bar(s), (unit.it_begin + it) * kBK, 0);
          if (T::kPackedByTma) {
            tma_load_2d(smem_u32(p_ptr(s)), &map_p, full_bar(s), (unit.it_begin + it) * T::kRowBytes,
                        unit.n_tile * kSkRows);
          }
          copy.advance(p.copy_stages);
          ++issued;
        }
      }
      if (*s_abort != 0) {
        // Drain: the copies already issued must land before the CTA may exit.
        const int pending = issued < p.copy_stages ? issued : p.copy_stages;
        for (int i = 0; i < pending; ++i) {
          // walk back from the last issued stage
          int s = copy.index - 1 - i;
          uint32_t phase = copy.phase;
          if (s < 0) {
            s += p.copy_stages;
            phase ^= 1u;
          }
          for (uint32_t spin = 0; spin < kSpinLimit && !mbar_try_wait(full_bar(s), phase); ++spin) {
          }
        }
      }
    }
  } else if (warp == kSkMmaWarp) {
    if (lane == 0) {
      const uint32_t idesc = instr_desc_tokens(p.n_pad, RTN);
      SkinnyRing copy;
      SkinnyRing slot;
      int local = 0;  // units this CTA has started
      bool ok = true;
      for (int u = blockIdx.x; u < p.units && ok; u += gridDim.x, ++local) {
        const SkinnyUnit unit = skinny_unit(p, u);
        const int buf = local & 1;
        // the epilogue must have drained this accumulator (two units ago)
        ok = mbar_wait(acc_empty_bar(buf), ((local >> 1) & 1u) ^ 1u, s_abort, 16);
        if (!ok) {
          break;
        }
        tc_fence_after();
        const uint32_t acc = tmem_base + buf * acc_cols;
        for (int it = 0; it < unit.iters; ++it) {
          const int s = copy.index;
          const int w = slot.index;
          ok = mbar_wait(full_bar(s), copy.phase, s_abort, 12) &&
               mbar_wait(ready_bar(w), slot.phase, s_abort, 13);
          if (!ok) {
            break;
          }
          tc_fence_after();
#pragma unroll
          for (int j = 0; j < kBK / 16; ++j) {
            const uint64_t dw = smem_desc_k_sw128(w_addr(w) + j * 32);
            const uint64_t dx = smem_desc_k_sw128(x_addr(s) + j * 32);
            umma_f16(acc, dw, dx, idesc, (it > 0 || j > 0) ? 1u : 0u);
          }
          // the expanders finished with the packed tile before they signalled `ready`
          umma_commit(free_bar(w));
          umma_commit(empty_bar(s));
          copy.advance(p.copy_stages);
          slot.advance(p.slots);
        }
        if (ok) {
          umma_commit(acc_full_bar(buf));
        }
      }
    }
  } else if (warp < kSkExpanderWarps) {
    // ---- expanders: 2 threads per weight row ----
    constexpr int kBytesPerThread = T::kRowBytes / 2;
    constexpr int kWords = kBytesPerThread / 4;
    constexpr int kGroups = (kBK / 8) / 2;
    const int row = threadIdx.x >> 1;
    const int part = threadIdx.x & 1;
    RegTable table;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint32_t hi = 0;
      uint32_t lo = 0;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int idx = 4 * q + e;
        const float c = (BITS <= 4 && idx < (1 << BITS)) ? s_cent[idx] : 0.0f;
        const uint32_t bits = __half_as_ushort(__float2half_rn(c * table_scale));
        hi |= (bits >> 8) << (8 * e);
        lo |= (bits & 0xffu) << (8 * e);
      }
      table.hi[q] = hi;
      table.lo[q] = lo;
    }
    // RTN: the table holds the integers -8 .. 7 as bf16 (exact); a decoded pair is then
    // multiplied by the row's scale of this k step with one bf16x2 multiply.  (i - 8) * scale
    // is exact in fp32 (a 4-bit integer times an 8-bit significand), so the single rounding of
    // mul.rn.bf16x2 equals the reference's bf16((i - 8) * scale) (packed_adaln_cpu.cpp:61-73).
    if (RTN) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint32_t hi = 0;
        uint32_t lo = 0;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const uint32_t bits = __bfloat16_as_ushort(__float2bfloat16_rn(static_cast<float>(4 * q + e - 8)));
          hi |= (bits >> 8) << (8 * e);
          lo |= (bits & 0xffu) << (8 * e);
        }
        table.hi[q] = hi;
        table.lo[q] = lo;
      }
    }
    auto rtn_scale = [&](uint4 &v, uint32_t scale2) {
      const __nv_bfloat162 sc = *reinterpret_cast<const __nv_bfloat162 *>(&scale2);
      uint32_t *w = reinterpret_cast<uint32_t *>(&v);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const __nv_bfloat162 prod = __hmul2(*reinterpret_cast<const __nv_bfloat162 *>(&w[e]), sc);
        w[e] = *reinterpret_cast<const uint32_t *>(&prod);
      }
    };
    const uint16_t *lane_lut = s_lut + (BITS == 6 ? lane : (lane & 7));
    // sign-symmetric 4-bit tables (every Lloyd-Max codebook; not the RTN integers) take the
    // shorter decode, the whole warp or none of it
    const bool symmetric = BITS == 4 && !RTN && __all_sync(0xffffffffu, table_is_symmetric(table));
    const uint32_t row_off = (row >> 3) * 1024 + (row & 7) * 128;
    SkinnyRing copy;
    SkinnyRing slot;
    bool ok = true;
    for (int u = blockIdx.x; u < p.units && ok; u += gridDim.x) {
      const SkinnyUnit unit = skinny_unit(p, u);
      // 3-bit rows come straight from global memory (4-byte loads, one k step ahead)
      const int64_t n_global = static_cast<int64_t>(unit.n_tile) * kSkRows + row;
      const bool row_valid = n_global < p.out_features;
      const uint8_t *grow = p.packed + n_global * (static_cast<int64_t>(p.k_iters) * T::kRowBytes) +
                            static_cast<int64_t>(unit.it_begin) * T::kRowBytes + part * kBytesPerThread;
      uint32_t words[kWords];
      auto load_global = [&](int it, uint32_t (&dst)[kWords]) {
#pragma unroll
        for (int q = 0; q < kWords; ++q) {
          dst[q] = (row_valid && it < unit.iters)
                       ? __ldg(reinterpret_cast<const uint32_t *>(grow + static_cast<int64_t>(it) * T::kRowBytes) + q)
                       : 0u;
        }
      };
      if (!T::kPackedByTma) {
        load_global(0, words);
      }
      // RTN: this row's scale of every k step, fetched one step ahead
      const __nv_bfloat16 *scale_row =
          RTN ? p.rtn_scales + (row_valid ? n_global : 0) * p.k_iters + unit.it_begin : nullptr;
      uint32_t scale_now = RTN ? __bfloat16_as_ushort(scale_row[0]) : 0u;
      for (int it = 0; it < unit.iters; ++it) {
        const int s = copy.index;
        const int w = slot.index;
        uint32_t next_words[kWords];
        if (!T::kPackedByTma) {
          load_global(it + 1, next_words);
        }
        uint32_t scale_next = 0u;
        if (RTN) {
          scale_next = it + 1 < unit.iters ? __bfloat16_as_ushort(scale_row[it + 1]) : 0u;
        }
        if (!mbar_wait(full_bar(s), copy.phase, s_abort, 14)) {
          ok = false;
          break;
        }
        if (!mbar_wait(free_bar(w), slot.phase ^ 1u, s_abort, 17)) {
          ok = false;
          break;
        }
        if (T::kPackedByTma) {
          const unsigned char *src = p_ptr(s) + row * T::kRowBytes + part * kBytesPerThread;
          if (kBytesPerThread % 16 == 0) {
#pragma unroll
            for (int q = 0; q < kWords / 4; ++q) {
              const uint4 v = reinterpret_cast<const uint4 *>(src)[q];
              words[4 * q + 0] = v.x;
              words[4 * q + 1] = v.y;
              words[4 * q + 2] = v.z;
              words[4 * q + 3] = v.w;
            }
          } else if (kBytesPerThread % 8 == 0) {
#pragma unroll
            for (int q = 0; q < kWords / 2; ++q) {
              const uint2 v = reinterpret_cast<const uint2 *>(src)[q];
              words[2 * q] = v.x;
              words[2 * q + 1] = v.y;
            }
          } else {
#pragma unroll
            for (int q = 0; q < kWords; ++q) {
              words[q] = reinterpret_cast<const uint32_t *>(src)[q];
            }
          }
        }
        const uint32_t dst_row = w_addr(w) + row_off;
        // Decode every group first and store afterwards: the stores are volatile asm, which the
        // compiler keeps in program order, and a decode-store-decode-store sequence would chain
        // the (latency-bound) byte-permute sequences one after the other instead of overlapping them.
        uint4 expanded[kGroups];
#pragma unroll
        for (int c = 0; c < kGroups; ++c) {
          uint32_t lo;
          uint32_t hi;
          group_bits<BITS, kWords>(words, c, lo, hi);
          if (symmetric) {
            decode8_w4_symmetric(lo, table, expanded[c]);
          } else if (BITS == 4) {
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
          if (RTN) {
            rtn_scale(expanded[c], scale_now | (scale_now << 16));
          }
        }
#pragma unroll
        for (int c = 0; c < kGroups; ++c) {
          const int chunk = part * kGroups + c;
          const uint32_t dst = dst_row + (((chunk ^ (row & 7)) & 7) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(expanded[c].x),
                       "r"(expanded[c].y), "r"(expanded[c].z), "r"(expanded[c].w)
                       : "memory");
        }
        if (!T::kPackedByTma) {
#pragma unroll
          for (int q = 0; q < kWords; ++q) {
            words[q] = next_words[q];
          }
        }
        scale_now = scale_next;
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(ready_bar(w));
        }
        copy.advance(p.copy_stages);
        slot.advance(p.slots);
      }
    }
  } else {
    // ---- epilogue warps: tensor-memory lane = weight row, column = token ----
    const int quarter = warp & 3;
    int local = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < p.units && ok; u += gridDim.x, ++local) {
      const SkinnyUnit unit = skinny_unit(p, u);
      const int buf = local & 1;
      const int64_t n = static_cast<int64_t>(unit.n_tile) * kSkRows + quarter * 32 + lane;
      const bool n_ok = n < p.out_features;
      float scale_n = 0.0f;
      float bias_n = 0.0f;
      if (n_ok) {
        scale_n = RTN ? 1.0f : __fdiv_rn(__bfloat162float(p.row_norms[n]), table_scale);
        bias_n = p.bias_dtype >= 0 ? load_bias(p.bias, p.bias_dtype, n) : 0.0f;
      }
      if (!mbar_wait(acc_full_bar(buf), (local >> 1) & 1u, s_abort, 15)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t acc = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * acc_cols;
      __nv_bfloat16 *out = static_cast<__nv_bfloat16 *>(p.out);
      float *part = p.partial + static_cast<int64_t>(unit.split) * p.n_pad * p.out_features + n;
#pragma unroll 1
      for (int c0 = 0; c0 < p.n_pad; c0 += 16) {
        uint32_t v[16];
        tmem_ld_32x32b_x16(acc + c0, v);
        tmem_ld_wait();
        if (n_ok) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int tok = c0 + j;
            if (tok < p.rows) {
              if (p.splits == 1) {
                out[static_cast<int64_t>(tok) * p.out_features + n] =
                    __float2bfloat16_rn(fmaf(__uint_as_float(v[j]), s_tok[tok] * scale_n, bias_n));
              } else {
                part[static_cast<int64_t>(tok) * p.out_features] = __uint_as_float(v[j]);
              }
            }
          }
        }
      }
      // this accumulator may be overwritten now
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(acc_empty_bar(buf));
      }
      if (p.splits > 1) {
        // Whichever CTA finishes the LAST slice of these 32 weight rows adds all the slices
        // -- always in slice order, so the result does not depend on who that is.
        __threadfence();
        __syncwarp();
        int done = 0;
        if (lane == 0) {
          done = atomicAdd(p.counters + unit.n_tile * 4 + quarter, 1);
        }
        done = __shfl_sync(0xffffffffu, done, 0);
        if (done == p.splits - 1) {
          __threadfence();
          if (n_ok) {
            // eight tokens at a time, so that 8 x (unrolled slices) loads are in flight
            const float *all = p.partial + n;
            const int64_t tok_stride = p.out_features;
            const int64_t slice_stride = static_cast<int64_t>(p.n_pad) * p.out_features;
            for (int tok0 = 0; tok0 < p.rows; tok0 += 8) {
              float sum[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll 4
              for (int sl = 0; sl < p.splits; ++sl) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  // rows past the last token are inside the buffer (n_pad rows) but unwritten;
                  // their sums are never stored
                  sum[j] += __ldcg(all + sl * slice_stride + (tok0 + j) * tok_stride);
                }
              }
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const int tok = tok0 + j;
                if (tok < p.rows) {
                  out[static_cast<int64_t>(tok) * p.out_features + n] =
                      __float2bfloat16_rn(fmaf(sum[j], s_tok[tok] * scale_n, bias_n));
                }
              }
            }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kSkMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, tmem_cols);
  }
}

struct SkinnyPlan {
  int n_pad;
  int n_tiles;
  int splits;
  int chunk_iters;
};

inline SkinnyPlan skinny_plan(int64_t rows, int64_t in_features, int64_t out_features, int sm_count) {
  SkinnyPlan plan;
  plan.n_pad = static_cast<int>((rows + 15) / 16 * 16);
  plan.n_tiles = static_cast<int>((out_features + kSkRows - 1) / kSkRows);
  const int k_iters = static_cast<int>(in_features / kBK);
  // at least two units per resident CTA, with at least kSkMinItersPerSplit k steps each
  int per_sm = 4;
  if (tunable(OQ_TUNE_SKINNY_UNITS_PER_SM) > 0) {
    per_sm = tunable(OQ_TUNE_SKINNY_UNITS_PER_SM);
  }
  const int wanted = per_sm * sm_count;
  int splits = (wanted + plan.n_tiles - 1) / plan.n_tiles;
  int min_iters = kSkMinItersPerSplit;
  if (tunable(OQ_TUNE_SKINNY_MIN_ITERS) > 0) {
    min_iters = tunable(OQ_TUNE_SKINNY_MIN_ITERS);
  }
  int most = k_iters / min_iters > 0 ? k_iters / min_iters : 1;
  // every slice writes (and the reduction re-reads) n_pad x 128 fp32 partial sums per unit:
  // keep that traffic under about half of the packed weight bytes
  const int64_t traffic_cap = in_features / (32 * static_cast<int64_t>(plan.n_pad));
  most = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(most, traffic_cap)));
  splits = splits < 1 ? 1 : (splits > most ? most : splits);
  plan.chunk_iters = (k_iters + splits - 1) / splits;
  plan.splits = (k_iters + plan.chunk_iters - 1) / plan.chunk_iters;
  return plan;
}

// Workspace of the sliced reduction: [4 counters per weight tile, padded to 256 bytes]
// [partial sums].
inline size_t skinny_counter_bytes(const SkinnyPlan &plan) {
  return (static_cast<size_t>(plan.n_tiles) * 4 * sizeof(int) + 255) / 256 * 256;
}

inline size_t skinny_partial_bytes(const SkinnyPlan &plan, int64_t out_features) {
  return plan.splits > 1
             ? skinny_counter_bytes(plan) +
                   static_cast<size_t>(plan.splits) * plan.n_pad * out_features * sizeof(float)
             : 0;
}

template <int BITS, bool RTN = false>
int launch_skinny_bits(const CUtensorMap &map_x, const CUtensorMap &map_p, SkinnyParams p,
                       int sm_count, cudaStream_t stream) {
  using T = SkinnyTile<BITS>;
  static std::once_flag once;
  static cudaError_t attr_status = cudaSuccess;
  std::call_once(once, [] {
    attr_status = cudaFuncSetAttribute(skinny_tcgen05_kernel<BITS, RTN>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       232448);
  });
  OQ_CHECK_CUDA(attr_status);
  p.copy_stages = T::copy_stages(p.n_pad);
  p.copy_stage_bytes = T::copy_stage_bytes(p.n_pad);
  p.slots = T::slots(p.n_pad);
  if (p.copy_stages < 2) {
    return fail(OQ_ERR_UNSUPPORTED, "the few-token kernel's tiles do not fit in shared memory");
  }
  p.units = p.n_tiles * p.splits;
  const int smem = T::smem_bytes(p.n_pad);
  const int resident = smem <= 113 * 1024 ? 2 : 1;
  const int grid = p.units < resident * sm_count ? p.units : resident * sm_count;
  // Programmatic stream serialization: the grid may start while the kernel before it in the
  // stream is still running (once that kernel has executed griddepcontrol.launch_dependents
  // in every CTA); griddepcontrol.wait inside orders every dependent read after its end.
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(grid);
  config.blockDim = dim3(kSkThreads);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attr;
  config.numAttrs = 1;
  OQ_CHECK_CUDA(cudaLaunchKernelEx(&config, skinny_tcgen05_kernel<BITS, RTN>, map_x, map_p, p));
  count_launch();
  return OQ_OK;
}
