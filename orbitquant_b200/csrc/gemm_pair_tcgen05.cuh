// Large-row codebook-decode GEMM on a PAIR of CTAs (tcgen05 cta_group::2).  Included by
// gemm_tcgen05.cu inside its anonymous namespace; uses that file's PTX wrappers and decode
// routines.
//
// The single-CTA kernel is co-limited by the index decode: expanding a 256 x 64 weight tile
// costs its eight expander warps about as long as the MMAs that tile feeds.  Here two CTAs of
// a cluster share every expanded tile: a pair computes a 512 x 256 output tile, each CTA
// holds 256 of the rows (two 128 x 256 accumulators in its tensor memory, as before) but
// expands only HALF of the weight tile (128 rows).  One thread of the leader CTA issues
// tcgen05.mma.cta_group::2 (M = 256: 128 rows from each CTA's activation tile; N = 256: 128
// weight rows from each CTA's expanded tile), so per unit of MMA work the decode is halved.
//
//   per CTA and k step: TMA of its own 256 x 64 activation tile and its own 128-row packed
//   tile -> local `full[s]`; its expanders write its half of the f16 weight tile and arrive
//   on the LEADER's `bready[s]` (16 arrivals: 8 local warps + 8 of the peer, the peer's
//   through mapa + a cluster-scope mbarrier arrive); the leader's MMA thread issues 2 x 4
//   MMAs and one tcgen05.commit arrives on both CTAs' `empty[s]` (and, at the end, `acc_full`).
//
// Every TMA load is an ordinary per-CTA load into the issuing CTA's own shared memory.
// Waits are bounded as in the single-CTA kernel; the two cluster-wide barriers (after barrier
// init, before tensor-memory release) are hardware barriers that every thread of both CTAs
// reaches on every path.

template <int BITS>
struct PairTile {
  static constexpr int kBN = 256;      // pair tile width
  static constexpr int kHalfN = 128;   // weight rows expanded by one CTA
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = kHalfN * kBK * 2;
  static constexpr int kRowBytes = kBK * BITS / 8;
  static constexpr int kPBytes = kHalfN * kRowBytes;
  static constexpr bool kPackedByTma = BITS != 3;
  static constexpr int kLutBytes = BITS == 6 ? 64 * 32 * 2 : (BITS == 8 ? 256 * 8 * 2 : 0);
  static constexpr int kStageBytes = (kABytes + kBBytes + kPBytes + 1023) / 1024 * 1024;
  static constexpr int kHeaderBytes = 256 + 2 * kBN * 4 + 256 * 4 + kLutBytes;
  static constexpr int kFit = (232448 - kHeaderBytes - 1024) / kStageBytes;
  static constexpr int kStages = kFit > 4 ? 4 : kFit;
  static_assert(kStages >= 2, "tile does not fit in shared memory");
  static constexpr int kSmemBytes = kHeaderBytes + 1024 + kStages * kStageBytes;
  static constexpr int kTmemCols = 512;
  static constexpr int kExpanderWarps = 8;  // 2 threads per weight row
  static constexpr int kProducerWarp = kExpanderWarps;
  static constexpr int kMmaWarp = kExpanderWarps + 1;
  static constexpr int kThreads = (kExpanderWarps + 2) * 32;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Address of the same shared-memory location in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(addr), "r"(rank));
  return out;
}

__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}

// Bounded wait with cluster-scope acquire (the arrivals come from the peer CTA too).
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity,
                                                  volatile int *abort_flag, int code) {
  for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
    if (mbar_try_wait_cluster(bar, parity)) {
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

__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
               "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols)
               : "memory");
}

__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                              uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Arrives on the barrier at this shared-memory offset in every CTA of `mask`.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar, uint16_t mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(bar), "h"(mask)
      : "memory");
}

// Instruction descriptor of the pair MMA: f32 accumulator, f16 x f16, K-major, M = 256.
__host__ __device__ constexpr uint32_t instr_desc_pair(int n) {
  return (1u << 4) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(256 >> 4) << 24);
}

template <int BITS>
__global__ void __launch_bounds__((PairTile<BITS>::kThreads), 1)
gemm_pair_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a,
                         const __grid_constant__ CUtensorMap map_p, const GemmParams p) {
  using T = PairTile<BITS>;
  constexpr int BN = T::kBN;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem_raw);
  uint32_t *s_tmem = reinterpret_cast<uint32_t *>(smem_raw + 192);
  volatile int *s_abort = reinterpret_cast<volatile int *>(smem_raw + 200);
  float *s_scale = reinterpret_cast<float *>(smem_raw + 256);
  float *s_bias = s_scale + BN;
  float *s_cent = s_bias + BN;
  uint16_t *s_lut = reinterpret_cast<uint16_t *>(s_cent + 256);
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
  const uint32_t rank = cluster_ctarank();          // 0 = leader (issues the MMAs)
  const int pair = blockIdx.x >> 1;
  const int m_pair = pair % p.m_tiles;              // m_tiles = 512-row pair tiles here
  const int n_tile = pair / p.m_tiles;
  const int64_t m0 = static_cast<int64_t>(m_pair) * (2 * kBM) + rank * kBM;  // this CTA's 256 rows
  const int64_t n0 = static_cast<int64_t>(n_tile) * BN;                      // the pair's columns
  const int64_t nb0 = n0 + rank * T::kHalfN;        // the weight rows this CTA expands

  if (threadIdx.x == 0) {
    for (int s = 0; s < T::kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
      mbar_init(bready_bar(s), 2 * T::kExpanderWarps);  // used in the leader only
    }
    mbar_init(acc_full_bar, 1);
    *s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == T::kMmaWarp) {
    tmem_alloc_pair(smem_u32(s_tmem), T::kTmemCols);
  }
  if (warp == T::kProducerWarp && lane == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_p) : "memory");
  }
  for (int i = threadIdx.x; i < (1 << BITS); i += T::kThreads) {
    s_cent[i] = p.centroids[i];
  }
  // no CTA may arrive on the peer's barriers before they exist
  tc_fence_before();
  cluster_sync_all();
  tc_fence_after();
  asm volatile("griddepcontrol.wait;" ::: "memory");  // see the single-CTA kernel
  const float table_scale = p.table_scale != nullptr ? __ldg(p.table_scale) : kCentroidScale;
  if (BITS == 6) {
    for (int i = threadIdx.x; i < 64 * 32; i += T::kThreads) {
      s_lut[i] = __half_as_ushort(__float2half_rn(s_cent[i >> 5] * table_scale));
    }
  } else if (BITS == 8) {
    for (int i = threadIdx.x; i < 256 * 8; i += T::kThreads) {
      s_lut[i] = __half_as_ushort(__float2half_rn(s_cent[i >> 3] * table_scale));
    }
  }
  for (int i = threadIdx.x; i < BN; i += T::kThreads) {
    const int64_t n = n0 + i;
    const bool ok = n < p.out_features;
    s_scale[i] = ok ? __fdiv_rn(__bfloat162float(p.row_norms[n]), table_scale) : 0.0f;
    s_bias[i] = (ok && p.bias_dtype >= 0) ? load_bias(p.bias, p.bias_dtype, n) : 0.0f;
  }
  __syncthreads();
  const uint32_t tmem_base = *s_tmem;

  if (warp == T::kProducerWarp) {
    if (lane == 0) {
      int issued = 0;
      for (int it = 0; it < p.k_iters; ++it) {
        const int s = it % T::kStages;
        const uint32_t phase = (it / T::kStages) & 1u;
        if (!mbar_wait(empty_bar(s), phase ^ 1u, s_abort, 21)) {
          break;
        }
        mbar_arrive_expect_tx(full_bar(s), T::kABytes + (T::kPackedByTma ? T::kPBytes : 0));
        tma_load_2d(a_addr(s), &map_a, full_bar(s), it * kBK, static_cast<int>(m0));
        if (T::kPackedByTma) {
          tma_load_2d(smem_u32(p_ptr(s)), &map_p, full_bar(s), it * T::kRowBytes, static_cast<int>(nb0));
        }
        issued = it + 1;
      }
      if (*s_abort != 0) {
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
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = instr_desc_pair(BN);
      bool ok = true;
      for (int it = 0; it < p.k_iters && ok; ++it) {
        const int s = it % T::kStages;
        const uint32_t phase = (it / T::kStages) & 1u;
        // 16 arrivals: every expander warp of both CTAs, each of which has seen its own
        // CTA's activation and packed tiles land before expanding
        ok = mbar_wait_cluster(bready_bar(s), phase, s_abort, 23);
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
            umma_f16_pair(tmem_base + half * BN, da, db, idesc, (it > 0 || j > 0) ? 1u : 0u);
          }
        }
        umma_commit_pair(empty_bar(s), 3);
      }
      if (ok) {
        umma_commit_pair(acc_full_bar, 3);
      }
    }
  } else {
    // ---- expanders: this CTA's 128 weight rows, 2 threads per row ----
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
    const uint16_t *lane_lut = s_lut + (BITS == 6 ? lane : (lane & 7));
    const uint32_t row_off = (row >> 3) * 1024 + (row & 7) * 128;
    const int64_t n_global = nb0 + row;
    const bool row_valid = n_global < p.out_features;
    const uint8_t *grow = p.packed + n_global * (static_cast<int64_t>(p.k_iters) * T::kRowBytes) +
                          part * kBytesPerThread;
    uint32_t words[kWords];
    auto load_global = [&](int it, uint32_t (&dst)[kWords]) {
#pragma unroll
      for (int q = 0; q < kWords; ++q) {
        dst[q] = (row_valid && it < p.k_iters)
                     ? __ldg(reinterpret_cast<const uint32_t *>(grow + static_cast<int64_t>(it) * T::kRowBytes) + q)
                     : 0u;
      }
    };
    const uint32_t leader_bready0 = map_to_cta(bready_bar(0), 0);
    bool ok = true;
    if (!T::kPackedByTma) {
      load_global(0, words);
    }
    for (int it = 0; it < p.k_iters; ++it) {
      const int s = it % T::kStages;
      const uint32_t phase = (it / T::kStages) & 1u;
      uint32_t next_words[kWords];
      if (!T::kPackedByTma) {
        load_global(it + 1, next_words);
      }
      if (!mbar_wait(full_bar(s), phase, s_abort, 24)) {
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
      const uint32_t dst_row = b_addr(s) + row_off;
      uint4 expanded[kGroups];
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
#pragma unroll
      for (int c = 0; c < (p.debug_skip ? 0 : kGroups); ++c) {
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
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive_cluster(leader_bready0 + 8u * s);
      }
    }

    // ---- epilogue: as in the single-CTA kernel, on this CTA's 256 rows ----
    constexpr int kPitch = BN * 2 + 16;
    static_assert(kEpilogueWarps * 32 * kPitch <= T::kStages * T::kStageBytes, "epilogue staging space");
    if (ok && mbar_wait(acc_full_bar, 0, s_abort, 25)) {
      tc_fence_after();
      const int half = warp >> 2;
      const int quarter = warp & 3;
      const int64_t m_first = m0 + half * 128 + quarter * 32;
      const int64_t m = m_first + lane;
      const float row_scale = m < p.rows ? p.row_scale[m] : 0.0f;
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
            const float a = fmaf(__uint_as_float(v[2 * j]), row_scale * s_scale[c0 + 2 * j],
                                 s_bias[c0 + 2 * j]);
            const float b = fmaf(__uint_as_float(v[2 * j + 1]), row_scale * s_scale[c0 + 2 * j + 1],
                                 s_bias[c0 + 2 * j + 1]);
            const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
            w[e] = *reinterpret_cast<const uint32_t *>(&h);
          }
          dst[q] = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
      __syncwarp();
      const bool vec_ok = (p.out_features % 8) == 0 && (p.out_ld % 8) == 0 && (p.out_col % 8) == 0;
      const int64_t n = n0 + lane * 8;
      const bool lane_full = n + 8 <= p.out_features;
      const int64_t rows_here = p.rows - m_first < 32 ? p.rows - m_first : 32;
      for (int d = 0; d < p.n_outs; ++d) {
        __nv_bfloat16 *out = static_cast<__nv_bfloat16 *>(p.outs[d]) + p.out_col + n;
#pragma unroll 4
        for (int r = 0; r < rows_here; ++r) {
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

  // Neither CTA may release tensor memory (or exit) while the pair's MMAs or the peer's
  // remote arrivals can still touch it.
  tc_fence_before();
  cluster_sync_all();
  if (warp == T::kMmaWarp) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, T::kTmemCols);
  }
}

template <int BITS>
int launch_pair_bits(const CUtensorMap &map_a, const CUtensorMap &map_p, const GemmParams &p,
                     int pairs, cudaStream_t stream) {
  using T = PairTile<BITS>;
  static std::once_flag once;
  static cudaError_t attr_status = cudaSuccess;
  std::call_once(once, [] {
    attr_status = cudaFuncSetAttribute(gemm_pair_tcgen05_kernel<BITS>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, T::kSmemBytes);
  });
  OQ_CHECK_CUDA(attr_status);
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(2 * pairs);
  config.blockDim = dim3(T::kThreads);
  config.dynamicSmemBytes = T::kSmemBytes;
  config.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attr;
  config.numAttrs = 2;
  OQ_CHECK_CUDA(cudaLaunchKernelEx(&config, gemm_pair_tcgen05_kernel<BITS>, map_a, map_p, p));
  count_launch();
  return OQ_OK;
}
