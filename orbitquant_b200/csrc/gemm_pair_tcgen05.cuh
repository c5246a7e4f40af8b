// Large-row codebook-decode GEMM on a PAIR of CTAs (tcgen05 cta_group::2).  Included by
// gemm_tcgen05.cu inside its anonymous namespace; uses that file's PTX wrappers, its expander
// loop and its epilogue.
//
// The single-CTA kernel moves 160 KB through shared memory per k step (activation tile in and
// out once, expanded weight tile in once and out twice, because each of its two 128-row MMAs
// reads the whole 256-row B operand) -- as long as the MMAs themselves take -- and its
// expander warps need about as long again for the index decode.  A pair halves both: the two
// CTAs of a cluster compute a 512 x 256 output tile, each holds 256 of the rows (two
// 128 x 256 accumulators in its tensor memory, as before) but expands and stores only HALF
// of the weight tile (128 rows), and one thread of the leader CTA issues
// tcgen05.mma.cta_group::2 (M = 256: 128 rows from each CTA's activation tile; N = 256: 128
// weight rows from each CTA's expanded tile).
//
//   per CTA and k step   TMA of its own 256 x 64 activation tile and its own 128-row packed
//                        tile -> local `full[s]`; its expanders write its half of the weight
//                        tile and arrive on the local `bready[s]`.
//   hand-over            the peer CTA's otherwise idle MMA-warp thread waits for the peer's
//                        `full[s]` and `bready[s]` and forwards ONE arrival to `peer[s]` in the
//                        leader, released at CTA scope (see mbar_arrive_remote).  A
//                        cluster-scope release from every expander warp instead (sixteen per k
//                        step) stalls the expanders on a memory barrier of about a microsecond
//                        each time: measured 4 stall cycles per issued instruction and a
//                        tensor pipe 50 % busy, slower than one CTA.
//   MMA                  the leader waits for its `full[s]`, `bready[s]` and `peer[s]`, issues
//                        2 x 4 MMAs, and one tcgen05.commit arrives on both CTAs' `empty[s]`
//                        (and, at the end, `acc_full`).
//
// Every TMA load is an ordinary per-CTA load into the issuing CTA's own shared memory.
// Waits are bounded as in the single-CTA kernel; the two cluster-wide barriers (after barrier
// init, before tensor-memory release) are hardware barriers that every thread of both CTAs
// reaches on every path.

// I8: INT8 operands (kind::i8, 32-bit integer accumulators) -- a k step is 128 values, i.e. the
// same 128-byte operand rows as 64 values of a 16-bit type.
template <int BN, int BITS, bool I8 = false>
struct PairTile {
  static constexpr int kBN = BN;           // pair tile width (256 or 192)
  static constexpr int kHalfN = BN / 2;    // weight rows expanded by one CTA
  static constexpr bool kI8 = I8;
  static constexpr int kStepElems = I8 ? 2 * kBK : kBK;   // k values per pipeline step
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = kHalfN * kBK * 2;
  static constexpr int kRowBytes = kStepElems * BITS / 8;
  static_assert(!I8 || BITS == 4, "INT8 code tables exist for 4-bit indices");
  static constexpr bool kPackedByTma = BITS != 3;
  static constexpr int kPBytes = kPackedByTma ? kHalfN * kRowBytes : 0;
  static constexpr int kStageBytes = (kABytes + kBBytes + kPBytes + 1023) / 1024 * 1024;
  static constexpr int kCentFloats = 1 << BITS;
  static constexpr int kHeaderBytes = 256 + 2 * kBN * 4 + kCentFloats * 4;
  static constexpr int kFit = (232448 - kHeaderBytes - 1024) / kStageBytes;
  static constexpr int kStages = kFit > 4 ? 4 : kFit;
  static_assert(kStages >= 2, "tile does not fit in shared memory");
  static_assert((4 * kStages + 1) * 8 <= 192, "barrier block");
  static_assert(kHalfN % 8 == 0 && BN % 16 == 0, "operand layout");
  static constexpr int kSmemBytes = kHeaderBytes + 1024 + kStages * kStageBytes;
  static constexpr int kTmemCols = 512;
  static constexpr int kTpr = 2;            // expander threads per weight row
  static constexpr int kExpanderWarps = kHalfN * kTpr / 32;   // 8 or 6
  // warps 0..7 run the epilogue; those beyond the expander warps idle through the k loop
  static constexpr int kProducerWarp = kEpilogueWarps;
  static constexpr int kMmaWarp = kEpilogueWarps + 1;
  static constexpr int kThreads = (kEpilogueWarps + 2) * 32;
  static_assert(kExpanderWarps <= kEpilogueWarps, "warp roles");
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

// Arrival on a barrier of the peer CTA.  Release at CTA scope: what the arrival publishes
// (this CTA's shared memory, written by its own threads and its own TMA copies) lives in this
// SM, so it is complete for any reader once it is complete here; a cluster-scope release
// would add a memory barrier of about a microsecond to every hand-over.
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
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

__device__ __forceinline__ void umma_i8_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                             uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
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

// Instruction descriptor of the INT8 pair MMA: 32-bit integer accumulator (format code 2),
// A = B = signed 8-bit (format code 1), K-major, M = 256, 32 k values per instruction.
__host__ __device__ constexpr uint32_t instr_desc_pair_i8(int n) {
  return (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(256 >> 4) << 24);
}

// Instruction descriptor of the pair MMA: as instr_desc(), M = 256.
__host__ __device__ constexpr uint32_t instr_desc_pair(int n, bool bf16_operands) {
  return (1u << 4) | ((bf16_operands ? 1u : 0u) << 7) | ((bf16_operands ? 1u : 0u) << 10) |
         (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(256 >> 4) << 24);
}

template <int BN, int BITS, bool SCALED, bool I8 = false>
__global__ void __launch_bounds__((PairTile<BN, BITS, I8>::kThreads), 1)
gemm_pair_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a,
                         const __grid_constant__ CUtensorMap map_p, const GemmParams p) {
  using T = PairTile<BN, BITS, I8>;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  // header: barriers | scale[BN] | bias[BN] | codebook
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem_raw);
  uint32_t *s_tmem = reinterpret_cast<uint32_t *>(smem_raw + 192);
  volatile int *s_abort = reinterpret_cast<volatile int *>(smem_raw + 200);
  float *s_scale = reinterpret_cast<float *>(smem_raw + 256);
  float *s_bias = s_scale + BN;
  float *s_cent = s_bias + BN;
  const uint32_t header_end = smem_u32(smem_raw) + T::kHeaderBytes;
  const uint32_t stage_base = (header_end + 1023u) & ~1023u;
  unsigned char *stage_ptr = smem_raw + (stage_base - smem_u32(smem_raw));

  // full | empty | bready as the expander loop expects them, then peer | acc_full
  const uint32_t bar_base = smem_u32(bars);
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (T::kStages + s); };
  auto bready_bar = [&](int s) { return bar_base + 8u * (2 * T::kStages + s); };
  auto peer_bar = [&](int s) { return bar_base + 8u * (3 * T::kStages + s); };   // leader only
  const uint32_t acc_full_bar = bar_base + 8u * (4 * T::kStages);

  auto a_addr = [&](int s) { return stage_base + s * T::kStageBytes; };
  auto b_addr = [&](int s) { return stage_base + s * T::kStageBytes + T::kABytes; };
  auto p_addr = [&](int s) { return stage_base + s * T::kStageBytes + T::kABytes + T::kBBytes; };

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();          // 0 = leader (issues the MMAs)
  const int pair = blockIdx.x >> 1;
  // p.m_tiles counts 512-row pair tiles, p.n_tiles 256-column tiles
  const int m_pair = p.columns_fastest ? pair / p.n_tiles : pair % p.m_tiles;
  const int n_tile = p.columns_fastest ? pair % p.n_tiles : pair / p.m_tiles;
  const int64_t m0 = static_cast<int64_t>(m_pair) * (2 * kBM) + rank * kBM;  // this CTA's 256 rows
  const int64_t n0 = static_cast<int64_t>(n_tile) * BN;                      // the pair's columns
  const int64_t nb0 = n0 + rank * T::kHalfN;        // the weight rows this CTA expands

  if (threadIdx.x == 0) {
    for (int s = 0; s < T::kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
      mbar_init(bready_bar(s), T::kExpanderWarps);
      mbar_init(peer_bar(s), 1);
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
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // see the single-CTA kernel
  asm volatile("griddepcontrol.wait;" ::: "memory");
  // the copies of the first stages leave before the tables below are built
  int issued_early = 0;
  if (warp == T::kProducerWarp && lane == 0) {
    for (; issued_early < T::kStages && issued_early < p.k_iters; ++issued_early) {
      const int s = issued_early;
      mbar_arrive_expect_tx(full_bar(s), T::kABytes + T::kPBytes);
      tma_load_2d(a_addr(s), &map_a, full_bar(s), s * T::kStepElems, static_cast<int>(m0));
      if (T::kPackedByTma) {
        tma_load_2d(p_addr(s), &map_p, full_bar(s), s * T::kRowBytes, static_cast<int>(nb0));
      }
    }
  }
  const float table_scale =
      SCALED ? 1.0f : (p.table_scale != nullptr ? __ldg(p.table_scale) : kCentroidScale);
  for (int i = threadIdx.x; i < BN; i += T::kThreads) {
    const int64_t n = n0 + i;
    const bool ok = n < p.out_features;
    s_scale[i] = ok ? (SCALED ? 1.0f : __fdiv_rn(__bfloat162float(p.row_norms[n]), table_scale)) : 0.0f;
    s_bias[i] = (ok && p.bias_dtype >= 0) ? load_bias(p.bias, p.bias_dtype, n) : 0.0f;
  }
  __syncthreads();
  const uint32_t tmem_base = *s_tmem;

  if (warp == T::kProducerWarp) {
    if (lane == 0) {
      int issued = issued_early;
      for (int it = issued_early; it < p.k_iters; ++it) {
        const int s = it % T::kStages;
        const uint32_t phase = (it / T::kStages) & 1u;
        if (!mbar_wait(empty_bar(s), phase ^ 1u, s_abort, 21)) {
          break;
        }
        mbar_arrive_expect_tx(full_bar(s), T::kABytes + T::kPBytes);
        tma_load_2d(a_addr(s), &map_a, full_bar(s), it * T::kStepElems, static_cast<int>(m0));
        if (T::kPackedByTma) {
          tma_load_2d(p_addr(s), &map_p, full_bar(s), it * T::kRowBytes, static_cast<int>(nb0));
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
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = I8 ? instr_desc_pair_i8(BN) : instr_desc_pair(BN, SCALED);
      bool ok = true;
      for (int it = 0; it < p.k_iters && ok; ++it) {
        const int s = it % T::kStages;
        const uint32_t phase = (it / T::kStages) & 1u;
        ok = mbar_wait(full_bar(s), phase, s_abort, 22) && mbar_wait(bready_bar(s), phase, s_abort, 23) &&
             mbar_wait(peer_bar(s), phase, s_abort, 24);
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
            // four instructions of 32 operand bytes each: 16 k values of a 16-bit type, 32 of INT8
            if (I8) {
              umma_i8_pair(tmem_base + half * BN, da, db, idesc, (it > 0 || j > 0) ? 1u : 0u);
            } else {
              umma_f16_pair(tmem_base + half * BN, da, db, idesc, (it > 0 || j > 0) ? 1u : 0u);
            }
          }
        }
        umma_commit_pair(empty_bar(s), 3);
      }
      if (ok) {
        umma_commit_pair(acc_full_bar, 3);
      }
    } else if (lane == 0) {
      // The peer's hand-over thread: its activation tile has landed and its half of the weight
      // tile is written -> one arrival in the leader.
      const uint32_t leader_peer0 = map_to_cta(peer_bar(0), 0);
      for (int it = 0; it < p.k_iters; ++it) {
        const int s = it % T::kStages;
        const uint32_t phase = (it / T::kStages) & 1u;
        if (!(mbar_wait(full_bar(s), phase, s_abort, 25) && mbar_wait(bready_bar(s), phase, s_abort, 26))) {
          break;
        }
        mbar_arrive_remote(leader_peer0 + 8u * s);
      }
    }
  } else {
    // ---- expanders (this CTA's 128 weight rows), then the epilogue of this CTA's 256 rows ----
    const bool ok = expand_weight_tiles<T, BITS, SCALED>(p, nb0, stage_base, bar_base, s_cent, nullptr,
                                                         table_scale, s_abort, warp, lane);
    store_output_tile<T, BN, SCALED>(p, m0, n0, tmem_base, stage_ptr, acc_full_bar, s_scale, s_bias,
                                     s_abort, ok, warp, lane);
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

template <int BN, int BITS, bool SCALED, bool I8 = false>
int launch_pair_bn(const CUtensorMap &map_a, const CUtensorMap &map_p, const GemmParams &p,
                   int pairs, cudaStream_t stream) {
  using T = PairTile<BN, BITS, I8>;
  static std::once_flag once;
  static cudaError_t attr_status = cudaSuccess;
  std::call_once(once, [] {
    attr_status = cudaFuncSetAttribute(gemm_pair_tcgen05_kernel<BN, BITS, SCALED, I8>,
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
  OQ_CHECK_CUDA(cudaLaunchKernelEx(&config, gemm_pair_tcgen05_kernel<BN, BITS, SCALED, I8>, map_a, map_p, p));
  count_launch();
  return OQ_OK;
}

template <int BITS, bool SCALED>
int launch_pair_bits(int bn, const CUtensorMap &map_a, const CUtensorMap &map_p, const GemmParams &p,
                     int pairs, cudaStream_t stream) {
  return bn == 256 ? launch_pair_bn<256, BITS, SCALED>(map_a, map_p, p, pairs, stream)
                   : launch_pair_bn<192, BITS, SCALED>(map_a, map_p, p, pairs, stream);
}
