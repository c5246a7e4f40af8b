// Rotate-and-quantize for large token counts: one warp transforms one rotation block.
//
// Same arithmetic, operation order and therefore the same bits as the kernels in prologue.cu
// (bf16 rows, dim a multiple of 256, block 256 .. 4096, x_q output only).  What differs is
// the organisation, chosen so that no CTA-wide barrier and no serial phase sits on the
// critical path:
//
//   norm warps (8, 9)       work ahead of the others on alternate batches of R tokens: wait
//                           for the batch's bulk copy (cp.async.bulk into one of S
//                           shared-memory slots, completion on an mbarrier), compute the
//                           token norms in the reference's AVX-512 order (16
//                           fused-multiply-add chains per token, two per lane, eight lanes per
//                           token, then the 8/4/2/1 fold -- a chain of dim/16 dependent
//                           operations, which is why there are two such warps) and tabulate
//                           every token's possible outputs; then signal `normed[slot]`.
//   transform warps (0..7)  each takes whole 1024-element chunks of a token (one or several
//                           rotation blocks): lane l gathers the 32 values of positions
//                           32l .. 32l+31 through a permutation table kept in shared memory
//                           (index and sign in one word), runs butterfly widths 1 .. 16 in
//                           registers, transposes through a swizzled 4 KB scratch (one 16-byte
//                           store per 4 values, conflict-free reads), runs widths 32 .. 512,
//                           quantises, and the 2 KB of results leave by one bulk store.  For
//                           blocks of 2048 / 4096 a team of 2 / 4 warps shares a block and a
//                           third pass (widths 1024, 2048) follows a team barrier.  The warp
//                           that finishes a batch last refills its slot with the batch S
//                           further on, so copies run S - 1 batches ahead of their use.
//
// Inside every phase all shared-memory loads come first and all stores last (the compiler
// cannot prove that the regions differ and would otherwise wait for each load before the next
// store), and shared memory is addressed with 32-bit addresses throughout.
//
// Quantising replaces the dependent 2^bits-way boundary search by ONE table step: the value
// is mapped linearly onto C cells (a fused multiply-add whose result's low mantissa bits are
// the cell number), every cell holds at most one boundary, and the cell's entry gives that
// boundary plus, per token, the two candidate outputs.  The cell table is derived by the
// kernel itself from the boundaries with the very instruction sequence that later reads it
// (binary search over float bit patterns for each cell's first value), so it is exact for
// any codebook; if some cell would hold two boundaries even with twice the cells, the kernel
// falls back to the boundary search.
#pragma once

namespace oq {

__device__ int g_prologue_status = 0;  // 0 = ok; otherwise the code of the first wait that gave up

namespace {

constexpr int kPwWarps = 8;                       // transform warps (16 in the wide variant)
constexpr int kPwWideWarps = 16;
constexpr int kPwNormWarps = 2;
__host__ __device__ constexpr int pw_threads(int transform_warps) {
  return (transform_warps + kPwNormWarps) * 32;
}
constexpr int kPwChunk = 1024;
constexpr int kPwRowPad = 32;                     // bytes between the rows of a slot
constexpr int kPwMaxRows = 4;                     // tokens per batch
constexpr int kPwMaxSlots = 4;
constexpr uint32_t kPwSpinLimit = 1u << 22;

__host__ __device__ constexpr int pw_max_cells(int bits) {
  return bits >= 8 ? 1024 : (4 << bits);
}

struct WarpPrologueParams {
  const uint16_t *x;
  uint16_t *xq;
  float *row_scale;  // f16 operand mode: per-token factor 2^(E-14); INT8 mode: norm * out_scale
  const int8_t *code_map;  // INT8 mode: output byte of every quantisation level
  float out_scale;         // INT8 mode: factor applied to the token norm
  const int32_t *perm;
  const int8_t *signs;
  const float *boundaries;
  const float *centroids;
  int64_t rows;
  int dim;
  int log2_block;
  int batch_rows;
  int slots;
  float eps;
  float inv_sqrt_block;
  const float *w_centroids;
  int w_bits;
  float *table_scale_out;
  int *zero_words;
  int zero_count;
};

// Shared-memory layout (byte offsets from a 128-byte aligned base).
struct PwLayout {
  int cent, bnd, cell_bnd, cell_meta, slot_meta, outtab, pairs, perm, slots, work;
  int row_pitch, slot_bytes, team_bytes, total;
};

__host__ __device__ inline PwLayout pw_layout(int dim, int block, int batch_rows, int slots, int bits,
                                              int transform_warps = kPwWarps) {
  PwLayout l;
  const int cells = pw_max_cells(bits);
  int at = 128;  // barriers, counters and flags
  l.cent = at;       at += 256 * 4;
  l.bnd = at;        at += 256 * 4;
  l.cell_bnd = at;   at += cells * 4;
  l.cell_meta = at;  at += (cells * 2 + 127) / 128 * 128;
  l.slot_meta = at;  at += kPwMaxSlots * kPwMaxRows * 16;             // norm, inv, opscale, -
  l.outtab = at;     at += (slots * batch_rows * (2 << bits) + 127) / 128 * 128;
  l.pairs = at;      at += slots * batch_rows * cells * 4;
  at = (at + 127) / 128 * 128;
  l.perm = at;       at += (dim + kPwChunk - 1) / kPwChunk * kPwChunk * 4;   // whole chunks
  l.row_pitch = dim * 2 + kPwRowPad;
  l.slot_bytes = batch_rows * l.row_pitch;
  l.slots = at;      at += slots * l.slot_bytes;
  at = (at + 127) / 128 * 128;
  const int team = block > kPwChunk ? block / kPwChunk : 1;
  l.team_bytes = team * kPwChunk * 6;                                  // fp32 scratch + 16-bit results
  l.work = at;       at += (transform_warps / team) * l.team_bytes;
  l.total = at + 128;                                                  // alignment slack
  return l;
}

__device__ __forceinline__ uint32_t pw_smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- shared memory through 32-bit addresses ----
__device__ __forceinline__ uint32_t pw_lds_u16(uint32_t a) {
  uint32_t v;   // a 32-bit destination: the loaded halfword arrives zero-extended
  asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ uint32_t pw_lds_u32(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ float pw_lds_f32(uint32_t a) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ uint4 pw_lds_v4(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}
__device__ __forceinline__ void pw_sts_v4f(uint32_t a, float x, float y, float z, float w) {
  asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(a), "f"(x), "f"(y), "f"(z), "f"(w) : "memory");
}
__device__ __forceinline__ void pw_sts_f32(uint32_t a, float v) {
  asm volatile("st.shared.f32 [%0], %1;" ::"r"(a), "f"(v) : "memory");
}
__device__ __forceinline__ void pw_sts_u16(uint32_t a, uint32_t v) {
  asm volatile("st.shared.u16 [%0], %1;" ::"r"(a), "r"(v) : "memory");   // low halfword of v
}
__device__ __forceinline__ void pw_sts_u8(uint32_t a, uint32_t v) {
  asm volatile("st.shared.u8 [%0], %1;" ::"r"(a), "r"(v) : "memory");    // low byte of v
}

__device__ __forceinline__ void pw_mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}

__device__ __forceinline__ void pw_mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void pw_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool pw_mbar_try_wait(uint32_t bar, uint32_t parity) {
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

// Bounded wait: gives up after the spin limit (or when another role has given up), raising the
// CTA's abort flag and the device status word.
__device__ __forceinline__ bool pw_mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int code) {
  for (uint32_t spin = 0; spin < kPwSpinLimit; ++spin) {
    if (pw_mbar_try_wait(bar, parity)) {
      return true;
    }
    if ((spin & 63u) == 63u && *abort_flag != 0) {
      return false;
    }
  }
  *abort_flag = code;
  atomicCAS(&g_prologue_status, 0, code);
  return false;
}

__device__ __forceinline__ void pw_bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}

__device__ __forceinline__ void pw_bulk_store(void *dst, uint32_t src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src), "r"(bytes)
               : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

__device__ __forceinline__ void pw_bulk_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}

__device__ __forceinline__ void pw_fence_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// Barrier among the warps of one team (teams 0 .. 3 use the named barriers 1 .. 4; the ids are
// literals so that the kernel reserves only those).
__device__ __forceinline__ void pw_team_barrier(int team, int threads) {
  switch (team) {
    case 0: asm volatile("bar.sync 1, %0;" ::"r"(threads) : "memory"); break;
    case 1: asm volatile("bar.sync 2, %0;" ::"r"(threads) : "memory"); break;
    case 2: asm volatile("bar.sync 3, %0;" ::"r"(threads) : "memory"); break;
    default: asm volatile("bar.sync 4, %0;" ::"r"(threads) : "memory"); break;
  }
}

// Linear map of a value onto cell numbers: clamp to [lo, hi] (NaN goes to hi, as the
// reference counts NaN above every boundary), then one fused multiply-add whose rounded
// result is 2^23 + cell.
struct PwCellMap {
  float lo, hi, scale, offset;
};

__device__ __forceinline__ PwCellMap pw_cell_map(float lo, float hi, int cells) {
  PwCellMap m;
  m.lo = lo;
  m.hi = hi;
  m.scale = __fdiv_rn(static_cast<float>(cells - 3), __fsub_rn(hi, lo));
  m.offset = __fmaf_rn(-lo, m.scale, 8388609.0f);  // 2^23 + 1: nominal cells 1 .. cells - 2
  return m;
}

__device__ __forceinline__ uint32_t pw_cell_bits(float d, const PwCellMap &m) {
  const float clamped = fmaxf(fminf(d, m.hi), m.lo);
  return __float_as_uint(__fmaf_rn(clamped, m.scale, m.offset));
}

// Order-preserving map between floats and unsigned integers.
__device__ __forceinline__ uint32_t pw_float_key(float v) {
  const uint32_t b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ float pw_key_float(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

// Butterfly widths 1, 2, ... 2^(STAGES-1) over S register values.
template <int S, int STAGES>
__device__ __forceinline__ void pw_butterflies(float (&v)[S]) {
#pragma unroll
  for (int stage = 0; stage < STAGES; ++stage) {
    const int h = 1 << stage;
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

// What a transform thread needs to quantise values of one token.
struct PwQuant {
  PwCellMap map;
  // shared addresses of the per-cell boundaries (float) and of this token's candidate pairs,
  // both minus 4 * 0x4B000000: the cell number arrives as 2^23 + cell in a float's bits
  uint32_t cell_bnd;
  uint32_t pairs;
  const float *bnd;    // boundaries (fallback search)
  const uint16_t *outtab;  // this token's 2^bits outputs (fallback search)
  float isb;
};

// Quantises N register values in place (the results replace the values as raw 16-bit patterns).
template <int BITS, bool CELLS, int N>
__device__ __forceinline__ void pw_quantize_all(float (&w)[N], const PwQuant &q) {
  if (CELLS) {
    // groups of up to 8: the table reads of a group are in flight together, and the register
    // budget stays within two CTAs per SM
    constexpr int kGroup = N < 8 ? N : 8;
#pragma unroll
    for (int a0 = 0; a0 < N; a0 += kGroup) {
      float d[kGroup];
      float b[kGroup];
      uint32_t pair[kGroup];
#pragma unroll
      for (int a = 0; a < kGroup; ++a) {
        d[a] = __fmul_rn(w[a0 + a], q.isb);
        const uint32_t off = pw_cell_bits(d[a], q.map) << 2;
        b[a] = pw_lds_f32(q.cell_bnd + off);
        pair[a] = pw_lds_u32(q.pairs + off);
      }
#pragma unroll
      for (int a = 0; a < kGroup; ++a) {
        w[a0 + a] = __uint_as_float(!(d[a] <= b[a]) ? (pair[a] >> 16) : pair[a]);
      }
    }
  } else {
#pragma unroll
    for (int a = 0; a < N; ++a) {
      const float d = __fmul_rn(w[a], q.isb);
      int pos = 0;
#pragma unroll
      for (int step = 1 << (BITS - 1); step >= 1; step >>= 1) {
        pos += !(d <= q.bnd[pos + step - 1]) ? step : 0;
      }
      w[a] = __uint_as_float(static_cast<uint32_t>(q.outtab[pos]));
    }
  }
}

// Pass B of one chunk (and, for blocks up to 1024, the quantisation): lane b owns column b of
// the 32 x 32 arrangement held in the warp's scratch.
template <int BITS, bool CELLS, int STAGES, bool FINAL, bool OUT8 = false>
__device__ __forceinline__ void pw_pass_b(uint32_t scratch, uint32_t result, int lane, int active_rows,
                                          const PwQuant &q) {
  float w[32];
  const uint32_t column = scratch + ((lane & 3) << 2);
  const uint32_t group = static_cast<uint32_t>(lane >> 2);
#pragma unroll
  for (int a = 0; a < 32; ++a) {
    w[a] = pw_lds_f32(column + a * 128 + ((group ^ (a & 7)) << 4));
  }
  pw_butterflies<32, STAGES>(w);
  if (FINAL) {
    pw_quantize_all<BITS, CELLS, 32>(w, q);
    if (lane == 0) {
      pw_bulk_store_wait_read();   // the previous chunk's results have left the staging area
    }
    __syncwarp();
    // results in position order: 16-bit values, or (OUT8) bytes
    const uint32_t dst = result + lane * (OUT8 ? 1 : 2);
    if (active_rows == 32) {
#pragma unroll
      for (int a = 0; a < 32; ++a) {
        if (OUT8) {
          pw_sts_u8(dst + a * 32, __float_as_uint(w[a]));
        } else {
          pw_sts_u16(dst + a * 64, __float_as_uint(w[a]));
        }
      }
    } else {
#pragma unroll
      for (int a = 0; a < 32; ++a) {
        if (a < active_rows) {
          if (OUT8) {
            pw_sts_u8(dst + a * 32, __float_as_uint(w[a]));
          } else {
            pw_sts_u16(dst + a * 64, __float_as_uint(w[a]));
          }
        }
      }
    }
  } else {
    __syncwarp();   // every lane has read its column before the scratch is rewritten
    const uint32_t dst = scratch + lane * 4;
#pragma unroll
    for (int a = 0; a < 32; ++a) {
      pw_sts_f32(dst + a * 128, w[a]);
    }
  }
}

// Pass C of a team block: widths 1024 (and 2048) across the team's TEAM chunks, then the
// quantisation.  Thread tt of the team owns positions tt, tt + threads, ...
template <int BITS, bool CELLS, int TEAM, bool OUT8 = false>
__device__ __forceinline__ void pw_pass_c(uint32_t scratch, uint32_t result, int tt, const PwQuant &q) {
  constexpr int kThreads = TEAM * 32;
  constexpr int kPer = kPwChunk / kThreads;   // positions per thread: 16 (two chunks) or 8 (four)
  constexpr int kBatch = 8 / TEAM;            // positions handled together: TEAM * kBatch = 8 values
  constexpr int kStages = TEAM == 2 ? 1 : 2;
#pragma unroll 1
  for (int i0 = 0; i0 < kPer; i0 += kBatch) {
    float c[kBatch][TEAM];
#pragma unroll
    for (int i = 0; i < kBatch; ++i) {
#pragma unroll
      for (int t = 0; t < TEAM; ++t) {
        c[i][t] = pw_lds_f32(scratch + (t * kPwChunk + tt + kThreads * (i0 + i)) * 4);
      }
    }
#pragma unroll
    for (int i = 0; i < kBatch; ++i) {
      pw_butterflies<TEAM, kStages>(c[i]);
      pw_quantize_all<BITS, CELLS, TEAM>(c[i], q);
    }
#pragma unroll
    for (int i = 0; i < kBatch; ++i) {
#pragma unroll
      for (int t = 0; t < TEAM; ++t) {
        if (OUT8) {
          pw_sts_u8(result + (t * kPwChunk + tt + kThreads * (i0 + i)), __float_as_uint(c[i][t]));
        } else {
          pw_sts_u16(result + (t * kPwChunk + tt + kThreads * (i0 + i)) * 2, __float_as_uint(c[i][t]));
        }
      }
    }
  }
}

// F16OP: output = the f16 operand of the tensor-core GEMM (+ per-token factor).  OUT8: output =
// one byte per element, the INT8 code `code_map[level]` (+ per-token factor norm * out_scale),
// the operand of the INT8 tensor-core GEMM.  Neither: x_q in bf16.
template <int BITS, bool F16OP, int TW = kPwWarps, bool OUT8 = false>
__global__ void __launch_bounds__(pw_threads(TW), (TW == kPwWarps ? 2 : 1))
rotate_quantize_warp_kernel(const WarpPrologueParams p) {
  static_assert(!(F16OP && OUT8), "one output format");
  constexpr int kPwThreads = pw_threads(TW);

  extern __shared__ unsigned char pw_smem_raw[];
  constexpr int kLevels = 1 << BITS;
  constexpr int kMaxCells = pw_max_cells(BITS);
  const uint32_t raw_addr = pw_smem_u32(pw_smem_raw);
  unsigned char *smem = pw_smem_raw + (((raw_addr + 127u) & ~127u) - raw_addr);
  const uint32_t smem_addr = pw_smem_u32(smem);
  const int dim = p.dim;
  const int block = 1 << p.log2_block;
  const int R = p.batch_rows;
  const int S = p.slots;
  const PwLayout lay = pw_layout(dim, block, R, S, BITS, TW);

  // bytes 0..63: full[4] normed[4] barriers; 64..79: done counters; 80..: flags
  int *s_done = reinterpret_cast<int *>(smem + 64);
  volatile int *s_fallback = reinterpret_cast<volatile int *>(smem + 80);
  volatile int *s_abort = reinterpret_cast<volatile int *>(smem + 84);
  volatile int *s_cells = reinterpret_cast<volatile int *>(smem + 88);
  float *s_cent = reinterpret_cast<float *>(smem + lay.cent);
  float *s_bnd = reinterpret_cast<float *>(smem + lay.bnd);
  float *s_cell_bnd = reinterpret_cast<float *>(smem + lay.cell_bnd);
  uint16_t *s_cell_meta = reinterpret_cast<uint16_t *>(smem + lay.cell_meta);
  float *s_slot_meta = reinterpret_cast<float *>(smem + lay.slot_meta);   // [S][4]{norm, inv, opscale, -}
  uint16_t *s_outtab = reinterpret_cast<uint16_t *>(smem + lay.outtab);   // [S][R][levels]
  uint32_t *s_pairs = reinterpret_cast<uint32_t *>(smem + lay.pairs);     // [S][R][max cells]
  uint32_t *s_perm = reinterpret_cast<uint32_t *>(smem + lay.perm);
  float *s_dmin = reinterpret_cast<float *>(smem + lay.work);             // set-up only

  auto full_bar = [&](int s) { return smem_addr + 8u * s; };
  auto normed_bar = [&](int s) { return smem_addr + 32u + 8u * s; };

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // The last CTA of the grid does nothing but the table-scale search and the counter
  // clearing for the kernel that follows (both off every token's critical path).
  const int workers = static_cast<int>(gridDim.x) - (p.table_scale_out != nullptr ? 1 : 0);
  if (static_cast<int>(blockIdx.x) == workers) {
    // its outputs live in the workspace, which the kernel before this one may still read
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (threadIdx.x < 256) {
      for (int i = threadIdx.x; i < p.zero_count; i += 256) {
        p.zero_words[i] = 0;
      }
      search_table_scale(p.w_centroids, p.w_bits, p.table_scale_out, reinterpret_cast<float *>(smem + 128));
    }
    return;
  }

  const int64_t n_batches = (p.rows + R - 1) / R;
  // CTA-local batch b is global batch blockIdx.x + b * workers
  const int my_batches = static_cast<int>((n_batches - blockIdx.x + workers - 1) / workers);
  auto issue_load = [&](int local_batch) {   // one thread
    const int slot = local_batch % S;
    const int64_t row0 = (static_cast<int64_t>(blockIdx.x) + static_cast<int64_t>(local_batch) * workers) * R;
    const int nrows = static_cast<int>(min(static_cast<int64_t>(R), p.rows - row0));
    pw_mbar_expect_tx(full_bar(slot), static_cast<uint32_t>(nrows) * dim * 2);
    for (int rr = 0; rr < nrows; ++rr) {
      pw_bulk_load(smem_addr + lay.slots + slot * lay.slot_bytes + rr * lay.row_pitch,
                   p.x + (row0 + rr) * dim, static_cast<uint32_t>(dim) * 2, full_bar(slot));
    }
  };

  // ---- set-up: barriers and the first copies, codebook, permutation table, cell table ----
  if (threadIdx.x == 0) {
    for (int s = 0; s < kPwMaxSlots; ++s) {
      pw_mbar_init(full_bar(s), 1);
      pw_mbar_init(normed_bar(s), 1);
      s_done[s] = 0;
    }
    *s_fallback = 0;
    *s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int i = threadIdx.x; i < kLevels; i += kPwThreads) {
    s_cent[i] = p.centroids[i];
    s_bnd[i] = i < kLevels - 1 ? p.boundaries[i] : 0.0f;
  }
  // entry of rotated position i: byte offset of its source element in the row | sign << 31.
  // Stored so that lane l's 16-byte read of group g of a chunk is conflict-free:
  // [chunk][g = (i % 32) / 4][lane = (i % 1024) / 32][i % 4].
  // Four positions per 16-byte read, four reads in flight per thread before any is used (the
  // table build is pure global-memory latency otherwise).
  {
    const int groups = dim >> 2;
    const int4 *perm4 = reinterpret_cast<const int4 *>(p.perm);
    const uint32_t *signs4 = reinterpret_cast<const uint32_t *>(p.signs);
    for (int g0 = threadIdx.x; g0 < groups; g0 += 4 * kPwThreads) {
      int4 pv[4];
      uint32_t sv[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int g = g0 + u * kPwThreads;
        if (g < groups) {
          pv[u] = __ldg(perm4 + g);
          sv[u] = __ldg(signs4 + g);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int g = g0 + u * kPwThreads;
        if (g < groups) {
          const int i = g << 2;   // positions i .. i + 3 share a lane and a 16-byte group
          const int within = i & (kPwChunk - 1);
          const int slot_index = (i - within) + ((within & 31) >> 2) * 128 + (within >> 5) * 4;
          const int src[4] = {pv[u].x, pv[u].y, pv[u].z, pv[u].w};
          uint4 entry;
          uint32_t *e = reinterpret_cast<uint32_t *>(&entry);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            e[q] = (static_cast<uint32_t>(src[q]) << 1) | ((sv[u] << (24 - 8 * q)) & 0x80000000u);
          }
          *reinterpret_cast<uint4 *>(s_perm + slot_index) = entry;
        }
      }
    }
  }
  __syncthreads();

  const float lo = s_bnd[0];
  const float hi = s_bnd[kLevels - 2];
  int cells = kMaxCells / 2;
  bool use_cells = false;
  for (int attempt = 0; attempt < 2 && !use_cells; ++attempt, cells *= 2) {
    const PwCellMap map = pw_cell_map(lo, hi, cells);
    const uint32_t first_cell = pw_cell_bits(lo, map) - 0x4B000000u;
    const uint32_t last_cell = pw_cell_bits(hi, map) - 0x4B000000u;
    const bool range_ok = hi > lo && first_cell < static_cast<uint32_t>(cells) &&
                          last_cell < static_cast<uint32_t>(cells) && first_cell <= last_cell;
    if (range_ok) {
      // first value of every cell: the smallest float whose cell number is >= c
      for (int c = threadIdx.x; c <= cells; c += kPwThreads) {
        float dmin;
        if (c == cells || static_cast<uint32_t>(c) > last_cell) {
          dmin = __int_as_float(0x7f800000);           // never reached
        } else if (static_cast<uint32_t>(c) <= first_cell) {
          dmin = __int_as_float(0xff800000);           // everything below lo lands in lo's cell
        } else {
          uint32_t below = pw_float_key(lo);           // cell(below) < c
          uint32_t reach = pw_float_key(hi);           // cell(reach) >= c
          // start from the inverse of the map where a narrow bracket around it holds
          const float guess = __fmaf_rn(__fdiv_rn(static_cast<float>(c) - 1.5f, map.scale), 1.0f, lo);
          const uint32_t centre = pw_float_key(fmaxf(fminf(guess, hi), lo));
          const uint32_t near_lo = centre - below > 256u ? centre - 256u : below;
          const uint32_t near_hi = reach - centre > 256u ? centre + 256u : reach;
          if (pw_cell_bits(pw_key_float(near_lo), map) - 0x4B000000u < static_cast<uint32_t>(c)) {
            below = near_lo;
          }
          if (pw_cell_bits(pw_key_float(near_hi), map) - 0x4B000000u >= static_cast<uint32_t>(c)) {
            reach = near_hi;
          }
          while (reach - below > 1u) {
            const uint32_t mid = below + ((reach - below) >> 1);
            const uint32_t cell = pw_cell_bits(pw_key_float(mid), map) - 0x4B000000u;
            if (cell >= static_cast<uint32_t>(c)) {
              reach = mid;
            } else {
              below = mid;
            }
          }
          dmin = pw_key_float(reach);
        }
        s_dmin[c] = dmin;
      }
    }
    __syncthreads();
    if (range_ok) {
      for (int c = threadIdx.x; c < cells; c += kPwThreads) {
        const float d0 = s_dmin[c];
        const float d1 = s_dmin[c + 1];
        int base = 0;
        int upper = 0;
        for (int j = 0; j < kLevels - 1; ++j) {
          base += s_bnd[j] < d0 ? 1 : 0;
          upper += s_bnd[j] < d1 ? 1 : 0;
        }
        const int count = upper - base;
        if (count > 1) {
          *s_fallback = attempt + 1;
        }
        s_cell_bnd[c] = count >= 1 ? s_bnd[base] : __int_as_float(0x7f800000);
        s_cell_meta[c] = static_cast<uint16_t>(base | (count >= 1 ? 0x100 : 0));
      }
    }
    __syncthreads();
    use_cells = range_ok && *s_fallback != attempt + 1;
    if (use_cells && threadIdx.x == 0) {
      *s_cells = cells;
    }
    __syncthreads();
  }
  if (use_cells) {
    cells = *s_cells;
  }
  const PwCellMap map = pw_cell_map(lo, hi, use_cells ? cells : 8);
  const int units_per_row = block > kPwChunk ? dim / block : (dim + kPwChunk - 1) / kPwChunk;

  // Everything above read constants only (codebook, permutation, signs) and may have run while
  // the kernel before this one in the stream was still busy.  From here on the kernel reads x and
  // writes its outputs, which that kernel may have produced or may still be reading.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (threadIdx.x == 0) {
    for (int b = 0; b < S && b < my_batches; ++b) {
      issue_load(b);
    }
  }

  if (warp >= TW) {
    // ================= norm warps: alternate batches =================
    const int r = lane >> 3;
    const int t = lane & 7;
    for (int bi = warp - TW; bi < my_batches; bi += kPwNormWarps) {
      const int slot = bi % S;
      const uint32_t use = static_cast<uint32_t>(bi / S);
      const int64_t row0 = (static_cast<int64_t>(blockIdx.x) + static_cast<int64_t>(bi) * workers) * R;
      const int nrows = static_cast<int>(min(static_cast<int64_t>(R), p.rows - row0));
      if (!pw_mbar_wait(full_bar(slot), use & 1u, s_abort, 2)) {
        break;
      }
      // chains 2t and 2t+1 of token r: x[16 i + 2t], x[16 i + 2t + 1], i ascending
      float acc0 = 0.0f;
      float acc1 = 0.0f;
      if (r < nrows) {
        const uint32_t src = smem_addr + lay.slots + slot * lay.slot_bytes + r * lay.row_pitch + t * 4;
        const int iters = dim >> 4;
        int i = 0;
        for (; i + 8 <= iters; i += 8) {
          uint32_t w[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            w[u] = pw_lds_u32(src + (i + u) * 32);
          }
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const float a = __uint_as_float(w[u] << 16);
            const float b = __uint_as_float(w[u] & 0xffff0000u);
            acc0 = __fmaf_rn(a, a, acc0);
            acc1 = __fmaf_rn(b, b, acc1);
          }
        }
        for (; i < iters; ++i) {
          const uint32_t w = pw_lds_u32(src + i * 32);
          const float a = __uint_as_float(w << 16);
          const float b = __uint_as_float(w & 0xffff0000u);
          acc0 = __fmaf_rn(a, a, acc0);
          acc1 = __fmaf_rn(b, b, acc1);
        }
      }
      // the 16-lane fold 8, 4, 2, 1: chain j pairs with j^8, j^4, j^2 (lanes t^4, t^2, t^1), then
      // with j^1 (the thread's other chain)
#pragma unroll
      for (int m = 4; m >= 1; m >>= 1) {
        acc0 = __fadd_rn(acc0, __shfl_xor_sync(0xffffffffu, acc0, m));
        acc1 = __fadd_rn(acc1, __shfl_xor_sync(0xffffffffu, acc1, m));
      }
      const float total = __fadd_rn(acc0, acc1);
      float *meta = s_slot_meta + (slot * kPwMaxRows + r) * 4;
      if (r < nrows && t == 0) {
        const float norm = __fsqrt_rn(total);
        float mult = 1.0f;
        if (F16OP) {
          float back = 1.0f;
          if (norm > 0.0f && norm < __int_as_float(0x7f800000)) {
            const int e = max(ilogbf(norm) + 1, -100);
            mult = ldexpf(1.0f, 14 - e);
            back = ldexpf(1.0f, e - 14);
          }
          p.row_scale[row0 + r] = back;
        } else if (OUT8) {
          p.row_scale[row0 + r] = __fmul_rn(norm, p.out_scale);
        }
        meta[0] = norm;
        meta[1] = __fdiv_rn(1.0f, __fadd_rn(norm, p.eps));
        meta[2] = mult;
      }
      __syncwarp();
      // every token's 2^BITS possible outputs, then the candidate pair of every cell
      uint16_t *outtab = s_outtab + slot * R * kLevels;
      for (int i = lane; i < nrows * kLevels; i += 32) {
        const int rr = i >> BITS;
        const float *m = s_slot_meta + (slot * kPwMaxRows + rr) * 4;
        const float q = __fmul_rn(s_cent[i & (kLevels - 1)], m[0]);
        const __nv_bfloat16 qb = __float2bfloat16_rn(q);
        outtab[i] = OUT8 ? static_cast<uint16_t>(static_cast<uint8_t>(p.code_map[i & (kLevels - 1)]))
                         : (F16OP ? __half_as_ushort(__float2half_rn(__fmul_rn(__bfloat162float(qb), m[2])))
                                  : __bfloat16_as_ushort(qb));
      }
      __syncwarp();
      if (use_cells) {
        uint32_t *pairs = s_pairs + slot * R * kMaxCells;
        for (int i = lane; i < nrows * cells; i += 32) {
          const int rr = i / cells;
          const int c = i - rr * cells;
          const uint32_t meta16 = s_cell_meta[c];
          const int base = meta16 & 0xff;
          const int next = min(base + static_cast<int>(meta16 >> 8), kLevels - 1);
          pairs[rr * kMaxCells + c] = static_cast<uint32_t>(outtab[rr * kLevels + base]) |
                                      (static_cast<uint32_t>(outtab[rr * kLevels + next]) << 16);
        }
      }
      __syncwarp();
      if (lane == 0) {
        pw_mbar_arrive(normed_bar(slot));
      }
    }
    return;
  }

  // ================= transform warps =================
  const int team_size = block > kPwChunk ? block / kPwChunk : 1;
  const int n_teams = TW / team_size;
  const int team = warp / team_size;
  const int tw = warp - team * team_size;
  const int team_threads = team_size * 32;
  const int tt = tw * 32 + lane;
  const uint32_t scratch = smem_addr + lay.work + team * lay.team_bytes;        // [team][1024] fp32
  const uint32_t result = scratch + team_size * kPwChunk * 4;                    // [team][1024] 16-bit
  const uint32_t my_scratch = scratch + tw * kPwChunk * 4;
  const uint32_t my_rows = my_scratch + lane * 128;
  const uint32_t perm_base = smem_addr + lay.perm + lane * 16;

  PwQuant quant;
  quant.map = map;
  quant.cell_bnd = smem_addr + lay.cell_bnd - 0x2C000000u;
  quant.bnd = s_bnd;
  quant.isb = p.inv_sqrt_block;

  int64_t unit_base = 0;   // units of this CTA before the current batch
  for (int bi = 0; bi < my_batches; ++bi) {
    const int slot = bi % S;
    const uint32_t use = static_cast<uint32_t>(bi / S);
    const int64_t row0 = (static_cast<int64_t>(blockIdx.x) + static_cast<int64_t>(bi) * workers) * R;
    const int nrows = static_cast<int>(min(static_cast<int64_t>(R), p.rows - row0));
    const int units = nrows * units_per_row;
    if (!pw_mbar_wait(normed_bar(slot), use & 1u, s_abort, 3)) {
      break;
    }
    const uint32_t slot_addr = smem_addr + lay.slots + slot * lay.slot_bytes;
    const int first = static_cast<int>((team - unit_base % n_teams + n_teams) % n_teams);
    for (int j = first; j < units; j += n_teams) {
      const int r = j / units_per_row;
      const int u = j - r * units_per_row;
      const float inv = s_slot_meta[(slot * kPwMaxRows + r) * 4 + 1];
      quant.pairs = smem_addr + lay.pairs + ((slot * R + r) * kMaxCells) * 4 - 0x2C000000u;
      quant.outtab = s_outtab + (slot * R + r) * kLevels;
      const uint32_t row_addr = slot_addr + r * lay.row_pitch;
      // this warp's 1024-element chunk: positions chunk_first .. chunk_first + chunk_len
      const int chunk_index = team_size > 1 ? u * team_size + tw : u;
      const int chunk_first = chunk_index * kPwChunk;
      const int chunk_len = min(kPwChunk, dim - chunk_first);
      const int active_lanes = chunk_len >> 5;

      // ---- pass A: gather, widths 1 .. 16, transposing store ----
      {
        float v[32];
        if (lane < active_lanes) {
          const uint32_t entries = perm_base + chunk_first * 4;
          uint32_t e[32];
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            const uint4 e4 = pw_lds_v4(entries + g * 512);
            e[4 * g] = e4.x;
            e[4 * g + 1] = e4.y;
            e[4 * g + 2] = e4.z;
            e[4 * g + 3] = e4.w;
          }
          uint32_t raw[32];
#pragma unroll
          for (int q = 0; q < 32; ++q) {
            raw[q] = pw_lds_u16(row_addr + (e[q] & 0xffffu));
          }
#pragma unroll
          for (int q = 0; q < 32; ++q) {
            v[q] = __fmul_rn(__uint_as_float((raw[q] << 16) ^ (e[q] & 0x80000000u)), inv);
          }
        } else {
#pragma unroll
          for (int q = 0; q < 32; ++q) {
            v[q] = 0.0f;
          }
        }
        pw_butterflies<32, 5>(v);
        // 16-byte group g of lane l goes to slot g ^ (l & 7) of the lane's 128-byte row
        const uint32_t swz = static_cast<uint32_t>(lane & 7);
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          pw_sts_v4f(my_rows + ((g ^ swz) << 4), v[4 * g], v[4 * g + 1], v[4 * g + 2], v[4 * g + 3]);
        }
      }
      __syncwarp();
      if (team_size == 1) {
        // ---- pass B with the quantisation; widths up to the block ----
        if (use_cells) {
          switch (p.log2_block) {
            case 8: pw_pass_b<BITS, true, 3, true, OUT8>(my_scratch, result, lane, active_lanes, quant); break;
            case 9: pw_pass_b<BITS, true, 4, true, OUT8>(my_scratch, result, lane, active_lanes, quant); break;
            default: pw_pass_b<BITS, true, 5, true, OUT8>(my_scratch, result, lane, active_lanes, quant); break;
          }
        } else {
          switch (p.log2_block) {
            case 8: pw_pass_b<BITS, false, 3, true, OUT8>(my_scratch, result, lane, active_lanes, quant); break;
            case 9: pw_pass_b<BITS, false, 4, true, OUT8>(my_scratch, result, lane, active_lanes, quant); break;
            default: pw_pass_b<BITS, false, 5, true, OUT8>(my_scratch, result, lane, active_lanes, quant); break;
          }
        }
        pw_fence_async();
        __syncwarp();
        if (lane == 0) {
          if (OUT8) {
            pw_bulk_store(reinterpret_cast<uint8_t *>(p.xq) + (row0 + r) * dim + chunk_first, result,
                          static_cast<uint32_t>(chunk_len));
          } else {
            pw_bulk_store(p.xq + (row0 + r) * dim + chunk_first, result, static_cast<uint32_t>(chunk_len) * 2);
          }
        }
      } else {
        // ---- pass B (widths 32 .. 512) back into the scratch, then pass C across the team ----
        pw_pass_b<BITS, true, 5, false>(my_scratch, result, lane, 32, quant);
        if (tt == 0) {
          pw_bulk_store_wait_read();
        }
        pw_team_barrier(team, team_threads);
        if (use_cells) {
          if (team_size == 2) {
            pw_pass_c<BITS, true, 2, OUT8>(scratch, result, tt, quant);
          } else {
            pw_pass_c<BITS, true, 4, OUT8>(scratch, result, tt, quant);
          }
        } else if (team_size == 2) {
          pw_pass_c<BITS, false, 2, OUT8>(scratch, result, tt, quant);
        } else {
          pw_pass_c<BITS, false, 4, OUT8>(scratch, result, tt, quant);
        }
        pw_fence_async();
        pw_team_barrier(team, team_threads);   // results complete; scratch free for the next unit
        if (tt == 0) {
          if (OUT8) {
            pw_bulk_store(reinterpret_cast<uint8_t *>(p.xq) + (row0 + r) * dim + static_cast<int64_t>(u) * block,
                          result, static_cast<uint32_t>(block));
          } else {
            pw_bulk_store(p.xq + (row0 + r) * dim + static_cast<int64_t>(u) * block, result,
                          static_cast<uint32_t>(block) * 2);
          }
        }
      }
    }
    unit_base += units;
    // The warp that finishes the batch last refills the slot with the batch S further on.
    __syncwarp();
    if (lane == 0) {
      __threadfence_block();
      if (atomicAdd(&s_done[slot], 1) == TW - 1) {
        atomicExch(&s_done[slot], 0);
        if (bi + S < my_batches) {
          pw_fence_async();
          issue_load(bi + S);
        }
      }
    }
  }
  if (lane == 0) {
    pw_bulk_store_wait_read();   // staging memory must outlive the last store's read
  }
}

inline bool warp_prologue_supported(int x_dtype, int64_t dim, int64_t block, int bits) {
  return x_dtype == OQ_DTYPE_BF16 && dim % 256 == 0 && dim <= 32768 && block >= 256 && block <= 4096 &&
         (bits == 2 || bits == 3 || bits == 4 || bits == 6 || bits == 8);
}

}  // namespace
}  // namespace oq
