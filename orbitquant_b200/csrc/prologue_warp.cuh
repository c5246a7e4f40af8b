// Rotate-and-quantize for large token counts: one warp transforms one rotation block.
//
// Same arithmetic, operation order and therefore the same bits as the kernels in prologue.cu
// (bf16 rows, dim a multiple of 256, block 256 .. 4096, x_q output only).  What differs is
// the organisation, chosen so that no CTA-wide barrier and no serial phase sits on the
// critical path:
//
//   norm warp (warp 8)      works one batch of R tokens AHEAD of the others: bulk-copies the
//                           batch into a shared-memory slot (cp.async.bulk, completion on an
//                           mbarrier), computes the token norms in the reference's AVX-512
//                           order (16 fused-multiply-add chains per token, two per lane, eight
//                           lanes per token, then the 8/4/2/1 fold) and tabulates every
//                           token's possible outputs; then signals `normed[slot]`.
//   transform warps (0..7)  each takes whole 1024-element chunks of a token (one or several
//                           rotation blocks): lane l gathers the 32 values of positions
//                           32l .. 32l+31 through a permutation table kept in shared memory
//                           (index and sign in one word), runs butterfly widths 1 .. 16 in
//                           registers, transposes through a swizzled 4 KB scratch (one 16-byte
//                           store per 4 values, conflict-free reads), runs widths 32 .. 512,
//                           quantises, and the 2 KB of results leave by one bulk store.  For
//                           blocks of 2048 / 4096 a team of 2 / 4 warps shares a block and a
//                           third pass (widths 1024, 2048) follows a team barrier.
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

constexpr int kPwWarps = 8;                       // transform warps
constexpr int kPwThreads = (kPwWarps + 1) * 32;   // + the norm warp
constexpr int kPwNormWarp = kPwWarps;
constexpr int kPwChunk = 1024;
constexpr int kPwRowPad = 32;                     // bytes between the rows of a slot
constexpr int kPwMaxRows = 4;                     // tokens per batch
constexpr uint32_t kPwSpinLimit = 1u << 22;

__host__ __device__ constexpr int pw_max_cells(int bits) {
  return bits >= 8 ? 1024 : (4 << bits);
}

struct WarpPrologueParams {
  const uint16_t *x;
  uint16_t *xq;
  float *row_scale;  // f16 operand mode: per-token factor 2^(E-14)
  const int32_t *perm;
  const int8_t *signs;
  const float *boundaries;
  const float *centroids;
  int64_t rows;
  int dim;
  int log2_block;
  int batch_rows;
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

__host__ __device__ inline PwLayout pw_layout(int dim, int block, int batch_rows, int bits) {
  PwLayout l;
  const int cells = pw_max_cells(bits);
  int at = 128;  // barriers and flags
  l.cent = at;       at += 256 * 4;
  l.bnd = at;        at += 256 * 4;
  l.cell_bnd = at;   at += cells * 4;
  l.cell_meta = at;  at += (cells * 2 + 127) / 128 * 128;
  l.slot_meta = at;  at += 2 * kPwMaxRows * 16;                       // norm, inv, opscale, -
  l.outtab = at;     at += (2 * batch_rows * (2 << bits) + 127) / 128 * 128;
  l.pairs = at;      at += 2 * batch_rows * cells * 4;
  at = (at + 127) / 128 * 128;
  l.perm = at;       at += (dim + kPwChunk - 1) / kPwChunk * kPwChunk * 4;   // whole chunks
  l.row_pitch = dim * 2 + kPwRowPad;
  l.slot_bytes = batch_rows * l.row_pitch;
  l.slots = at;      at += 2 * l.slot_bytes;
  at = (at + 127) / 128 * 128;
  const int team = block > kPwChunk ? block / kPwChunk : 1;
  l.team_bytes = team * kPwChunk * 6;                                  // fp32 scratch + 16-bit results
  l.work = at;       at += (kPwWarps / team) * l.team_bytes;
  l.total = at + 128;                                                  // alignment slack
  return l;
}

__device__ __forceinline__ uint32_t pw_smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
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

template <int S>
__device__ __forceinline__ void pw_butterflies(float (&v)[S], int limit) {
#pragma unroll
  for (int h = 1; h < S; h <<= 1) {
    if (h < limit) {
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
}

// State a transform thread needs to quantise values of one token.
struct PwQuant {
  PwCellMap map;
  const unsigned char *cell_bnd;   // float per cell
  const unsigned char *pairs;      // this token's candidate pair per cell
  const float *bnd;                // boundaries (fallback search)
  const uint16_t *outtab;          // this token's 2^bits outputs (fallback search)
  float isb;
  bool use_cells;
};

template <int BITS>
__device__ __forceinline__ uint16_t pw_quantize(float value, const PwQuant &q) {
  const float d = __fmul_rn(value, q.isb);
  if (q.use_cells) {
    const uint32_t off = (pw_cell_bits(d, q.map) << 2) - 0x2C000000u;  // 4 * (bits - 0x4B000000)
    const float b = *reinterpret_cast<const float *>(q.cell_bnd + off);
    const uint32_t pair = *reinterpret_cast<const uint32_t *>(q.pairs + off);
    return static_cast<uint16_t>(!(d <= b) ? (pair >> 16) : pair);
  }
  int pos = 0;
#pragma unroll
  for (int step = 1 << (BITS - 1); step >= 1; step >>= 1) {
    pos += !(d <= q.bnd[pos + step - 1]) ? step : 0;
  }
  return q.outtab[pos];
}

template <int BITS, bool F16OP>
__global__ void __launch_bounds__(kPwThreads, 2)
rotate_quantize_warp_kernel(const WarpPrologueParams p) {
  extern __shared__ unsigned char pw_smem_raw[];
  constexpr int kLevels = 1 << BITS;
  constexpr int kMaxCells = pw_max_cells(BITS);
  const uint32_t raw_addr = pw_smem_u32(pw_smem_raw);
  unsigned char *smem = pw_smem_raw + (((raw_addr + 127u) & ~127u) - raw_addr);
  const int dim = p.dim;
  const int block = 1 << p.log2_block;
  const int R = p.batch_rows;
  const PwLayout lay = pw_layout(dim, block, R, BITS);

  uint64_t *bars = reinterpret_cast<uint64_t *>(smem);
  volatile int *s_fallback = reinterpret_cast<volatile int *>(smem + 64);
  volatile int *s_abort = reinterpret_cast<volatile int *>(smem + 68);
  volatile int *s_cells = reinterpret_cast<volatile int *>(smem + 72);
  float *s_cent = reinterpret_cast<float *>(smem + lay.cent);
  float *s_bnd = reinterpret_cast<float *>(smem + lay.bnd);
  float *s_cell_bnd = reinterpret_cast<float *>(smem + lay.cell_bnd);
  uint16_t *s_cell_meta = reinterpret_cast<uint16_t *>(smem + lay.cell_meta);
  float *s_slot_meta = reinterpret_cast<float *>(smem + lay.slot_meta);   // [2][R]{norm, inv, opscale, -}
  uint16_t *s_outtab = reinterpret_cast<uint16_t *>(smem + lay.outtab);   // [2][R][levels]
  uint32_t *s_pairs = reinterpret_cast<uint32_t *>(smem + lay.pairs);     // [2][R][max cells]
  uint32_t *s_perm = reinterpret_cast<uint32_t *>(smem + lay.perm);
  unsigned char *s_slots = smem + lay.slots;
  unsigned char *s_work = smem + lay.work;
  float *s_dmin = reinterpret_cast<float *>(s_work);                       // set-up only

  const uint32_t bar_base = pw_smem_u32(bars);
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto normed_bar = [&](int s) { return bar_base + 16u + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 32u + 8u * s; };

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // The last CTA of the grid does nothing but the table-scale search and the counter
  // clearing for the kernel that follows (both off every token's critical path).
  const int workers = static_cast<int>(gridDim.x) - (p.table_scale_out != nullptr ? 1 : 0);
  if (static_cast<int>(blockIdx.x) == workers) {
    if (threadIdx.x < 256) {
      for (int i = threadIdx.x; i < p.zero_count; i += 256) {
        p.zero_words[i] = 0;
      }
      search_table_scale(p.w_centroids, p.w_bits, p.table_scale_out, reinterpret_cast<float *>(smem + 128));
    }
    return;
  }

  // ---- set-up: barriers, codebook, permutation table, cell table ----
  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      pw_mbar_init(full_bar(s), 1);
      pw_mbar_init(normed_bar(s), 1);
      pw_mbar_init(empty_bar(s), kPwWarps);
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
  for (int i = threadIdx.x; i < dim; i += kPwThreads) {
    const uint32_t entry = (static_cast<uint32_t>(p.perm[i]) << 1) | (p.signs[i] < 0 ? 0x80000000u : 0u);
    const int within = i & (kPwChunk - 1);
    const int slot_index = (i - within) + ((within & 31) >> 2) * 128 + (within >> 5) * 4 + (within & 3);
    s_perm[slot_index] = entry;
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
  const int64_t n_batches = (p.rows + R - 1) / R;

  if (warp == kPwNormWarp) {
    // ================= norm warp =================
    const int r = lane >> 3;
    const int t = lane & 7;
    int bi = 0;
    for (int64_t batch = blockIdx.x; batch < n_batches; batch += workers, ++bi) {
      const int slot = bi & 1;
      const uint32_t use = static_cast<uint32_t>(bi >> 1);
      const int64_t row0 = batch * R;
      const int nrows = static_cast<int>(min(static_cast<int64_t>(R), p.rows - row0));
      if (!pw_mbar_wait(empty_bar(slot), (use & 1u) ^ 1u, s_abort, 1)) {
        break;
      }
      unsigned char *slot_ptr = s_slots + slot * lay.slot_bytes;
      if (lane == 0) {
        pw_mbar_expect_tx(full_bar(slot), static_cast<uint32_t>(nrows) * dim * 2);
        for (int rr = 0; rr < nrows; ++rr) {
          pw_bulk_load(pw_smem_u32(slot_ptr + rr * lay.row_pitch), p.x + (row0 + rr) * dim,
                       static_cast<uint32_t>(dim) * 2, full_bar(slot));
        }
      }
      if (!pw_mbar_wait(full_bar(slot), use & 1u, s_abort, 2)) {
        break;
      }
      // chains 2t and 2t+1 of token r: x[16 i + 2t], x[16 i + 2t + 1], i ascending
      float acc0 = 0.0f;
      float acc1 = 0.0f;
      if (r < nrows) {
        const uint32_t *src = reinterpret_cast<const uint32_t *>(slot_ptr + r * lay.row_pitch) + t;
        const int iters = dim >> 4;
        int i = 0;
        for (; i + 8 <= iters; i += 8) {
          uint32_t w[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            w[u] = src[(i + u) * 8];
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
          const uint32_t w = src[i * 8];
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
        outtab[i] = F16OP ? __half_as_ushort(__float2half_rn(__fmul_rn(__bfloat162float(qb), m[2])))
                          : __bfloat16_as_ushort(qb);
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
  const int n_teams = kPwWarps / team_size;
  const int team = warp / team_size;
  const int tw = warp - team * team_size;
  const int team_threads = team_size * 32;
  const int tt = tw * 32 + lane;
  float *scratch = reinterpret_cast<float *>(s_work + team * lay.team_bytes);          // [team][1024] fp32
  uint16_t *result = reinterpret_cast<uint16_t *>(scratch + team_size * kPwChunk);     // [team][1024]
  float *my_scratch = scratch + tw * kPwChunk;
  const int passb_limit = block >= kPwChunk ? 32 : (block >> 5);  // butterfly widths of pass B, in rows of 32

  PwQuant quant;
  quant.map = map;
  quant.cell_bnd = reinterpret_cast<const unsigned char *>(s_cell_bnd);
  quant.bnd = s_bnd;
  quant.isb = p.inv_sqrt_block;
  quant.use_cells = use_cells;

  int bi = 0;
  int64_t unit_base = 0;   // units of this CTA before the current batch
  bool ok = true;
  for (int64_t batch = blockIdx.x; batch < n_batches && ok; batch += workers, ++bi) {
    const int slot = bi & 1;
    const uint32_t use = static_cast<uint32_t>(bi >> 1);
    const int64_t row0 = batch * R;
    const int nrows = static_cast<int>(min(static_cast<int64_t>(R), p.rows - row0));
    const int units = nrows * units_per_row;
    if (!pw_mbar_wait(normed_bar(slot), use & 1u, s_abort, 3)) {
      ok = false;
      break;
    }
    const unsigned char *slot_ptr = s_slots + slot * lay.slot_bytes;
    int first = static_cast<int>((team - unit_base % n_teams + n_teams) % n_teams);
    for (int j = first; j < units; j += n_teams) {
      const int r = j / units_per_row;
      const int u = j - r * units_per_row;
      const float inv = s_slot_meta[(slot * kPwMaxRows + r) * 4 + 1];
      quant.pairs = reinterpret_cast<const unsigned char *>(s_pairs + (slot * R + r) * kMaxCells);
      quant.outtab = s_outtab + (slot * R + r) * kLevels;
      const unsigned char *row_ptr = slot_ptr + r * lay.row_pitch;
      // this warp's 1024-element chunk: positions chunk_first .. chunk_first + chunk_len
      const int chunk_index = team_size > 1 ? u * team_size + tw : u;
      const int chunk_first = chunk_index * kPwChunk;
      const int chunk_len = min(kPwChunk, dim - chunk_first);
      const int active_lanes = chunk_len >> 5;

      // ---- pass A: gather, widths 1 .. 16 ----
      float v[32];
      if (lane < active_lanes) {
        const uint4 *entries = reinterpret_cast<const uint4 *>(s_perm + chunk_first) + lane;
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const uint4 e4 = entries[g * 32];
          const uint32_t e[4] = {e4.x, e4.y, e4.z, e4.w};
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const uint32_t raw = *reinterpret_cast<const uint16_t *>(row_ptr + (e[q] & 0xffffu));
            v[4 * g + q] = __fmul_rn(__uint_as_float((raw << 16) ^ (e[q] & 0x80000000u)), inv);
          }
        }
      } else {
#pragma unroll
        for (int q = 0; q < 32; ++q) {
          v[q] = 0.0f;
        }
      }
      pw_butterflies<32>(v, 32);
      // transpose through the scratch: 16-byte group g of lane l goes to slot g ^ (l & 7)
      {
        float4 *dst = reinterpret_cast<float4 *>(my_scratch + lane * 32);
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          dst[g ^ (lane & 7)] = make_float4(v[4 * g], v[4 * g + 1], v[4 * g + 2], v[4 * g + 3]);
        }
      }
      __syncwarp();
      // ---- pass B: lane b owns column b of the 32 x 32 arrangement, widths 32 .. 512 ----
      float w[32];
#pragma unroll
      for (int a = 0; a < 32; ++a) {
        w[a] = my_scratch[a * 32 + ((((lane >> 2) ^ (a & 7)) << 2) | (lane & 3))];
      }
      pw_butterflies<32>(w, passb_limit);
      if (team_size == 1) {
        if (lane == 0) {
          pw_bulk_store_wait_read();   // the previous chunk's results have left the staging area
        }
        __syncwarp();
#pragma unroll
        for (int a = 0; a < 32; ++a) {
          if (a < active_lanes) {
            result[a * 32 + lane] = pw_quantize<BITS>(w[a], quant);
          }
        }
        pw_fence_async();
        __syncwarp();
        if (lane == 0) {
          pw_bulk_store(p.xq + (row0 + r) * dim + chunk_first, pw_smem_u32(result),
                        static_cast<uint32_t>(chunk_len) * 2);
        }
      } else {
        // ---- pass C: widths 1024 (and 2048) across the team's chunks ----
        __syncwarp();   // every lane has read its column before the scratch is rewritten
#pragma unroll
        for (int a = 0; a < 32; ++a) {
          my_scratch[a * 32 + lane] = w[a];
        }
        if (tt == 0) {
          pw_bulk_store_wait_read();
        }
        pw_team_barrier(team, team_threads);
        const int per_thread = kPwChunk / team_threads;   // 16 (two chunks) or 8 (four)
        if (team_size == 2) {
#pragma unroll 4
          for (int i = 0; i < per_thread; ++i) {
            const int pos = tt + team_threads * i;
            float c[2] = {scratch[pos], scratch[kPwChunk + pos]};
            pw_butterflies<2>(c, 2);
            result[pos] = pw_quantize<BITS>(c[0], quant);
            result[kPwChunk + pos] = pw_quantize<BITS>(c[1], quant);
          }
        } else {
#pragma unroll 4
          for (int i = 0; i < per_thread; ++i) {
            const int pos = tt + team_threads * i;
            float c[4] = {scratch[pos], scratch[kPwChunk + pos], scratch[2 * kPwChunk + pos],
                          scratch[3 * kPwChunk + pos]};
            pw_butterflies<4>(c, 4);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              result[q * kPwChunk + pos] = pw_quantize<BITS>(c[q], quant);
            }
          }
        }
        pw_fence_async();
        pw_team_barrier(team, team_threads);   // results complete; scratch free for the next unit
        if (tt == 0) {
          pw_bulk_store(p.xq + (row0 + r) * dim + static_cast<int64_t>(u) * block, pw_smem_u32(result),
                        static_cast<uint32_t>(block) * 2);
        }
      }
    }
    unit_base += units;
    __syncwarp();
    if (lane == 0) {
      pw_mbar_arrive(empty_bar(slot));
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
