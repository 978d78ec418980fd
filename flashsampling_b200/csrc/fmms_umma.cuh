// Tensor-core kernel: tcgen05.mma with TMEM accumulators, fed by TMA.
//
// Orientation: the batch sits on the MMA M axis (128 TMEM lanes = 128 hidden-state
// rows, zero-extended) and the vocabulary on the N axis (up to 256 TMEM columns per
// tile).  D[128, NT] = Hs[128, 64] * Wt[NT, 64]^T per 64-wide slice of the hidden
// dimension, both operands K-major in shared memory with the 128-byte swizzle that
// TMA writes and the MMA descriptor names.  An epilogue thread therefore owns ONE
// batch row and walks vocabulary columns in order: the Gumbel-max scan is a running
// (max, index) in two registers, with no cross-lane traffic until the kernel ends.
//
// Warp roles (640 threads, one CTA per SM, persistent over a contiguous range of
// vocabulary tiles):
//   warp 0, 2   TMA producers: W tile / hidden-state tile(s) of each pipeline stage
//   warp 1      TMEM allocation, then one elected thread issues tcgen05.mma/commit
//   warp 3      idle
//   warps 4-19  epilogue (four warpgroups that split a tile's columns): tcgen05.ld ->
//               scale, noise, running argmax.  TMEM accumulators are multi-buffered
//               so the epilogue of tile i overlaps the mainloop of tile i+1.
// Batches above 128 use two M tiles that share every W tile (MT = 2).
//
// Row replicas (batches of at most 64 rows).  An epilogue warp can only read its own quadrant of
// 32 TMEM lanes, so with 64 (32) batch rows half (three quarters) of the epilogue warps - and of
// the SM's four schedulers - would have no rows.  Instead of one MMA over the whole tile the issuer
// then runs R = 2 (4) MMAs per K step, each over 1/R of the tile's columns, and shifts the A
// operand of replica k back by k * 128/R rows: rows k*128/R .. of that operand are the hidden
// states (the rows before them are whatever precedes the hidden-state tile in the stage, i.e. W
// bytes; their accumulator lanes are never read).  Replica k's columns therefore hold the batch
// rows in lanes k*128/R .., and every quadrant scans 1/R of the columns of the same rows.  No
// extra shared memory, no extra TMA traffic, the same tensor-core work.
#pragma once

#include <cuda.h>

#include "fmms_common.cuh"
#include "fmms_gemv.cuh"  // SampleParams

namespace fmms {

constexpr int kUmmaThreads = 640;
constexpr int kUmmaEpiWarp0 = 4;       // first epilogue warp
constexpr int kUmmaEpiWarps = 16;      // four warpgroups: four warps per scheduler keep the epilogue's
                                       // long dependency chains (Philox, logarithms) overlapped
constexpr int kUmmaEpiGroups = kUmmaEpiWarps / 4;
constexpr int kUmmaBK = 64;            // hidden-dimension slice per stage (128 B of bf16)
constexpr int kUmmaHTileMax = 128 * 128;  // the MMA always reads 128 hidden-state rows (16 KiB)
constexpr int kUmmaMaxStages = 12;
constexpr int kTmemCols = 512;

struct UmmaPlan {
  int grid;           // persistent CTAs
  int units_total;    // ceil(V / 16): the vocabulary in units of 16 rows (the MMA N granule)
  int tiles_per_cta;  // T: every CTA cuts its contiguous range of units into T tiles
  int q_units;        // tiles are q_units or q_units - 1 units high
  int nt_cap;         // TMEM columns reserved per accumulator (256 or 128)
  int stages;         // shared-memory ring depth
  int h_rows;         // rows of the hidden-state TMA box (MT = 1: ceil8(B); MT = 2: 128)
  int mt;             // M tiles (1 or 2)
  int slabs;          // 64-column K slabs per pipeline stage (one TMA operation fetches them all)
  int copies;         // row replicas R (1, 2 or 4): MMAs per K step, each over 1/R of the tile's columns
  int m_rows;         // rows of the MMA's M axis: 128, or 64 for some batches of at most 64 rows (see umma_plan)
  size_t smem;
};

// Shared memory: [barriers 1 KiB][stages x (W tile: tallest tile x 128 B | MT hidden-state tiles:
// h_rows x 128 B)][8 or 16 KiB slack].  With fewer hidden-state rows than the MMA's M (64 or 128) the
// A operand runs past its tile into whatever follows (the next stage, or the slack after the last
// one); those accumulator lanes belong to no batch row and are never read.
__host__ __device__ inline size_t umma_stage_bytes(int mt, int q_units, int h_rows, int slabs) {
  return (size_t)slabs * ((size_t)q_units * 16 * 128 + (size_t)mt * h_rows * 128);
}

// Work split.  The vocabulary is dealt out in units of 16 rows: CTA c gets a contiguous range
// of U_c = units_total / grid (+1 for the first units_total % grid CTAs) units and cuts it into
// T near-equal tiles, so no CTA walks more than 16 rows beyond the average.  All tiles of all
// CTAs are then q or q - 1 units high, which two TMA descriptors (two box heights) cover.
__host__ inline UmmaPlan umma_plan(int V, int B, int num_sms, int max_smem, int stages_cap = 0,
                                   int mt2_nt_cap = 256, int nt_target = 0, int min_tiles = 1, int D = 0, int slabs_force = 0,
                                   int copies_cap = 0, int m_force = -1) {
  UmmaPlan pl{};
  pl.mt = B > 128 ? 2 : 1;
  // Two M tiles share each W tile.  Wide tiles (one 2 x 256-column accumulator, epilogue not
  // overlapped) re-read the hidden states least; mt2_nt_cap = 128 selects two double-buffered
  // 128-column accumulators instead.
  pl.nt_cap = pl.mt == 1 ? 256 : mt2_nt_cap;
  pl.units_total = (V + 15) / 16;
  pl.grid = pl.units_total < num_sms ? pl.units_total : num_sms;
  int u_max = (pl.units_total + pl.grid - 1) / pl.grid;
  pl.h_rows = pl.mt == 2 ? 128 : ((B + 7) / 8 * 8);
  if (pl.h_rows < 16) pl.h_rows = 16;  // an 8-row hidden-state box measured 2-4 us slower than a 16-row one (half of it zero fill)
  // M = 64 MMAs (at most 64 batch rows, no row replicas; m_force = 0 keeps M = 128) read half the A operand and
  // leave 16 rows in the lower half of every TMEM lane quadrant; the epilogue splits every chunk of columns
  // between the two half-warps, so twice as many lanes scan as with the same rows in an M = 128 accumulator.
  // Measured against M = 128 in the same run (Qwen head): B = 16 197.6 -> 194.1 us, B = 32 199.7 -> 196.6,
  // B = 64 217 -> 197.6, four draws per row at B = 64 253 -> 232.
  pl.m_rows = (pl.mt == 1 && copies_cap < 2 && pl.h_rows <= 64 && m_force != 0) ? 64 : 128;
  // Behind the last stage: room for the rows the MMA's A operand reads beyond its hidden-state tile
  // ((m_rows - h_rows) x 128 B; with row replicas up to 16 KiB), which the epilogue reuses for the rows' pivots
  // (top-k) and the CTA's winners (at most 8 KiB).
  const size_t slack = (copies_cap >= 2 || (pl.mt == 1 && pl.m_rows - pl.h_rows > 56)) ? kUmmaHTileMax : kUmmaHTileMax / 2;
  int cap_units = pl.nt_cap / 16;
  if (pl.mt == 1 && pl.h_rows <= 64 && D > 0 && D % 64 == 0) {
    // keep tiles low enough for two K slabs per stage and three stages (the 52 KiB operations
    // are worth more than the last 48 rows of tile height)
    const long long per_stage = ((long long)max_smem - (1024 + 1024 + (long long)slack)) / 3;
    const int fit = (int)((per_stage / 2 - (long long)pl.h_rows * 128) / (16 * 128));
    if (fit >= 8 && fit < cap_units) cap_units = fit;
  }
  if (nt_target >= 16 && nt_target / 16 < cap_units) cap_units = nt_target / 16;
  pl.tiles_per_cta = (u_max + cap_units - 1) / cap_units;
  // min_tiles > 1 cuts small per-CTA ranges into several tiles so that epilogues overlap the next
  // mainloop; measured slower on the small shards of 8-way tensor parallelism, because W boxes
  // under ~16 KiB run into the per-thread TMA issue rate.
  if (pl.tiles_per_cta < min_tiles && u_max >= 4 * min_tiles) pl.tiles_per_cta = min_tiles;
  pl.q_units = (u_max + pl.tiles_per_cta - 1) / pl.tiles_per_cta;
  // One thread sustains only about three TMA operations per microsecond, so short tiles fetch
  // several 64-column slabs of the hidden dimension per operation (a 3-D box), aiming at >= 40 KiB
  // of W per operation (measured: 52 KiB operations stream the Qwen head 4% faster than 26 KiB ones).  Needs D % 64 == 0 (a slab index must not run into the next row).
  pl.slabs = 1;
  const size_t fixed = 1024 /*barriers*/ + 1024 /*alignment*/ + slack;
  if (D > 0 && D % 64 == 0) {
    const int w_slab = pl.q_units * 16 * 128;
    int sk = slabs_force > 0 ? slabs_force : (40 * 1024 + w_slab - 1) / w_slab;
    if (sk > 4) sk = 4;
    if (sk > D / 64) sk = D / 64;
    if (sk < 1) sk = 1;
    // keep at least three stages in the ring
    const int min_stages = (stages_cap == 2) ? 2 : 3;
    while (sk > 1 && min_stages * umma_stage_bytes(pl.mt, pl.q_units, pl.h_rows, sk) + fixed > (size_t)max_smem) --sk;
    pl.slabs = sk;
  }
  const size_t sb = umma_stage_bytes(pl.mt, pl.q_units, pl.h_rows, pl.slabs);
  int stages = stages_cap > 1 ? stages_cap : kUmmaMaxStages;
  if (stages > kUmmaMaxStages) stages = kUmmaMaxStages;
  while (stages > 2 && stages * sb + fixed > (size_t)max_smem) --stages;
  pl.stages = stages;
  pl.smem = stages * sb + fixed;
  // Row replicas: the A operand of replica k starts k * (16 KiB / R) bytes before the hidden-state
  // slab, which must still lie inside the stage: the W slabs in front of it have to be that long
  // even for the lower of the two tile heights.
  // Off unless asked for (copies_cap = 2 or 4): measured on the Qwen head, B = 64, the epilogue of a
  // tile drops from 9.5 to 4.9 (2.8) us with 2 (4) replicas, but every MMA re-reads its 128-row A
  // operand, and the mainloop slows from 171 to 236 (344) us.
  int r = 1;
  if (pl.mt == 1 && copies_cap >= 2) {
    r = pl.h_rows <= 32 ? 4 : (pl.h_rows <= 64 ? 2 : 1);
    if (r > copies_cap) r = 2;
  }
  const int low_units = pl.q_units > 1 ? pl.q_units - 1 : pl.q_units;
  while (r > 1 && (size_t)pl.slabs * low_units * 16 * 128 < (size_t)(r - 1) * (16384 / r)) r >>= 1;
  pl.copies = r;
  if (r > 1) pl.m_rows = 128;
  return pl;
}

// The tile schedule of one CTA, recomputed identically by every warp role.
struct TileInfo {
  int v0;  // first vocabulary row
  int nt;  // rows (0: nothing, skip)
};

struct TileWalk {
  int u_next;  // first unit of the next tile
  int base, extra, i, T;
  __device__ __forceinline__ TileWalk(int units_total, int T_) {
    const int per = units_total / (int)gridDim.x, rem = units_total % (int)gridDim.x;
    const int c = blockIdx.x;
    const int u_cnt = per + (c < rem ? 1 : 0);
    u_next = c * per + min(c, rem);
    T = T_;
    base = u_cnt / T;
    extra = u_cnt % T;
    i = 0;
  }
  __device__ __forceinline__ int count() const { return T; }
  __device__ __forceinline__ TileInfo next() {
    const int units = base + (i < extra ? 1 : 0);
    TileInfo t{u_next * 16, units * 16};
    u_next += units;
    ++i;
    return t;
  }
};

// Columns [begin, end) of a tile of `nt` rows (a multiple of 16) that replica k of R scans:
// the tile's 16-row units dealt out as evenly as possible.
__device__ __forceinline__ void replica_columns(int nt, int R, int k, int& begin, int& end) {
  const int units = nt >> 4, per = units / R, rem = units % R;
  begin = (k * per + min(k, rem)) * 16;
  end = begin + (per + (k < rem ? 1 : 0)) * 16;
}

// ---- tcgen05 wrappers ----------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// The same with e4m3 operands (kind::f8f6f4): 32 values of K per instruction, again 32 bytes of each row.
__device__ __forceinline__ void umma_e4m3(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
      "}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// K-major operand tile in shared memory, rows of 128 bytes, 128-byte swizzle:
// 8-row groups are 1024 bytes apart (stride byte offset), descriptor version 1.
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// kind::f16 instruction descriptor: fp32 accumulate, bf16 x bf16, both K-major, M = 128 (or 64).
// With fp8 the operand formats are e4m3 (format code 0 of kind::f8f6f4) instead of bf16 (code 1 of kind::f16).
__host__ __device__ inline uint32_t umma_idesc(int n, int m = 128, bool fp8 = false) {
  const uint32_t fmt = fp8 ? 0u : ((1u << 7) | (1u << 10));
  return (1u << 4) | fmt | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// CW (16 or 32) accumulator columns of the warp's 32 lanes, starting at TMEM address taddr
template <int CW>
__device__ __forceinline__ void tmem_ld_chunk(uint32_t taddr, uint32_t (&r)[CW]) {
  if constexpr (CW == 32) tmem_ld32(taddr, r);
  else tmem_ld16(taddr, r);
}

// ---- epilogue scan shared by the tensor-core kernels ---------------------------------------
struct EpiRow {
  int b;          // batch row this thread owns
  bool row_ok;    // b < B
  bool greedy, ext, ret_logits, quad_aligned;
  float inv_t;
  bool noisy;     // false for a row whose temperature is <= 0: that row is decoded greedily
  unsigned long long seed;
  const float* w_scale = nullptr;  // fp8 weights: per-vocabulary-row scales (null: bf16 weights)
  float h_scale = 1.f;             // fp8 weights: scale of this thread's quantised hidden-state row
};

// CW accumulator columns of the thread's row, as logits: with fp8 weights the raw sums are multiplied by the
// scales of the hidden-state row and of each vocabulary row (columns beyond V keep an arbitrary finite factor;
// no scan uses them).
template <int CW>
__device__ __forceinline__ void load_logit_chunk(const SampleParams& p, const EpiRow& e, uint32_t taddr, int vbase,
                                                 uint32_t (&acc)[CW]) {
  tmem_ld_chunk<CW>(taddr, acc);
  if (e.w_scale != nullptr && e.row_ok) {
    if (vbase + CW <= p.V) {
      const float4* ws = reinterpret_cast<const float4*>(e.w_scale + vbase);  // vbase is a multiple of 16
#pragma unroll
      for (int i = 0; i < CW / 4; ++i) {
        const float4 w = __ldg(ws + i);
        acc[4 * i + 0] = __float_as_uint(__uint_as_float(acc[4 * i + 0]) * (w.x * e.h_scale));
        acc[4 * i + 1] = __float_as_uint(__uint_as_float(acc[4 * i + 1]) * (w.y * e.h_scale));
        acc[4 * i + 2] = __float_as_uint(__uint_as_float(acc[4 * i + 2]) * (w.z * e.h_scale));
        acc[4 * i + 3] = __float_as_uint(__uint_as_float(acc[4 * i + 3]) * (w.w * e.h_scale));
      }
    } else {
#pragma unroll
      for (int i = 0; i < CW; ++i) {
        const float w = __ldg(e.w_scale + min(vbase + i, p.V - 1));
        acc[i] = __float_as_uint(__uint_as_float(acc[i]) * (w * e.h_scale));
      }
    }
  }
}

// kFlagLogprob: fold the first n_ok of NC scaled logits into the thread's running log-sum-exp - one maximum and
// one rescale per chunk.
template <int NC>
__device__ __forceinline__ void lse_chunk(const uint32_t (&acc)[NC], int n_ok, float sc, float& lse_m, float& lse_l) {
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < NC; ++i)
    if (i < n_ok) mx = fmaxf(mx, __uint_as_float(acc[i]));
  if (mx > -INFINITY) {
    const float mn = fmaxf(lse_m, mx * sc);
    float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
    for (int i = 0; i < NC; i += 2) {
      if (i < n_ok) sum0 += ex2_approx(fmaf(__uint_as_float(acc[i]), sc, -mn));
      if (i + 1 < n_ok) sum1 += ex2_approx(fmaf(__uint_as_float(acc[i + 1]), sc, -mn));
    }
    lse_l = lse_l * ex2_approx(lse_m - mn) + (sum0 + sum1);
    lse_m = mn;
  }
}

// The upper 16 columns of a 32-column chunk move from the lanes that hold the rows (0..15) to lanes 16..31, so that
// both half-warps work on an M = 64 accumulator; afterwards every lane holds 16 columns of the row of (lane & 15),
// the first of them column 0 of the chunk in lanes 0..15 and column 16 in lanes 16..31.
__device__ __forceinline__ void split_chunk(const uint32_t (&acc)[32], uint32_t (&half)[16]) {
  const int lane = (int)(threadIdx.x & 31);
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const uint32_t up = __shfl_sync(0xffffffffu, acc[16 + i], lane & 15);
    half[i] = (lane & 16) ? up : acc[i];
  }
}

// kFlagLogprob: fold the scaled logits of columns [c_begin, c_end) of the accumulator tile into the thread's running
// log-sum-exp.  A pass of its own over the tile (TMEM reads are cheap), so that the sampling scan keeps its
// registers.  `split`: see scan_tile_columns; the two lanes of a row keep separate sums.
template <int CW = 32>
__device__ __forceinline__ void lse_tile_columns(const SampleParams& p, const EpiRow& e, uint32_t t_addr,
                                                 int c_begin, int c_end, int v0, float& lse_m, float& lse_l,
                                                 bool split = false) {
  const float sc = e.inv_t * kLog2e;  // > 0: the largest logit gives the largest scaled logit
  for (int c = c_begin; c < c_end; c += CW) {
    uint32_t acc[CW];
    load_logit_chunk<CW>(p, e, t_addr + (uint32_t)c, v0 + c, acc);
    if constexpr (CW == 32) {
      if (split) {
        uint32_t half[16];
        split_chunk(acc, half);
        const int cc = c + (int)(threadIdx.x & 16);
        if (e.row_ok) lse_chunk<16>(half, min(c_end - cc, p.V - (v0 + cc)), sc, lse_m, lse_l);
        continue;
      }
    }
    if (e.row_ok) lse_chunk<CW>(acc, min(c_end - c, p.V - (v0 + c)), sc, lse_m, lse_l);
  }
}

// NC consecutive columns of the thread's row, starting at column c of the tile (vocabulary row v0 + c of this shard),
// for draw `s`: scale, add noise, keep the running (max, id).
template <int NC>
__device__ __forceinline__ void scan_chunk(const SampleParams& p, const EpiRow& e, const uint32_t (&acc)[NC], int c, int c_end,
                                           int v0, int s, float& bv, int& bi) {
  const int vbase = v0 + c;
  if (e.ret_logits && s == 0) {
#pragma unroll
    for (int i = 0; i < NC; ++i)
      if (c + i < c_end && vbase + i < p.V)
        p.logits_out[(size_t)e.b * p.V + vbase + i] = __uint_as_float(acc[i]);
  }
  if (e.greedy) {
#pragma unroll
    for (int i = 0; i < NC; ++i) {
      const float y = __uint_as_float(acc[i]);
      if (c + i < c_end && vbase + i < p.V && y > bv) {
        bv = y;
        bi = vbase + i;
      }
    }
  } else if (e.ext) {
    const float* nz = p.ext_noise + (size_t)s * p.noise_s_stride + (size_t)e.b * p.noise_ld + vbase;
#pragma unroll
    for (int i = 0; i < NC; ++i) {
      if (c + i < c_end && vbase + i < p.V) {
        const float y = fmaf(__uint_as_float(acc[i]), e.inv_t, e.noisy ? nz[i] : 0.f);
        if (y > bv) {
          bv = y;
          bi = vbase + i;
        }
      }
    }
  } else if (!e.noisy) {
    // a row with temperature <= 0 inside a sampled batch: plain argmax, no noise to draw
#pragma unroll
    for (int i = 0; i < NC; ++i) {
      const float y = __uint_as_float(acc[i]) * e.inv_t;
      if (c + i < c_end && vbase + i < p.V && y > bv) {
        bv = y;
        bi = vbase + i;
      }
    }
  } else if (e.quad_aligned) {
    const unsigned long long q0 = (unsigned long long)(p.v_offset + vbase) >> 2;
    const int n_ok = min(c_end - c, p.V - vbase);  // valid columns of this chunk
    int li = -1;  // column (inside the chunk) of a new running maximum: the selects then take immediates
#pragma unroll
    for (int g = 0; g < NC / 4; ++g) {
      const uint4 q = noise_block(e.seed, s, e.b + p.b_offset, q0 + g);
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
      // (A cheap screen in front of the exact comparison - the leading random bits against
      // 2^((x / T - best) log2 e), one ex2 instead of a conversion and two logarithms, exact path for the
      // survivors - was measured and dropped: the last tile of a 5-tile range got 16 % faster, but a
      // CTA's first tile, where new records are frequent and the warp runs both paths, got 14 %
      // slower, and short tensor-parallel shards consist of that tile alone.)
      if (n_ok >= NC) {  // an interior chunk: no column masks
#pragma unroll
        for (int wi = 0; wi < 4; ++wi) {
          const int i = g * 4 + wi;
          const float y = fmaf(__uint_as_float(acc[i]), e.inv_t, gumbel_from_bits(w[wi]));
          if (y > bv) {
            bv = y;
            li = i;
          }
        }
      } else {
#pragma unroll
        for (int wi = 0; wi < 4; ++wi) {
          const int i = g * 4 + wi;
          const float y = fmaf(__uint_as_float(acc[i]), e.inv_t, gumbel_from_bits(w[wi]));
          if (i < n_ok && y > bv) {
            bv = y;
            li = i;
          }
        }
      }
    }
    if (li >= 0) bi = vbase + li;
  } else {
#pragma unroll
    for (int i = 0; i < NC; ++i) {
      const unsigned long long vg = (unsigned long long)(p.v_offset + vbase + i);
      const uint4 q = noise_block(e.seed, s, e.b + p.b_offset, vg >> 2);
      const float y = fmaf(__uint_as_float(acc[i]), e.inv_t, e.noisy ? gumbel_from_bits(pick_word(q, (uint32_t)vg & 3u)) : 0.f);
      if (c + i < c_end && vbase + i < p.V && y > bv) {
        bv = y;
        bi = vbase + i;
      }
    }
  }
}

// Scan columns [c_begin, c_end) of the accumulator tile at TMEM address `t_addr` (this warp's lane
// quadrant, first column of the tile) for draw `s`.  `split` (M = 64 accumulators: only lanes 0..15 of a quadrant
// hold rows): lanes 16..31 fetch the upper 16 columns of each 32-column chunk from the lane that holds the row
// (16 shuffles) and scan them for that row, so that both halves of the warp work; the two lanes of a row keep
// separate running winners, which meet in the row's packed key at the end of the kernel.
template <int CW = 32>
__device__ __forceinline__ void scan_tile_columns(const SampleParams& p, const EpiRow& e, uint32_t t_addr,
                                                  int c_begin, int c_end, int v0, int s, float& bv, int& bi,
                                                  bool split = false) {
  for (int c = c_begin; c < c_end; c += CW) {
    uint32_t acc[CW];
    load_logit_chunk<CW>(p, e, t_addr + (uint32_t)c, v0 + c, acc);
    if constexpr (CW == 32) {
      if (split) {
        uint32_t half[16];
        split_chunk(acc, half);
        if (e.row_ok) scan_chunk<16>(p, e, half, c + (int)(threadIdx.x & 16), c_end, v0, s, bv, bi);
        continue;
      }
    }
    if (e.row_ok) scan_chunk<CW>(p, e, acc, c, c_end, v0, s, bv, bi);
  }
}

// kFlagTopk: scan columns [c_begin, c_end) of the accumulator tile: z = logit / T; track the largest z
// seen (`tmax`) and, when `append`, keep every z >= pivot in the thread's own segment of the row's candidates
// (`seg`, `seg_n` entries so far).  No atomics: appends through a shared per-row counter were measured first -
// their round trips fill the SM's memory-instruction queue, which the mbarrier and TMA instructions of the
// producer and MMA warps share, and slowed the weight stream by 25-40 us.
template <int CW = 32>
__device__ __forceinline__ void topk_scan_columns(const SampleParams& p, const EpiRow& e, uint32_t t_addr, int c_begin,
                                                  int c_end, int v0, float pivot, bool append,
                                                  unsigned long long* seg, int& seg_n, float& tmax) {
  for (int c = c_begin; c < c_end; c += CW) {
    uint32_t acc[CW];
    load_logit_chunk<CW>(p, e, t_addr + (uint32_t)c, v0 + c, acc);
    if (e.row_ok) {
      const int vbase = v0 + c;
#pragma unroll
      for (int i = 0; i < CW; ++i) {
        if (c + i < c_end && vbase + i < p.V) {
          const float z = __uint_as_float(acc[i]) * e.inv_t;
          tmax = fmaxf(tmax, z);
          if (append && z >= pivot) {
            if (seg_n < kTopkSegCap) {
              seg[seg_n] = cand_key(z, vbase + i);
            } else if (seg_n < kTopkSpillDead) {
              // a full segment (large logits clustered in this CTA's vocabulary range): the row's shared spill list
              const unsigned int pos = atomicAdd(&p.topk.extra_count[e.b], 1u);
              if (pos < (unsigned int)kTopkExtraCap) p.topk.extra[(size_t)e.b * kTopkExtraCap + pos] = cand_key(z, vbase + i);
              else seg_n = kTopkSpillDead;  // that list is full too (the count says so): the row goes to the exact pass
            }
            ++seg_n;
          }
        }
      }
    }
  }
}

// The rows' pivots: the smallest of each row's class maxima.  Every class maximum is a different vocabulary
// entry, so at least kTopkSlots entries are >= the pivot and the top_k-th largest logit (top_k <= kTopkSlots)
// cannot lie below it.  An empty class means no bound yet (-inf).  The 16 epilogue warps of the CTA share the
// work: a warp reads a row's 64 class maxima with two coalesced loads, reduces them with shuffles and leaves the
// pivot in shared memory.  (First version: every thread read its own row's 256 bytes, 32 different lines per
// load instruction, four column-group warps each - 262 KB per CTA and tile from a few hot L2 lines, which slowed
// the weight stream by 25-40 us.)
__device__ __forceinline__ void topk_refresh_pivots(const SampleParams& p, float* pivots, int ew, int lane) {
  for (int r = ew; r < p.B; r += kUmmaEpiWarps) {
    const unsigned int* t = p.topk.table + (size_t)r * kTopkSlots;
    uint32_t a, c;
    asm volatile("ld.global.cg.u32 %0, [%1];" : "=r"(a) : "l"(t + lane));
    asm volatile("ld.global.cg.u32 %0, [%1];" : "=r"(c) : "l"(t + 32 + lane));
    uint32_t lo = min(a, c);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) lo = min(lo, __shfl_xor_sync(0xffffffffu, lo, off));
    if (lane == 0) pivots[r] = lo == 0u ? -INFINITY : float_key_decode(lo);
  }
}

// Columns [c_begin, c_end) of the range [r_begin, r_end) that column group `g` of `groups` scans:
// whole CW-column chunks, dealt out evenly.
template <int CW>
__device__ __forceinline__ void group_columns(int r_begin, int r_end, int g, int groups, int& c_begin, int& c_end) {
  const int chunks = (r_end - r_begin + CW - 1) / CW;
  const int per_group = (chunks + groups - 1) / groups;
  c_begin = min(r_begin + g * per_group * CW, r_end);
  c_end = min(c_begin + per_group * CW, r_end);
}

// ---- the kernel ------------------------------------------------------------------
template <int MT, bool LSE = false, bool TOPK = false>
__global__ void __launch_bounds__(kUmmaThreads, 1)
umma_sample_kernel(const __grid_constant__ CUtensorMap w_map_q, const __grid_constant__ CUtensorMap w_map_q1,
                   const __grid_constant__ CUtensorMap h_map, const SampleParams p, const int nt_cap,
                   const int units_total, const int q_units, const int h_rows, const int SK, const int R_,
                   const int m_rows) {
  if (p.run_if) {  // conditional launch: the flag is the previous kernel's to write
    griddep_wait();
    if (*reinterpret_cast<const volatile unsigned int*>(p.run_if) == 0u) return;
  }
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int stages = p.stages;
  const int n_tiles = p.tiles_per_cta;  // tiles of zero rows (tiny vocabularies) are skipped
  const int R = (MT == 1) ? R_ : 1;     // row replicas (see the head of this file)
  // M = 64 (MT = 1, at most 64 batch rows, no replicas): accumulator row i sits in TMEM lane 32 * (i / 16) + i % 16,
  // i.e. 16 rows in the lower half of every lane quadrant
  const bool m64 = (MT == 1) && m_rows == 64;
  // The non-epilogue warps.  (Moving the MMA issuer and the W producer to the warps whose schedulers have no
  // epilogue rows at B <= 64 was measured: no difference.)
  constexpr int mma_warp = 1, w_warp = 0, h_warp = 2;
  // stage = [SK W slabs][MT x SK hidden-state slabs]; SK > 1 means the maps are 3-D (slab = dim 2)
  const size_t h_slab_bytes = (size_t)h_rows * 128;
  const size_t stage_bytes = umma_stage_bytes(MT, q_units, h_rows, SK);
  const int slabs_total = (p.D + kUmmaBK - 1) / kUmmaBK;
  const int KB = (slabs_total + SK - 1) / SK;  // pipeline steps per tile
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem);
  smem += 1024;  // stages start 1 KiB-aligned behind the barriers
  uint64_t* empty_bar = full_bar + stages;
  uint64_t* acc_full = empty_bar + stages;
  uint64_t* acc_empty = acc_full + 4;
  uint64_t* epi_bar = acc_empty + 4;  // two barriers of the epilogue warps (top-k: before / after the grid-wide wait)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(epi_bar + 3);  // a third one: the per-tile pivot refresh
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int acc_stages = kTmemCols / (MT * nt_cap);

  const int cta = blockIdx.x;

  if (tid == 0) {
    for (int i = 0; i < stages; ++i) {
      mbar_init(&full_bar[i], 2);  // W producer + hidden-state producer
      mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < 4; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], kUmmaEpiWarps);
    }
    mbar_init(&epi_bar[0], kUmmaEpiWarps);
    mbar_init(&epi_bar[1], kUmmaEpiWarps);
    mbar_init(&epi_bar[2], kUmmaEpiWarps);
    *abort_flag = 0;
    fence_mbar_init();
    stamp(p, 0);
  }
  if (warp == mma_warp) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  // S > 1 keeps the running candidates of each (row, draw) in global memory: one row per CTA and
  // epilogue warpgroup, which start as "none"
  if (!TOPK && p.S > 1) {
    const int n = kUmmaEpiGroups * p.S * p.cand_rows;
    float* cv = p.cand_val + (size_t)cta * n;
    int* ci = p.cand_idx + (size_t)cta * n;
    for (int i = tid; i < n; i += kUmmaThreads) {
      cv[i] = -INFINITY;
      ci[i] = kIdxNone;
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (tid == 0) stamp(p, 1);

  if (warp == w_warp || warp == h_warp) {
    // ------------------------------ TMA producers -----------------------------
    // Two threads issue the loads of a stage, warp 0 the W tile and warp 2 the
    // hidden-state tile(s): a single thread sustains only about three bulk-tensor
    // operations per microsecond, which would cap the weight stream.
    if (lane == 0) {
      const bool is_w = (warp == w_warp);
      if (is_w) {
        prefetch_tmap(&w_map_q);
        prefetch_tmap(&w_map_q1);
      } else {
        prefetch_tmap(&h_map);
      }
      const uint64_t pol = is_w ? policy_evict_first() : policy_evict_last();
      // The hidden states may be the output of the kernel just before this one (quantised for e4m3 weights,
      // or gathered from host memory): their producer waits for it; the weight stream does not.
      if (!is_w) griddep_wait();
      int it = 0;
      int st = 0;          // ring slot of the next K step, and the parity of its "empty" barrier
      uint32_t phase = 1;
      bool ok = true;
      TileWalk walk(units_total, n_tiles);
      const bool flat = (SK == 1);  // one slab per stage: 2-D maps
      for (int t = 0; t < n_tiles && ok; ++t) {
        const TileInfo ti = walk.next();
        const int v0 = ti.v0, NT = ti.nt;
        if (NT == 0) continue;
        const uint32_t tx = (uint32_t)SK * (is_w ? (uint32_t)NT * 128u : (uint32_t)MT * (uint32_t)h_rows * 128u);
        const CUtensorMap* wm = (NT == q_units * 16) ? &w_map_q : &w_map_q1;
        const size_t h_off = (size_t)SK * NT * 128;   // hidden-state slabs follow the W slabs
        for (int kb = 0; kb < KB; ++kb, ++it) {
          if (!mbar_wait(&empty_bar[st], phase, abort_flag, p.status_dev)) {
            ok = false;
            break;
          }
          uint8_t* sw = smem + st * stage_bytes;
          mbar_arrive_expect_tx(&full_bar[st], tx);
          if (is_w) {
            if (flat) tma_load_2d_hint(sw, wm, kb * kUmmaBK, v0, &full_bar[st], pol);
            else tma_load_3d_hint(sw, wm, 0, v0, kb * SK, &full_bar[st], pol);
          } else {
#pragma unroll
            for (int m = 0; m < MT; ++m) {
              uint8_t* dst = sw + h_off + (size_t)m * SK * h_slab_bytes;
              if (flat) tma_load_2d_hint(dst, &h_map, kb * kUmmaBK, m * 128, &full_bar[st], pol);
              else tma_load_3d_hint(dst, &h_map, 0, m * 128, kb * SK, &full_bar[st], pol);
            }
          }
          if (++st == stages) {
            st = 0;
            phase ^= 1u;
          }
        }
      }
      if (*abort_flag) {
        for (int st = 0; st < min(it, stages); ++st) {
          const int last_it = ((it - 1 - st) / stages) * stages + st;
          mbar_wait_plain(&full_bar[st], (uint32_t)(last_it / stages) & 1u, 100000000ull);
        }
      }
    }
  } else if (warp == mma_warp) {
    // ------------------------------ MMA issuer --------------------------------
    // One thread feeds the tensor core, and a K step's MMA takes about as long as the HBM needs for that step's
    // bytes: the loop between two tcgen05.mma is kept free of divisions and repeated branches (per-tile
    // constants are hoisted, ring slot and phase are counted, the operand kind is decided once per K step).
    if (lane == 0) {
      bool ok = true;
      TileWalk walk(units_total, n_tiles);
      const uint32_t a_shift = (uint32_t)(16384 / R);  // bytes by which each further replica's A operand starts earlier
      const bool fp8 = (p.flags & kFlagFp8) != 0;
      const uint32_t smem0 = smem_u32(smem);
      int st = 0;            // ring slot of the next K step
      uint32_t phase = 0;    // its parity
      bool first = true;
      int j = 0;             // accumulator buffer of the next tile
      uint32_t acc_phase = 0;
      for (int t = 0; t < n_tiles && ok; ++t) {
        const TileInfo ti = walk.next();
        const int NT = ti.nt;
        if (NT == 0) continue;
        const uint32_t h_off = (uint32_t)(SK * NT * 128);
        const uint32_t w_pitch = (uint32_t)(NT * 128);  // TMA packs the slabs of a box back to back: the pitch follows the tile height
        // the column ranges (and instruction descriptors) of the replicas; R = 1: the whole tile
        int cb[4] = {0, 0, 0, 0};
        uint32_t idesc[4] = {0, 0, 0, 0};
        for (int r = 0; r < R; ++r) {
          int ce;
          replica_columns(NT, R, r, cb[r], ce);
          idesc[r] = ce > cb[r] ? umma_idesc(ce - cb[r], m64 ? 64 : 128, fp8) : 0u;
        }
        const uint32_t idesc_full = umma_idesc(NT, 128, fp8);
        if (!mbar_wait(&acc_empty[j], acc_phase ^ 1u, abort_flag, p.status_dev)) break;
        tc_fence_after();
        for (int kb = 0; kb < KB; ++kb) {
          if (!mbar_wait(&full_bar[st], phase, abort_flag, p.status_dev)) {
            ok = false;
            break;
          }
          tc_fence_after();
          if (first) {
            stamp(p, 2);
            first = false;
          }
          const uint32_t sw = smem0 + (uint32_t)st * (uint32_t)stage_bytes;
          for (int sl = 0; sl < SK; ++sl) {
            const uint32_t w_slab = sw + (uint32_t)sl * w_pitch;
            const uint32_t acc0 = (kb | sl) != 0 ? 1u : 0u;
            if (MT == 1) {
              const uint32_t a_slab = sw + h_off + (uint32_t)(sl * h_slab_bytes);
              for (int r = 0; r < R; ++r) {
                if (idesc[r] == 0u) continue;
                const uint64_t adesc = umma_smem_desc(a_slab - (uint32_t)r * a_shift);
                const uint64_t bdesc = umma_smem_desc(w_slab + (uint32_t)(cb[r] * 128));
                const uint32_t d_tmem = tmem_base + (uint32_t)(j * nt_cap + cb[r]);
                // advance both descriptors by 16 bf16 (32 e4m3) = 32 bytes inside the swizzled row
                if (fp8) {
                  umma_e4m3(d_tmem, adesc, bdesc, idesc[r], acc0);
                  umma_e4m3(d_tmem, adesc + 2, bdesc + 2, idesc[r], 1u);
                  umma_e4m3(d_tmem, adesc + 4, bdesc + 4, idesc[r], 1u);
                  umma_e4m3(d_tmem, adesc + 6, bdesc + 6, idesc[r], 1u);
                } else {
                  umma_bf16(d_tmem, adesc, bdesc, idesc[r], acc0);
                  umma_bf16(d_tmem, adesc + 2, bdesc + 2, idesc[r], 1u);
                  umma_bf16(d_tmem, adesc + 4, bdesc + 4, idesc[r], 1u);
                  umma_bf16(d_tmem, adesc + 6, bdesc + 6, idesc[r], 1u);
                }
              }
            } else {
              const uint64_t bdesc = umma_smem_desc(w_slab);
#pragma unroll
              for (int m = 0; m < MT; ++m) {
                const uint64_t adesc = umma_smem_desc(sw + h_off + (uint32_t)((m * SK + sl) * h_slab_bytes));
                const uint32_t d_tmem = tmem_base + (uint32_t)((j * MT + m) * nt_cap);
                if (fp8) {
                  umma_e4m3(d_tmem, adesc, bdesc, idesc_full, acc0);
                  umma_e4m3(d_tmem, adesc + 2, bdesc + 2, idesc_full, 1u);
                  umma_e4m3(d_tmem, adesc + 4, bdesc + 4, idesc_full, 1u);
                  umma_e4m3(d_tmem, adesc + 6, bdesc + 6, idesc_full, 1u);
                } else {
                  umma_bf16(d_tmem, adesc, bdesc, idesc_full, acc0);
                  umma_bf16(d_tmem, adesc + 2, bdesc + 2, idesc_full, 1u);
                  umma_bf16(d_tmem, adesc + 4, bdesc + 4, idesc_full, 1u);
                  umma_bf16(d_tmem, adesc + 6, bdesc + 6, idesc_full, 1u);
                }
              }
            }
          }
          umma_commit(&empty_bar[st]);  // stage reusable once these MMAs have read it
          if (++st == stages) {
            st = 0;
            phase ^= 1u;
          }
        }
        if (ok) umma_commit(&acc_full[j]);  // accumulator complete
        if (++j == acc_stages) {
          j = 0;
          acc_phase ^= 1u;
        }
      }
      stamp(p, 3);
    }
  } else if (warp >= kUmmaEpiWarp0) {
    // -------------------------------- epilogue --------------------------------
    griddep_wait();  // temperatures and scales may come from the kernel just before this one
    const int ew = warp - kUmmaEpiWarp0;  // 0..15
    const int wg = ew >> 2;               // epilogue warpgroup 0..3
    const int quad = warp & 3;            // TMEM lane quadrant this warp may read
    // MT = 1: the four warpgroups split the columns four ways; MT = 2: two per M tile
    const int m_tile = (MT == 2) ? (wg & 1) : 0;
    const int col_group = (MT == 2) ? (wg >> 1) : wg;
    constexpr int kColGroups = (MT == 2) ? kUmmaEpiGroups / 2 : kUmmaEpiGroups;
    // the replica whose rows sit in this quadrant's lanes, and the batch row of this thread
    const int lanes_per_replica = 128 / R;
    const int replica = (quad * 32) / lanes_per_replica;
    // M = 64 accumulators keep rows in lanes 0..15 of each quadrant only.  The sampling scan then splits every
    // chunk of columns between the two half-warps (lanes 16..31 work for the row of lane - 16), and so does the
    // log-sum-exp scan; the top-k scan leaves the upper lanes idle.
    const bool split = m64 && !TOPK;
    const int b = m64 ? quad * 16 + (lane & 15) : m_tile * 128 + quad * 32 + lane - replica * lanes_per_replica;
    const bool holds_acc = !m64 || lane < 16;               // this lane's TMEM lane carries a batch row
    const bool row_ok = b < p.B && (split || holds_acc);    // this thread scans for row b
    const bool acc_ok = b < p.B && holds_acc;
    const bool warp_ok = m64 ? quad * 16 < p.B : (m_tile * 128 + quad * 32 - replica * lanes_per_replica) < p.B;
    // row of the S > 1 scratch: replicas, and the two lanes of a split row, must not share one
    const int cand_row = (R > 1 || split) ? quad * 32 + lane : b;

    const bool greedy = (p.flags & kFlagGreedy) != 0;
    const bool ext = (p.flags & kFlagExtNoise) != 0;
    const bool ret_logits = (p.flags & kFlagReturnLogits) != 0;
    const bool quad_aligned = (p.v_offset & 3) == 0;
    float invT = 1.0f;
    bool noisy = true;
    if (row_ok && !greedy) {
      const float temp = p.temperature[(size_t)b * p.temp_stride];
      noisy = temp > 0.f;  // temperature <= 0 selects greedy decoding for this row
      invT = noisy ? 1.0f / temp : 1.0f;
    }
    EpiRow row{b, row_ok, greedy, ext, ret_logits, quad_aligned, invT, noisy, resolve_seed(p.seed, p.flags)};
    if (p.flags & kFlagFp8) {
      row.w_scale = p.w_scale;
      row.h_scale = row_ok ? p.h_scale[b] : 1.f;
    }
    const int S = p.S;
    const size_t slot_row = ((size_t)cta * kUmmaEpiGroups + wg) * ((size_t)S * p.cand_rows);
    const bool narrow = (R == 4);  // four replicas leave ~50 columns per quadrant: deal them out in 16-column chunks

    float best_val = -INFINITY;  // S == 1: lives in registers for the whole kernel
    int best_idx = kIdxNone;
    float lse_m = -INFINITY, lse_l = 0.f;  // kFlagLogprob: this thread's share of the row's log-sum-exp
    bool topk_started = false;             // kFlagTopk: the CTA's first tile has been through the grid-wide step
    // kFlagTopk: this thread's private segment of its row's candidates
    // (with two M tiles a thread scans half of every tile, four times the columns of a thread of the one-M-tile
    // layout: it owns two segments and fills them on alternate tiles, which keeps a segment's expected load -
    // a few entries - far from its capacity even for a row whose early pivots come out low)
    constexpr int kSegsPerThread = (MT == 2) ? 2 : 1;
    const int topk_seg_id = (cta * kColGroups + col_group) * kSegsPerThread;
    unsigned long long* topk_seg =
        TOPK && row_ok ? p.topk.list + ((size_t)b * kTopkMaxSegs + topk_seg_id) * kTopkSegCap : nullptr;
    int topk_seg_n = 0, topk_seg_n2 = 0;
    // the rows' pivots live in the slack behind the last pipeline stage (the MMA reads that area as operand rows
    // that belong to no batch row; nothing else uses it)
    float* topk_pivots = reinterpret_cast<float*>(smem + (size_t)stages * stage_bytes);
    uint32_t pivot_phase = 0;

    TileWalk walk(units_total, n_tiles);
    for (int t = 0, ta = 0; t < n_tiles; ++t) {
      const TileInfo ti = walk.next();
      const int v0 = ti.v0, NT = ti.nt;
      if (NT == 0) continue;
      // column range of this warp inside the tile: the replica's columns, dealt out to the column groups
      int r_begin = 0, r_end = NT, c_begin, c_end;
      if (R > 1) replica_columns(NT, R, replica, r_begin, r_end);
      if (narrow) group_columns<16>(r_begin, r_end, col_group, kColGroups, c_begin, c_end);
      else group_columns<32>(r_begin, r_end, col_group, kColGroups, c_begin, c_end);
      const int j = ta % acc_stages;
      const uint32_t un = (uint32_t)(ta / acc_stages);
      ++ta;
      if (!mbar_wait(&acc_full[j], un & 1u, abort_flag, p.status_dev)) break;
      tc_fence_after();
      if (ew == 0 && lane == 0 && t == n_tiles - 1) stamp(p, 4);
      if constexpr (TOPK) {
        // Candidates for top-k: everything at or above the row's pivot goes into this thread's segment of the
        // row's candidates.  The pivot is the smallest of kTopkSlots class maxima, to which every (CTA, column
        // group, tile) contributes the largest scaled logit it has seen.  The first tile is scanned twice: once
        // for its maxima, then - after every CTA of the grid has published its own - for the candidates;
        // later tiles refresh the pivots, collect, and publish their maximum afterwards.
        const uint32_t t_addr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)((j * MT + m_tile) * nt_cap);
        // odd multipliers: every row reaches all slots, and every slot hears from all column groups (whose
        // shares of a tile differ in width), so that no class is made of narrow shares only
        const int slot = (cta * 5 + (m_tile * kColGroups + col_group) * 17 + 37 * t) & (kTopkSlots - 1);
        float tmax = -INFINITY;
        const bool first_tile = !topk_started;
        if (first_tile) {
          if (warp_ok) topk_scan_columns<32>(p, row, t_addr, c_begin, c_end, v0, 0.f, false, topk_seg, topk_seg_n, tmax);
          if (row_ok && tmax > -INFINITY) atomicMax(&p.topk.table[(size_t)b * kTopkSlots + slot], float_key(tmax));
          __threadfence();
          __syncwarp();
          if (lane == 0) mbar_arrive(&epi_bar[0]);
          bool ok = mbar_wait(&epi_bar[0], 0u, abort_flag, p.status_dev);
          if (ok && ew == 0 && lane == 0) {
            // grid-wide: all CTAs are resident (one per SM), so every one of them arrives
            atomicAdd(p.topk.gbar, 1u);
            const unsigned long long t0 = global_timer_ns();
            unsigned int spins = 0;
            while (*reinterpret_cast<volatile unsigned int*>(p.topk.gbar) < gridDim.x) {
              if ((++spins & 0xffu) == 0 && (*abort_flag || global_timer_ns() - t0 > kWaitLimitNs)) {
                *abort_flag = 1;
                if (p.status_dev) atomicExch(p.status_dev, kErrTimeout);
                break;
              }
            }
            __threadfence();
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(&epi_bar[1]);
          ok = ok && mbar_wait(&epi_bar[1], 0u, abort_flag, p.status_dev);
          if (!ok) break;
          topk_started = true;
        }
        // this tile's pivots, computed by all epilogue warps together
        topk_refresh_pivots(p, topk_pivots, ew, lane);
        __syncwarp();
        if (lane == 0) mbar_arrive(&epi_bar[2]);
        if (!mbar_wait(&epi_bar[2], pivot_phase, abort_flag, p.status_dev)) break;
        pivot_phase ^= 1u;
        const float pivot = row_ok ? topk_pivots[b] : INFINITY;
        if (warp_ok) {
          if (kSegsPerThread == 2 && (t & 1))
            topk_scan_columns<32>(p, row, t_addr, c_begin, c_end, v0, pivot, true, topk_seg + kTopkSegCap, topk_seg_n2, tmax);
          else
            topk_scan_columns<32>(p, row, t_addr, c_begin, c_end, v0, pivot, true, topk_seg, topk_seg_n, tmax);
        }
        // later tiles publish their maximum after the scan (the first tile's went out before the grid-wide wait)
        if (!first_tile && row_ok && tmax > -INFINITY)
          atomicMax(&p.topk.table[(size_t)b * kTopkSlots + slot], float_key(tmax));
      } else if (warp_ok) {
        const uint32_t t_addr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)((j * MT + m_tile) * nt_cap);
        if constexpr (LSE) {
          if (narrow) lse_tile_columns<16>(p, row, t_addr, c_begin, c_end, v0, lse_m, lse_l);
          else lse_tile_columns<32>(p, row, t_addr, c_begin, c_end, v0, lse_m, lse_l, split);
        }
        for (int s = 0; s < S; ++s) {
          float bv = best_val;
          int bi = best_idx;
          if (S > 1) {
            bv = -INFINITY;
            bi = kIdxNone;
          }
          if (narrow) scan_tile_columns<16>(p, row, t_addr, c_begin, c_end, v0, s, bv, bi);
          else scan_tile_columns<32>(p, row, t_addr, c_begin, c_end, v0, s, bv, bi, split);
          if (S > 1) {
            if (row_ok) {
              const size_t o = slot_row + (size_t)s * p.cand_rows + cand_row;
              if (bv > p.cand_val[o]) {  // later tiles have larger indices: strict compare keeps the lowest
                p.cand_val[o] = bv;
                p.cand_idx[o] = bi;
              }
            }
          } else {
            best_val = bv;
            best_idx = bi;
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[j]);
    }
    if (ew == 0 && lane == 0) stamp(p, 5);
    if (LSE && split) {
      // the upper half-warp's sums join those of the lanes that hold the rows
      const float m2 = __shfl_down_sync(0xffffffffu, lse_m, 16), l2 = __shfl_down_sync(0xffffffffu, lse_l, 16);
      if (lane < 16) lse_merge(lse_m, lse_l, m2, l2);
    }
    if (TOPK && row_ok) {
      p.topk.seg_count[(size_t)b * kTopkMaxSegs + topk_seg_id] = (unsigned int)topk_seg_n;
      if (kSegsPerThread == 2) p.topk.seg_count[(size_t)b * kTopkMaxSegs + topk_seg_id + 1] = (unsigned int)topk_seg_n2;
    }
    // merge this thread's winners into the per-(row, draw) keys
    if (!TOPK && S == 1 && R == 1) {
      // One key per row and CTA: the winners of a row's column groups (and half-warps) meet in shared memory,
      // in the slack behind the last pipeline stage, before one thread per row merges them into the global key.
      unsigned long long* cta_keys = reinterpret_cast<unsigned long long*>(smem + (size_t)stages * stage_bytes);
      const int halves = split ? 2 : 1;
      if (row_ok)
        cta_keys[(size_t)(col_group * halves + (split ? (lane >> 4) : 0)) * (MT * 128) + b] =
            best_idx != kIdxNone ? cand_key(best_val, best_idx) : 0ull;
      __syncwarp();
      if (lane == 0) mbar_arrive(&epi_bar[0]);
      if (mbar_wait(&epi_bar[0], 0u, abort_flag, p.status_dev)) {
        const int r = ew * 32 + lane;
        if (r < MT * 128 && r < p.B) {
          unsigned long long k = 0ull;
          for (int g = 0; g < kColGroups * halves; ++g) k = max(k, cta_keys[(size_t)g * (MT * 128) + r]);
          if (k != 0ull) atomicMax(&p.keys[r], k);
        }
      }
    }
    if (!TOPK && row_ok) {
      if (S == 1) {
        if (R > 1 && best_idx != kIdxNone) atomicMax(&p.keys[b], cand_key(best_val, best_idx));
      } else {
        for (int s = 0; s < S; ++s) {
          const size_t o = slot_row + (size_t)s * p.cand_rows + cand_row;
          const int ci = p.cand_idx[o];
          if (ci != kIdxNone) atomicMax(&p.keys[(size_t)s * p.B + b], cand_key(p.cand_val[o], ci));
        }
      }
      // every tile has been multiplied, so the pipeline's first stage is free: it collects the
      // partial sums of each row, one per (replica, column group)
      if (LSE && acc_ok)
        reinterpret_cast<unsigned long long*>(smem)[(replica * kColGroups + col_group) * (MT * 128) + b] =
            lse_pack(lse_m, lse_l);
    }
  }

  griddep_wait();  // every thread, before the tail reads or writes anything the previous kernel may have touched
  tc_fence_before();
  __threadfence();
  __syncthreads();
  if (warp == mma_warp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  if constexpr (LSE) {
    // one partial row per CTA: the (replica, column group) sums merged in a fixed order
    constexpr int kGroups = (MT == 2) ? kUmmaEpiGroups / 2 : kUmmaEpiGroups;
    const unsigned long long* part = reinterpret_cast<const unsigned long long*>(smem);
    for (int r = tid; r < MT * 128 && r < p.B; r += kUmmaThreads) {
      float m = -INFINITY, l = 0.f;
      for (int g = 0; g < kGroups * R; ++g) lse_merge_packed(m, l, part[g * (MT * 128) + r]);
      p.lse[(size_t)cta * p.B + r] = lse_pack(m, l);
    }
  }
  if (!TOPK && !(p.flags & kFlagTwoStage)) {
    volatile int* is_last = abort_flag + 1;
    finish_sample<LSE>(p, tid, kUmmaThreads, [] { __syncthreads(); }, is_last, /*fenced_and_synced=*/!LSE);
  }
}

}  // namespace fmms
