// Small-batch weight-streaming kernel (batch rows <= 8) and the pieces every sampling kernel
// shares: the parameter block and the tail that decodes the winners (and, with tensor
// parallelism, exchanges them over NVLink).
//
// A persistent grid of one CTA per SM.  A producer warp streams row groups of W[V, D] - 32 rows
// (64 for two to four batch rows) by one or two 256-column chunks per TMA operation
// (cp.async.bulk.tensor, 16 to 64 KiB) - through a shared-memory ring with mbarriers; eight
// consumer warps each own four (eight) rows of the group and accumulate fp32 dot products
// (packed fma.rn.f32x2) against the hidden states, which sit in shared memory for the whole
// kernel.  When a group is complete the sums are reduced across the warp, scaled by 1/T,
// perturbed with Gumbel noise and folded into a running (max, index) per (row b, draw s) that
// lives in registers for the whole CTA.  Groups are dealt out 7/8 statically (contiguous ranges)
// and 1/8 through an atomic counter, because SMs do not all get the same share of the HBM
// bandwidth.  One packed candidate per (b, s) per CTA reaches global memory (atomicMax).
#pragma once

#include <cuda.h>

#include "fmms_common.cuh"
#include "fmms_tp.cuh"

namespace fmms {

constexpr int kGemvConsumerWarps = 8;
constexpr int kGemvCols = 256;  // columns per stage
// Rows of a group that one warp owns: 8 for two to four batch rows (more independent
// accumulation chains per warp and half the hidden-state reloads); 4 for a single row, where
// the finer 32-row groups balance better over the SMs, and above four rows (registers).
__host__ __device__ constexpr int gemv_rows_per_warp(int NB) { return (NB >= 2 && NB <= 4) ? 8 : 4; }
__host__ __device__ constexpr int gemv_rows(int NB) { return kGemvConsumerWarps * gemv_rows_per_warp(NB); }
__host__ __device__ constexpr int gemv_stage_bytes(int NB) { return gemv_rows(NB) * kGemvCols * 2; }
constexpr int kGemvThreads = (kGemvConsumerWarps + 1) * 32;       // + producer warp
constexpr int kGemvMaxBatch = 8;
constexpr int kGemvMaxStages = 6;  // ring depth cap: ~96-128 KiB in flight per SM, deeper rings measured slower

constexpr int kLseMaxSplit = 16;  // partial sums per row left by the first merge step
constexpr int kLseMaxRows = 256;  // batch rows per launch

struct SampleParams {
  const __nv_bfloat16* H;    // [B, D]
  const float* temperature;  // [1] or [B]
  int temp_stride;           // 0 or 1
  int V, D, B, S;
  unsigned long long seed;
  long long v_offset;        // global vocabulary id of row 0
  int flags;
  const float* ext_noise;    // element (s, b, v) at s * noise_s_stride + b * noise_ld + v
  long long noise_ld;
  long long noise_s_stride;
  int b_offset;              // batch row of this call's row 0 inside the caller's batch (keys the noise)
  float* logits_out;         // [B, V]
  unsigned long long* keys;  // [S * B] packed winners, zero on entry and on exit (atomicMax target)
  unsigned int* ticket;      // CTAs-done counter, zero on entry and on exit
  unsigned int* sched;       // dynamic work counter, zero on entry and on exit
  float* cand_val;           // [4 * gridDim.x, S * cand_rows] running per-CTA candidates (tensor-core path, S > 1)
  int* cand_idx;
  int cand_rows;             // rows of that scratch: B, or 128 (one per TMEM lane) with 64-row accumulators or row replicas
  long long* out_idx;        // [B, S]
  float* out_val;            // [B, S] or null
  // kFlagLogprob: per-CTA partial log-sum-exps, the rows' normalisers, and the outputs
  unsigned long long* lse;   // [lse_parts, B] packed (m, l); every launch writes all it reads
  unsigned long long* lse2;  // [kLseMaxSplit, kLseMaxRows] scratch of the last CTA's two-step merge
  int lse_parts;             // CTAs (CTA pairs) that write a partial row
  float* out_logprob;        // [B, S] ln p(sampled id)
  float* out_lse;            // [B] ln sum_v exp(logit_v / T), or null
  int* status_dev;
  int* status_mirror;        // optional: host-mapped copy of *status_dev, written by the last CTA when it is done
  unsigned long long* stamps;  // optional [gridDim.x][8] %globaltimer stamps of the kernel's phases (null = off)
  int stages;                // shared-memory ring depth
  int gemv_chunks;           // weight-streaming kernel: 256-column chunks fetched per TMA operation
  int tile_rows;             // tensor-core path: vocabulary rows per tile
  int tiles_per_cta;         // tensor-core path
  // tensor parallelism (tp_world > 1): the last CTA also runs the cross-rank exchange
  int tp_rank, tp_world, tp_max_items;
  unsigned int tp_epoch;
  unsigned long long tp_wait_ns;
  TpPeers tp_peers;
  // fp8 weights (kFlagFp8): logit = accumulator * w_scale[v] * h_scale[b]
  const float* w_scale;      // [V] one scale per vocabulary row
  const float* h_scale;      // [B] one scale per (quantised) hidden-state row
  // top-k / top-p (kFlagTopk): the pass collects candidates, other kernels finish the rows
  TopkArgs topk;
  const unsigned int* run_if;  // optional: the kernel returns at once when this word is zero
};

// Last step of a sampling kernel, run by `nthreads` threads of every CTA after their packed
// candidates went into p.keys with atomicMax: the CTA that takes the last ticket decodes the
// winners into the output and leaves keys and ticket zero for the next launch.
__device__ __forceinline__ void stamp(const SampleParams& p, int slot) {
  if (p.stamps) p.stamps[(size_t)blockIdx.x * 8 + slot] = global_timer_ns();
}

// Log-probability of a decoded winner (kFlagLogprob): the perturbed value minus the winner's
// own noise, which is a pure function of (seed, draw, row, id), gives logit / T; the row's
// log-sum-exp slot gives the normaliser.
__device__ __forceinline__ float winner_logit(const SampleParams& p, int b, int s, float y, int idx) {
  if (idx < 0 || idx >= p.V) return __int_as_float(0x7fc00000);  // no candidate: NaN
  float g = 0.f;
  if (!(p.flags & kFlagGreedy) && p.temperature[(size_t)b * p.temp_stride] > 0.f) {
    if (p.flags & kFlagExtNoise) {
      g = p.ext_noise[(size_t)s * p.noise_s_stride + (size_t)b * p.noise_ld + idx];
    } else {
      const unsigned long long vg = (unsigned long long)(p.v_offset + idx);
      const uint4 q = noise_block(resolve_seed(p.seed, p.flags), s, b + p.b_offset, vg >> 2);
      g = gumbel_from_bits(pick_word(q, (uint32_t)vg & 3u));
    }
  }
  return y - g;
}
__device__ __forceinline__ float winner_logprob(const SampleParams& p, int b, int s, float y, int idx, float lse) {
  return winner_logit(p, b, s, y, idx) - lse;
}

template <bool LSE = false, class SyncFn>
__device__ __forceinline__ void finish_sample(const SampleParams& p, int tid, int nthreads, SyncFn sync,
                                              volatile int* is_last, bool fenced_and_synced = false) {
  if (!fenced_and_synced) {
    __threadfence();
    sync();
  }
  if (tid == 0) {
    // Tensor parallel with the step counter kept on the device: fetch it now, so that its latency
    // overlaps the ticket's (only the CTA that turns out to be last uses it; is_last[1] carries it)
    unsigned int step = p.tp_epoch;
    if (p.tp_world > 1 && step == 0u)
      step = tp_load_counter(reinterpret_cast<const unsigned int*>(
                 reinterpret_cast<const unsigned char*>(p.tp_peers.slots[p.tp_rank]) +
                 tp_counter_offset(p.tp_world, p.tp_max_items))) + 1u;
    *is_last = (atomicAdd(p.ticket, 1u) == gridDim.x - 1) ? 1 : 0;
    is_last[1] = (int)step;
  }
  sync();
  if (tid == 0) stamp(p, 6);
  if (!*is_last) return;
  __threadfence();
  const int n = p.B * p.S;
  // kFlagLogprob, first step: the CTAs' partial sums [lse_parts][B] shrink to [lse_k][B].  A warp
  // takes up to 32 consecutive rows (coalesced loads; with fewer rows the spare lanes share the
  // partial rows and a shuffle tree joins them) and every lse_k-th share of the partial rows.  The
  // merge order is fixed: with statically tiled kernels the result is reproducible bit for bit.
  int lse_k = 1;
  if constexpr (LSE) {
    const int lane = tid & 31, warp = tid >> 5, nwarps = nthreads >> 5;
    const int nblk = (p.B + 31) >> 5;  // <= 8 <= nwarps
    lse_k = min(nwarps / nblk, kLseMaxSplit);
    int rows = 32;  // rows per warp: 32, or the batch rounded up to a power of two
    if (p.B < 32) {
      rows = 1;
      while (rows < p.B) rows <<= 1;
    }
    if (warp < nblk * lse_k) {  // warp-uniform
      const int per_row = 32 / rows;  // lanes that share a row
      const int b = (warp % nblk) * 32 + (lane & (rows - 1)), j = warp / nblk;
      const int step = lse_k * per_row;
      float m = -INFINITY, l = 0.f;
      if (b < p.B) {
        int part = j * per_row + lane / rows;
        for (; part + 3 * step < p.lse_parts; part += 4 * step) {  // four loads in flight
          unsigned long long x[4];
#pragma unroll
          for (int u = 0; u < 4; ++u)
            x[u] = *reinterpret_cast<volatile unsigned long long*>(&p.lse[(size_t)(part + u * step) * p.B + b]);
#pragma unroll
          for (int u = 0; u < 4; ++u) lse_merge_packed(m, l, x[u]);
        }
        for (; part < p.lse_parts; part += step)
          lse_merge_packed(m, l, *reinterpret_cast<volatile unsigned long long*>(&p.lse[(size_t)part * p.B + b]));
      }
      for (int off = rows; off < 32; off <<= 1) {
        const float m2 = __shfl_xor_sync(0xffffffffu, m, off);
        const float l2 = __shfl_xor_sync(0xffffffffu, l, off);
        lse_merge(m, l, m2, l2);
      }
      if (lane < rows && b < p.B) p.lse2[(size_t)j * kLseMaxRows + b] = lse_pack(m, l);
    }
    __threadfence_block();
    sync();
  }
  if (p.tp_world <= 1) {
    for (int item = tid; item < n; item += nthreads) {
      const unsigned long long k = atomicExch(&p.keys[item], 0ull);
      float v;
      int idx;
      cand_key_decode(k, v, idx);
      const int s = item / p.B, b = item - s * p.B;
      p.out_idx[(size_t)b * p.S + s] = p.v_offset + idx;
      if (p.out_val) p.out_val[(size_t)b * p.S + s] = v;
      if constexpr (LSE) {
        // second step: the row's lse_k partial sums, then the winner's log-probability
        float m = -INFINITY, l = 0.f;
        for (int j = 0; j < lse_k; ++j)
          lse_merge_packed(m, l, *reinterpret_cast<volatile unsigned long long*>(&p.lse2[(size_t)j * kLseMaxRows + b]));
        const float lse = lse_value(m, l);
        p.out_logprob[(size_t)b * p.S + s] = winner_logprob(p, b, s, v, idx, lse);
        if (s == 0 && p.out_lse) p.out_lse[b] = lse;
      }
    }
    if (tid == 0) {
      *p.ticket = 0u;
      *p.sched = 0u;
      stamp(p, 7);
      // every other CTA has finished its waits before this one took the last ticket
      if (p.status_mirror && p.status_dev) *p.status_mirror = *reinterpret_cast<volatile int*>(p.status_dev);
    }
    return;
  }
  // Tensor parallel: this rank's winners go straight into every rank's exchange buffer (see
  // fmms_tp.cuh for the protocol), then the same threads wait for the peers' records and keep
  // the maximum.  Items are processed in rounds of `nthreads`: send a round, then receive it.
  const int world = p.tp_world, rank = p.tp_rank;
  // this step's number: the caller's, or one more than the count kept in the rank's own buffer (a captured
  // launch then advances by itself on every replay); fetched by thread 0 before the ticket
  const unsigned int epoch = (unsigned int)is_last[1];
  unsigned int* counter = reinterpret_cast<unsigned int*>(reinterpret_cast<unsigned char*>(p.tp_peers.slots[rank]) +
                                                          tp_counter_offset(world, p.tp_max_items));
  if (tid == 0) *counter = epoch;
  const int parity = (int)(epoch & 1u);
  const size_t my_row = ((size_t)parity * world + rank) * p.tp_max_items;
  const TpRecord* mine = p.tp_peers.slots[rank] + (size_t)parity * world * p.tp_max_items;
  // kFlagLogprob: two more regions - every item's unperturbed winning logit, every row's (m, l)
  const size_t logit_region = tp_logit_region(world, p.tp_max_items);
  const size_t lse_region = tp_lse_region(world, p.tp_max_items);
  const size_t lse_parity = lse_region + (size_t)parity * world * kTpMaxRows;
  for (int item = tid; item < n; item += nthreads) {
    const unsigned long long k = atomicExch(&p.keys[item], 0ull);
    float v;
    int idx;
    cand_key_decode(k, v, idx);
    tp_send(p.tp_peers, world, my_row + item, v, p.v_offset + idx, epoch);
    if constexpr (LSE) {
      const int s = item / p.B, b = item - s * p.B;
      tp_send_words(p.tp_peers, world, logit_region + my_row + item, winner_logit(p, b, s, v, idx), 0u, epoch);
      if (s == 0) {  // this shard's log-sum-exp of row b
        float m = -INFINITY, l = 0.f;
        for (int j = 0; j < lse_k; ++j)
          lse_merge_packed(m, l, *reinterpret_cast<volatile unsigned long long*>(&p.lse2[(size_t)j * kLseMaxRows + b]));
        tp_send_words(p.tp_peers, world, lse_parity + (size_t)rank * kTpMaxRows + b, m, __float_as_uint(l), epoch);
      }
    }
  }
  if (tid == 0) {
    *p.ticket = 0u;
    *p.sched = 0u;
  }
  for (int item = tid; item < n; item += nthreads) {
    float bv;
    long long bi;
    int win = 0;
    bool ok = tp_recv_max(mine, world, p.tp_max_items, item, epoch, p.tp_wait_ns, bv, bi, &win);
    const int s = item / p.B, b = item - s * p.B;
    if constexpr (LSE) {
      // the winner's logit from the rank that owns it, and the row's normaliser: the shards' partial
      // sums merged in rank order, so that every rank computes the same bits
      float logit = 0.f, m = -INFINITY, l = 0.f;
      TpRecord rec;
      if (ok) ok = tp_wait_record(p.tp_peers.slots[rank] + logit_region + ((size_t)parity * world + win) * p.tp_max_items + item,
                                  epoch, p.tp_wait_ns, rec);
      if (ok) logit = __uint_as_float(rec.val_bits);
      for (int r = 0; r < world && ok; ++r) {
        ok = tp_wait_record(p.tp_peers.slots[rank] + lse_parity + (size_t)r * kTpMaxRows + b, epoch, p.tp_wait_ns, rec);
        if (ok) lse_merge(m, l, __uint_as_float(rec.val_bits), __uint_as_float(rec.idx));
      }
      const float lse = ok ? lse_value(m, l) : __int_as_float(0x7fc00000);
      p.out_logprob[(size_t)b * p.S + s] = ok ? logit - lse : lse;
      if (s == 0 && p.out_lse) p.out_lse[b] = lse;
    }
    if (!ok) {
      if (p.status_dev) atomicExch(p.status_dev, kErrTimeout);
      bi = -1;
    }
    p.out_idx[(size_t)b * p.S + s] = bi;
    if (p.out_val) p.out_val[(size_t)b * p.S + s] = bv;
  }
  if (tid == 0) stamp(p, 7);
  if (p.status_mirror && p.status_dev) {
    sync();  // the receive loop above may have recorded a time-out
    if (tid == 0) *p.status_mirror = *reinterpret_cast<volatile int*>(p.status_dev);
  }
}

__host__ __device__ inline int gemv_dpad(int D, int chunks) {
  const int w = kGemvCols * chunks;
  return (D + w - 1) / w * w;
}

__host__ __device__ inline size_t gemv_smem_bytes(int NB, int D, int stages, int chunks) {
  return (size_t)stages * chunks * gemv_stage_bytes(NB) + (size_t)NB * gemv_dpad(D, chunks) * 2 +
         16 * (size_t)stages + kGemvConsumerWarps * 32 * 8 + 16 + 4 * (size_t)stages;
}

__device__ __forceinline__ float2 bf16x2_to_float2(uint32_t x) {
  return make_float2(__uint_as_float(x << 16), __uint_as_float(x & 0xffff0000u));
}

template <int NB, bool LSE = false>
__global__ void __launch_bounds__(kGemvThreads, 1)
gemv_sample_kernel(const __grid_constant__ CUtensorMap w_map, const SampleParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  constexpr int kGemvRowsPerWarp = gemv_rows_per_warp(NB);
  constexpr int kGemvRows = gemv_rows(NB);
  constexpr int kChunkBytes = gemv_stage_bytes(NB);  // one rows x 256-column chunk
  const int CK = p.gemv_chunks;                      // chunks per stage (CK > 1: the map is 3-D)
  const int kGemvStageBytes = CK * kChunkBytes;
  constexpr int kRowShift = (kGemvRowsPerWarp == 8) ? 3 : 2;
  // (row, b, s) results a lane may own: rows_per_warp * NB * S <= rows_per_warp * 32
  constexpr int kGemvItemsPerLane = kGemvRowsPerWarp;
  const int stages = p.stages;
  const int KC = ((p.D + kGemvCols - 1) / kGemvCols + CK - 1) / CK;  // pipeline steps per row group
  const int Dpad = KC * CK * kGemvCols;

  uint8_t* w_tiles = smem;
  __nv_bfloat16* hs = reinterpret_cast<__nv_bfloat16*>(smem + (size_t)stages * kGemvStageBytes);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(hs) + (size_t)NB * Dpad * 2);
  uint64_t* empty_bar = full_bar + stages;
  float* red_val = reinterpret_cast<float*>(empty_bar + stages);
  int* red_idx = reinterpret_cast<int*>(red_val + kGemvConsumerWarps * 32);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(red_idx + kGemvConsumerWarps * 32);
  volatile int* stage_group = abort_flag + 4;  // row group carried by each ring slot (-1: no more work)

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;

  // Work split: every CTA first walks a contiguous range holding 7/8 of its even share of the
  // 32(64)-row groups; the remaining groups form a pool that CTAs claim one at a time through an
  // atomic counter, which evens out the differences in the bandwidth individual SMs get.
  const int groups_total = (p.V + kGemvRows - 1) / kGemvRows;
  const int g_static = (int)(((long long)groups_total * 7 / 8) / (int)gridDim.x);
  const int cta = blockIdx.x;
  const int g_begin = cta * g_static;
  const int g_end = g_begin + g_static;
  const int pool_begin = (int)gridDim.x * g_static;

  if (tid == 0) {
    for (int i = 0; i < stages; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], kGemvConsumerWarps);
    }
    *abort_flag = 0;
    fence_mbar_init();
    stamp(p, 0);
  }
  // hidden states -> shared memory, zero padded to [NB][Dpad] (they may come from the kernel just before this one)
  griddep_wait();
  {
    const int chunks_per_row = Dpad / 8;
    const int d_chunks = p.D / 8;  // D % 8 == 0 is checked on the host
    for (int i = tid; i < NB * chunks_per_row; i += kGemvThreads) {
      const int b = i / chunks_per_row, c = i - b * chunks_per_row;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (b < p.B && c < d_chunks) v = *reinterpret_cast<const uint4*>(p.H + (size_t)b * p.D + c * 8);
      *reinterpret_cast<uint4*>(hs + (size_t)b * Dpad + c * 8) = v;
    }
  }
  __syncthreads();

  if (warp == kGemvConsumerWarps) {
    // ------------------------------ producer ------------------------------
    if (lane == 0) {
      prefetch_tmap(&w_map);
      const uint64_t pol = policy_evict_first();
      int it = 0;
      int g = g_begin < g_end ? g_begin : -1;
      int claimed = -1;  // pool group claimed ahead of time (the atomic's latency hides behind a group)
      bool from_pool = false;
      if (g < 0) {
        g = pool_begin + (int)atomicAdd(p.sched, 1u);
        from_pool = true;
      }
      while (g < groups_total && !*abort_flag) {
        // claim the next group before streaming this one
        int g_next;
        if (!from_pool && g + 1 < g_end) {
          g_next = g + 1;
        } else {
          claimed = pool_begin + (int)atomicAdd(p.sched, 1u);
          g_next = claimed;
        }
        for (int kc = 0; kc < KC; ++kc, ++it) {
          const int st = it % stages;
          const uint32_t n = (uint32_t)(it / stages);
          if (!mbar_wait(&empty_bar[st], (n & 1u) ^ 1u, abort_flag, p.status_dev)) break;
          stage_group[st] = g;
          mbar_arrive_expect_tx(&full_bar[st], kGemvStageBytes);
          if (CK == 1)
            tma_load_2d_hint(w_tiles + (size_t)st * kGemvStageBytes, &w_map, kc * kGemvCols, g * kGemvRows,
                             &full_bar[st], pol);
          else
            tma_load_3d_hint(w_tiles + (size_t)st * kGemvStageBytes, &w_map, 0, g * kGemvRows, kc * CK,
                             &full_bar[st], pol);
        }
        if (g_next == claimed) from_pool = true;
        g = g_next;
      }
      if (!*abort_flag) {
        // end marker: one more ring slot, no data
        const int st = it % stages;
        const uint32_t n = (uint32_t)(it / stages);
        if (mbar_wait(&empty_bar[st], (n & 1u) ^ 1u, abort_flag, p.status_dev)) {
          stage_group[st] = -1;
          mbar_arrive(&full_bar[st]);
        }
      }
      if (*abort_flag) {
        // A wait ran out somewhere: before the CTA may retire, give the copies that
        // are still in flight a bounded chance to land in shared memory.
        for (int st = 0; st < min(it, stages); ++st) {
          const int last_it = ((it - 1 - st) / stages) * stages + st;
          mbar_wait_plain(&full_bar[st], (uint32_t)(last_it / stages) & 1u, 100000000ull);
        }
      }
    }
    return;
  }

  // -------------------------------- consumers --------------------------------
  const bool greedy = (p.flags & kFlagGreedy) != 0;
  const bool ext = (p.flags & kFlagExtNoise) != 0;
  const bool ret_logits = (p.flags & kFlagReturnLogits) != 0;
  const int n_items = kGemvRowsPerWarp * NB * p.S;
  const unsigned long long seed = resolve_seed(p.seed, p.flags);

  // Lane l owns the items i = j * 32 + l (j < kGemvItemsPerLane) of the warp's
  // rows_per_warp x NB x S results: row r = i % rows_per_warp, then b, then s.  Only the running
  // best of each item lives in registers; the coordinates are recomputed when needed.
  float best_val[kGemvItemsPerLane];
  int best_idx[kGemvItemsPerLane];
#pragma unroll
  for (int j = 0; j < kGemvItemsPerLane; ++j) {
    best_val[j] = -INFINITY;
    best_idx[j] = kIdxNone;
  }
  // kFlagLogprob: running log-sum-exp of the items of draw 0 (one per vocabulary row and batch row)
  float lse_m[LSE ? kGemvItemsPerLane : 1], lse_l[LSE ? kGemvItemsPerLane : 1];
  if constexpr (LSE) {
#pragma unroll
    for (int j = 0; j < kGemvItemsPerLane; ++j) {
      lse_m[j] = -INFINITY;
      lse_l[j] = 0.f;
    }
  }

  int st = 0;          // ring slot of the next pipeline step and the parity of its "full" barrier (counted, not divided)
  uint32_t phase = 0;
  for (;;) {
    // the first ring slot of a group tells which group it is
    if (!mbar_wait(&full_bar[st], phase, abort_flag, p.status_dev)) break;
    const int g = stage_group[st];
    if (g < 0) break;
    float2 acc[kGemvRowsPerWarp][NB];
#pragma unroll
    for (int r = 0; r < kGemvRowsPerWarp; ++r)
#pragma unroll
      for (int b = 0; b < NB; ++b) acc[r][b] = make_float2(0.f, 0.f);

    for (int kc = 0; kc < KC; ++kc) {
      mbar_wait(&full_bar[st], phase, abort_flag, p.status_dev);

      for (int c = 0; c < CK; ++c) {
        float2 hreg[NB][4];
#pragma unroll
        for (int b = 0; b < NB; ++b) {
          const uint4 hv = *reinterpret_cast<const uint4*>(hs + (size_t)b * Dpad + (kc * CK + c) * kGemvCols + lane * 8);
          hreg[b][0] = bf16x2_to_float2(hv.x);
          hreg[b][1] = bf16x2_to_float2(hv.y);
          hreg[b][2] = bf16x2_to_float2(hv.z);
          hreg[b][3] = bf16x2_to_float2(hv.w);
        }
        const uint8_t* tile = w_tiles + (size_t)st * kGemvStageBytes + (size_t)c * kChunkBytes + (size_t)(warp * kGemvRowsPerWarp) * (kGemvCols * 2) + lane * 16;
#pragma unroll
        for (int r = 0; r < kGemvRowsPerWarp; ++r) {
          const uint4 wv = *reinterpret_cast<const uint4*>(tile + r * (kGemvCols * 2));
          const float2 w0 = bf16x2_to_float2(wv.x), w1 = bf16x2_to_float2(wv.y);
          const float2 w2 = bf16x2_to_float2(wv.z), w3 = bf16x2_to_float2(wv.w);
#pragma unroll
          for (int b = 0; b < NB; ++b) {
            float2 a = acc[r][b];
            a = __ffma2_rn(w0, hreg[b][0], a);
            a = __ffma2_rn(w1, hreg[b][1], a);
            a = __ffma2_rn(w2, hreg[b][2], a);
            a = __ffma2_rn(w3, hreg[b][3], a);
            acc[r][b] = a;
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[st]);
      if (++st == stages) {
        st = 0;
        phase ^= 1u;
      }
    }

    // warp-wide sums: every lane ends up with all 4 * NB logits of the warp's rows
    float sum[kGemvRowsPerWarp][NB];
#pragma unroll
    for (int r = 0; r < kGemvRowsPerWarp; ++r)
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        float x = acc[r][b].x + acc[r][b].y;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) x += __shfl_xor_sync(0xffffffffu, x, off);
        sum[r][b] = x;
      }

    const int v_warp = g * kGemvRows + warp * kGemvRowsPerWarp;
#pragma unroll
    for (int j = 0; j < kGemvItemsPerLane; ++j) {
      const int i = j * 32 + lane;
      const int item_r = i & (kGemvRowsPerWarp - 1);
      const int item_b = (i >> kRowShift) % NB;
      const int item_s = (i >> kRowShift) / NB;
      const int v = v_warp + item_r;
      if (i < n_items && item_b < p.B && v < p.V) {
        float val = 0.f;
#pragma unroll
        for (int r = 0; r < kGemvRowsPerWarp; ++r)
#pragma unroll
          for (int b = 0; b < NB; ++b)
            if (item_r == r && item_b == b) val = sum[r][b];
        if (ret_logits && item_s == 0) p.logits_out[(size_t)item_b * p.V + v] = val;
        float y;
        if (greedy) {
          y = val;
          if constexpr (LSE)
            if (item_s == 0) lse_push(lse_m[j], lse_l[j], val * kLog2e);
        } else {
          const float temp = p.temperature[(size_t)item_b * p.temp_stride];
          if constexpr (LSE)
            if (item_s == 0) lse_push(lse_m[j], lse_l[j], val * ((temp > 0.f ? 1.0f / temp : 1.0f) * kLog2e));
          if (temp <= 0.f) {
            y = val;  // temperature <= 0 selects greedy decoding for this row
          } else if (ext) {
            y = fmaf(val, 1.0f / temp, p.ext_noise[(size_t)item_s * p.noise_s_stride + (size_t)item_b * p.noise_ld + v]);
          } else {
            const unsigned long long vg = (unsigned long long)(p.v_offset + v);
            const uint4 q = noise_block(seed, item_s, item_b + p.b_offset, vg >> 2);
            y = fmaf(val, 1.0f / temp, gumbel_from_bits(pick_word(q, (uint32_t)vg & 3u)));
          }
        }
        if (y > best_val[j]) {
          best_val[j] = y;
          best_idx[j] = v;
        }
      }
    }
  }

  if (tid == 0) stamp(p, 5);
  // ---- CTA-level reduction of the running candidates: rows (shuffles), warps (smem) ----
#pragma unroll
  for (int j = 0; j < kGemvItemsPerLane; ++j) {
#pragma unroll
    for (int off = 1; off < kGemvRowsPerWarp; off <<= 1) {
      const float v2 = __shfl_xor_sync(0xffffffffu, best_val[j], off);
      const int i2 = __shfl_xor_sync(0xffffffffu, best_idx[j], off);
      cand_merge(best_val[j], best_idx[j], v2, i2);
    }
  }
  const int n_slots = NB * p.S;  // <= 32, slot = b + NB * s
#pragma unroll
  for (int j = 0; j < kGemvItemsPerLane; ++j) {
    const int i = j * 32 + lane;
    if ((i & (kGemvRowsPerWarp - 1)) == 0 && (i >> kRowShift) < n_slots) {
      red_val[warp * 32 + (i >> kRowShift)] = best_val[j];
      red_idx[warp * 32 + (i >> kRowShift)] = best_idx[j];
    }
  }
  asm volatile("bar.sync 1, %0;" ::"r"(kGemvConsumerWarps * 32) : "memory");
  if (tid < n_slots) {
    float bv = red_val[tid];
    int bi = red_idx[tid];
#pragma unroll
    for (int w = 1; w < kGemvConsumerWarps; ++w) cand_merge(bv, bi, red_val[w * 32 + tid], red_idx[w * 32 + tid]);
    const int b = tid % NB, s = tid / NB;
    if (b < p.B && bi != kIdxNone) atomicMax(&p.keys[(size_t)s * p.B + b], cand_key(bv, bi));
  }
  if constexpr (LSE) {
    // the same two steps for the log-sum-exp of draw 0: rows of a warp by shuffles, then warps
#pragma unroll
    for (int j = 0; j < kGemvItemsPerLane; ++j) {
#pragma unroll
      for (int off = 1; off < kGemvRowsPerWarp; off <<= 1) {
        const float m2 = __shfl_xor_sync(0xffffffffu, lse_m[j], off);
        const float l2 = __shfl_xor_sync(0xffffffffu, lse_l[j], off);
        lse_merge(lse_m[j], lse_l[j], m2, l2);
      }
    }
    asm volatile("bar.sync 1, %0;" ::"r"(kGemvConsumerWarps * 32) : "memory");  // red_* have been read
    float* red_l = reinterpret_cast<float*>(red_idx);
#pragma unroll
    for (int j = 0; j < kGemvItemsPerLane; ++j) {
      const int i = j * 32 + lane;
      if ((i & (kGemvRowsPerWarp - 1)) == 0 && (i >> kRowShift) < NB) {  // slots of draw 0: slot = b
        red_val[warp * 32 + (i >> kRowShift)] = lse_m[j];
        red_l[warp * 32 + (i >> kRowShift)] = lse_l[j];
      }
    }
    asm volatile("bar.sync 1, %0;" ::"r"(kGemvConsumerWarps * 32) : "memory");
    if (tid < NB && tid < p.B) {
      float m = red_val[tid], l = red_l[tid];
#pragma unroll
      for (int w = 1; w < kGemvConsumerWarps; ++w) lse_merge(m, l, red_val[w * 32 + tid], red_l[w * 32 + tid]);
      p.lse[(size_t)blockIdx.x * p.B + tid] = lse_pack(m, l);  // this CTA's partial row
    }
  }
  if (!(p.flags & kFlagTwoStage)) {
    volatile int* is_last = abort_flag + 1;
    finish_sample<LSE>(
        p, tid, kGemvConsumerWarps * 32,
        [] { asm volatile("bar.sync 1, %0;" ::"r"(kGemvConsumerWarps * 32) : "memory"); }, is_last);
  }
}

// ---------------------------------------------------------------------------------
// Stand-alone second stage (FMMS_FLAG_TWO_STAGE): the sampling kernel only merges its
// candidates into p.keys; this kernel decodes the winners and clears the keys.
// ---------------------------------------------------------------------------------
__global__ void reduce_candidates_kernel(unsigned long long* __restrict__ keys, unsigned int* __restrict__ sched,
                                         int B, int S, long long v_offset, long long* __restrict__ out_idx,
                                         float* __restrict__ out_val) {
  const int item = blockIdx.x * blockDim.x + threadIdx.x;  // s * B + b
  if (item == 0) *sched = 0u;  // the sampling kernel's dynamic work counter
  if (item >= B * S) return;
  const unsigned long long k = keys[item];
  keys[item] = 0ull;
  float v;
  int idx;
  cand_key_decode(k, v, idx);
  const int s = item / B, b = item - s * B;
  out_idx[(size_t)b * S + s] = v_offset + idx;
  if (out_val) out_val[(size_t)b * S + s] = v;
}

}  // namespace fmms
