// Tensor-core kernel for 129..256 batch rows: CTA pairs (clusters of two) and tcgen05.mma
// cta_group::2.
//
// One MMA spans both SMs of a pair: M = 256 batch rows (128 TMEM lanes in each CTA), N = the
// vocabulary tile (up to 256 columns in each CTA's TMEM).  Each CTA loads only ITS half of the
// W tile (NT/2 rows) and ITS 128 hidden-state rows, so per streamed W byte the pair moves half
// the hidden-state bytes and reads fewer shared-memory operand bytes than the single-CTA kernel
// with two M tiles, and its accumulators stay double-buffered.  At 256 rows the step is bound by
// the tensor pipe (2*V*D*256 flop); measured on the Qwen head 269 us against 300 us for the
// two-M-tile kernel, tensor pipe 57 % against 50 % active.  The leader CTA (rank 0) issues every MMA; completion is signalled to both CTAs
// with one tcgen05.commit per CTA.  Loads are ordinary (non-multicast) TMA operations whose
// transaction bytes are counted on the leader's mbarrier.  Epilogue, candidate keys and the tail
// are those of the single-CTA kernel: each CTA scans its own 128 rows.
#pragma once

#include <cuda.h>

#include "fmms_common.cuh"
#include "fmms_gemv.cuh"
#include "fmms_umma.cuh"

namespace fmms {

constexpr int kPairUnitRows = 32;  // vocabulary granule of a pair tile (16 rows per CTA)

struct PairPlan {
  int grid;           // CTAs (even)
  int units_total;    // ceil(V / 32)
  int tiles_per_pair;
  int q_units;        // tiles are q_units or q_units - 1 granules high
  int slabs, stages;
  size_t smem;
};

__host__ __device__ inline size_t pair_stage_bytes(int q_units, int slabs) {
  return (size_t)slabs * ((size_t)q_units * 16 * 128 + (size_t)kUmmaHTileMax);
}

__host__ inline PairPlan pair_plan(int V, int D, int num_sms, int max_smem, int slabs_force = 0) {
  PairPlan pl{};
  pl.units_total = (V + kPairUnitRows - 1) / kPairUnitRows;
  int pairs = num_sms / 2;
  if (pairs > pl.units_total) pairs = pl.units_total;
  pl.grid = pairs * 2;
  const int u_max = (pl.units_total + pairs - 1) / pairs;
  pl.tiles_per_pair = (u_max + 7) / 8;  // at most 256 rows per tile
  pl.q_units = (u_max + pl.tiles_per_pair - 1) / pl.tiles_per_pair;
  const size_t fixed = 1024 + 1024;
  int sk = slabs_force > 0 ? slabs_force : 2;
  if (sk > D / 64) sk = D / 64;
  if (sk < 1) sk = 1;
  while (sk > 1 && 3 * pair_stage_bytes(pl.q_units, sk) + fixed > (size_t)max_smem) --sk;
  pl.slabs = sk;
  int stages = kUmmaMaxStages;
  while (stages > 2 && stages * pair_stage_bytes(pl.q_units, sk) + fixed > (size_t)max_smem) --stages;
  pl.stages = stages;
  pl.smem = stages * pair_stage_bytes(pl.q_units, sk) + fixed;
  return pl;
}

// ---- cluster helpers ------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t mapa_shared(uint32_t saddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx_remote(uint32_t cluster_addr, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(cluster_addr), "r"(bytes)
               : "memory");
}
// 3-D tiled TMA load of a CTA pair: data into this CTA's shared memory, bytes counted on the
// mbarrier at cluster address `bar_cluster_addr` (the leader's).
__device__ __forceinline__ void tma_pair_load_3d(void* smem_dst, const void* tmap, int x, int y, int z,
                                                 uint32_t bar_cluster_addr, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1, {%2, %3, %4}], [%5], %6;" ::"r"(smem_u32(smem_dst)),
      "l"(tmap), "r"(x), "r"(y), "r"(z), "r"(bar_cluster_addr), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_pair_commit(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr)
               : "memory");
}
__device__ __forceinline__ void umma_pair_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_pair_e4m3(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
      "}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// fp32 accumulate, bf16 x bf16 (or e4m3 x e4m3: format code 0 of kind::f8f6f4), both K-major, M = 256 (128 rows in
// each CTA of the pair)
__host__ __device__ inline uint32_t umma_pair_idesc(int n, bool fp8 = false) {
  const uint32_t fmt = fp8 ? 0u : ((1u << 7) | (1u << 10));
  return (1u << 4) | fmt | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}

// Tile schedule of one pair: granules of 32 rows, T near-equal tiles (see TileWalk).
struct PairWalk {
  int u_next, base, extra, i;
  __device__ __forceinline__ PairWalk(int units_total, int T) {
    const int pairs = (int)gridDim.x / 2, c = (int)blockIdx.x / 2;
    const int per = units_total / pairs, rem = units_total % pairs;
    const int u_cnt = per + (c < rem ? 1 : 0);
    u_next = c * per + min(c, rem);
    base = u_cnt / T;
    extra = u_cnt % T;
    i = 0;
  }
  __device__ __forceinline__ void next(int& v0, int& nt) {
    const int units = base + (i < extra ? 1 : 0);
    v0 = u_next * kPairUnitRows;
    nt = units * kPairUnitRows;
    u_next += units;
    ++i;
  }
};

template <bool LSE = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kUmmaThreads, 1)
umma_pair_sample_kernel(const __grid_constant__ CUtensorMap w_map_q, const __grid_constant__ CUtensorMap w_map_q1,
                        const __grid_constant__ CUtensorMap h_map, const SampleParams p, const int units_total,
                        const int q_units, const int SK) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int stages = p.stages;
  const int n_tiles = p.tiles_per_cta;
  constexpr int nt_cap = 256, acc_stages = 2;
  // stage = [SK half-W slabs (q_units * 16 rows)][SK hidden-state slabs (128 rows)]
  const size_t w_slab_cap = (size_t)q_units * 16 * 128, h_slab_bytes = kUmmaHTileMax;
  const size_t w_tile_bytes = SK * w_slab_cap;
  const size_t stage_bytes = w_tile_bytes + SK * h_slab_bytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem);
  smem += 1024;
  uint64_t* empty_bar = full_bar + stages;
  uint64_t* acc_full = empty_bar + stages;
  uint64_t* acc_empty = acc_full + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const bool leader = rank == 0;
  const int KB = (p.D / kUmmaBK + SK - 1) / SK;  // D % 64 == 0 is required by the launcher
  const int cta = blockIdx.x;

  if (tid == 0) {
    for (int i = 0; i < stages; ++i) {
      mbar_init(&full_bar[i], 4);   // W and hidden-state producers of both CTAs (used in the leader)
      mbar_init(&empty_bar[i], 1);  // one commit per CTA
    }
    for (int i = 0; i < 4; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 2 * kUmmaEpiWarps);  // epilogue warps of both CTAs (used in the leader)
    }
    *abort_flag = 0;
    fence_mbar_init();
    stamp(p, 0);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, kTmemCols);
    tmem_relinquish_pair();
  }
  if (p.S > 1) {
    const int n = kUmmaEpiGroups * p.S * p.B;
    float* cv = p.cand_val + (size_t)cta * n;
    int* ci = p.cand_idx + (size_t)cta * n;
    for (int i = tid; i < n; i += kUmmaThreads) {
      cv[i] = -INFINITY;
      ci[i] = kIdxNone;
    }
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anyone signals across the pair
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (tid == 0) stamp(p, 1);

  if (warp == 0 || warp == 2) {
    // ------------------------------ TMA producers (both CTAs) -----------------------------
    if (lane == 0) {
      const bool is_w = (warp == 0);
      if (is_w) {
        prefetch_tmap(&w_map_q);
        prefetch_tmap(&w_map_q1);
      } else {
        prefetch_tmap(&h_map);
      }
      const uint64_t pol = is_w ? policy_evict_first() : policy_evict_last();
      if (!is_w) griddep_wait();  // the hidden states may come from the kernel just before this one
      int st = 0;          // ring slot of the next K step and the parity of its "empty" barrier (no divisions here)
      uint32_t phase = 1;
      bool ok = true;
      PairWalk walk(units_total, n_tiles);
      for (int t = 0; t < n_tiles && ok; ++t) {
        int v0, NT;
        walk.next(v0, NT);
        if (NT == 0) continue;
        const int half = NT / 2;
        const uint32_t tx = (uint32_t)SK * (is_w ? (uint32_t)half * 128u : (uint32_t)h_slab_bytes);
        const CUtensorMap* wm = (NT == q_units * kPairUnitRows) ? &w_map_q : &w_map_q1;
        for (int kb = 0; kb < KB; ++kb) {
          if (!mbar_wait(&empty_bar[st], phase, abort_flag, p.status_dev)) {
            ok = false;
            break;
          }
          uint8_t* sw = smem + st * stage_bytes;
          const uint32_t bar = mapa_shared(smem_u32(&full_bar[st]), 0);  // the leader's barrier
          mbar_arrive_expect_tx_remote(bar, tx);
          if (is_w)
            tma_pair_load_3d(sw, wm, 0, v0 + (int)rank * half, kb * SK, bar, pol);
          else
            tma_pair_load_3d(sw + w_tile_bytes, &h_map, 0, (int)rank * 128, kb * SK, bar, pol);
          if (++st == stages) {
            st = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA only) --------------------------
    if (leader && lane == 0) {
      // the loop between two tcgen05.mma is kept free of divisions: ring slot, parity and accumulator buffer are counted
      int st = 0, j = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool first = true;
      bool ok = true;
      const uint32_t smem0 = smem_u32(smem);
      const bool fp8 = (p.flags & kFlagFp8) != 0;
      PairWalk walk(units_total, n_tiles);
      for (int t = 0; t < n_tiles && ok; ++t) {
        int v0, NT;
        walk.next(v0, NT);
        if (NT == 0) continue;
        const uint32_t idesc = umma_pair_idesc(NT, fp8);
        const uint32_t w_pitch = (uint32_t)((NT / 2) * 128);
        if (!mbar_wait(&acc_empty[j], acc_phase ^ 1u, abort_flag, p.status_dev)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(j * nt_cap);
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
            const uint64_t bdesc = umma_smem_desc(sw + (uint32_t)sl * w_pitch);
            const uint64_t adesc = umma_smem_desc(sw + (uint32_t)(w_tile_bytes + sl * h_slab_bytes));
            // both descriptors advance by 16 bf16 (32 e4m3) = 32 bytes inside the swizzled row
            if (fp8) {
              umma_pair_e4m3(d_tmem, adesc, bdesc, idesc, (kb | sl) != 0 ? 1u : 0u);
              umma_pair_e4m3(d_tmem, adesc + 2, bdesc + 2, idesc, 1u);
              umma_pair_e4m3(d_tmem, adesc + 4, bdesc + 4, idesc, 1u);
              umma_pair_e4m3(d_tmem, adesc + 6, bdesc + 6, idesc, 1u);
            } else {
              umma_pair_bf16(d_tmem, adesc, bdesc, idesc, (kb | sl) != 0 ? 1u : 0u);
              umma_pair_bf16(d_tmem, adesc + 2, bdesc + 2, idesc, 1u);
              umma_pair_bf16(d_tmem, adesc + 4, bdesc + 4, idesc, 1u);
              umma_pair_bf16(d_tmem, adesc + 6, bdesc + 6, idesc, 1u);
            }
          }
          // the stage is free in BOTH CTAs once these MMAs have read it
          umma_pair_commit(smem_u32(&empty_bar[st]));
          umma_pair_commit(mapa_shared(smem_u32(&empty_bar[st]), 1));
          if (++st == stages) {
            st = 0;
            phase ^= 1u;
          }
        }
        if (ok) {
          umma_pair_commit(smem_u32(&acc_full[j]));
          umma_pair_commit(mapa_shared(smem_u32(&acc_full[j]), 1));
        }
        if (++j == acc_stages) {
          j = 0;
          acc_phase ^= 1u;
        }
      }
      stamp(p, 3);
    }
  } else if (warp >= kUmmaEpiWarp0) {
    // -------------------------------- epilogue (both CTAs) --------------------------------
    griddep_wait();  // temperatures may come from the kernel just before this one
    const int ew = warp - kUmmaEpiWarp0;
    const int wg = ew >> 2;
    const int quad = warp & 3;
    const int b = (int)rank * 128 + quad * 32 + lane;
    const bool row_ok = b < p.B;
    const bool warp_ok = ((int)rank * 128 + quad * 32) < p.B;
    const bool greedy = (p.flags & kFlagGreedy) != 0;
    float invT = 1.0f;
    bool noisy = true;
    if (row_ok && !greedy) {
      const float temp = p.temperature[(size_t)b * p.temp_stride];
      noisy = temp > 0.f;
      invT = noisy ? 1.0f / temp : 1.0f;
    }
    EpiRow row{b, row_ok, greedy, (p.flags & kFlagExtNoise) != 0, (p.flags & kFlagReturnLogits) != 0,
               (p.v_offset & 3) == 0, invT, noisy, resolve_seed(p.seed, p.flags)};
    if (p.flags & kFlagFp8) {  // e4m3 operands: the accumulator is rescaled per vocabulary row and batch row
      row.w_scale = p.w_scale;
      row.h_scale = row_ok ? p.h_scale[b] : 1.f;
    }
    const int S = p.S;
    const size_t slot_row = ((size_t)cta * kUmmaEpiGroups + wg) * ((size_t)S * p.B);
    float best_val = -INFINITY;
    int best_idx = kIdxNone;
    float lse_m = -INFINITY, lse_l = 0.f;  // kFlagLogprob: this thread's share of the row's log-sum-exp

    PairWalk walk(units_total, n_tiles);
    for (int t = 0, ta = 0; t < n_tiles; ++t) {
      int v0, NT;
      walk.next(v0, NT);
      if (NT == 0) continue;
      const int chunks = (NT + 31) / 32;
      const int per_group = (chunks + kUmmaEpiGroups - 1) / kUmmaEpiGroups;
      const int c_begin = min(wg * per_group * 32, NT);
      const int c_end = min(c_begin + per_group * 32, NT);
      const int j = ta % acc_stages;
      const uint32_t un = (uint32_t)(ta / acc_stages);
      ++ta;
      if (!mbar_wait(&acc_full[j], un & 1u, abort_flag, p.status_dev)) break;
      tc_fence_after();
      if (ew == 0 && lane == 0 && t == n_tiles - 1) stamp(p, 4);
      if (warp_ok) {
        const uint32_t t_addr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(j * nt_cap);
        if constexpr (LSE) lse_tile_columns(p, row, t_addr, c_begin, c_end, v0, lse_m, lse_l);
        for (int s = 0; s < S; ++s) {
          float bv = best_val;
          int bi = best_idx;
          if (S > 1) {
            bv = -INFINITY;
            bi = kIdxNone;
          }
          scan_tile_columns(p, row, t_addr, c_begin, c_end, v0, s, bv, bi);
          if (S > 1) {
            if (row_ok) {
              const size_t o = slot_row + (size_t)s * p.B + b;
              if (bv > p.cand_val[o]) {
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
      if (lane == 0) mbar_arrive_remote(mapa_shared(smem_u32(&acc_empty[j]), 0));
    }
    if (ew == 0 && lane == 0) stamp(p, 5);
    if (row_ok) {
      if (S == 1) {
        if (best_idx != kIdxNone) atomicMax(&p.keys[b], cand_key(best_val, best_idx));
      } else {
        for (int s = 0; s < S; ++s) {
          const size_t o = slot_row + (size_t)s * p.B + b;
          const int ci = p.cand_idx[o];
          if (ci != kIdxNone) atomicMax(&p.keys[(size_t)s * p.B + b], cand_key(p.cand_val[o], ci));
        }
      }
      // every tile has been multiplied, so the pipeline's first stage is free: it collects the
      // warpgroups' partial sums of this CTA's 128 rows
      if constexpr (LSE)
        reinterpret_cast<unsigned long long*>(smem)[wg * 128 + quad * 32 + lane] = lse_pack(lse_m, lse_l);
    }
  }

  griddep_wait();
  tc_fence_before();
  __threadfence();
  __syncthreads();
  cluster_sync_all();  // the peer has stopped reading TMEM and signalling this CTA's barriers
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
  if constexpr (LSE) {
    // one partial row per CTA pair: each CTA fills in its own 128 batch rows
    const unsigned long long* part = reinterpret_cast<const unsigned long long*>(smem);
    for (int r = tid; r < 128; r += kUmmaThreads) {
      const int b = (int)rank * 128 + r;
      if (b >= p.B) continue;
      float m = -INFINITY, l = 0.f;
#pragma unroll
      for (int g = 0; g < kUmmaEpiGroups; ++g) lse_merge_packed(m, l, part[g * 128 + r]);
      p.lse[(size_t)(cta >> 1) * p.B + b] = lse_pack(m, l);
    }
  }
  if (!(p.flags & kFlagTwoStage)) {
    volatile int* is_last = abort_flag + 1;
    finish_sample<LSE>(p, tid, kUmmaThreads, [] { __syncthreads(); }, is_last, /*fenced_and_synced=*/!LSE);
  }
}

}  // namespace fmms
