// Top-k / top-p sampling from the fused pass.
//
// The reference restricts sampling to the k largest logits of a row (and, with top-p, to the
// smallest prefix of them whose softmax mass reaches p) by writing a top-k list per vocabulary
// tile to memory and merging the lists afterwards (tl_fused_mm_topk.py:25-107).  Here the
// tensor-core pass itself filters: only logits at or above the row's pivot, a running lower bound
// of its k-th largest logit, are kept (see the epilogue of umma_sample_kernel), typically ~1e3 of
// the 1.5e5 entries of a row, each epilogue thread in a segment of its own.  The kernels in this
// file finish the rows:
//
//   topk_finish_kernel   one CTA per row: gather the row's candidates, keep the k largest, apply the
//                        temperature-scaled softmax and the nucleus mask, and draw every sample as
//                        a Gumbel-max over the surviving ids with the SAME noise stream as the
//                        unrestricted sampler (noise keyed by seed, draw, row and global id), so a
//                        restricted draw equals the unrestricted one whenever that one survives.
//   topk_exact_kernel    rows that overflowed (logits rising steadily over the vocabulary defeat any
//                        running bound): exact radix selection over the row's full logits, which a
//                        conditional second pass has written to scratch memory.
//   topk_overflow_kernel the same rows when the caller gave no scratch for that second pass: the
//                        ids become -1 and the status word reports it.
#pragma once

#include "fmms_common.cuh"
#include "fmms_gemv.cuh"  // SampleParams

namespace fmms {

constexpr int kTopkFinishThreads = 256;
constexpr int kTopkExactThreads = 1024;
constexpr int kErrTopkOverflow = 8;  // FMMS_ERR_TOPK_OVERFLOW

// Shared result of the selection step of one row.
struct TopkRowShared {
  float z[kTopkSlots];  // scaled logits of the kept candidates, descending
  int id[kTopkSlots];   // their local vocabulary ids
  int allowed;          // candidates that survive top-k and top-p
  float lse;            // natural-log normaliser over the survivors
};

// In-place bitonic sort, descending, of n (a power of two) 64-bit keys in shared memory.
__device__ __forceinline__ void bitonic_sort_desc(unsigned long long* keys, int n, int tid, int nthreads) {
  for (int size = 2; size <= n; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      __syncthreads();
      for (int i = tid; i < (n >> 1); i += nthreads) {
        const int lo = 2 * i - (i & (stride - 1));
        const int hi = lo + stride;
        const bool desc = ((lo & size) == 0);
        const unsigned long long a = keys[lo], c = keys[hi];
        if ((a < c) == desc) {
          keys[lo] = c;
          keys[hi] = a;
        }
      }
    }
  }
  __syncthreads();
}

// Given the row's candidates sorted descending (at least min(k, n) valid ones first), compute the
// survivors and draw the row's S samples.  Called by every thread of the CTA.
__device__ __forceinline__ void topk_finish_row(const SampleParams& p, int b, const unsigned long long* sorted, int n,
                                                TopkRowShared* sh, int tid, int nthreads) {
  const int kk = min(p.topk.k, n);
  const bool greedy_flag = (p.flags & kFlagGreedy) != 0;
  float temp = 1.f;
  if (!greedy_flag) temp = p.temperature[(size_t)b * p.temp_stride];
  const bool noisy = !greedy_flag && temp > 0.f;
  if (tid < 32) {
    // softmax over the kk largest (two per lane), inclusive prefix sums in rank order, nucleus mask
    const int i0 = tid, i1 = tid + 32;
    float z0 = -INFINITY, z1 = -INFINITY;
    int id0 = 0, id1 = 0;
    if (i0 < kk) cand_key_decode(sorted[i0], z0, id0);
    if (i1 < kk) cand_key_decode(sorted[i1], z1, id1);
    const float zmax = __shfl_sync(0xffffffffu, z0, 0);
    const float e0 = i0 < kk ? __expf(z0 - zmax) : 0.f, e1 = i1 < kk ? __expf(z1 - zmax) : 0.f;
    float s0 = e0, s1 = e1;  // inclusive scans over lanes
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const float a = __shfl_up_sync(0xffffffffu, s0, off), c = __shfl_up_sync(0xffffffffu, s1, off);
      if (tid >= off) {
        s0 += a;
        s1 += c;
      }
    }
    const float first32 = __shfl_sync(0xffffffffu, s0, 31);
    s1 += first32;
    const float total = __shfl_sync(0xffffffffu, s1, 31);
    bool keep0 = i0 < kk, keep1 = i1 < kk;
    if (p.topk.top_p > 0.f && p.topk.top_p < 1.f) {
      // keep rank i while the mass BEFORE it is below top_p; rank 0 always stays (tl_fused_mm_topk.py:93-96)
      const float lim = p.topk.top_p * total;
      keep0 = keep0 && (i0 == 0 || (s0 - e0) < lim);
      keep1 = keep1 && ((s1 - e1) < lim);
    }
    if (!noisy) {  // greedy row: the largest logit alone
      keep0 = keep0 && i0 == 0;
      keep1 = false;
    }
    const int a = __popc(__ballot_sync(0xffffffffu, keep0)) + __popc(__ballot_sync(0xffffffffu, keep1));
    // mass of the survivors (a prefix of the ranks)
    float kept = (keep0 ? e0 : 0.f) + (keep1 ? e1 : 0.f);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) kept += __shfl_xor_sync(0xffffffffu, kept, off);
    sh->z[i0] = z0;
    sh->z[i1] = z1;
    sh->id[i0] = id0;
    sh->id[i1] = id1;
    if (tid == 0) {
      sh->allowed = a;
      sh->lse = zmax + __logf(kept);
    }
  }
  __syncthreads();
  const int a = sh->allowed;
  const unsigned long long seed = resolve_seed(p.seed, p.flags);
  const bool ext = (p.flags & kFlagExtNoise) != 0;
  if (p.S < nthreads) {
    // few draws: one warp per draw, the candidates spread over its lanes
    const int lane = tid & 31;
    for (int s = tid >> 5; s < p.S; s += nthreads >> 5) {
      float best = -INFINITY, best_z = 0.f;
      int best_id = 0x7fffffff;
      for (int i = lane; i < a; i += 32) {
        const float z = sh->z[i];
        const int id = sh->id[i];
        float g = 0.f;
        if (noisy) {
          if (ext) {
            g = p.ext_noise[(size_t)s * p.noise_s_stride + (size_t)b * p.noise_ld + id];
          } else {
            const unsigned long long vg = (unsigned long long)(p.v_offset + id);
            const uint4 q = noise_block(seed, s, b + p.b_offset, vg >> 2);
            g = gumbel_from_bits(pick_word(q, (uint32_t)vg & 3u));
          }
        }
        const float y = z + g;
        if (y > best) {  // ranks ascend within a lane: equal values keep the more probable candidate
          best = y;
          best_z = z;
          best_id = id;
        }
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) {
        const float y2 = __shfl_xor_sync(0xffffffffu, best, off), z2 = __shfl_xor_sync(0xffffffffu, best_z, off);
        const int id2 = __shfl_xor_sync(0xffffffffu, best_id, off);
        if (y2 > best || (y2 == best && id2 < best_id)) {
          best = y2;
          best_z = z2;
          best_id = id2;
        }
      }
      if (lane == 0) {
        const size_t o = (size_t)b * p.S + s;
        p.out_idx[o] = a > 0 ? p.v_offset + best_id : -1;
        if (p.out_val) p.out_val[o] = best;
        if (p.out_logprob) p.out_logprob[o] = best_z - sh->lse;
      }
    }
    if (tid == 0 && p.out_lse) p.out_lse[b] = sh->lse;
    return;
  }
  for (int s = tid; s < p.S; s += nthreads) {
    float best = -INFINITY, best_z = 0.f;
    int best_id = 0;
    for (int i = 0; i < a; ++i) {
      const float z = sh->z[i];
      const int id = sh->id[i];
      float g = 0.f;
      if (noisy) {
        if (ext) {
          g = p.ext_noise[(size_t)s * p.noise_s_stride + (size_t)b * p.noise_ld + id];
        } else {
          const unsigned long long vg = (unsigned long long)(p.v_offset + id);
          const uint4 q = noise_block(seed, s, b + p.b_offset, vg >> 2);
          g = gumbel_from_bits(pick_word(q, (uint32_t)vg & 3u));
        }
      }
      const float y = z + g;
      if (y > best) {
        best = y;
        best_z = z;
        best_id = id;
      }
    }
    const size_t o = (size_t)b * p.S + s;
    p.out_idx[o] = a > 0 ? p.v_offset + best_id : -1;
    if (p.out_val) p.out_val[o] = best;
    if (p.out_logprob) p.out_logprob[o] = best_z - sh->lse;
  }
  if (tid == 0 && p.out_lse) p.out_lse[b] = sh->lse;
}

// Count `bin` in a shared-memory histogram for the lanes with `in` set.  Lanes of a warp that hit the
// same bin are merged into one atomic: the logits of a row share a few exponents, so the first
// radix step would otherwise send almost every element to the same three or four counters.  All 32
// lanes of the warp must call this together.
__device__ __forceinline__ void hist_add_merged(unsigned int* hist, uint32_t bin, bool in) {
  const unsigned int peers = __match_any_sync(0xffffffffu, in ? bin : 0xffffffffu);
  if (in && (int)(threadIdx.x & 31) == __ffs(peers) - 1) atomicAdd(&hist[bin], (unsigned int)__popc(peers));
}

// The 32-bit value key of the k-th largest of n packed candidates (radix selection
// over the value halves: 11 + 11 + 10 bits, one 2048-bin histogram per step), and how many
// candidates equal to it belong to the k largest.  Called by every thread of a CTA of at least 256
// threads; 1 <= k <= n.
__device__ __forceinline__ void select_kth_key(const unsigned long long* keys, int n, int k, unsigned int* hist,
                                               unsigned int* warp_sums, unsigned int* sh_prefix, unsigned int* sh_need,
                                               int tid, int nthreads, uint32_t& tau, unsigned int& need_eq) {
  if (tid == 0) {
    *sh_prefix = 0u;
    *sh_need = (unsigned int)k;
  }
  uint32_t mask = 0u;
  const int shifts[3] = {21, 10, 0}, bits[3] = {11, 11, 10};
  for (int pass = 0; pass < 3; ++pass) {
    for (int i = tid; i < 2048; i += nthreads) hist[i] = 0u;
    __syncthreads();
    const uint32_t prefix = *sh_prefix, binmask = (1u << bits[pass]) - 1u;
    for (int base = 0; base < n; base += nthreads) {  // whole warps stay together for the merged count
      const int i = base + tid;
      const uint32_t key = i < n ? (uint32_t)(keys[i] >> 32) : 0u;
      hist_add_merged(hist, (key >> shifts[pass]) & binmask, i < n && (key & mask) == prefix);
    }
    __syncthreads();
    {
      // Which bin holds the `need`-th largest?  Thread t sums bins [hi - 8t - 7, hi - 8t] (from the top),
      // a block-wide inclusive scan of those sums finds the thread whose share crosses `need`, and that
      // thread walks its eight bins.  (2048 bins = 256 threads x 8; fewer bins leave the upper threads idle.)
      const unsigned int need = *sh_need;
      const int hi = (int)binmask;
      unsigned int mine = 0;
      if (tid < 256) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int bin = hi - 8 * tid - j;
          if (bin >= 0) mine += hist[bin];
        }
      }
      unsigned int incl = mine;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const unsigned int v = __shfl_up_sync(0xffffffffu, incl, off);
        if ((tid & 31) >= off) incl += v;
      }
      if ((tid & 31) == 31 && tid < 256) warp_sums[tid >> 5] = incl;
      __syncthreads();
      if (tid < 256) {
        unsigned int before = incl - mine;
        for (int w = 0; w < (tid >> 5); ++w) before += warp_sums[w];
        if (before < need && before + mine >= need) {  // exactly one thread (or none: fewer than `need` entries)
          unsigned int cum = before;
          int bin = hi - 8 * tid;
          for (int j = 0; j < 8 && bin - j >= 0; ++j) {
            if (cum + hist[bin - j] >= need) {
              *sh_need = need - cum;
              *sh_prefix = prefix | ((uint32_t)(bin - j) << shifts[pass]);
              break;
            }
            cum += hist[bin - j];
          }
        }
      }
    }
    mask |= binmask << shifts[pass];
    __syncthreads();
  }
  tau = *sh_prefix;
  need_eq = *sh_need;
}

// One CTA per batch row.  Dynamic shared memory: kTopkListCap keys.
__global__ void __launch_bounds__(kTopkFinishThreads) topk_finish_kernel(const SampleParams p) {
  griddep_wait();  // launched behind its producer with programmatic stream serialisation
  extern __shared__ unsigned long long topk_keys[];
  __shared__ unsigned int hist[2048];
  __shared__ unsigned long long picked[2 * kTopkSlots];
  __shared__ unsigned int sh_prefix, sh_need, sh_count, sh_total, sh_overflow, warp_sums[8];
  __shared__ TopkRowShared sh;
  const int b = blockIdx.x, tid = threadIdx.x;
  if (tid == 0) {
    sh_total = 0u;
    sh_overflow = 0u;
    sh_count = 0u;
  }
  for (int i = tid; i < 2 * kTopkSlots; i += kTopkFinishThreads) picked[i] = 0ull;
  __syncthreads();
  // gather the row's candidates from the segments the epilogue threads filled (order does not matter)
  const unsigned int* counts = p.topk.seg_count + (size_t)b * kTopkMaxSegs;
  const unsigned long long* segs = p.topk.list + (size_t)b * kTopkMaxSegs * kTopkSegCap;
  for (int sg = tid; sg < p.topk.nseg; sg += kTopkFinishThreads) {
    const unsigned int n = min(counts[sg], (unsigned int)kTopkSegCap);  // what did not fit is in the spill list
    if (n) {
      const unsigned int pos = atomicAdd(&sh_total, n);
      for (unsigned int i = 0; i < n; ++i)
        if (pos + i < (unsigned int)kTopkListCap) topk_keys[pos + i] = segs[(size_t)sg * kTopkSegCap + i];
    }
  }
  __syncthreads();
  {
    // the row's spill list: entries of threads whose segments were full
    const unsigned int ex = p.topk.extra_count[b], base = sh_total;
    const unsigned long long* extra = p.topk.extra + (size_t)b * kTopkExtraCap;
    for (unsigned int i = tid; i < min(ex, (unsigned int)kTopkExtraCap); i += kTopkFinishThreads)
      if (base + i < (unsigned int)kTopkListCap) topk_keys[base + i] = extra[i];
    __syncthreads();
    if (tid == 0) {
      if (ex > (unsigned int)kTopkExtraCap) sh_overflow = 1u;
      sh_total = base + ex;
      p.topk.extra_count[b] = 0u;  // as the next call expects it
    }
    __syncthreads();
  }
  if (sh_overflow || sh_total > (unsigned int)kTopkListCap) {
    // the running bound did not keep up with this row (more candidates than the lists hold): leave it to the
    // exact pass
    if (tid == 0) {
      p.topk.row_fallback[b] = 1;
      atomicExch(p.topk.need_fallback, 1u);
    }
  } else {
    // the k largest of the row's n candidates: threshold by radix selection, then a sort of the few survivors
    const int n = (int)sh_total, k = min(p.topk.k, n);
    uint32_t tau = 0u;
    unsigned int need_eq = 0u;
    if (k > 0) select_kth_key(topk_keys, n, k, hist, warp_sums, &sh_prefix, &sh_need, tid, kTopkFinishThreads, tau, need_eq);
    // everything above the threshold (fewer than k), then entries equal to it while there is room: which of
    // several exactly equal logits at the k-th place are taken is not specified (nor is it by the reference)
    for (int pass = 0; pass < 2 && k > 0; ++pass) {
      for (int i = tid; i < n; i += kTopkFinishThreads) {
        const uint32_t vk = (uint32_t)(topk_keys[i] >> 32);
        if (pass == 0 ? vk > tau : vk == tau) {
          const unsigned int pos = atomicAdd(&sh_count, 1u);
          if (pos < 2u * kTopkSlots) picked[pos] = topk_keys[i];
        }
      }
      __syncthreads();
    }
    bitonic_sort_desc(picked, 2 * kTopkSlots, tid, kTopkFinishThreads);
    topk_finish_row(p, b, picked, k, &sh, tid, kTopkFinishThreads);
  }
  // leave the row's scratch as the next call expects it
  for (int i = tid; i < kTopkSlots; i += kTopkFinishThreads) p.topk.table[(size_t)b * kTopkSlots + i] = 0u;
  if (tid == 0 && b == 0) *p.topk.gbar = 0u;
}

// Rows that overflowed, from their full logits [B, V] (fp32, unscaled): exact radix selection of the
// k-th largest scaled logit, then the k largest (equal values: lowest ids first), then the same tail.
__global__ void __launch_bounds__(kTopkExactThreads) topk_exact_kernel(const SampleParams p, const float* __restrict__ logits) {
  griddep_wait();  // launched behind its producer with programmatic stream serialisation
  __shared__ unsigned int hist[2048];
  __shared__ unsigned long long picked[2 * kTopkSlots];
  __shared__ unsigned int sh_prefix, sh_need, sh_count, sh_scan[kTopkExactThreads / 32], sh_taken;
  __shared__ TopkRowShared sh;
  const int b = blockIdx.x, tid = threadIdx.x;
  // the conditional pass that wrote the logits has read this word; nobody reads it in this kernel
  if (b == 0 && tid == 0) *p.topk.need_fallback = 0u;
  if (!p.topk.row_fallback[b]) return;
  const float* row = logits + (size_t)b * p.V;
  float inv_t = 1.f;
  if (!(p.flags & kFlagGreedy)) {
    const float temp = p.temperature[(size_t)b * p.temp_stride];
    if (temp > 0.f) inv_t = 1.f / temp;
  }
  const int k = min(p.topk.k, p.V);
  if (tid == 0) {
    sh_prefix = 0u;
    sh_need = (unsigned int)k;
  }
  uint32_t mask = 0u;
  const int shifts[3] = {21, 10, 0}, bits[3] = {11, 11, 10};
  for (int pass = 0; pass < 3; ++pass) {
    for (int i = tid; i < 2048; i += kTopkExactThreads) hist[i] = 0u;
    __syncthreads();
    const uint32_t prefix = sh_prefix, binmask = (1u << bits[pass]) - 1u;
    for (int base = 0; base < p.V; base += kTopkExactThreads) {
      const int v = base + tid;
      const uint32_t key = v < p.V ? float_key(row[v] * inv_t) : 0u;
      hist_add_merged(hist, (key >> shifts[pass]) & binmask, v < p.V && (key & mask) == prefix);
    }
    __syncthreads();
    if (tid == 0) {
      unsigned int need = sh_need, cum = 0;
      int bin = (int)binmask;
      for (; bin > 0; --bin) {
        if (cum + hist[bin] >= need) break;
        cum += hist[bin];
      }
      sh_need = need - cum;  // how many of this bin are still wanted
      sh_prefix = prefix | ((uint32_t)bin << shifts[pass]);
    }
    mask |= binmask << shifts[pass];
    __syncthreads();
  }
  const uint32_t tau = sh_prefix;       // key of the k-th largest scaled logit
  const unsigned int need_eq = sh_need;  // entries equal to it that belong to the k largest
  if (tid == 0) {
    sh_count = 0u;
    sh_taken = 0u;
  }
  for (int i = tid; i < 2 * kTopkSlots; i += kTopkExactThreads) picked[i] = 0ull;
  __syncthreads();
  // entries above the threshold (fewer than k), in any order
  for (int v = tid; v < p.V; v += kTopkExactThreads) {
    const float z = row[v] * inv_t;
    if (float_key(z) > tau) {
      const unsigned int pos = atomicAdd(&sh_count, 1u);
      if (pos < (unsigned int)kTopkSlots) picked[pos] = cand_key(z, v);
    }
  }
  __syncthreads();
  const unsigned int n_gt = sh_count;
  // entries equal to the threshold, lowest ids first: an ordered compaction, one block-wide scan per 1024 ids
  for (int base = 0; base < p.V; base += kTopkExactThreads) {
    const int v = base + tid;
    float z = 0.f;
    bool hit = false;
    if (v < p.V) {
      z = row[v] * inv_t;
      hit = float_key(z) == tau;
    }
    const unsigned int ballot = __ballot_sync(0xffffffffu, hit);
    if ((tid & 31) == 0) sh_scan[tid >> 5] = __popc(ballot);
    __syncthreads();
    unsigned int before = sh_taken, total = 0;
    for (int w = 0; w < kTopkExactThreads / 32; ++w) {
      if (w < (tid >> 5)) before += sh_scan[w];
      total += sh_scan[w];
    }
    before += __popc(ballot & ((1u << (tid & 31)) - 1u));
    if (hit && before < need_eq) picked[n_gt + before] = cand_key(z, v);
    __syncthreads();
    if (tid == 0) sh_taken += total;
    __syncthreads();
    if (sh_taken >= need_eq) break;
  }
  __syncthreads();
  bitonic_sort_desc(picked, 2 * kTopkSlots, tid, kTopkExactThreads);
  topk_finish_row(p, b, picked, k, &sh, tid, kTopkExactThreads);
  if (tid == 0) p.topk.row_fallback[b] = 0;
}

// Rows that overflowed when there is no scratch for the exact pass: ids -1 and an error status.
__global__ void topk_overflow_kernel(const SampleParams p) {
  griddep_wait();  // launched behind its producer with programmatic stream serialisation
  const int b = blockIdx.x, tid = threadIdx.x;
  if (b == 0 && tid == 0) *p.topk.need_fallback = 0u;
  if (!p.topk.row_fallback[b]) return;
  for (int s = tid; s < p.S; s += blockDim.x) {
    p.out_idx[(size_t)b * p.S + s] = -1;
    if (p.out_val) p.out_val[(size_t)b * p.S + s] = -INFINITY;
  }
  if (tid == 0) {
    if (p.status_dev) atomicExch(p.status_dev, kErrTopkOverflow);
    p.topk.row_fallback[b] = 0;
  }
}

}  // namespace fmms
