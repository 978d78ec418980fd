// Device-side building blocks shared by the sampling kernels: the counter-based
// noise stream, candidate ordering, and thin wrappers over the sm_100a PTX used
// for mbarriers, TMA (cp.async.bulk.tensor) and tcgen05/TMEM.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fmms {

// ------------------------------------------------------------------------------------
// status / flags (mirrors include/fmms_b200.h)
// ------------------------------------------------------------------------------------
constexpr int kOk = 0, kErrTimeout = 1, kErrBadArg = 2, kErrUnsupported = 3, kErrWorkspace = 4,
              kErrCuda = 5, kErrArch = 6;
constexpr int kFlagGreedy = 1, kFlagExtNoise = 2, kFlagReturnLogits = 4, kFlagForceGemv = 8,
              kFlagForceMma = 16, kFlagTwoStage = 32, kFlagSeedDev = 64, kFlagLogprob = 128;

constexpr int kFlagFp8 = 2048;   // W (and the staged hidden states) are e4m3 bytes with per-row scales
constexpr int kFlagTopk = 1024;  // internal: the launch collects top-k candidates instead of sampling

constexpr int kIdxNone = 0x7fffffff;  // candidate index meaning "no candidate yet"

// ------------------------------------------------------------------------------------
// Top-k / top-p: per-row scratch shared by the candidate-collecting pass and the kernels
// that finish the rows (see fmms_topk.cuh).  Everything here is zero between calls.
// ------------------------------------------------------------------------------------
constexpr int kTopkSlots = 64;       // class maxima per row; also the largest top_k
constexpr int kTopkSegCap = 16;      // candidates one epilogue thread can keep for its row (its private segment)
constexpr int kTopkMaxSegs = 640;    // segments per row: persistent CTAs x column groups
constexpr int kTopkListCap = 4096;   // candidates per row that the finish kernel gathers from the segments
constexpr int kTopkSpillDead = 1 << 24;  // a thread's segment count from the moment it found the spill list full
constexpr int kTopkExtraCap = 2048;  // entries of a row's spill list (logits clustered in a few CTAs' vocabulary ranges)
struct TopkArgs {
  int k;                        // top_k (1..kTopkSlots); 0 = off
  float top_p;                  // nucleus mass in (0, 1); anything else = off
  int nseg;                     // segments per row in this launch (CTAs x column groups)
  unsigned int* table;          // [B][kTopkSlots] order-preserving keys of class maxima (0 = empty)
  unsigned int* seg_count;      // [B][kTopkMaxSegs] candidates each thread found (above kTopkSegCap: overflow);
                                // every launch writes all nseg entries of every row it reads
  unsigned long long* list;     // [B][kTopkMaxSegs][kTopkSegCap] packed (scaled logit, local id)
  unsigned int* extra_count;    // [B] candidates that did not fit into their thread's segment ...
  unsigned long long* extra;    // ... and went to the row's shared spill list [B][kTopkExtraCap] instead
  unsigned int* gbar;           // grid-wide arrival counter of the collecting pass
  unsigned int* need_fallback;  // != 0: some row overflowed and the exact pass has to run
  unsigned char* row_fallback;  // [B] rows that overflowed
};

// Bounded waits: a wait gives up after this many nanoseconds of wall-clock time,
// records kErrTimeout and lets the kernel run to its end on whatever data it has.
constexpr unsigned long long kWaitLimitNs = 2000000000ull;

// ------------------------------------------------------------------------------------
// Noise: Philox-4x32-10 keyed by (seed + sample), counter = (v >> 2, b, v >> 34, 0)
// ------------------------------------------------------------------------------------
constexpr uint32_t kPhiloxM0 = 0xD2511F53u, kPhiloxM1 = 0xCD9E8D57u;
constexpr uint32_t kPhiloxW0 = 0x9E3779B9u, kPhiloxW1 = 0xBB67AE85u;

__device__ __forceinline__ uint4 philox4x32_10(uint4 c, uint2 k) {
#pragma unroll
  for (int i = 0; i < 10; ++i) {
    // one 32 x 32 -> 64-bit multiply per product (mul.wide.u32), not a high and a low multiply
    const unsigned long long p0 = (unsigned long long)kPhiloxM0 * c.x, p1 = (unsigned long long)kPhiloxM1 * c.z;
    const uint32_t hi0 = (uint32_t)(p0 >> 32), lo0 = (uint32_t)p0;
    const uint32_t hi1 = (uint32_t)(p1 >> 32), lo1 = (uint32_t)p1;
    c = make_uint4(hi1 ^ c.y ^ k.x, lo1, hi0 ^ c.w ^ k.y, lo0);
    k.x += kPhiloxW0;
    k.y += kPhiloxW1;
  }
  return c;
}

// The four 32-bit words for global vocabulary ids 4q .. 4q+3 of row b, draw s.
__device__ __forceinline__ uint4 noise_block(unsigned long long seed, int s, int b,
                                             unsigned long long v_quad) {
  const unsigned long long stream = seed + (unsigned long long)s;
  return philox4x32_10(make_uint4((uint32_t)v_quad, (uint32_t)b, (uint32_t)(v_quad >> 32), 0u),
                       make_uint2((uint32_t)stream, (uint32_t)(stream >> 32)));
}

// The seed of a call: the value itself, or (kFlagSeedDev) a uint64 read from device memory, so that
// a launch captured in a CUDA graph draws fresh noise on every replay.
__device__ __forceinline__ unsigned long long resolve_seed(unsigned long long seed_or_ptr, int flags) {
  if (flags & kFlagSeedDev) return *reinterpret_cast<const volatile unsigned long long*>(seed_or_ptr);
  return seed_or_ptr;
}

// .ftz: no rescaling code around the instruction for subnormal inputs, which the callers never produce (the
// arguments are 1 - w >= 2^-24 or exactly 0, and unit exponentials >= 2^-33)
__device__ __forceinline__ float lg2_approx(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Standard Gumbel variate from 32 random bits.  w = (r + 0.5) 2^-32; the unit
// exponential E = -log1p(-w) is a cubic in w below 2^-7 (fp32 keeps the full
// relative precision of small w, which is the winning upper tail of the Gumbel)
// and -ln(1 - w) above; G = -ln E.  w == 1 after rounding gives G = -inf, which
// simply never wins.
__device__ __forceinline__ float gumbel_from_bits(uint32_t r) {
  constexpr float kLn2 = 0.6931471805599453f;
  const float w = fmaf(__uint2float_rn(r), 0x1p-32f, 0x1p-33f);
  const float e_small = w * fmaf(w, fmaf(w, 0.3333333333f, 0.5f), 1.0f);
  const float e_big = -kLn2 * lg2_approx(1.0f - w);
  const float e = (w < 0x1p-7f) ? e_small : e_big;
  return -kLn2 * lg2_approx(e);
}

__device__ __forceinline__ uint32_t pick_word(const uint4& q, uint32_t i) {
  return i == 0 ? q.x : (i == 1 ? q.y : (i == 2 ? q.z : q.w));
}

// Candidate order: larger value wins, equal values resolve to the lower index.
__device__ __forceinline__ bool cand_better(float v1, int i1, float v2, int i2) {
  return (v1 > v2) || (v1 == v2 && i1 < i2);
}

__device__ __forceinline__ void cand_merge(float& v, int& i, float v2, int i2) {
  if (cand_better(v2, i2, v, i)) {
    v = v2;
    i = i2;
  }
}

__device__ __forceinline__ void warp_cand_allreduce(float& v, int& i) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const float v2 = __shfl_xor_sync(0xffffffffu, v, off);
    const int i2 = __shfl_xor_sync(0xffffffffu, i, off);
    cand_merge(v, i, v2, i2);
  }
}

// A candidate packed into 64 bits so that one atomicMax keeps the winner: the high word is
// the value mapped to an order-preserving unsigned integer, the low word the complemented
// index (equal values resolve to the lower index).  Zero means "no candidate".
__device__ __forceinline__ unsigned long long cand_key(float v, int idx) {
  uint32_t b = __float_as_uint(v);
  b = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
  return ((unsigned long long)b << 32) | (unsigned long long)(~(uint32_t)idx);
}

// The value half of a candidate key on its own: an order-preserving 32-bit image of a float.
__device__ __forceinline__ uint32_t float_key(float v) {
  const uint32_t b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float float_key_decode(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

__device__ __forceinline__ void cand_key_decode(unsigned long long k, float& v, int& idx) {
  if (k == 0ull) {
    v = -INFINITY;
    idx = 0;
    return;
  }
  uint32_t b = (uint32_t)(k >> 32);
  b = (b & 0x80000000u) ? (b & 0x7fffffffu) : ~b;
  v = __uint_as_float(b);
  idx = (int)(~(uint32_t)k);
}

// ------------------------------------------------------------------------------------
// Running log-sum-exp of one batch row (kFlagLogprob), in base-2 units: the pair (m, l) stands
// for l * 2^m with l = sum_v 2^(x_v * log2(e) - m); l == 0 means "nothing accumulated yet".
// ------------------------------------------------------------------------------------
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2f = 0.6931471805599453f;

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// (m, l) <- (m, l) + (m2, l2)
__device__ __forceinline__ void lse_merge(float& m, float& l, float m2, float l2) {
  if (!(l2 > 0.f)) return;
  if (!(l > 0.f)) {
    m = m2;
    l = l2;
    return;
  }
  const float mn = fmaxf(m, m2);
  l = l * ex2_approx(m - mn) + l2 * ex2_approx(m2 - mn);
  m = mn;
}

// Fold one scaled logit x2 = logit / T * log2(e) into (m, l); m starts at -inf, l at 0.
__device__ __forceinline__ void lse_push(float& m, float& l, float x2) {
  const float mn = fmaxf(m, x2);
  l = l * ex2_approx(m - mn) + ex2_approx(x2 - mn);
  m = mn;
}

// A partial sum as one 64-bit word (m in the high half, l in the low half; zero = empty).
__device__ __forceinline__ unsigned long long lse_pack(float m, float l) {
  return ((unsigned long long)__float_as_uint(m) << 32) | __float_as_uint(l);
}
__device__ __forceinline__ void lse_merge_packed(float& m, float& l, unsigned long long bits) {
  lse_merge(m, l, __uint_as_float((uint32_t)(bits >> 32)), __uint_as_float((uint32_t)bits));
}

// Natural-log normaliser ln(sum_v exp(logit_v / T)).
__device__ __forceinline__ float lse_value(float m, float l) { return (m + log2f(l)) * kLn2f; }

// ------------------------------------------------------------------------------------
// PTX wrappers
// ------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded mbarrier wait.  `abort_flag` lives in shared memory: once any wait of
// the CTA has timed out every later wait returns at once, so the kernel drains
// instead of stacking time-outs.  Returns false on time-out.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          int* status_dev) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_timer_ns();
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 0x3ffu) == 0) {
      if (*abort_flag) return false;
      if (global_timer_ns() - t0 > kWaitLimitNs) {
        *abort_flag = 1;
        if (status_dev) atomicExch(status_dev, kErrTimeout);
        return false;
      }
    }
  }
  return true;
}

// Bounded wait that ignores the abort flag (used while draining after a time-out).
__device__ __forceinline__ bool mbar_wait_plain(uint64_t* bar, uint32_t parity,
                                                unsigned long long limit_ns) {
  const unsigned long long t0 = global_timer_ns();
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 0x3ffu) == 0 && global_timer_ns() - t0 > limit_ns) return false;
  }
  return true;
}

// 2-D tiled TMA load, completion signalled on an mbarrier (bytes of the full box).
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const void* tmap, int x, int y,
                                            uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];" ::"r"(smem_u32(smem_dst)),
      "l"(tmap), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}

__device__ __forceinline__ void tma_load_2d_hint(void* smem_dst, const void* tmap, int x, int y,
                                                 uint64_t* bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1, {%2, %3}], [%4], %5;" ::"r"(smem_u32(smem_dst)),
      "l"(tmap), "r"(x), "r"(y), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}

__device__ __forceinline__ void tma_load_3d_hint(void* smem_dst, const void* tmap, int x, int y, int z,
                                                 uint64_t* bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1, {%2, %3, %4}], [%5], %6;" ::"r"(smem_u32(smem_dst)),
      "l"(tmap), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}

__device__ __forceinline__ uint64_t policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}

__device__ __forceinline__ uint64_t policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}

// Programmatic dependent launch.  A kernel launched with the programmatic-serialisation attribute may start
// while the kernel before it on the stream still runs; griddep_wait() blocks until that kernel has completed
// and its writes are visible (it returns at once in a kernel launched the ordinary way).  The earlier kernel
// calls griddep_launch_dependents() to let the next one start.
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ void prefetch_tmap(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

}  // namespace fmms
