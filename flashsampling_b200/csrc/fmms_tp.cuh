// Tensor-parallel exchange of per-row winners over NVLink peer memory.
//
// Every rank owns a symmetric buffer: `slots[2][world][max_items]` of 16-byte records
// (fp32 value, int64 global id) followed by `flags[world]` (one 128-byte line each).
// A step with epoch e uses slot parity e & 1.  Rank r writes its records into
// slots[e & 1][r] of EVERY rank with plain 16-byte stores through peer pointers, then
// release-stores e into flags[r] of every rank; it then waits (bounded) until all of its
// own flags show e and takes the maximum over the `world` records of each item.  All loads
// are local; the only traffic that crosses NVLink is 16 bytes per item per peer plus the
// flags.  Epochs only grow, so flags are never reset, and the two parities keep a fast rank
// from overwriting records a slow rank is still reading (a rank can be at most one step
// ahead, because its own step e+1 cannot finish before every rank has signalled e+1).
#pragma once

#include "fmms_common.cuh"

namespace fmms {

constexpr int kTpMaxWorld = 8;
constexpr int kTpFlagStride = 32;  // uint32 per flag line (128 bytes)

struct TpRecord {
  float val;
  int pad;
  long long idx;
};
static_assert(sizeof(TpRecord) == 16, "record must be one 16-byte store");

struct TpPeers {
  TpRecord* slots[kTpMaxWorld];
  unsigned int* flags[kTpMaxWorld];
};

__host__ __device__ inline size_t tp_buffer_bytes(int world, int max_items) {
  return (size_t)2 * world * max_items * sizeof(TpRecord) + (size_t)world * kTpFlagStride * 4;
}

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ TpRecord ld_record_volatile(const TpRecord* p) {
  TpRecord r;
  int a, b, c, d;
  asm volatile("ld.volatile.global.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "l"(p) : "memory");
  r.val = __int_as_float(a);
  r.pad = b;
  r.idx = (long long)(((unsigned long long)(unsigned int)d << 32) | (unsigned int)c);
  return r;
}

// One CTA.  local_idx/local_val: this rank's winners [n_items] (item = b * S + s).
__global__ void tp_exchange_kernel(const long long* __restrict__ local_idx, const float* __restrict__ local_val,
                                   int n_items, int max_items, int rank, int world, TpPeers peers,
                                   unsigned int epoch, unsigned long long wait_limit_ns,
                                   long long* __restrict__ out_idx, float* __restrict__ out_val, int* status_dev) {
  const int tid = threadIdx.x;
  const int parity = (int)(epoch & 1u);
  const size_t my_row = ((size_t)parity * world + rank) * max_items;
  for (int i = tid; i < n_items; i += blockDim.x) {
    const float v = local_val[i];
    const long long id = local_idx[i];
    const int4 rec = make_int4(__float_as_int(v), 0, (int)(unsigned int)(unsigned long long)id,
                               (int)(unsigned int)((unsigned long long)id >> 32));
    for (int p = 0; p < world; ++p) *reinterpret_cast<int4*>(peers.slots[p] + my_row + i) = rec;
  }
  __threadfence_system();
  __syncthreads();
  if (tid < world) st_release_sys(peers.flags[tid] + (size_t)rank * kTpFlagStride, epoch);
  __shared__ int timed_out;
  if (tid == 0) timed_out = 0;
  __syncthreads();
  if (tid < world) {
    const unsigned int* f = peers.flags[rank] + (size_t)tid * kTpFlagStride;
    const unsigned long long t0 = global_timer_ns();
    unsigned int spins = 0;
    while ((int)(ld_acquire_sys(f) - epoch) < 0) {
      if ((++spins & 0xffu) == 0 && global_timer_ns() - t0 > wait_limit_ns) {
        timed_out = 1;
        if (status_dev) atomicExch(status_dev, kErrTimeout);
        break;
      }
    }
  }
  __syncthreads();
  const TpRecord* mine = peers.slots[rank] + (size_t)parity * world * max_items;
  for (int i = tid; i < n_items; i += blockDim.x) {
    float bv = -INFINITY;
    long long bi = 0x7fffffffffffffffll;
    for (int r = 0; r < world; ++r) {
      const TpRecord rec = ld_record_volatile(mine + (size_t)r * max_items + i);
      if (rec.val > bv || (rec.val == bv && rec.idx < bi)) {
        bv = rec.val;
        bi = rec.idx;
      }
    }
    if (timed_out) bi = -1;  // never hand out an id computed from stale records
    out_idx[i] = bi;
    if (out_val) out_val[i] = bv;
  }
}

}  // namespace fmms
