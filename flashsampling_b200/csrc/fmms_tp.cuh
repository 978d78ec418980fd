// Tensor-parallel exchange of per-row winners over NVLink peer memory.
//
// Every rank owns a symmetric buffer of 16-byte records in three regions: winners
// `[2][world][max_items]`, the winners' unperturbed logits `[2][world][max_items]` and the rows'
// log-sum-exp partials `[2][world][256]` (the last two only travel when log-probabilities are
// asked for).  A record
// carries its own validity: {value bits, epoch, global id, epoch}, each half an 8-byte word that
// NVLink delivers atomically, so no separate flag and no fence is needed (the "low-latency"
// protocol of collective libraries).  In step `epoch` rank r stores its records into
// slots[epoch & 1][r] of EVERY rank with plain peer stores and then reads its own buffer, spinning
// (bounded) on each record until both halves show this epoch, and keeps the maximum over ranks.
// All loads are local; 16 bytes per item and peer cross NVLink, once, one way.  Epochs only grow
// (0 = never written), and the two parities keep a fast rank from overwriting records a slow rank
// has not read yet: a rank cannot finish step e+1 before every rank has sent its step-e+1 records,
// which each rank does only after reading all of step e.
#pragma once

#include "fmms_common.cuh"

namespace fmms {

constexpr int kTpMaxWorld = 8;
constexpr int kTpMaxRows = 256;    // batch rows per launch (log-sum-exp records)
constexpr int kTpFlagStride = 32;  // the buffer ends with world * 128 reserved bytes; the first word is the
                                   // rank's own step counter (used when the caller passes epoch 0)

struct TpRecord {
  unsigned int val_bits, epoch0, idx, epoch1;
};
static_assert(sizeof(TpRecord) == 16, "record must be one 16-byte store");

struct TpPeers {
  TpRecord* slots[kTpMaxWorld];
};

__host__ __device__ inline size_t tp_record_count(int world, int max_items) {
  return (size_t)2 * world * ((size_t)2 * max_items + kTpMaxRows);
}

__host__ __device__ inline size_t tp_buffer_bytes(int world, int max_items) {
  return tp_record_count(world, max_items) * sizeof(TpRecord) + (size_t)world * kTpFlagStride * 4;
}

__host__ __device__ inline size_t tp_counter_offset(int world, int max_items) {
  return tp_record_count(world, max_items) * sizeof(TpRecord);
}

// first record of the logit region / of the log-sum-exp region of a rank's buffer
__host__ __device__ inline size_t tp_logit_region(int world, int max_items) { return (size_t)2 * world * max_items; }
__host__ __device__ inline size_t tp_lse_region(int world, int max_items) { return (size_t)4 * world * max_items; }

// Epoch of this step: the caller's, or (caller passed 0) one more than the count kept in the
// rank's own buffer, which makes a captured launch replayable: every replay advances by itself.
__device__ __forceinline__ unsigned int tp_load_counter(const unsigned int* counter) {
  unsigned int v;
  asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
  return v;
}

__device__ __forceinline__ void st_record(TpRecord* p, float v, unsigned int idx, unsigned int epoch) {
  asm volatile("st.volatile.global.v4.b32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(__float_as_uint(v)), "r"(epoch),
               "r"(idx), "r"(epoch)
               : "memory");
}

__device__ __forceinline__ TpRecord ld_record(const TpRecord* p) {
  TpRecord r;
  asm volatile("ld.volatile.global.v4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(r.val_bits), "=r"(r.epoch0), "=r"(r.idx), "=r"(r.epoch1)
               : "l"(p)
               : "memory");
  return r;
}

// Send one record (two payload words) to the same place in every rank's buffer.
__device__ __forceinline__ void tp_send_words(const TpPeers& peers, int world, size_t record, float a, unsigned int b,
                                              unsigned int epoch) {
  for (int q = 0; q < world; ++q) st_record(peers.slots[q] + record, a, b, epoch);
}

// Wait (bounded) until the record at `src` carries this epoch.  Returns false on time-out.
__device__ __forceinline__ bool tp_wait_record(const TpRecord* src, unsigned int epoch, unsigned long long wait_limit_ns,
                                               TpRecord& rec) {
  rec = ld_record(src);
  unsigned int spins = 0;
  unsigned long long t0 = 0;
  while (rec.epoch0 != epoch || rec.epoch1 != epoch) {
    if ((++spins & 0x3fu) == 0) {
      if (t0 == 0) t0 = global_timer_ns();
      else if (global_timer_ns() - t0 > wait_limit_ns) return false;
    }
    rec = ld_record(src);
  }
  return true;
}

// Send this rank's record of `item` to every rank.
__device__ __forceinline__ void tp_send(const TpPeers& peers, int world, size_t row_item, float v, long long gid,
                                        unsigned int epoch) {
  for (int q = 0; q < world; ++q) st_record(peers.slots[q] + row_item, v, (unsigned int)gid, epoch);
}

// Wait (bounded) for all ranks' records of `item` in this rank's buffer and reduce them.
// Returns false on time-out.
__device__ __forceinline__ bool tp_recv_max(const TpRecord* mine, int world, int max_items, int item,
                                            unsigned int epoch, unsigned long long wait_limit_ns, float& bv,
                                            long long& bi, int* winner_rank = nullptr) {
  bv = -INFINITY;
  bi = 0x7fffffffffffffffll;
  unsigned long long t0 = 0;
  for (int r = 0; r < world; ++r) {
    const TpRecord* src = mine + (size_t)r * max_items + item;
    TpRecord rec = ld_record(src);
    unsigned int spins = 0;
    while (rec.epoch0 != epoch || rec.epoch1 != epoch) {
      if ((++spins & 0x3fu) == 0) {
        if (t0 == 0) t0 = global_timer_ns();
        else if (global_timer_ns() - t0 > wait_limit_ns) return false;
      }
      rec = ld_record(src);
    }
    const float v = __uint_as_float(rec.val_bits);
    const long long id = (long long)rec.idx;
    if (v > bv || (v == bv && id < bi)) {
      bv = v;
      bi = id;
      if (winner_rank) *winner_rank = r;
    }
  }
  return true;
}

// One CTA.  local_idx/local_val: this rank's winners [n_items] (item = b * S + s).
__global__ void tp_exchange_kernel(const long long* __restrict__ local_idx, const float* __restrict__ local_val,
                                   int n_items, int max_items, int rank, int world, TpPeers peers,
                                   unsigned int epoch, unsigned long long wait_limit_ns,
                                   long long* __restrict__ out_idx, float* __restrict__ out_val, int* status_dev) {
  const int tid = threadIdx.x;
  unsigned int* counter = reinterpret_cast<unsigned int*>(reinterpret_cast<unsigned char*>(peers.slots[rank]) +
                                                          tp_counter_offset(world, max_items));
  if (epoch == 0u) epoch = tp_load_counter(counter) + 1u;
  __syncthreads();  // every thread has read the counter before thread 0 advances it
  if (tid == 0) *counter = epoch;
  const int parity = (int)(epoch & 1u);
  const size_t my_row = ((size_t)parity * world + rank) * max_items;
  const TpRecord* mine = peers.slots[rank] + (size_t)parity * world * max_items;
  for (int i = tid; i < n_items; i += blockDim.x) tp_send(peers, world, my_row + i, local_val[i], local_idx[i], epoch);
  for (int i = tid; i < n_items; i += blockDim.x) {
    float bv;
    long long bi;
    if (!tp_recv_max(mine, world, max_items, i, epoch, wait_limit_ns, bv, bi)) {
      if (status_dev) atomicExch(status_dev, kErrTimeout);
      bi = -1;  // never hand out an id computed from stale records
    }
    out_idx[i] = bi;
    if (out_val) out_val[i] = bv;
  }
}

}  // namespace fmms
