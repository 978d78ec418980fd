// C ABI of the fused LM-head sampling library (see include/fmms_b200.h): argument
// checks, kernel selection, TMA descriptor cache and launches.  No torch types, no
// allocation on the sampling path, no synchronisation.
#include <cuda.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "../../include/fmms_b200.h"
#include "fmms_common.cuh"
#include "fmms_tp.cuh"
#include "fmms_gemv.cuh"
#include "fmms_umma.cuh"
#include "fmms_umma2.cuh"
#include "fmms_topk.cuh"

namespace fmms {

constexpr int kVersion = 1000;
constexpr int kMaxParts = 640;      // upper bound on candidate rows in the workspace (4 per persistent CTA)
constexpr int kMaxDevices = 16;
constexpr int kGemvAutoMaxBatch = 4;  // auto-dispatch: batches up to this use the weight-streaming kernel where its shared memory
                                      // allows (measured, Qwen head: B = 3 187 vs 198 us, B = 4 189 vs 198, B = 5 262 vs 200)

static thread_local int g_last_path = FMMS_PATH_NONE;
static unsigned long long* g_stamps = nullptr;  // see fmms_debug_stamps()

struct DeviceInfo {
  std::atomic<bool> ready{false};
  int num_sms = 0;
  int cc_major = 0;
  int max_smem_optin = 0;
  bool gemv_attr[2][kGemvMaxBatch + 1] = {};  // [with log-probabilities][batch rows]
  bool umma_attr[3][8] = {};  // [plain | log-probabilities | top-k][M tiles; 3 = pair kernel]
};

static std::mutex g_mu;
static DeviceInfo g_dev[kMaxDevices];

static int device_info(DeviceInfo** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return kErrCuda;
  if (dev < 0 || dev >= kMaxDevices) return kErrUnsupported;
  DeviceInfo& d = g_dev[dev];
  if (!d.ready.load(std::memory_order_acquire)) {
    std::lock_guard<std::mutex> lk(g_mu);
    if (!d.ready.load(std::memory_order_relaxed)) {
      if (cudaDeviceGetAttribute(&d.num_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return kErrCuda;
      if (cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return kErrCuda;
      if (cudaDeviceGetAttribute(&d.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess) return kErrCuda;
      d.ready.store(true, std::memory_order_release);
    }
  }
  *out = &d;
  return kOk;
}

// ---- TMA descriptors ------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                   CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill);

static EncodeTiledFn lookup_encode_fn() {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
      q == cudaDriverEntryPointSuccess)
    return reinterpret_cast<EncodeTiledFn>(p);
  return nullptr;
}

static EncodeTiledFn encode_fn() {
  static const EncodeTiledFn fn = lookup_encode_fn();  // initialised once, thread-safe
  return fn;
}

struct MapKey {
  const void* ptr;
  long long rows, cols;
  int box_rows, box_cols, swizzle;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && box_rows == o.box_rows &&
           box_cols == o.box_cols && swizzle == o.swizzle;
  }
};
struct MapEntry {
  MapKey key;
  CUtensorMap map;
};
// Two caches: descriptors of weight matrices (few, long-lived) and of hidden-state matrices.  A
// serving engine may hand over a fresh hidden-state tensor every step: those misses cost one
// host-side encode each and must never evict a weight descriptor.
struct MapCache {
  std::vector<MapEntry> entries;
  size_t capacity;
};
static MapCache g_maps_w{{}, 64}, g_maps_h{{}, 16};

static bool map_cache_find(MapCache& c, const MapKey& key, CUtensorMap* out) {
  std::lock_guard<std::mutex> lk(g_mu);
  for (const MapEntry& e : c.entries)
    if (e.key == key) {
      *out = e.map;
      return true;
    }
  return false;
}
static void map_cache_put(MapCache& c, const MapKey& key, const CUtensorMap& m) {
  std::lock_guard<std::mutex> lk(g_mu);
  if (c.entries.size() >= c.capacity) c.entries.erase(c.entries.begin());
  c.entries.push_back(MapEntry{key, m});
}

// Row-major [rows, cols] bf16 matrix, box = box_rows x box_cols, out-of-range elements read as zero.
static int get_tensor_map(const void* ptr, long long rows, long long cols, int box_rows, int box_cols,
                          CUtensorMapSwizzle swz, CUtensorMap* out, bool hidden = false) {
  MapCache& cache = hidden ? g_maps_h : g_maps_w;
  const MapKey key{ptr, rows, cols, box_rows, box_cols, (int)swz};
  if (map_cache_find(cache, key, out)) return kOk;
  EncodeTiledFn fn = encode_fn();
  if (!fn) return kErrCuda;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMap m;
  CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return kErrCuda;
  map_cache_put(cache, key, m);
  *out = m;
  return kOk;
}

// Workspace layout, a function of the workspace SIZE only (so calls of different shapes that
// share one workspace agree on it): [ticket: 256 B][log-sum-exp scratch: kLseMaxSplit x 256 u64 of
// the last CTA's merge, then kMaxLseParts x 256 u64 per-CTA partial sums][keys: cap u64][running candidates:
// kMaxParts * cap * (f32 + i32)], cap = the number of (row, draw) items the size can hold.
// Ticket and keys must be zero when a call starts; every call leaves them zero again.  The
// log-sum-exp scratch needs no initial state: a launch writes every entry it later reads.
constexpr int kMaxBatchPerLaunch = 256;
constexpr int kMaxLseParts = kMaxParts / 4;  // one partial row per CTA (or CTA pair)
static_assert(kMaxBatchPerLaunch == kLseMaxRows, "the log-sum-exp scratch is sized for one launch's rows");
constexpr size_t kWsLse2Offset = 256;
constexpr size_t kWsLseOffset = kWsLse2Offset + (size_t)kLseMaxSplit * kLseMaxRows * 8;
constexpr size_t kWsHeadBytes = kWsLseOffset + (size_t)kMaxLseParts * kMaxBatchPerLaunch * 8;
static size_t workspace_bytes_for(int B, int S) {
  return kWsHeadBytes + (size_t)B * (size_t)S * 8 * (1 + (size_t)kMaxParts);
}
static size_t workspace_item_capacity(size_t bytes) {
  return (bytes - kWsHeadBytes) / (8 * (1 + (size_t)kMaxParts));
}

// [rows, cols] bf16 matrix seen as (inner columns, rows, cols / inner groups); box = inner x box_rows x groups.
static int get_tensor_map_3d(const void* ptr, long long rows, long long cols, int inner, int box_rows, int slabs,
                             CUtensorMapSwizzle swz, CUtensorMap* out, bool hidden = false) {
  MapCache& cache = hidden ? g_maps_h : g_maps_w;
  const MapKey key{ptr, rows, cols, box_rows, inner + 1000 * slabs, (int)swz};
  if (map_cache_find(cache, key, out)) return kOk;
  EncodeTiledFn fn = encode_fn();
  if (!fn) return kErrCuda;
  cuuint64_t dims[3] = {(cuuint64_t)inner, (cuuint64_t)rows, (cuuint64_t)(cols / inner)};
  cuuint64_t strides[2] = {(cuuint64_t)cols * 2, (cuuint64_t)inner * 2};
  cuuint32_t box[3] = {(cuuint32_t)inner, (cuuint32_t)box_rows, (cuuint32_t)slabs};
  cuuint32_t estr[3] = {1, 1, 1};
  CUtensorMap m;
  CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return kErrCuda;
  map_cache_put(cache, key, m);
  *out = m;
  return kOk;
}
static int get_tensor_map_slabs(const void* ptr, long long rows, long long cols, int box_rows, int slabs,
                                CUtensorMap* out, bool hidden = false) {
  return get_tensor_map_3d(ptr, rows, cols, 64, box_rows, slabs, CU_TENSOR_MAP_SWIZZLE_128B, out, hidden);
}
static int get_tensor_map_chunks(const void* ptr, long long rows, long long cols, int box_rows, int chunks,
                                 CUtensorMap* out) {
  return get_tensor_map_3d(ptr, rows, cols, 256, box_rows, chunks, CU_TENSOR_MAP_SWIZZLE_NONE, out);
}

// ---- fp8 weights: the hidden states are quantised per row on the way in -----------------
// One CTA per hidden-state row: q = e4m3(h * 448 / amax) (round to nearest even), scale = amax / 448.
// The same arithmetic, in the same order, as the CPU oracle's quantiser, so both produce the same bytes.
__global__ void __launch_bounds__(256) quantize_rows_e4m3_kernel(const __nv_bfloat16* __restrict__ h, int D,
                                                                 unsigned char* __restrict__ q, float* __restrict__ scale) {
  __shared__ float warp_max[8];
  griddep_launch_dependents();  // the sampling kernel behind this one may start its weight stream now
  const int b = blockIdx.x, tid = threadIdx.x;
  const __nv_bfloat16* row = h + (size_t)b * D;
  float amax = 0.f;
  for (int i = tid; i < D; i += 256) amax = fmaxf(amax, fabsf(__bfloat162float(row[i])));
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
  if ((tid & 31) == 0) warp_max[tid >> 5] = amax;
  __syncthreads();
  amax = warp_max[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) amax = fmaxf(amax, warp_max[w]);
  amax = fmaxf(amax, 1e-12f);
  const float inv = 448.0f / amax;
  if (tid == 0) scale[b] = amax / 448.0f;
  for (int i = tid; i < D; i += 256)
    q[(size_t)b * D + i] = (unsigned char)__nv_cvt_float_to_fp8(__bfloat162float(row[i]) * inv, __NV_SATFINITE, __NV_E4M3);
}

struct Fp8Args {
  const float* w_scale;  // [V_local]
  void* staging;         // device memory for the quantised hidden states and their scales
  size_t staging_bytes;
};
static size_t fp8_staging_bytes(int D, int B) { return (((size_t)B * D + 255) & ~(size_t)255) + (size_t)B * 4; }

// ---- launches ---------------------------------------------------------------------
// g_overlap_next: the next sampling kernel may start while the kernel enqueued just before it (the hidden-state
// quantiser or the host-buffer gather, both of which release their dependents at once) still runs; the sampling
// kernels wait (griddepcontrol.wait) before they touch anything that kernel writes.  Consumed by one launch.
static thread_local bool g_overlap_next = false;

template <class... KArgs, class... Args>
static cudaError_t launch_kernel(void (*kernel)(KArgs...), int grid, int block, size_t smem, cudaStream_t stream,
                                 Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3((unsigned)block);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  if (g_overlap_next) {
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    g_overlap_next = false;
  }
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ---- GEMV launch ----------------------------------------------------------------
template <int NB, bool LSE>
static int launch_gemv_nb_lse(DeviceInfo& d, const CUtensorMap& map, SampleParams& p, int grid, size_t smem,
                              cudaStream_t stream) {
  if (!d.gemv_attr[LSE][NB]) {
    if (cudaFuncSetAttribute(gemv_sample_kernel<NB, LSE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             d.max_smem_optin) != cudaSuccess)
      return kErrCuda;
    d.gemv_attr[LSE][NB] = true;
  }
  return launch_kernel(gemv_sample_kernel<NB, LSE>, grid, kGemvThreads, smem, stream, map, p) == cudaSuccess ? kOk : kErrCuda;
}

// The kernels that also accumulate the log-sum-exp (kFlagLogprob) are separate instantiations,
// so that the plain sampling kernels carry none of that code.
template <int NB>
static int launch_gemv_nb(DeviceInfo& d, const CUtensorMap& map, SampleParams& p, int grid, size_t smem,
                          cudaStream_t stream) {
  return (p.flags & kFlagLogprob) ? launch_gemv_nb_lse<NB, true>(d, map, p, grid, smem, stream)
                                  : launch_gemv_nb_lse<NB, false>(d, map, p, grid, smem, stream);
}

// Tuning knobs (read once): FMMS_GEMV_STAGES / FMMS_UMMA_STAGES cap the shared-memory ring depth.
static int env_int(const char* name) {
  const char* v = std::getenv(name);
  return v ? std::atoi(v) : 0;
}
static int gemv_stage_cap() {
  static const int v = env_int("FMMS_GEMV_STAGES");
  return v;
}
static int umma_stage_cap() {
  static const int v = env_int("FMMS_UMMA_STAGES");
  return v;
}
static int umma_nt_target() {
  static const int v = env_int("FMMS_UMMA_NT");
  return v;
}
static int umma_min_tiles() {
  static const int v = env_int("FMMS_UMMA_MIN_TILES") > 0 ? env_int("FMMS_UMMA_MIN_TILES") : 1;
  return v;
}
static int umma_mt2_nt_cap() {
  static const int v = env_int("FMMS_UMMA_MT2_NTCAP") == 128 ? 128 : 256;
  return v;
}

static int gemv_chunks(int NB, int D) {
  static const int forced = env_int("FMMS_GEMV_CHUNKS");
  if (D % kGemvCols != 0 || D / kGemvCols < 2) return 1;  // the 3-D view needs whole chunks
  if (forced == 1 || forced == 2) return forced;
  return 2;  // 32-64 KiB per TMA operation (measured: B = 1 on the Qwen head 218 -> 183 us)
}

static int gemv_stages(const DeviceInfo& d, int NB, int D) {
  // about 96-128 KiB of W in flight per SM
  const int ck = gemv_chunks(NB, D);
  const int want = (int)(131072 / ((size_t)ck * gemv_stage_bytes(NB)));
  int stages = gemv_stage_cap() >= 3 ? gemv_stage_cap() : (want < 3 ? 3 : (want > kGemvMaxStages ? kGemvMaxStages : want));
  while (stages >= 3 && gemv_smem_bytes(NB, D, stages, ck) > (size_t)d.max_smem_optin) --stages;
  return stages >= 3 ? stages : 0;
}

static bool gemv_eligible(const DeviceInfo& d, int D, int B, int S) {
  return B <= kGemvMaxBatch && (long long)B * S <= 32 && gemv_stages(d, B, D) > 0;
}

static int launch_gemv(DeviceInfo& d, const void* W, SampleParams& p, cudaStream_t stream) {
  CUtensorMap map;
  const int NB = p.B;
  const int kGemvRows = gemv_rows(NB);
  p.gemv_chunks = gemv_chunks(NB, p.D);
  int rc;
  if (p.gemv_chunks > 1)
    rc = get_tensor_map_chunks(W, p.V, p.D, kGemvRows, p.gemv_chunks, &map);
  else
    rc = get_tensor_map(W, p.V, p.D, kGemvRows, kGemvCols, CU_TENSOR_MAP_SWIZZLE_NONE, &map);
  if (rc != kOk) return -rc;
  p.stages = gemv_stages(d, NB, p.D);
  const size_t smem = gemv_smem_bytes(NB, p.D, p.stages, p.gemv_chunks);
  const int groups = (p.V + kGemvRows - 1) / kGemvRows;
  const int grid = groups < d.num_sms ? groups : d.num_sms;
  if ((p.flags & kFlagLogprob) && grid > kMaxLseParts) return -kErrUnsupported;
  p.lse_parts = grid;
  switch (NB) {
    case 1: rc = launch_gemv_nb<1>(d, map, p, grid, smem, stream); break;
    case 2: rc = launch_gemv_nb<2>(d, map, p, grid, smem, stream); break;
    case 3: rc = launch_gemv_nb<3>(d, map, p, grid, smem, stream); break;
    case 4: rc = launch_gemv_nb<4>(d, map, p, grid, smem, stream); break;
    case 5: rc = launch_gemv_nb<5>(d, map, p, grid, smem, stream); break;
    case 6: rc = launch_gemv_nb<6>(d, map, p, grid, smem, stream); break;
    case 7: rc = launch_gemv_nb<7>(d, map, p, grid, smem, stream); break;
    case 8: rc = launch_gemv_nb<8>(d, map, p, grid, smem, stream); break;
    default: return -kErrUnsupported;
  }
  if (rc != kOk) return -rc;
  return grid;  // > 0: number of candidate rows written
}

// ---- tensor-core launch -----------------------------------------------------------
struct UmmaMaps {
  CUtensorMap wq, wq1, hm;
};

template <int MT, bool LSE, bool TOPK>
static int launch_umma_variant(DeviceInfo& d, const UmmaMaps& mp, SampleParams& p, const UmmaPlan& pl,
                               cudaStream_t stream) {
  bool& attr_set = d.umma_attr[TOPK ? 2 : (LSE ? 1 : 0)][MT];
  if (!attr_set) {
    if (cudaFuncSetAttribute(umma_sample_kernel<MT, LSE, TOPK>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             d.max_smem_optin) != cudaSuccess)
      return kErrCuda;
    attr_set = true;
  }
  return launch_kernel(umma_sample_kernel<MT, LSE, TOPK>, pl.grid, kUmmaThreads, pl.smem, stream, mp.wq, mp.wq1, mp.hm, p,
                       pl.nt_cap, pl.units_total, pl.q_units, pl.h_rows, pl.slabs, pl.copies, pl.m_rows) == cudaSuccess
             ? kOk
             : kErrCuda;
}

// The kernels that also accumulate the log-sum-exp (kFlagLogprob) or collect top-k candidates
// (kFlagTopk) are separate instantiations, so that the plain sampling kernels carry none of that code.
template <int MT>
static int launch_umma_mt(DeviceInfo& d, const UmmaMaps& mp, SampleParams& p, const UmmaPlan& pl,
                          cudaStream_t stream) {
  if (p.flags & kFlagTopk) return launch_umma_variant<MT, false, true>(d, mp, p, pl, stream);
  return (p.flags & kFlagLogprob) ? launch_umma_variant<MT, true, false>(d, mp, p, pl, stream)
                                  : launch_umma_variant<MT, false, false>(d, mp, p, pl, stream);
}

static int umma_slabs_force() {
  static const int v = env_int("FMMS_UMMA_SLABS");
  return v;
}

static int umma_m64() {
  static const int v = std::getenv("FMMS_UMMA_M64") ? env_int("FMMS_UMMA_M64") : -1;  // 0 / 1 force M = 128 / 64 (B <= 64)
  return v;
}
static int umma_copies_cap() {
  static const int v = env_int("FMMS_UMMA_COPIES");  // 0 (default): no row replicas; 2 / 4: up to that many
  return v;
}

static int build_umma_maps(const void* W, const void* H, const SampleParams& p, const UmmaPlan& pl, UmmaMaps* mp) {
  int rc;
  if (pl.slabs > 1) {
    rc = get_tensor_map_slabs(W, p.V, p.D, pl.q_units * 16, pl.slabs, &mp->wq);
    if (rc != kOk) return rc;
    mp->wq1 = mp->wq;
    if (pl.q_units > 1) {
      rc = get_tensor_map_slabs(W, p.V, p.D, (pl.q_units - 1) * 16, pl.slabs, &mp->wq1);
      if (rc != kOk) return rc;
    }
    rc = get_tensor_map_slabs(H, p.B, p.D, pl.h_rows, pl.slabs, &mp->hm, /*hidden=*/true);
    if (rc != kOk) return rc;
  } else {
    rc = get_tensor_map(W, p.V, p.D, pl.q_units * 16, kUmmaBK, CU_TENSOR_MAP_SWIZZLE_128B, &mp->wq);
    if (rc != kOk) return rc;
    mp->wq1 = mp->wq;  // a CTA only uses the lower box when some tile is one unit shorter
    if (pl.q_units > 1) {
      rc = get_tensor_map(W, p.V, p.D, (pl.q_units - 1) * 16, kUmmaBK, CU_TENSOR_MAP_SWIZZLE_128B, &mp->wq1);
      if (rc != kOk) return rc;
    }
    rc = get_tensor_map(H, p.B, p.D, pl.h_rows, kUmmaBK, CU_TENSOR_MAP_SWIZZLE_128B, &mp->hm, /*hidden=*/true);
    if (rc != kOk) return rc;
  }
  return kOk;
}

static int launch_umma(DeviceInfo& d, const void* W, const void* H, SampleParams& p, cudaStream_t stream,
                       size_t cand_capacity) {
  // Row replicas keep the S > 1 scratch by TMEM lane (128 rows): without room for that, run without them.
  const int copies_cap =
      ((p.flags & kFlagTopk) || (p.S > 1 && (size_t)128 * p.S > cand_capacity)) ? 1 : umma_copies_cap();
  // The split epilogue of 64-row accumulators keeps the S > 1 scratch by TMEM lane as well.
  int m_force = umma_m64();
  if (p.S > 1 && !(p.flags & kFlagTopk) && (size_t)128 * p.S > cand_capacity) m_force = 0;
  UmmaPlan pl = umma_plan(p.V, p.B, d.num_sms, d.max_smem_optin, umma_stage_cap(), umma_mt2_nt_cap(),
                          umma_nt_target(), umma_min_tiles(), p.D, umma_slabs_force(), copies_cap, m_force);
  if (pl.grid * kUmmaEpiGroups > kMaxParts) return -kErrUnsupported;
  UmmaMaps mp;
  int rc = build_umma_maps(W, H, p, pl, &mp);
  if (rc != kOk && pl.slabs > 1) {
    // the driver refused the 3-D view: fall back to one slab per operation
    pl = umma_plan(p.V, p.B, d.num_sms, d.max_smem_optin, umma_stage_cap(), umma_mt2_nt_cap(), umma_nt_target(),
                   umma_min_tiles(), 0, 0, copies_cap, m_force);
    rc = build_umma_maps(W, H, p, pl, &mp);
  }
  if (rc != kOk) return -rc;
  if (pl.copies > 1 || (pl.m_rows == 64 && p.S > 1 && !(p.flags & kFlagTopk))) {
    p.cand_rows = 128;
    p.cand_idx = reinterpret_cast<int*>(p.cand_val + (size_t)kMaxParts * 128 * p.S);
  }
  p.stages = pl.stages;
  p.tile_rows = pl.q_units * 16;
  p.tiles_per_cta = pl.tiles_per_cta;
  p.lse_parts = pl.grid;
  rc = pl.mt == 1 ? launch_umma_mt<1>(d, mp, p, pl, stream) : launch_umma_mt<2>(d, mp, p, pl, stream);
  if (rc != kOk) return -rc;
  return pl.grid * kUmmaEpiGroups;
}

// ---- CTA-pair tensor-core launch (129..256 batch rows) -----------------------------------
static int pair_enabled() {
  static const int v = std::getenv("FMMS_UMMA_PAIR") ? env_int("FMMS_UMMA_PAIR") : 1;
  return v;
}

// CTA pairs pay off once a pair has several tiles to walk; short shards stay on the single-CTA
// kernel with two M tiles (measured on a 18992-row shard: 56 us vs 60 us).  FMMS_UMMA_PAIR=0
// switches the pair kernel off, =2 forces it for every batch above 128.
static bool use_pair_kernel(int V, int D, int B, int num_sms) {
  if (B <= 128 || D % 64 != 0 || num_sms < 2 || pair_enabled() == 0) return false;
  return pair_enabled() == 2 || V >= 32768;
}

static int launch_umma_pair(DeviceInfo& d, const void* W, const void* H, SampleParams& p, cudaStream_t stream) {
  const PairPlan pl = pair_plan(p.V, p.D, d.num_sms, d.max_smem_optin, umma_slabs_force());
  if (pl.grid * kUmmaEpiGroups > kMaxParts) return -kErrUnsupported;
  CUtensorMap wq, wq1, hm;
  int rc = get_tensor_map_slabs(W, p.V, p.D, pl.q_units * 16, pl.slabs, &wq);
  if (rc != kOk) return -rc;
  wq1 = wq;
  if (pl.q_units > 1) {
    rc = get_tensor_map_slabs(W, p.V, p.D, (pl.q_units - 1) * 16, pl.slabs, &wq1);
    if (rc != kOk) return -rc;
  }
  rc = get_tensor_map_slabs(H, p.B, p.D, 128, pl.slabs, &hm, /*hidden=*/true);
  if (rc != kOk) return -rc;
  const bool lse = (p.flags & kFlagLogprob) != 0;
  if (!d.umma_attr[lse][3]) {
    if (cudaFuncSetAttribute(lse ? umma_pair_sample_kernel<true> : umma_pair_sample_kernel<false>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, d.max_smem_optin) != cudaSuccess)
      return -kErrCuda;
    d.umma_attr[lse][3] = true;
  }
  p.stages = pl.stages;
  p.tile_rows = pl.q_units * kPairUnitRows;
  p.tiles_per_cta = pl.tiles_per_pair;
  p.lse_parts = pl.grid / 2;
  const cudaError_t err =
      lse ? launch_kernel(umma_pair_sample_kernel<true>, pl.grid, kUmmaThreads, pl.smem, stream, wq, wq1, hm, p,
                          pl.units_total, pl.q_units, pl.slabs)
          : launch_kernel(umma_pair_sample_kernel<false>, pl.grid, kUmmaThreads, pl.smem, stream, wq, wq1, hm, p,
                          pl.units_total, pl.q_units, pl.slabs);
  if (err != cudaSuccess) return -kErrCuda;
  return pl.grid * kUmmaEpiGroups;
}

// ---- measurement helper: evict L2 with a read-only sweep (leaves no dirty lines behind) ----
__global__ void l2_sweep_kernel(const uint4* __restrict__ p, size_t n16, unsigned int* sink) {
  unsigned int acc = 0;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (size_t)gridDim.x * blockDim.x) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p + i));
    acc ^= v.x ^ v.y ^ v.z ^ v.w;
  }
  if (acc == 0x9e3779b9u && sink) *sink = acc;  // keeps the loads alive; practically never true
}

// ---- built-in scratch for callers that cannot allocate --------------------------------
// Candidate scratch of fmms_sample_static(): room for kMaxParts candidate rows of up to
// kStaticMaxItems (batch rows x draws) entries, 8 bytes each.  Every GPU on which the
// library's module is loaded holds these bytes until the process exits.
constexpr int kStaticMaxItems = 1024;
constexpr size_t kStaticScratchBytes = kWsHeadBytes + (size_t)kStaticMaxItems * 8 * (1 + (size_t)kMaxParts);
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// In host code `g_static_scratch` is only a handle for the runtime, not a device address;
// the address is looked up once per device (with that device current) and cached here.
static void* g_static_scratch_ptr[kMaxDevices] = {};

static int static_scratch_ptr(void** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return kErrCuda;
  if (dev < 0 || dev >= kMaxDevices) return kErrUnsupported;
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_static_scratch_ptr[dev]) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_static_scratch) != cudaSuccess || !ptr) return kErrCuda;
    g_static_scratch_ptr[dev] = ptr;
  }
  *out = g_static_scratch_ptr[dev];
  return kOk;
}

}  // namespace fmms

using namespace fmms;

extern "C" {

int fmms_version(void) { return kVersion; }

const char* fmms_strerror(int status) {
  switch (status) {
    case FMMS_OK: return "ok";
    case FMMS_ERR_TIMEOUT: return "a bounded device-side wait timed out";
    case FMMS_ERR_BAD_ARG: return "bad argument";
    case FMMS_ERR_UNSUPPORTED: return "unsupported shape or alignment";
    case FMMS_ERR_WORKSPACE: return "workspace missing or too small";
    case FMMS_ERR_CUDA: return "CUDA call failed";
    case FMMS_ERR_ARCH: return "device is not compute capability 10.x (sm_100a)";
    case FMMS_ERR_TOO_LARGE: return "batch rows x draws exceeds the built-in scratch (fmms_static_max_items)";
    case FMMS_ERR_TOPK_OVERFLOW: return "a row's top-k candidate list overflowed and no scratch for the exact pass was given";
    default: return "unknown status";
  }
}

int fmms_num_sms(int* num_sms) {
  if (!num_sms) return FMMS_ERR_BAD_ARG;
  DeviceInfo* d = nullptr;
  int rc = device_info(&d);
  if (rc != kOk) return rc;
  *num_sms = d->num_sms;
  return FMMS_OK;
}

int fmms_query_workspace(int V_local, int D, int B, int S, size_t* bytes) {
  if (!bytes || V_local <= 0 || D <= 0 || B <= 0 || S <= 0) return FMMS_ERR_BAD_ARG;
  // With several draws per row the tensor-core kernel keeps running candidates in the workspace, one
  // row per TMEM lane (128) for a batch of at most 64 rows: with 64-row accumulators two lanes scan for
  // each row and keep separate candidates.
  const int rows = B > 256 ? 256 : ((S > 1 && B <= 64) ? 128 : B);
  *bytes = workspace_bytes_for(rows, S);
  return FMMS_OK;
}

int fmms_last_path(void) { return g_last_path; }

int fmms_plan(int V_local, int D, int B, int S, int flags, int num_sms, int max_smem_bytes, int* plan) {
  if (!plan || V_local <= 0 || D <= 0 || B <= 0 || S <= 0 || num_sms <= 0 || max_smem_bytes <= 0)
    return FMMS_ERR_BAD_ARG;
  if (D % 8 != 0 || B > 256) return FMMS_ERR_UNSUPPORTED;
  DeviceInfo d;
  d.num_sms = num_sms;
  d.max_smem_optin = max_smem_bytes;
  const bool can_gemv = gemv_eligible(d, D, B, S);
  bool use_gemv = can_gemv && B <= kGemvAutoMaxBatch;
  if (flags & FMMS_FLAG_FORCE_GEMV) {
    if (!can_gemv) return FMMS_ERR_UNSUPPORTED;
    use_gemv = true;
  }
  if (flags & FMMS_FLAG_FORCE_MMA) use_gemv = false;
  for (int i = 0; i < 8; ++i) plan[i] = 0;
  if (use_gemv) {
    const int kGemvRows = gemv_rows(B);
    const int groups = (V_local + kGemvRows - 1) / kGemvRows;
    plan[0] = FMMS_PATH_GEMV;
    plan[1] = groups < num_sms ? groups : num_sms;
    plan[2] = kGemvRows;
    plan[3] = (groups + plan[1] - 1) / plan[1];
    plan[4] = gemv_stages(d, B, D);
    plan[5] = 1;
    plan[6] = (int)gemv_smem_bytes(B, D, plan[4], gemv_chunks(B, D));
    plan[7] = plan[1];
  } else {
    if (use_pair_kernel(V_local, D, B, num_sms)) {
      const PairPlan pp = pair_plan(V_local, D, num_sms, max_smem_bytes, 0);
      plan[0] = FMMS_PATH_MMA;
      plan[1] = pp.grid;
      plan[2] = pp.q_units * kPairUnitRows;
      plan[3] = pp.tiles_per_pair;
      plan[4] = pp.stages;
      plan[5] = 2;
      plan[6] = (int)pp.smem;
      plan[7] = pp.grid * kUmmaEpiGroups;
      return FMMS_OK;
    }
    const UmmaPlan pl = umma_plan(V_local, B, num_sms, max_smem_bytes, 0, 256, 0, 1, D, 0, umma_copies_cap());
    plan[0] = FMMS_PATH_MMA;
    plan[1] = pl.grid;
    plan[2] = pl.q_units * 16;
    plan[3] = pl.tiles_per_cta;
    plan[4] = pl.stages;
    plan[5] = pl.mt;
    plan[6] = (int)pl.smem;
    plan[7] = pl.grid * kUmmaEpiGroups;
  }
  return FMMS_OK;
}

struct TpArgs;
static int sample_rows(const void* W_bf16, const void* H_bf16, const float* temperature, int temp_stride,
                       int V_local, int D, int B, int S, unsigned long long seed, long long v_global_offset,
                       int flags, const float* ext_noise, long long noise_ld, long long noise_s_stride, int b_offset,
                       float* logits_out, long long* out_idx, float* out_val, void* workspace,
                       size_t workspace_bytes, int* status_dev, void* stream_v, const TpArgs* tpa,
                       float* out_logprob, float* out_lse, int* status_mirror, const Fp8Args* fp8);

struct TpArgs {
  int rank, world, max_items;
  void* const* peer_buffers;
  unsigned int epoch;
  unsigned long long wait_limit_ns;
};

static int sample_impl(const void* W_bf16, const void* H_bf16, const float* temperature, int temp_stride,
                       int V_local, int D, int B, int S, unsigned long long seed, long long v_global_offset,
                       int flags, const float* ext_noise, long long noise_ld, float* logits_out,
                       long long* out_idx, float* out_val, void* workspace, size_t workspace_bytes,
                       int* status_dev, void* stream_v, const TpArgs* tpa, float* out_logprob = nullptr,
                       float* out_lse = nullptr, int* status_mirror = nullptr, const Fp8Args* fp8 = nullptr) {
  g_last_path = FMMS_PATH_NONE;
  if (!W_bf16 || !H_bf16 || !out_idx || V_local <= 0 || D <= 0 || B <= 0 || S <= 0) return FMMS_ERR_BAD_ARG;
  const bool greedy = flags & FMMS_FLAG_GREEDY, ext = flags & FMMS_FLAG_EXT_NOISE;
  if (!greedy && !temperature) return FMMS_ERR_BAD_ARG;
  if (temp_stride != 0 && temp_stride != 1) return FMMS_ERR_BAD_ARG;
  if (ext && !greedy && (!ext_noise || noise_ld < V_local)) return FMMS_ERR_BAD_ARG;
  if ((flags & FMMS_FLAG_RETURN_LOGITS) && !logits_out) return FMMS_ERR_BAD_ARG;
  if ((flags & FMMS_FLAG_FORCE_GEMV) && (flags & FMMS_FLAG_FORCE_MMA)) return FMMS_ERR_BAD_ARG;
  if (v_global_offset < 0) return FMMS_ERR_BAD_ARG;
  if (flags & FMMS_FLAG_LOGPROB) {
    if (!out_logprob) return FMMS_ERR_BAD_ARG;
    // the log-sum-exp is merged and decoded by the last CTA (under tensor parallelism after the
    // exchange of the shards' partial sums), which the stand-alone second stage does not do
    if (flags & FMMS_FLAG_TWO_STAGE) return FMMS_ERR_UNSUPPORTED;
  }
  if (D % 8 != 0 || ((uintptr_t)W_bf16 & 15) || ((uintptr_t)H_bf16 & 15)) return FMMS_ERR_UNSUPPORTED;
  if (fp8) {
    if (!fp8->w_scale || !fp8->staging || ((uintptr_t)fp8->staging & 255) || ((uintptr_t)fp8->w_scale & 15)) return FMMS_ERR_BAD_ARG;
    if (fp8->staging_bytes < fp8_staging_bytes(D, B > kMaxBatchPerLaunch ? kMaxBatchPerLaunch : B)) return FMMS_ERR_WORKSPACE;
    if (D % 16 != 0 || (flags & (FMMS_FLAG_FORCE_GEMV | FMMS_FLAG_TWO_STAGE))) return FMMS_ERR_UNSUPPORTED;
  }
  if (B > kMaxBatchPerLaunch) {
    // Larger batches run as consecutive launches over blocks of 256 rows (each streams W again,
    // as the reference's 64-row tiles do); the noise stays keyed by the caller's row numbers.
    if (tpa) return FMMS_ERR_UNSUPPORTED;
    for (int b0 = 0; b0 < B; b0 += kMaxBatchPerLaunch) {
      const int nb = B - b0 < kMaxBatchPerLaunch ? B - b0 : kMaxBatchPerLaunch;
      Fp8Args f8{};
      if (fp8) f8 = Fp8Args{fp8->w_scale, fp8->staging, fp8->staging_bytes};
      const int rc = sample_rows(W_bf16, reinterpret_cast<const __nv_bfloat16*>(H_bf16) + (size_t)b0 * D,
                                 temperature ? temperature + (size_t)b0 * temp_stride : nullptr, temp_stride, V_local,
                                 D, nb, S, seed, v_global_offset, flags,
                                 ext_noise ? ext_noise + (size_t)b0 * noise_ld : nullptr, noise_ld,
                                 (long long)B * noise_ld, b0, logits_out ? logits_out + (size_t)b0 * V_local : nullptr,
                                 out_idx + (size_t)b0 * S, out_val ? out_val + (size_t)b0 * S : nullptr, workspace,
                                 workspace_bytes, status_dev, stream_v, nullptr,
                                 out_logprob ? out_logprob + (size_t)b0 * S : nullptr,
                                 out_lse ? out_lse + b0 : nullptr, status_mirror, fp8 ? &f8 : nullptr);
      if (rc != FMMS_OK) return rc;
    }
    return FMMS_OK;
  }
  return sample_rows(W_bf16, H_bf16, temperature, temp_stride, V_local, D, B, S, seed, v_global_offset, flags,
                     ext_noise, noise_ld, (long long)B * noise_ld, 0, logits_out, out_idx, out_val, workspace,
                     workspace_bytes, status_dev, stream_v, tpa, out_logprob, out_lse, status_mirror, fp8);
}

static int sample_rows(const void* W_bf16, const void* H_bf16, const float* temperature, int temp_stride,
                       int V_local, int D, int B, int S, unsigned long long seed, long long v_global_offset,
                       int flags, const float* ext_noise, long long noise_ld, long long noise_s_stride, int b_offset,
                       float* logits_out, long long* out_idx, float* out_val, void* workspace,
                       size_t workspace_bytes, int* status_dev, void* stream_v, const TpArgs* tpa,
                       float* out_logprob, float* out_lse, int* status_mirror, const Fp8Args* fp8) {
  const bool greedy = flags & FMMS_FLAG_GREEDY;
  (void)greedy;
  const size_t need = workspace_bytes_for(B, S);  // the least that works; fmms_query_workspace may ask for more
  if (!workspace || workspace_bytes < need || ((uintptr_t)workspace & 255)) return FMMS_ERR_WORKSPACE;

  DeviceInfo* d = nullptr;
  int rc = device_info(&d);
  if (rc != kOk) return rc;
  if (d->cc_major != 10) return FMMS_ERR_ARCH;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);

  SampleParams p{};
  p.H = reinterpret_cast<const __nv_bfloat16*>(H_bf16);
  p.temperature = temperature;
  p.temp_stride = temp_stride;
  p.V = V_local;
  p.D = D;
  p.B = B;
  p.S = S;
  p.seed = seed;
  p.v_offset = v_global_offset;
  p.flags = flags;
  p.ext_noise = ext_noise;
  p.noise_ld = noise_ld;
  p.noise_s_stride = noise_s_stride;
  p.b_offset = b_offset;
  p.logits_out = logits_out;
  unsigned char* ws = reinterpret_cast<unsigned char*>(workspace);
  const size_t cap = workspace_item_capacity(workspace_bytes);
  p.ticket = reinterpret_cast<unsigned int*>(ws);
  p.sched = p.ticket + 1;
  p.lse = reinterpret_cast<unsigned long long*>(ws + kWsLseOffset);
  p.lse2 = reinterpret_cast<unsigned long long*>(ws + kWsLse2Offset);
  p.out_logprob = out_logprob;
  p.out_lse = out_lse;
  p.keys = reinterpret_cast<unsigned long long*>(ws + kWsHeadBytes);
  p.cand_val = reinterpret_cast<float*>(ws + kWsHeadBytes + cap * 8);
  p.cand_idx = reinterpret_cast<int*>(p.cand_val + (size_t)kMaxParts * B * S);
  p.cand_rows = B;
  p.out_idx = out_idx;
  p.out_val = out_val;
  p.tp_world = 1;
  if (tpa) {
    if (tpa->world < 1 || tpa->world > kTpMaxWorld || tpa->rank < 0 || tpa->rank >= tpa->world || !tpa->peer_buffers)
      return FMMS_ERR_BAD_ARG;
    if ((long long)B * S > tpa->max_items || (flags & FMMS_FLAG_TWO_STAGE)) return FMMS_ERR_UNSUPPORTED;
    p.tp_rank = tpa->rank;
    p.tp_world = tpa->world;
    p.tp_max_items = tpa->max_items;
    p.tp_epoch = tpa->epoch;
    p.tp_wait_ns = tpa->wait_limit_ns ? tpa->wait_limit_ns : kWaitLimitNs;
    for (int r = 0; r < tpa->world; ++r) {
      if (!tpa->peer_buffers[r]) return FMMS_ERR_BAD_ARG;
      p.tp_peers.slots[r] = reinterpret_cast<TpRecord*>(tpa->peer_buffers[r]);
    }
    if (v_global_offset + (long long)V_local > 0xffffffffll) return FMMS_ERR_UNSUPPORTED;  // ids travel as 32 bits
  }
  p.status_dev = status_dev;
  p.status_mirror = status_mirror;
  p.stamps = g_stamps;

  if (fp8) {
    // e4m3 weights: quantise the hidden states (per-row scale) into the staging area, then run the tensor-core
    // kernel on byte matrices that the TMA sees as [rows, D / 2] 16-bit matrices (the same bytes)
    unsigned char* hq = reinterpret_cast<unsigned char*>(fp8->staging);
    float* hs = reinterpret_cast<float*>(hq + (((size_t)B * D + 255) & ~(size_t)255));
    quantize_rows_e4m3_kernel<<<B, 256, 0, stream>>>(p.H, D, hq, hs);
    if (cudaGetLastError() != cudaSuccess) return FMMS_ERR_CUDA;
    p.flags |= kFlagFp8;
    p.w_scale = fp8->w_scale;
    p.h_scale = hs;
    p.D = D / 2;
    g_overlap_next = true;  // the weight stream starts while the quantiser runs
    const int parts8 = use_pair_kernel(V_local, p.D, B, d->num_sms) ? launch_umma_pair(*d, W_bf16, hq, p, stream)
                                                                     : launch_umma(*d, W_bf16, hq, p, stream, cap);
    g_overlap_next = false;
    g_last_path = FMMS_PATH_MMA;
    if (parts8 <= 0) return parts8 == 0 ? FMMS_ERR_CUDA : -parts8;
    return FMMS_OK;
  }
  const bool can_gemv = gemv_eligible(*d, D, B, S);
  bool use_gemv;
  if (flags & FMMS_FLAG_FORCE_GEMV) {
    if (!can_gemv) return FMMS_ERR_UNSUPPORTED;
    use_gemv = true;
  } else if (flags & FMMS_FLAG_FORCE_MMA) {
    use_gemv = false;
  } else {
    use_gemv = can_gemv && B <= kGemvAutoMaxBatch;
  }

  int parts;
  if (use_gemv) {
    parts = launch_gemv(*d, W_bf16, p, stream);
    g_last_path = FMMS_PATH_GEMV;
  } else {
    if (use_pair_kernel(V_local, D, B, d->num_sms))
      parts = launch_umma_pair(*d, W_bf16, H_bf16, p, stream);
    else
      parts = launch_umma(*d, W_bf16, H_bf16, p, stream, cap);
    g_last_path = FMMS_PATH_MMA;
  }
  if (parts <= 0) return parts == 0 ? FMMS_ERR_CUDA : -parts;

  if (flags & FMMS_FLAG_TWO_STAGE) {
    const int n = B * S;
    reduce_candidates_kernel<<<(n + 127) / 128, 128, 0, stream>>>(p.keys, p.sched, B, S, v_global_offset, out_idx,
                                                                   out_val);
    return cudaGetLastError() == cudaSuccess ? FMMS_OK : FMMS_ERR_CUDA;
  }
  return FMMS_OK;
}

int fmms_sample(const void* W_bf16, const void* H_bf16, const float* temperature, int temp_stride,
                int V_local, int D, int B, int S, unsigned long long seed, long long v_global_offset,
                int flags, const float* ext_noise, long long noise_ld, float* logits_out,
                long long* out_idx, float* out_val, void* workspace, size_t workspace_bytes,
                int* status_dev, void* stream) {
  return sample_impl(W_bf16, H_bf16, temperature, temp_stride, V_local, D, B, S, seed, v_global_offset, flags,
                     ext_noise, noise_ld, logits_out, out_idx, out_val, workspace, workspace_bytes, status_dev,
                     stream, nullptr);
}

int fmms_sample_tp(const void* W_bf16, const void* H_bf16, const float* temperature, int temp_stride,
                   int V_local, int D, int B, int S, unsigned long long seed, long long v_global_offset,
                   int flags, const float* ext_noise, long long noise_ld, float* logits_out,
                   long long* out_idx, float* out_val, void* workspace, size_t workspace_bytes,
                   int* status_dev, void* stream, int rank, int world, int max_items,
                   void* const* peer_buffers, unsigned int epoch, unsigned long long wait_limit_ns) {
  const TpArgs tpa{rank, world, max_items, peer_buffers, epoch, wait_limit_ns};
  return sample_impl(W_bf16, H_bf16, temperature, temp_stride, V_local, D, B, S, seed, v_global_offset, flags,
                     ext_noise, noise_ld, logits_out, out_idx, out_val, workspace, workspace_bytes, status_dev,
                     stream, &tpa);
}
int fmms_sample_logprobs(const void* W_bf16, const void* H_bf16, const float* temperature, int temp_stride,
                         int V_local, int D, int B, int S, unsigned long long seed, long long v_global_offset,
                         int flags, const float* ext_noise, long long noise_ld, float* logits_out,
                         long long* out_idx, float* out_val, void* workspace, size_t workspace_bytes,
                         int* status_dev, void* stream, float* out_logprob, float* out_lse) {
  return sample_impl(W_bf16, H_bf16, temperature, temp_stride, V_local, D, B, S, seed, v_global_offset,
                     flags | FMMS_FLAG_LOGPROB, ext_noise, noise_ld, logits_out, out_idx, out_val, workspace,
                     workspace_bytes, status_dev, stream, nullptr, out_logprob, out_lse);
}

// ---- one descriptor for every variant; host-memory inputs and outputs --------------------
static size_t align256(size_t n) { return (n + 255) & ~(size_t)255; }

struct StagingLayout {
  size_t h, t, idx, val, lp, lse, total;
};
static StagingLayout staging_layout(int D, int B, int S) {
  StagingLayout l{};
  size_t off = 0;
  l.h = off;   off += align256((size_t)B * D * 2);
  l.t = off;   off += align256((size_t)B * 4);
  l.idx = off; off += align256((size_t)B * S * 8);
  l.val = off; off += align256((size_t)B * S * 4);
  l.lp = off;  off += align256((size_t)B * S * 4);
  l.lse = off; off += align256((size_t)B * 4);
  l.total = off;
  return l;
}

int fmms_query_staging(int D, int B, int S, size_t* bytes) {
  if (!bytes || D <= 0 || B <= 0 || S <= 0) return FMMS_ERR_BAD_ARG;
  *bytes = staging_layout(D, B, S).total;  // also covers the quantised hidden states of FMMS_FLAG_W_FP8
  return FMMS_OK;
}

// ---- top-k / top-p -----------------------------------------------------------------------
// Scratch layout: a head that is zero between calls, laid out for 256 rows whatever the batch (calls of
// different batch sizes share one scratch, and the parts behind the head keep stale data):
// [table 256 x 64 u32][segment counts 256 x 640 u32][gbar, need_fallback: 256 B][row_fallback 256][ids of the
// conditional pass 256 x 8][spill counts 256 u32], then [segments B x 640 x 16 x 8][spill lists B x 2048 x 8]
// [logits B x V x 4].
struct TopkLayout {
  size_t table, count, words, rows, dummy_idx, extra_count, list, extra, logits, total_small, total_full;
};
static TopkLayout topk_layout(int V, int B) {
  TopkLayout l{};
  size_t off = 0;
  const size_t rows = kMaxBatchPerLaunch;
  l.table = off;     off += align256(rows * kTopkSlots * 4);
  l.count = off;     off += align256(rows * kTopkMaxSegs * 4);
  l.words = off;     off += 256;
  l.rows = off;      off += align256(rows);
  l.dummy_idx = off; off += align256(rows * 8);
  l.extra_count = off; off += align256(rows * 4);
  l.list = off;      off += align256((size_t)B * kTopkMaxSegs * kTopkSegCap * 8);
  l.extra = off;     off += align256((size_t)B * kTopkExtraCap * 8);
  l.total_small = off;
  l.logits = off;    off += align256((size_t)B * V * 4);
  l.total_full = off;
  return l;
}

int fmms_query_topk_workspace(int V_local, int B, size_t* bytes, size_t* bytes_without_exact_pass) {
  if (!bytes || V_local <= 0 || B <= 0) return FMMS_ERR_BAD_ARG;
  const TopkLayout l = topk_layout(V_local, B > kMaxBatchPerLaunch ? kMaxBatchPerLaunch : B);
  *bytes = l.total_full;
  if (bytes_without_exact_pass) *bytes_without_exact_pass = l.total_small;
  return FMMS_OK;
}

// One block of at most 256 rows: candidate pass, finish, conditional exact pass.
static int topk_rows(const fmms_call_t& c, int b0, int nb) {
  DeviceInfo* d = nullptr;
  int rc = device_info(&d);
  if (rc != kOk) return rc;
  if (d->cc_major != 10) return FMMS_ERR_ARCH;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(c.stream);
  const TopkLayout l = topk_layout(c.V_local, nb);
  if (c.topk_workspace_bytes < l.total_small) return FMMS_ERR_WORKSPACE;
  const bool exact_pass = c.topk_workspace_bytes >= l.total_full;
  unsigned char* tw = reinterpret_cast<unsigned char*>(c.topk_workspace);
  unsigned char* ws = reinterpret_cast<unsigned char*>(c.workspace);

  SampleParams p{};
  p.H = reinterpret_cast<const __nv_bfloat16*>(c.H_bf16) + (size_t)b0 * c.D;
  p.temperature = c.temperature ? c.temperature + (size_t)b0 * c.temp_stride : nullptr;
  p.temp_stride = c.temp_stride;
  p.V = c.V_local;
  p.D = c.D;
  p.B = nb;
  p.S = c.S;
  p.seed = c.seed;
  p.v_offset = c.v_global_offset;
  p.flags = (c.flags & (FMMS_FLAG_GREEDY | FMMS_FLAG_EXT_NOISE | FMMS_FLAG_SEED_DEVICE)) | kFlagTopk;
  p.ext_noise = c.ext_noise ? c.ext_noise + (size_t)b0 * c.noise_ld : nullptr;
  p.noise_ld = c.noise_ld;
  p.noise_s_stride = (long long)c.B * c.noise_ld;
  p.b_offset = b0;
  p.ticket = reinterpret_cast<unsigned int*>(ws);
  p.sched = p.ticket + 1;
  p.keys = reinterpret_cast<unsigned long long*>(ws + kWsHeadBytes);
  p.cand_val = reinterpret_cast<float*>(ws + kWsHeadBytes + workspace_item_capacity(c.workspace_bytes) * 8);
  p.cand_idx = reinterpret_cast<int*>(p.cand_val);
  p.cand_rows = nb;
  p.lse = reinterpret_cast<unsigned long long*>(ws + kWsLseOffset);
  p.lse2 = reinterpret_cast<unsigned long long*>(ws + kWsLse2Offset);
  p.out_idx = c.out_idx + (size_t)b0 * c.S;
  p.out_val = c.out_val ? c.out_val + (size_t)b0 * c.S : nullptr;
  p.out_logprob = c.out_logprob ? c.out_logprob + (size_t)b0 * c.S : nullptr;
  p.out_lse = c.out_lse ? c.out_lse + b0 : nullptr;
  p.status_dev = c.status_dev;
  p.stamps = g_stamps;
  p.tp_world = 1;
  p.topk.k = c.top_k;
  p.topk.top_p = c.top_p;
  p.topk.table = reinterpret_cast<unsigned int*>(tw + l.table);
  p.topk.seg_count = reinterpret_cast<unsigned int*>(tw + l.count);
  p.topk.gbar = reinterpret_cast<unsigned int*>(tw + l.words);
  p.topk.need_fallback = p.topk.gbar + 1;
  p.topk.row_fallback = tw + l.rows;
  p.topk.list = reinterpret_cast<unsigned long long*>(tw + l.list);
  p.topk.extra_count = reinterpret_cast<unsigned int*>(tw + l.extra_count);
  p.topk.extra = reinterpret_cast<unsigned long long*>(tw + l.extra);

  const void* h_operand = p.H;
  if (c.flags & FMMS_FLAG_W_FP8) {
    // e4m3 weights: quantised hidden states in the staging area, byte matrices seen as [rows, D / 2] (see sample_rows)
    if (!c.w_scale || !c.staging || ((uintptr_t)c.staging & 255) || c.staging_bytes < fp8_staging_bytes(c.D, nb))
      return FMMS_ERR_WORKSPACE;
    if (c.D % 16 != 0) return FMMS_ERR_UNSUPPORTED;
    unsigned char* hq = reinterpret_cast<unsigned char*>(c.staging);
    float* hs = reinterpret_cast<float*>(hq + (((size_t)nb * c.D + 255) & ~(size_t)255));
    quantize_rows_e4m3_kernel<<<nb, 256, 0, stream>>>(p.H, c.D, hq, hs);
    if (cudaGetLastError() != cudaSuccess) return FMMS_ERR_CUDA;
    p.flags |= kFlagFp8;
    p.w_scale = c.w_scale;
    p.h_scale = hs;
    p.D = c.D / 2;
    h_operand = hq;
    g_overlap_next = true;
  }
  // 1. candidate pass (tensor-core kernel, never the CTA-pair variant), 2. one CTA per row finishes
  int parts = launch_umma(*d, c.W_bf16, h_operand, p, stream, 0);
  g_overlap_next = false;
  if (parts <= 0) return parts == 0 ? FMMS_ERR_CUDA : -parts;
  p.topk.nseg = parts;  // CTAs x column groups x segments per thread: 4 x 1 with one M tile, 2 x 2 with two
  // The follow-up kernels are launched with programmatic stream serialisation: each becomes resident while its
  // producer still runs and waits (griddepcontrol.wait) for it before touching anything, which hides their launch
  // latencies behind one another.
  g_overlap_next = true;
  if (launch_kernel(topk_finish_kernel, nb, kTopkFinishThreads, kTopkListCap * sizeof(unsigned long long), stream, p) !=
      cudaSuccess)
    return FMMS_ERR_CUDA;
  // 3. rows whose list overflowed: a conditional greedy pass writes all logits, then exact selection
  if (exact_pass) {
    SampleParams q = p;
    q.flags = FMMS_FLAG_GREEDY | FMMS_FLAG_RETURN_LOGITS | (p.flags & kFlagFp8);
    q.S = 1;
    q.logits_out = reinterpret_cast<float*>(tw + l.logits);
    q.out_idx = reinterpret_cast<long long*>(tw + l.dummy_idx);
    q.out_val = q.out_logprob = q.out_lse = nullptr;
    q.run_if = p.topk.need_fallback;
    q.topk = TopkArgs{};
    g_overlap_next = true;
    parts = launch_umma(*d, c.W_bf16, h_operand, q, stream, 0);
    g_overlap_next = false;
    if (parts <= 0) return parts == 0 ? FMMS_ERR_CUDA : -parts;
    g_overlap_next = true;
    if (launch_kernel(topk_exact_kernel, nb, kTopkExactThreads, 0, stream, p, (const float*)q.logits_out) != cudaSuccess)
      return FMMS_ERR_CUDA;
  } else {
    g_overlap_next = true;
    if (launch_kernel(topk_overflow_kernel, nb, 128, 0, stream, p) != cudaSuccess) return FMMS_ERR_CUDA;
  }
  g_last_path = FMMS_PATH_MMA;
  return cudaGetLastError() == cudaSuccess ? FMMS_OK : FMMS_ERR_CUDA;
}

static int topk_impl(const fmms_call_t& c) {
  g_last_path = FMMS_PATH_NONE;
  if (!c.W_bf16 || !c.H_bf16 || !c.out_idx || c.V_local <= 0 || c.D <= 0 || c.B <= 0 || c.S <= 0) return FMMS_ERR_BAD_ARG;
  if (c.top_k < 1 || c.top_k > kTopkSlots) return FMMS_ERR_UNSUPPORTED;
  const bool greedy = c.flags & FMMS_FLAG_GREEDY, ext = c.flags & FMMS_FLAG_EXT_NOISE;
  if (!greedy && !c.temperature) return FMMS_ERR_BAD_ARG;
  if (c.temp_stride != 0 && c.temp_stride != 1) return FMMS_ERR_BAD_ARG;
  if (ext && !greedy && (!c.ext_noise || c.noise_ld < c.V_local)) return FMMS_ERR_BAD_ARG;
  if (c.tp_world > 1 || (c.flags & (FMMS_FLAG_RETURN_LOGITS | FMMS_FLAG_TWO_STAGE | FMMS_FLAG_HOST_IO | FMMS_FLAG_FORCE_GEMV)))
    return FMMS_ERR_UNSUPPORTED;
  if (c.D % 8 != 0 || ((uintptr_t)c.W_bf16 & 15) || ((uintptr_t)c.H_bf16 & 15)) return FMMS_ERR_UNSUPPORTED;
  if (!c.workspace || c.workspace_bytes < workspace_bytes_for(1, 1) || ((uintptr_t)c.workspace & 255)) return FMMS_ERR_WORKSPACE;
  if (!c.topk_workspace || ((uintptr_t)c.topk_workspace & 255)) return FMMS_ERR_WORKSPACE;
  for (int b0 = 0; b0 < c.B; b0 += kMaxBatchPerLaunch) {
    const int nb = c.B - b0 < kMaxBatchPerLaunch ? c.B - b0 : kMaxBatchPerLaunch;
    const int rc = topk_rows(c, b0, nb);
    if (rc != FMMS_OK) return rc;
  }
  return FMMS_OK;
}

// Device-visible address of a host pointer (pinned or registered memory under unified addressing),
// or null for pageable memory.  Asked afresh on every call: an address that was pinned memory once
// may be pageable memory later.
static void* host_ptr_on_device(const void* host) {
  if (!host) return nullptr;
  cudaPointerAttributes a{};
  if (cudaPointerGetAttributes(&a, host) == cudaSuccess && a.type == cudaMemoryTypeHost) return a.devicePointer;
  cudaGetLastError();  // pageable memory is not an error here
  return nullptr;
}

// Hidden states and temperatures from device-visible host memory into the staging buffer: one small
// kernel in place of two copy-engine operations (each of which costs a hand-over between the copy
// and the compute engine, several microseconds, before the sampling kernel may start).
static __global__ void stage_host_inputs_kernel(const uint4* __restrict__ h_src, uint4* __restrict__ h_dst, size_t n16,
                                         const float* __restrict__ t_src, float* __restrict__ t_dst, int nt) {
  griddep_launch_dependents();  // the sampling kernel behind this one may start its weight stream now
  const size_t i0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = i0; i < n16; i += stride) h_dst[i] = h_src[i];
  for (size_t i = i0; i < (size_t)nt; i += stride) t_dst[i] = t_src[i];
}

int fmms_run(const fmms_call_t* c) {
  if (!c || c->struct_bytes != sizeof(fmms_call_t)) return FMMS_ERR_BAD_ARG;
  if (c->top_k != 0) return topk_impl(*c);
  const int kernel_flags = c->flags & ~(FMMS_FLAG_HOST_IO | FMMS_FLAG_NO_SYNC);
  TpArgs tpa{c->tp_rank, c->tp_world, c->tp_max_items, c->tp_peer_buffers, c->tp_epoch, c->tp_wait_limit_ns};
  const TpArgs* tp = c->tp_world > 1 ? &tpa : nullptr;
  const Fp8Args f8{c->w_scale, c->staging, c->staging_bytes};
  const bool fp8 = (c->flags & FMMS_FLAG_W_FP8) != 0;
  if (fp8 && (c->flags & FMMS_FLAG_HOST_IO)) return FMMS_ERR_UNSUPPORTED;
  if (!(c->flags & FMMS_FLAG_HOST_IO))
    return sample_impl(c->W_bf16, c->H_bf16, c->temperature, c->temp_stride, c->V_local, c->D, c->B, c->S, c->seed,
                       c->v_global_offset, kernel_flags & ~FMMS_FLAG_W_FP8, c->ext_noise, c->noise_ld, c->logits_out,
                       c->out_idx, c->out_val, c->workspace, c->workspace_bytes, c->status_dev, c->stream, tp,
                       c->out_logprob, c->out_lse, nullptr, fp8 ? &f8 : nullptr);
  // host-memory hidden states, temperatures and results
  if (!c->H_bf16 || !c->out_idx || c->D <= 0 || c->B <= 0 || c->S <= 0 || c->D % 8 != 0) return FMMS_ERR_BAD_ARG;
  const StagingLayout l = staging_layout(c->D, c->B, c->S);
  if (!c->staging || c->staging_bytes < l.total || ((uintptr_t)c->staging & 255)) return FMMS_ERR_WORKSPACE;
  if ((c->flags & FMMS_FLAG_LOGPROB) && !c->out_logprob) return FMMS_ERR_BAD_ARG;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(c->stream);
  unsigned char* st = reinterpret_cast<unsigned char*>(c->staging);
  const size_t n_items = (size_t)c->B * c->S;
  const size_t h_bytes = (size_t)c->B * c->D * 2;
  const int nt = c->temperature ? (c->temp_stride ? c->B : 1) : 0;

  // Inputs.  Device-visible (pinned) host memory, 16-byte aligned: one gather kernel; else copies.
  void* h_map = host_ptr_on_device(c->H_bf16);
  void* t_map = nt ? host_ptr_on_device(c->temperature) : nullptr;
  const float* temp_dev = nt ? reinterpret_cast<const float*>(st + l.t) : nullptr;
  if (h_map && (!nt || t_map) && !((uintptr_t)h_map & 15)) {
    const size_t n16 = h_bytes / 16;
    int blocks = (int)((n16 + 255) / 256);
    if (blocks > 296) blocks = 296;
    if (blocks < 1) blocks = 1;
    stage_host_inputs_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<const uint4*>(h_map),
                                                         reinterpret_cast<uint4*>(st + l.h), n16,
                                                         reinterpret_cast<const float*>(t_map),
                                                         reinterpret_cast<float*>(st + l.t), nt);
    if (cudaGetLastError() != cudaSuccess) return FMMS_ERR_CUDA;
    g_overlap_next = true;  // the sampling kernel's weight stream starts while the gather runs
  } else {
    if (cudaMemcpyAsync(st + l.h, c->H_bf16, h_bytes, cudaMemcpyHostToDevice, stream) != cudaSuccess) return FMMS_ERR_CUDA;
    if (nt && cudaMemcpyAsync(st + l.t, c->temperature, (size_t)nt * 4, cudaMemcpyHostToDevice, stream) != cudaSuccess)
      return FMMS_ERR_CUDA;
  }

  // Outputs.  Into device-visible host memory the kernel's last CTA writes directly (a few hundred
  // bytes over the bus, no copy operation behind the kernel); pageable memory goes through staging.
  long long* idx_map = reinterpret_cast<long long*>(host_ptr_on_device(c->out_idx));
  float* val_map = c->out_val ? reinterpret_cast<float*>(host_ptr_on_device(c->out_val)) : nullptr;
  float* lp_map = c->out_logprob ? reinterpret_cast<float*>(host_ptr_on_device(c->out_logprob)) : nullptr;
  float* lse_map = c->out_lse ? reinterpret_cast<float*>(host_ptr_on_device(c->out_lse)) : nullptr;
  int* status_map = (c->status_host && c->status_dev) ? reinterpret_cast<int*>(host_ptr_on_device(c->status_host)) : nullptr;
  const bool direct = idx_map && (!c->out_val || val_map) && (!c->out_logprob || lp_map) && (!c->out_lse || lse_map) &&
                      (!(c->status_host && c->status_dev) || status_map);
  int rc;
  struct ClearOverlap {
    ~ClearOverlap() { g_overlap_next = false; }
  } clear_overlap;  // whatever path the call takes from here
  if (direct) {
    rc = sample_impl(c->W_bf16, st + l.h, temp_dev, c->temp_stride, c->V_local, c->D, c->B, c->S, c->seed,
                     c->v_global_offset, kernel_flags, c->ext_noise, c->noise_ld, c->logits_out, idx_map, val_map,
                     c->workspace, c->workspace_bytes, c->status_dev, c->stream, tp, lp_map, lse_map, status_map);
    if (rc != FMMS_OK) return rc;
  } else {
    rc = sample_impl(c->W_bf16, st + l.h, temp_dev, c->temp_stride, c->V_local, c->D, c->B, c->S, c->seed,
                     c->v_global_offset, kernel_flags, c->ext_noise, c->noise_ld, c->logits_out,
                     reinterpret_cast<long long*>(st + l.idx),
                     c->out_val ? reinterpret_cast<float*>(st + l.val) : nullptr, c->workspace, c->workspace_bytes,
                     c->status_dev, c->stream, tp, c->out_logprob ? reinterpret_cast<float*>(st + l.lp) : nullptr,
                     c->out_lse ? reinterpret_cast<float*>(st + l.lse) : nullptr);
    if (rc != FMMS_OK) return rc;
    bool ok = cudaMemcpyAsync(c->out_idx, st + l.idx, n_items * 8, cudaMemcpyDeviceToHost, stream) == cudaSuccess;
    if (c->out_val) ok = ok && cudaMemcpyAsync(c->out_val, st + l.val, n_items * 4, cudaMemcpyDeviceToHost, stream) == cudaSuccess;
    if (c->out_logprob) ok = ok && cudaMemcpyAsync(c->out_logprob, st + l.lp, n_items * 4, cudaMemcpyDeviceToHost, stream) == cudaSuccess;
    if (c->out_lse) ok = ok && cudaMemcpyAsync(c->out_lse, st + l.lse, (size_t)c->B * 4, cudaMemcpyDeviceToHost, stream) == cudaSuccess;
    if (c->status_host && c->status_dev)
      ok = ok && cudaMemcpyAsync(c->status_host, c->status_dev, 4, cudaMemcpyDeviceToHost, stream) == cudaSuccess;
    if (!ok) return FMMS_ERR_CUDA;
  }
  if (!(c->flags & FMMS_FLAG_NO_SYNC) && cudaStreamSynchronize(stream) != cudaSuccess) return FMMS_ERR_CUDA;
  return FMMS_OK;
}

// ---- tensor-parallel exchange -----------------------------------------------------------
int fmms_tp_buffer_bytes(int world, int max_items, size_t* bytes) {
  if (!bytes || world < 1 || world > kTpMaxWorld || max_items < 1) return FMMS_ERR_BAD_ARG;
  *bytes = tp_buffer_bytes(world, max_items);
  return FMMS_OK;
}

int fmms_tp_alloc(size_t bytes, void** dev_ptr, void* ipc_handle_64) {
  if (!dev_ptr || !ipc_handle_64 || bytes == 0) return FMMS_ERR_BAD_ARG;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle is 64 bytes");
  void* p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess) return FMMS_ERR_CUDA;
  if (cudaMemset(p, 0, bytes) != cudaSuccess) {
    cudaFree(p);
    return FMMS_ERR_CUDA;
  }
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) {
    cudaFree(p);
    return FMMS_ERR_CUDA;
  }
  memcpy(ipc_handle_64, &h, 64);
  *dev_ptr = p;
  return FMMS_OK;
}

int fmms_tp_open(const void* ipc_handle_64, void** peer_ptr) {
  if (!ipc_handle_64 || !peer_ptr) return FMMS_ERR_BAD_ARG;
  cudaIpcMemHandle_t h;
  memcpy(&h, ipc_handle_64, 64);
  void* p = nullptr;
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) return FMMS_ERR_CUDA;
  *peer_ptr = p;
  return FMMS_OK;
}

int fmms_tp_close(void* peer_ptr) {
  if (!peer_ptr) return FMMS_ERR_BAD_ARG;
  return cudaIpcCloseMemHandle(peer_ptr) == cudaSuccess ? FMMS_OK : FMMS_ERR_CUDA;
}

int fmms_tp_free(void* dev_ptr) {
  if (!dev_ptr) return FMMS_ERR_BAD_ARG;
  return cudaFree(dev_ptr) == cudaSuccess ? FMMS_OK : FMMS_ERR_CUDA;
}

int fmms_tp_exchange(const long long* local_idx, const float* local_val, int n_items, int max_items, int rank,
                     int world, void* const* peer_buffers, unsigned int epoch,
                     unsigned long long wait_limit_ns, long long* out_idx, float* out_val, int* status_dev,
                     void* stream) {
  if (!local_idx || !local_val || !out_idx || !peer_buffers) return FMMS_ERR_BAD_ARG;
  if (world < 1 || world > kTpMaxWorld || rank < 0 || rank >= world) return FMMS_ERR_BAD_ARG;
  if (n_items < 1 || n_items > max_items) return FMMS_ERR_BAD_ARG;
  TpPeers peers{};
  for (int r = 0; r < world; ++r) {
    if (!peer_buffers[r]) return FMMS_ERR_BAD_ARG;
    peers.slots[r] = reinterpret_cast<TpRecord*>(peer_buffers[r]);
  }
  const int threads = n_items >= 1024 ? 1024 : ((n_items + 31) / 32 * 32 < 32 ? 32 : (n_items + 31) / 32 * 32);
  tp_exchange_kernel<<<1, threads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      local_idx, local_val, n_items, max_items, rank, world, peers, epoch,
      wait_limit_ns ? wait_limit_ns : kWaitLimitNs, out_idx, out_val, status_dev);
  return cudaGetLastError() == cudaSuccess ? FMMS_OK : FMMS_ERR_CUDA;
}

int fmms_debug_stamps(unsigned long long* stamps_dev) {
  g_stamps = stamps_dev;
  return FMMS_OK;
}

int fmms_l2_sweep(const void* buffer, size_t bytes, void* stream) {
  if (!buffer || bytes < 16 || ((uintptr_t)buffer & 15)) return FMMS_ERR_BAD_ARG;
  DeviceInfo* d = nullptr;
  const int rc = device_info(&d);
  if (rc != kOk) return rc;
  l2_sweep_kernel<<<d->num_sms * 8, 512, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint4*>(buffer), bytes / 16, nullptr);
  return cudaGetLastError() == cudaSuccess ? FMMS_OK : FMMS_ERR_CUDA;
}

int fmms_static_max_items(void) { return kStaticMaxItems; }

int fmms_static_reset(void* stream) {
  void* scratch = nullptr;
  const int rc = static_scratch_ptr(&scratch);
  if (rc != kOk) return rc;
  // the part that calls rely on being zero: CTA counter, work counter and the packed winners
  const size_t head = kWsHeadBytes + (size_t)kStaticMaxItems * 8;
  return cudaMemsetAsync(scratch, 0, head, reinterpret_cast<cudaStream_t>(stream)) == cudaSuccess ? FMMS_OK : FMMS_ERR_CUDA;
}

int fmms_sample_static(const void* W_bf16, const void* H_bf16, const float* temperature, int temp_stride,
                       int V_local, int D, int B, int S, unsigned long long seed, long long v_global_offset,
                       int flags, const float* ext_noise, long long noise_ld, float* logits_out,
                       long long* out_idx, float* out_val, int* status_dev, void* stream) {
  if (B <= 0 || S <= 0) return FMMS_ERR_BAD_ARG;
  if ((long long)B * (long long)S > kStaticMaxItems) return FMMS_ERR_TOO_LARGE;
  void* scratch = nullptr;
  const int rc = static_scratch_ptr(&scratch);  // first call on a device: symbol-address look-up
  if (rc != kOk) return rc;
  // The head of the scratch (packed winners and the CTA counter) has to be zero when a call
  // starts: the array is zero when the module is loaded, and every call's last CTA puts the
  // zeros back after decoding, so nothing is cleared here.  The running candidates behind it
  // are initialised by the kernel that uses them.
  return fmms_sample(W_bf16, H_bf16, temperature, temp_stride, V_local, D, B, S, seed, v_global_offset, flags,
                     ext_noise, noise_ld, logits_out, out_idx, out_val, scratch, kStaticScratchBytes, status_dev,
                     stream);
}

}  // extern "C"
