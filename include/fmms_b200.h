/*
 * fmms_b200.h - C ABI of the B200 (sm_100a) fused LM-head sampling library.
 *
 * One pass over a bf16 LM-head weight W[V, D] computes, for every hidden-state
 * row h_b, token ids distributed as softmax(W h_b / T_b) without ever writing
 * logits to memory: logits are formed tile by tile, Gumbel noise is added on
 * chip and only (max, index) candidates survive (Gumbel-max trick).
 *
 * Conventions for every entry point
 *   - plain C types only; all data pointers are DEVICE pointers owned by the
 *     caller; nothing is allocated or freed on the sampling path;
 *   - work is enqueued on the given cudaStream_t (passed as void*), the call
 *     never synchronises and never throws; the return value is a status code
 *     (0 = ok), fmms_strerror() names it;
 *   - `status_dev` (nullable) is an int in device memory that a kernel sets
 *     to FMMS_ERR_TIMEOUT if one of its bounded waits ran out; the host reads
 *     it whenever it likes.
 *
 * Each declaration cites the reference interface it replaces (paths relative
 * to the reference project, src/fused_mm_sampling/...).
 */
#ifndef FMMS_B200_H_
#define FMMS_B200_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* status codes */
#define FMMS_OK 0
#define FMMS_ERR_TIMEOUT 1       /* a bounded device-side wait ran out          */
#define FMMS_ERR_BAD_ARG 2       /* null pointer, non-positive size, bad flags  */
#define FMMS_ERR_UNSUPPORTED 3   /* shape/alignment the kernels do not handle   */
#define FMMS_ERR_WORKSPACE 4     /* workspace missing or too small              */
#define FMMS_ERR_CUDA 5          /* a CUDA runtime/driver call failed           */
#define FMMS_ERR_ARCH 6          /* device is not compute capability 10.x       */
#define FMMS_ERR_TOO_LARGE 7     /* B * S exceeds the built-in scratch          */
#define FMMS_ERR_TOPK_OVERFLOW 8 /* status word only: a row's top-k candidates overflowed and no scratch
                                    for the exact second pass was given (see fmms_query_topk_workspace) */

/* flags of fmms_sample / fmms_sample_tp */
#define FMMS_FLAG_GREEDY 1         /* argmax of raw logits (core.py GREEDY_SAMPLING, :569-600) */
#define FMMS_FLAG_EXT_NOISE 2      /* add caller-supplied fp32 noise instead of Philox noise   */
#define FMMS_FLAG_RETURN_LOGITS 4  /* also store fp32 logits (core.py RETURN_LOGITS, :568-573) */
#define FMMS_FLAG_FORCE_GEMV 8     /* use the small-batch weight-streaming kernel              */
#define FMMS_FLAG_FORCE_MMA 16     /* use the tcgen05 tensor-core kernel                       */
#define FMMS_FLAG_SEED_DEVICE 64   /* `seed` is a DEVICE POINTER to a uint64 seed that the kernel reads:
                                      a launch captured in a CUDA graph then draws fresh noise on every
                                      replay once the caller advances the value between replays       */
#define FMMS_FLAG_TWO_STAGE 32     /* decode the winners in a second kernel (the reference's
                                      stage 2, core.py:359-370) instead of the last CTA        */
#define FMMS_FLAG_LOGPROB 128      /* set by fmms_sample_logprobs(): the pass also accumulates each
                                      row's log-sum-exp and reports ln p(sampled id)            */

#define FMMS_FLAG_HOST_IO 256      /* fmms_run() only: H_bf16, temperature and the outputs out_idx / out_val /
                                      out_logprob / out_lse are HOST pointers (pinned memory recommended); the
                                      call copies them through the caller's device `staging` buffer           */
#define FMMS_FLAG_NO_SYNC 512      /* with FMMS_FLAG_HOST_IO: do not wait for the stream before returning   */
#define FMMS_FLAG_W_FP8 2048       /* fmms_run() only: W_bf16 points to e4m3 bytes [V_local, D] with one fp32
                                      scale per row in `w_scale` (weight = byte value * scale); see fmms_call_t */

/* kernel paths reported by fmms_last_path() */
#define FMMS_PATH_NONE 0
#define FMMS_PATH_GEMV 1
#define FMMS_PATH_MMA 2

/* Library/ABI version (major * 1000 + minor). No reference counterpart. */
int fmms_version(void);

/* Text for a status code. No reference counterpart (the reference raises
 * Python exceptions: core.py:235-241). */
const char* fmms_strerror(int status);

/* Number of SMs of the current device (persistent-grid size). Replaces
 * num_sms_cached(), core.py:212-214. */
int fmms_num_sms(int* num_sms);

/* Bytes of scratch the sampling call needs. Replaces the per-call torch.empty of
 * `maxs` / `maxs_idx` [num_samples, cdiv(V,128), H] in core.py:262-270. Here every
 * CTA folds its winners into one packed 64-bit key per (row, draw) with atomicMax.
 * THE WORKSPACE MUST BE ZERO BEFORE ITS FIRST USE (one cudaMemset when it is
 * created); every call leaves it ready for the next one. After a call that reported
 * FMMS_ERR_TIMEOUT, zero it again. */
int fmms_query_workspace(int V_local, int D, int B, int S, size_t* bytes);

/*
 * The fused sampling step on one GPU (or on one vocabulary shard).
 * Replaces fused_mm_sample_triton(), core.py:224-348 (stage-1 kernel
 * core.py:480-635 plus stage-2 _local_reduce core.py:359-370).
 *
 *   W_bf16        [V_local, D] bf16 row-major, 16-byte aligned, D % 8 == 0
 *   H_bf16        [B, D] bf16 row-major, 16-byte aligned; more than 256 rows run as
 *                 consecutive launches over blocks of 256 rows
 *   temperature   fp32; temp_stride 0 = one value for all rows (the
 *                 reference's 0-d tensor, core.py:228,513), 1 = one per row
 *   S             draws per row (num_samples)
 *   seed          draw s uses the random stream `seed + s` (core.py:644)
 *   v_global_offset  global vocabulary id of W's row 0 (tp_rank * vocab_size
 *                 at core.py:603); also keys the noise so that a sharded run
 *                 reproduces the unsharded one
 *   ext_noise     [S, B, noise_ld] fp32, used when FMMS_FLAG_EXT_NOISE;
 *                 element (s, b, v) is added to logit (b, v) / T_b
 *   logits_out    [B, V_local] fp32, written when FMMS_FLAG_RETURN_LOGITS
 *   out_idx       [B, S] int64 global token ids
 *   out_val       [B, S] fp32 winning perturbed logits (nullable)
 *   workspace     >= fmms_query_workspace() bytes, 256-byte aligned, zeroed once
 *                 when created (see fmms_query_workspace)
 */
int fmms_sample(const void* W_bf16, const void* H_bf16, const float* temperature, int temp_stride,
                int V_local, int D, int B, int S, unsigned long long seed,
                long long v_global_offset, int flags, const float* ext_noise, long long noise_ld,
                float* logits_out, long long* out_idx, float* out_val, void* workspace,
                size_t workspace_bytes, int* status_dev, void* stream);

/* Which kernel the last fmms_sample / fmms_sample_tp call of this thread
 * dispatched to (FMMS_PATH_*). No reference counterpart (the reference has one
 * kernel and autotunes its tile shape, core.py:442-476). */
int fmms_last_path(void);

/* Measurement helper: read `bytes` of `buffer` once with streaming loads, which evicts the
 * L2 cache without leaving dirty lines behind (a memset-based flush makes the next kernel pay
 * for the write-back).  Counterpart of the 256 MB `cache.zero_()` flush of the reference's
 * bench harness (bench/triton_benchmark_lib.py:237-249). */
int fmms_l2_sweep(const void* buffer, size_t bytes, void* stream);

/* Profiling aid: while `stamps_dev` (device memory, 8 x 8 bytes per persistent CTA, at least
 * 320 CTAs) is set, every sampling kernel records %globaltimer at its phases for each CTA:
 * [0] entry, [1] prologue done, [2] first operands landed, [3] last MMA issued, [4] last
 * accumulator complete, [5] epilogue done, [6] CTA done, [7] winners decoded (last CTA only).
 * Pass NULL to switch it off (the default).  Counterpart of the reference's Proton
 * intra-kernel scopes (benchmarking/insert_proton_records.py). */
int fmms_debug_stamps(unsigned long long* stamps_dev);

/* Host-only: the launch plan fmms_sample would use on a device with `num_sms`
 * SMs and `max_smem_bytes` of opt-in shared memory per block; needs no GPU.
 * plan[0] = FMMS_PATH_*, [1] = persistent CTAs, [2] = vocabulary rows of the tallest tile
 * (row group), [3] = tiles (row groups) of the busiest CTA, [4] = pipeline stages, [5] = M tiles,
 * [6] = dynamic shared memory bytes, [7] = candidate rows handed to the
 * cross-CTA reduction.  Replaces the tile heuristics bsz_h() (core.py:876-881)
 * and the autotune table (core.py:442-470). */
int fmms_plan(int V_local, int D, int B, int S, int flags, int num_sms, int max_smem_bytes, int* plan);

/* ---- tensor parallelism: vocabulary shards on the GPUs of one NVLink domain ------------
 *
 * Each rank samples its own block with fmms_sample() (v_global_offset = first global row of
 * the block, out_val requested) and then calls fmms_tp_exchange(): every rank writes its
 * per-row (value, id, epoch) records into every rank's symmetric buffer with plain peer
 * stores, waits (bounded) until the records of all ranks in its own buffer carry this
 * step's epoch, and keeps the largest value per row (ids below 2^32).  All ranks end with the same ids.  This replaces the symmetric-memory
 * fan-out of per-tile candidates plus host-launched barrier and reduce of the reference:
 * allocate_symm_mem_outputs / tp_post_kernel_reduce (tensor_parallel_reduce.py:21-85) and
 * the in-kernel peer stores (core.py:614-632).
 */

/* fmms_sample() with the exchange folded into the sampling kernel: the CTA that finishes last
 * writes this rank's winners into every rank's buffer, signals, waits (bounded) for the peers
 * and writes the global winners to out_idx / out_val - one launch per step and rank, no host
 * barrier.  Arguments as fmms_sample() plus those of fmms_tp_exchange(); B * S must not exceed
 * `max_items`.  Replaces fused_mm_sample_triton() with tp.size > 1 (core.py:250-260,
 * :614-632, :323-340). */
int fmms_sample_tp(const void* W_bf16, const void* H_bf16, const float* temperature, int temp_stride,
                   int V_local, int D, int B, int S, unsigned long long seed,
                   long long v_global_offset, int flags, const float* ext_noise, long long noise_ld,
                   float* logits_out, long long* out_idx, float* out_val, void* workspace,
                   size_t workspace_bytes, int* status_dev, void* stream, int rank, int world,
                   int max_items, void* const* peer_buffers, unsigned int epoch,
                   unsigned long long wait_limit_ns);

/* fmms_sample() that also reports, from the same pass over W, the log-probability of every
 * sampled id under softmax(logits / T) and each row's log-normaliser:
 *   out_logprob [B, S] fp32 (required)  ln p(out_idx[b, s]) = logit / T - out_lse[b]
 *   out_lse     [B]    fp32 (nullable)  ln sum_v exp(logit_v / T) over this call's V_local rows
 * Rows decoded greedily (FMMS_FLAG_GREEDY, or temperature <= 0) use T = 1.  The kernels keep a
 * running (max, sum) per row next to the running argmax; every CTA leaves one partial sum per
 * row in the workspace and the CTA that finishes last merges them in a fixed order (bit for bit
 * reproducible with the tensor-core kernels; to fp32 rounding with the weight-streaming kernel,
 * whose CTAs share part of the work dynamically); the winner's logit is its perturbed value minus its own noise, which is a
 * pure function of (seed, draw, row, id).  The sampled ids are those of fmms_sample().  Not combined
 * with FMMS_FLAG_TWO_STAGE (FMMS_ERR_UNSUPPORTED).  This entry point has no tensor-parallel
 * arguments: under tensor parallelism use fmms_run() with FMMS_FLAG_LOGPROB and tp_world > 1 (the
 * winner's logit and every rank's log-sum-exp travel in the same fused exchange as the winners), or
 * call this on the local shard and combine out_lse across ranks on the host.
 * The reference has no counterpart: it lists log-probabilities as unavailable without the full
 * logits (findings/vllm-integration.md:99); the accumulation is the online log-sum-exp that its
 * paper's appendix on optional outputs describes. */
int fmms_sample_logprobs(const void* W_bf16, const void* H_bf16, const float* temperature, int temp_stride,
                         int V_local, int D, int B, int S, unsigned long long seed,
                         long long v_global_offset, int flags, const float* ext_noise, long long noise_ld,
                         float* logits_out, long long* out_idx, float* out_val, void* workspace,
                         size_t workspace_bytes, int* status_dev, void* stream, float* out_logprob,
                         float* out_lse);

/*
 * One call descriptor for every variant of the sampling step: fmms_run(&call) is fmms_sample(),
 * fmms_sample_tp() (tp_world > 1) or fmms_sample_logprobs() (FMMS_FLAG_LOGPROB) with the
 * arguments taken from the structure, which a host keeps and updates in place between steps
 * (only H_bf16, temperature, seed and the output pointers change from step to step).  Set
 * `struct_bytes = sizeof(fmms_call_t)`; fields a call does not use are zero.
 *
 * With FMMS_FLAG_HOST_IO the hidden states, the temperatures and the results live in HOST
 * memory: the call enqueues the host-to-device copies into `staging` (device memory of at
 * least fmms_query_staging() bytes, 256-byte aligned), the sampling kernel, and the
 * device-to-host copies of the ids (and of out_val / out_logprob / out_lse when given, and of
 * the status word into `status_host` when given), then waits for the stream unless
 * FMMS_FLAG_NO_SYNC is set.  W_bf16, ext_noise, logits_out, workspace and status_dev stay device
 * pointers.  This is the whole decode-side hand-over of an engine whose hidden states arrive in
 * host memory, in one library call.  The reference has no counterpart (its entry point takes
 * CUDA tensors, core.py:224-235).
 */
typedef struct fmms_call {
  size_t struct_bytes;
  const void* W_bf16;
  const void* H_bf16;
  const float* temperature;
  int temp_stride;
  int V_local, D, B, S;
  unsigned long long seed;
  long long v_global_offset;
  int flags;
  const float* ext_noise;
  long long noise_ld;
  float* logits_out;
  long long* out_idx;
  float* out_val;
  float* out_logprob; /* FMMS_FLAG_LOGPROB */
  float* out_lse;     /* FMMS_FLAG_LOGPROB, nullable */
  void* workspace;
  size_t workspace_bytes;
  int* status_dev;
  void* stream;
  /* tensor parallelism: tp_world > 1 selects the fused exchange of fmms_sample_tp() */
  int tp_rank, tp_world, tp_max_items;
  void* const* tp_peer_buffers;
  unsigned int tp_epoch;
  unsigned long long tp_wait_limit_ns;
  /* FMMS_FLAG_HOST_IO */
  void* staging;
  size_t staging_bytes;
  int* status_host;
  /* top-k / top-p sampling: top_k in 1..64 switches it on (see fmms_query_topk_workspace) */
  int top_k;
  float top_p;              /* nucleus mass in (0, 1); any other value: top-k only */
  void* topk_workspace;     /* device memory, 256-byte aligned, ZERO before its first use */
  size_t topk_workspace_bytes;
  /* FMMS_FLAG_W_FP8: e4m3 weights.  `W_bf16` then holds V_local x D bytes (D % 16 == 0), `w_scale` one fp32
   * scale per vocabulary row (16-byte aligned); the call quantises the bf16 hidden states per row to e4m3
   * (scale = max|h| / 448) into `staging` (device memory of fmms_query_staging() bytes; no other use of it in
   * this mode), multiplies with tcgen05.mma kind::f8f6f4 and applies both scales to the fp32 sums before the
   * temperature.  Half the bytes of the bf16 stream.  Works with tensor parallelism, log-probabilities and
   * top-k; not with FMMS_FLAG_HOST_IO, FMMS_FLAG_TWO_STAGE or the small-batch kernel.  The reference has no
   * counterpart (it names quantised LM heads as future work, findings/cutlass-fmms-kernel-plan.md:1076-1077). */
  const float* w_scale;
} fmms_call_t;

int fmms_run(const fmms_call_t* call);

/*
 * Top-k / top-p sampling (fmms_run() with call.top_k in 1..64).  Replaces the reference's
 * fused_mm_topk_and_sample(): per-tile top-k lists written by fused_mm_topk_kernel
 * (tl_fused_mm_topk.py:146-238) and merged, filtered and sampled by _topk_merge_and_sample
 * (tl_fused_mm_topk.py:76-107).  Same distribution: softmax of logits / T over the k largest
 * logits of a row, optionally cut to the smallest prefix (in descending order) whose mass before
 * each kept entry is below top_p (the most probable entry always stays), renormalised.
 *
 * Here the tensor-core pass keeps, per row, only the logits at or above a running lower bound of
 * the row's k-th largest logit (about 1e3 of 1.5e5 entries; every epilogue thread has a segment of
 * 16 entries per row); one small kernel per call then gathers each row's candidates, selects the
 * k largest, applies softmax and the nucleus cut and draws the samples as a
 * Gumbel-max over the surviving ids, with the noise stream of fmms_sample() (so a draw equals the
 * unrestricted draw for the same seed whenever that one survives the cut).  A row that overflows
 * (more than 4096 candidates, or more than 16 in one thread's share of ~300 vocabulary entries;
 * logits that rise steadily over the vocabulary do that) is redone exactly by a
 * second pass that materialises its logits - launched with every call, it returns at once when
 * no row needs it.  out_logprob / out_lse, when given, refer to the truncated distribution.
 *
 * The scratch: `bytes` includes room for those logits (B x V_local x 4); with only
 * `bytes_without_exact_pass` an overflowing row gets ids of -1 and FMMS_ERR_TOPK_OVERFLOW in the
 * status word instead.  Zero the memory once; every call leaves it ready for the next.
 * Not combined with tensor parallelism, FMMS_FLAG_RETURN_LOGITS, FMMS_FLAG_TWO_STAGE or
 * FMMS_FLAG_HOST_IO (FMMS_ERR_UNSUPPORTED).
 */
int fmms_query_topk_workspace(int V_local, int B, size_t* bytes, size_t* bytes_without_exact_pass);

/* Bytes of device staging that fmms_run() needs with FMMS_FLAG_HOST_IO for B rows of D hidden
 * values and S draws. No reference counterpart. */
int fmms_query_staging(int D, int B, int S, size_t* bytes);

/* Size of one rank's symmetric buffer for `world` ranks and up to `max_items` (B * S)
 * items per step. */
int fmms_tp_buffer_bytes(int world, int max_items, size_t* bytes);

/* Set-up, not on the sampling path: allocate (and zero) this rank's buffer and produce the
 * 64-byte CUDA IPC handle that the other ranks open.  Replaces
 * symm_mem.get_symm_mem_workspace (tensor_parallel_reduce.py:45-48). */
int fmms_tp_alloc(size_t bytes, void** dev_ptr, void* ipc_handle_64);
int fmms_tp_open(const void* ipc_handle_64, void** peer_ptr);
int fmms_tp_close(void* peer_ptr);
int fmms_tp_free(void* dev_ptr);

/* The exchange step (one small kernel).  `peer_buffers[world]` are the device pointers of
 * every rank's buffer as seen from this process (own buffer at index `rank`); `epoch` is
 * either 0 - the step number is then kept in the rank's own buffer and advanced by the kernel,
 * so a launch captured in a CUDA graph can be replayed - or the caller's own counter, the
 * same on all ranks and growing by one per step from 1 (do not mix the two on one buffer); `wait_limit_ns` bounds
 * the wait for the peers' records (0 = 2 s), after which FMMS_ERR_TIMEOUT is written to `status_dev` and the
 * ids are set to -1.  Replaces symm_mem_hdl.barrier() + _local_reduce over world * tiles
 * (tensor_parallel_reduce.py:77-84). */
int fmms_tp_exchange(const long long* local_idx, const float* local_val, int n_items, int max_items,
                     int rank, int world, void* const* peer_buffers, unsigned int epoch,
                     unsigned long long wait_limit_ns, long long* out_idx, float* out_val,
                     int* status_dev, void* stream);

/*
 * fmms_sample() for callers that cannot hand over a workspace because they cannot
 * allocate device memory at all: a plugin inside a serving process that reserved the
 * whole GPU for its own pool at start-up, a plain C host with no allocator of its own,
 * or a decode loop in which cudaMalloc (and the device-wide synchronisation it implies)
 * is forbidden once serving has begun.  It has no counterpart in the reference, which
 * allocates its candidate buffers with torch.empty on every call.
 *
 * Same arguments and results as fmms_sample() minus `workspace`: the candidate scratch
 * is an array built into the library's device image (about 5.4 MiB, resident on every
 * GPU that loads the library until the process exits).  The call itself allocates
 * nothing, on the device or through any library.
 *
 *   - limit: B * S <= fmms_static_max_items() (1024); larger problems return
 *     FMMS_ERR_TOO_LARGE and launch nothing;
 *   - the first call on each device looks the array's device address up (with that
 *     device current) and caches it; make that first call before any stream capture
 *     is begun on the device;
 *   - all calls on a device share the one array: two calls whose kernels overlap on the
 *     GPU (different streams without an ordering between them) race on it.  Calls on
 *     one stream, or ordered by events, are safe.  The array keeps the last call's
 *     running candidates; the part that must start at zero (packed winners, CTA
 *     counter) is zero when the library is loaded and is zeroed again by each call's
 *     last CTA, so the caller never clears anything;
 *   - after a call whose status word reported FMMS_ERR_TIMEOUT the array is normally clean
 *     as well (a CTA whose wait ran out still takes its ticket, and the last one still
 *     clears the head), but a caller that wants certainty - or whose launch was cut short
 *     from outside - calls fmms_static_reset() before the next sample.
 */
int fmms_sample_static(const void* W_bf16, const void* H_bf16, const float* temperature, int temp_stride,
                       int V_local, int D, int B, int S, unsigned long long seed,
                       long long v_global_offset, int flags, const float* ext_noise, long long noise_ld,
                       float* logits_out, long long* out_idx, float* out_val, int* status_dev,
                       void* stream);

/* Largest B * S that fmms_sample_static() accepts. No reference counterpart. */
int fmms_static_max_items(void);

/* Zero the part of the built-in array that fmms_sample_static() expects to be zero (one
 * cudaMemsetAsync on `stream`; allocates nothing).  The counterpart of "zero the workspace
 * again" for callers that own no workspace.  No reference counterpart. */
int fmms_static_reset(void* stream);

#ifdef __cplusplus
}
#endif

#endif /* FMMS_B200_H_ */
