/* C ABI of libmercury_b200.so: B200 (sm_100a) attention ops for the code that
 * Mercury's CommIR PyTorch backend emits for ring, double-ring and GQA
 * schedules.
 *
 * Every entry point takes plain pointers and sizes, enqueues its work on the
 * given CUDA stream of the current device and returns at once with one of the
 * MB_* codes below; none of them aborts, traps or throws.  Device-side waits
 * are bounded: a wait that runs out is reported through the status word read
 * by mb_status_fetch().
 *
 * Tensors are bf16 unless stated, with the head dimension contiguous; the other
 * strides are given in elements.  Citations name files of the reference
 * project (ChandlerGuan/mercury_artifact) whose call this entry point replaces.
 */
#ifndef MERCURY_B200_H_
#define MERCURY_B200_H_

#include <stdint.h>

#if defined(__GNUC__)
#define MB_API __attribute__((visibility("default")))
#else
#define MB_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

#define MB_SUCCESS 0
#define MB_E_INVALID (-1)     /* bad argument (null pointer, negative size, too many segments) */
#define MB_E_UNSUPPORTED (-2) /* shape or option outside what the kernels implement */
#define MB_E_CUDA (-3)        /* a CUDA runtime call failed */
#define MB_E_TENSORMAP (-4)   /* a TMA descriptor could not be encoded (alignment/stride) */
#define MB_E_DEVICE (-5)      /* the status word reported a device-side timeout */
#define MB_E_TOO_LARGE (-6)   /* problem exceeds the fixed scratch of an allocation-free entry point */

#define MB_MAX_SEGMENTS 32 /* K/V (or stream) shards per launch: 8 ranks x ring_divide 4, or a 32-way mesh */
#define MB_MAX_JOBS 40      /* query shards per mb_attn_fwd_multi launch */

/* One sequence shard of K and V: [batch, sk, hkv, head_dim] views. */
typedef struct mb_kv_segment {
  const void* k;
  const void* v;
  int64_t stride_b, stride_s, stride_h; /* shared by k and v */
  int32_t sk;                           /* keys in this shard */
  int32_t k_off;                        /* global position of key 0 (causal rule only) */
  /* Optional arrival flag (device word on this GPU): the kernel does not touch the shard
   * before *ready_flag >= ready_value.  NULL: the shard is already in place.  Lets one launch
   * overlap compute on early shards with the transfer of later ones (see mb_flag_signal). */
  const int32_t* ready_flag;
  int32_t ready_value;
  int32_t reserved;
} mb_kv_segment;

typedef struct mb_attn_fwd_args {
  const void* q; /* [batch, sq, hq, head_dim] */
  int64_t q_stride_b, q_stride_s, q_stride_h;
  void* o; /* [batch, sq, hq, head_dim] bf16, written */
  int64_t o_stride_b, o_stride_s, o_stride_h;
  float* lse; /* [batch, hq, sq] fp32, written: ln sum exp(scale * q.k); sq contiguous */
  int64_t lse_stride_b, lse_stride_h; /* element strides; 0, 0 selects the contiguous layout */
  int32_t batch, sq, hq, hkv, head_dim;
  int32_t q_off;  /* global position of query row 0 (causal rule only) */
  int32_t causal; /* key visible iff k_off + j <= q_off + i */
  float softmax_scale;
  int32_t nseg;
  mb_kv_segment seg[MB_MAX_SEGMENTS];
  int32_t* status; /* device word for timeouts; NULL selects the library's own word */
} mb_attn_fwd_args;

/* Attention forward of one query shard against nseg K/V shards, in segment
 * order, with the online-softmax state carried on chip across shards.
 * nseg == 1 replaces the per-step block call
 *   _flash_attn_forward(**params)            utils/flash_attn_dsl.py:174
 * (also :120, :229, :285, :392, :457), and nseg == P replaces the whole
 * generated loop body of one rank -- block call plus update_out_and_lse
 * (utils/flash_attn_dsl.py:51-71) -- once the shards are reachable.
 * A row that sees no key gets o = 0 and lse = -inf. */
MB_API int mb_attn_fwd(const mb_attn_fwd_args* args, void* cuda_stream);

/* One query shard of a multi-shard forward launch, with where its results go. */
typedef struct mb_fwd_job {
  const void* q; /* [batch, sq, hq, head_dim] */
  int64_t q_stride_b, q_stride_s, q_stride_h;
  void* o; /* [batch, sq, hq, head_dim] bf16, written; may be a peer GPU's memory mapped here */
  int64_t o_stride_b, o_stride_s, o_stride_h;
  float* lse; /* [batch, hq, sq] fp32, written; may be peer memory */
  int64_t lse_stride_b, lse_stride_h; /* 0, 0 selects the contiguous layout */
  int32_t sq;
  int32_t q_off;     /* global position of query row 0 (causal rule only) */
  uint32_t seg_mask; /* bit s set: this job attends to segment s (0 selects all segments) */
  int32_t reserved;
  /* Optional arrival flag of the query shard (a word on this GPU), as ready_flag of mb_kv_segment. */
  const int32_t* q_ready_flag;
  int32_t q_ready_value;
  /* Optional completion flag: once every CTA of this job has stored its rows, the kernel stores
   * done_value to *done_flag with release semantics at system scope (the word may live on the GPU that
   * owns the rows).  Needs done_counter: a zero-initialised word on this GPU that the kernel uses to
   * count finished CTAs and leaves at zero again. */
  int32_t done_value;
  int32_t* done_flag;
  int32_t* done_counter;
  /* Optional carried state.  A job with state_out != 0 does not write o / lse (they may be NULL) but
   * stores the online-softmax state of its rows: unnormalised output rows in state_o
   * [batch, hq, sq, head_dim] fp32 (16-byte aligned) and (reference maximum in raw score units, running
   * sum) pairs in state_ml [batch, hq, sq, 2] fp32.  A job with state_in != 0 starts from that state
   * instead of the empty one (same q rows, same buffers; in place is fine).  A chain of such jobs, one
   * per K/V shard in arrival order, gives the same bits as one job over all the shards, and lets the
   * CTAs of a launch be ordered shard by shard, so that none holds an SM while it waits for a shard
   * that is still in flight.  If the jobs of a chain are in ONE launch, give them chain: int32 words
   * [batch, hq, ceil(sq / 256)] on this GPU; a job with state_out stores chain_set to its CTA's word
   * after its state (release), a job with state_in waits (bounded, status 109) until the word is
   * >= chain_wait.  The continuing job must come later in job[] (CTAs are dispatched in job order), and the
   * values must grow from launch to launch (or the words be cleared in between): a word left at an old value
   * that already satisfies the wait lets a link start before the link before it has stored its state.
   * With chain == NULL the jobs must be in different launches of one stream. */
  float* state_o;
  float* state_ml;
  int32_t state_in, state_out;
  int32_t* chain;
  int32_t chain_wait, chain_set;
} mb_fwd_job;

typedef struct mb_attn_fwd_multi_args {
  int32_t batch, hq, hkv, head_dim;
  int32_t causal;
  float softmax_scale;
  int32_t njobs;
  int32_t nseg;
  mb_fwd_job job[MB_MAX_JOBS];
  mb_kv_segment seg[MB_MAX_SEGMENTS];
  int32_t* status;
} mb_attn_fwd_multi_args;

/* mb_attn_fwd for up to MB_MAX_JOBS query shards in ONE launch (CTAs of the jobs are scheduled together,
 * first job first).  The balanced causal ring uses it: a rank computes two query half-shards that belong
 * to other ranks against the K/V shards they can see, writes o / lse straight into the owners' memory and
 * raises each owner's completion flag from the kernel.  It replaces the same reference calls as
 * mb_attn_fwd; the re-assignment of query rows has no counterpart in the reference (whose generated
 * loop is only correct for causal = False, utils/flash_attn_dsl.py:167). */
MB_API int mb_attn_fwd_multi(const mb_attn_fwd_multi_args* args, void* cuda_stream);

/* ---- backward ------------------------------------------------------------------------- */

typedef struct mb_bwd_preprocess_args {
  const void* dout; /* [batch, sq, hq, head_dim] bf16 */
  int64_t dout_stride_b, dout_stride_s, dout_stride_h;
  const void* out; /* forward output, same shape */
  int64_t out_stride_b, out_stride_s, out_stride_h;
  const float* lse; /* [batch, hq, sq] fp32: the FINAL log-sum-exp of these query rows */
  float* lse2;      /* [batch, hq, stat_pad] fp32, written: -lse * log2(e); -inf for rows without keys and padding */
  float* delta;     /* [batch, hq, stat_pad] fp32, written: rowsum(dout * out), 0 in the padding */
  int32_t batch, sq, hq, head_dim;
  int32_t stat_pad; /* sq rounded up to a multiple of 64 */
} mb_bwd_preprocess_args;

/* Per-row statistics the backward kernels need; run once per query shard (in a ring, once
 * per rank: every block call of the generated loop receives the same out and softmax_lse,
 * utils/attn_bwd_dsl.py:91-92). */
MB_API int mb_attn_bwd_preprocess(const mb_bwd_preprocess_args* args, void* cuda_stream);

#define MB_BWD_MODE_DKV 1 /* owner = one K/V shard, stream = query shards: writes dK (out1) and dV (out2) */
#define MB_BWD_MODE_DQ 0  /* owner = one query shard, stream = K/V shards: writes dQ (out1) */
#define MB_BWD_MODE_FUSED 2 /* like DKV, and each streamed query shard's dQ contributions are ADDED (fp32,
                             * red.global.add) into its segment's dq_accum: scores are computed once, 5 tile
                             * products per block instead of 7.  dQ then depends on the order of fp32
                             * additions (not bitwise reproducible); finish with mb_attn_bwd_dq_convert. */
#define MB_OUT_BF16 0
#define MB_OUT_F32 1
#define MB_OUT_F32_ACCUM 2 /* out += result (each element is owned by one CTA: no atomics) */

/* One streamed shard.  Mode DKV: str = q, str_g = dout (hq heads) with that shard's lse2/delta;
 * mode DQ: str = k, str_g = v (hkv heads), lse2/delta unused. */
typedef struct mb_bwd_segment {
  const void* str;
  const void* str_g;
  int64_t stride_b, stride_s, stride_h;
  int32_t rows;
  int32_t pos_off; /* global position of row 0 (causal rule) */
  const float* lse2;
  const float* delta;
  int32_t stat_pad;
  int32_t ready_value;
  const int32_t* ready_flag; /* optional arrival flag, as in mb_kv_segment */
  /* MB_BWD_MODE_FUSED only: fp32 [batch, hq, stat_pad, head_dim], zero-filled by the caller (or holding a
   * partial sum to add to): receives this query shard's UNSCALED dQ contributions. */
  float* dq_accum;
} mb_bwd_segment;

typedef struct mb_attn_bwd_args {
  int32_t mode; /* MB_BWD_MODE_* */
  int32_t out_mode; /* MB_OUT_* */
  const void* own;   /* DKV: k; DQ: q      [batch, own_rows, heads, head_dim] */
  const void* own_g; /* DKV: v; DQ: dout   same strides */
  int64_t own_stride_b, own_stride_s, own_stride_h;
  const float* own_lse2; /* DQ mode only: statistics of the owner's query rows */
  const float* own_delta;
  int32_t own_stat_pad;
  int32_t own_rows;
  int32_t own_off; /* global position of owner row 0 */
  int32_t batch, hq, hkv, head_dim;
  int32_t causal; /* key visible iff k_pos <= q_pos */
  float softmax_scale;
  void* out1; /* DKV: dk; DQ: dq   [batch, own_rows, heads, head_dim] */
  void* out2; /* DKV: dv */
  int64_t out_stride_b, out_stride_s, out_stride_h;
  int32_t nseg;
  int32_t reserved;
  mb_bwd_segment seg[MB_MAX_SEGMENTS];
  int32_t* status;
} mb_attn_bwd_args;

/* Gradients of one owner shard against nseg streamed shards.  One DQ call plus one DKV call
 * with a single segment replace the block call
 *   _flash_attn_backward(**params)           utils/attn_bwd_dsl.py:115
 * and, with one segment per rank, the whole generated backward loop including its fp32
 * accumulation and the rotating dK/dV buffer (mercury/backend/pytorch/codegen.py:99-190). */
MB_API int mb_attn_bwd(const mb_attn_bwd_args* args, void* cuda_stream);

/* dq[b, s, h, :] = softmax_scale * dq_accum[b, h, s, :]: the last step of MB_BWD_MODE_FUSED.
 * dq is bf16 (MB_OUT_BF16) or fp32 (MB_OUT_F32) with the given element strides; dq_accum has row pitch
 * stat_pad per (batch, head). */
MB_API int mb_attn_bwd_dq_convert(const float* dq_accum, void* dq, int64_t dq_stride_b, int64_t dq_stride_s,
                                  int64_t dq_stride_h, int32_t batch, int32_t sq, int32_t hq, int32_t stat_pad,
                                  int32_t out_mode, float softmax_scale, void* cuda_stream);

typedef struct mb_attn_bwd_block_args {
  const void* dout; /* [batch, sq, hq, head_dim] bf16; dout and out use q's strides */
  const void* q;
  const void* out;
  int64_t q_stride_b, q_stride_s, q_stride_h;
  const void* k; /* [batch, sk, hkv, head_dim] bf16 */
  const void* v;
  int64_t kv_stride_b, kv_stride_s, kv_stride_h;
  const float* lse; /* [batch, hq, sq] fp32, final log-sum-exp of the query rows */
  void* dq;         /* like q, written */
  int64_t dq_stride_b, dq_stride_s, dq_stride_h;
  void* dk; /* like k, written; dk and dv share strides */
  void* dv;
  int64_t dkv_stride_b, dkv_stride_s, dkv_stride_h;
  int32_t batch, sq, sk, hq, hkv, head_dim;
  int32_t q_off, k_off; /* global positions of query row 0 / key 0 (causal rule) */
  int32_t causal;
  int32_t out_mode; /* MB_OUT_BF16 or MB_OUT_F32 */
  float softmax_scale;
  int32_t* status;
} mb_attn_bwd_block_args;

/* Block backward (dq, dk, dv of one query shard against one K/V shard) that performs no
 * allocation of any kind.  It has no counterpart in the reference.
 *
 * Who needs it: callers that are not allowed to obtain device memory at the point where they
 * run the backward -- code executing under a memory pool that is already fully planned, inside
 * a framework's allocator callback, or in a serving process whose memory budget is fixed at
 * start-up -- and that therefore cannot provide the per-row statistics workspace
 * (2 x batch x hq x pad64(sq) floats) that mb_attn_bwd_preprocess / mb_attn_bwd expect from
 * the caller.  Here that workspace is a fixed 8 MiB array inside the library, resident on every
 * GPU that loads it until the process exits.
 *
 * Limit: batch * hq * pad64(sq) <= 1 048 576 rows (for example batch 1, 32 heads, 32 768 query
 * rows); anything larger is refused with MB_E_TOO_LARGE and nothing is launched.
 * The first call on a device looks up the array's device address and sets kernel attributes;
 * make that first call before any stream capture begins.  Every call uses the same array and
 * overwrites all of the part it needs (nothing has to be cleared beforehand), so two calls whose
 * kernels overlap on the GPU -- different streams, or different host threads -- race on it;
 * calls queued on one stream are safe.  Inputs and outputs are the caller's, as elsewhere. */
MB_API int mb_attn_bwd_block_noalloc(const mb_attn_bwd_block_args* args, void* cuda_stream);

#define MB_DTYPE_BF16 0
#define MB_DTYPE_F32 1

typedef struct mb_merge_args {
  float* out;            /* [batch, seq, heads, head_dim] fp32 contiguous, updated in place */
  float* lse;            /* [batch, seq, heads, 1] fp32 contiguous, updated in place */
  const void* block_out; /* [batch, seq, heads, head_dim], bf16 or fp32 */
  int64_t block_stride_b, block_stride_s, block_stride_h;
  const float* block_lse; /* [batch, heads, seq] fp32 contiguous */
  int32_t batch, seq, heads, head_dim;
  int32_t first;       /* non-zero: adopt the block (the reference's out-is-None call) */
  int32_t block_dtype; /* MB_DTYPE_* of block_out */
} mb_merge_args;

/* One step of the running out/LSE merge:
 *   out <- out - sigmoid(block_lse - lse) * (out - block_out)
 *   lse <- lse - logsigmoid(lse - block_lse)
 * Replaces update_out_and_lse / _update_out_and_lse, utils/flash_attn_dsl.py:31-71.
 * Rows whose block_lse is -inf are left unchanged; rows whose lse is -inf adopt the block. */
MB_API int mb_merge_out_lse(const mb_merge_args* args, void* cuda_stream);

/* Merge of two packed fp32 buffers of `rows` rows, each row = head_dim_plus_1 floats
 * [out | lse]; out may alias lhs.  Replaces flash_reduce, utils/flash_attn_dsl.py:293-305 (the
 * reduce op of the ring-over-Q schedule, mercury/backend/pytorch/codegen.py:116-190). */
MB_API int mb_flash_reduce(const float* lhs, const float* rhs, float* out, int64_t rows, int32_t head_dim_plus_1,
                           void* cuda_stream);

/* One-shot merge of n (<= 16) packed fp32 buffers [rows, head_dim_plus_1] into out:
 * lse* = log sum_r exp(lse_r), out* = sum_r exp(lse_r - lse*) out_r.  srcs is a HOST array of n
 * device pointers; they may be peer mappings (the kernel then reads over NVLink).  out must not
 * alias a source another rank is still reading.  Replaces update_out_and_lse_collective,
 * utils/flash_attn_dsl.py:307-324 (the tree / all-reduce merge emitted at
 * mercury/backend/pytorch/codegen.py:427-440). */
MB_API int mb_tree_merge(const float* const* srcs, int32_t n, float* out, int64_t rows, int32_t head_dim_plus_1,
                         void* cuda_stream);

/* ---- peer memory over NVLink (one process per GPU) ------------------------------------
 * Together these replace SendRecv.send_recv / commit / wait of
 * mercury/backend/pytorch/utils.py:9-39 (NCCL batch_isend_irecv): a send is a copy into the
 * peer's inbox followed by mb_flag_signal on the peer's flag; a wait is mb_flag_wait on the
 * local flag. */

/* cudaMalloc-backed allocation that mb_ipc_export can share with the other ranks. */
MB_API int mb_mem_alloc(void** ptr, uint64_t bytes);
MB_API int mb_mem_free(void* ptr);
MB_API int mb_mem_zero(void* ptr, uint64_t bytes, void* cuda_stream);
/* 64-byte handle of an mb_mem_alloc allocation / mapping of a peer's handle into this process. */
MB_API int mb_ipc_export(void* ptr, unsigned char* handle64);
MB_API int mb_ipc_import(const unsigned char* handle64, void** ptr);
MB_API int mb_ipc_release(void* ptr);
/* Stream-ordered copy; either side may be a peer mapping (copy engines over NVLink). */
MB_API int mb_copy_async(void* dst, const void* src, uint64_t bytes, void* cuda_stream);
/* The same for `height` rows of `width` bytes with row pitches dpitch / spitch (one head group of a
 * [batch, seq, heads, head_dim] tensor is such a rectangle); all four 16-byte aligned. */
MB_API int mb_copy2d_async(void* dst, uint64_t dpitch, const void* src, uint64_t spitch, uint64_t width,
                           uint64_t height, void* cuda_stream);
/* Stream-ordered release-store of `value` to a flag word (local or peer mapping). */
MB_API int mb_flag_signal(int32_t* flag, int32_t value, void* cuda_stream);
/* Stream-ordered wait until *flag >= value.  After timeout_ns the wait gives up, writes a
 * timeout code to `status` (NULL: the library's word) and lets the stream continue. */
MB_API int mb_flag_wait(const int32_t* flag, int32_t value, uint64_t timeout_ns, int32_t* status,
                        void* cuda_stream);

/* The same for up to 32 flags with ONE kernel launch: flags / values are HOST arrays of n entries. */
MB_API int mb_flags_signal(int32_t* const* flags, const int32_t* values, int32_t n, void* cuda_stream);
MB_API int mb_flags_wait(const int32_t* const* flags, const int32_t* values, int32_t n, uint64_t timeout_ns,
                         int32_t* status, void* cuda_stream);

/* One contiguous byte range of a pull: src may be a peer mapping; both addresses and the size are
 * multiples of 16. */
typedef struct mb_pull_range {
  const void* src;
  void* dst;
  uint64_t bytes;
} mb_pull_range;

#define MB_MAX_PULL_RANGES 8
#define MB_MAX_PULL_FLAGS 4

typedef struct mb_pull_args {
  int32_t nranges;
  int32_t nflags;
  mb_pull_range range[MB_MAX_PULL_RANGES];
  const int32_t* wait_flag; /* optional: do not read before *wait_flag >= wait_value (the source's "published" word) */
  int32_t wait_value;
  int32_t ctas; /* CTAs to use; 0 selects one per SM */
  int32_t* flag[MB_MAX_PULL_FLAGS]; /* raised (release, system scope) once every byte has landed; may be peer memory */
  int32_t value[MB_MAX_PULL_FLAGS];
  int32_t* counter; /* zero-initialised word on this GPU; counts finished CTAs and is left at zero again */
  int32_t* status;  /* NULL selects the library's word */
} mb_pull_args;

/* SM-driven pull over NVLink: a grid of one-warp CTAs copies the ranges in 8 KiB chunks with bulk
 * copies peer -> shared memory -> local memory (three chunks in flight per CTA), waits first (bounded)
 * for the source's flag, and the last CTA to finish raises the completion flags -- wait, transfer and
 * signal in ONE launch.  The CTAs are small enough (25 KiB of shared memory, 32 threads) to run beside a
 * resident attention CTA on every SM.  The alternative to mb_flag_wait + mb_copy_async + mb_flags_signal
 * (copy engines); both replace the transfer inside SendRecv, mercury/backend/pytorch/utils.py:22-39. */
MB_API int mb_pull_sm(const mb_pull_args* args, void* cuda_stream);

/* How long a kernel waits for a shard that another GPU has to deliver (the ready_flag of a segment or of
 * a job's queries) before it gives up with status 109.  Process-wide, applies to launches made afterwards.
 * Default 30 000 ms: ranks of a job may be seconds apart (first-call module load, data loading, a
 * checkpoint on one rank), and the reference's NCCL path would simply wait.  Waits inside one CTA keep
 * their fixed budget of about a second. */
MB_API int mb_set_peer_wait_ms(uint32_t milliseconds);

/* Enqueue a copy of the status word of the current device into *pinned_host_dst (page-locked host
 * memory) on `cuda_stream`, without synchronising and without clearing the word.  Lets a caller notice a
 * timed-out wait of an earlier call at its next call instead of paying a synchronisation per call. */
MB_API int mb_status_peek_async(int32_t* pinned_host_dst, void* cuda_stream);

/* Synchronise `cuda_stream`, copy the library's status word of the current
 * device into *out (0 = no device-side timeout so far) and clear it. */
MB_API int mb_status_fetch(int32_t* out, void* cuda_stream);

/* Text of the CUDA runtime error behind the calling thread's latest MB_E_CUDA, e.g.
 * "launch attn_bwd_fused_kernel: cudaErrorLaunchOutOfResources (too many resources requested for launch)".
 * Empty when there was none. */
MB_API int mb_last_cuda_error(char* buf, int32_t len);

/* Library version, major * 1000 + minor. */
MB_API int mb_version(void);

#ifdef __cplusplus
}
#endif
#endif /* MERCURY_B200_H_ */
