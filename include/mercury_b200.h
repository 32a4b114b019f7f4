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

#define MB_MAX_SEGMENTS 8

/* One sequence shard of K and V: [batch, sk, hkv, head_dim] views. */
typedef struct mb_kv_segment {
  const void* k;
  const void* v;
  int64_t stride_b, stride_s, stride_h; /* shared by k and v */
  int32_t sk;                           /* keys in this shard */
  int32_t k_off;                        /* global position of key 0 (causal rule only) */
} mb_kv_segment;

typedef struct mb_attn_fwd_args {
  const void* q; /* [batch, sq, hq, head_dim] */
  int64_t q_stride_b, q_stride_s, q_stride_h;
  void* o; /* [batch, sq, hq, head_dim] bf16, written */
  int64_t o_stride_b, o_stride_s, o_stride_h;
  float* lse; /* [batch, hq, sq] fp32 contiguous, written: ln sum exp(scale * q.k) */
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

/* Synchronise `cuda_stream`, copy the library's status word of the current
 * device into *out (0 = no device-side timeout so far) and clear it. */
MB_API int mb_status_fetch(int32_t* out, void* cuda_stream);

/* Library version, major * 1000 + minor. */
MB_API int mb_version(void);

#ifdef __cplusplus
}
#endif
#endif /* MERCURY_B200_H_ */
