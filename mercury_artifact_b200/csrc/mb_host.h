// Host-side declarations shared by the translation units of libmercury_b200.so.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <string.h>

#include "mercury_b200.h"

namespace mb {

// Encode a tiled bf16 TMA descriptor with 128-byte swizzle.  Returns 0 on success.
int encode_tiled_bf16(CUtensorMap* map, void* base, int rank, const cuuint64_t* dims, const cuuint64_t* strides_bytes,
                      const cuuint32_t* box, const cuuint32_t* elem_strides);

// Remember a failed CUDA runtime call for mb_last_cuda_error(); returns true when `e` is cudaSuccess.
bool cuda_ok(cudaError_t e, const char* what);

// Device address of the library's status word on the current device (nullptr on failure).
int* default_status_word();

int launch_attn_fwd(const mb_attn_fwd_args* args, cudaStream_t stream);
int launch_attn_fwd_multi(const mb_attn_fwd_multi_args* args, cudaStream_t stream);

// Budget of in-kernel waits for data that other GPUs deliver (mb_set_peer_wait_ms), in SM cycles.
void set_peer_wait_ms(unsigned ms);
long long peer_wait_cycles();
int launch_merge(const mb_merge_args* args, cudaStream_t stream);
int launch_tree_merge(const float* const* srcs, int n, float* out, long long rows, int width, cudaStream_t stream);
int launch_flash_reduce(const float* lhs, const float* rhs, float* out, long long rows, int width, cudaStream_t stream);
int launch_bwd_preprocess(const mb_bwd_preprocess_args* args, cudaStream_t stream);
int launch_attn_bwd(const mb_attn_bwd_args* args, cudaStream_t stream);
int launch_dq_convert(const float* acc, void* dq, long long sb, long long ss, long long sh, int batch, int sq, int hq,
                      int pad, int out_mode, float scale, cudaStream_t stream);
int launch_bwd_block_noalloc(const mb_attn_bwd_block_args* args, cudaStream_t stream);

}  // namespace mb
