// extern "C" surface of libmercury_b200.so and the few host utilities the
// kernels share (TMA descriptor encoding, the per-device status word).
#include <cudaTypedefs.h>
#include <stdio.h>

#include "mb_host.h"

namespace mb {

__device__ int g_status_word = 0;

static thread_local char g_last_cuda_error[256] = "";

bool cuda_ok(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return true;
  snprintf(g_last_cuda_error, sizeof(g_last_cuda_error), "%s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
  cudaGetLastError();  // clear the non-sticky error so that it is not reported again by a later call
  return false;
}

int* default_status_word() {
  static int* cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (cached[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) return nullptr;
    cached[dev] = static_cast<int*>(p);
  }
  return cached[dev];
}

int encode_tiled_bf16(CUtensorMap* map, void* base, int rank, const cuuint64_t* dims, const cuuint64_t* strides_bytes,
                      const cuuint32_t* box, const cuuint32_t* elem_strides) {
  static PFN_cuTensorMapEncodeTiled_v12000 encode = nullptr;
  if (encode == nullptr) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess || fn == nullptr)
      return -1;
    encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
  }
  CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, static_cast<cuuint32_t>(rank), base, dims, strides_bytes,
                      box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -1;
}

}  // namespace mb

extern "C" {

int mb_version(void) { return 1001; }

int mb_last_cuda_error(char* buf, int32_t len) {
  if (buf == nullptr || len <= 0) return MB_E_INVALID;
  strncpy(buf, mb::g_last_cuda_error, static_cast<size_t>(len) - 1);
  buf[len - 1] = 0;
  return MB_SUCCESS;
}

int mb_attn_fwd(const mb_attn_fwd_args* args, void* cuda_stream) {
  return mb::launch_attn_fwd(args, static_cast<cudaStream_t>(cuda_stream));
}

int mb_attn_fwd_multi(const mb_attn_fwd_multi_args* args, void* cuda_stream) {
  return mb::launch_attn_fwd_multi(args, static_cast<cudaStream_t>(cuda_stream));
}

int mb_set_peer_wait_ms(uint32_t milliseconds) {
  mb::set_peer_wait_ms(milliseconds);
  return MB_SUCCESS;
}

int mb_status_peek_async(int32_t* pinned_host_dst, void* cuda_stream) {
  if (pinned_host_dst == nullptr) return MB_E_INVALID;
  int* word = mb::default_status_word();
  if (word == nullptr) return MB_E_CUDA;
  return cudaMemcpyAsync(pinned_host_dst, word, sizeof(int), cudaMemcpyDeviceToHost,
                         static_cast<cudaStream_t>(cuda_stream)) == cudaSuccess
             ? MB_SUCCESS
             : MB_E_CUDA;
}

int mb_attn_bwd_preprocess(const mb_bwd_preprocess_args* args, void* cuda_stream) {
  return mb::launch_bwd_preprocess(args, static_cast<cudaStream_t>(cuda_stream));
}

int mb_attn_bwd(const mb_attn_bwd_args* args, void* cuda_stream) {
  return mb::launch_attn_bwd(args, static_cast<cudaStream_t>(cuda_stream));
}

int mb_attn_bwd_dq_convert(const float* dq_accum, void* dq, int64_t dq_stride_b, int64_t dq_stride_s, int64_t dq_stride_h,
                           int32_t batch, int32_t sq, int32_t hq, int32_t stat_pad, int32_t out_mode,
                           float softmax_scale, void* cuda_stream) {
  return mb::launch_dq_convert(dq_accum, dq, dq_stride_b, dq_stride_s, dq_stride_h, batch, sq, hq, stat_pad, out_mode,
                               softmax_scale, static_cast<cudaStream_t>(cuda_stream));
}

int mb_attn_bwd_block_noalloc(const mb_attn_bwd_block_args* args, void* cuda_stream) {
  return mb::launch_bwd_block_noalloc(args, static_cast<cudaStream_t>(cuda_stream));
}

int mb_flash_reduce(const float* lhs, const float* rhs, float* out, int64_t rows, int32_t head_dim_plus_1,
                    void* cuda_stream) {
  return mb::launch_flash_reduce(lhs, rhs, out, rows, head_dim_plus_1, static_cast<cudaStream_t>(cuda_stream));
}

int mb_tree_merge(const float* const* srcs, int32_t n, float* out, int64_t rows, int32_t head_dim_plus_1,
                  void* cuda_stream) {
  return mb::launch_tree_merge(srcs, n, out, rows, head_dim_plus_1, static_cast<cudaStream_t>(cuda_stream));
}

int mb_merge_out_lse(const mb_merge_args* args, void* cuda_stream) {
  return mb::launch_merge(args, static_cast<cudaStream_t>(cuda_stream));
}

int mb_status_fetch(int32_t* out, void* cuda_stream) {
  if (out == nullptr) return MB_E_INVALID;
  int* word = mb::default_status_word();
  if (word == nullptr) return MB_E_CUDA;
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  int host = 0;
  if (cudaMemcpyAsync(&host, word, sizeof(int), cudaMemcpyDeviceToHost, st) != cudaSuccess) return MB_E_CUDA;
  if (cudaStreamSynchronize(st) != cudaSuccess) return MB_E_CUDA;
  if (host != 0 && cudaMemsetAsync(word, 0, sizeof(int), st) != cudaSuccess) return MB_E_CUDA;
  *out = host;
  return MB_SUCCESS;
}

}  // extern "C"
