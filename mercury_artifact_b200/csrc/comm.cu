// Peer-memory plumbing for one-process-per-GPU jobs on an NVSwitch box:
// IPC-shareable allocations, handle export/import, stream-ordered flag
// signal/wait kernels with system-scope release/acquire, and async copies that
// the copy engines run over NVLink.
//
// Together these replace the reference's SendRecv helper
// (mercury/backend/pytorch/utils.py:9-39: NCCL batch_isend_irecv + req.wait):
// a send becomes "copy into the peer's inbox slot, then raise the peer's flag",
// a wait becomes "wait on my own flag".  The wait is bounded: when the budget
// runs out the kernel writes MB_ERR_TIMEOUT_FLAG to the status word and returns,
// leaving the context usable.
#include "mb_common.cuh"
#include "mb_host.h"

namespace mb {

__global__ void flag_signal_kernel(int* flag, int value) {
  __threadfence_system();
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(flag), "r"(value) : "memory");
}

__global__ void flag_wait_kernel(const int* flag, int value, unsigned long long timeout_ns, int* status) {
  unsigned long long t0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  unsigned spins = 0;
  for (;;) {
    int seen;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(flag) : "memory");
    if (seen >= value) return;
    if (((++spins) & 255u) == 0u) {
      unsigned long long now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      if (now - t0 > timeout_ns) {
        if (status != nullptr) atomicCAS(status, 0, MB_ERR_TIMEOUT_FLAG);
        return;
      }
    }
    __nanosleep(200);
  }
}

// Up to 32 flags per launch: lane i handles flag i.
struct FlagBatch {
  int* flag[32];
  int value[32];
  int n;
};

__global__ void flags_signal_kernel(const __grid_constant__ FlagBatch b) {
  __threadfence_system();
  const int i = threadIdx.x;
  if (i < b.n) asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(b.flag[i]), "r"(b.value[i]) : "memory");
}

__global__ void flags_wait_kernel(const __grid_constant__ FlagBatch b, unsigned long long timeout_ns, int* status) {
  const int i = threadIdx.x;
  if (i >= b.n) return;
  unsigned long long t0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  unsigned spins = 0;
  for (;;) {
    int seen;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(b.flag[i]) : "memory");
    if (seen >= b.value[i]) return;
    if (((++spins) & 255u) == 0u) {
      unsigned long long now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      if (now - t0 > timeout_ns) {
        if (status != nullptr) atomicCAS(status, 0, MB_ERR_TIMEOUT_FLAG);
        return;
      }
    }
    __nanosleep(200);
  }
}

// The flag kernels must be able to start while an attention kernel fills every SM.  An SM
// only co-hosts kernels that agree on its shared-memory carve-out, and the attention
// kernels run with the largest one, so the flag kernels ask for the same.
static void prefer_max_smem_carveout_once() {
  static bool done[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64 || done[dev]) return;
  cudaFuncSetAttribute(flag_signal_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                       cudaSharedmemCarveoutMaxShared);
  cudaFuncSetAttribute(flag_wait_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                       cudaSharedmemCarveoutMaxShared);
  cudaFuncSetAttribute(flags_signal_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                       cudaSharedmemCarveoutMaxShared);
  cudaFuncSetAttribute(flags_wait_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                       cudaSharedmemCarveoutMaxShared);
  done[dev] = true;
}

}  // namespace mb

extern "C" {

int mb_mem_alloc(void** ptr, uint64_t bytes) {
  if (ptr == nullptr) return MB_E_INVALID;
  *ptr = nullptr;
  if (bytes == 0) return MB_SUCCESS;
  return cudaMalloc(ptr, bytes) == cudaSuccess ? MB_SUCCESS : MB_E_CUDA;
}

int mb_mem_free(void* ptr) {
  if (ptr == nullptr) return MB_SUCCESS;
  return cudaFree(ptr) == cudaSuccess ? MB_SUCCESS : MB_E_CUDA;
}

int mb_mem_zero(void* ptr, uint64_t bytes, void* cuda_stream) {
  if (ptr == nullptr && bytes != 0) return MB_E_INVALID;
  if (bytes == 0) return MB_SUCCESS;
  return cudaMemsetAsync(ptr, 0, bytes, static_cast<cudaStream_t>(cuda_stream)) == cudaSuccess ? MB_SUCCESS
                                                                                                : MB_E_CUDA;
}

int mb_ipc_export(void* ptr, unsigned char* handle64) {
  if (ptr == nullptr || handle64 == nullptr) return MB_E_INVALID;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, ptr) != cudaSuccess) return MB_E_CUDA;
  memcpy(handle64, &h, 64);
  return MB_SUCCESS;
}

int mb_ipc_import(const unsigned char* handle64, void** ptr) {
  if (ptr == nullptr || handle64 == nullptr) return MB_E_INVALID;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  *ptr = nullptr;
  return cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess ? MB_SUCCESS : MB_E_CUDA;
}

int mb_ipc_release(void* ptr) {
  if (ptr == nullptr) return MB_SUCCESS;
  return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? MB_SUCCESS : MB_E_CUDA;
}

int mb_copy_async(void* dst, const void* src, uint64_t bytes, void* cuda_stream) {
  if (bytes == 0) return MB_SUCCESS;
  if (dst == nullptr || src == nullptr) return MB_E_INVALID;
  return cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, static_cast<cudaStream_t>(cuda_stream)) == cudaSuccess
             ? MB_SUCCESS
             : MB_E_CUDA;
}

int mb_flag_signal(int32_t* flag, int32_t value, void* cuda_stream) {
  if (flag == nullptr) return MB_E_INVALID;
  mb::prefer_max_smem_carveout_once();
  mb::flag_signal_kernel<<<1, 1, 0, static_cast<cudaStream_t>(cuda_stream)>>>(flag, value);
  return cudaGetLastError() == cudaSuccess ? MB_SUCCESS : MB_E_CUDA;
}

int mb_flag_wait(const int32_t* flag, int32_t value, uint64_t timeout_ns, int32_t* status, void* cuda_stream) {
  if (flag == nullptr) return MB_E_INVALID;
  int* st = status ? status : mb::default_status_word();
  mb::prefer_max_smem_carveout_once();
  mb::flag_wait_kernel<<<1, 1, 0, static_cast<cudaStream_t>(cuda_stream)>>>(flag, value, timeout_ns, st);
  return cudaGetLastError() == cudaSuccess ? MB_SUCCESS : MB_E_CUDA;
}

static int fill_batch(mb::FlagBatch* b, const int32_t* const* flags, const int32_t* values, int32_t n) {
  if (flags == nullptr || values == nullptr || n < 0 || n > 32) return MB_E_INVALID;
  memset(b, 0, sizeof(*b));
  for (int i = 0; i < n; ++i) {
    if (flags[i] == nullptr) return MB_E_INVALID;
    b->flag[i] = const_cast<int*>(flags[i]);
    b->value[i] = values[i];
  }
  b->n = n;
  return MB_SUCCESS;
}

int mb_flags_signal(int32_t* const* flags, const int32_t* values, int32_t n, void* cuda_stream) {
  mb::FlagBatch b;
  int rc = fill_batch(&b, flags, values, n);
  if (rc != MB_SUCCESS || n == 0) return rc;
  mb::prefer_max_smem_carveout_once();
  mb::flags_signal_kernel<<<1, 32, 0, static_cast<cudaStream_t>(cuda_stream)>>>(b);
  return cudaGetLastError() == cudaSuccess ? MB_SUCCESS : MB_E_CUDA;
}

int mb_flags_wait(const int32_t* const* flags, const int32_t* values, int32_t n, uint64_t timeout_ns, int32_t* status,
                  void* cuda_stream) {
  mb::FlagBatch b;
  int rc = fill_batch(&b, flags, values, n);
  if (rc != MB_SUCCESS || n == 0) return rc;
  int* st = status ? status : mb::default_status_word();
  mb::prefer_max_smem_carveout_once();
  mb::flags_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(cuda_stream)>>>(b, timeout_ns, st);
  return cudaGetLastError() == cudaSuccess ? MB_SUCCESS : MB_E_CUDA;
}

}  // extern "C"
