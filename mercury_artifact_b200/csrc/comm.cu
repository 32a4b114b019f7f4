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

// ---------------------------------------------------------------------------
// SM-driven pull: peer memory -> shared memory -> local memory with bulk copies
// ---------------------------------------------------------------------------
constexpr int kPullChunk = 8192;
constexpr int kPullDepth = 3;
constexpr int kPullSmemBytes = kPullDepth * kPullChunk;

struct PullArgs {
  const uint8_t* src[MB_MAX_PULL_RANGES];
  uint8_t* dst[MB_MAX_PULL_RANGES];
  unsigned long long bytes[MB_MAX_PULL_RANGES];
  int first_chunk[MB_MAX_PULL_RANGES + 1];  // prefix sums of the ranges' chunk counts
  int nranges;
  const int* wait_flag;
  int wait_value;
  int* flag[MB_MAX_PULL_FLAGS];
  int value[MB_MAX_PULL_FLAGS];
  int nflags;
  int* counter;
  long long wait_cycles;
  int* status;
};

__global__ void __launch_bounds__(32) pull_kernel(const __grid_constant__ PullArgs a) {
  extern __shared__ __align__(128) uint8_t pull_smem[];
  __shared__ uint64_t bar[kPullDepth];
  __shared__ int abort_word;
  if (threadIdx.x == 0) {
    abort_word = 0;
    for (int i = 0; i < kPullDepth; ++i) mbar_init(&bar[i], 1);
    fence_barrier_init();
    fence_proxy_async_smem();
    bool ok = true;
    if (a.wait_flag != nullptr) {
      ok = flag_wait_ge(a.wait_flag, a.wait_value, &abort_word, MB_ERR_TIMEOUT_FLAG, a.wait_cycles);
      asm volatile("fence.proxy.async;" ::: "memory");
    }
    const int total = a.first_chunk[a.nranges];
    // chunk c of this CTA's list: global chunk index blockIdx.x + c * gridDim.x
    auto chunk_of = [&](int idx, const uint8_t** src, uint8_t** dst, unsigned* nbytes) {
      int r = 0;
      while (r + 1 < a.nranges && idx >= a.first_chunk[r + 1]) ++r;
      const unsigned long long off = static_cast<unsigned long long>(idx - a.first_chunk[r]) * kPullChunk;
      const unsigned long long left = a.bytes[r] - off;
      *src = a.src[r] + off;
      *dst = a.dst[r] + off;
      *nbytes = static_cast<unsigned>(left < kPullChunk ? left : kPullChunk);
    };
    const int mine = ok && (int)blockIdx.x < total ? (total - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    // kPullDepth buffers: one being drained by a store, the others receiving loads.  Chunk c + kPullDepth - 1
    // goes into the buffer chunk c - 1 was stored from; that store is the second most recent bulk group
    // when the refill is issued (right after the store of chunk c), hence wait_group.read 1.
    int issued = 0;
    auto issue_load = [&](int c) {
      const uint8_t* src;
      uint8_t* dst;
      unsigned nbytes;
      chunk_of(blockIdx.x + c * gridDim.x, &src, &dst, &nbytes);
      const int b = c % kPullDepth;
      mbar_expect_tx(&bar[b], nbytes);
      bulk_load(pull_smem + b * kPullChunk, src, nbytes, &bar[b]);
      ++issued;
    };
    for (int c = 0; c < kPullDepth - 1 && c < mine; ++c) issue_load(c);
    for (int c = 0; c < mine && ok; ++c) {
      const int b = c % kPullDepth;
      ok = mbar_wait(&bar[b], (c / kPullDepth) & 1, &abort_word, MB_ERR_TIMEOUT_MISC, a.wait_cycles);
      if (!ok) break;
      const uint8_t* src;
      uint8_t* dst;
      unsigned nbytes;
      chunk_of(blockIdx.x + c * gridDim.x, &src, &dst, &nbytes);
      asm volatile(
          "cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;\n\t"
          "cp.async.bulk.commit_group;" ::"l"(dst),
          "r"(smem_u32(pull_smem + b * kPullChunk)), "r"(nbytes)
          : "memory");
      const int nxt = c + kPullDepth - 1;
      if (nxt < mine) {
        if (c >= 1) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
        issue_load(nxt);
      }
    }
    if (!ok) {
      // loads still in flight must land before the CTA (and its shared memory) goes away: bounded
      for (int m = 0; m < kPullDepth; ++m) {
        const long long t0 = clock64();
        while (issued > m && !mbar_try_wait(&bar[m], ((issued - 1 - m) / kPullDepth) & 1) &&
               clock64() - t0 < kWaitCycleLimit / 16) {
        }
      }
    }
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // every store of this CTA is complete
    if (abort_word != 0 && a.status != nullptr) atomicCAS(a.status, 0, abort_word);
    // count this CTA; the last one publishes (a CTA that gave up still counts, the status word tells the host)
    __threadfence();
    int prev;
    asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(prev) : "l"(a.counter) : "memory");
    if (prev == (int)gridDim.x - 1) {
      *a.counter = 0;
      __threadfence_system();
      for (int i = 0; i < a.nflags; ++i)
        asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(a.flag[i]), "r"(a.value[i]) : "memory");
    }
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
  cudaFuncSetAttribute(pull_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
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

int mb_copy2d_async(void* dst, uint64_t dpitch, const void* src, uint64_t spitch, uint64_t width, uint64_t height,
                    void* cuda_stream) {
  if (width == 0 || height == 0) return MB_SUCCESS;
  if (dst == nullptr || src == nullptr || dpitch < width || spitch < width) return MB_E_INVALID;
  if ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src) | dpitch | spitch | width) & 15u)
    return MB_E_INVALID;
  return mb::cuda_ok(cudaMemcpy2DAsync(dst, dpitch, src, spitch, width, height, cudaMemcpyDefault,
                                       static_cast<cudaStream_t>(cuda_stream)),
                     "cudaMemcpy2DAsync")
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

int mb_pull_sm(const mb_pull_args* x, void* cuda_stream) {
  if (x == nullptr || x->nranges < 0 || x->nranges > MB_MAX_PULL_RANGES || x->nflags < 0 ||
      x->nflags > MB_MAX_PULL_FLAGS || x->counter == nullptr || x->ctas < 0)
    return MB_E_INVALID;
  mb::PullArgs a;
  memset(&a, 0, sizeof(a));
  int n = 0, chunks = 0;
  for (int r = 0; r < x->nranges; ++r) {
    const mb_pull_range& g = x->range[r];
    if (g.bytes == 0) continue;
    if (g.src == nullptr || g.dst == nullptr) return MB_E_INVALID;
    if ((reinterpret_cast<uintptr_t>(g.src) | reinterpret_cast<uintptr_t>(g.dst) | g.bytes) & 15u) return MB_E_INVALID;
    a.src[n] = static_cast<const uint8_t*>(g.src);
    a.dst[n] = static_cast<uint8_t*>(g.dst);
    a.bytes[n] = g.bytes;
    a.first_chunk[n] = chunks;
    chunks += static_cast<int>((g.bytes + mb::kPullChunk - 1) / mb::kPullChunk);
    ++n;
  }
  a.first_chunk[n] = chunks;
  a.nranges = n;
  a.wait_flag = x->wait_flag;
  a.wait_value = x->wait_value;
  for (int i = 0; i < x->nflags; ++i) {
    if (x->flag[i] == nullptr) return MB_E_INVALID;
    a.flag[i] = x->flag[i];
    a.value[i] = x->value[i];
  }
  a.nflags = x->nflags;
  a.counter = x->counter;
  a.wait_cycles = mb::peer_wait_cycles();
  a.status = x->status ? x->status : mb::default_status_word();
  if (a.status == nullptr) return MB_E_CUDA;
  int dev = 0, sms = 148;
  if (!mb::cuda_ok(cudaGetDevice(&dev), "cudaGetDevice")) return MB_E_CUDA;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int grid = x->ctas > 0 ? x->ctas : sms;
  if (chunks > 0 && grid > chunks) grid = chunks;
  if (grid < 1) grid = 1;
  mb::prefer_max_smem_carveout_once();
  mb::pull_kernel<<<grid, 32, mb::kPullSmemBytes, static_cast<cudaStream_t>(cuda_stream)>>>(a);
  return mb::cuda_ok(cudaGetLastError(), "launch pull_kernel") ? MB_SUCCESS : MB_E_CUDA;
}

}  // extern "C"
