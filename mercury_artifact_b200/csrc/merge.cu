// Running out/LSE merge of partial attention results (HBM-bound, element-wise).
//
// Replaces update_out_and_lse / _update_out_and_lse of the reference
// (utils/flash_attn_dsl.py:31-71): the generated ring loop calls it once per
// step on the fp32 state out[B,S,H,D], lse[B,S,H,1] with the block result
// block_out[B,S,H,D] (input dtype) and block_lse[B,H,S] (fp32, note the
// transposed layout).  The reference spends about eight eager element-wise
// kernels per step on this; here it is one pass: 4+2 bytes read and 4 bytes
// written per output element.
#include <cuda_bf16.h>

#include "mb_host.h"

namespace mb {

struct MergeArgs {
  float* out;             // [B,S,H,D] contiguous
  float* lse;             // [B,S,H] contiguous (the reference's [B,S,H,1])
  const void* block_out;  // bf16 or fp32, strides in elements, D contiguous
  long long bo_sb, bo_ss, bo_sh;
  const float* block_lse;  // [B,H,S] contiguous
  int B, S, H, D;
  int first;         // 1: adopt the block (first ring step)
  int block_is_f32;  // dtype of block_out
};

// A warp takes kRowsPerWarp consecutive (b, s, h) rows per iteration: lanes 0..3 fetch the rows' two
// log-sum-exp words and work out the weights at the same time, and every lane issues the float4 loads of all
// four rows before it uses any of them.  The weights of the NEXT group of rows are fetched and computed while
// the loads of the current group are in flight, so an iteration waits for memory once, not twice (with 68
// registers per thread only 24 warps fit an SM; two dependent round trips per iteration left the kernel at
// half the HBM rate).
constexpr int kRowsPerWarp = 4;

__device__ __forceinline__ void merge_weights(const MergeArgs& a, long long row0, long long rows, int lane, float& my_w,
                                              long long& my_brow) {
  my_w = 0.f;
  my_brow = 0;
  if (lane < kRowsPerWarp && row0 + lane < rows) {
    const long long row = row0 + lane;
    const int h = static_cast<int>(row % a.H);
    const long long bs = row / a.H;
    const int s = static_cast<int>(bs % a.S);
    const int b = static_cast<int>(bs / a.S);
    const float bl = a.block_lse[(static_cast<long long>(b) * a.H + h) * a.S + s];
    const float l = a.first ? -INFINITY : a.lse[row];
    float new_l;
    if (l == -INFINITY) {  // nothing accumulated yet for this row
      my_w = 1.f;
      new_l = bl;
    } else if (bl == -INFINITY) {  // the block saw no key for this row
      my_w = 0.f;
      new_l = l;
    } else {
      const float x = bl - l;
      // fast intrinsics: their error (2^-21 relative in the exponential, ~1e-7 absolute in the logarithm
      // of a number in [1, 2]) is far below the bf16 block they weigh, and they keep the register count low
      my_w = __fdividef(1.f, 1.f + __expf(-x));                 // sigmoid(block_lse - lse)
      new_l = l + fmaxf(x, 0.f) + __logf(1.f + __expf(-fabsf(x)));  // lse - logsigmoid(lse - block_lse)
    }
    a.lse[row] = new_l;
    my_brow = b * a.bo_sb + s * a.bo_ss + h * a.bo_sh;
  }
}

// The block's values stay in the form they were loaded in (bf16 pairs: half the registers) until they are used.
template <bool kBlockF32>
struct BlockVec;
template <>
struct BlockVec<true> {
  float4 v;
  __device__ __forceinline__ void load(const void* base, long long idx) {
    v = *reinterpret_cast<const float4*>(static_cast<const float*>(base) + idx);
  }
  __device__ __forceinline__ float4 get() const { return v; }
};
template <>
struct BlockVec<false> {
  uint2 raw;
  __device__ __forceinline__ void load(const void* base, long long idx) {
    raw = *reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(base) + idx);
  }
  __device__ __forceinline__ float4 get() const {
    float4 r;
    r.x = __uint_as_float(raw.x << 16);
    r.y = __uint_as_float(raw.x & 0xffff0000u);
    r.z = __uint_as_float(raw.y << 16);
    r.w = __uint_as_float(raw.y & 0xffff0000u);
    return r;
  }
};

#ifndef MB_MERGE_BLOCKS_PER_SM
#define MB_MERGE_BLOCKS_PER_SM 4
#endif

template <bool kBlockF32>
__global__ void __launch_bounds__(256, MB_MERGE_BLOCKS_PER_SM) merge_kernel(const MergeArgs a) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const long long rows = static_cast<long long>(a.B) * a.S * a.H;
  const long long step = nwarps * kRowsPerWarp;
  float my_w;
  long long my_brow;
  merge_weights(a, warp0 * kRowsPerWarp, rows, lane, my_w, my_brow);
  for (long long row0 = warp0 * kRowsPerWarp; row0 < rows; row0 += step) {
    float w[kRowsPerWarp];
    long long brow[kRowsPerWarp];
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
      w[r] = __shfl_sync(0xffffffffu, my_w, r);
      brow[r] = __shfl_sync(0xffffffffu, my_brow, r);
    }
    for (int d = lane * 4; d < a.D; d += 128) {
      BlockVec<kBlockF32> bo[kRowsPerWarp];
      float4 o[kRowsPerWarp];
#pragma unroll
      for (int r = 0; r < kRowsPerWarp; ++r) {
        if (row0 + r < rows) {
          bo[r].load(a.block_out, brow[r] + d);
          // w == 1 adopts the block: the old state (uninitialised on the first step) is not read
          if (w[r] != 1.f) o[r] = *reinterpret_cast<const float4*>(a.out + (row0 + r) * a.D + d);
        }
      }
      // the next group's weights, while this group's rows are on their way (once per group)
      if (d == lane * 4 && row0 + step < rows) merge_weights(a, row0 + step, rows, lane, my_w, my_brow);
#pragma unroll
      for (int r = 0; r < kRowsPerWarp; ++r) {
        if (row0 + r < rows) {
          const float4 bv = bo[r].get();
          float4 v = bv;
          if (w[r] != 1.f) {
            v = o[r];
            v.x -= w[r] * (v.x - bv.x);
            v.y -= w[r] * (v.y - bv.y);
            v.z -= w[r] * (v.z - bv.z);
            v.w -= w[r] * (v.w - bv.w);
          }
          *reinterpret_cast<float4*>(a.out + (row0 + r) * a.D + d) = v;
        }
      }
    }
  }
}

// Packed merge of two [rows, D+1] fp32 buffers, each row = [out (D values) | lse]:
// the reference's flash_reduce (utils/flash_attn_dsl.py:293-305), used by the ring-over-Q
// schedule whose reduce buffer rotates with the queries.  One warp per row; rows of D+1 floats
// are not 16-byte aligned, so lanes read consecutive floats (coalesced 128-byte lines).
// `out` may be the same buffer as `lhs` (the C ABI says so), hence no __restrict__ on those two: every
// element is read and written by the same lane, and the row's lse word is read by all lanes before the
// __syncwarp() that precedes lane 0's store of the merged value.
__global__ void __launch_bounds__(256) flash_reduce_kernel(const float* lhs, const float* __restrict__ rhs,
                                                           float* out, long long rows, int width) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const int d = width - 1;
  for (long long row = warp0; row < rows; row += nwarps) {
    const float* l = lhs + row * width;
    const float* r = rhs + row * width;
    float* o = out + row * width;
    const float ll = l[d], rl = r[d];
    __syncwarp();
    float w, new_l;
    if (ll == -INFINITY) {
      w = 1.f;
      new_l = rl;
    } else if (rl == -INFINITY) {
      w = 0.f;
      new_l = ll;
    } else {
      const float x = rl - ll;
      w = 1.f / (1.f + expf(-x));                            // sigmoid(r_lse - l_lse)
      new_l = ll + fmaxf(x, 0.f) + log1pf(expf(-fabsf(x)));  // l_lse - logsigmoid(l_lse - r_lse)
    }
    for (int c = lane; c < d; c += 32) {
      const float lo = l[c];
      o[c] = lo - w * (lo - r[c]);
    }
    if (lane == 0) o[d] = new_l;
  }
}

int launch_flash_reduce(const float* lhs, const float* rhs, float* out, long long rows, int width,
                        cudaStream_t stream) {
  if (rows < 0 || width < 2) return MB_E_INVALID;
  if (rows == 0) return MB_SUCCESS;
  if (lhs == nullptr || rhs == nullptr || out == nullptr) return MB_E_INVALID;
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long want = (rows + 7) / 8;
  const long long cap = static_cast<long long>(sms) * 8;
  flash_reduce_kernel<<<static_cast<int>(want < cap ? want : cap), 256, 0, stream>>>(lhs, rhs, out, rows, width);
  return cudaGetLastError() == cudaSuccess ? MB_SUCCESS : MB_E_CUDA;
}

// One-shot merge of n packed [rows, D+1] fp32 buffers (row = [out | lse]) into `out`:
//   lse* = log sum_r exp(lse_r),   out* = sum_r exp(lse_r - lse*) out_r
// which is what the reference's tree merge computes with three collectives
// (update_out_and_lse_collective, utils/flash_attn_dsl.py:307-324: all_reduce(MAX) of the LSE,
// then all_reduce(SUM) of the rescaled outputs and of the weights).  The source pointers may
// be other ranks' buffers mapped into this process: the loads then cross NVLink inside the
// kernel, each rank reading every peer once.  One warp per row, n <= 16.
struct TreeArgs {
  const float* src[16];
  float* out;
  long long rows;
  int n, width;
};

__global__ void __launch_bounds__(256) tree_merge_kernel(const TreeArgs a) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const int d = a.width - 1;
  for (long long row = warp0; row < a.rows; row += nwarps) {
    const long long base = row * a.width;
    float m = -INFINITY;
    float lse_r[16];
#pragma unroll
    for (int r = 0; r < 16; ++r) {
      lse_r[r] = r < a.n ? a.src[r][base + d] : -INFINITY;
      m = fmaxf(m, lse_r[r]);
    }
    float denom = 0.f;
#pragma unroll
    for (int r = 0; r < 16; ++r) {
      lse_r[r] = (r < a.n && m != -INFINITY) ? expf(lse_r[r] - m) : 0.f;  // now the weight of rank r
      denom += lse_r[r];
    }
    const float inv = denom > 0.f ? 1.f / denom : 0.f;
    for (int c = lane; c < d; c += 32) {
      float acc = 0.f;
#pragma unroll
      for (int r = 0; r < 16; ++r)
        if (r < a.n) acc += lse_r[r] * a.src[r][base + c];
      a.out[base + c] = acc * inv;
    }
    if (lane == 0) a.out[base + d] = denom > 0.f ? m + logf(denom) : -INFINITY;
  }
}

int launch_tree_merge(const float* const* srcs, int n, float* out, long long rows, int width, cudaStream_t stream) {
  if (n < 1 || n > 16 || rows < 0 || width < 2) return MB_E_INVALID;
  if (rows == 0) return MB_SUCCESS;
  if (srcs == nullptr || out == nullptr) return MB_E_INVALID;
  TreeArgs a;
  for (int r = 0; r < 16; ++r) a.src[r] = r < n ? srcs[r] : nullptr;
  for (int r = 0; r < n; ++r)
    if (a.src[r] == nullptr) return MB_E_INVALID;
  a.out = out;
  a.rows = rows;
  a.n = n;
  a.width = width;
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long want = (rows + 7) / 8;
  const long long cap = static_cast<long long>(sms) * 8;
  tree_merge_kernel<<<static_cast<int>(want < cap ? want : cap), 256, 0, stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? MB_SUCCESS : MB_E_CUDA;
}

int launch_merge(const mb_merge_args* x, cudaStream_t stream) {
  if (x == nullptr || x->out == nullptr || x->lse == nullptr || x->block_out == nullptr || x->block_lse == nullptr)
    return MB_E_INVALID;
  if (x->batch < 0 || x->seq < 0 || x->heads < 0 || x->head_dim <= 0) return MB_E_INVALID;
  if (x->head_dim % 4 != 0) return MB_E_UNSUPPORTED;
  if (x->block_dtype != MB_DTYPE_BF16 && x->block_dtype != MB_DTYPE_F32) return MB_E_UNSUPPORTED;
  const long long rows = static_cast<long long>(x->batch) * x->seq * x->heads;
  if (rows == 0) return MB_SUCCESS;
  MergeArgs a;
  a.out = x->out;
  a.lse = x->lse;
  a.block_out = x->block_out;
  a.bo_sb = x->block_stride_b;
  a.bo_ss = x->block_stride_s;
  a.bo_sh = x->block_stride_h;
  a.block_lse = x->block_lse;
  a.B = x->batch;
  a.S = x->seq;
  a.H = x->heads;
  a.D = x->head_dim;
  a.first = x->first ? 1 : 0;
  a.block_is_f32 = x->block_dtype == MB_DTYPE_F32;
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long want = (rows + 8 * kRowsPerWarp - 1) / (8 * kRowsPerWarp);  // 8 warps per block
  const long long cap = static_cast<long long>(sms) * MB_MERGE_BLOCKS_PER_SM;  // one resident wave, grid-stride loop
  const int grid = static_cast<int>(want < cap ? want : cap);
  if (a.block_is_f32) merge_kernel<true><<<grid, 256, 0, stream>>>(a);
  else merge_kernel<false><<<grid, 256, 0, stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? MB_SUCCESS : MB_E_CUDA;
}

}  // namespace mb
