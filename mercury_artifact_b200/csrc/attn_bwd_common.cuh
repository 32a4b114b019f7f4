// Pieces shared by the backward attention kernels (two-pass and single-pass): tile geometry, kernel
// arguments, the causal step range, the MMA group issue helpers and the element-wise math.
#pragma once

#include "mb_common.cuh"
#include "mb_host.h"

namespace mb {

constexpr int kOwnRows = 128;
constexpr int kStrRows = 64;
constexpr int kBD = 128;                              // head dim
constexpr int kOwnTileBytes = kOwnRows * kBD * 2;     // 32 KiB, two 64-column halves of 16 KiB
constexpr int kOwnHalfBytes = kOwnTileBytes / 2;
constexpr int kStrTileBytes = kStrRows * kBD * 2;     // 16 KiB, two halves of 8 KiB
constexpr int kStrHalfBytes = kStrTileBytes / 2;
constexpr int kStatBytes = 2 * kStrRows * 4;          // lse2[64] + delta[64]
constexpr int kBwdStageBytes = 2 * kStrTileBytes + 1024;  // Str + StrG + stats (padded)
constexpr int kBwdStages = 4;
constexpr int kBwdThreads = 320;                      // 8 element-wise warps + MMA warp + loader warp

struct BwdMaps {
  CUtensorMap own, own_g;                 // box 128 rows
  CUtensorMap str[MB_MAX_SEGMENTS];       // box 64 rows
  CUtensorMap str_g[MB_MAX_SEGMENTS];
};

struct BwdArgs {
  int mode_dkv;  // 1: owner = K/V, stream = Q/dO; 0: owner = Q/dO, stream = K/V
  int B, own_rows, Hq, Hkv, group;
  int own_off;  // global position of owner row 0
  int causal;
  float scale, scale_log2;
  int nseg;
  int seg_rows[MB_MAX_SEGMENTS];
  int seg_off[MB_MAX_SEGMENTS];                 // global position of the segment's row 0
  const float* seg_lse2[MB_MAX_SEGMENTS];       // dKV mode: stats of the segment's queries [B,Hq,pad]
  const float* seg_delta[MB_MAX_SEGMENTS];
  int seg_stat_pad[MB_MAX_SEGMENTS];            // padded row count of those arrays
  float* seg_dq[MB_MAX_SEGMENTS];               // single-pass mode: fp32 dQ accumulation [B,Hq,pad,D] of the segment
  const int* seg_flag[MB_MAX_SEGMENTS];
  int seg_flag_value[MB_MAX_SEGMENTS];
  long long peer_wait_cycles;                   // budget of a wait for a shard another GPU delivers
  long long wait_cycles;                        // budget of a wait inside the CTA (plus the above with flags)
  const float* own_lse2;                        // dQ mode: stats of the owner's queries [B,Hq,own_pad]
  const float* own_delta;
  int own_stat_pad;
  // outputs: acc1 -> (dK | dQ), acc2 -> dV.  [B, rows, heads, D], strides in elements.
  void* out1;
  void* out2;
  long long o_sb, o_ss, o_sh;
  int out_mode;  // 0 bf16 store, 1 fp32 store, 2 fp32 accumulate
  int* status;
};

struct BwdSmem {
  uint64_t own_full;
  uint64_t str_full[kBwdStages];
  uint64_t str_empty[kBwdStages];
  uint64_t xy_full[2];
  uint64_t pd_full[2];
  uint64_t acc_full;
  uint64_t drain;
  uint32_t tmem_base;
  int abort_word;
  int seg_first[MB_MAX_SEGMENTS];  // first and one-past-last 64-row step of each segment for this owner tile
  int seg_last[MB_MAX_SEGMENTS];
};

constexpr int kBwdSmemBytes = 2 * kOwnTileBytes + kBwdStages * kBwdStageBytes + 1024 + 1024;

// Range of 64-row stream steps of a segment that can interact with the owner tile.
__device__ __forceinline__ void step_range(const BwdArgs& a, int own0, int s, int* first, int* last) {
  const int rows = a.seg_rows[s];
  int f = 0, l = (rows + kStrRows - 1) / kStrRows;
  if (own0 >= a.own_rows || rows <= 0) {
    *first = 0;
    *last = 0;
    return;
  }
  if (a.causal) {
    const int own_lo = a.own_off + own0;
    const int own_hi = a.own_off + min(own0 + kOwnRows, a.own_rows) - 1;
    if (a.mode_dkv) {
      // stream = queries: a query row sees the owner's keys iff q_pos >= k_pos; need q_pos >= own_lo
      long long need = (long long)own_lo - a.seg_off[s];  // first local query row that can see key own_lo
      if (need > 0) f = (int)min((long long)l, need / kStrRows);
    } else {
      // stream = keys: visible iff k_pos <= q_pos; need k_pos <= own_hi
      long long maxk = (long long)own_hi - a.seg_off[s];
      if (maxk < 0) l = 0;
      else l = (int)min((long long)l, maxk / kStrRows + 1);
    }
  }
  if (f > l) f = l;
  *first = f;
  *last = l;
}

// Groups of MMAs issued from one asm block by a converged warp (one elected lane issues): the
// descriptors of the k-steps differ only in the start-address field (16-byte units), so each is
// one 64-bit add away, and a converged warp lets that arithmetic run on the uniform datapath.

// X (or Y) = Own * Stream^T for a 128 x 64 tile: 8 MMAs (K = 16) over the two 64-column halves.
// Offsets: owner tile half pitch 16 KiB (1024 units), stream tile half pitch 8 KiB (512 units).
__device__ __forceinline__ void issue_xy_group(uint32_t d_tmem, uint64_t own_desc, uint64_t str_desc,
                                               uint32_t idesc) {
  asm volatile(
      "{\n\t"
      ".reg .pred pe, pt, pf;\n\t"
      ".reg .b64 oa, sb;\n\t"
      "elect.sync _|pe, 0xffffffff;\n\t"
      "setp.eq.u32 pt, 0, 0;\n\t"
      "setp.ne.u32 pf, 0, 0;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, pf;\n\t"
      "add.s64 oa, %1, 2;\n\t add.s64 sb, %2, 2;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], oa, sb, %3, pt;\n\t"
      "add.s64 oa, %1, 4;\n\t add.s64 sb, %2, 4;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], oa, sb, %3, pt;\n\t"
      "add.s64 oa, %1, 6;\n\t add.s64 sb, %2, 6;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], oa, sb, %3, pt;\n\t"
      "add.s64 oa, %1, 1024;\n\t add.s64 sb, %2, 512;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], oa, sb, %3, pt;\n\t"
      "add.s64 oa, %1, 1026;\n\t add.s64 sb, %2, 514;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], oa, sb, %3, pt;\n\t"
      "add.s64 oa, %1, 1028;\n\t add.s64 sb, %2, 516;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], oa, sb, %3, pt;\n\t"
      "add.s64 oa, %1, 1030;\n\t add.s64 sb, %2, 518;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], oa, sb, %3, pt;\n\t"
      "}"
      :
      : "r"(d_tmem), "l"(own_desc), "l"(str_desc), "r"(idesc)
      : "memory");
}
static_assert(kOwnHalfBytes / 16 == 1024 && kStrHalfBytes / 16 == 512, "issue_xy_group hard-codes the tile pitches");

// Acc (+)= A[tmem] * Stream for the 64 stream rows of a step: 4 MMAs of 16 rows.  The bf16 A
// operand sits in columns [0,16) (rows 0..31) and [32,48) (rows 32..63) of its 64-column buffer;
// the stream tile is read MN-major, 16 rows = 2048 bytes = 128 descriptor units apart.
__device__ __forceinline__ void issue_acc_group(uint32_t d_tmem, uint32_t a_tmem, uint64_t str_desc, uint32_t idesc,
                                                uint32_t accumulate_first) {
  asm volatile(
      "{\n\t"
      ".reg .pred pe, pt, p0;\n\t"
      ".reg .b64 sb;\n\t"
      ".reg .b32 pa;\n\t"
      "elect.sync _|pe, 0xffffffff;\n\t"
      "setp.eq.u32 pt, 0, 0;\n\t"
      "setp.ne.u32 p0, %4, 0;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p0;\n\t"
      "add.s64 sb, %2, 128;\n\t add.u32 pa, %1, 8;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [pa], sb, %3, pt;\n\t"
      "add.s64 sb, %2, 256;\n\t add.u32 pa, %1, 32;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [pa], sb, %3, pt;\n\t"
      "add.s64 sb, %2, 384;\n\t add.u32 pa, %1, 40;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [pa], sb, %3, pt;\n\t"
      "}"
      :
      : "r"(d_tmem), "r"(a_tmem), "l"(str_desc), "r"(idesc), "r"(accumulate_first)
      : "memory");
}

#ifndef MB_BWD_PACKED
#define MB_BWD_PACKED 1
#endif

// p = exp2(x*c + nlse2), ds = p * (y - delta) for the 32 columns a thread owns; bf16 pairs out.
// kDkv: the statistics vary per column (read from the stage's shared-memory copy); otherwise they
// are the thread's row constants.  kMask: columns outside [lo, hi) are invisible (causal diagonal).
template <bool kDkv, bool kMask>
__device__ __forceinline__ void ew_compute(const uint32_t (&xr)[32], const uint32_t (&yr)[32], uint32_t (&pk)[16],
                                           uint32_t (&dk)[16], float c, const float* nl_col, const float* d_col,
                                           float row_nl, float row_d, int lo, int hi) {
#if MB_BWD_PACKED
  const uint64_t c2 = pack2(c, c);
  const uint64_t row_nl2 = pack2(row_nl, row_nl), row_d2 = pack2(row_d, row_d);
#pragma unroll
  for (int e = 0; e < 32; e += 2) {
    // per-column statistics: one 16-byte broadcast load serves two pairs (the arrays are 16-byte aligned)
    uint64_t nl2 = row_nl2, d2 = row_d2;
    if (kDkv) {
      const ulonglong2 nl4 = *reinterpret_cast<const ulonglong2*>(nl_col + (e & ~3));
      const ulonglong2 d4 = *reinterpret_cast<const ulonglong2*>(d_col + (e & ~3));
      nl2 = (e & 2) ? nl4.y : nl4.x;
      d2 = (e & 2) ? d4.y : d4.x;
    }
    const uint64_t t2 = fma2(pack2(__uint_as_float(xr[e]), __uint_as_float(xr[e + 1])), c2, nl2);
    float t0, t1;
    unpack2(t2, t0, t1);
    float p0 = fast_exp2(t0), p1 = fast_exp2(t1);
    if (kMask) {
      if (e < lo || e >= hi) p0 = 0.f;
      if (e + 1 < lo || e + 1 >= hi) p1 = 0.f;
    }
    const uint64_t s2 = mul2(pack2(p0, p1), sub2(pack2(__uint_as_float(yr[e]), __uint_as_float(yr[e + 1])), d2));
    float s0, s1;
    unpack2(s2, s0, s1);
    pk[e >> 1] = pack_bf16x2(p0, p1);
    dk[e >> 1] = pack_bf16x2(s0, s1);
  }
#else
#pragma unroll
  for (int e = 0; e < 32; e += 2) {
    float nl0 = row_nl, nl1 = row_nl, d0 = row_d, d1 = row_d;
    if (kDkv) {
      const float2 nv = *reinterpret_cast<const float2*>(nl_col + e);
      const float2 dv = *reinterpret_cast<const float2*>(d_col + e);
      nl0 = nv.x; nl1 = nv.y; d0 = dv.x; d1 = dv.y;
    }
    float p0 = fast_exp2(fmaf(__uint_as_float(xr[e]), c, nl0));
    float p1 = fast_exp2(fmaf(__uint_as_float(xr[e + 1]), c, nl1));
    if (kMask) {
      if (e < lo || e >= hi) p0 = 0.f;
      if (e + 1 < lo || e + 1 >= hi) p1 = 0.f;
    }
    const float s0 = p0 * (__uint_as_float(yr[e]) - d0);
    const float s1 = p1 * (__uint_as_float(yr[e + 1]) - d1);
    pk[e >> 1] = pack_bf16x2(p0, p1);
    dk[e >> 1] = pack_bf16x2(s0, s1);
  }
#endif
}

// single-pass kernel (attn_bwd_fused.cu), launched by launch_attn_bwd for MB_BWD_MODE_FUSED
int launch_attn_bwd_fused(const BwdMaps& maps, const BwdArgs& a, dim3 grid, cudaStream_t stream);

}  // namespace mb
