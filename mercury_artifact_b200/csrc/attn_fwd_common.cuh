// Pieces shared by the forward attention kernels: tile geometry, kernel arguments, the causal
// tile count, and the MMA group issue helpers.
#pragma once

#include "mb_common.cuh"
#include "mb_host.h"

namespace mb {

constexpr int kBM = 128;            // query rows per tile
constexpr int kBN = 128;            // keys per tile
constexpr int kD = 128;             // head dimension
constexpr int kTileBytes = kBN * kD * 2;  // 32 KiB, stored as two 64-column halves
constexpr int kHalfBytes = kTileBytes / 2;
#ifndef MB_FWD_STAGES
#define MB_FWD_STAGES 4
#endif
constexpr int kFwdStages = MB_FWD_STAGES;  // 32 KiB K or V tiles in flight (3, 4 and 5 measured alike)
constexpr int kFwdThreads = 384;  // 8 softmax warps + one auxiliary warpgroup (2 MMA issuers, loader, 1 idle)
constexpr float kRescaleThreshold = 8.0f;  // lazy rescale: tolerate p up to 2^8
constexpr int kMaxJobs = MB_MAX_JOBS;
constexpr int kMaxQMaps = 16;  // distinct query tensors per launch (jobs over the same rows share a map)

struct FwdMaps {
  CUtensorMap q[kMaxQMaps];
  CUtensorMap k[MB_MAX_SEGMENTS];
  CUtensorMap v[MB_MAX_SEGMENTS];
};

// One query shard of the launch and where its results go.
struct FwdJob {
  __nv_bfloat16* o;
  long long o_sb, o_ss, o_sh;  // element strides
  float* lse;                  // [B, Hq, Sq], row-contiguous
  long long lse_sb, lse_sh;    // element strides of lse
  int Sq, q_off;
  unsigned seg_mask;           // segments this job attends to
  int x_begin, n_pairs;        // first CTA of the job in the (one-dimensional) grid; query tile pairs
  const int* q_flag;           // arrival flag of the query shard (nullptr: in place)
  int q_flag_value;
  int done_value;              // stored to *done_flag by the job's last CTA
  int* done_flag;
  int* done_counter;
  int n_ctas;
  // Carried online-softmax state (see mb_fwd_job): unnormalised rows [B, Hq, Sq, D] and (maximum, sum)
  // pairs [B, Hq, Sq, 2], both fp32; chain words [B, Hq, n_pairs].
  float* st_o;
  float* st_ml;
  int* chain;
  int chain_wait, chain_set;
  int st_in, st_out;
  int qmap;  // index of the job's query tensor map
};

struct FwdArgs {
  FwdJob job[kMaxJobs];
  int njobs;
  int B, Hq, group;
  int nseg;
  int seg_sk[MB_MAX_SEGMENTS];
  int seg_koff[MB_MAX_SEGMENTS];
  const int* seg_flag[MB_MAX_SEGMENTS];  // arrival flag of a staged shard (nullptr: already in place)
  int seg_flag_value[MB_MAX_SEGMENTS];
  int causal;
  float scale;       // softmax scale
  float scale_log2;  // softmax scale * log2(e)
  long long peer_wait_cycles;  // budget of a wait for data another GPU delivers
  long long wait_cycles;       // budget of a wait inside the CTA (plus the above when the launch has flags)
  int* status;
};

struct FwdSmem {
  uint64_t q_full;
  uint64_t kv_full[kFwdStages];
  uint64_t kv_empty[kFwdStages];
  uint64_t s_full[2];
  uint64_t s_free;        // the one score region is handed from user to user (4 warp arrivals per use)
  uint64_t p_full[2][2];  // [query tile][half of the keys of a K/V tile]
  uint64_t o_full[2];
  uint64_t drain;
  uint32_t tmem_base;
  int abort_word;
  int jid;
  int pair, h, b;  // this CTA's query tile pair, head and batch entry
  int n_tiles[2][MB_MAX_SEGMENTS];  // K/V tiles of each segment that query tile i takes part in
  FwdJob job;                       // this CTA's job (a copy: read with fixed offsets, no registers held)
};

constexpr int kFwdSmemBytes = 2 * kTileBytes + kFwdStages * kTileBytes + 1024 /*alignment slack*/ + 1024 /*FwdSmem*/;
static_assert(sizeof(FwdSmem) <= 1024, "control block too large");
static_assert(kFwdSmemBytes <= 232448, "shared memory budget of one CTA");

// Number of K/V tiles of a segment that a query tile starting at row q0 can see.
__device__ __forceinline__ int visible_tiles(int q0, int Sq, int q_off, int causal, int sk, int koff) {
  if (q0 >= Sq || sk <= 0) return 0;
  int nt = (sk + kBN - 1) / kBN;
  if (causal) {
    int last_row = min(q0 + kBM - 1, Sq - 1);
    long long max_k = (long long)q_off + last_row - koff;  // largest visible local key index
    if (max_k < 0) return 0;
    long long lim = max_k / kBN + 1;
    if (lim < nt) nt = (int)lim;
  }
  return nt;
}

// Called by a converged warp; one elected lane issues.  Keeping the warp converged lets the
// descriptor arithmetic run on the uniform datapath (tcgen05.mma takes its descriptors from uniform
// registers), and one asm block per group of MMAs keeps the instruction count low: the
// shared-memory descriptors of the k-steps differ from the first one only in the start-address
// field (bits 0-13, in 16-byte units), so each is one 64-bit add away.

// S = Q K^T for one 128x128 tile: 8 MMAs (K = 16 each) over the two 64-column halves of Q and K.
// Offsets in 16-byte units: k-step k -> (k >> 2) * (kHalfBytes / 16) + (k & 3) * 2.
__device__ __forceinline__ void issue_qk(uint32_t d_tmem, uint64_t q_desc, uint64_t k_desc, uint32_t idesc) {
  asm volatile(
      "{\n\t"
      ".reg .pred pe, pt, pf;\n\t"
      ".reg .b64 qa, kb;\n\t"
      "elect.sync _|pe, 0xffffffff;\n\t"
      "setp.eq.u32 pt, 0, 0;\n\t"
      "setp.ne.u32 pf, 0, 0;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, pf;\n\t"
      "add.s64 qa, %1, 2;\n\t add.s64 kb, %2, 2;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], qa, kb, %3, pt;\n\t"
      "add.s64 qa, %1, 4;\n\t add.s64 kb, %2, 4;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], qa, kb, %3, pt;\n\t"
      "add.s64 qa, %1, 6;\n\t add.s64 kb, %2, 6;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], qa, kb, %3, pt;\n\t"
      "add.s64 qa, %1, 1024;\n\t add.s64 kb, %2, 1024;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], qa, kb, %3, pt;\n\t"
      "add.s64 qa, %1, 1026;\n\t add.s64 kb, %2, 1026;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], qa, kb, %3, pt;\n\t"
      "add.s64 qa, %1, 1028;\n\t add.s64 kb, %2, 1028;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], qa, kb, %3, pt;\n\t"
      "add.s64 qa, %1, 1030;\n\t add.s64 kb, %2, 1030;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], qa, kb, %3, pt;\n\t"
      "}"
      :
      : "r"(d_tmem), "l"(q_desc), "l"(k_desc), "r"(idesc)
      : "memory");
}
static_assert(kHalfBytes / 16 == 1024, "issue_qk hard-codes the half-tile pitch");

// O (+)= P V for 64 keys (half of a K/V tile): 4 MMAs of 16 keys.  P comes from tensor memory
// (8 columns per 16 keys); V is read MN-major, 16 keys = 2048 bytes = 128 descriptor units apart.
// p_tmem and v_desc already point at the half to process.
__device__ __forceinline__ void issue_pv_half(uint32_t d_tmem, uint32_t p_tmem, uint64_t v_desc, uint32_t idesc,
                                              uint32_t accumulate_first) {
  asm volatile(
      "{\n\t"
      ".reg .pred pe, pt, p0;\n\t"
      ".reg .b64 vb;\n\t"
      ".reg .b32 pa;\n\t"
      "elect.sync _|pe, 0xffffffff;\n\t"
      "setp.eq.u32 pt, 0, 0;\n\t"
      "setp.ne.u32 p0, %4, 0;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p0;\n\t"
      "add.s64 vb, %2, 128;\n\t add.u32 pa, %1, 8;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [pa], vb, %3, pt;\n\t"
      "add.s64 vb, %2, 256;\n\t add.u32 pa, %1, 16;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [pa], vb, %3, pt;\n\t"
      "add.s64 vb, %2, 384;\n\t add.u32 pa, %1, 24;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [pa], vb, %3, pt;\n\t"
      "}"
      :
      : "r"(d_tmem), "r"(p_tmem), "l"(v_desc), "r"(idesc), "r"(accumulate_first)
      : "memory");
}

}  // namespace mb
