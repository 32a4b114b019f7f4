// Forward attention over a list of K/V segments for sm_100a.
//
// One CTA owns two 128-row query tiles of one (batch, query-head) and streams
// every K/V tile of every segment through them, keeping the online-softmax
// state (row max, row sum, fp32 output accumulator) on chip for the whole list.
// A "segment" is one sequence shard of K and V: the per-step block of the ring
// schedule is a one-segment call, and the whole ring (or double ring) for one
// rank is an nseg-segment call whose segment order is the rank's arrival order.
// Because the running state never leaves the SM, the per-step out/LSE merge of
// the generated ring loop (utils/flash_attn_dsl.py:31-71 in the reference)
// disappears from the fused path.
//
// Roles inside the CTA (384 threads, three warpgroups):
//   warps 0-3  softmax + epilogue for query tile 0 (one thread per row)
//   warps 4-7  softmax + epilogue for query tile 1
//   warp  8    tcgen05.mma issuer for query tile 0 (lane 0) and tensor-memory owner
//   warp  9    TMA loader (lane 0)
//   warp 10    tcgen05.mma issuer for query tile 1 (lane 0); one issuing thread for both tiles
//              cannot feed the tensor pipe (measured ~95 cycles per MMA instruction issued)
//   warp 11    idle; the auxiliary warpgroup's registers go to the softmax warps (setmaxnreg)
// Tensor memory (512 columns): S0 | S1 | O0 | O1, 128 fp32 columns each.  The
// bf16 probabilities overwrite the first 64 columns of their score tile and are
// consumed from tensor memory as the A operand of the P.V product.
#include "mb_common.cuh"
#include "mb_host.h"

namespace mb {

constexpr int kBM = 128;            // query rows per tile
constexpr int kBN = 128;            // keys per tile
constexpr int kD = 128;             // head dimension
constexpr int kTileBytes = kBN * kD * 2;  // 32 KiB, stored as two 64-column halves
constexpr int kHalfBytes = kTileBytes / 2;
constexpr int kFwdStages = 4;
constexpr int kFwdThreads = 384;  // 8 softmax warps + one auxiliary warpgroup (MMA, loader, 2 idle)
constexpr float kRescaleThreshold = 8.0f;  // lazy rescale: tolerate p up to 2^8
#ifndef MB_POLY_EVERY
#define MB_POLY_EVERY 0
#endif
constexpr int kPolyEvery = MB_POLY_EVERY;
#ifndef MB_TAKE_TURNS
#define MB_TAKE_TURNS 1
#endif
constexpr bool kTakeTurns = MB_TAKE_TURNS != 0;  // every n-th pair of exponentials goes to the FMA pipe (0: none)

// Optional timeline capture for kernel tuning (compiled in only with -DMB_TRACE): CTA (0,0,0)
// records clock64() at fixed points of the first kTraceIters K/V iterations.
#ifdef MB_TRACE
constexpr int kTraceIters = 24;
__device__ long long g_fwd_trace[3][kTraceIters][12];
#define MB_TRACE_AT(role, it, ev)                                                              \
  do {                                                                                         \
    if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (it) < kTraceIters)           \
      g_fwd_trace[role][it][ev] = clock64();                                                   \
  } while (0)
#else
#define MB_TRACE_AT(role, it, ev) \
  do {                            \
  } while (0)
#endif

struct FwdMaps {
  CUtensorMap q;
  CUtensorMap k[MB_MAX_SEGMENTS];
  CUtensorMap v[MB_MAX_SEGMENTS];
};

struct FwdArgs {
  __nv_bfloat16* o;
  long long o_sb, o_ss, o_sh;  // element strides
  float* lse;                  // [B, Hq, Sq], row-contiguous
  long long lse_sb, lse_sh;    // element strides of lse
  int B, Sq, Hq, group;
  int nseg;
  int seg_sk[MB_MAX_SEGMENTS];
  int seg_koff[MB_MAX_SEGMENTS];
  const int* seg_flag[MB_MAX_SEGMENTS];  // arrival flag of a staged shard (nullptr: already in place)
  int seg_flag_value[MB_MAX_SEGMENTS];
  int q_off;
  int causal;
  float scale;       // softmax scale
  float scale_log2;  // softmax scale * log2(e)
  int* status;
};

struct FwdSmem {
  uint64_t q_full;
  uint64_t kv_full[kFwdStages];
  uint64_t kv_empty[kFwdStages];
  uint64_t s_full[2];
  uint64_t p_full[2][2];  // [query tile][half of the keys of a K/V tile]
  uint64_t o_full[2];
  uint64_t turn[2];  // exp2-phase token passed between the two softmax warpgroups
  uint64_t drain;
  uint32_t tmem_base;
  int abort_word;
  int n_tiles[2][MB_MAX_SEGMENTS];  // K/V tiles of each segment that query tile i takes part in
};

constexpr int kFwdSmemBytes = 2 * kTileBytes + kFwdStages * kTileBytes + 1024 /*alignment slack*/ + 1024 /*FwdSmem*/;
static_assert(sizeof(FwdSmem) <= 1024, "control block too large");

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

// 160 registers/thread at launch (not the 168 that 384 threads would allow): the few warps' worth
// left free on the SM let the transfer stream's one-thread flag kernels start beside a resident CTA.
__global__ void __maxnreg__(160)
attn_fwd_kernel(const __grid_constant__ FwdMaps maps, const FwdArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sKV = smem + 2 * kTileBytes;
  FwdSmem* ctl = reinterpret_cast<FwdSmem*>(smem + 2 * kTileBytes + kFwdStages * kTileBytes);
  volatile int* abort_word = &ctl->abort_word;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  // Heavier (later) query rows first when causal.
  const int pair = a.causal ? (gridDim.x - 1 - blockIdx.x) : blockIdx.x;
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int hkv = h / a.group;
  const int q0 = pair * 2 * kBM;

  if (tid == 0) {
    mbar_init(&ctl->q_full, 1);
    for (int s = 0; s < kFwdStages; ++s) {
      mbar_init(&ctl->kv_full[s], 1);
      mbar_init(&ctl->kv_empty[s], 2);  // one arrival from each of the two MMA-issuing warps
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&ctl->s_full[i], 1);
      mbar_init(&ctl->p_full[i][0], 128);
      mbar_init(&ctl->p_full[i][1], 128);
      mbar_init(&ctl->o_full[i], 1);
      mbar_init(&ctl->turn[i], 128);
    }
    mbar_init(&ctl->drain, 2);
    ctl->abort_word = 0;
    for (int i = 0; i < 2; ++i)
      for (int s = 0; s < MB_MAX_SEGMENTS; ++s)
        ctl->n_tiles[i][s] =
            s < a.nseg ? visible_tiles(q0 + i * kBM, a.Sq, a.q_off, a.causal, a.seg_sk[s], a.seg_koff[s]) : 0;
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == 8) {
    tmem_alloc(&ctl->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  const uint32_t tmem = ctl->tmem_base;  // columns: S0 [0,128) S1 [128,256) O0 [256,384) O1 [384,512)

  bool any_work = false;
  for (int s = 0; s < a.nseg; ++s) any_work |= (ctl->n_tiles[0][s] | ctl->n_tiles[1][s]) != 0;

  // Registers move from the auxiliary warpgroup (warps 8-11) to the two softmax
  // warpgroups; each role changes its own budget as the first thing it does.
  if (warp == 11) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 48;");
  } else if (warp == 9) {
    // ------------------------------------------------------------------ loader
    asm volatile("setmaxnreg.dec.sync.aligned.u32 48;");
    if (lane == 0 && any_work) {
      tma_prefetch_desc(&maps.q);
      const int act0 = q0 < a.Sq, act1 = q0 + kBM < a.Sq;
      mbar_expect_tx(&ctl->q_full, (act0 + act1) * kTileBytes);
      for (int i = 0; i < 2; ++i) {
        if (q0 + i * kBM < a.Sq) {
          tma_load_4d(sQ + i * kTileBytes, &maps.q, &ctl->q_full, 0, h, q0 + i * kBM, b);
          tma_load_4d(sQ + i * kTileBytes + kHalfBytes, &maps.q, &ctl->q_full, 64, h, q0 + i * kBM, b);
        }
      }
      int n = 0;
      bool ok = true;
      for (int s = 0; s < a.nseg && ok; ++s) {
        const int nmax = max(ctl->n_tiles[0][s], ctl->n_tiles[1][s]);
        if (nmax > 0 && a.seg_flag[s] != nullptr) {
          // The shard is being staged by another stream: wait (bounded) for its arrival flag,
          // then order the TMA reads (async proxy) after the flag read.
          ok = flag_wait_ge(a.seg_flag[s], a.seg_flag_value[s], abort_word, MB_ERR_TIMEOUT_SEGMENT);
          asm volatile("fence.proxy.async;" ::: "memory");
        }
        for (int jt = 0; jt < nmax && ok; ++jt) {
          for (int which = 0; which < 2; ++which) {
            const int stage = n % kFwdStages;
            const int round = n / kFwdStages;
            if (round > 0 && !mbar_wait(&ctl->kv_empty[stage], (round - 1) & 1, abort_word, MB_ERR_TIMEOUT_KV_EMPTY)) {
              ok = false;
              break;
            }
            const CUtensorMap* map = which ? &maps.v[s] : &maps.k[s];
            uint8_t* dst = sKV + stage * kTileBytes;
            mbar_expect_tx(&ctl->kv_full[stage], kTileBytes);
            tma_load_4d(dst, map, &ctl->kv_full[stage], 0, hkv, jt * kBN, b);
            tma_load_4d(dst + kHalfBytes, map, &ctl->kv_full[stage], 64, hkv, jt * kBN, b);
            ++n;
          }
        }
      }
      if (!ok) {
        // Give copies already in flight a bounded chance to land before the CTA exits.
        const int first = n > kFwdStages ? n - kFwdStages : 0;
        for (int m = first; m < n; ++m) {
          const long long t0 = clock64();
          while (!mbar_try_wait(&ctl->kv_full[m % kFwdStages], (m / kFwdStages) & 1) &&
                 clock64() - t0 < kWaitCycleLimit / 16) {
          }
        }
      }
    }
  } else if (warp == 8 || warp == 10) {
    // ------------------------------------------- MMA issuers: warp 8 -> query tile 0, warp 10 -> tile 1
    // Each walks every K/V stage in load order (K0 V0 K1 V1 ...): it waits for the stage, uses it if
    // its query tile takes part in that K/V tile, and arrives on the stage's "empty" barrier either
    // way, so the barrier always sees one arrival per issuing warp.
    asm volatile("setmaxnreg.dec.sync.aligned.u32 48;");
    if (any_work) {  // whole warp, converged
      const int i = (warp - 8) >> 1;
      constexpr uint32_t idesc_qk = umma_idesc_bf16(kBM, kBN, false, false);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(kBM, kD, false, true);
      const uint32_t tSi = tmem + i * 128, tOi = tmem + 256 + i * 128;
      const uint64_t q_desc = umma_smem_desc(smem_u32(sQ) + i * kTileBytes, 16, 1024);
      const uint64_t k_desc0 = umma_smem_desc(smem_u32(sKV), 16, 1024);          // K-major view of stage 0
      const uint64_t v_desc0 = umma_smem_desc(smem_u32(sKV), kHalfBytes, 1024);  // MN-major view of stage 0
      constexpr uint32_t kStageUnits = kTileBytes / 16;
      uint64_t* p_full0 = &ctl->p_full[i][0];
      uint64_t* p_full1 = &ctl->p_full[i][1];
      int cnt = 0;   // tiles this query tile has taken part in
      int n = 0;     // next stage index in load order
      bool ok = mbar_wait_warp(&ctl->q_full, 0, abort_word, MB_ERR_TIMEOUT_Q);
      bool first = true;
      for (int s = 0; s < a.nseg && ok; ++s) {
        const int mine = ctl->n_tiles[i][s];
        const int nmax = max(ctl->n_tiles[0][s], ctl->n_tiles[1][s]);
        for (int jt = 0; jt < nmax; ++jt) {
          const bool part = jt < mine;
          // ---- K tile of this iteration
          {
            const int stage = n % kFwdStages;
            ok = mbar_wait_warp(&ctl->kv_full[stage], (n / kFwdStages) & 1, abort_word, MB_ERR_TIMEOUT_KV_FULL);
            if (!ok) break;
            if (part) {
              tc_fence_after();
              issue_qk(tSi, q_desc, k_desc0 + stage * kStageUnits, idesc_qk);
              umma_commit_elect(&ctl->s_full[i]);
              umma_commit_elect(&ctl->kv_empty[stage]);
              MB_TRACE_AT(2, cnt, i * 6 + 5);
            } else {
              mbar_arrive_elect(&ctl->kv_empty[stage]);
            }
            ++n;
          }
          // ---- V tile of this iteration
          {
            const int stage = n % kFwdStages;
            ok = mbar_wait_warp(&ctl->kv_full[stage], (n / kFwdStages) & 1, abort_word, MB_ERR_TIMEOUT_KV_FULL);
            if (!ok) break;
            if (part) {
              const uint64_t v_desc = v_desc0 + stage * kStageUnits;
              MB_TRACE_AT(2, cnt, i * 6 + 0);
              ok = mbar_wait_warp(p_full0, cnt & 1, abort_word, MB_ERR_TIMEOUT_P);
              if (!ok) break;
              MB_TRACE_AT(2, cnt, i * 6 + 1);
              tc_fence_after();
              issue_pv_half(tOi, tSi, v_desc, idesc_pv, first ? 0u : 1u);
              MB_TRACE_AT(2, cnt, i * 6 + 2);
              ok = mbar_wait_warp(p_full1, cnt & 1, abort_word, MB_ERR_TIMEOUT_P);
              if (!ok) break;
              MB_TRACE_AT(2, cnt, i * 6 + 3);
              tc_fence_after();
              issue_pv_half(tOi, tSi + 32, v_desc + 4 * 128, idesc_pv, 1u);
              umma_commit_elect(&ctl->o_full[i]);
              umma_commit_elect(&ctl->kv_empty[stage]);
              MB_TRACE_AT(2, cnt, i * 6 + 4);
              first = false;
              ++cnt;
            } else {
              mbar_arrive_elect(&ctl->kv_empty[stage]);
            }
            ++n;
          }
        }
      }
      if (!ok) {
        // Let tensor-core work already issued finish (bounded) before tensor memory is released.
        umma_commit_elect(&ctl->drain);
        const long long t0 = clock64();
        while (!mbar_try_wait(&ctl->drain, 0) && clock64() - t0 < kWaitCycleLimit / 16) {
        }
        __syncwarp();
      }
    }
  } else {
    // ------------------------------------------------------ softmax + epilogue
    asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
    // All control flow below is warp-uniform (the tensor-memory loads and
    // stores are warp-collective); only global stores are predicated per row.
    const int i = warp >> 2;                    // query tile
    const int row = ((warp & 3) << 5) | lane;   // row inside the tile == tensor-memory lane
    const uint32_t lane_field = static_cast<uint32_t>((warp & 3) << 5) << 16;
    const uint32_t tSi = tmem + i * 128 + lane_field;
    const uint32_t tOi = tmem + 256 + i * 128 + lane_field;
    const int qrow = q0 + i * kBM + row;        // row inside this rank's Q
    const int qpos = a.q_off + qrow;            // global position used by the causal rule

    float m_ref = -INFINITY;  // reference max (raw score units)
    float l = 0.f;            // running sum of exp2
    int cnt = 0;
    int shared_cnt = 0;       // K/V tiles both query tiles took part in so far
    bool ok = true;

    for (int s = 0; s < a.nseg && ok; ++s) {
      const int nt = ctl->n_tiles[i][s];
      const int nt_both = min(ctl->n_tiles[0][s], ctl->n_tiles[1][s]);
      const int sk = a.seg_sk[s];
      const int koff = a.seg_koff[s];
      for (int jt = 0; jt < nt; ++jt) {
        if (row == 0) MB_TRACE_AT(i, cnt, 0);
        ok = mbar_wait_warp(&ctl->s_full[i], cnt & 1, abort_word, MB_ERR_TIMEOUT_S);
        if (!ok) break;
        if (row == 0) MB_TRACE_AT(i, cnt, 1);
        tc_fence_after();
        uint32_t sr[4][32];
        tmem_ld32(tSi + 0, sr[0]);
        tmem_ld32(tSi + 32, sr[1]);
        tmem_ld32(tSi + 64, sr[2]);
        tmem_ld32(tSi + 96, sr[3]);
        tmem_wait_ld();
        if (row == 0) MB_TRACE_AT(i, cnt, 2);

        // masking: only tiles that cross the segment end or the causal diagonal
        const int k0 = jt * kBN;
        const bool tile_needs_mask =
            (k0 + kBN > sk) || (a.causal && (koff + k0 + kBN - 1 > a.q_off + q0 + i * kBM));
        if (tile_needs_mask) {
          int limit = sk - k0;  // columns >= limit are invisible
          if (a.causal) limit = min(limit, qpos - koff - k0 + 1);
#pragma unroll
          for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int e = 0; e < 32; ++e)
              if (c * 32 + e >= limit) sr[c][e] = 0xff800000u;  // -inf
        }

        float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          mx0 = max3(mx0, __uint_as_float(sr[0][e]), __uint_as_float(sr[0][e + 1]));
          mx1 = max3(mx1, __uint_as_float(sr[1][e]), __uint_as_float(sr[1][e + 1]));
          mx2 = max3(mx2, __uint_as_float(sr[2][e]), __uint_as_float(sr[2][e + 1]));
          mx3 = max3(mx3, __uint_as_float(sr[3][e]), __uint_as_float(sr[3][e + 1]));
        }
        const float m_tile = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
        if (row == 0) MB_TRACE_AT(i, cnt, 3);

        if (cnt == 0) {
          m_ref = m_tile;
        } else {
          const float m_new = fmaxf(m_ref, m_tile);
          const bool need = (m_new - m_ref) * a.scale_log2 > kRescaleThreshold;
          if (__any_sync(0xffffffffu, need)) {
            // O of the previous step must be complete before it is rescaled.
            ok = mbar_wait_warp(&ctl->o_full[i], (cnt - 1) & 1, abort_word, MB_ERR_TIMEOUT_O);
            if (!ok) break;
            tc_fence_after();
            const float f = need ? fast_exp2((m_ref - m_new) * a.scale_log2) : 1.f;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              uint32_t orow[32];
              tmem_ld32(tOi + c * 32, orow);
              tmem_wait_ld();
#pragma unroll
              for (int e = 0; e < 32; ++e) orow[e] = __float_as_uint(__uint_as_float(orow[e]) * f);
              tmem_st32(tOi + c * 32, orow);
            }
            tmem_wait_st();
            if (need) {
              l *= f;
              m_ref = m_new;
            }
          }
        }

        // The two warpgroups take turns in the exp2 phase: the 16-lane MUFU is the scarce unit, and
        // if both tiles reach this phase together they share it, finish together and then leave it
        // idle while both wait for the tensor pipe.  Alternating keeps one tile in its MUFU phase
        // while the other tile's MMAs run.  Only K/V tiles that both query tiles process take part,
        // so the two warpgroups always agree on the turn count.
        const bool take_turns = kTakeTurns && jt < nt_both;
        if (take_turns) {
          ok = mbar_wait_warp(&ctl->turn[i], (shared_cnt & 1) ^ (i == 0 ? 1 : 0), abort_word, MB_ERR_TIMEOUT_MISC);
          if (!ok) break;
        }

        // p = exp2(s * c - m * c): the scale/subtract and the row sum run as packed pairs; every
        // kPolyEvery-th pair of exponentials is evaluated on the FMA pipe, the rest on the MUFU.
        const float m_scaled = (m_ref == -INFINITY) ? 0.f : m_ref * a.scale_log2;
        const uint64_t c2 = pack2(a.scale_log2, a.scale_log2);
        const uint64_t nm2 = pack2(-m_scaled, -m_scaled);
        uint64_t sum_a = pack2(0.f, 0.f), sum_b = pack2(0.f, 0.f);
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t pk[32];
#pragma unroll
          for (int cc = 0; cc < 2; ++cc) {
            const int c = half * 2 + cc;
#pragma unroll
            for (int e = 0; e < 32; e += 2) {
              const uint64_t x2 = fma2(pack2(__uint_as_float(sr[c][e]), __uint_as_float(sr[c][e + 1])), c2, nm2);
              uint64_t p2;
              if (kPolyEvery > 0 && ((e >> 1) % (kPolyEvery > 0 ? kPolyEvery : 1)) == kPolyEvery - 1) {
                p2 = exp2_poly2(x2);
              } else {
                float x0, x1;
                unpack2(x2, x0, x1);
                p2 = pack2(fast_exp2(x0), fast_exp2(x1));
              }
              if ((e >> 1) & 1) sum_b = add2(sum_b, p2);
              else sum_a = add2(sum_a, p2);
              float p0, p1;
              unpack2(p2, p0, p1);
              pk[cc * 16 + (e >> 1)] = pack_bf16x2(p0, p1);
            }
          }
          if (half == 1 && take_turns) {
            mbar_arrive(&ctl->turn[i ^ 1]);  // my exponentials are issued: the other warpgroup's turn
            ++shared_cnt;
          }
          tmem_st32(tSi + half * 32, pk);
          tmem_wait_st();
          tc_fence_before();
          mbar_arrive(&ctl->p_full[i][half]);
          if (row == 0) MB_TRACE_AT(i, cnt, 4 + half);
        }
        {
          float s0, s1;
          unpack2(add2(sum_a, sum_b), s0, s1);
          l += s0 + s1;
        }
        ++cnt;
      }
    }

    // epilogue: O / l -> bf16, LSE = ln(sum exp(scale * s)).  Tiles whose rows all lie past Sq skip it.
    if (ok && q0 + i * kBM < a.Sq) {
      bool have = cnt > 0;
      if (have) {
        have = mbar_wait_warp(&ctl->o_full[i], (cnt - 1) & 1, abort_word, MB_ERR_TIMEOUT_O);
        ok = have;
      }
      if (ok) {
        const bool store = qrow < a.Sq;
        const float inv_l = (have && l > 0.f) ? 1.f / l : 0.f;
        __nv_bfloat16* optr = a.o + (long long)b * a.o_sb + (long long)qrow * a.o_ss + (long long)h * a.o_sh;
        if (have) tc_fence_after();
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t orow[32];
          if (have) {
            tmem_ld32(tOi + c * 32, orow);
            tmem_wait_ld();
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) orow[e] = 0u;
          }
          if (store) {
            uint4* dst = reinterpret_cast<uint4*>(optr + c * 32);
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint4 w;
              w.x = pack_bf16x2(__uint_as_float(orow[v * 8 + 0]) * inv_l, __uint_as_float(orow[v * 8 + 1]) * inv_l);
              w.y = pack_bf16x2(__uint_as_float(orow[v * 8 + 2]) * inv_l, __uint_as_float(orow[v * 8 + 3]) * inv_l);
              w.z = pack_bf16x2(__uint_as_float(orow[v * 8 + 4]) * inv_l, __uint_as_float(orow[v * 8 + 5]) * inv_l);
              w.w = pack_bf16x2(__uint_as_float(orow[v * 8 + 6]) * inv_l, __uint_as_float(orow[v * 8 + 7]) * inv_l);
              dst[v] = w;
            }
          }
        }
        if (store) {
          const float lse = (have && l > 0.f) ? (m_ref * a.scale + __logf(l)) : -INFINITY;
          a.lse[(long long)b * a.lse_sb + (long long)h * a.lse_sh + qrow] = lse;
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 8) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
  if (tid == 0 && ctl->abort_word != 0 && a.status != nullptr) atomicCAS(a.status, 0, ctl->abort_word);
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
static int make_tile_map(CUtensorMap* map, const void* ptr, int D, int H, int S, int B, long long sb, long long ss,
                         long long sh) {
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)H, (cuuint64_t)S, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)sh * 2, (cuuint64_t)ss * 2, (cuuint64_t)sb * 2};
  cuuint32_t box[4] = {64, 1, (cuuint32_t)kBN, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  return encode_tiled_bf16(map, const_cast<void*>(ptr), 4, dims, strides, box, estr);
}

int launch_attn_fwd(const mb_attn_fwd_args* x, cudaStream_t stream) {
  if (x == nullptr) return MB_E_INVALID;
  if (x->head_dim != kD) return MB_E_UNSUPPORTED;
  if (x->batch <= 0 || x->hq <= 0 || x->hkv <= 0 || x->hq % x->hkv != 0) return MB_E_INVALID;
  if (x->nseg < 0 || x->nseg > MB_MAX_SEGMENTS) return MB_E_INVALID;
  if (x->sq < 0) return MB_E_INVALID;
  if (x->sq == 0) return MB_SUCCESS;
  if (x->q == nullptr || x->o == nullptr || x->lse == nullptr) return MB_E_INVALID;

  static bool attr_set[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return MB_E_CUDA;
  if (dev < 64 && !attr_set[dev]) {
    if (cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kFwdSmemBytes) !=
        cudaSuccess)
      return MB_E_CUDA;
    attr_set[dev] = true;
  }

  FwdMaps maps;
  FwdArgs a;
  memset(&maps, 0, sizeof(maps));
  memset(&a, 0, sizeof(a));
  if (make_tile_map(&maps.q, x->q, kD, x->hq, x->sq, x->batch, x->q_stride_b, x->q_stride_s, x->q_stride_h))
    return MB_E_TENSORMAP;
  int nseg = 0;
  for (int s = 0; s < x->nseg; ++s) {
    const mb_kv_segment& g = x->seg[s];
    if (g.sk < 0) return MB_E_INVALID;
    if (g.sk == 0) continue;  // an empty shard contributes nothing
    if (g.k == nullptr || g.v == nullptr) return MB_E_INVALID;
    if (make_tile_map(&maps.k[nseg], g.k, kD, x->hkv, g.sk, x->batch, g.stride_b, g.stride_s, g.stride_h))
      return MB_E_TENSORMAP;
    if (make_tile_map(&maps.v[nseg], g.v, kD, x->hkv, g.sk, x->batch, g.stride_b, g.stride_s, g.stride_h))
      return MB_E_TENSORMAP;
    a.seg_sk[nseg] = g.sk;
    a.seg_koff[nseg] = g.k_off;
    a.seg_flag[nseg] = g.ready_flag;
    a.seg_flag_value[nseg] = g.ready_value;
    ++nseg;
  }
  a.nseg = nseg;
  a.o = reinterpret_cast<__nv_bfloat16*>(x->o);
  a.o_sb = x->o_stride_b;
  a.o_ss = x->o_stride_s;
  a.o_sh = x->o_stride_h;
  a.lse = x->lse;
  a.lse_sh = x->lse_stride_h ? x->lse_stride_h : x->sq;
  a.lse_sb = x->lse_stride_b ? x->lse_stride_b : (long long)x->hq * x->sq;
  a.B = x->batch;
  a.Sq = x->sq;
  a.Hq = x->hq;
  a.group = x->hq / x->hkv;
  a.q_off = x->q_off;
  a.causal = x->causal ? 1 : 0;
  a.scale = x->softmax_scale;
  a.scale_log2 = x->softmax_scale * 1.4426950408889634f;
  a.status = x->status ? x->status : default_status_word();
  if (a.status == nullptr) return MB_E_CUDA;

  dim3 grid((x->sq + 2 * kBM - 1) / (2 * kBM), x->hq, x->batch);
  attn_fwd_kernel<<<grid, kFwdThreads, kFwdSmemBytes, stream>>>(maps, a);
  return cudaGetLastError() == cudaSuccess ? MB_SUCCESS : MB_E_CUDA;
}

}  // namespace mb

#ifdef MB_TRACE
extern "C" __attribute__((visibility("default"))) int mb_debug_fetch_fwd_trace(long long* host_out) {
  return cudaMemcpyFromSymbol(host_out, mb::g_fwd_trace, sizeof(mb::g_fwd_trace)) == cudaSuccess ? 0 : -3;
}
#endif
