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
//   warp  8    tcgen05.mma issuer for the Q.K^T products of both query tiles, tensor-memory owner
//   warp  9    TMA loader (lane 0)
//   warp 10    tcgen05.mma issuer for the P.V products of both query tiles
//   warp 11    idle; the auxiliary warpgroup's registers go to the softmax warps (setmaxnreg)
//
// Tensor memory (512 columns): S | P0 | P1 | O0 | O1 = 128 + 64 + 64 + 128 + 128.  There is ONE
// fp32 score region, used by the two query tiles in turn: a softmax thread copies its whole score
// row into registers as soon as the tile is complete and hands the region on, so the next Q.K^T
// product (of the other query tile) starts while this tile is still in its exponentials.  The bf16
// probabilities have a region of their own per query tile, so that the next score tile of a query
// tile does not have to wait for its P.V product either.  What remains serial is the hand-over of
// the score region: copy-out -> issuing warp wakes -> 8 MMAs -> tensor-pipe latency -> softmax warp
// wakes, about 1 100-1 300 cycles per use, two uses per K/V tile.
//
// K/V tiles are loaded in the order K0 K1 V0 K2 V1 K3 V2 ...: the score product of K/V tile g+1 is
// issued before the P.V product of tile g needs its V tile.
//
// A launch may carry several "jobs": query shards with their own output pointers, sharing the segment
// list.  blockIdx.x runs through the query-tile pairs of job 0, then of job 1, ...  A job can name an
// arrival flag for its queries (they may still be in flight from another GPU) and a completion flag,
// which the job's last CTA raises with a release store at system scope once every row of the job has
// been stored -- the rows, and the flag, may live in another GPU's memory.
#include <climits>

#include "attn_fwd_common.cuh"

namespace mb {

// Position in the CTA's list of K/V tiles: every tile of every segment that at least one of the two
// query tiles takes part in, in segment order.
struct TileIter {
  int s, jt;
};
__device__ __forceinline__ int seg_tiles(const FwdSmem* ctl, int s) {
  return max(ctl->n_tiles[0][s], ctl->n_tiles[1][s]);
}
__device__ __forceinline__ TileIter iter_first(const FwdSmem* ctl, int nseg) {
  TileIter it{0, 0};
  while (it.s < nseg && seg_tiles(ctl, it.s) == 0) ++it.s;
  return it;
}
__device__ __forceinline__ void iter_next(const FwdSmem* ctl, int nseg, TileIter& it) {
  if (++it.jt >= seg_tiles(ctl, it.s)) {
    it.jt = 0;
    ++it.s;
    while (it.s < nseg && seg_tiles(ctl, it.s) == 0) ++it.s;
  }
}

// Register budgets.  setmaxnreg can only redistribute the registers the CTA was launched with
// (threads x launch budget); an increase beyond that pool would block forever, hence the check.
#define MB_FWD_LAUNCH_REGS 160
#define MB_FWD_SOFTMAX_REGS 216
#define MB_FWD_AUX_REGS 48
#define MB_STR2(x) #x
#define MB_STR(x) MB_STR2(x)
static_assert(8 * 32 * MB_FWD_SOFTMAX_REGS + 4 * 32 * MB_FWD_AUX_REGS <= kFwdThreads * MB_FWD_LAUNCH_REGS,
              "setmaxnreg budgets exceed the registers the CTA is launched with");

// 160 registers/thread at launch (not the 168 that 384 threads would allow): the few warps' worth
// left free on the SM let the transfer stream's one-thread flag kernels start beside a resident CTA.
__global__ void __maxnreg__(MB_FWD_LAUNCH_REGS)
attn_fwd_kernel(const __grid_constant__ FwdMaps maps, const __grid_constant__ FwdArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sKV = smem + 2 * kTileBytes;
  FwdSmem* ctl = reinterpret_cast<FwdSmem*>(smem + 2 * kTileBytes + kFwdStages * kTileBytes);
  volatile int* abort_word = &ctl->abort_word;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  // Which job this CTA belongs to; within a job the heavier (later) query rows come first when causal.
  if (tid == 0) {
    int jid = 0;
    while (jid + 1 < a.njobs && (int)blockIdx.x >= a.job[jid + 1].x_begin) ++jid;
    ctl->jid = jid;
    ctl->job = a.job[jid];
    // CTAs are dispatched in grid order: job by job, inside a job batch entry by batch entry and head by
    // head (the CTAs running at one time share a few heads' K/V through L2), heavier query rows first.
    const int local = (int)blockIdx.x - a.job[jid].x_begin;
    const int np = a.job[jid].n_pairs;
    const int pidx = local % np;
    ctl->pair = a.causal ? (np - 1 - pidx) : pidx;
    ctl->h = (local / np) % a.Hq;
    ctl->b = (local / np) / a.Hq;
  }
  __syncthreads();
  const FwdJob& J = ctl->job;
  // (pair, head, batch entry) stay in shared memory: the roles read them where they need them, so that
  // they occupy no registers across the softmax loop
  const int q0 = ctl->pair * 2 * kBM;

  if (tid == 0) {
    mbar_init(&ctl->q_full, 1);
    for (int s = 0; s < kFwdStages; ++s) {
      mbar_init(&ctl->kv_full[s], 1);
      mbar_init(&ctl->kv_empty[s], 1);  // released by the one warp that consumes the stage
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&ctl->s_full[i], 1);
      mbar_init(&ctl->p_full[i][0], 128);
      mbar_init(&ctl->p_full[i][1], 128);
      mbar_init(&ctl->o_full[i], 1);
    }
    mbar_init(&ctl->s_free, 4);
    mbar_init(&ctl->drain, 2);
    ctl->abort_word = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  // K/V tiles of each segment that each of the two query tiles takes part in: one thread per entry
  // (computed by one thread this was ~4 000 cycles of a CTA's prologue at 32 segments)
  if (tid < 2 * MB_MAX_SEGMENTS) {
    const int i = tid / MB_MAX_SEGMENTS, s = tid % MB_MAX_SEGMENTS;
    ctl->n_tiles[i][s] = (s < a.nseg && ((J.seg_mask >> s) & 1u))
                             ? visible_tiles(q0 + i * kBM, J.Sq, J.q_off, a.causal, a.seg_sk[s], a.seg_koff[s])
                             : 0;
  }
  if (warp == 8) {
    tmem_alloc(&ctl->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  const uint32_t tmem = ctl->tmem_base;  // columns: S [0,128) P0 [128,192) P1 [192,256) O0 [256,384) O1 [384,512)

  bool any_work = false;
  for (int s = 0; s < a.nseg; ++s) any_work |= (ctl->n_tiles[0][s] | ctl->n_tiles[1][s]) != 0;

  // Registers move from the auxiliary warpgroup (warps 8-11) to the two softmax
  // warpgroups; each role changes its own budget as the first thing it does.
  if (warp == 11) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 " MB_STR(MB_FWD_AUX_REGS) ";");
  } else if (warp == 9) {
    // ------------------------------------------------------------------ loader
    asm volatile("setmaxnreg.dec.sync.aligned.u32 " MB_STR(MB_FWD_AUX_REGS) ";");
    if (lane == 0 && any_work) {
      bool ok = true;
      const CUtensorMap* qmap = &maps.q[J.qmap];
      tma_prefetch_desc(qmap);
      if (J.q_flag != nullptr) {
        // The queries are being staged from another GPU: wait (bounded) for their arrival flag.  On a
        // timeout the Q load is skipped; every other role then runs into the abort word and returns.
        ok = flag_wait_ge(J.q_flag, J.q_flag_value, abort_word, MB_ERR_TIMEOUT_SEGMENT, a.peer_wait_cycles);
        asm volatile("fence.proxy.async;" ::: "memory");
      }
      if (ok) {
        const int act0 = q0 < J.Sq, act1 = q0 + kBM < J.Sq;
        mbar_expect_tx(&ctl->q_full, (act0 + act1) * kTileBytes);
        for (int i = 0; i < 2; ++i) {
          if (q0 + i * kBM < J.Sq) {
            tma_load_4d(sQ + i * kTileBytes, qmap, &ctl->q_full, 0, ctl->h, q0 + i * kBM, ctl->b);
            tma_load_4d(sQ + i * kTileBytes + kHalfBytes, qmap, &ctl->q_full, 64, ctl->h, q0 + i * kBM, ctl->b);
          }
        }
      }
      int n = 0;
      const int b_ = ctl->b, hkv = ctl->h / a.group;
      // One K or V tile into the next stage of the ring.
      auto load_tile = [&](int which, const TileIter& it) {
        if (which == 0 && it.jt == 0 && a.seg_flag[it.s] != nullptr) {
          // The shard is being staged by another stream: wait (bounded) for its arrival flag,
          // then order the TMA reads (async proxy) after the flag read.
          ok = flag_wait_ge(a.seg_flag[it.s], a.seg_flag_value[it.s], abort_word, MB_ERR_TIMEOUT_SEGMENT,
                            a.peer_wait_cycles);
          asm volatile("fence.proxy.async;" ::: "memory");
          if (!ok) return;
        }
        const int stage = n % kFwdStages;
        const int round = n / kFwdStages;
        if (round > 0 && !mbar_wait(&ctl->kv_empty[stage], (round - 1) & 1, abort_word, MB_ERR_TIMEOUT_KV_EMPTY, a.wait_cycles)) {
          ok = false;
          return;
        }
        const CUtensorMap* map = which ? &maps.v[it.s] : &maps.k[it.s];
        uint8_t* dst = sKV + stage * kTileBytes;
        mbar_expect_tx(&ctl->kv_full[stage], kTileBytes);
        tma_load_4d(dst, map, &ctl->kv_full[stage], 0, hkv, it.jt * kBN, b_);
        tma_load_4d(dst + kHalfBytes, map, &ctl->kv_full[stage], 64, hkv, it.jt * kBN, b_);
        ++n;
      };
      TileIter nxt = iter_first(ctl, a.nseg);
      TileIter cur = nxt;
      if (ok && nxt.s < a.nseg) {
        load_tile(0, nxt);
        iter_next(ctl, a.nseg, nxt);
      }
      while (ok && cur.s < a.nseg) {
        if (nxt.s < a.nseg) load_tile(0, nxt);
        if (ok) load_tile(1, cur);
        cur = nxt;
        if (nxt.s < a.nseg) iter_next(ctl, a.nseg, nxt);
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
    // ------------------------------------------- MMA issuers: warp 8 issues every Q.K^T product,
    // warp 10 every P.V product, of both query tiles.  (One warp per query tile issuing both kinds
    // held its P.V products back while it sat in the issue of its next score product, and the
    // products of the two tiles then fell into the same stretch of time, with the tensor pipe idle
    // in between.)  Positions in the ring of K/V stages follow the load order K0 K1 V0 K2 V1 ...
    asm volatile("setmaxnreg.dec.sync.aligned.u32 " MB_STR(MB_FWD_AUX_REGS) ";");
    if (any_work) {  // whole warp, converged
      constexpr uint32_t kStageUnits = kTileBytes / 16;
      int total = 0;  // K/V tiles this CTA walks through
      for (int s = 0; s < a.nseg; ++s) total += seg_tiles(ctl, s);
      bool ok = true;
      if (warp == 8) {
        constexpr uint32_t idesc_qk = umma_idesc_bf16(kBM, kBN, false, false);
        const uint64_t q_desc = umma_smem_desc(smem_u32(sQ), 16, 1024);
        const uint64_t k_desc0 = umma_smem_desc(smem_u32(sKV), 16, 1024);  // K-major view of stage 0
        int g = 0;    // K/V tile index over all segments
        int use = 0;  // uses of the score region so far, by either query tile
        ok = mbar_wait_warp(&ctl->q_full, 0, abort_word, MB_ERR_TIMEOUT_Q, a.wait_cycles);
        for (int s = 0; s < a.nseg && ok; ++s) {
          const int n0 = ctl->n_tiles[0][s], n1 = ctl->n_tiles[1][s];
          const int nmax = max(n0, n1);
          for (int jt = 0; jt < nmax && ok; ++jt, ++g) {
            const int pos = g == 0 ? 0 : 2 * g - 1;
            const int stage = pos % kFwdStages;
            ok = mbar_wait_warp(&ctl->kv_full[stage], (pos / kFwdStages) & 1, abort_word, MB_ERR_TIMEOUT_KV_FULL, a.wait_cycles);
            if (!ok) break;
#pragma unroll
            for (int i = 0; i < 2; ++i) {
              if (jt < (i ? n1 : n0)) {
                // the score region's previous user must have copied its scores out
                if (use > 0) {
                  ok = mbar_wait_warp(&ctl->s_free, (use - 1) & 1, abort_word, MB_ERR_TIMEOUT_S, a.wait_cycles);
                  if (!ok) break;
                }
                tc_fence_after();
                issue_qk(tmem, q_desc + i * kStageUnits, k_desc0 + stage * kStageUnits, idesc_qk);
                umma_commit_elect(&ctl->s_full[i]);
                ++use;
              }
            }
            if (!ok) break;
            umma_commit_elect(&ctl->kv_empty[stage]);
          }
        }
      } else {
        constexpr uint32_t idesc_pv = umma_idesc_bf16(kBM, kD, false, true);
        const uint64_t v_desc0 = umma_smem_desc(smem_u32(sKV), kHalfBytes, 1024);  // MN-major view of stage 0
        int g = 0;
        int cnt0 = 0, cnt1 = 0;  // P.V products issued per query tile
        for (int s = 0; s < a.nseg && ok; ++s) {
          const int n0 = ctl->n_tiles[0][s], n1 = ctl->n_tiles[1][s];
          const int nmax = max(n0, n1);
          for (int jt = 0; jt < nmax && ok; ++jt, ++g) {
            const int pos = g == total - 1 ? 2 * total - 1 : 2 * g + 2;
            const int stage = pos % kFwdStages;
            ok = mbar_wait_warp(&ctl->kv_full[stage], (pos / kFwdStages) & 1, abort_word, MB_ERR_TIMEOUT_KV_FULL, a.wait_cycles);
            if (!ok) break;
            const uint64_t v_desc = v_desc0 + stage * kStageUnits;
#pragma unroll
            for (int i = 0; i < 2; ++i) {
              if (jt < (i ? n1 : n0)) {
                const int cnt = i ? cnt1 : cnt0;
                const uint32_t tPi = tmem + 128 + i * 64, tOi = tmem + 256 + i * 128;
                ok = mbar_wait_warp(&ctl->p_full[i][0], cnt & 1, abort_word, MB_ERR_TIMEOUT_P, a.wait_cycles);
                if (!ok) break;
                tc_fence_after();
                issue_pv_half(tOi, tPi, v_desc, idesc_pv, (cnt == 0 && !J.st_in) ? 0u : 1u);
                ok = mbar_wait_warp(&ctl->p_full[i][1], cnt & 1, abort_word, MB_ERR_TIMEOUT_P, a.wait_cycles);
                if (!ok) break;
                tc_fence_after();
                issue_pv_half(tOi, tPi + 32, v_desc + 4 * 128, idesc_pv, 1u);
                umma_commit_elect(&ctl->o_full[i]);
                if (i) ++cnt1;
                else ++cnt0;
              }
            }
            if (!ok) break;
            umma_commit_elect(&ctl->kv_empty[stage]);
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
    asm volatile("setmaxnreg.inc.sync.aligned.u32 " MB_STR(MB_FWD_SOFTMAX_REGS) ";");
    // All control flow below is warp-uniform (the tensor-memory loads and
    // stores are warp-collective); only global stores are predicated per row.
    const int i = warp >> 2;                    // query tile
    const int row = ((warp & 3) << 5) | lane;   // row inside the tile == tensor-memory lane
    const uint32_t lane_field = static_cast<uint32_t>((warp & 3) << 5) << 16;
    const uint32_t tS = tmem + lane_field;
    const uint32_t tPi = tmem + 128 + i * 64 + lane_field;
    const uint32_t tOi = tmem + 256 + i * 128 + lane_field;
    // global position used by the causal rule; the row inside the job's Q is qpos - J.q_off
    const int qpos = J.q_off + q0 + i * kBM + row;

    float m_ref = -INFINITY;  // reference max (raw score units)
    float l = 0.f;            // running sum of exp2
    int cnt = 0;
    bool ok = true;
    if (J.st_in && q0 + i * kBM < J.Sq) {
      const int qrow = qpos - J.q_off;  // row inside the job's Q
      const long long st_row = ((long long)ctl->b * a.Hq + ctl->h) * J.Sq + qrow;
      // Continue where an earlier job stopped: its unnormalised rows go back into tensor memory, its
      // maximum and sum into registers.  With chain words that job may be part of this launch (a CTA
      // with a lower index); its release store is acquired here.
      if (J.chain != nullptr) {
        if (lane == 0)
          ok = flag_wait_ge(J.chain + ((long long)ctl->b * a.Hq + ctl->h) * J.n_pairs + ctl->pair, J.chain_wait, abort_word,
                            MB_ERR_TIMEOUT_SEGMENT, a.peer_wait_cycles);
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      }
      if (ok) {
        const bool valid = qrow < J.Sq;
        const float4* src = reinterpret_cast<const float4*>(J.st_o + st_row * kD);
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t orow[32];
#pragma unroll
          for (int v = 0; v < 8; ++v) {
            const float4 w = valid ? src[c * 8 + v] : make_float4(0.f, 0.f, 0.f, 0.f);
            orow[v * 4 + 0] = __float_as_uint(w.x);
            orow[v * 4 + 1] = __float_as_uint(w.y);
            orow[v * 4 + 2] = __float_as_uint(w.z);
            orow[v * 4 + 3] = __float_as_uint(w.w);
          }
          tmem_st32(tOi + c * 32, orow);
        }
        tmem_wait_st();
        if (valid) {
          const float2 ml = *reinterpret_cast<const float2*>(J.st_ml + st_row * 2);
          m_ref = ml.x;
          l = ml.y;
        }
      }
    }

    for (int s = 0; s < a.nseg && ok; ++s) {
      const int nt = ctl->n_tiles[i][s];
      const int sk = a.seg_sk[s];
      const int koff = a.seg_koff[s];
      for (int jt = 0; jt < nt; ++jt) {
        ok = mbar_wait_warp(&ctl->s_full[i], cnt & 1, abort_word, MB_ERR_TIMEOUT_S, a.wait_cycles);
        if (!ok) break;
        tc_fence_after();
        uint32_t sr[4][32];
        tmem_ld32(tS + 0, sr[0]);
        tmem_ld32(tS + 32, sr[1]);
        tmem_ld32(tS + 64, sr[2]);
        tmem_ld32(tS + 96, sr[3]);
        tmem_wait_ld();
        // The scores are in registers: hand the score region to its next user.
        tc_fence_before();
        mbar_arrive_elect(&ctl->s_free);

        // masking: only tiles that cross the segment end or the causal diagonal
        const int k0 = jt * kBN;
        const bool tile_needs_mask =
            (k0 + kBN > sk) || (a.causal && (koff + k0 + kBN - 1 > qpos - row));  // qpos - row: the tile's first row
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

        if (cnt == 0 && __all_sync(0xffffffffu, m_ref == -INFINITY)) {
          m_ref = m_tile;  // nothing accumulated yet (a carried state of rows without keys is all zero)
        } else {
          // The previous P.V product of this query tile must be complete before its probabilities
          // are overwritten, and before O is rescaled (a carried state is already in place).
          if (cnt > 0) {
            ok = mbar_wait_warp(&ctl->o_full[i], (cnt - 1) & 1, abort_word, MB_ERR_TIMEOUT_O, a.wait_cycles);
            if (!ok) break;
            tc_fence_after();
          }
          const float m_new = fmaxf(m_ref, m_tile);
          const bool need = (m_new - m_ref) * a.scale_log2 > kRescaleThreshold;
          if (__any_sync(0xffffffffu, need)) {
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

        // p = exp2(s * c - m * c): the scale/subtract and the row sum run as packed pairs.  (Taking
        // turns between the two warpgroups in this MUFU-bound phase, and moving part of the
        // exponentials to a polynomial on the FMA pipe, were both measured as losses.)
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
              float x0, x1;
              unpack2(x2, x0, x1);
              const uint64_t p2 = pack2(fast_exp2(x0), fast_exp2(x1));
              if ((e >> 1) & 1) sum_b = add2(sum_b, p2);
              else sum_a = add2(sum_a, p2);
              float p0, p1;
              unpack2(p2, p0, p1);
              pk[cc * 16 + (e >> 1)] = pack_bf16x2(p0, p1);
            }
          }
          tmem_st32(tPi + half * 32, pk);
          tmem_wait_st();
          tc_fence_before();
          mbar_arrive(&ctl->p_full[i][half]);
        }
        {
          float s0, s1;
          unpack2(add2(sum_a, sum_b), s0, s1);
          l += s0 + s1;
        }
        ++cnt;
      }
    }

    // epilogue.  Final job: O / l -> bf16, LSE = ln(sum exp(scale * s)).  Job that hands its state on:
    // the unnormalised rows, the maximum and the sum, as they are.  Tiles whose rows all lie past Sq skip it.
    const int qrow = qpos - J.q_off;  // row inside the job's Q
    if (ok && qrow - row < J.Sq) {
      const long long st_row = ((long long)ctl->b * a.Hq + ctl->h) * J.Sq + qrow;
      const bool have_acc = cnt > 0 || J.st_in;   // tensor memory holds this tile's rows
      if (cnt > 0) ok = mbar_wait_warp(&ctl->o_full[i], (cnt - 1) & 1, abort_word, MB_ERR_TIMEOUT_O, a.wait_cycles);
      if (ok) {
        const bool store = qrow < J.Sq;
        if (have_acc) tc_fence_after();
        if (J.st_out) {
          float4* dst = reinterpret_cast<float4*>(J.st_o + st_row * kD);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t orow[32];
            if (have_acc) {
              tmem_ld32(tOi + c * 32, orow);
              tmem_wait_ld();
            } else {
#pragma unroll
              for (int e = 0; e < 32; ++e) orow[e] = 0u;
            }
            if (store) {
#pragma unroll
              for (int v = 0; v < 8; ++v)
                dst[c * 8 + v] = make_float4(__uint_as_float(orow[v * 4 + 0]), __uint_as_float(orow[v * 4 + 1]),
                                             __uint_as_float(orow[v * 4 + 2]), __uint_as_float(orow[v * 4 + 3]));
            }
          }
          if (store) *reinterpret_cast<float2*>(J.st_ml + st_row * 2) = make_float2(m_ref, l);
        } else {
          const float inv_l = (have_acc && l > 0.f) ? 1.f / l : 0.f;
          __nv_bfloat16* optr = J.o + (long long)ctl->b * J.o_sb + (long long)qrow * J.o_ss + (long long)ctl->h * J.o_sh;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t orow[32];
            if (have_acc) {
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
            const float lse = (have_acc && l > 0.f) ? (m_ref * a.scale + __logf(l)) : -INFINITY;
            J.lse[(long long)ctl->b * J.lse_sb + (long long)ctl->h * J.lse_sh + qrow] = lse;
          }
        }
      }
    }
    if (J.st_out && J.chain != nullptr) {
      // Publish the state to the job that continues it: every softmax thread's stores, then one release
      // store of the chain word.  (A CTA that gave up publishes too, so that nothing downstream waits out
      // its budget; the status word tells the host.)
      __threadfence();
      asm volatile("bar.sync 1, 256;" ::: "memory");
      if (warp == 0 && lane == 0)
        asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(J.chain + ((long long)ctl->b * a.Hq + ctl->h) * J.n_pairs + ctl->pair),
                     "r"(J.chain_set)
                     : "memory");
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 8) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
  if (tid == 0 && ctl->abort_word != 0 && a.status != nullptr) atomicCAS(a.status, 0, ctl->abort_word);
  if (tid == 0 && J.done_flag != nullptr) {
    // Every thread's result stores precede the barrier above; this fence makes them visible at system
    // scope (they may have gone to another GPU) before the arrival is counted.  The CTA that counts the
    // last arrival publishes the job: the flag's reader then sees every row of every CTA.  A CTA that
    // gave up still counts, so that the word returns to zero; the status word tells the host.
    __threadfence_system();
    int prev;
    asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(prev) : "l"(J.done_counter) : "memory");
    if (prev == J.n_ctas - 1) {
      *J.done_counter = 0;
      __threadfence_system();
      asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(J.done_flag), "r"(J.done_value) : "memory");
    }
  }
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

static long long g_peer_wait_ms = 30000;

void set_peer_wait_ms(unsigned ms) { g_peer_wait_ms = ms == 0 ? 1 : ms; }

// Cycle budget of waits for data other GPUs deliver: the SM clock never exceeds 2 GHz here, so
// 2e6 cycles per millisecond is at least the requested time.
long long peer_wait_cycles() { return g_peer_wait_ms * 2000000LL; }

int launch_attn_fwd_multi(const mb_attn_fwd_multi_args* x, cudaStream_t stream) {
  if (x == nullptr) return MB_E_INVALID;
  if (x->head_dim != kD) return MB_E_UNSUPPORTED;
  if (x->batch <= 0 || x->hq <= 0 || x->hkv <= 0 || x->hq % x->hkv != 0) return MB_E_INVALID;
  if (x->nseg < 0 || x->nseg > MB_MAX_SEGMENTS) return MB_E_INVALID;
  if (x->njobs < 1 || x->njobs > MB_MAX_JOBS) return MB_E_INVALID;

  static bool attr_set[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return MB_E_CUDA;
  if (dev < 64 && !attr_set[dev]) {
    if (cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kFwdSmemBytes) !=
        cudaSuccess)
      return MB_E_CUDA;
    attr_set[dev] = true;
  }

  // Kernel parameters (8.7 KB of tensor maps + 1.3 KB of scalars) are assembled in static storage:
  // the launch copies them, and launches of one process are issued from one thread at a time per device.
  static thread_local FwdMaps maps;
  static thread_local FwdArgs a;
  memset(&a, 0, sizeof(a));
  // empty segments are dropped; a job's segment mask is re-indexed accordingly
  int seg_new[MB_MAX_SEGMENTS];
  int nseg = 0;
  for (int s = 0; s < x->nseg; ++s) {
    const mb_kv_segment& g = x->seg[s];
    seg_new[s] = -1;
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
    seg_new[s] = nseg++;
  }
  a.nseg = nseg;
  int njobs = 0, x_total = 0, nqmaps = 0;
  const mb_fwd_job* qmap_of[kMaxQMaps];
  for (int j = 0; j < x->njobs; ++j) {
    const mb_fwd_job& g = x->job[j];
    if (g.sq < 0) return MB_E_INVALID;
    if (g.sq == 0) {
      // nothing to compute, but a completion flag must still be raised: only allowed without one
      if (g.done_flag != nullptr) return MB_E_INVALID;
      continue;
    }
    if (g.q == nullptr) return MB_E_INVALID;
    if (!g.state_out && (g.o == nullptr || g.lse == nullptr)) return MB_E_INVALID;
    if ((g.state_in || g.state_out) && (g.state_o == nullptr || g.state_ml == nullptr)) return MB_E_INVALID;
    if ((reinterpret_cast<uintptr_t>(g.state_o) & 15u) || (reinterpret_cast<uintptr_t>(g.state_ml) & 7u)) return MB_E_INVALID;
    if (g.done_flag != nullptr && g.done_counter == nullptr) return MB_E_INVALID;
    // jobs over the same query rows (the links of a state chain) share one tensor map
    int qmap = -1;
    for (int m = 0; m < nqmaps && qmap < 0; ++m) {
      const mb_fwd_job& o = *qmap_of[m];
      if (o.q == g.q && o.sq == g.sq && o.q_stride_b == g.q_stride_b && o.q_stride_s == g.q_stride_s &&
          o.q_stride_h == g.q_stride_h)
        qmap = m;
    }
    if (qmap < 0) {
      if (nqmaps == kMaxQMaps) return MB_E_INVALID;
      if (make_tile_map(&maps.q[nqmaps], g.q, kD, x->hq, g.sq, x->batch, g.q_stride_b, g.q_stride_s, g.q_stride_h))
        return MB_E_TENSORMAP;
      qmap_of[nqmaps] = &g;
      qmap = nqmaps++;
    }
    FwdJob& J = a.job[njobs];
    J.qmap = qmap;
    J.o = reinterpret_cast<__nv_bfloat16*>(g.o);
    J.o_sb = g.o_stride_b;
    J.o_ss = g.o_stride_s;
    J.o_sh = g.o_stride_h;
    J.lse = g.lse;
    J.lse_sh = g.lse_stride_h ? g.lse_stride_h : g.sq;
    J.lse_sb = g.lse_stride_b ? g.lse_stride_b : (long long)x->hq * g.sq;
    J.Sq = g.sq;
    J.q_off = g.q_off;
    unsigned mask = 0;
    for (int s = 0; s < x->nseg; ++s)
      if (seg_new[s] >= 0 && (g.seg_mask == 0 || ((g.seg_mask >> s) & 1u))) mask |= 1u << seg_new[s];
    J.seg_mask = mask;
    J.x_begin = x_total;
    J.n_pairs = (g.sq + 2 * kBM - 1) / (2 * kBM);
    J.q_flag = g.q_ready_flag;
    J.q_flag_value = g.q_ready_value;
    J.done_flag = g.done_flag;
    J.done_value = g.done_value;
    J.done_counter = g.done_counter;
    J.n_ctas = J.n_pairs * x->hq * x->batch;
    J.st_o = g.state_o;
    J.st_ml = g.state_ml;
    J.st_in = g.state_in ? 1 : 0;
    J.st_out = g.state_out ? 1 : 0;
    J.chain = g.chain;
    J.chain_wait = g.chain_wait;
    J.chain_set = g.chain_set;
    if (x_total > INT_MAX - J.n_ctas) return MB_E_INVALID;
    x_total += J.n_ctas;
    ++njobs;
  }
  if (njobs == 0) return MB_SUCCESS;
  a.njobs = njobs;
  a.B = x->batch;
  a.Hq = x->hq;
  a.group = x->hq / x->hkv;
  a.causal = x->causal ? 1 : 0;
  a.scale = x->softmax_scale;
  a.scale_log2 = x->softmax_scale * 1.4426950408889634f;
  a.peer_wait_cycles = peer_wait_cycles();
  bool has_flags = false;
  for (int s = 0; s < nseg; ++s) has_flags |= a.seg_flag[s] != nullptr;
  for (int j = 0; j < njobs; ++j) has_flags |= a.job[j].q_flag != nullptr || (a.job[j].chain != nullptr && a.job[j].st_in);
  a.wait_cycles = kWaitCycleLimit + (has_flags ? a.peer_wait_cycles : 0);
  a.status = x->status ? x->status : default_status_word();
  if (a.status == nullptr) return MB_E_CUDA;

  dim3 grid(x_total, 1, 1);
  attn_fwd_kernel<<<grid, kFwdThreads, kFwdSmemBytes, stream>>>(maps, a);
  return cuda_ok(cudaGetLastError(), "launch attn_fwd_kernel") ? MB_SUCCESS : MB_E_CUDA;
}

// One query shard: the single-job form of the launch above.
int launch_attn_fwd(const mb_attn_fwd_args* x, cudaStream_t stream) {
  if (x == nullptr) return MB_E_INVALID;
  if (x->nseg < 0 || x->nseg > MB_MAX_SEGMENTS) return MB_E_INVALID;
  if (x->sq < 0) return MB_E_INVALID;
  if (x->sq == 0) {
    if (x->head_dim != kD) return MB_E_UNSUPPORTED;
    if (x->batch <= 0 || x->hq <= 0 || x->hkv <= 0 || x->hq % x->hkv != 0) return MB_E_INVALID;
    return MB_SUCCESS;
  }
  static thread_local mb_attn_fwd_multi_args m;
  memset(&m, 0, sizeof(m));
  m.batch = x->batch; m.hq = x->hq; m.hkv = x->hkv; m.head_dim = x->head_dim;
  m.causal = x->causal; m.softmax_scale = x->softmax_scale;
  m.njobs = 1; m.nseg = x->nseg;
  mb_fwd_job& j = m.job[0];
  j.q = x->q; j.q_stride_b = x->q_stride_b; j.q_stride_s = x->q_stride_s; j.q_stride_h = x->q_stride_h;
  j.o = x->o; j.o_stride_b = x->o_stride_b; j.o_stride_s = x->o_stride_s; j.o_stride_h = x->o_stride_h;
  j.lse = x->lse; j.lse_stride_b = x->lse_stride_b; j.lse_stride_h = x->lse_stride_h;
  j.sq = x->sq; j.q_off = x->q_off;
  for (int s = 0; s < x->nseg; ++s) m.seg[s] = x->seg[s];
  m.status = x->status;
  return launch_attn_fwd_multi(&m, stream);
}

}  // namespace mb
