// Single-pass backward attention for sm_100a: dK, dV AND the dQ contributions of one K/V tile
// against a list of query shards in one sweep -- scores and probabilities are computed once
// (5 tile products per 128x128 block instead of the 7 of the two-launch form in attn_bwd.cu).
//
// Owner = K_j, V_j (128 keys), stream = Q, dO (64 query rows per step), as in mode dKV of the
// two-pass kernel:
//     X = K Q^T = S^T        Y = V dO^T = dP^T            (rows: keys, columns: queries)
//     P^T = exp2(X*c + lse2[q]),   dS^T = P^T * (Y - delta[q])
//     dV += P^T dO           dK += dS^T Q
// plus, per step,
//     dQ^T(step) = K^T dS^T  (rows: head-dim, columns: the 64 queries of the step)
// which is not accumulated on chip (every step has other queries) but added into an fp32 buffer
// [batch, hq, rows, head_dim] in global memory: the drain warps transpose it through shared memory
// into 32 query rows x 128 floats (16 KiB, contiguous in the buffer) and one thread adds it with a
// bulk reduction (cp.reduce.async.bulk ... add.f32).  Per-element red.global.add from registers was
// measured first: it cost 18 % of the kernel.  Each query row receives one contribution per K/V
// tile that it can see.  A small kernel afterwards scales and converts the
// buffer to bf16.  The order of those fp32 additions varies from run to run, so dQ is not
// bitwise reproducible (dK and dV are); the two-launch form stays available for callers that
// need determinism.
//
// Tensor memory (512 columns): dK | dV | X0 | X1 | Y | dQ^T = 128 + 128 + 4 x 64.  X is
// double-buffered; Y has one buffer, which the element-wise warps copy to registers together with X
// at the start of a step and hand back at once, so Y of the next step is produced while this step
// computes; dQ^T has one, drained by four dedicated warps a step behind.  The bf16 P^T and dS^T
// overwrite the X buffer they came from (each thread writes only columns it has itself read) and are
// the tensor-memory A operand of the dV / dK products; dS^T is also written to shared memory
// ([128 keys][64 queries], 128-byte swizzle, two buffers) as the MN-major B operand of the dQ^T
// product, whose A operand is the K tile read MN-major.
//
// Every hand-over between roles costs a few hundred cycles of latency (a timeline of the first
// version showed the element-wise warps waiting for about 1 100 of the 2 850 cycles of a step), so a
// step has as few as possible: the element-wise warps wait once (X, Y and the stage's statistics
// are all there), give Y back, and arrive once when P^T and dS^T are both in place; the issuing warp
// waits for that one event per step.  Issue order per step t: Y(t+1) | dV, dK, dQ^T of step t |
// X(t+2); the tensor pipe runs in issue order, which is what makes X(t)'s completion imply that the
// dQ^T product of step t-2 has finished reading the shared-memory dS^T buffer step t reuses.
//
// 16 warps in four warpgroups: 0-7 element-wise (lane quarter x column half), 8 MMA issuer and
// tensor-memory owner, 9 TMA loader, 10-11 idle, 12-15 drain dQ^T.  Registers are allocated per
// warpgroup (a CTA of 14 warps is charged for 16), so the CTA launches with 512 x 128 registers and
// setmaxnreg moves them to where they are needed: 168 for the element-wise warpgroups, 88 for the
// other two.  That is every register of the SM.  A launch whose stream segments carry arrival flags
// uses a second instantiation with 120 / 160 / 80 (1 % slower): the one-warp kernels that raise those
// flags from the transfer stream must be able to start beside a resident CTA.
// Every wait is bounded, as in the other kernels.
#include "attn_bwd_common.cuh"

namespace mb {

constexpr int kFusedThreads = 512;
static_assert(8 * 32 * 168 + 8 * 32 * 88 <= kFusedThreads * 128 && 8 * 32 * 160 + 8 * 32 * 80 <= kFusedThreads * 120,
              "setmaxnreg budgets exceed the registers the CTA is launched with");

// Register budgets of the roles, by the launch budget of the instantiation.
template <int kLaunchRegs>
__device__ __forceinline__ void fused_regs_aux() {
  if constexpr (kLaunchRegs == 128) asm volatile("setmaxnreg.dec.sync.aligned.u32 88;");
  else asm volatile("setmaxnreg.dec.sync.aligned.u32 80;");
}
template <int kLaunchRegs>
__device__ __forceinline__ void fused_regs_ew() {
  if constexpr (kLaunchRegs == 128) asm volatile("setmaxnreg.inc.sync.aligned.u32 168;");
  else asm volatile("setmaxnreg.inc.sync.aligned.u32 160;");
}
constexpr int kFusedStages = 3;
constexpr int kDsBytes = kOwnRows * kStrRows * 2;  // 16 KiB: dS^T as [128 keys][64 queries] bf16
constexpr int kDqStageBytes = 32 * kBD * 4;          // 16 KiB: 32 query rows x 128 floats on their way to the reduction
constexpr int kFusedSmemBytes =
    2 * kOwnTileBytes + kFusedStages * kBwdStageBytes + 2 * kDsBytes + kDqStageBytes + 1024 + 1024;
static_assert(kFusedSmemBytes <= 232448, "shared memory budget of one CTA");

struct FusedSmem {
  uint64_t own_full;
  uint64_t str_full[kFusedStages];
  uint64_t str_empty[kFusedStages];
  // Per-step events alternate between two barriers (step t uses [t & 1], phase t >> 1), so that a
  // role one step ahead of its partner can never complete a phase the partner has yet to look at.
  uint64_t x_full[2];
  uint64_t y_full[2];
  uint64_t y_free[2];   // 256 arrivals: every element-wise thread has copied its part of Y
  uint64_t pd_full[2];  // 256 arrivals: P^T and dS^T of the step are in tensor memory, dS^T also in shared memory
  uint64_t dq_full[2];  // the dQ^T product of the step (and everything issued before it) is complete
  uint64_t dq_free[2];  // 128 arrivals: the drain warps have copied dQ^T out
  uint64_t acc_full;
  uint64_t drain;
  uint32_t tmem_base;
  int abort_word;
  int seg_first[MB_MAX_SEGMENTS];
  int seg_last[MB_MAX_SEGMENTS];
};
static_assert(sizeof(FusedSmem) <= 1024, "control block too large");

// dQ^T = K^T dS^T for one step: 8 MMAs of 16 keys (M = 128 head-dim, N = 64 queries).  Both operands
// are read MN-major from shared memory; 16 keys are 16 rows of 128 bytes = 128 descriptor units in
// either tile.
__device__ __forceinline__ void issue_dq_group(uint32_t d_tmem, uint64_t k_desc, uint64_t ds_desc, uint32_t idesc) {
  asm volatile(
      "{\n\t"
      ".reg .pred pe, pt, pf;\n\t"
      ".reg .b64 ka, sb;\n\t"
      "elect.sync _|pe, 0xffffffff;\n\t"
      "setp.eq.u32 pt, 0, 0;\n\t"
      "setp.ne.u32 pf, 0, 0;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, pf;\n\t"
      "add.s64 ka, %1, 128;\n\t add.s64 sb, %2, 128;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], ka, sb, %3, pt;\n\t"
      "add.s64 ka, %1, 256;\n\t add.s64 sb, %2, 256;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], ka, sb, %3, pt;\n\t"
      "add.s64 ka, %1, 384;\n\t add.s64 sb, %2, 384;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], ka, sb, %3, pt;\n\t"
      "add.s64 ka, %1, 512;\n\t add.s64 sb, %2, 512;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], ka, sb, %3, pt;\n\t"
      "add.s64 ka, %1, 640;\n\t add.s64 sb, %2, 640;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], ka, sb, %3, pt;\n\t"
      "add.s64 ka, %1, 768;\n\t add.s64 sb, %2, 768;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], ka, sb, %3, pt;\n\t"
      "add.s64 ka, %1, 896;\n\t add.s64 sb, %2, 896;\n\t"
      "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], ka, sb, %3, pt;\n\t"
      "}"
      :
      : "r"(d_tmem), "l"(k_desc), "l"(ds_desc), "r"(idesc)
      : "memory");
}

template <int kLaunchRegs>
__global__ void __maxnreg__(kLaunchRegs) attn_bwd_fused_kernel(const __grid_constant__ BwdMaps maps,
                                                       const __grid_constant__ BwdArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sOwn = smem;                   // K tile
  uint8_t* sOwnG = smem + kOwnTileBytes;  // V tile
  uint8_t* sStage = smem + 2 * kOwnTileBytes;
  uint8_t* sDs = sStage + kFusedStages * kBwdStageBytes;  // two buffers; 1024-byte aligned: every piece before it is
  float* sDq = reinterpret_cast<float*>(sDs + 2 * kDsBytes);  // staging of the dQ reduction
  FusedSmem* ctl = reinterpret_cast<FusedSmem*>(sDs + 2 * kDsBytes + kDqStageBytes);
  volatile int* abort_word = &ctl->abort_word;
  static_assert((kFusedStages * kBwdStageBytes) % 1024 == 0, "dS^T tile must stay 1024-byte aligned");

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int own0 = blockIdx.x * kOwnRows;
  const int h_own = blockIdx.y;  // K/V head
  const int b = blockIdx.z;
  const int n_sub = a.group;     // query heads streamed per segment
  const int h_str_base = h_own * a.group;

  if (tid == 0) {
    mbar_init(&ctl->own_full, 1);
    for (int s = 0; s < kFusedStages; ++s) {
      mbar_init(&ctl->str_full[s], 1);
      mbar_init(&ctl->str_empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&ctl->x_full[i], 1);
      mbar_init(&ctl->y_full[i], 1);
      mbar_init(&ctl->y_free[i], 256);
      mbar_init(&ctl->pd_full[i], 256);
      mbar_init(&ctl->dq_full[i], 1);
      mbar_init(&ctl->dq_free[i], 128);
    }
    mbar_init(&ctl->acc_full, 1);
    mbar_init(&ctl->drain, 1);
    ctl->abort_word = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (tid < MB_MAX_SEGMENTS) {  // one thread per segment: its range of 64-row steps for this owner tile
    int f = 0, l = 0;
    if (tid < a.nseg) step_range(a, own0, tid, &f, &l);
    ctl->seg_first[tid] = f;
    ctl->seg_last[tid] = l;
  }
  if (warp == 8) {
    tmem_alloc(&ctl->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  // columns: dK [0,128) dV [128,256) X0 [256,320) X1 [320,384) Y [384,448) dQ^T [448,512)
  const uint32_t tmem = ctl->tmem_base;
  constexpr uint32_t kColX = 256, kColY = 384, kColDq = 448;

  int total_steps = 0;
  for (int s = 0; s < a.nseg; ++s) total_steps += (ctl->seg_last[s] - ctl->seg_first[s]) * n_sub;

  // Every role changes its register budget as the first thing it does (a warpgroup-wide instruction: all
  // four warps of a warpgroup execute the same one).
  if (warp == 9) {
    // ------------------------------------------------------------------ loader
    fused_regs_aux<kLaunchRegs>();
    if (lane == 0 && total_steps > 0) {
      mbar_expect_tx(&ctl->own_full, 2 * kOwnTileBytes);
      tma_load_4d(sOwn, &maps.own, &ctl->own_full, 0, h_own, own0, b);
      tma_load_4d(sOwn + kOwnHalfBytes, &maps.own, &ctl->own_full, 64, h_own, own0, b);
      tma_load_4d(sOwnG, &maps.own_g, &ctl->own_full, 0, h_own, own0, b);
      tma_load_4d(sOwnG + kOwnHalfBytes, &maps.own_g, &ctl->own_full, 64, h_own, own0, b);
      int n = 0;
      bool ok = true;
      for (int s = 0; s < a.nseg && ok; ++s) {
        const int f = ctl->seg_first[s], l = ctl->seg_last[s];
        if (l > f && a.seg_flag[s] != nullptr) {
          ok = flag_wait_ge(a.seg_flag[s], a.seg_flag_value[s], abort_word, MB_ERR_TIMEOUT_SEGMENT,
                            a.peer_wait_cycles);
          asm volatile("fence.proxy.async;" ::: "memory");
        }
        for (int g = 0; g < n_sub && ok; ++g) {
          const int h_str = h_str_base + g;
          for (int t = f; t < l; ++t) {
            const int stage = n % kFusedStages, round = n / kFusedStages;
            if (round > 0 && !mbar_wait(&ctl->str_empty[stage], (round - 1) & 1, abort_word, MB_ERR_TIMEOUT_KV_EMPTY,
                                        a.wait_cycles)) {
              ok = false;
              break;
            }
            uint8_t* dst = sStage + stage * kBwdStageBytes;
            mbar_expect_tx(&ctl->str_full[stage], 2 * kStrTileBytes + kStatBytes);
            const int r0 = t * kStrRows;
            tma_load_4d(dst, &maps.str[s], &ctl->str_full[stage], 0, h_str, r0, b);
            tma_load_4d(dst + kStrHalfBytes, &maps.str[s], &ctl->str_full[stage], 64, h_str, r0, b);
            tma_load_4d(dst + kStrTileBytes, &maps.str_g[s], &ctl->str_full[stage], 0, h_str, r0, b);
            tma_load_4d(dst + kStrTileBytes + kStrHalfBytes, &maps.str_g[s], &ctl->str_full[stage], 64, h_str, r0, b);
            const long long soff = ((long long)b * a.Hq + h_str) * a.seg_stat_pad[s] + r0;
            bulk_load(dst + 2 * kStrTileBytes, a.seg_lse2[s] + soff, kStrRows * 4, &ctl->str_full[stage]);
            bulk_load(dst + 2 * kStrTileBytes + kStrRows * 4, a.seg_delta[s] + soff, kStrRows * 4,
                      &ctl->str_full[stage]);
            ++n;
          }
        }
      }
      if (!ok) {
        const int first = n > kFusedStages ? n - kFusedStages : 0;
        for (int m = first; m < n; ++m) {
          const long long t0 = clock64();
          while (!mbar_try_wait(&ctl->str_full[m % kFusedStages], (m / kFusedStages) & 1) &&
                 clock64() - t0 < kWaitCycleLimit / 16) {
          }
        }
      }
    }
  } else if (warp == 8) {
    // -------------------------------------------------------------- MMA issuer
    fused_regs_aux<kLaunchRegs>();
    if (total_steps > 0) {  // whole warp, converged; one elected lane issues
      constexpr uint32_t idesc_xy = umma_idesc_bf16(kOwnRows, kStrRows, false, false);  // 128 x 64, both K-major
      constexpr uint32_t idesc_acc = umma_idesc_bf16(kOwnRows, kBD, false, true);       // 128 x 128, B MN-major
      constexpr uint32_t idesc_dq = umma_idesc_bf16(kBD, kStrRows, true, true);         // 128 x 64, both MN-major
      const uint64_t k_desc = umma_smem_desc(smem_u32(sOwn), 16, 1024);                   // K, K-major (for X)
      const uint64_t v_desc = umma_smem_desc(smem_u32(sOwnG), 16, 1024);                  // V, K-major (for Y)
      const uint64_t kt_desc = umma_smem_desc(smem_u32(sOwn), kOwnHalfBytes, 1024);       // K, MN-major (for dQ^T)
      const uint64_t ds_desc = umma_smem_desc(smem_u32(sDs), kStrHalfBytes, 1024);        // dS^T, MN-major
      const uint64_t str_k_desc0 = umma_smem_desc(smem_u32(sStage), 16, 1024);             // stage 0, K-major
      const uint64_t str_mn_desc0 = umma_smem_desc(smem_u32(sStage), kStrHalfBytes, 1024);  // stage 0, MN-major
      constexpr uint32_t kStageUnits = kBwdStageBytes / 16, kStrGUnits = kStrTileBytes / 16;
      const int T = total_steps;
      bool ok = mbar_wait_warp(&ctl->own_full, 0, abort_word, MB_ERR_TIMEOUT_Q, a.wait_cycles);

      auto stage_units = [&](int t) { return static_cast<uint32_t>(t % kFusedStages) * kStageUnits; };
      auto wait_stage = [&](int t) {
        return mbar_wait_warp(&ctl->str_full[t % kFusedStages], (t / kFusedStages) & 1, abort_word,
                              MB_ERR_TIMEOUT_KV_FULL, a.wait_cycles);
      };
      auto issue_x = [&](int t) {  // X(t) = K Q(t)^T
        issue_xy_group(tmem + kColX + (t & 1) * 64, k_desc, str_k_desc0 + stage_units(t), idesc_xy);
        umma_commit_elect(&ctl->x_full[t & 1]);
      };
      auto issue_y = [&](int t) {  // Y(t) = V dO(t)^T
        issue_xy_group(tmem + kColY, v_desc, str_k_desc0 + stage_units(t) + kStrGUnits, idesc_xy);
        umma_commit_elect(&ctl->y_full[t & 1]);
      };

      // prologue: X(0), Y(0), X(1)
      if (ok) ok = wait_stage(0);
      if (ok) {
        tc_fence_after();
        issue_x(0);
        issue_y(0);
      }
      if (ok && T > 1) {
        ok = wait_stage(1);
        if (ok) {
          tc_fence_after();
          issue_x(1);
        }
      }
      for (int t = 0; t < T && ok; ++t) {
        const uint32_t tx = tmem + kColX + (t & 1) * 64;
        const uint32_t su = stage_units(t);
        // Y of the next step: its buffer is free once every thread holds Y(t) in registers, which
        // happens at the start of the element-wise step (its stage arrived before X(t+1) was issued)
        if (t + 1 < T) {
          ok = mbar_wait_warp(&ctl->y_free[t & 1], (t >> 1) & 1, abort_word, MB_ERR_TIMEOUT_S, a.wait_cycles);
          if (!ok) break;
          tc_fence_after();
          issue_y(t + 1);
        }
        // dV += P^T dO, dK += dS^T Q, dQ^T = K^T dS^T
        ok = mbar_wait_warp(&ctl->pd_full[t & 1], (t >> 1) & 1, abort_word, MB_ERR_TIMEOUT_P, a.wait_cycles);
        if (!ok) break;
        tc_fence_after();
        issue_acc_group(tmem + 128, tx, str_mn_desc0 + su + kStrGUnits, idesc_acc, t > 0 ? 1u : 0u);
        issue_acc_group(tmem + 0, tx + 16, str_mn_desc0 + su, idesc_acc, t > 0 ? 1u : 0u);
        if (t > 0) {  // the drain warps must have copied dQ^T(t-1) out
          ok = mbar_wait_warp(&ctl->dq_free[(t - 1) & 1], ((t - 1) >> 1) & 1, abort_word, MB_ERR_TIMEOUT_O,
                              a.wait_cycles);
          if (!ok) break;
          tc_fence_after();
        }
        issue_dq_group(tmem + kColDq, kt_desc, ds_desc + (t & 1) * (kDsBytes / 16), idesc_dq);
        umma_commit_elect(&ctl->dq_full[t & 1]);
        umma_commit_elect(&ctl->str_empty[t % kFusedStages]);
        // X of step t+2 into the buffer whose P^T / dS^T the products above read (in issue order)
        if (t + 2 < T) {
          ok = wait_stage(t + 2);
          if (!ok) break;
          tc_fence_after();
          issue_x(t + 2);
        }
      }
      if (ok) {
        umma_commit_elect(&ctl->acc_full);
      } else {
        umma_commit_elect(&ctl->drain);
        const long long t0 = clock64();
        while (!mbar_try_wait(&ctl->drain, 0) && clock64() - t0 < kWaitCycleLimit / 16) {
        }
        __syncwarp();
      }
    }
  } else if (warp == 10 || warp == 11) {
    // idle: these two warps only complete the third warpgroup
    fused_regs_aux<kLaunchRegs>();
  } else if (warp >= 12) {
    // ------------------------------------------------ drain dQ^T: tensor memory -> red.global.add
    fused_regs_aux<kLaunchRegs>();
    const int quarter = warp & 3;
    const int d = (quarter << 5) | lane;  // head-dim index == tensor-memory lane
    const uint32_t tq = tmem + kColDq + (static_cast<uint32_t>(quarter << 5) << 16);
    const bool issuer = warp == 12 && lane == 0;
    bool ok = true;
    int t = 0;
    for (int s = 0; s < a.nseg && ok; ++s) {
      const int f = ctl->seg_first[s], l = ctl->seg_last[s];
      const int rows = a.seg_rows[s];
      for (int g = 0; g < n_sub && ok; ++g) {
        float* acc_base = a.seg_dq[s] + ((long long)b * a.Hq + (h_str_base + g)) * a.seg_stat_pad[s] * kBD;
        for (int st = f; st < l; ++st, ++t) {
          ok = mbar_wait_warp(&ctl->dq_full[t & 1], (t >> 1) & 1, abort_word, MB_ERR_TIMEOUT_O, a.wait_cycles);
          {
            // The four drain warps meet at named barriers below, so they must leave the loop together:
            // agree on the outcome of the (bounded) wait.  Every warp always reaches this point.
            uint32_t all_ok;
            asm volatile(
                "{\n\t"
                ".reg .pred pin, pout;\n\t"
                "setp.ne.u32 pin, %1, 0;\n\t"
                "bar.red.and.pred pout, 2, 128, pin;\n\t"
                "selp.u32 %0, 1, 0, pout;\n\t"
                "}"
                : "=r"(all_ok)
                : "r"(ok ? 1u : 0u)
                : "memory");
            ok = all_ok != 0;
          }
          if (!ok) break;
          tc_fence_after();
          uint32_t v[2][32];
          tmem_ld32(tq, v[0]);
          tmem_ld32(tq + 32, v[1]);
          tmem_wait_ld();
          tc_fence_before();
          mbar_arrive(&ctl->dq_free[t & 1]);
          const int r0 = st * kStrRows;
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            const int nrow = min(32, rows - (r0 + hh * 32));  // rows past the shard's end carry zeros: skipped
            // the staging tile is free once the previous bulk reduction has read it
            if (issuer) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            asm volatile("bar.sync 1, 128;" ::: "memory");
            // transpose: lane d of the tile's column e becomes element [e][d] (conflict-free rows of 128 floats)
#pragma unroll
            for (int e = 0; e < 32; ++e) sDq[e * kBD + d] = __uint_as_float(v[hh][e]);
            fence_proxy_async_smem();
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (issuer && nrow > 0) {
              float* dst = acc_base + (long long)(r0 + hh * 32) * kBD;
              asm volatile(
                  "cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;\n\t"
                  "cp.async.bulk.commit_group;"
                  :
                  : "l"(dst), "r"(smem_u32(sDq)), "r"(nrow * kBD * 4)
                  : "memory");
            }
          }
        }
      }
    }
    // the last reduction must have left shared memory before the CTA exits (its global side completes on its own)
    if (issuer) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  } else {
    // ------------------------------------------------ element-wise warps (0..7) + epilogue
    fused_regs_ew<kLaunchRegs>();
    const int quarter = warp & 3, half = warp >> 2;
    const int row = (quarter << 5) | lane;  // key row == tensor-memory lane
    const uint32_t lane_field = static_cast<uint32_t>(quarter << 5) << 16;
    const int own_pos = a.own_off + own0 + row;
    // my row of the dS^T tile in shared memory: four 16-byte chunks (32 queries), 128-byte swizzle
    const int swz = row & 7;
    bool ok = true;

    int t = 0;
    for (int s = 0; s < a.nseg && ok; ++s) {
      const int f = ctl->seg_first[s], l = ctl->seg_last[s];
      const int seg_off = a.seg_off[s];
      for (int g = 0; g < n_sub && ok; ++g) {
        for (int st = f; st < l; ++st, ++t) {
          const int buf = t & 1, stage = t % kFusedStages;
          const uint32_t tx = tmem + kColX + buf * 64 + lane_field + half * 32;
          const uint32_t ty = tmem + kColY + lane_field + half * 32;
          // One wait per step: the stage (its statistics are read below; it landed long ago, this only
          // orders those reads after the bulk copy), X and Y.
          ok = mbar_wait_warp(&ctl->str_full[stage], (t / kFusedStages) & 1, abort_word, MB_ERR_TIMEOUT_KV_FULL,
                              a.wait_cycles) &&
               mbar_wait_warp(&ctl->x_full[buf], (t >> 1) & 1, abort_word, MB_ERR_TIMEOUT_S, a.wait_cycles) &&
               mbar_wait_warp(&ctl->y_full[buf], (t >> 1) & 1, abort_word, MB_ERR_TIMEOUT_S, a.wait_cycles);
          if (!ok) break;
          tc_fence_after();
          uint32_t xr[32], yr[32];
          tmem_ld32(tx, xr);
          tmem_ld32(ty, yr);
          tmem_wait_ld();
          tc_fence_before();
          mbar_arrive(&ctl->y_free[buf]);   // Y(t+1) may overwrite the buffer from here on

          const int c0 = st * kStrRows + half * 32;  // first query row (local to the segment) of my columns
          int lo = 0;
          if (a.causal) lo = own_pos - (seg_off + c0);  // query c visible iff seg_off + c0 + c >= own_pos
          const bool need_mask = __any_sync(0xffffffffu, lo > 0);
          const float* stats = reinterpret_cast<const float*>(sStage + stage * kBwdStageBytes + 2 * kStrTileBytes);
          const float* nl_col = stats + half * 32;            // -lse*log2(e) of my 32 columns
          const float* d_col = stats + kStrRows + half * 32;  // delta of my 32 columns

          // p = exp2(x*c + nlse2), ds = p * (y - delta): packed pairs, bf16 pairs out
          uint32_t pk[16], dk[16];
          if (need_mask) ew_compute<true, true>(xr, yr, pk, dk, a.scale_log2, nl_col, d_col, 0.f, 0.f, lo, 32);
          else ew_compute<true, false>(xr, yr, pk, dk, a.scale_log2, nl_col, d_col, 0.f, 0.f, lo, 32);
          tmem_st16(tx, pk);
          tmem_st16(tx + 16, dk);
          // dS^T also to shared memory.  Buffer t & 1 was last read by the dQ^T product of step t-2, which
          // the tensor pipe finished before it produced X(t) (issue order), so no further wait is needed.
          uint8_t* ds_row = sDs + buf * kDsBytes + row * 128;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int chunk = (half * 4 + c) ^ swz;
            *reinterpret_cast<uint4*>(ds_row + chunk * 16) = make_uint4(dk[c * 4], dk[c * 4 + 1], dk[c * 4 + 2], dk[c * 4 + 3]);
          }
          fence_proxy_async_smem();
          tmem_wait_st();
          tc_fence_before();
          mbar_arrive(&ctl->pd_full[buf]);
        }
      }
    }

    // epilogue: each warp stores its lane quarter x column half of dK and dV
    if (ok && own0 < a.own_rows) {
      const bool have = total_steps > 0;
      if (have) ok = mbar_wait_warp(&ctl->acc_full, 0, abort_word, MB_ERR_TIMEOUT_O, a.wait_cycles);
      if (ok) {
        if (have) tc_fence_after();
        const bool store = own0 + row < a.own_rows;
        for (int which = 0; which < 2; ++which) {
          void* base = which ? a.out2 : a.out1;
          const float mul = which ? 1.f : a.scale;  // dK carries the softmax scale, dV does not
          const long long off = (long long)b * a.o_sb + (long long)(own0 + row) * a.o_ss + (long long)h_own * a.o_sh;
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            uint32_t acc[32];
            if (have) {
              tmem_ld32(tmem + which * 128 + lane_field + half * 64 + c * 32, acc);
              tmem_wait_ld();
            } else {
#pragma unroll
              for (int e = 0; e < 32; ++e) acc[e] = 0u;
            }
            if (!store) continue;
            const int col = half * 64 + c * 32;
            if (a.out_mode == 0) {
              uint4* dst = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(base) + off + col);
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                uint4 w;
                w.x = pack_bf16x2(__uint_as_float(acc[v * 8 + 0]) * mul, __uint_as_float(acc[v * 8 + 1]) * mul);
                w.y = pack_bf16x2(__uint_as_float(acc[v * 8 + 2]) * mul, __uint_as_float(acc[v * 8 + 3]) * mul);
                w.z = pack_bf16x2(__uint_as_float(acc[v * 8 + 4]) * mul, __uint_as_float(acc[v * 8 + 5]) * mul);
                w.w = pack_bf16x2(__uint_as_float(acc[v * 8 + 6]) * mul, __uint_as_float(acc[v * 8 + 7]) * mul);
                dst[v] = w;
              }
            } else {
              float4* dst = reinterpret_cast<float4*>(static_cast<float*>(base) + off + col);
#pragma unroll
              for (int v = 0; v < 8; ++v) {
                float4 w = make_float4(__uint_as_float(acc[v * 4 + 0]) * mul, __uint_as_float(acc[v * 4 + 1]) * mul,
                                       __uint_as_float(acc[v * 4 + 2]) * mul, __uint_as_float(acc[v * 4 + 3]) * mul);
                if (a.out_mode == 2) {
                  const float4 old = dst[v];
                  w.x += old.x; w.y += old.y; w.z += old.z; w.w += old.w;
                }
                dst[v] = w;
              }
            }
          }
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
// dq[b, s, h, :] = scale * acc[b, h, s, :]  (fp32 accumulation buffer -> the caller's dq tensor)
// ---------------------------------------------------------------------------
struct DqConvertArgs {
  const float* acc;  // [B, Hq, pad, D]
  void* dq;          // [B, Sq, Hq, D] bf16 or fp32, strides in elements
  long long sb, ss, sh;
  int B, Sq, Hq, pad, f32_out;
  float scale;
};

// One warp per (b, h, row): a row is 128 floats = 4 per lane.
__global__ void __launch_bounds__(256) dq_convert_kernel(const DqConvertArgs a) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int row = blockIdx.x * 8 + w;
  const int h = blockIdx.y, b = blockIdx.z;
  if (row >= a.Sq) return;
  const float4 v = *reinterpret_cast<const float4*>(a.acc + (((long long)b * a.Hq + h) * a.pad + row) * kBD + lane * 4);
  const long long off = b * a.sb + row * a.ss + h * a.sh + lane * 4;
  if (a.f32_out) {
    *reinterpret_cast<float4*>(static_cast<float*>(a.dq) + off) =
        make_float4(v.x * a.scale, v.y * a.scale, v.z * a.scale, v.w * a.scale);
  } else {
    uint2 o;
    o.x = pack_bf16x2(v.x * a.scale, v.y * a.scale);
    o.y = pack_bf16x2(v.z * a.scale, v.w * a.scale);
    *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(a.dq) + off) = o;
  }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
int launch_attn_bwd_fused(const BwdMaps& maps, const BwdArgs& a, dim3 grid, cudaStream_t stream) {
  static bool done[64] = {};
  int dev = 0;
  if (!cuda_ok(cudaGetDevice(&dev), "cudaGetDevice")) return MB_E_CUDA;
  if (dev >= 0 && dev < 64 && !done[dev]) {
    if (!cuda_ok(cudaFuncSetAttribute(attn_bwd_fused_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      kFusedSmemBytes),
                 "shared-memory attribute of attn_bwd_fused_kernel") ||
        !cuda_ok(cudaFuncSetAttribute(attn_bwd_fused_kernel<120>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      kFusedSmemBytes),
                 "shared-memory attribute of attn_bwd_fused_kernel"))
      return MB_E_CUDA;
    done[dev] = true;
  }
  // arrival flags are raised by one-warp kernels of the transfer stream: leave them room on every SM
  bool has_flags = false;
  for (int s = 0; s < a.nseg; ++s) has_flags |= a.seg_flag[s] != nullptr;
  if (has_flags) attn_bwd_fused_kernel<120><<<grid, kFusedThreads, kFusedSmemBytes, stream>>>(maps, a);
  else attn_bwd_fused_kernel<128><<<grid, kFusedThreads, kFusedSmemBytes, stream>>>(maps, a);
  return cuda_ok(cudaGetLastError(), "launch attn_bwd_fused_kernel") ? MB_SUCCESS : MB_E_CUDA;
}

int launch_dq_convert(const float* acc, void* dq, long long sb, long long ss, long long sh, int batch, int sq, int hq,
                      int pad, int out_mode, float scale, cudaStream_t stream) {
  if (acc == nullptr || dq == nullptr || batch <= 0 || hq <= 0 || sq < 0 || pad < sq) return MB_E_INVALID;
  if (out_mode != MB_OUT_BF16 && out_mode != MB_OUT_F32) return MB_E_INVALID;
  if (sq == 0) return MB_SUCCESS;
  DqConvertArgs a;
  a.acc = acc; a.dq = dq; a.sb = sb; a.ss = ss; a.sh = sh;
  a.B = batch; a.Sq = sq; a.Hq = hq; a.pad = pad; a.f32_out = out_mode == MB_OUT_F32 ? 1 : 0; a.scale = scale;
  dim3 grid((sq + 7) / 8, hq, batch);
  dq_convert_kernel<<<grid, 256, 0, stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? MB_SUCCESS : MB_E_CUDA;
}

}  // namespace mb
