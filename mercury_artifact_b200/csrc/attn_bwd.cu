// Backward attention for sm_100a: dQ, dK, dV of one query shard against a list
// of K/V shards (dQ) and of one K/V shard against a list of query shards (dK/dV).
//
// One kernel template runs in two modes.  An "owner" tile of 128 rows keeps its
// accumulators in tensor memory while "stream" tiles of 64 rows pass by:
//
//   mode dKV: owner = K_j, V_j (128 keys); stream = Q, dO (64 query rows per step)
//       X = K Q^T = S^T     Y = V dO^T = dP^T          (rows: keys, columns: queries)
//       P^T = exp2(X*c + lse2[q]),  dS^T = P^T * (Y - delta[q])
//       dV += P^T dO        dK += dS^T Q
//   mode dQ:  owner = Q_i, dO_i (128 query rows); stream = K, V (64 keys per step)
//       X = Q K^T = S       Y = dO V^T = dP
//       P = exp2(X*c + lse2[q]),    dS = P * (Y - delta[q])
//       dQ += dS K
//
// lse2 is stored NEGATED, -lse * log2(e) (and -inf for rows without keys and for padding, so
// that P = exp2(X*c + lse2) = 0 there); it and delta = rowsum(dO * O) come from a small
// preprocess kernel.  X and Y
// are double-buffered in tensor memory (2 x 2 x 64 columns); the bf16 P and dS
// overwrite them in place and feed the accumulating MMAs as the tensor-memory A
// operand; the stream tile in shared memory is read once K-major (for X, Y) and
// once MN-major (for the accumulation).  Scores are recomputed in both modes
// (7 tile MMAs per 128x128 block instead of 5), which buys an atomic-free,
// deterministic kernel with no fp32 dQ scratch.
//
// The stream is a list of segments (shards), each with an optional arrival flag,
// exactly like the forward kernel: the backward of a whole ring for one rank is
// two launches (dQ over all K/V shards, dK/dV over all query shards) and the
// reference's rotating fp32 dK/dV accumulator (codegen.py:116-190) is not needed:
// every gradient tile is owned by exactly one CTA.
//
// Replaces _flash_attn_backward(**params), utils/attn_bwd_dsl.py:115 of the reference.
#include "attn_bwd_common.cuh"

namespace mb {

template <int kDummy>
__global__ void __maxnreg__(160) attn_bwd_kernel(const __grid_constant__ BwdMaps maps,
                                                 const __grid_constant__ BwdArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sOwn = smem;
  uint8_t* sOwnG = smem + kOwnTileBytes;
  uint8_t* sStage = smem + 2 * kOwnTileBytes;
  BwdSmem* ctl = reinterpret_cast<BwdSmem*>(sStage + kBwdStages * kBwdStageBytes);
  volatile int* abort_word = &ctl->abort_word;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int own0 = blockIdx.x * kOwnRows;
  const int h_own = blockIdx.y;  // dKV: kv head; dQ: query head
  const int b = blockIdx.z;
  const int n_sub = a.mode_dkv ? a.group : 1;  // query heads streamed per segment
  const int h_str_base = a.mode_dkv ? h_own * a.group : h_own / a.group;

  if (tid == 0) {
    mbar_init(&ctl->own_full, 1);
    for (int s = 0; s < kBwdStages; ++s) {
      mbar_init(&ctl->str_full[s], 1);
      mbar_init(&ctl->str_empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&ctl->xy_full[i], 1);
      mbar_init(&ctl->pd_full[i], 256);
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
  const uint32_t tmem = ctl->tmem_base;  // Acc1 [0,128) Acc2 [128,256) X0 [256,320) Y0 [320,384) X1 [384,448) Y1 [448,512)

  int total_steps = 0;
  for (int s = 0; s < a.nseg; ++s) total_steps += (ctl->seg_last[s] - ctl->seg_first[s]) * n_sub;

  if (warp == 9) {
    // ------------------------------------------------------------------ loader
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
            const int stage = n % kBwdStages, round = n / kBwdStages;
            if (round > 0 &&
                !mbar_wait(&ctl->str_empty[stage], (round - 1) & 1, abort_word, MB_ERR_TIMEOUT_KV_EMPTY, a.wait_cycles)) {
              ok = false;
              break;
            }
            uint8_t* dst = sStage + stage * kBwdStageBytes;
            mbar_expect_tx(&ctl->str_full[stage], 2 * kStrTileBytes + (a.mode_dkv ? kStatBytes : 0));
            const int r0 = t * kStrRows;
            tma_load_4d(dst, &maps.str[s], &ctl->str_full[stage], 0, h_str, r0, b);
            tma_load_4d(dst + kStrHalfBytes, &maps.str[s], &ctl->str_full[stage], 64, h_str, r0, b);
            tma_load_4d(dst + kStrTileBytes, &maps.str_g[s], &ctl->str_full[stage], 0, h_str, r0, b);
            tma_load_4d(dst + kStrTileBytes + kStrHalfBytes, &maps.str_g[s], &ctl->str_full[stage], 64, h_str, r0, b);
            if (a.mode_dkv) {
              const long long soff = ((long long)b * a.Hq + h_str) * a.seg_stat_pad[s] + r0;
              bulk_load(dst + 2 * kStrTileBytes, a.seg_lse2[s] + soff, kStrRows * 4, &ctl->str_full[stage]);
              bulk_load(dst + 2 * kStrTileBytes + kStrRows * 4, a.seg_delta[s] + soff, kStrRows * 4,
                        &ctl->str_full[stage]);
            }
            ++n;
          }
        }
      }
      if (!ok) {
        const int first = n > kBwdStages ? n - kBwdStages : 0;
        for (int m = first; m < n; ++m) {
          const long long t0 = clock64();
          while (!mbar_try_wait(&ctl->str_full[m % kBwdStages], (m / kBwdStages) & 1) &&
                 clock64() - t0 < kWaitCycleLimit / 16) {
          }
        }
      }
    }
  } else if (warp == 8) {
    // -------------------------------------------------------------- MMA issuer
    if (total_steps > 0) {  // whole warp, converged; one elected lane issues
      constexpr uint32_t idesc_xy = umma_idesc_bf16(kOwnRows, kStrRows, false, false);  // 128 x 64, both K-major
      constexpr uint32_t idesc_acc = umma_idesc_bf16(kOwnRows, kBD, false, true);       // 128 x 128, B MN-major
      const uint64_t own_desc = umma_smem_desc(smem_u32(sOwn), 16, 1024);
      const uint64_t own_g_desc = umma_smem_desc(smem_u32(sOwnG), 16, 1024);
      const uint64_t str_k_desc0 = umma_smem_desc(smem_u32(sStage), 16, 1024);             // K-major view, stage 0
      const uint64_t str_mn_desc0 = umma_smem_desc(smem_u32(sStage), kStrHalfBytes, 1024);  // MN-major view, stage 0
      constexpr uint32_t kStageUnits = kBwdStageBytes / 16, kStrGUnits = kStrTileBytes / 16;
      const int T = total_steps;
      const bool dkv = a.mode_dkv != 0;
      bool ok = mbar_wait_warp(&ctl->own_full, 0, abort_word, MB_ERR_TIMEOUT_Q, a.wait_cycles);

      auto issue_xy = [&](int t) {
        const uint32_t su = (t % kBwdStages) * kStageUnits;
        const uint32_t tx = tmem + 256 + (t & 1) * 128;
        issue_xy_group(tx, own_desc, str_k_desc0 + su, idesc_xy);
        issue_xy_group(tx + 64, own_g_desc, str_k_desc0 + su + kStrGUnits, idesc_xy);
        umma_commit_elect(&ctl->xy_full[t & 1]);
      };
      auto issue_acc = [&](int t) {
        const int stage = t % kBwdStages;
        const uint32_t su = stage * kStageUnits;
        const uint32_t tx = tmem + 256 + (t & 1) * 128;
        // dS overlays Y, P overlays X
        issue_acc_group(tmem + 0, tx + 64, str_mn_desc0 + su, idesc_acc, t > 0 ? 1u : 0u);
        if (dkv) issue_acc_group(tmem + 128, tx, str_mn_desc0 + su + kStrGUnits, idesc_acc, t > 0 ? 1u : 0u);
        umma_commit_elect(&ctl->str_empty[stage]);
      };

      for (int t = 0; t < 2 && t < T && ok; ++t) {
        ok = mbar_wait_warp(&ctl->str_full[t % kBwdStages], 0, abort_word, MB_ERR_TIMEOUT_KV_FULL, a.wait_cycles);
        if (ok) {
          tc_fence_after();
          issue_xy(t);
        }
      }
      for (int t = 0; t < T && ok; ++t) {
        ok = mbar_wait_warp(&ctl->pd_full[t & 1], (t >> 1) & 1, abort_word, MB_ERR_TIMEOUT_P, a.wait_cycles);
        if (!ok) break;
        tc_fence_after();
        issue_acc(t);
        if (t + 2 < T) {
          const int n = t + 2;
          ok = mbar_wait_warp(&ctl->str_full[n % kBwdStages], (n / kBwdStages) & 1, abort_word,
                              MB_ERR_TIMEOUT_KV_FULL, a.wait_cycles);
          if (!ok) break;
          tc_fence_after();
          issue_xy(n);
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
  } else {
    // ------------------------------------------------ element-wise warps (0..7) + epilogue
    const int quarter = warp & 3, half = warp >> 2;
    const int row = (quarter << 5) | lane;  // owner row == tensor-memory lane
    const uint32_t lane_field = static_cast<uint32_t>(quarter << 5) << 16;
    const int own_pos = a.own_off + own0 + row;
    bool ok = true;

    const bool dkv_mode = a.mode_dkv != 0;
    float row_nl = 0.f, row_d = 0.f;
    if (!dkv_mode) {
      const int r = min(own0 + row, a.own_stat_pad - 1);
      const long long soff = ((long long)b * a.Hq + h_own) * a.own_stat_pad + r;
      row_nl = a.own_lse2[soff];
      row_d = a.own_delta[soff];
    }

    int t = 0;
    for (int s = 0; s < a.nseg && ok; ++s) {
      const int f = ctl->seg_first[s], l = ctl->seg_last[s];
      const int seg_off = a.seg_off[s];
      for (int g = 0; g < n_sub && ok; ++g) {
        for (int st = f; st < l; ++st, ++t) {
          const int buf = t & 1, stage = t % kBwdStages;
          ok = mbar_wait_warp(&ctl->xy_full[buf], (t >> 1) & 1, abort_word, MB_ERR_TIMEOUT_S, a.wait_cycles);
          if (!ok) break;
          // the stage's statistics arrived with the stream tile (completed long ago; cheap re-check)
          if (a.mode_dkv) {
            ok = mbar_wait_warp(&ctl->str_full[stage], (t / kBwdStages) & 1, abort_word, MB_ERR_TIMEOUT_KV_FULL, a.wait_cycles);
            if (!ok) break;
          }
          tc_fence_after();
          const uint32_t tx = tmem + 256 + buf * 128 + lane_field, ty = tx + 64;
          uint32_t xr[32], yr[32];
          tmem_ld32(tx + half * 32, xr);
          tmem_ld32(ty + half * 32, yr);
          tmem_wait_ld();

          const int c0 = st * kStrRows + half * 32;  // first stream row (local to the segment) of my columns
          // causal limits on my 32 columns: dKV mode masks queries before the key, dQ mode keys after the query
          int lo = 0, hi = 32;
          if (a.causal) {
            if (a.mode_dkv) lo = own_pos - (seg_off + c0);        // query c visible iff seg_off+c0+c >= own_pos
            else hi = own_pos - (seg_off + c0) + 1;               // key c visible iff seg_off+c0+c <= own_pos
          }
          const bool need_mask = __any_sync(0xffffffffu, lo > 0 || hi < 32);  // only steps crossing the diagonal
          const float* stats = reinterpret_cast<const float*>(sStage + stage * kBwdStageBytes + 2 * kStrTileBytes);
          const float* nl_col = stats + half * 32;            // -lse2 of my 32 columns (dKV mode)
          const float* d_col = stats + kStrRows + half * 32;  // delta of my 32 columns
          uint32_t pk[16], dk[16];
          if (dkv_mode) {
            if (need_mask) ew_compute<true, true>(xr, yr, pk, dk, a.scale_log2, nl_col, d_col, 0.f, 0.f, lo, hi);
            else ew_compute<true, false>(xr, yr, pk, dk, a.scale_log2, nl_col, d_col, 0.f, 0.f, lo, hi);
          } else {
            if (need_mask) ew_compute<false, true>(xr, yr, pk, dk, a.scale_log2, nl_col, d_col, row_nl, row_d, lo, hi);
            else ew_compute<false, false>(xr, yr, pk, dk, a.scale_log2, nl_col, d_col, row_nl, row_d, lo, hi);
          }
          tmem_st16(tx + half * 32, pk);
          tmem_st16(ty + half * 32, dk);
          tmem_wait_st();
          tc_fence_before();
          mbar_arrive(&ctl->pd_full[buf]);
        }
      }
    }

    // epilogue: each warp stores its lane quarter x column half of the accumulators
    if (ok && own0 < a.own_rows) {
      const bool have = total_steps > 0;
      if (have) ok = mbar_wait_warp(&ctl->acc_full, 0, abort_word, MB_ERR_TIMEOUT_O, a.wait_cycles);
      if (ok) {
        if (have) tc_fence_after();
        const bool store = own0 + row < a.own_rows;
        const int n_out = a.mode_dkv ? 2 : 1;
        for (int which = 0; which < n_out; ++which) {
          void* base = which ? a.out2 : a.out1;
          const float mul = which ? 1.f : a.scale;  // dK and dQ carry the softmax scale, dV does not
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
// preprocess: delta = rowsum(dO * O), lse2 = -lse * log2(e)  ->  [B, Hq, pad] fp32 each
// ---------------------------------------------------------------------------
struct PreArgs {
  const __nv_bfloat16* dout;
  const __nv_bfloat16* out;
  long long do_sb, do_ss, do_sh, o_sb, o_ss, o_sh;
  const float* lse;  // [B,Hq,Sq]
  float* lse2;       // [B,Hq,pad]
  float* delta;      // [B,Hq,pad]
  int B, Sq, Hq, pad;
};

// One warp per (b, h, row); a block covers 8 consecutive rows of one (b, h).
__global__ void __launch_bounds__(256) bwd_preprocess_kernel(const PreArgs a) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int row = blockIdx.x * 8 + w;
  const int h = blockIdx.y, b = blockIdx.z;
  if (row >= a.pad) return;
  const long long sidx = ((long long)b * a.Hq + h) * a.pad + row;
  if (row >= a.Sq) {
    if (lane == 0) {
      a.lse2[sidx] = -INFINITY;
      a.delta[sidx] = 0.f;
    }
    return;
  }
  const uint2 dv = *reinterpret_cast<const uint2*>(a.dout + b * a.do_sb + row * a.do_ss + h * a.do_sh + lane * 4);
  const uint2 ov = *reinterpret_cast<const uint2*>(a.out + b * a.o_sb + row * a.o_ss + h * a.o_sh + lane * 4);
  float acc = __uint_as_float(dv.x << 16) * __uint_as_float(ov.x << 16) +
              __uint_as_float(dv.x & 0xffff0000u) * __uint_as_float(ov.x & 0xffff0000u) +
              __uint_as_float(dv.y << 16) * __uint_as_float(ov.y << 16) +
              __uint_as_float(dv.y & 0xffff0000u) * __uint_as_float(ov.y & 0xffff0000u);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) {
    const float l = a.lse[((long long)b * a.Hq + h) * a.Sq + row];
    a.lse2[sidx] = (l == -INFINITY) ? -INFINITY : -l * 1.4426950408889634f;
    a.delta[sidx] = acc;
  }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
static int make_map(CUtensorMap* map, const void* ptr, int H, int S, int B, long long sb, long long ss, long long sh,
                    int box_rows) {
  cuuint64_t dims[4] = {(cuuint64_t)kBD, (cuuint64_t)H, (cuuint64_t)S, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)sh * 2, (cuuint64_t)ss * 2, (cuuint64_t)sb * 2};
  cuuint32_t box[4] = {64, 1, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  return encode_tiled_bf16(map, const_cast<void*>(ptr), 4, dims, strides, box, estr);
}

static int set_smem_attr_once() {
  static bool done[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return MB_E_CUDA;
  if (dev >= 0 && dev < 64 && !done[dev]) {
    if (cudaFuncSetAttribute(attn_bwd_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, kBwdSmemBytes) !=
        cudaSuccess)
      return MB_E_CUDA;
    done[dev] = true;
  }
  return MB_SUCCESS;
}

int launch_bwd_preprocess(const mb_bwd_preprocess_args* x, cudaStream_t stream) {
  if (x == nullptr || x->dout == nullptr || x->out == nullptr || x->lse == nullptr || x->lse2 == nullptr ||
      x->delta == nullptr)
    return MB_E_INVALID;
  if (x->head_dim != kBD) return MB_E_UNSUPPORTED;
  if (x->batch <= 0 || x->hq <= 0 || x->sq < 0 || x->stat_pad < x->sq || x->stat_pad % kStrRows != 0)
    return MB_E_INVALID;
  if (x->stat_pad == 0) return MB_SUCCESS;
  PreArgs a;
  a.dout = static_cast<const __nv_bfloat16*>(x->dout);
  a.out = static_cast<const __nv_bfloat16*>(x->out);
  a.do_sb = x->dout_stride_b; a.do_ss = x->dout_stride_s; a.do_sh = x->dout_stride_h;
  a.o_sb = x->out_stride_b; a.o_ss = x->out_stride_s; a.o_sh = x->out_stride_h;
  a.lse = x->lse; a.lse2 = x->lse2; a.delta = x->delta;
  a.B = x->batch; a.Sq = x->sq; a.Hq = x->hq; a.pad = x->stat_pad;
  dim3 grid((x->stat_pad + 7) / 8, x->hq, x->batch);
  bwd_preprocess_kernel<<<grid, 256, 0, stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? MB_SUCCESS : MB_E_CUDA;
}

int launch_attn_bwd(const mb_attn_bwd_args* x, cudaStream_t stream) {
  if (x == nullptr) return MB_E_INVALID;
  if (x->head_dim != kBD) return MB_E_UNSUPPORTED;
  if (x->batch <= 0 || x->hq <= 0 || x->hkv <= 0 || x->hq % x->hkv != 0) return MB_E_INVALID;
  if (x->nseg < 0 || x->nseg > MB_MAX_SEGMENTS || x->own_rows < 0) return MB_E_INVALID;
  if (x->out_mode < 0 || x->out_mode > 2) return MB_E_INVALID;
  if (x->own_rows == 0) return MB_SUCCESS;
  if (x->own == nullptr || x->own_g == nullptr || x->out1 == nullptr) return MB_E_INVALID;
  const bool fused = x->mode == MB_BWD_MODE_FUSED;
  const bool dkv = x->mode == MB_BWD_MODE_DKV || fused;
  if (!dkv && x->mode != MB_BWD_MODE_DQ) return MB_E_INVALID;
  if (dkv && x->out2 == nullptr) return MB_E_INVALID;
  if (!dkv && (x->own_lse2 == nullptr || x->own_delta == nullptr || x->own_stat_pad < x->own_rows))
    return MB_E_INVALID;
  int rc = set_smem_attr_once();
  if (rc != MB_SUCCESS) return rc;

  static thread_local BwdMaps maps;  // 8.4 KB of tensor maps: the launch copies them
  static thread_local BwdArgs a;
  memset(&a, 0, sizeof(a));
  a.peer_wait_cycles = peer_wait_cycles();
  const int h_own = dkv ? x->hkv : x->hq;
  const int h_str = dkv ? x->hq : x->hkv;
  if (make_map(&maps.own, x->own, h_own, x->own_rows, x->batch, x->own_stride_b, x->own_stride_s, x->own_stride_h,
               kOwnRows) ||
      make_map(&maps.own_g, x->own_g, h_own, x->own_rows, x->batch, x->own_stride_b, x->own_stride_s,
               x->own_stride_h, kOwnRows))
    return MB_E_TENSORMAP;
  int nseg = 0;
  for (int s = 0; s < x->nseg; ++s) {
    const mb_bwd_segment& g = x->seg[s];
    if (g.rows < 0) return MB_E_INVALID;
    if (g.rows == 0) continue;
    if (g.str == nullptr || g.str_g == nullptr) return MB_E_INVALID;
    if (dkv && (g.lse2 == nullptr || g.delta == nullptr || g.stat_pad < g.rows || g.stat_pad % kStrRows != 0))
      return MB_E_INVALID;
    if (fused && g.dq_accum == nullptr) return MB_E_INVALID;
    if (make_map(&maps.str[nseg], g.str, h_str, g.rows, x->batch, g.stride_b, g.stride_s, g.stride_h, kStrRows) ||
        make_map(&maps.str_g[nseg], g.str_g, h_str, g.rows, x->batch, g.stride_b, g.stride_s, g.stride_h, kStrRows))
      return MB_E_TENSORMAP;
    a.seg_rows[nseg] = g.rows;
    a.seg_off[nseg] = g.pos_off;
    a.seg_lse2[nseg] = g.lse2;
    a.seg_delta[nseg] = g.delta;
    a.seg_stat_pad[nseg] = g.stat_pad;
    a.seg_dq[nseg] = g.dq_accum;
    a.seg_flag[nseg] = g.ready_flag;
    a.seg_flag_value[nseg] = g.ready_value;
    ++nseg;
  }
  a.nseg = nseg;
  bool has_flags = false;
  for (int s = 0; s < nseg; ++s) has_flags |= a.seg_flag[s] != nullptr;
  a.wait_cycles = kWaitCycleLimit + (has_flags ? a.peer_wait_cycles : 0);
  a.mode_dkv = dkv ? 1 : 0;
  a.B = x->batch;
  a.own_rows = x->own_rows;
  a.Hq = x->hq;
  a.Hkv = x->hkv;
  a.group = x->hq / x->hkv;
  a.own_off = x->own_off;
  a.causal = x->causal ? 1 : 0;
  a.scale = x->softmax_scale;
  a.scale_log2 = x->softmax_scale * 1.4426950408889634f;
  a.own_lse2 = x->own_lse2;
  a.own_delta = x->own_delta;
  a.own_stat_pad = x->own_stat_pad;
  a.out1 = x->out1;
  a.out2 = x->out2;
  a.o_sb = x->out_stride_b;
  a.o_ss = x->out_stride_s;
  a.o_sh = x->out_stride_h;
  a.out_mode = x->out_mode;
  a.status = x->status ? x->status : default_status_word();
  if (a.status == nullptr) return MB_E_CUDA;

  dim3 grid((x->own_rows + kOwnRows - 1) / kOwnRows, h_own, x->batch);
  if (fused) return launch_attn_bwd_fused(maps, a, grid, stream);
  attn_bwd_kernel<0><<<grid, kBwdThreads, kBwdSmemBytes, stream>>>(maps, a);
  return cuda_ok(cudaGetLastError(), "launch attn_bwd_kernel") ? MB_SUCCESS : MB_E_CUDA;
}

// ---------------------------------------------------------------------------
// allocation-free block backward
// ---------------------------------------------------------------------------
// Row statistics (lse2, delta) for the allocation-free entry point live in this fixed array
// instead of caller-provided memory: 2 x 1 Mi floats = 8 MiB, held by every GPU that loads
// the library until the process exits.
constexpr long long kStaticStatRows = 1ll << 20;  // batch * hq * pad64(sq) must not exceed this
static __device__ __align__(256) float g_bwd_static_stats[2 * kStaticStatRows];

// Host code cannot use the array's name as an address (it is only a stand-in on the host side):
// look the device address up once per device, with that device current.
static float* static_stats_address(int* rc) {
  static float* cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    *rc = MB_E_CUDA;
    return nullptr;
  }
  if (cached[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_bwd_static_stats) != cudaSuccess || p == nullptr) {
      *rc = MB_E_CUDA;
      return nullptr;
    }
    cached[dev] = static_cast<float*>(p);
  }
  *rc = MB_SUCCESS;
  return cached[dev];
}

int launch_bwd_block_noalloc(const mb_attn_bwd_block_args* x, cudaStream_t stream) {
  if (x == nullptr) return MB_E_INVALID;
  if (x->head_dim != kBD) return MB_E_UNSUPPORTED;
  if (x->batch <= 0 || x->hq <= 0 || x->hkv <= 0 || x->hq % x->hkv != 0 || x->sq < 0 || x->sk < 0) return MB_E_INVALID;
  if (x->out_mode != MB_OUT_BF16 && x->out_mode != MB_OUT_F32) return MB_E_INVALID;
  if (x->dout == nullptr || x->q == nullptr || x->k == nullptr || x->v == nullptr || x->out == nullptr ||
      x->lse == nullptr || x->dq == nullptr || x->dk == nullptr || x->dv == nullptr)
    return MB_E_INVALID;
  const long long pad = (x->sq + kStrRows - 1) / kStrRows * (long long)kStrRows;
  const long long rows = (long long)x->batch * x->hq * (pad > 0 ? pad : kStrRows);
  if (rows > kStaticStatRows) return MB_E_TOO_LARGE;
  if (x->sq == 0 && x->sk == 0) return MB_SUCCESS;
  int rc = MB_SUCCESS;
  float* stats = static_stats_address(&rc);
  if (stats == nullptr) return rc;
  const int stat_pad = static_cast<int>(pad > 0 ? pad : kStrRows);
  float* lse2 = stats;
  float* delta = stats + kStaticStatRows;

  if (x->sq > 0) {
    mb_bwd_preprocess_args p;
    memset(&p, 0, sizeof(p));
    p.dout = x->dout; p.dout_stride_b = x->q_stride_b; p.dout_stride_s = x->q_stride_s; p.dout_stride_h = x->q_stride_h;
    p.out = x->out; p.out_stride_b = x->q_stride_b; p.out_stride_s = x->q_stride_s; p.out_stride_h = x->q_stride_h;
    p.lse = x->lse; p.lse2 = lse2; p.delta = delta;
    p.batch = x->batch; p.sq = x->sq; p.hq = x->hq; p.head_dim = x->head_dim; p.stat_pad = stat_pad;
    rc = launch_bwd_preprocess(&p, stream);
    if (rc != MB_SUCCESS) return rc;
  }

  mb_attn_bwd_args a;
  memset(&a, 0, sizeof(a));
  a.batch = x->batch; a.hq = x->hq; a.hkv = x->hkv; a.head_dim = x->head_dim;
  a.causal = x->causal; a.softmax_scale = x->softmax_scale; a.out_mode = x->out_mode; a.status = x->status;
  // dQ: owner = q/dout, stream = k/v
  a.mode = MB_BWD_MODE_DQ;
  a.own = x->q; a.own_g = x->dout;
  a.own_stride_b = x->q_stride_b; a.own_stride_s = x->q_stride_s; a.own_stride_h = x->q_stride_h;
  a.own_lse2 = lse2; a.own_delta = delta; a.own_stat_pad = stat_pad;
  a.own_rows = x->sq; a.own_off = x->q_off;
  a.out1 = x->dq; a.out2 = nullptr;
  a.out_stride_b = x->dq_stride_b; a.out_stride_s = x->dq_stride_s; a.out_stride_h = x->dq_stride_h;
  a.nseg = 1;
  a.seg[0].str = x->k; a.seg[0].str_g = x->v;
  a.seg[0].stride_b = x->kv_stride_b; a.seg[0].stride_s = x->kv_stride_s; a.seg[0].stride_h = x->kv_stride_h;
  a.seg[0].rows = x->sk; a.seg[0].pos_off = x->k_off;
  rc = launch_attn_bwd(&a, stream);
  if (rc != MB_SUCCESS) return rc;
  // dK/dV: owner = k/v, stream = q/dout with the statistics just computed
  a.mode = MB_BWD_MODE_DKV;
  a.own = x->k; a.own_g = x->v;
  a.own_stride_b = x->kv_stride_b; a.own_stride_s = x->kv_stride_s; a.own_stride_h = x->kv_stride_h;
  a.own_lse2 = nullptr; a.own_delta = nullptr; a.own_stat_pad = 0;
  a.own_rows = x->sk; a.own_off = x->k_off;
  a.out1 = x->dk; a.out2 = x->dv;
  a.out_stride_b = x->dkv_stride_b; a.out_stride_s = x->dkv_stride_s; a.out_stride_h = x->dkv_stride_h;
  a.seg[0].str = x->q; a.seg[0].str_g = x->dout;
  a.seg[0].stride_b = x->q_stride_b; a.seg[0].stride_s = x->q_stride_s; a.seg[0].stride_h = x->q_stride_h;
  a.seg[0].rows = x->sq; a.seg[0].pos_off = x->q_off;
  a.seg[0].lse2 = lse2; a.seg[0].delta = delta; a.seg[0].stat_pad = stat_pad;
  return launch_attn_bwd(&a, stream);
}

}  // namespace mb
