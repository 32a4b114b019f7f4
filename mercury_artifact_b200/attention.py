"""Tensor-level wrappers over the C ABI: forward attention over K/V segments.

Tensors are torch CUDA tensors; torch is used for memory and streams only.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence, Tuple

import torch

from . import _lib


def _stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def _check_bshd(t: torch.Tensor, name: str) -> None:
    if t.dim() != 4:
        raise ValueError(f"{name} must be [batch, seq, heads, head_dim], got {tuple(t.shape)}")
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if t.dtype != torch.bfloat16:
        raise TypeError(f"{name} must be bfloat16, got {t.dtype}")
    if t.stride(3) != 1:
        raise ValueError(f"{name}: head_dim must be contiguous")


def attn_fwd_segments(
    q: torch.Tensor,
    segments: Sequence[tuple],
    softmax_scale: float,
    causal: bool = False,
    q_off: int = 0,
    out: Optional[torch.Tensor] = None,
    lse: Optional[torch.Tensor] = None,
    out_raw: Optional[tuple] = None,
    lse_raw: Optional[tuple] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """softmax(scale * q k^T) v over the concatenation of `segments`.

    out_raw = (address, stride_b, stride_s, stride_h) and lse_raw = (address, stride_b, stride_h)
    direct the results to raw device addresses instead of tensors (for example another rank's
    memory mapped into this process); the function then returns (None, None).

    segments: (k, v, k_off) or (k, v, k_off, flag_ptr, flag_value) with k, v of shape
    [batch, sk, hkv, head_dim]; k_off is the global position of the shard's first key and
    matters only when `causal` (key visible iff k_off + j <= q_off + i); flag_ptr, when
    given, is the address of a device int32 that reaches flag_value once the shard has
    arrived (the kernel waits for it before reading the shard).  Returns
    (o bf16 [b, sq, hq, d], lse fp32 [b, hq, sq]).
    """
    _check_bshd(q, "q")
    b, sq, hq, d = q.shape
    if len(segments) > _lib.MB_MAX_SEGMENTS:
        raise ValueError(f"at most {_lib.MB_MAX_SEGMENTS} K/V segments per call")
    raw = out_raw is not None
    if raw != (lse_raw is not None):
        raise ValueError("out_raw and lse_raw go together")
    if not raw:
        if out is None:
            out = torch.empty_like(q)
        else:
            _check_bshd(out, "out")
        if lse is None:
            lse = torch.empty((b, hq, sq), dtype=torch.float32, device=q.device)
        elif lse.dtype != torch.float32 or lse.stride(2) != 1 or tuple(lse.shape) != (b, hq, sq):
            raise ValueError("lse must be an fp32 [batch, hq, sq] tensor with contiguous rows")
        out_raw = (out.data_ptr(), out.stride(0), out.stride(1), out.stride(2))
        lse_raw = (lse.data_ptr(), lse.stride(0), lse.stride(1))

    args = _lib.AttnFwdArgs()
    args.q = q.data_ptr()
    args.q_stride_b, args.q_stride_s, args.q_stride_h = q.stride(0), q.stride(1), q.stride(2)
    args.o, args.o_stride_b, args.o_stride_s, args.o_stride_h = out_raw
    args.lse, args.lse_stride_b, args.lse_stride_h = lse_raw
    args.batch, args.sq, args.hq, args.head_dim = b, sq, hq, d
    args.q_off = int(q_off)
    args.causal = 1 if causal else 0
    args.softmax_scale = float(softmax_scale)
    args.nseg = len(segments)
    args.status = None
    hkv = None
    for i, segment in enumerate(segments):
        k, v, k_off = segment[:3]
        flag_ptr, flag_value = (segment[3], segment[4]) if len(segment) >= 5 and segment[3] else (None, 0)
        _check_bshd(k, "k")
        _check_bshd(v, "v")
        if k.shape != v.shape or k.stride() != v.stride():
            raise ValueError("k and v of one segment must share shape and strides")
        if k.shape[0] != b or k.shape[3] != d:
            raise ValueError("segment batch/head_dim mismatch with q")
        if hkv is None:
            hkv = k.shape[2]
        elif hkv != k.shape[2]:
            raise ValueError("all segments must have the same number of K/V heads")
        seg = args.seg[i]
        seg.k, seg.v = k.data_ptr(), v.data_ptr()
        seg.stride_b, seg.stride_s, seg.stride_h = k.stride(0), k.stride(1), k.stride(2)
        seg.sk = k.shape[1]
        seg.k_off = int(k_off)
        seg.ready_flag = flag_ptr
        seg.ready_value = int(flag_value)
    args.hkv = hkv if hkv is not None else hq
    with torch.cuda.device(q.device):
        _lib.check(_lib.lib.mb_attn_fwd(C.byref(args), C.c_void_p(_stream_ptr())), "mb_attn_fwd")
    return (None, None) if raw else (out, lse)


def attn_fwd_multi(jobs: Sequence[dict], segments: Sequence[tuple], softmax_scale: float, causal: bool,
                   batch: int, hq: int, hkv: int, head_dim: int, device: torch.device) -> None:
    """Several query shards against one list of K/V segments in ONE launch (mb_attn_fwd_multi).

    jobs: dicts with
      q            tensor [batch, sq, hq, d] (a view is fine)
      q_off        global position of its row 0
      out_raw      (address, stride_b, stride_s, stride_h) of the bf16 result, lse_raw (address, stride_b,
                   stride_h) of the fp32 log-sum-exp -- raw addresses, so that they can point into another
                   rank's memory mapped into this process
      q_flag       optional (address, value): arrival flag of the query shard
      done         optional (flag address, value, counter address): completion flag raised by the kernel
      seg_mask     optional bit mask of the segments the job attends to (default: all)
      state        optional (state_o, state_ml): fp32 tensors [batch, hq, sq, d] and [batch, hq, sq, 2] that
                   carry the online-softmax state between jobs over the same query rows
      state_in / state_out   start from that state / store it instead of the result (out_raw and lse_raw
                   may then be omitted)
      chain        optional (address of int32 words [batch, hq, ceil(sq/256)], wait value, set value): lets
                   the job that continues a state be part of the same launch (later in `jobs`)
    segments: as in attn_fwd_segments.  CTAs are dispatched job by job, job 0 first."""
    if not 1 <= len(jobs) <= _lib.MB_MAX_JOBS:
        raise ValueError(f"1..{_lib.MB_MAX_JOBS} jobs per launch")
    if len(segments) > _lib.MB_MAX_SEGMENTS:
        raise ValueError(f"at most {_lib.MB_MAX_SEGMENTS} K/V segments per call")
    a = _lib.AttnFwdMultiArgs()
    a.batch, a.hq, a.hkv, a.head_dim = batch, hq, hkv, head_dim
    a.causal = 1 if causal else 0
    a.softmax_scale = float(softmax_scale)
    a.njobs, a.nseg = len(jobs), len(segments)
    a.status = None
    for i, jb in enumerate(jobs):
        q = jb["q"]
        _check_bshd(q, "q")
        if q.shape[0] != batch or q.shape[2] != hq or q.shape[3] != head_dim:
            raise ValueError("job q does not match batch / hq / head_dim")
        j = a.job[i]
        j.q = q.data_ptr()
        j.q_stride_b, j.q_stride_s, j.q_stride_h = q.stride(0), q.stride(1), q.stride(2)
        if jb.get("out_raw") is not None:
            j.o, j.o_stride_b, j.o_stride_s, j.o_stride_h = jb["out_raw"]
            j.lse, j.lse_stride_b, j.lse_stride_h = jb["lse_raw"]
        elif not jb.get("state_out"):
            raise ValueError("a job needs out_raw / lse_raw unless it stores its state")
        if jb.get("state") is not None:
            so, sml = jb["state"]
            if so.dtype != torch.float32 or sml.dtype != torch.float32 or not so.is_contiguous() or \
                    not sml.is_contiguous() or tuple(so.shape) != (batch, hq, q.shape[1], head_dim) or \
                    tuple(sml.shape) != (batch, hq, q.shape[1], 2):
                raise ValueError("state must be contiguous fp32 [batch, hq, sq, d] and [batch, hq, sq, 2]")
            j.state_o, j.state_ml = so.data_ptr(), sml.data_ptr()
            j.state_in, j.state_out = int(bool(jb.get("state_in"))), int(bool(jb.get("state_out")))
            if jb.get("chain"):
                j.chain, j.chain_wait, j.chain_set = jb["chain"][0], int(jb["chain"][1]), int(jb["chain"][2])
        elif jb.get("state_in") or jb.get("state_out"):
            raise ValueError("state_in / state_out need the state tensors")
        j.sq, j.q_off = q.shape[1], int(jb.get("q_off", 0))
        j.seg_mask = int(jb.get("seg_mask", 0))
        if jb.get("q_flag"):
            j.q_ready_flag, j.q_ready_value = jb["q_flag"][0], int(jb["q_flag"][1])
        if jb.get("done"):
            j.done_flag, j.done_value, j.done_counter = jb["done"][0], int(jb["done"][1]), jb["done"][2]
    for i, segment in enumerate(segments):
        k, v, k_off = segment[:3]
        flag_ptr, flag_value = (segment[3], segment[4]) if len(segment) >= 5 and segment[3] else (None, 0)
        _check_bshd(k, "k")
        _check_bshd(v, "v")
        if k.shape != v.shape or k.stride() != v.stride():
            raise ValueError("k and v of one segment must share shape and strides")
        if k.shape[0] != batch or k.shape[2] != hkv or k.shape[3] != head_dim:
            raise ValueError("segment does not match batch / hkv / head_dim")
        seg = a.seg[i]
        seg.k, seg.v = k.data_ptr(), v.data_ptr()
        seg.stride_b, seg.stride_s, seg.stride_h = k.stride(0), k.stride(1), k.stride(2)
        seg.sk, seg.k_off = k.shape[1], int(k_off)
        seg.ready_flag, seg.ready_value = flag_ptr, int(flag_value)
    with torch.cuda.device(device):
        _lib.check(_lib.lib.mb_attn_fwd_multi(C.byref(a), C.c_void_p(_stream_ptr())), "mb_attn_fwd_multi")


# ------------------------------------------------------------------------------------------
# backward
# ------------------------------------------------------------------------------------------
class RowStats:
    """lse2 = -lse*log2(e) (stored negated) and delta = rowsum(dout*out) of one query shard, padded to 64 rows."""

    def __init__(self, lse2: torch.Tensor, delta: torch.Tensor, rows: int, pad: Optional[int] = None):
        self.lse2, self.delta, self.rows = lse2, delta, rows
        # row pitch of the [batch, hq, pad] arrays; a view that starts at a later row keeps the pitch
        self.pad = lse2.shape[-1] if pad is None else pad


def _pad64(n: int) -> int:
    return max(64, (n + 63) // 64 * 64)


def bwd_preprocess(dout: torch.Tensor, out: torch.Tensor, lse: torch.Tensor,
                   workspace: Optional[torch.Tensor] = None) -> RowStats:
    """Per-row statistics for the backward kernels.  `out` and `lse` are the FINAL forward results
    of these query rows.  workspace: optional fp32 [2, batch, hq, pad64(sq)] to write into."""
    _check_bshd(dout, "dout")
    _check_bshd(out, "out")
    b, sq, hq, d = dout.shape
    pad = _pad64(sq)
    if workspace is None:
        workspace = torch.empty((2, b, hq, pad), dtype=torch.float32, device=dout.device)
    elif tuple(workspace.shape) != (2, b, hq, pad) or workspace.dtype != torch.float32 or not workspace.is_contiguous():
        raise ValueError(f"workspace must be contiguous fp32 {(2, b, hq, pad)}")
    lse = lse.contiguous()
    if tuple(lse.shape) != (b, hq, sq) or lse.dtype != torch.float32:
        raise ValueError("lse must be fp32 [batch, hq, sq]")
    a = _lib.BwdPreprocessArgs()
    a.dout = dout.data_ptr()
    a.dout_stride_b, a.dout_stride_s, a.dout_stride_h = dout.stride(0), dout.stride(1), dout.stride(2)
    a.out = out.data_ptr()
    a.out_stride_b, a.out_stride_s, a.out_stride_h = out.stride(0), out.stride(1), out.stride(2)
    a.lse, a.lse2, a.delta = lse.data_ptr(), workspace[0].data_ptr(), workspace[1].data_ptr()
    a.batch, a.sq, a.hq, a.head_dim, a.stat_pad = b, sq, hq, d, pad
    with torch.cuda.device(dout.device):
        _lib.check(_lib.lib.mb_attn_bwd_preprocess(C.byref(a), C.c_void_p(_stream_ptr())), "mb_attn_bwd_preprocess")
    return RowStats(workspace[0], workspace[1], sq)


_OUT_MODES = {torch.bfloat16: _lib.MB_OUT_BF16, torch.float32: _lib.MB_OUT_F32}


def _bwd_launch(mode, own, own_g, own_off, segments, hq, hkv, scale, causal, out1, out2, accumulate, own_stats=None):
    """One mb_attn_bwd launch.  Segment dicts: str, str_g, off, optional stats (RowStats), flag / flag_value,
    and dq_accum (fp32 tensor, single-pass mode)."""
    _check_bshd(own, "owner")
    _check_bshd(own_g, "owner_g")
    if own.shape != own_g.shape or own.stride() != own_g.stride():
        raise ValueError("the two owner tensors must share shape and strides")
    if len(segments) > _lib.MB_MAX_SEGMENTS:
        raise ValueError(f"at most {_lib.MB_MAX_SEGMENTS} segments per call")
    b, rows, _, d = own.shape
    a = _lib.AttnBwdArgs()
    a.mode = mode
    if out1.dtype not in _OUT_MODES:
        raise TypeError("gradient outputs must be bf16 or fp32")
    if accumulate and out1.dtype != torch.float32:
        raise TypeError("accumulation needs fp32 gradient buffers")
    a.out_mode = _lib.MB_OUT_F32_ACCUM if accumulate else _OUT_MODES[out1.dtype]
    a.own, a.own_g = own.data_ptr(), own_g.data_ptr()
    a.own_stride_b, a.own_stride_s, a.own_stride_h = own.stride(0), own.stride(1), own.stride(2)
    if own_stats is not None:
        a.own_lse2, a.own_delta, a.own_stat_pad = own_stats.lse2.data_ptr(), own_stats.delta.data_ptr(), own_stats.pad
    a.own_rows, a.own_off = rows, int(own_off)
    a.batch, a.hq, a.hkv, a.head_dim = b, hq, hkv, d
    a.causal = 1 if causal else 0
    a.softmax_scale = float(scale)
    a.out1 = out1.data_ptr()
    if out2 is not None:
        if out2.shape != out1.shape or out2.stride() != out1.stride() or out2.dtype != out1.dtype:
            raise ValueError("dk and dv must share shape, strides and dtype")
        a.out2 = out2.data_ptr()
    if out1.stride(3) != 1 or tuple(out1.shape) != tuple(own.shape):
        raise ValueError("gradient output must match the owner's shape with a contiguous head_dim")
    a.out_stride_b, a.out_stride_s, a.out_stride_h = out1.stride(0), out1.stride(1), out1.stride(2)
    a.nseg = len(segments)
    for i, sg in enumerate(segments):
        s, s_g, off = sg["str"], sg["str_g"], sg["off"]
        _check_bshd(s, "stream")
        _check_bshd(s_g, "stream_g")
        if s.shape != s_g.shape or s.stride() != s_g.stride():
            raise ValueError("the two stream tensors of a segment must share shape and strides")
        seg = a.seg[i]
        seg.str, seg.str_g = s.data_ptr(), s_g.data_ptr()
        seg.stride_b, seg.stride_s, seg.stride_h = s.stride(0), s.stride(1), s.stride(2)
        seg.rows, seg.pos_off = s.shape[1], int(off)
        st = sg.get("stats")
        if st is not None:
            seg.lse2, seg.delta, seg.stat_pad = st.lse2.data_ptr(), st.delta.data_ptr(), st.pad
        if sg.get("flag"):
            seg.ready_flag, seg.ready_value = sg["flag"], int(sg["flag_value"])
        if sg.get("dq_accum") is not None:
            acc = sg["dq_accum"]
            if acc.dtype != torch.float32 or not acc.is_contiguous() or tuple(acc.shape) != (b, hq, seg.stat_pad, d):
                raise ValueError(f"dq_accum must be contiguous fp32 {(b, hq, seg.stat_pad, d)}")
            seg.dq_accum = acc.data_ptr()
    with torch.cuda.device(own.device):
        _lib.check(_lib.lib.mb_attn_bwd(C.byref(a), C.c_void_p(_stream_ptr())), "mb_attn_bwd")


def attn_bwd_dq(q, dout, stats: RowStats, kv_segments, softmax_scale, causal=False, q_off=0, dq=None,
                accumulate=False, hkv=None):
    """dQ of one query shard against K/V segments [(k, v, k_off) or dicts]; dq bf16/fp32 like q."""
    if dq is None:
        dq = torch.empty_like(q)
    segs = []
    for sg in kv_segments:
        if isinstance(sg, dict):
            segs.append(sg)
        else:
            segs.append({"str": sg[0], "str_g": sg[1], "off": sg[2],
                         "flag": sg[3] if len(sg) > 3 else None, "flag_value": sg[4] if len(sg) > 4 else 0})
    hkv = hkv if hkv is not None else (segs[0]["str"].shape[2] if segs else q.shape[2])
    _bwd_launch(_lib.MB_BWD_MODE_DQ, q, dout, q_off, segs, q.shape[2], hkv, softmax_scale, causal, dq, None,
                accumulate, own_stats=stats)
    return dq


def attn_bwd_dkv(k, v, q_segments, softmax_scale, causal=False, k_off=0, dk=None, dv=None, accumulate=False, hq=None):
    """dK, dV of one K/V shard against query segments [(q, dout, stats, q_off[, flag, value])]."""
    if dk is None:
        dk = torch.empty_like(k)
    if dv is None:
        dv = torch.empty_like(v)
    segs = []
    for sg in q_segments:
        if isinstance(sg, dict):
            segs.append(sg)
        else:
            segs.append({"str": sg[0], "str_g": sg[1], "stats": sg[2], "off": sg[3],
                         "flag": sg[4] if len(sg) > 4 else None, "flag_value": sg[5] if len(sg) > 5 else 0})
    hq = hq if hq is not None else (segs[0]["str"].shape[2] if segs else k.shape[2])
    _bwd_launch(_lib.MB_BWD_MODE_DKV, k, v, k_off, segs, hq, k.shape[2], softmax_scale, causal, dk, dv, accumulate)
    return dk, dv


def dq_convert_raw(dq_accum: torch.Tensor, dq_ptr: int, strides: Sequence[int], batch: int, sq: int, hq: int, pad: int,
                   softmax_scale: float, out_dtype=torch.bfloat16) -> None:
    """Finish a single-sweep backward: scale the fp32 dq accumulation [batch, hq, pad, d] and store it as
    [batch, sq, hq, d] rows at a raw address with element strides (batch, row, head) -- the address may
    be another rank's memory mapped into this process (mb_attn_bwd_dq_convert)."""
    with torch.cuda.device(dq_accum.device):
        _lib.check(_lib.lib.mb_attn_bwd_dq_convert(dq_accum.data_ptr(), dq_ptr, strides[0], strides[1], strides[2],
                                                   batch, sq, hq, pad, _OUT_MODES[out_dtype], float(softmax_scale),
                                                   C.c_void_p(_stream_ptr())),
                   "mb_attn_bwd_dq_convert")


def attn_bwd_fused(q, dout, stats: RowStats, k, v, softmax_scale, causal=False, q_off=0, k_off=0, dq=None, dk=None,
                   dv=None, dq_accum: Optional[torch.Tensor] = None):
    """dQ, dK, dV of one query shard against one K/V shard in a single sweep (MB_BWD_MODE_FUSED): scores
    and probabilities are computed once; the dQ contributions of every K/V tile are added into an fp32
    buffer (`dq_accum`, [batch, hq, pad64(sq), d], allocated and zeroed here unless given) and converted
    at the end.  The order of those additions varies, so dq is not bitwise reproducible run to run
    (dk and dv are); attn_bwd_dq + attn_bwd_dkv is the deterministic two-launch form."""
    if dq is None:
        dq = torch.empty_like(q)
    if dk is None:
        dk = torch.empty_like(k)
    if dv is None:
        dv = torch.empty_like(v)
    b, sq, hq, d = q.shape
    if dq_accum is None:
        dq_accum = torch.zeros((b, hq, stats.pad, d), dtype=torch.float32, device=q.device)
    seg = {"str": q, "str_g": dout, "stats": stats, "off": q_off, "dq_accum": dq_accum}
    _bwd_launch(_lib.MB_BWD_MODE_FUSED, k, v, k_off, [seg], hq, k.shape[2], softmax_scale, causal, dk, dv, False)
    if dq.dtype not in _OUT_MODES or dq.stride(3) != 1 or tuple(dq.shape) != tuple(q.shape):
        raise ValueError("dq must be bf16 or fp32, shaped like q, with a contiguous head_dim")
    with torch.cuda.device(q.device):
        _lib.check(_lib.lib.mb_attn_bwd_dq_convert(dq_accum.data_ptr(), dq.data_ptr(), dq.stride(0), dq.stride(1),
                                                   dq.stride(2), b, sq, hq, stats.pad, _OUT_MODES[dq.dtype],
                                                   float(softmax_scale), C.c_void_p(_stream_ptr())),
                   "mb_attn_bwd_dq_convert")
    return dq, dk, dv
