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
) -> Tuple[torch.Tensor, torch.Tensor]:
    """softmax(scale * q k^T) v over the concatenation of `segments`.

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
    if out is None:
        out = torch.empty_like(q)
    else:
        _check_bshd(out, "out")
    if lse is None:
        lse = torch.empty((b, hq, sq), dtype=torch.float32, device=q.device)
    elif lse.dtype != torch.float32 or not lse.is_contiguous() or tuple(lse.shape) != (b, hq, sq):
        raise ValueError("lse must be a contiguous fp32 [batch, hq, sq] tensor")

    args = _lib.AttnFwdArgs()
    args.q = q.data_ptr()
    args.q_stride_b, args.q_stride_s, args.q_stride_h = q.stride(0), q.stride(1), q.stride(2)
    args.o = out.data_ptr()
    args.o_stride_b, args.o_stride_s, args.o_stride_h = out.stride(0), out.stride(1), out.stride(2)
    args.lse = lse.data_ptr()
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
    return out, lse
