"""Drop-in ops under the names the generated code resolves at exec time.

The reference's DSL bodies call `_flash_attn_forward(**params)`,
`update_out_and_lse(...)` and `get_default_args(...)` as free names looked up in
the namespace handed to `exec` (example.py:153-156 of the reference).  The
functions here have the same names, keyword sets, return shapes and error
behaviour, and run on the sm_100a kernels of libmercury_b200.so.
"""
from __future__ import annotations

import ctypes as C
import inspect
from functools import lru_cache
from typing import Optional, Tuple

import torch

from . import _lib
from .attention import (_stream_ptr, attn_bwd_dkv, attn_bwd_dq, attn_bwd_fused, attn_fwd_segments,
                        bwd_preprocess)


# -- get_default_args -----------------------------------------------------------------------
@lru_cache(maxsize=None)
def _defaults_of(func):
    spec = inspect.getfullargspec(func)
    defaults = spec.defaults or ()
    values = (None,) * (len(spec.args) - len(defaults)) + tuple(defaults)
    table = dict(zip(spec.args, values))
    if "softcap" in table:
        table["softcap"] = 0.0
    return table


def get_default_args(func):
    """Argument-name -> default table of `func` (None where it has no default, softcap forced to
    0.0), like utils/flash_attn_dsl.py:14-29.  Custom-op wrappers are unwrapped via `_init_fn`."""
    return _defaults_of(func if inspect.isfunction(func) else func._init_fn)


def _reject_unsupported(dropout_p, window_size_left, window_size_right, softcap, alibi_slopes, causal=False):
    if dropout_p:
        raise NotImplementedError("dropout_p must be 0 (the ring schedules never set it)")
    # window_size_right == 0 is how flash-attn spells "causal" internally; without causal=True it would be
    # a window, which these kernels do not implement
    right_ok = (-1, 0, None) if causal else (-1, None)
    if window_size_left not in (-1, None) or window_size_right not in right_ok:
        raise NotImplementedError("sliding-window attention is not implemented")
    if softcap:
        raise NotImplementedError("softcap must be 0")
    if alibi_slopes is not None:
        raise NotImplementedError("alibi_slopes must be None")


# -- block forward --------------------------------------------------------------------------
def _flash_attn_forward(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    dropout_p: float,
    softmax_scale: float,
    causal: bool,
    window_size_left: int = -1,
    window_size_right: int = -1,
    softcap: float = 0.0,
    alibi_slopes: Optional[torch.Tensor] = None,
    return_softmax: bool = False,
) -> Tuple[torch.Tensor, torch.Tensor, None, None]:
    """Block attention forward, the per-step call of every generated loop
    (utils/flash_attn_dsl.py:174).  q [B,Sq,Hq,D], k/v [B,Sk,Hkv,D] bf16 ->
    (out like q, softmax_lse [B,Hq,Sq] fp32, None, None).

    causal=True aligns the mask to the bottom-right corner like the flash-attn op.
    Unlike flash-attn, a row without any visible key returns lse = -inf (not +inf).
    """
    _reject_unsupported(dropout_p, window_size_left, window_size_right, softcap, alibi_slopes, causal)
    if return_softmax:
        raise NotImplementedError("return_softmax is only meaningful with dropout")
    if softmax_scale is None:
        softmax_scale = q.shape[-1] ** -0.5
    q_off = k.shape[1] - q.shape[1] if causal else 0
    out, lse = attn_fwd_segments(q, [(k, v, 0)], softmax_scale, causal=bool(causal), q_off=q_off)
    return out, lse, None, None


# -- block backward -------------------------------------------------------------------------
def _flash_attn_backward(
    dout: torch.Tensor,
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    out: torch.Tensor,
    softmax_lse: torch.Tensor,
    dq: Optional[torch.Tensor],
    dk: Optional[torch.Tensor],
    dv: Optional[torch.Tensor],
    dropout_p: float,
    softmax_scale: float,
    causal: bool,
    window_size_left: int = -1,
    window_size_right: int = -1,
    softcap: float = 0.0,
    alibi_slopes: Optional[torch.Tensor] = None,
    deterministic: bool = False,
    rng_state: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Block attention backward, the per-step call of the generated backward loop
    (utils/attn_bwd_dsl.py:115).  Writes dq, dk, dv IN PLACE (dk/dv may be the two halves of
    a packed [2,...] buffer) and returns softmax_d = rowsum(dout * out) as [B, Hq, pad64(Sq)].
    `out` and `softmax_lse` are the final forward results of the query rows, which need not come
    from this K/V block alone.  deterministic=False (the generated code's default) runs the
    single-sweep kernel, whose dq depends on the order of fp32 additions; deterministic=True runs
    the two-launch form, which has no atomics and is bitwise reproducible."""
    _reject_unsupported(dropout_p, window_size_left, window_size_right, softcap, alibi_slopes, causal)
    if softmax_scale is None:
        softmax_scale = q.shape[-1] ** -0.5
    if dq is None:
        dq = torch.empty_like(q)
    if dk is None:
        dk = torch.empty_like(k)
    if dv is None:
        dv = torch.empty_like(v)
    q_off = k.shape[1] - q.shape[1] if causal else 0
    stats = bwd_preprocess(dout, out, softmax_lse)
    if deterministic or q.shape[1] == 0 or k.shape[1] == 0:
        attn_bwd_dq(q, dout, stats, [(k, v, 0)], softmax_scale, causal=bool(causal), q_off=q_off, dq=dq)
        attn_bwd_dkv(k, v, [(q, dout, stats, q_off)], softmax_scale, causal=bool(causal), k_off=0, dk=dk, dv=dv)
    else:
        attn_bwd_fused(q, dout, stats, k, v, softmax_scale, causal=bool(causal), q_off=q_off, k_off=0, dq=dq, dk=dk,
                       dv=dv)
    return stats.delta


# -- merge ----------------------------------------------------------------------------------
def _merge_launch(out, lse, block_out, block_lse, first: bool) -> None:
    b, s, h, d = out.shape
    if block_out.shape != out.shape:
        raise ValueError(f"block_out {tuple(block_out.shape)} does not match out {tuple(out.shape)}")
    if tuple(block_lse.shape) != (b, h, s):
        raise ValueError(f"block_lse must be [B,H,S] = {(b, h, s)}, got {tuple(block_lse.shape)}")
    if block_out.stride(3) != 1:
        block_out = block_out.contiguous()
    if block_out.dtype not in (torch.bfloat16, torch.float32):
        block_out = block_out.float()
    block_lse = block_lse.contiguous().float()
    a = _lib.MergeArgs()
    a.out, a.lse = out.data_ptr(), lse.data_ptr()
    a.block_out = block_out.data_ptr()
    a.block_stride_b, a.block_stride_s, a.block_stride_h = block_out.stride(0), block_out.stride(1), block_out.stride(2)
    a.block_lse = block_lse.data_ptr()
    a.batch, a.seq, a.heads, a.head_dim = b, s, h, d
    a.first = 1 if first else 0
    a.block_dtype = _lib.MB_DTYPE_F32 if block_out.dtype == torch.float32 else _lib.MB_DTYPE_BF16
    with torch.cuda.device(out.device):
        _lib.check(_lib.lib.mb_merge_out_lse(C.byref(a), C.c_void_p(_stream_ptr())), "mb_merge_out_lse")


def update_out_and_lse(
    out: Optional[torch.Tensor],
    lse: Optional[torch.Tensor],
    block_out: torch.Tensor,
    block_lse: torch.Tensor,
    slice_=None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Running merge with the reference's calling convention (utils/flash_attn_dsl.py:51-71):
    the first call (out is None) returns a fresh fp32 copy of the block and its LSE as
    [B,S,H,1]; later calls update the state IN PLACE and return it."""
    if not block_out.is_cuda:
        raise ValueError("update_out_and_lse: CUDA tensors only (there is no CPU path)")
    if out is None:
        if slice_ is not None:
            raise RuntimeError("first update_out_and_lse should not pass slice_ args")
        b, s, h, d = block_out.shape
        out = torch.empty((b, s, h, d), dtype=torch.float32, device=block_out.device)
        lse = torch.empty((b, s, h, 1), dtype=torch.float32, device=block_out.device)
        _merge_launch(out, lse, block_out, block_lse, first=True)
        return out, lse
    if slice_ is not None:
        so, sl = out[slice_], lse[slice_]
        if so.is_contiguous() and sl.is_contiguous():
            _merge_launch(so, sl, block_out, block_lse, first=False)
        else:
            co, cl = so.contiguous(), sl.contiguous()
            _merge_launch(co, cl, block_out, block_lse, first=False)
            out[slice_], lse[slice_] = co, cl
        return out, lse
    if not (out.is_contiguous() and lse.is_contiguous() and out.dtype == torch.float32):
        raise ValueError("update_out_and_lse: running state must be contiguous fp32")
    _merge_launch(out, lse, block_out, block_lse, first=False)
    return out, lse


def flash_reduce(lhs: torch.Tensor, rhs: torch.Tensor) -> torch.Tensor:
    """Merge of two packed fp32 [..., D+1] = [out | lse] buffers, the reduce op of the ring-over-Q
    schedule (utils/flash_attn_dsl.py:293-305).  Returns a new tensor, like the reference."""
    if not (lhs.is_cuda and rhs.is_cuda):
        raise ValueError("flash_reduce: CUDA tensors only (there is no CPU path)")
    if lhs.shape != rhs.shape or lhs.dtype != torch.float32 or rhs.dtype != torch.float32:
        raise ValueError("flash_reduce: both operands must be fp32 with the same [..., D+1] shape")
    lhs, rhs = lhs.contiguous(), rhs.contiguous()
    out = torch.empty_like(lhs)
    width = lhs.shape[-1]
    rows = lhs.numel() // width if width else 0
    with torch.cuda.device(lhs.device):
        _lib.check(_lib.lib.mb_flash_reduce(lhs.data_ptr(), rhs.data_ptr(), out.data_ptr(), rows, width,
                                            C.c_void_p(_stream_ptr())), "mb_flash_reduce")
    return out
