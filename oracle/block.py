"""Block attention forward/backward in fp32 on the CPU (test infrastructure).

Shapes follow the call sites of the reference (utils/flash_attn_dsl.py:160-176,
utils/attn_bwd_dsl.py:86-115): q [B, Sq, Hq, D]; k, v [B, Sk, Hkv, D] with
Hq = Hkv * group; out like q; lse [B, Hq, Sq] fp32 = ln sum_j exp(scale * q_i.k_j).
The block math itself is the third-party flash-attn op (not in the reference
tree); this is the published algorithm written out directly.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch


def _expand_kv(x: torch.Tensor, hq: int) -> torch.Tensor:
    """[B, S, Hkv, D] -> [B, Hq, S, D] fp32, each K/V head repeated for its query group."""
    hkv = x.shape[2]
    x = x.float().permute(0, 2, 1, 3)
    if hkv != hq:
        x = x.repeat_interleave(hq // hkv, dim=1)
    return x


def visibility(sq: int, sk: int, q_off: int, k_off: int, device=None) -> torch.Tensor:
    """[Sq, Sk] bool: key j visible to query i iff k_off + j <= q_off + i."""
    qpos = torch.arange(sq, device=device) + q_off
    kpos = torch.arange(sk, device=device) + k_off
    return kpos[None, :] <= qpos[:, None]


def block_attn_fwd(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    softmax_scale: float,
    causal: bool = False,
    q_off: Optional[int] = None,
    k_off: int = 0,
    q_chunk: int = 1024,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns (out in q.dtype, lse fp32 [B, Hq, Sq]).

    With causal=True and no offsets the mask is aligned to the bottom-right
    corner (q_off = Sk - Sq), the convention of the flash-attn op the reference
    calls.  A row that sees no key yields out = 0 and lse = -inf.
    """
    b, sq, hq, d = q.shape
    sk = k.shape[1]
    if q_off is None:
        q_off = sk - sq
    kf = _expand_kv(k, hq)
    vf = _expand_kv(v, hq)
    out = torch.empty((b, hq, sq, d), dtype=torch.float32)
    lse = torch.empty((b, hq, sq), dtype=torch.float32)
    for s0 in range(0, sq, q_chunk):
        s1 = min(sq, s0 + q_chunk)
        qf = q[:, s0:s1].float().permute(0, 2, 1, 3)
        scores = torch.matmul(qf, kf.transpose(-1, -2)) * softmax_scale
        if causal:
            vis = visibility(s1 - s0, sk, q_off + s0, k_off)
            scores = scores.masked_fill(~vis, float("-inf"))
        if sk > 0:
            blk_lse = torch.logsumexp(scores, dim=-1)
        else:
            blk_lse = torch.full(scores.shape[:-1], float("-inf"))
        p = torch.exp(scores - blk_lse.unsqueeze(-1))
        p = torch.nan_to_num(p, nan=0.0)  # rows with no visible key
        out[:, :, s0:s1] = torch.matmul(p, vf)
        lse[:, :, s0:s1] = blk_lse
    return out.permute(0, 2, 1, 3).contiguous().to(q.dtype), lse


def block_attn_bwd(
    dout: torch.Tensor,
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    out: torch.Tensor,
    lse: torch.Tensor,
    softmax_scale: float,
    causal: bool = False,
    q_off: Optional[int] = None,
    k_off: int = 0,
    q_chunk: int = 1024,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Gradients (dq, dk, dv) in fp32 for one (Q shard, K/V shard) pair.

    `out` and `lse` are the FINAL output and log-sum-exp of the Q rows (over all
    K/V shards), exactly what the generated backward passes to every block call
    (utils/attn_bwd_dsl.py:91-92): P = exp(scale*s - lse), dV = P^T dO,
    dP = dO V^T, delta = rowsum(dO * O), dS = P * (dP - delta),
    dQ = scale * dS K, dK = scale * dS^T Q.
    """
    b, sq, hq, d = q.shape
    sk, hkv = k.shape[1], k.shape[2]
    group = hq // hkv
    if q_off is None:
        q_off = sk - sq
    kf = _expand_kv(k, hq)
    vf = _expand_kv(v, hq)
    dq = torch.zeros((b, hq, sq, d), dtype=torch.float32)
    dk = torch.zeros((b, hq, sk, d), dtype=torch.float32)
    dv = torch.zeros((b, hq, sk, d), dtype=torch.float32)
    for s0 in range(0, sq, q_chunk):
        s1 = min(sq, s0 + q_chunk)
        qf = q[:, s0:s1].float().permute(0, 2, 1, 3)
        dof = dout[:, s0:s1].float().permute(0, 2, 1, 3)
        of = out[:, s0:s1].float().permute(0, 2, 1, 3)
        scores = torch.matmul(qf, kf.transpose(-1, -2)) * softmax_scale
        if causal:
            vis = visibility(s1 - s0, sk, q_off + s0, k_off)
            scores = scores.masked_fill(~vis, float("-inf"))
        p = torch.exp(scores - lse[:, :, s0:s1].float().unsqueeze(-1))
        p = torch.nan_to_num(p, nan=0.0, posinf=0.0)
        dv += torch.matmul(p.transpose(-1, -2), dof)
        dp = torch.matmul(dof, vf.transpose(-1, -2))
        delta = (dof * of).sum(dim=-1, keepdim=True)
        ds = p * (dp - delta)
        dq[:, :, s0:s1] = torch.matmul(ds, kf) * softmax_scale
        dk += torch.matmul(ds.transpose(-1, -2), qf) * softmax_scale
    if group != 1:
        dk = dk.view(b, hkv, group, sk, d).sum(dim=2)
        dv = dv.view(b, hkv, group, sk, d).sum(dim=2)
    return (
        dq.permute(0, 2, 1, 3).contiguous(),
        dk.permute(0, 2, 1, 3).contiguous(),
        dv.permute(0, 2, 1, 3).contiguous(),
    )


def full_attention(q, k, v, softmax_scale, causal=False):
    """Single-device fp32 attention over the whole sequence (the acceptance reference)."""
    return block_attn_fwd(q, k, v, softmax_scale, causal=causal, q_off=(k.shape[1] - q.shape[1]) if causal else 0)


def attn_flops(batch: int, hq: int, sq: int, sk: int, d: int, causal: bool) -> float:
    """Forward FLOPs, causal-adjusted: 4*B*H*Sq*Sk*D, halved when causal."""
    return 4.0 * batch * hq * sq * sk * d * (0.5 if causal else 1.0)
