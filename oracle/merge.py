"""Merge of partial attention results (test infrastructure).

Restates utils/flash_attn_dsl.py:31-71 (running out/LSE merge used by every
generated ring loop) and :293-305 (the same merge on a packed [..., D+1] buffer).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn.functional as F


def merge_step(out, lse, block_out, block_lse):
    """utils/flash_attn_dsl.py:31-49.

    out [B,S,H,D] fp32, lse [B,S,H,1] fp32; block_out [B,S,H,D] any float dtype,
    block_lse [B,H,S] fp32.  new = old - sigmoid(blse - lse) * (old - block);
    lse_new = lse - logsigmoid(lse - blse).
    """
    bo = block_out.to(torch.float32)
    bl = block_lse.transpose(-2, -1).unsqueeze(-1)
    new_out = out - torch.sigmoid(bl - lse) * (out - bo)
    new_lse = lse - F.logsigmoid(lse - bl)
    return new_out, new_lse


def update_out_and_lse(
    out: Optional[torch.Tensor],
    lse: Optional[torch.Tensor],
    block_out: torch.Tensor,
    block_lse: torch.Tensor,
    slice_=None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """utils/flash_attn_dsl.py:51-71: the first call adopts the block result
    (fp32 copy, LSE transposed to [B,S,H,1]); later calls merge, optionally into a slice."""
    if out is None:
        if slice_ is not None:
            raise RuntimeError("first update_out_and_lse should not pass slice_ args")
        return block_out.to(torch.float32), block_lse.transpose(-2, -1).unsqueeze(-1)
    if slice_ is not None:
        o, l = merge_step(out[slice_], lse[slice_], block_out, block_lse)
        out[slice_], lse[slice_] = o, l
        return out, lse
    return merge_step(out, lse, block_out, block_lse)


def flash_reduce(lhs: torch.Tensor, rhs: torch.Tensor) -> torch.Tensor:
    """utils/flash_attn_dsl.py:293-305: merge of two packed [..., D+1] = [out | lse] buffers."""
    lo, ll = lhs[..., :-1], lhs[..., -1:]
    ro, rl = rhs[..., :-1], rhs[..., -1:]
    out = lo - torch.sigmoid(rl - ll) * (lo - ro)
    lse = ll - F.logsigmoid(ll - rl)
    return torch.cat([out, lse], dim=-1)


def merge_exact(parts):
    """Order-independent merge of [(out [B,S,H,D], lse [B,H,S])...] by the log-sum-exp
    identity; used to cross-check merge_step and to merge causal partials where some rows
    of a block see no key (lse = -inf), which the reference formula cannot represent."""
    lses = torch.stack([p[1].float() for p in parts])             # [n,B,H,S]
    total = torch.logsumexp(lses, dim=0)                           # [B,H,S]
    w = torch.exp(lses - total.unsqueeze(0))
    w = torch.nan_to_num(w, nan=0.0)
    out = sum(p[0].float() * w[i].transpose(-2, -1).unsqueeze(-1) for i, p in enumerate(parts))
    return out, total


def tree_merge(packed_parts):
    """What update_out_and_lse_collective leaves on every rank (utils/flash_attn_dsl.py:307-324):
    with m = max_r lse_r and d_r = exp(lse_r - m):  out = sum_r d_r out_r / sum_r d_r,
    lse = m + log sum_r d_r.  packed_parts: list of [..., D+1] fp32 tensors, one per rank."""
    lses = torch.stack([p[..., -1:] for p in packed_parts])
    m = lses.max(dim=0).values
    d = torch.exp(lses - m)
    out = sum(p[..., :-1] * d[i] for i, p in enumerate(packed_parts)) / d.sum(dim=0)
    return torch.cat([out, m + torch.log(d.sum(dim=0))], dim=-1)
