"""Row-sampled fp32 attention for checking results at sizes where the full matrix is too big
(test infrastructure; runs on whatever device its inputs live on).

Same math as oracle/block.py (softmax(scale * q k^T) v with the natural log-sum-exp of the scaled
scores, and its analytic gradient as the generated backward uses it, utils/attn_bwd_dsl.py:86-115
of the reference: `out` and `lse` are the FINAL results of a query row), evaluated only for a
sample of query rows against ALL keys (forward, dQ) or for a sample of key rows against ALL
queries (dK, dV).  A key at global position j is visible to the query at global position i iff
j <= i when `causal`.
"""
from __future__ import annotations

from typing import Tuple

import torch


def _heads_chunks(hq: int, cols: int, rows: int, limit_elems: int = 1 << 28):
    """Query heads per slice so that a [heads, rows, cols] fp32 score block stays under the limit."""
    per = max(1, limit_elems // max(1, rows * cols))
    return [(h0, min(hq, h0 + per)) for h0 in range(0, hq, per)]


def sample_positions(length: int, n: int, seed: int, must: Tuple[int, ...] = ()) -> torch.Tensor:
    """Sorted unique positions in [0, length): the given ones plus seeded random ones up to n."""
    g = torch.Generator().manual_seed(seed)
    want = {int(p) for p in must if 0 <= int(p) < length}
    if length > 0:
        extra = torch.randint(0, length, (max(0, 2 * n),), generator=g).tolist()
        for p in extra:
            if len(want) >= n:
                break
            want.add(int(p))
    return torch.tensor(sorted(want), dtype=torch.long)


def fwd_rows(q_rows: torch.Tensor, q_pos: torch.Tensor, k: torch.Tensor, v: torch.Tensor, softmax_scale: float,
             causal: bool, k_off: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
    """q_rows [B, n, Hq, D] at global positions q_pos [n]; k, v [B, Sk, Hkv, D] with key 0 at global
    position k_off.  Returns (o [B, n, Hq, D] fp32, lse [B, Hq, n] fp32)."""
    b, n, hq, d = q_rows.shape
    sk, hkv = k.shape[1], k.shape[2]
    group = hq // hkv
    dev = q_rows.device
    o = torch.empty((b, n, hq, d), dtype=torch.float32, device=dev)
    lse = torch.empty((b, hq, n), dtype=torch.float32, device=dev)
    kpos = torch.arange(sk, device=dev) + k_off
    vis = (kpos[None, :] <= q_pos.to(dev)[:, None]) if causal else None
    for h0, h1 in _heads_chunks(hq, sk, n * b):
        qf = q_rows[:, :, h0:h1].float().permute(0, 2, 1, 3)                                # [B,h,n,D]
        kv_heads = torch.arange(h0, h1, device=dev) // group
        kf = k.index_select(2, kv_heads).float().permute(0, 2, 1, 3)                        # [B,h,Sk,D]
        vf = v.index_select(2, kv_heads).float().permute(0, 2, 1, 3)
        s = torch.matmul(qf, kf.transpose(-1, -2)) * softmax_scale
        if vis is not None:
            s = s.masked_fill(~vis, float("-inf"))
        l = torch.logsumexp(s, dim=-1) if sk > 0 else torch.full(s.shape[:-1], float("-inf"), device=dev)
        p = torch.nan_to_num(torch.exp(s - l.unsqueeze(-1)), nan=0.0)
        o[:, :, h0:h1] = torch.matmul(p, vf).permute(0, 2, 1, 3)
        lse[:, h0:h1] = l
    return o, lse


def dq_rows(q_rows: torch.Tensor, do_rows: torch.Tensor, o_rows: torch.Tensor, lse_rows: torch.Tensor,
            q_pos: torch.Tensor, k: torch.Tensor, v: torch.Tensor, softmax_scale: float, causal: bool,
            k_off: int = 0) -> torch.Tensor:
    """dQ [B, n, Hq, D] fp32 of the sampled query rows; o_rows/lse_rows ([B, Hq, n]) are their final
    forward results."""
    b, n, hq, d = q_rows.shape
    sk, hkv = k.shape[1], k.shape[2]
    group = hq // hkv
    dev = q_rows.device
    dq = torch.empty((b, n, hq, d), dtype=torch.float32, device=dev)
    kpos = torch.arange(sk, device=dev) + k_off
    vis = (kpos[None, :] <= q_pos.to(dev)[:, None]) if causal else None
    for h0, h1 in _heads_chunks(hq, sk, n * b):
        qf = q_rows[:, :, h0:h1].float().permute(0, 2, 1, 3)
        dof = do_rows[:, :, h0:h1].float().permute(0, 2, 1, 3)
        of = o_rows[:, :, h0:h1].float().permute(0, 2, 1, 3)
        kv_heads = torch.arange(h0, h1, device=dev) // group
        kf = k.index_select(2, kv_heads).float().permute(0, 2, 1, 3)
        vf = v.index_select(2, kv_heads).float().permute(0, 2, 1, 3)
        s = torch.matmul(qf, kf.transpose(-1, -2)) * softmax_scale
        if vis is not None:
            s = s.masked_fill(~vis, float("-inf"))
        p = torch.nan_to_num(torch.exp(s - lse_rows[:, h0:h1].float().unsqueeze(-1)), nan=0.0, posinf=0.0)
        dp = torch.matmul(dof, vf.transpose(-1, -2))
        delta = (dof * of).sum(-1, keepdim=True)
        ds = p * (dp - delta)
        dq[:, :, h0:h1] = (torch.matmul(ds, kf) * softmax_scale).permute(0, 2, 1, 3)
    return dq


def dkv_rows(k_rows: torch.Tensor, v_rows: torch.Tensor, k_pos: torch.Tensor, q: torch.Tensor, do: torch.Tensor,
             o: torch.Tensor, lse: torch.Tensor, softmax_scale: float, causal: bool,
             q_off: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
    """(dK, dV) [B, n, Hkv, D] fp32 of the sampled key rows at global positions k_pos [n], against
    ALL queries: q, do, o [B, Sq, Hq, D], lse [B, Hq, Sq], query 0 at global position q_off."""
    b, n, hkv, d = k_rows.shape
    sq, hq = q.shape[1], q.shape[2]
    group = hq // hkv
    dev = q.device
    dk = torch.zeros((b, n, hkv, d), dtype=torch.float32, device=dev)
    dv = torch.zeros((b, n, hkv, d), dtype=torch.float32, device=dev)
    qpos = torch.arange(sq, device=dev) + q_off
    vis = (k_pos.to(dev)[None, :] <= qpos[:, None]) if causal else None                       # [Sq, n]
    for h0, h1 in _heads_chunks(hq, n * b, sq):
        qf = q[:, :, h0:h1].float().permute(0, 2, 1, 3)                                      # [B,h,Sq,D]
        dof = do[:, :, h0:h1].float().permute(0, 2, 1, 3)
        of = o[:, :, h0:h1].float().permute(0, 2, 1, 3)
        kv_heads = torch.arange(h0, h1, device=dev) // group
        kf = k_rows.index_select(2, kv_heads).float().permute(0, 2, 1, 3)                    # [B,h,n,D]
        vf = v_rows.index_select(2, kv_heads).float().permute(0, 2, 1, 3)
        s = torch.matmul(qf, kf.transpose(-1, -2)) * softmax_scale                           # [B,h,Sq,n]
        if vis is not None:
            s = s.masked_fill(~vis, float("-inf"))
        p = torch.nan_to_num(torch.exp(s - lse[:, h0:h1].float().unsqueeze(-1)), nan=0.0, posinf=0.0)
        dp = torch.matmul(dof, vf.transpose(-1, -2))
        delta = (dof * of).sum(-1, keepdim=True)
        ds = p * (dp - delta)
        pdv = torch.matmul(p.transpose(-1, -2), dof)                                         # [B,h,n,D]
        pdk = torch.matmul(ds.transpose(-1, -2), qf) * softmax_scale
        # several query heads share a K/V head: their contributions add up
        dv.index_add_(2, kv_heads, pdv.permute(0, 2, 1, 3).contiguous())
        dk.index_add_(2, kv_heads, pdk.permute(0, 2, 1, 3).contiguous())
    return dk, dv


# ---------------------------------------------------------------------------
# one rank of a sequence-sharded job: gather what the check needs, compare a row sample
# ---------------------------------------------------------------------------
def gather_seq(x: torch.Tensor, seq_dim: int, world: int) -> torch.Tensor:
    """Concatenate every rank's shard along the sequence dimension (torch.distributed, any backend)."""
    if world == 1:
        return x
    import torch.distributed as dist

    x = x.contiguous()
    out = torch.empty((world,) + tuple(x.shape), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x)
    return torch.cat(list(out.unbind(0)), dim=seq_dim)


def check_forward_shard(q, kv, o, lse, rank: int, world: int, causal: bool, softmax_scale: float, rows: int = 64,
                        seed: int = 77) -> dict:
    """Max-abs error of a row sample of THIS rank's o / lse (shard `rank` of `world` contiguous equal
    shards; kv [2, B, L, Hkv, D]) against fp32 attention over the keys of all ranks.  The sample always
    holds the first and last row of the shard and of each of its halves.  Collective: every rank calls it."""
    L = q.shape[1]
    k_full, v_full = gather_seq(kv[0], 1, world), gather_seq(kv[1], 1, world)
    pos = sample_positions(L, rows, seed=seed + rank, must=(0, L // 2 - 1, L // 2, L - 1)).to(q.device)
    ro, rl = fwd_rows(q[:, pos], pos + rank * L, k_full, v_full, softmax_scale, causal)
    return {"o_max_abs": (o[:, pos].float() - ro).abs().max().item(),
            "lse_max_abs": (lse[:, :, pos] - rl).abs().max().item(), "rows": int(pos.numel())}


def check_backward_shard(q, kv, o, lse, dout, dq, dkv, rank: int, world: int, causal: bool, softmax_scale: float,
                         rows: int = 48, seed: int = 177) -> dict:
    """Max-abs error of a row sample of THIS rank's dq (its queries against all keys) and dk / dv (its
    keys against the queries of all ranks) against the fp32 gradients.  Collective."""
    L = q.shape[1]
    pos = sample_positions(L, rows, seed=seed + rank, must=(0, L // 2 - 1, L // 2, L - 1)).to(q.device)
    gpos = pos + rank * L
    k_full, v_full = gather_seq(kv[0], 1, world), gather_seq(kv[1], 1, world)
    rq = dq_rows(q[:, pos], dout[:, pos], o[:, pos], lse[:, :, pos], gpos, k_full, v_full, softmax_scale, causal)
    eq = (dq[:, pos].float() - rq).abs().max().item()
    del k_full, v_full, rq
    q_full, do_full = gather_seq(q, 1, world), gather_seq(dout, 1, world)
    o_full, lse_full = gather_seq(o, 1, world), gather_seq(lse, 2, world)
    rk, rv = dkv_rows(kv[0][:, pos], kv[1][:, pos], gpos, q_full, do_full, o_full, lse_full, softmax_scale, causal)
    return {"dq_max_abs": eq, "dk_max_abs": (dkv[0][:, pos].float() - rk).abs().max().item(),
            "dv_max_abs": (dkv[1][:, pos].float() - rv).abs().max().item(), "rows": int(pos.numel())}
