"""The per-rank ring schedules of the generated code, restated on the CPU (test infrastructure).

Two executions of the same protocol:
  * simulate_*: all P ranks inside one process, message passing modelled by list shuffles;
  * rank_*: one rank of a torch.distributed (gloo) job, messages by batched isend/irecv,
    which is what mercury/backend/pytorch/utils.py:9-39 (SendRecv) does.

Protocol sources: forward loop mercury/backend/pytorch/codegen.py:443-494 (post the next
transfer, compute on the held shard, merge), double-ring neighbour choice :480-491, backward
accumulators and write-back hop :99-190, index helpers utils.py:41-106 and :171-192.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

import torch

from . import block as _block
from . import merge as _merge


# ---------------------------------------------------------------------------
# mesh index helpers (mercury/backend/pytorch/utils.py:41-106): dimension 0 varies fastest
# ---------------------------------------------------------------------------
def coords_of(rank: int, shape: Sequence[int]) -> Tuple[int, ...]:
    out = []
    for n in shape:
        out.append(rank % n)
        rank //= n
    return tuple(out)


def rank_of(coords: Sequence[int], shape: Sequence[int]) -> int:
    r, mul = 0, 1
    for c, n in zip(coords, shape):
        r += c * mul
        mul *= n
    return r


def shift_coord(coords: Sequence[int], dim: int, delta: int, modulo: int) -> Tuple[int, ...]:
    c = list(coords)
    c[dim] = (c[dim] + delta) % modulo
    return tuple(c)


def writeback_src_dst(coords, shape, ring_dims) -> Tuple[int, int]:
    """utils.py:171-192: the extra hop that returns a rotating reduce buffer to its owner."""
    src, step = tuple(coords), 1
    for d in reversed(ring_dims):
        src = shift_coord(src, d, -step, shape[d])
        step = shape[d]
    dst, step = tuple(coords), 1
    for d in reversed(ring_dims):
        dst = shift_coord(dst, d, step, shape[d])
        step = shape[d]
    return rank_of(src, shape), rank_of(dst, shape)


def ring_steps(shape: Sequence[int]) -> List[Tuple[int, ...]]:
    """Loop nest order of the generated code: outermost mesh dim is the outermost loop,
    mesh dim 0 the innermost (`for outer: for inner:`)."""
    steps = [()]
    for n in reversed(shape):
        steps = [s + (i,) for s in steps for i in range(n)]
    # each tuple is (idx_of_last_dim, ..., idx_of_dim0); flip to mesh-dim order
    return [tuple(reversed(s)) for s in steps]


def hop_dim(step: Tuple[int, ...], shape: Sequence[int]) -> Optional[int]:
    """Which mesh dim the shard moves along after this step (codegen.py:480-491):
    the first dim (from 0) whose ring index is not at its end; None after the last step."""
    for d, n in enumerate(shape):
        if step[d] + 1 != n:
            return d
    return None


def kv_origin_schedule(rank: int, shape: Sequence[int]) -> List[int]:
    """Origin rank of the K/V shard that `rank` computes on at each step (relay semantics)."""
    p = 1
    for n in shape:
        p *= n
    held = list(range(p))
    out = []
    for st in ring_steps(shape):
        out.append(held[rank])
        d = hop_dim(st, shape)
        if d is not None:
            held = [held[rank_of(shift_coord(coords_of(r, shape), d, -1, shape[d]), shape)] for r in range(p)]
    return out


# ---------------------------------------------------------------------------
# forward, all ranks in one process
# ---------------------------------------------------------------------------
def simulate_ring_fwd(
    q_shards: Sequence[torch.Tensor],
    kv_shards: Sequence[torch.Tensor],
    softmax_scale: float,
    mesh_shape: Sequence[int],
    causal: bool = False,
    positional_causal: bool = False,
    block_fn: Callable = _block.block_attn_fwd,
):
    """q_shards[r] [B,S/P,Hq,D]; kv_shards[r] [2,B,S/P,Hkv,D].  Returns ([o_r], [lse_r [B,Hq,S/P]]).

    causal=True with positional_causal=False reproduces the reference literally: the flag is
    handed unchanged to every block (utils/flash_attn_dsl.py:167), which is only meaningful for
    causal=False.  positional_causal=True is this build's causal ring: block (r, origin) uses the
    global positions of its shards, blocks entirely in the future are skipped.
    """
    p = len(q_shards)
    held = [kv.clone() for kv in kv_shards]
    origin = list(range(p))
    outs: List[Optional[torch.Tensor]] = [None] * p
    lses: List[Optional[torch.Tensor]] = [None] * p
    parts: List[list] = [[] for _ in range(p)]
    shard_len = q_shards[0].shape[1]
    kv_len = kv_shards[0].shape[2]
    for st in ring_steps(mesh_shape):
        d = hop_dim(st, mesh_shape)
        if d is not None:
            src = [rank_of(shift_coord(coords_of(r, mesh_shape), d, -1, mesh_shape[d]), mesh_shape) for r in range(p)]
            nxt = [held[s] for s in src]
            nxt_origin = [origin[s] for s in src]
        for r in range(p):
            k, v = held[r][0], held[r][1]
            if positional_causal:
                q_off, k_off = r * shard_len, origin[r] * kv_len
                if k_off > q_off + shard_len - 1:
                    continue
                parts[r].append(block_fn(q_shards[r], k, v, softmax_scale, causal=True, q_off=q_off, k_off=k_off))
            else:
                bo, bl = block_fn(q_shards[r], k, v, softmax_scale, causal=causal)
                outs[r], lses[r] = _merge.update_out_and_lse(outs[r], lses[r], bo, bl)
        if d is not None:
            held, origin = nxt, nxt_origin
    res_o, res_l = [], []
    for r in range(p):
        if positional_causal:
            o, l = _merge.merge_exact(parts[r])
            res_o.append(o.to(q_shards[r].dtype))
            res_l.append(l)
        else:
            res_o.append(outs[r].to(q_shards[r].dtype))
            res_l.append(lses[r].squeeze(-1).transpose(1, 2).contiguous())
    return res_o, res_l


# ---------------------------------------------------------------------------
# ring over Q with a rotating packed reduce buffer (codegen.py:116-190, flash_reduce)
# ---------------------------------------------------------------------------
def simulate_ring_over_q(q_shards, kv_shards, softmax_scale: float, mesh_shape: Sequence[int],
                         block_fn: Callable = _block.block_attn_fwd):
    """K/V stay put; the query shard and a packed fp32 [B,S/P,H,D+1] = [out | lse] buffer rotate
    together.  Step 0 starts the buffer from the local block result, later steps merge the buffer
    that arrived with the queries (flash_reduce), and one extra hop (get_src_dst_ranks) returns
    each buffer to the rank that owns those queries.  Non-causal, as in the reference."""
    p = len(q_shards)
    ring_dims = list(range(len(mesh_shape)))
    held_q = [q.clone() for q in q_shards]
    buf: List[Optional[torch.Tensor]] = [None] * p
    incoming: List[Optional[torch.Tensor]] = [None] * p
    for idx, st in enumerate(ring_steps(mesh_shape)):
        d = hop_dim(st, mesh_shape)
        if d is not None:
            src = [rank_of(shift_coord(coords_of(r, mesh_shape), d, -1, mesh_shape[d]), mesh_shape) for r in range(p)]
        for r in range(p):
            bo, bl = block_fn(held_q[r], kv_shards[r][0], kv_shards[r][1], softmax_scale, causal=False)
            res = torch.cat([bo.to(torch.float32), bl.transpose(-2, -1).unsqueeze(-1)], dim=-1)
            buf[r] = res.contiguous() if idx == 0 else _merge.flash_reduce(incoming[r], res)
        if d is not None:
            held_q = [held_q[s] for s in src]
            incoming = [buf[s] for s in src]
        else:
            back = [writeback_src_dst(coords_of(r, mesh_shape), mesh_shape, ring_dims)[0] for r in range(p)]
            buf = [buf[s] for s in back]
    outs = [b[..., :-1].to(q_shards[r].dtype) for r, b in enumerate(buf)]
    lses = [b[..., -1].transpose(1, 2).contiguous() for b in buf]
    return outs, lses


# ---------------------------------------------------------------------------
# backward, all ranks in one process (codegen.py:99-190)
# ---------------------------------------------------------------------------
def simulate_ring_bwd(
    q_shards, kv_shards, o_shards, lse_shards, dout_shards, softmax_scale: float, mesh_shape: Sequence[int],
    positional_causal: bool = False, block_dtype: Optional[torch.dtype] = None,
    bwd_fn: Callable = _block.block_attn_bwd,
):
    """Returns ([dq_r], [dkv_r [2,B,S/P,H,D]]) in the dtype of q/kv.

    Per step every rank computes block gradients for (its Q shard, the held K/V shard) in
    `block_dtype` (the reference allocates block_dq/block_dkv in the input dtype,
    utils/attn_bwd_dsl.py:83-84), adds dq locally in fp32, adds dkv onto the fp32 accumulator
    that arrived from the previous rank and forwards it; one extra hop brings each
    accumulator home.  The reference calls the block with causal=False always (:100).
    """
    p = len(q_shards)
    ring_dims = list(range(len(mesh_shape)))
    held = [kv.clone() for kv in kv_shards]
    origin = list(range(p))
    acc_dq: List[Optional[torch.Tensor]] = [None] * p
    acc_dkv: List[Optional[torch.Tensor]] = [None] * p
    incoming: List[Optional[torch.Tensor]] = [None] * p
    steps = ring_steps(mesh_shape)
    shard_len = q_shards[0].shape[1]
    kv_len = kv_shards[0].shape[2]
    for idx, st in enumerate(steps):
        d = hop_dim(st, mesh_shape)
        if d is not None:
            src = [rank_of(shift_coord(coords_of(r, mesh_shape), d, -1, mesh_shape[d]), mesh_shape) for r in range(p)]
        for r in range(p):
            k, v = held[r][0], held[r][1]
            bdt = block_dtype or q_shards[r].dtype
            if positional_causal:
                q_off, k_off = r * shard_len, origin[r] * kv_len
                if k_off > q_off + shard_len - 1:
                    bdq = torch.zeros_like(q_shards[r], dtype=torch.float32)
                    bdk = torch.zeros_like(k, dtype=torch.float32)
                    bdv = torch.zeros_like(v, dtype=torch.float32)
                else:
                    bdq, bdk, bdv = bwd_fn(dout_shards[r], q_shards[r], k, v, o_shards[r], lse_shards[r],
                                           softmax_scale, causal=True, q_off=q_off, k_off=k_off)
            else:
                bdq, bdk, bdv = bwd_fn(dout_shards[r], q_shards[r], k, v, o_shards[r], lse_shards[r],
                                       softmax_scale, causal=False)
            bdq = bdq.to(bdt).float()
            bdkv = torch.stack([bdk, bdv]).to(bdt).float()
            acc_dq[r] = bdq if idx == 0 else acc_dq[r] + bdq
            acc_dkv[r] = bdkv if idx == 0 else incoming[r] + bdkv
        if d is not None:
            held = [held[s] for s in src]
            origin = [origin[s] for s in src]
            incoming = [acc_dkv[s] for s in src]
        else:
            back = [writeback_src_dst(coords_of(r, mesh_shape), mesh_shape, ring_dims)[0] for r in range(p)]
            acc_dkv = [acc_dkv[s] for s in back]
    dq = [acc_dq[r].to(q_shards[r].dtype) for r in range(p)]
    dkv = [acc_dkv[r].to(kv_shards[r].dtype) for r in range(p)]
    return dq, dkv


# ---------------------------------------------------------------------------
# one rank of a torch.distributed job (SendRecv restated: utils.py:9-39)
# ---------------------------------------------------------------------------
class _Exchange:
    """One outstanding batched send+recv, like the reference's SendRecv object."""

    def __init__(self):
        self._ops, self._reqs = [], None

    def post(self, to_rank: int, from_rank: int, tensor: torch.Tensor) -> torch.Tensor:
        import torch.distributed as dist

        recv = torch.empty_like(tensor)
        self._ops = [dist.P2POp(dist.isend, tensor.contiguous(), to_rank), dist.P2POp(dist.irecv, recv, from_rank)]
        self._reqs = dist.batch_isend_irecv(self._ops)
        return recv

    def wait(self):
        for r in self._reqs or []:
            r.wait()
        self._reqs, self._ops = None, []


def rank_ring_fwd(q, kv, softmax_scale, mesh_shape, causal=False, block_fn: Callable = _block.block_attn_fwd):
    """Forward ring for the calling rank of an initialised process group.  Returns (o, lse [B,Hq,S/P])."""
    import torch.distributed as dist

    rank = dist.get_rank()
    me = coords_of(rank, mesh_shape)
    held = kv.contiguous()
    out = lse = None
    ex = _Exchange()
    nxt = None
    for st in ring_steps(mesh_shape):
        d = hop_dim(st, mesh_shape)
        if d is not None:
            to_rank = rank_of(shift_coord(me, d, 1, mesh_shape[d]), mesh_shape)
            from_rank = rank_of(shift_coord(me, d, -1, mesh_shape[d]), mesh_shape)
            nxt = ex.post(to_rank, from_rank, held)
        bo, bl = block_fn(q, held[0], held[1], softmax_scale, causal=causal)
        out, lse = _merge.update_out_and_lse(out, lse, bo, bl)
        if d is not None:
            ex.wait()
            held = nxt
    return out.to(q.dtype), lse.squeeze(-1).transpose(1, 2).contiguous()
