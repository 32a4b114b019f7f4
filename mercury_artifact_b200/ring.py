"""Fused ring / double-ring / GQA attention for one rank: forward and backward (public API).

`RingAttention.forward` computes what the generated per-rank loop computes
(mercury/backend/pytorch/codegen.py:443-494 + utils/flash_attn_dsl.py:160-179 of
the reference) with ONE attention launch: the K/V shards of all ranks are the
segments of a single mb_attn_fwd call in the rank's arrival order, so the
online-softmax state stays on chip and no out/LSE merge kernel runs.
`RingAttention.backward` replaces the generated backward loop
(codegen.py:99-190, utils/attn_bwd_dsl.py:70-134) with two launches: dQ of the
local queries over all K/V shards, and dK/dV of the local keys over all query
shards.  Every gradient tile is owned by one CTA, so the reference's rotating
fp32 dK/dV accumulator and its write-back hop have no counterpart here.

Transport.  On an NVSwitch box every peer is one hop away, so a shard is pulled
straight from the rank that owns it instead of being relayed around the ring;
the order in which a rank consumes shards is still the reference's (single ring:
(r - t) mod P; nested rings: mesh.kv_origin_schedule).  The copy engines move
each remote shard over NVLink into a local staging buffer on a high-priority
side stream and a per-segment flag is raised behind it; the kernel's loader
waits (bounded) on that flag before its first TMA load of the segment, so
compute on the shards already here overlaps the transfers of the later ones
inside one launch.

World size 1 is the unsharded program: one segment, no transport.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

from . import mesh
from .attention import (RowStats, _pad64, attn_bwd_dkv, attn_bwd_dq, attn_fwd_segments, bwd_preprocess)
from .comm import PeerContext, SymmetricBuffer, _align, default_context

_FLAG_REGION = 4096


class _ShardExchange:
    """Publish one byte-slot per rank and epoch; pull peers' slots into local staging.

    Symmetric memory per rank: two slots (epoch parity) + flag words
        ready[origin] at +0     raised on every peer once `origin` has published its slot
        done[reader]  at +1024  raised on the owner once `reader` no longer needs the slot
    Local memory: world-1 staging slots and one arrival flag per staging slot.
    All flag values are epoch numbers, which only grow.
    """

    def __init__(self, ctx: PeerContext, slot_bytes: int):
        self.ctx = ctx
        self.world, self.rank = ctx.world, ctx.rank
        self.slot_bytes = _align(slot_bytes, 1024)
        self.sym = SymmetricBuffer(ctx, 2 * self.slot_bytes + _FLAG_REGION)
        self._flag_off = 2 * self.slot_bytes
        self.staging = torch.empty((max(self.world - 1, 1), self.slot_bytes), dtype=torch.uint8, device=ctx.device)
        self.seg_flags = torch.zeros(64, dtype=torch.int32, device=ctx.device)
        self.epoch = 0
        self._next_stage = 0
        self._stage_of = {}
        torch.cuda.synchronize(ctx.device)

    def _ready_ptr(self, on_rank: int, origin: int) -> int:
        return self.sym.ptr(on_rank, self._flag_off + 4 * origin)

    def _done_ptr(self, on_rank: int, reader: int) -> int:
        return self.sym.ptr(on_rank, self._flag_off + 1024 + 4 * reader)

    def local_slot(self) -> torch.Tensor:
        off = (self.epoch % 2) * self.slot_bytes
        return self.sym.local.bytes()[off:off + self.slot_bytes]

    def begin(self, main: torch.cuda.Stream, peers: Optional[Sequence[int]] = None) -> torch.Tensor:
        """Start a new epoch; returns this rank's byte slot to fill on the transfer stream.
        peers restricts the exchange to a sub-group of ranks (default: every rank)."""
        ctx, comm = self.ctx, self.ctx.comm_stream
        self.epoch += 1
        self._next_stage = 0
        self._stage_of = {}
        e = self.epoch
        comm.wait_stream(main)
        if e > 2:  # the slot was last used at epoch e-2: every peer has released it by now or soon
            for p in (peers if peers is not None else range(self.world)):
                if p != self.rank:
                    ctx.wait_flag(self._done_ptr(self.rank, p), e - 2, comm)
        return self.local_slot()

    def publish(self, peers: Optional[Sequence[int]] = None) -> torch.cuda.Event:
        """Announce the filled slot to every peer; the event fires once the local copy is in place."""
        ctx, comm = self.ctx, self.ctx.comm_stream
        ev = torch.cuda.Event()
        ev.record(comm)
        for p in (peers if peers is not None else range(self.world)):
            if p != self.rank:
                ctx.signal(self._ready_ptr(p, self.rank), self.epoch, comm)
        return ev

    def pull(self, origin: int, ranges: Optional[Sequence[Tuple[int, int]]] = None, final: bool = True,
             raise_flag: bool = True, piece: int = 0) -> Tuple[torch.Tensor, int]:
        """Copy `origin`'s slot of this epoch (or the given (offset, nbytes) ranges of it) into that
        origin's staging slot (copy engines over NVLink).  Returns (staging bytes, address of the
        arrival flag that reaches `epoch` behind the copy).  final=False keeps the owner's slot
        reserved for a later pull of the same epoch; raise_flag=False leaves the arrival flag alone
        (the caller orders its consumers with a stream event instead).  piece selects one of the
        staging slot's eight arrival flags, for a slot that is pulled in several pieces."""
        ctx, comm = self.ctx, self.ctx.comm_stream
        e = self.epoch
        if origin not in self._stage_of:
            self._stage_of[origin] = self._next_stage
            self._next_stage += 1
            ctx.wait_flag(self._ready_ptr(self.rank, origin), e, comm)
        idx = self._stage_of[origin]
        dst = self.staging[idx]
        base = (e % 2) * self.slot_bytes
        for off, nbytes in (ranges if ranges is not None else [(0, self.slot_bytes)]):
            ctx.copy(dst.data_ptr() + off, self.sym.ptr(origin, base + off), nbytes, comm)
        if not 0 <= piece < 8:
            raise ValueError("a staging slot has eight arrival flags")
        flag_ptr = self.seg_flags.data_ptr() + 4 * (8 * idx + piece)
        if raise_flag:
            ctx.signal(flag_ptr, e, comm)
        if final:
            ctx.signal(self._done_ptr(origin, self.rank), e, comm)
        return dst, flag_ptr

    def release(self, origin: int) -> None:
        """Tell `origin` that this rank will not read its slot of this epoch."""
        self.ctx.signal(self._done_ptr(origin, self.rank), self.epoch, self.ctx.comm_stream)


def _carve(buf: torch.Tensor, offset: int, shape, dtype) -> Tuple[torch.Tensor, int]:
    n = 1
    for s in shape:
        n *= int(s)
    nbytes = n * torch.empty((), dtype=dtype).element_size()
    return buf[offset:offset + nbytes].view(dtype).view(*shape), offset + _align(nbytes, 256)


class RingAttention:
    """Attention of one rank of a sequence-sharded job.

    mesh_shape (P,) is the single ring, (n_inner, n_outer) the double ring (inner ring over
    mesh dimension 0, rank = inner + n_inner * outer).  Shard k of the sequence lives on rank k.
    With causal=True a key is visible iff its global position is <= the query's.
    """

    def __init__(self, mesh_shape: Sequence[int], batch: int, seq_local: int, hq: int, hkv: int,
                 head_dim: int = 128, causal: bool = False, ctx: Optional[PeerContext] = None,
                 balance_causal: bool = True, ring_divide: int = 1):
        self.mesh_shape = tuple(int(n) for n in mesh_shape)
        self.world = 1
        for n in self.mesh_shape:
            self.world *= n
        self.batch, self.seq_local, self.hq, self.hkv, self.head_dim = batch, seq_local, hq, hkv, head_dim
        self.causal = bool(causal)
        self.ctx = ctx if ctx is not None else (default_context() if self.world > 1 else None)
        self.rank = self.ctx.rank if self.ctx is not None else 0
        if self.ctx is not None and self.ctx.world != self.world:
            raise ValueError(f"mesh {self.mesh_shape} needs {self.world} ranks, the process group has {self.ctx.world}")
        self.order = mesh.kv_origin_schedule(self.rank, self.mesh_shape)
        self.q_shape = (batch, seq_local, hq, head_dim)
        self.kv_shape = (2, batch, seq_local, hkv, head_dim)
        self.stat_pad = _pad64(seq_local)
        self.stat_shape = (2, batch, hq, self.stat_pad)
        self.launches_per_forward = 1
        self.launches_per_backward = 3
        self._fwd_x: Optional[_ShardExchange] = None
        self._bwd_x: Optional[_ShardExchange] = None
        self._bal_x: Optional[_ShardExchange] = None
        self._bal_inbox: Optional[SymmetricBuffer] = None
        # Causal attention over contiguous shards gives rank r (r + 1/2) blocks of work.  With
        # balancing, the forward re-assigns query half-shards so that every rank computes the same
        # amount (see _forward_balanced); inputs and outputs keep the contiguous layout.
        self.balanced = bool(balance_causal) and self.causal and self.world > 1 and seq_local % 2 == 0
        if self.balanced:
            self.launches_per_forward = 2
        # ring_divide (the rounds parameter of the reference's shift primitive, ir/primitives.py:33-45,
        # 101-102): every K/V shard travels as `ring_divide` sequence pieces, each with its own arrival
        # flag and its own segment of the launch, so work on a shard starts when its first piece is in.
        # One launch takes at most eight segments: 1 local + (world - 1) * ring_divide.
        self.ring_divide = int(ring_divide)
        if self.ring_divide < 1 or seq_local % self.ring_divide != 0:
            raise ValueError("ring_divide must divide the local sequence length")
        if self.ring_divide > 1:
            if self.balanced:
                raise ValueError("ring_divide > 1 is implemented for the plain (unbalanced) forward: "
                                 "pass balance_causal=False")
            if 1 + (self.world - 1) * self.ring_divide > 8:
                raise ValueError("1 + (world - 1) * ring_divide segments exceed the eight of one launch")

    # ------------------------------------------------------------------ helpers
    def _sees_keys_of(self, origin: int) -> bool:
        """Whether this rank's queries can see any key of `origin`'s shard."""
        return (not self.causal) or origin <= self.rank

    def _seen_by_queries_of(self, origin: int) -> bool:
        """Whether `origin`'s queries can see any key of this rank's shard."""
        return (not self.causal) or origin >= self.rank

    def _kv_bytes(self) -> int:
        return 2 * self.batch * self.seq_local * self.hkv * self.head_dim * 2

    def _bwd_slot_bytes(self) -> int:
        """Backward exchange slot: kv | q | dout | row statistics, each 256-byte aligned."""
        q_b = self.batch * self.seq_local * self.hq * self.head_dim * 2
        st_b = 2 * self.batch * self.hq * self.stat_pad * 4
        return _align(self._kv_bytes(), 256) + 2 * _align(q_b, 256) + _align(st_b, 256)

    # ------------------------------------------------------------------ forward
    def forward(self, q: torch.Tensor, kv: torch.Tensor, o: Optional[torch.Tensor] = None,
                lse: Optional[torch.Tensor] = None, softmax_scale: Optional[float] = None
                ) -> Tuple[torch.Tensor, torch.Tensor]:
        """q [B,S/P,Hq,D], kv [2,B,S/P,Hkv,D] bf16 on this rank's device -> (o, lse [B,Hq,S/P])."""
        if tuple(kv.shape) != self.kv_shape:
            raise ValueError(f"kv must have shape {self.kv_shape}, got {tuple(kv.shape)}")
        if softmax_scale is None:
            softmax_scale = self.head_dim ** -0.5
        L = self.seq_local
        if self.world == 1:
            return attn_fwd_segments(q, [(kv[0], kv[1], 0)], softmax_scale, causal=self.causal, q_off=0, out=o, lse=lse)

        if self.balanced:
            return self._forward_balanced(q, kv, o, lse, softmax_scale)

        if self._fwd_x is None:
            self._fwd_x = _ShardExchange(self.ctx, self._kv_bytes())
        x = self._fwd_x
        main = torch.cuda.current_stream()
        comm = self.ctx.comm_stream
        me = self.rank

        slot_bytes = x.begin(main)
        slot, _ = _carve(slot_bytes, 0, self.kv_shape, torch.bfloat16)
        with torch.cuda.stream(comm):
            slot.copy_(kv, non_blocking=True)
        local_ready = x.publish()

        segs: List[tuple] = [(slot[0], slot[1], me * L)]
        for t in range(1, self.world):
            origin = self.order[t]
            if self._sees_keys_of(origin) and self.ring_divide == 1:
                buf, flag_ptr = x.pull(origin)
                rkv, _ = _carve(buf, 0, self.kv_shape, torch.bfloat16)
                segs.append((rkv[0], rkv[1], origin * L, flag_ptr, x.epoch))
            elif self._sees_keys_of(origin):
                d, c = self.ring_divide, L // self.ring_divide
                row_b = self.hkv * self.head_dim * 2
                for j in range(d):
                    # rows [j c, (j+1) c) of K and of V, for every batch entry: 2 B contiguous ranges
                    ranges = [(((w * self.batch + b) * L + j * c) * row_b, c * row_b)
                              for w in range(2) for b in range(self.batch)]
                    buf, flag_ptr = x.pull(origin, ranges, final=(j == d - 1), piece=j)
                    rkv, _ = _carve(buf, 0, self.kv_shape, torch.bfloat16)
                    segs.append((rkv[0][:, j * c:(j + 1) * c], rkv[1][:, j * c:(j + 1) * c], origin * L + j * c,
                                 flag_ptr, x.epoch))
            else:
                x.release(origin)

        main.wait_event(local_ready)
        return attn_fwd_segments(q, segs, softmax_scale, causal=self.causal, q_off=me * L, out=o, lse=lse)

    # ------------------------------------------------------------------ balanced causal forward
    def _forward_balanced(self, q, kv, o, lse, softmax_scale):
        """Causal forward with equal work per rank.

        The sequence is cut into 2P half-shards; rank r computes the queries of half-shards r and
        2P-1-r (work (r + 1/2) + (2P-1-r + 1/2) = 2P units on every rank).  A rank pulls the query
        half-shards it computes and the K/V shards they can see, and its kernels write o and lse
        straight into the owning rank's result inbox through the peer mapping (stores over NVLink);
        a flag per half tells the owner when its rows are complete.  Layout seen by the caller is
        unchanged: shard k of q, kv, o, lse lives on rank k.
        """
        ctx, P, me, L = self.ctx, self.world, self.rank, self.seq_local
        Lh = L // 2
        B, Hq, D = self.batch, self.hq, self.head_dim
        kv_b = self._kv_bytes()
        q_b = B * L * Hq * D * 2
        lse_b = B * Hq * L * 4
        off_q = _align(kv_b, 256)
        if self._bal_x is None:
            self._bal_x = _ShardExchange(ctx, off_q + _align(q_b, 256))
            self._res_bytes = _align(q_b, 256) + _align(lse_b, 256)
            self._bal_inbox = SymmetricBuffer(ctx, 2 * self._res_bytes + _FLAG_REGION)
        x, inbox = self._bal_x, self._bal_inbox
        main = torch.cuda.current_stream()
        comm = ctx.comm_stream

        slot = x.begin(main)
        s_kv, _ = _carve(slot, 0, self.kv_shape, torch.bfloat16)
        s_q, _ = _carve(slot, off_q, self.q_shape, torch.bfloat16)
        with torch.cuda.stream(comm):
            s_kv.copy_(kv, non_blocking=True)
            s_q.copy_(q, non_blocking=True)
        local_ready = x.publish()
        e = x.epoch
        par = e % 2

        chunks = [2 * P - 1 - me, me]          # heavier half-shard first; its first segment is local
        max_shard = chunks[0] // 2               # K/V shards 0..max_shard are needed
        owners = {c: c // 2 for c in chunks}

        def q_ranges(c):
            half = c % 2
            row_b = Hq * D * 2
            return [(off_q + (b * L + half * Lh) * row_b, Lh * row_b) for b in range(B)]

        # 1. the query half-shards first (small), ordered before the kernels by a stream event
        for c in chunks:
            if owners[c] != me:
                x.pull(owners[c], q_ranges(c), final=False, raise_flag=False)
        q_ready = torch.cuda.Event()
        q_ready.record(comm)
        # 2. the K/V shards, staggered so that ranks start on different sources
        kv_of = {me: (s_kv, None)}
        for t in range(1, P):
            origin = (me - t) % P
            if origin <= max_shard:
                buf, flag_ptr = x.pull(origin, [(0, kv_b)])
                rkv, _ = _carve(buf, 0, self.kv_shape, torch.bfloat16)
                kv_of[origin] = (rkv, flag_ptr)
            elif origin in x._stage_of:
                x.release(origin)   # only its queries were needed
            else:
                x.release(origin)
        pull_order = [me] + [(me - t) % P for t in range(1, P)]

        res_o_off = par * self._res_bytes
        res_l_off = res_o_off + _align(q_b, 256)

        def res_flag(rank, half):
            return inbox.ptr(rank, 2 * self._res_bytes + 8 * par + 4 * half)

        main.wait_event(local_ready)
        main.wait_event(q_ready)
        for c in chunks:
            owner, half = owners[c], c % 2
            rows = slice(half * Lh, (half + 1) * Lh)
            if owner == me:
                qc = q[:, rows]
            else:
                stage = x.staging[x._stage_of[owner]]
                qc = _carve(stage, off_q, self.q_shape, torch.bfloat16)[0][:, rows]
            segs = []
            for origin in pull_order:
                if origin <= c // 2 and origin in kv_of:
                    rkv, flag_ptr = kv_of[origin]
                    segs.append((rkv[0], rkv[1], origin * L) if flag_ptr is None
                                else (rkv[0], rkv[1], origin * L, flag_ptr, e))
            # results go straight into the owner's inbox (its memory is mapped here): raw addresses
            attn_fwd_segments(
                qc, segs, softmax_scale, causal=True, q_off=c * Lh,
                out_raw=(inbox.ptr(owner, res_o_off + half * Lh * Hq * D * 2), L * Hq * D, Hq * D, D),
                lse_raw=(inbox.ptr(owner, res_l_off + half * Lh * 4), Hq * L, L))
            ctx.signal(res_flag(owner, half), e, main)

        # 3. my own rows: wait for whoever computed them, then hand them to the caller
        my_o, _ = _carve(inbox.local.bytes(), res_o_off, self.q_shape, torch.bfloat16)
        my_lse, _ = _carve(inbox.local.bytes(), res_l_off, (B, Hq, L), torch.float32)
        ctx.wait_flag(res_flag(me, 0), e, main)
        ctx.wait_flag(res_flag(me, 1), e, main)
        if o is None:
            o = torch.empty_like(q)
        if lse is None:
            lse = torch.empty((B, Hq, L), dtype=torch.float32, device=q.device)
        o.copy_(my_o, non_blocking=True)
        lse.copy_(my_lse, non_blocking=True)
        return o, lse

    # ------------------------------------------------------------------ backward
    def backward(self, dout: torch.Tensor, q: torch.Tensor, kv: torch.Tensor, o: torch.Tensor, lse: torch.Tensor,
                 dq: Optional[torch.Tensor] = None, dkv: Optional[torch.Tensor] = None,
                 softmax_scale: Optional[float] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """Gradients of this rank's shard: dq like q, dkv like kv ([2,B,S/P,Hkv,D]).
        o and lse are this rank's forward results (lse [B,Hq,S/P])."""
        if tuple(kv.shape) != self.kv_shape or tuple(q.shape) != self.q_shape:
            raise ValueError("q/kv do not match the shapes this object was built for")
        if softmax_scale is None:
            softmax_scale = self.head_dim ** -0.5
        if dq is None:
            dq = torch.empty_like(q)
        if dkv is None:
            dkv = torch.empty_like(kv)
        L = self.seq_local
        me = self.rank
        if self.world == 1:
            stats = bwd_preprocess(dout, o, lse)
            attn_bwd_dq(q, dout, stats, [(kv[0], kv[1], 0)], softmax_scale, causal=self.causal, q_off=0, dq=dq)
            attn_bwd_dkv(kv[0], kv[1], [(q, dout, stats, 0)], softmax_scale, causal=self.causal, k_off=0,
                         dk=dkv[0], dv=dkv[1])
            return dq, dkv

        kv_b = self._kv_bytes()
        q_b = self.batch * L * self.hq * self.head_dim * 2
        st_b = 2 * self.batch * self.hq * self.stat_pad * 4
        off_kv, off_q = 0, _align(kv_b, 256)
        off_do = off_q + _align(q_b, 256)
        off_st = off_do + _align(q_b, 256)
        if self._bwd_x is None:
            assert off_st + _align(st_b, 256) == self._bwd_slot_bytes()
            self._bwd_x = _ShardExchange(self.ctx, self._bwd_slot_bytes())
        x = self._bwd_x
        main = torch.cuda.current_stream()
        comm = self.ctx.comm_stream

        def views(buf):
            v_kv, _ = _carve(buf, off_kv, self.kv_shape, torch.bfloat16)
            v_q, _ = _carve(buf, off_q, self.q_shape, torch.bfloat16)
            v_do, _ = _carve(buf, off_do, self.q_shape, torch.bfloat16)
            v_st, _ = _carve(buf, off_st, self.stat_shape, torch.float32)
            return v_kv, v_q, v_do, v_st

        # statistics of my rows go straight into my slot (main stream), the tensors are copied beside them
        slot_bytes = x.begin(main)
        s_kv, s_q, s_do, s_st = views(slot_bytes)
        with torch.cuda.stream(comm):
            stats = bwd_preprocess(dout, o, lse, workspace=s_st)
            s_kv.copy_(kv, non_blocking=True)
            s_q.copy_(q, non_blocking=True)
            s_do.copy_(dout, non_blocking=True)
        local_ready = x.publish()

        kv_segs = [{"str": s_kv[0], "str_g": s_kv[1], "off": me * L}]
        q_segs = [{"str": s_q, "str_g": s_do, "stats": stats, "off": me * L}]
        for t in range(1, self.world):
            origin = self.order[t]
            need_kv, need_q = self._sees_keys_of(origin), self._seen_by_queries_of(origin)
            if not (need_kv or need_q):
                x.release(origin)
                continue
            ranges = ([(off_kv, kv_b)] if need_kv else []) + ([(off_q, off_st + st_b - off_q)] if need_q else [])
            buf, flag_ptr = x.pull(origin, ranges)
            r_kv, r_q, r_do, r_st = views(buf)
            if need_kv:
                kv_segs.append({"str": r_kv[0], "str_g": r_kv[1], "off": origin * L,
                                "flag": flag_ptr, "flag_value": x.epoch})
            if need_q:
                q_segs.append({"str": r_q, "str_g": r_do, "stats": RowStats(r_st[0], r_st[1], L), "off": origin * L,
                               "flag": flag_ptr, "flag_value": x.epoch})

        main.wait_event(local_ready)
        attn_bwd_dq(q, dout, stats, kv_segs, softmax_scale, causal=self.causal, q_off=me * L, dq=dq, hkv=self.hkv)
        attn_bwd_dkv(kv[0], kv[1], q_segs, softmax_scale, causal=self.causal, k_off=me * L, dk=dkv[0], dv=dkv[1],
                     hq=self.hq)
        return dq, dkv

    # ------------------------------------------------------------------ host-buffer entry
    def forward_host(self, q_host: torch.Tensor, kv_host: torch.Tensor, o_host: torch.Tensor, lse_host: torch.Tensor,
                     softmax_scale: Optional[float] = None, chunks: int = 16) -> None:
        """Forward with pinned HOST tensors in and out (same shapes as forward()).

        Single rank, batch 1: the sequence is cut into `chunks` pieces; chunk i is copied in while
        chunk i-1 is being computed (its queries against the K/V rows that have arrived so far, which
        are contiguous on the device and go in as one segment) and chunk i-2 is copied out, so the PCIe
        transfers in both directions overlap the kernels.  What stays exposed is the last chunk's
        kernel and copy-out, hence many small chunks rather than few large ones.
        Otherwise: copy in, forward(), copy out.  Returns after the results are in host memory.
        """
        dev = torch.device("cuda", torch.cuda.current_device()) if self.ctx is None else self.ctx.device
        if softmax_scale is None:
            softmax_scale = self.head_dim ** -0.5
        L = self.seq_local
        if not hasattr(self, "_host_bufs"):
            self._host_bufs = (torch.empty(self.q_shape, dtype=torch.bfloat16, device=dev),
                               torch.empty(self.kv_shape, dtype=torch.bfloat16, device=dev),
                               torch.empty(self.q_shape, dtype=torch.bfloat16, device=dev),
                               torch.empty((self.batch, self.hq, L), dtype=torch.float32, device=dev),
                               torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev))
        q, kv, o, lse, s_in, s_out = self._host_bufs
        main = torch.cuda.current_stream()
        n = max(1, min(chunks, 64))
        pipelined = self.world == 1 and self.batch == 1 and L % n == 0 and (L // n) % 128 == 0
        if not pipelined:
            q.copy_(q_host, non_blocking=True)
            kv.copy_(kv_host, non_blocking=True)
            self.forward(q, kv, o, lse, softmax_scale)
            o_host.copy_(o, non_blocking=True)
            lse_host.copy_(lse, non_blocking=True)
            main.synchronize()
            return
        c = L // n
        s_in.wait_stream(main)
        s_out.wait_stream(main)
        arrived = []
        for i in range(n):
            rows = slice(i * c, (i + 1) * c)
            with torch.cuda.stream(s_in):
                # contiguous pieces only: strided host<->device copies take a slow staged path
                q[:, rows].copy_(q_host[:, rows], non_blocking=True)
                kv[0][:, rows].copy_(kv_host[0][:, rows], non_blocking=True)
                kv[1][:, rows].copy_(kv_host[1][:, rows], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(s_in)
            arrived.append(ev)
        for i in range(n):
            rows = slice(i * c, (i + 1) * c)
            main.wait_event(arrived[i])
            if self.causal:
                segs = [(kv[0][:, :(i + 1) * c], kv[1][:, :(i + 1) * c], 0)]
            else:
                main.wait_event(arrived[-1])
                segs = [(kv[0], kv[1], 0)]
            attn_fwd_segments(q[:, rows], segs, softmax_scale, causal=self.causal, q_off=i * c, out=o[:, rows],
                              lse=lse[:, :, rows])
            done = torch.cuda.Event()
            done.record(main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                o_host[:, rows].copy_(o[:, rows], non_blocking=True)
                if i == n - 1:
                    lse_host.copy_(lse, non_blocking=True)
        s_out.synchronize()

    def memory_bytes(self, backward: bool = False) -> dict:
        """Device memory this object allocates per rank for its transfers, by kind (the counterpart of
        the reference's per-card buffer model, mercury/ir/calculate_memory.py:9-66, for symmetric slots
        and staging instead of the rotating double buffer): `symmetric` is mapped by every peer (two
        epoch slots per exchange), `staging` holds pulled shards (world - 1 slots per exchange),
        `inbox` receives results computed elsewhere (balanced causal forward).  Flag regions included."""
        if self.world == 1:
            return {"symmetric": 0, "staging": 0, "inbox": 0}
        q_b = self.batch * self.seq_local * self.hq * self.head_dim * 2
        lse_b = self.batch * self.hq * self.seq_local * 4
        kv_b = self._kv_bytes()

        def exchange(slot_bytes):
            slot = _align(slot_bytes, 1024)
            return 2 * slot + _FLAG_REGION, max(self.world - 1, 1) * slot

        sym = stage = inbox = 0
        if self.balanced:
            a, b = exchange(_align(kv_b, 256) + _align(q_b, 256))
            sym, stage = sym + a, stage + b
            inbox = 2 * (_align(q_b, 256) + _align(lse_b, 256)) + _FLAG_REGION
        else:
            a, b = exchange(kv_b)
            sym, stage = sym + a, stage + b
        if backward:
            a, b = exchange(self._bwd_slot_bytes())
            sym, stage = sym + a, stage + b
        return {"symmetric": sym, "staging": stage, "inbox": inbox}

    def check(self) -> None:
        """Synchronise and raise if a device-side wait timed out."""
        if self.ctx is not None:
            self.ctx.check()
        else:
            from . import _lib

            _lib.raise_on_status(torch.cuda.current_stream().cuda_stream)
