"""Fused ring / double-ring / GQA attention for one rank: forward and backward (public API).

`RingAttention.forward` computes what the generated per-rank loop computes
(mercury/backend/pytorch/codegen.py:443-494 + utils/flash_attn_dsl.py:160-179 of
the reference) with ONE attention launch: the K/V shards of all ranks are the
segments of a single launch in the rank's arrival order, so the online-softmax
state stays on chip and no out/LSE merge kernel runs.
`RingAttention.backward` replaces the generated backward loop
(codegen.py:99-190, utils/attn_bwd_dsl.py:70-134) with two launches: dQ of the
local queries over all K/V shards, and dK/dV of the local keys over all query
shards.  Every gradient tile is owned by one CTA, so the reference's rotating
fp32 dK/dV accumulator and its write-back hop have no counterpart here.

Transport.  On an NVSwitch box every peer is one hop away, so a shard is pulled
straight from the rank that owns it instead of being relayed around the ring;
the order in which a rank consumes shards is still the reference's (single ring:
(r - t) mod P; nested rings: mesh.kv_origin_schedule).  Every rank keeps ONE
symmetric slot [kv | q | dout | row statistics] that all peers map.  The copy
engines move each remote shard (or each of its `ring_divide` pieces) over NVLink
into a local staging buffer on high-priority side streams and raise a per-piece
arrival flag behind it; the kernel's loader waits (bounded) on that flag before
its first TMA load of the piece, so compute on what is already here overlaps the
transfers of what is not, inside one launch.  Completion travels the other way
without any host or stream involvement: the last CTA of a job stores the owner's
result flag from the kernel.

Zero-copy operation: `symmetric_buffers()` hands out q / kv / dout / o / lse
tensors that live inside the symmetric memory.  A caller that produces its
inputs there and reads its results from there pays no staging copy at all;
ordinary tensors work too and cost one device-to-device copy per tensor.

World size 1 is the unsharded program: one segment, no transport.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from . import _lib, mesh
from .attention import (RowStats, _bwd_launch, _pad64, attn_bwd_dkv, attn_bwd_dq, attn_bwd_fused, attn_fwd_multi,
                        attn_fwd_segments, bwd_preprocess, dq_convert_raw)
from .comm import PeerContext, SymmetricBuffer, _align, default_context

_FLAG_REGION = 4096
_MAX_PIECES = 32          # arrival flags per staging slot
_READY, _DONE, _RES = 0, 256, 512   # byte offsets of the flag groups inside the flag region


def _carve(buf: torch.Tensor, offset: int, shape, dtype) -> Tuple[torch.Tensor, int]:
    n = 1
    for s in shape:
        n *= int(s)
    nbytes = n * torch.empty((), dtype=dtype).element_size()
    return buf[offset:offset + nbytes].view(dtype).view(*shape), offset + _align(nbytes, 256)


class _Exchange:
    """One symmetric slot per rank plus an optional result inbox, local staging, and the flags.

    Symmetric memory of a rank: [slot | inbox | flag region].  Flag words (int32, values are epoch
    numbers, which only grow):
        ready[origin]  on every rank   `origin` has published its slot for this epoch
        done[reader]   on the owner    `reader` has finished pulling the owner's slot of this epoch
        res[i]         on the owner    result part i of this epoch is complete in the owner's inbox
    Local memory: world - 1 staging slots, and int32 words for piece arrival flags
    [stage * 32 + piece], query arrival flags and the kernels' completion counters.
    """

    def __init__(self, ctx: PeerContext, slot_bytes: int, inbox_bytes: int, staging: bool = True):
        self.ctx = ctx
        self.world, self.rank = ctx.world, ctx.rank
        self.slot_bytes = _align(slot_bytes, 1024)
        self.inbox_bytes = _align(inbox_bytes, 1024) if inbox_bytes else 0
        self.sym = SymmetricBuffer(ctx, self.slot_bytes + self.inbox_bytes + _FLAG_REGION)
        self._flag_off = self.slot_bytes + self.inbox_bytes
        self.staging = torch.empty((max(self.world - 1, 1) if staging else 0, self.slot_bytes), dtype=torch.uint8,
                                   device=ctx.device)
        # piece arrival flags | 16 auxiliary words
        self.words = torch.zeros(max(self.world - 1, 1) * _MAX_PIECES + 16, dtype=torch.int32, device=ctx.device)
        self.epoch = 0
        self._waited = set()
        torch.cuda.synchronize(ctx.device)

    # -- addresses ---------------------------------------------------------------------------
    def ready_ptr(self, on_rank: int, origin: int) -> int:
        return self.sym.ptr(on_rank, self._flag_off + _READY + 4 * origin)

    def done_ptr(self, on_rank: int, reader: int) -> int:
        return self.sym.ptr(on_rank, self._flag_off + _DONE + 4 * reader)

    def res_ptr(self, on_rank: int, part: int) -> int:
        return self.sym.ptr(on_rank, self._flag_off + _RES + 4 * part)

    def inbox_ptr(self, on_rank: int, offset: int = 0) -> int:
        return self.sym.ptr(on_rank, self.slot_bytes + offset)

    def slot(self) -> torch.Tensor:
        return self.sym.local.bytes()[:self.slot_bytes]

    def inbox(self) -> torch.Tensor:
        return self.sym.local.bytes()[self.slot_bytes:self.slot_bytes + self.inbox_bytes]

    def stage_index(self, origin: int) -> int:
        return origin if origin < self.rank else origin - 1

    def stage(self, origin: int) -> torch.Tensor:
        return self.staging[self.stage_index(origin)]

    def piece_flag_ptr(self, origin: int, piece: int = 0) -> int:
        if not 0 <= piece < _MAX_PIECES:
            raise ValueError(f"a staging slot has {_MAX_PIECES} arrival flags")
        return self.words.data_ptr() + 4 * (self.stage_index(origin) * _MAX_PIECES + piece)

    def aux_ptr(self, i: int) -> int:
        """Sixteen further local words: query arrival flags (0..7) and completion counters (8..15)."""
        return self.words.data_ptr() + 4 * (max(self.world - 1, 1) * _MAX_PIECES + i)

    def stream_of(self, origin: int) -> torch.cuda.Stream:
        """Every pull from one origin runs on one stream, so its last pull is behind all the others."""
        s = self.ctx.comm_streams
        return s[origin % len(s)]

    # -- protocol ----------------------------------------------------------------------------
    def begin(self, main: torch.cuda.Stream) -> int:
        """Start a new epoch: transfers are ordered behind everything queued on `main` so far (the
        previous epoch's kernels read the staging slots that are about to be overwritten)."""
        self.epoch += 1
        self._waited = set()
        for s in self.ctx.comm_streams:
            s.wait_stream(main)
        return self.epoch

    def wait_slot_free(self, peers: Sequence[int]) -> None:
        """Before overwriting my slot: every peer has finished pulling the previous epoch."""
        if self.epoch > 1:
            flags = [(self.done_ptr(self.rank, p), self.epoch - 1) for p in peers if p != self.rank]
            self.ctx.wait_many(flags, self.ctx.comm_stream)

    def publish(self, peers: Sequence[int]) -> torch.cuda.Event:
        """Announce my slot to every peer (one launch); the event fires once the slot is in place."""
        comm = self.ctx.comm_stream
        ev = torch.cuda.Event()
        ev.record(comm)
        self.ctx.signal_many([(self.ready_ptr(p, self.rank), self.epoch) for p in peers if p != self.rank], comm)
        return ev

    def pull(self, origin: int, ranges: Sequence[Tuple[int, int]], raise_after: Sequence[Tuple[int, int]] = (),
             last: bool = False) -> torch.Tensor:
        """Copy (offset, nbytes) ranges of `origin`'s slot into its staging slot over NVLink (copy
        engines), then raise the given (flag address, value) pairs with one launch.  last=True also
        tells the owner that this rank is done with its slot."""
        ctx, st = self.ctx, self.stream_of(origin)
        dst = self.stage(origin)
        flags = list(raise_after)
        if last:
            flags.append((self.done_ptr(origin, self.rank), self.epoch))
        if origin not in self._waited:
            self._waited.add(origin)
            ctx.wait_flag(self.ready_ptr(self.rank, origin), self.epoch, st)
        for off, nbytes in ranges:
            ctx.copy(dst.data_ptr() + off, self.sym.ptr(origin, off), nbytes, st)
        if flags:
            ctx.signal_many(flags, st)
        return dst

    def pull_rects(self, origin: int, rects: Sequence[Tuple[int, int, int, int, int]],
                   raise_after: Sequence[Tuple[int, int]] = (), last: bool = False) -> None:
        """Like pull, for rectangles (destination address, slot offset, slot row pitch, width, height) in
        bytes: `height` rows of `width` bytes of `origin`'s slot land densely packed at the destination (the
        origin's staging slot or any other local buffer)."""
        ctx, st = self.ctx, self.stream_of(origin)
        if origin not in self._waited:
            self._waited.add(origin)
            ctx.wait_flag(self.ready_ptr(self.rank, origin), self.epoch, st)
        for dst_ptr, src_off, spitch, width, height in rects:
            ctx.copy2d(dst_ptr, width, self.sym.ptr(origin, src_off), spitch, width, height, st)
        flags = list(raise_after)
        if last:
            flags.append((self.done_ptr(origin, self.rank), self.epoch))
        if flags:
            ctx.signal_many(flags, st)

    def release(self, origins: Sequence[int]) -> None:
        """Tell these owners that this rank will not read their slots of this epoch (one launch)."""
        flags = [(self.done_ptr(o, self.rank), self.epoch) for o in origins if o != self.rank]
        if flags:
            self.ctx.signal_many(flags, self.ctx.comm_stream)


class RingAttention:
    """Attention of one rank of a sequence-sharded job.

    mesh_shape (P,) is the single ring, (n_inner, n_outer) the double ring (inner ring over
    mesh dimension 0, rank = inner + n_inner * outer).  Shard k of the sequence lives on rank k.
    With causal=True a key is visible iff its global position is <= the query's.
    backward=True reserves room for dout and the row statistics in the symmetric slot; it is needed
    to call backward() on more than one rank.
    """

    def __init__(self, mesh_shape: Sequence[int], batch: int, seq_local: int, hq: int, hkv: int,
                 head_dim: int = 128, causal: bool = False, ctx: Optional[PeerContext] = None,
                 balance_causal: bool = True, ring_divide: int = 1, backward: bool = False,
                 schedule: Optional[str] = None):
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
        self.lse_shape = (batch, hq, seq_local)
        self.stat_pad = _pad64(seq_local)
        self.stat_shape = (2, batch, hq, self.stat_pad)
        self.with_backward = bool(backward)
        # Remote shards travel on the copy engines (cudaMemcpyAsync between a flag-wait and a flag-signal
        # kernel on per-origin streams): measured between two B200s they move 726 GB/s alone and 521 GB/s
        # beside a resident attention kernel, against 638 / 429 GB/s for the SM-issued bulk copies of
        # mb_pull_sm, and they take no SM resources.
        self.launches_per_forward = 1
        self.launches_per_backward = 3
        self._x: Optional[_Exchange] = None
        self._state: Optional[List[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]]] = None
        self._monitor = getattr(self.ctx, "monitor", None) or _lib.StatusMonitor()
        # Causal attention over contiguous shards gives rank r (r + 1/2) blocks of forward work.  With
        # balancing, the forward re-assigns query half-shards so that every rank computes the same
        # amount; inputs and outputs keep the contiguous layout.  The backward
        # needs no such re-assignment: rank r does (r + 1/2) blocks of dQ work and (P - r - 1/2) blocks
        # of dK/dV work, P blocks on every rank.
        self.balanced = bool(balance_causal) and self.causal and self.world > 1 and seq_local % 2 == 0
        # Forward schedule.  "ring": every rank keeps its query rows (or, balanced causal, two half-shards) and
        # pulls whole K/V shards.  "heads": every rank computes ALL query rows for hq / world of the heads; it
        # pulls that head group's slice of q, k and v from every peer (an all-to-all through NVSwitch, 1/world
        # of the bytes of the ring per shard) and its kernel stores the rows of other ranks straight into their
        # o / lse.  Causal work is then the same on every rank by construction.  It is the head-parallel split
        # of the reference's search space (mercury/search) applied inside the call: inputs and outputs keep
        # the sequence-sharded layout.  Default (None, or MB_SCHEDULE): "heads" on a one-dimensional mesh of up
        # to 8 ranks when both head counts divide by the world size and balance_causal is on, else "ring".
        # The heads schedule's backward is head-parallel too (_backward_heads).
        schedule = schedule or os.environ.get("MB_SCHEDULE") or None
        can_heads = (self.world > 1 and len(self.mesh_shape) == 1 and self.world <= 8 and hq % self.world == 0
                     and hkv % self.world == 0 and self.world <= _lib.MB_MAX_SEGMENTS)
        if schedule is None:
            schedule = "heads" if can_heads and balance_causal and int(ring_divide) == 1 else "ring"
        if schedule not in ("ring", "heads"):
            raise ValueError("schedule must be 'ring' or 'heads'")
        if schedule == "heads" and not can_heads:
            raise ValueError("the heads schedule needs a one-dimensional mesh of 2..8 ranks and head counts "
                             "that divide by the world size")
        self.schedule = schedule if self.world > 1 else "ring"
        self.heads = self.schedule == "heads"
        if self.heads:
            self.balanced = False
        self._inbox_layout = self.balanced or self.heads   # peers pull q, results arrive in a symmetric o / lse
        # ring_divide (the rounds parameter of the reference's shift primitive, ir/primitives.py:33-45,
        # 101-102): every K/V shard travels as `ring_divide` sequence pieces, each with its own arrival
        # flag and its own segment of the launch, so work on a shard starts when its first piece is in.
        # One launch takes at most MB_MAX_SEGMENTS segments: 1 local + (world - 1) * ring_divide.
        self.ring_divide = int(ring_divide)
        if self.ring_divide < 1 or seq_local % self.ring_divide != 0:
            raise ValueError("ring_divide must divide the local sequence length")
        if 1 + (self.world - 1) * self.ring_divide > _lib.MB_MAX_SEGMENTS or self.ring_divide > _MAX_PIECES:
            raise ValueError(f"1 + (world - 1) * ring_divide segments exceed the {_lib.MB_MAX_SEGMENTS} of one launch")
        # byte layout of the slot and of the inbox
        self._kv_b = 2 * batch * seq_local * hkv * head_dim * 2
        self._q_b = batch * seq_local * hq * head_dim * 2
        self._lse_b = batch * hq * seq_local * 4
        self._st_b = 2 * batch * hq * self.stat_pad * 4
        self._off_kv = 0
        self._off_q = _align(self._kv_b, 256)
        self._off_do = self._off_q + _align(self._q_b, 256)
        self._off_st = self._off_do + _align(self._q_b, 256)
        # the slot holds what peers pull: K/V always; the queries when peers compute some of this rank's rows
        # (balanced forward) or its keys' gradients (backward); dout and the statistics for the backward
        if self.with_backward:
            self._slot_bytes = self._off_st + _align(self._st_b, 256)
        else:
            self._slot_bytes = self._off_do if self._inbox_layout else self._off_q
        self._inbox_o, self._inbox_lse = 0, _align(self._q_b, 256)
        self._inbox_bytes = (self._inbox_lse + _align(self._lse_b, 256)) if self._inbox_layout else 0
        # heads schedule with backward: the gradients of this rank's rows arrive head group by head group
        self._inbox_dq = self._inbox_bytes
        self._inbox_dkv = self._inbox_dq + _align(self._q_b, 256)
        if self.heads and self.with_backward:
            self._inbox_bytes = self._inbox_dkv + _align(self._kv_b, 256)
        if self.with_backward and self.ring_divide > 1 and (seq_local // self.ring_divide) % 64 != 0:
            raise ValueError("with backward=True the pieces of ring_divide must be multiples of 64 rows "
                             "(the row statistics travel in 64-row blocks)")
        self.last_launches = 0   # kernels this object launched in its latest forward() / backward()
        # World size 1 runs the backward as one sweep whose dq depends on the order of fp32 additions; set
        # this to get the two-launch form, which is bitwise reproducible.  (On several ranks the ring
        # schedule always uses the two-launch form -- it needs no cross-rank reduction of dq contributions --
        # and the heads schedule always the sweep.)
        self.deterministic_backward = False

    # ------------------------------------------------------------------ helpers
    def _sees_keys_of(self, origin: int) -> bool:
        """Whether this rank's queries can see any key of `origin`'s shard."""
        return (not self.causal) or origin <= self.rank

    def _seen_by_queries_of(self, origin: int) -> bool:
        """Whether `origin`'s queries can see any key of this rank's shard."""
        return (not self.causal) or origin >= self.rank

    def _exchange(self) -> _Exchange:
        if self._x is None:
            self._x = _Exchange(self.ctx, self._slot_bytes, self._inbox_bytes)
            slot, inbox = self._x.slot(), self._x.inbox()
            self._s_kv, _ = _carve(slot, self._off_kv, self.kv_shape, torch.bfloat16)
            if self._slot_bytes > self._off_q:
                self._s_q, _ = _carve(slot, self._off_q, self.q_shape, torch.bfloat16)
            else:   # nobody pulls this rank's queries: an ordinary tensor serves symmetric_buffers()
                self._s_q = torch.empty(self.q_shape, dtype=torch.bfloat16, device=self.ctx.device)
            if self.with_backward:
                self._s_do, _ = _carve(slot, self._off_do, self.q_shape, torch.bfloat16)
                self._s_st, _ = _carve(slot, self._off_st, self.stat_shape, torch.float32)
            if self.heads and self.with_backward:
                self._s_dq, _ = _carve(inbox, self._inbox_dq, self.q_shape, torch.bfloat16)
                self._s_dkv, _ = _carve(inbox, self._inbox_dkv, self.kv_shape, torch.bfloat16)
            if self._inbox_layout:
                self._s_o, _ = _carve(inbox, self._inbox_o, self.q_shape, torch.bfloat16)
                self._s_lse, _ = _carve(inbox, self._inbox_lse, self.lse_shape, torch.float32)
            else:   # results are written by this rank's own kernel: ordinary tensors
                self._s_o, self._s_lse = self._plain_outputs(self.ctx.device)
        return self._x

    def _stage_views(self, origin: int):
        buf = self._x.stage(origin)
        kv, _ = _carve(buf, self._off_kv, self.kv_shape, torch.bfloat16)
        if self._slot_bytes <= self._off_q:     # K/V only: nobody pulls queries in this configuration
            return kv, None, None, None
        q, _ = _carve(buf, self._off_q, self.q_shape, torch.bfloat16)
        if not self.with_backward:
            return kv, q, None, None
        do, _ = _carve(buf, self._off_do, self.q_shape, torch.bfloat16)
        st, _ = _carve(buf, self._off_st, self.stat_shape, torch.float32)
        return kv, q, do, st

    def symmetric_buffers(self) -> Dict[str, torch.Tensor]:
        """Tensors inside this rank's symmetric memory: q, kv (and dout with backward=True) to produce
        the inputs in, o and lse to read the results from.  Passing exactly these to forward() /
        backward() skips every staging copy.  Peers read q / kv / dout straight from here, so before
        OVERWRITING them after a call, call inputs_writable(); o and lse are rewritten by the next
        forward() (by kernels on other ranks), so consume them on the current stream before calling it.
        World size 1 has no symmetric memory: ordinary tensors are returned."""
        if self.world == 1:
            dev = torch.device("cuda", torch.cuda.current_device())
            out = {"q": torch.empty(self.q_shape, dtype=torch.bfloat16, device=dev),
                   "kv": torch.empty(self.kv_shape, dtype=torch.bfloat16, device=dev),
                   "o": torch.empty(self.q_shape, dtype=torch.bfloat16, device=dev),
                   "lse": torch.empty(self.lse_shape, dtype=torch.float32, device=dev)}
            if self.with_backward:
                out["dout"] = torch.empty(self.q_shape, dtype=torch.bfloat16, device=dev)
            return out
        self._exchange()
        # o / lse: the symmetric inbox when results are computed on other ranks (balanced causal forward),
        # ordinary tensors of this object otherwise
        out = {"q": self._s_q, "kv": self._s_kv, "o": self._s_o, "lse": self._s_lse}
        if self.with_backward:
            out["dout"] = self._s_do
            if self.heads:      # gradients arrive here; passing these to backward() skips the copy-out
                out["dq"], out["dkv"] = self._s_dq, self._s_dkv
        return out

    def inputs_writable(self) -> None:
        """Make the current stream wait until every peer has finished reading this rank's symmetric
        q / kv / dout of the last call (one small kernel).  Call before overwriting those tensors."""
        if self.world > 1 and self._x is not None and self._x.epoch > 0:
            x = self._x
            flags = [(x.done_ptr(self.rank, p), x.epoch) for p in range(self.world) if p != self.rank]
            self.ctx.wait_many(flags, torch.cuda.current_stream())

    @staticmethod
    def _same(a: torch.Tensor, b: torch.Tensor) -> bool:
        return a.data_ptr() == b.data_ptr() and a.shape == b.shape and a.stride() == b.stride()

    def _kv_piece_ranges(self, j: int) -> List[Tuple[int, int]]:
        """Byte ranges of rows [j c, (j+1) c) of K and of V inside a slot, for every batch entry."""
        c = self.seq_local // self.ring_divide
        row_b = self.hkv * self.head_dim * 2
        return [(self._off_kv + ((w * self.batch + b) * self.seq_local + j * c) * row_b, c * row_b)
                for w in range(2) for b in range(self.batch)]

    def _q_rows_ranges(self, base_off: int, r0: int, r1: int) -> List[Tuple[int, int]]:
        """Byte ranges of query rows [r0, r1) of a [B, L, Hq, D] bf16 tensor at base_off in a slot."""
        row_b = self.hq * self.head_dim * 2
        return [(base_off + (b * self.seq_local + r0) * row_b, (r1 - r0) * row_b) for b in range(self.batch)]

    def _shard_major_jobs(self, chunks: List[dict], order: Sequence[int], shard_bits: dict, epoch: int,
                          chunk_step: Optional[Sequence[int]] = None, hq: Optional[int] = None) -> List[dict]:
        """Cut every query chunk's work into one job per K/V shard, in the order the shards arrive, and list
        the jobs shard by shard: CTAs are dispatched in job order, so the SMs first do everything that
        needs only the local shard, then everything that needs the first pulled shard, and so on -- no CTA
        holds an SM while it waits for a shard that is still in flight (a CTA that walks through all the
        shards itself does: the first wave consumes shards faster than NVLink delivers them).  The jobs
        of a chunk hand the online-softmax state on through fp32 scratch and chain words; the last one
        writes the result.  chunk_step[i] is the step at which chunk i's queries arrive (default 0: with
        the first shard); its first job then takes every shard that has arrived by then.  More shards than
        job slots: consecutive shards share a job."""
        L = self.seq_local
        hq = self.hq if hq is None else hq
        chunk_step = list(chunk_step) if chunk_step is not None else [0] * len(chunks)
        group = 1
        while True:
            steps = [list(order[i:i + group]) for i in range(0, len(order), group)]
            plan: List[Tuple[int, int, int]] = []             # (step, chunk index, segment mask)
            for t, shards in enumerate(steps):
                for ci, ch in enumerate(chunks):
                    first_t = chunk_step[ci] // group
                    if t < first_t:
                        continue
                    rows = ch["q"].shape[1]
                    mask = 0
                    for tt in (range(t + 1) if t == first_t else (t,)):
                        for og in steps[tt]:
                            if (not self.causal) or og * L <= ch["q_off"] + rows - 1:     # its first key is visible
                                mask |= shard_bits[og]
                    if mask:
                        plan.append((t, ci, mask))
            if len(plan) <= _lib.MB_MAX_JOBS or group >= len(order):
                break
            group += 1
        count = [sum(1 for _, ci, _ in plan if ci == i) for i in range(len(chunks))]
        if self._state is None:
            dev = chunks[0]["q"].device
            self._state = []
            for ch in chunks:
                rows = ch["q"].shape[1]
                self._state.append((torch.empty((self.batch, hq, rows, self.head_dim), dtype=torch.float32, device=dev),
                                    torch.empty((self.batch, hq, rows, 2), dtype=torch.float32, device=dev),
                                    torch.zeros((self.batch, hq, (rows + 255) // 256), dtype=torch.int32, device=dev)))
        base = (epoch % (1 << 24)) * 64                   # chain values only grow; restart with cleared words
        if base == 0:
            for _, _, chain in self._state:
                chain.zero_()
        seen = [0] * len(chunks)
        out: List[dict] = []
        for t, ci, mask in plan:
            ch = chunks[ci]
            p, n = seen[ci], count[ci]
            seen[ci] += 1
            jb = {"q": ch["q"], "q_off": ch["q_off"], "seg_mask": mask}
            if "q_flag" in ch:
                jb["q_flag"] = ch["q_flag"]
            if n > 1:
                so, sml, chain = self._state[ci]
                jb.update(state=(so, sml), state_in=p > 0, state_out=p < n - 1,
                          chain=(chain.data_ptr(), base + p, base + p + 1))
            if p == n - 1:
                jb["out_raw"], jb["lse_raw"] = ch["out_raw"], ch["lse_raw"]
                if "done" in ch:
                    jb["done"] = ch["done"]
            out.append(jb)
        for ci, ch in enumerate(chunks):
            if count[ci] == 0:                            # sees no key at all: one job that writes zeros / -inf
                out.append({k: v for k, v in ch.items()} | {"seg_mask": 0})
        return out

    def _launch_heads(self, q: torch.Tensor, kv: torch.Tensor, x: _Exchange, e: int, softmax_scale: float) -> None:
        """Forward of the heads schedule: this rank computes ALL query rows for heads
        [rank * hq / P, (rank + 1) * hq / P).  From every peer it pulls that head group's rectangle of q and
        of k | v (rows of hq/P * D resp. hkv/P * D elements out of rows of hq * D resp. hkv * D) into the
        peer's staging slot, densely packed, and raises one arrival flag per peer.  One launch: a chain of
        jobs per peer's query rows, ordered by arrival; the last job of a chain stores o / lse for this head
        group straight into the owner's memory and raises the owner's flag for this rank."""
        P, me, L, B, D = self.world, self.rank, self.seq_local, self.batch, self.head_dim
        Hl, hkl = self.hq // P, self.hkv // P
        q_w, kv_w = Hl * D * 2, hkl * D * 2                       # bytes per row of a head group
        q_rect_b = B * L * q_w
        order = [me] + [(me - t) % P for t in range(1, P)]        # every rank starts at another origin
        segs: List[tuple] = []
        chunks: List[dict] = []
        shard_bits = {}
        for n, og in enumerate(order):
            if og == me:
                qv = q[:, :, me * Hl:(me + 1) * Hl]
                kvv = kv[:, :, :, me * hkl:(me + 1) * hkl]
                flag = None
            else:
                buf = x.stage(og)
                flag = x.piece_flag_ptr(og, 0)
                x.pull_rects(og, [(buf.data_ptr(), self._off_q + me * q_w, self.hq * D * 2, q_w, B * L),
                                  (buf.data_ptr() + _align(q_rect_b, 256), self._off_kv + me * kv_w, self.hkv * D * 2,
                                   kv_w, 2 * B * L)],
                             raise_after=[(flag, e)], last=True)
                qv, _ = _carve(buf, 0, (B, L, Hl, D), torch.bfloat16)
                kvv, _ = _carve(buf, _align(q_rect_b, 256), (2, B, L, hkl, D), torch.bfloat16)
            segs.append((kvv[0], kvv[1], og * L) + ((flag, e) if flag is not None else ()))
            shard_bits[og] = 1 << n
            ch = {"q": qv, "q_off": og * L,
                  "out_raw": (x.inbox_ptr(og, self._inbox_o + me * q_w), L * self.hq * D, self.hq * D, D),
                  "lse_raw": (x.inbox_ptr(og, self._inbox_lse + me * Hl * L * 4), self.hq * L, L),
                  "done": (x.res_ptr(og, me), e, x.aux_ptr(8 + n))}
            if flag is not None:
                ch["q_flag"] = (flag, e)
            chunks.append(ch)
        jobs = self._shard_major_jobs(chunks, order, shard_bits, e, chunk_step=list(range(P)), hq=Hl)
        attn_fwd_multi(jobs, segs, softmax_scale, self.causal, B, Hl, hkl, D, q.device)

    # ------------------------------------------------------------------ forward
    def forward(self, q: torch.Tensor, kv: torch.Tensor, o: Optional[torch.Tensor] = None,
                lse: Optional[torch.Tensor] = None, softmax_scale: Optional[float] = None
                ) -> Tuple[torch.Tensor, torch.Tensor]:
        """q [B,S/P,Hq,D], kv [2,B,S/P,Hkv,D] bf16 on this rank's device -> (o, lse [B,Hq,S/P])."""
        if tuple(kv.shape) != self.kv_shape or tuple(q.shape) != self.q_shape:
            raise ValueError(f"q / kv must have shapes {self.q_shape} / {self.kv_shape}, "
                             f"got {tuple(q.shape)} / {tuple(kv.shape)}")
        if softmax_scale is None:
            softmax_scale = self.head_dim ** -0.5
        self._monitor.poll()
        L = self.seq_local
        if self.world == 1:
            res = attn_fwd_segments(q, [(kv[0], kv[1], 0)], softmax_scale, causal=self.causal, q_off=0, out=o, lse=lse)
            self._monitor.post(torch.cuda.current_stream())
            return res

        ctx, P, me = self.ctx, self.world, self.rank
        x = self._exchange()
        launches0 = ctx.launch_count
        main = torch.cuda.current_stream()
        comm = ctx.comm_stream
        e = x.begin(main)
        peers = range(P)
        zero_in = self._same(kv, self._s_kv) and (not self._inbox_layout or self._same(q, self._s_q))
        if not zero_in:
            x.wait_slot_free(peers)
            with torch.cuda.stream(comm):
                self._s_kv.copy_(kv, non_blocking=True)
                if self._inbox_layout:
                    self._s_q.copy_(q, non_blocking=True)
        x.publish(peers)

        B, Hq, D = self.batch, self.hq, self.head_dim
        if o is None:
            o = self._s_o if self._inbox_layout else torch.empty_like(q)
        if lse is None:
            lse = self._s_lse if self._inbox_layout else torch.empty(self.lse_shape, dtype=torch.float32,
                                                                    device=q.device)
        if tuple(lse.shape) != self.lse_shape or lse.dtype != torch.float32 or lse.stride(2) != 1:
            raise ValueError("lse must be an fp32 [batch, hq, seq] tensor with contiguous rows")
        if tuple(o.shape) != self.q_shape or o.dtype != torch.bfloat16 or o.stride(3) != 1:
            raise ValueError("o must be a bf16 tensor shaped like q with a contiguous head_dim")

        if self.heads:
            self._launch_heads(q, kv, x, e, softmax_scale)    # the local head group is read from the caller's tensors
            # my rows: every rank (this one included) delivers its head group
            ctx.wait_many([(x.res_ptr(me, p), e) for p in range(P)], main)
            if not self._same(o, self._s_o):
                o.copy_(self._s_o, non_blocking=True)
            if not self._same(lse, self._s_lse):
                lse.copy_(self._s_lse, non_blocking=True)
            self._monitor.post(main)
            self.last_launches = ctx.launch_count - launches0 + 1
            return o, lse

        # ---- which query rows this rank computes, and where their results go
        jobs: List[dict] = []
        q_pulls: List[Tuple[int, List[Tuple[int, int]], int]] = []   # (owner, ranges, index of the arrival flag)
        if self.balanced:
            # The sequence is cut into 2P half-shards; rank r computes the queries of half-shards 2P-1-r and
            # r: (2P-1-r + 1/2) + (r + 1/2) = 2P units of work on every rank.  Results go straight into the
            # owning rank's inbox through the peer mapping (stores over NVLink from the kernel's epilogue),
            # and the job's last CTA raises the owner's flag for that half.
            Lh = L // 2
            for idx, c in enumerate((2 * P - 1 - me, me)):      # heavier half-shard first
                owner, half = c // 2, c % 2
                rows = slice(half * Lh, (half + 1) * Lh)
                job = {"q_off": c * Lh,
                       "out_raw": (x.inbox_ptr(owner, self._inbox_o + half * Lh * Hq * D * 2), L * Hq * D, Hq * D, D),
                       "lse_raw": (x.inbox_ptr(owner, self._inbox_lse + half * Lh * 4), Hq * L, L),
                       "done": (x.res_ptr(owner, half), e, x.aux_ptr(8 + idx))}
                if owner == me:
                    job["q"] = q[:, rows]
                else:
                    job["q"] = self._stage_views(owner)[1][:, rows]
                    job["q_flag"] = (x.aux_ptr(idx), e)
                    q_pulls.append((owner, self._q_rows_ranges(self._off_q, half * Lh, (half + 1) * Lh), idx))
                jobs.append(job)
            max_shard = (2 * P - 1 - me) // 2       # K/V shards 0..max_shard are visible to some query here
            # Pull order: every rank starts at another origin.  Up to four ranks (me+1, me+2, ...): the ranks near
            # P-1 -- which see nothing of their own shard and whose work is almost all on the low shards -- get
            # shards 0, 1, ... first (measured at four GPUs: 2.34 ms against 2.42 for the other direction).  Beyond
            # that (me-1, me-2, ...): a fluid model of the transfers (shared egress of an origin, one ingress
            # stream per rank) that reproduces both four-GPU figures puts it ahead at eight ranks, where the step
            # is bound by the 7 x 64 MiB that ranks 0 and 1 receive.  MB_PULL_ORDER=up|down overrides.
            sign = {"up": 1, "down": -1}.get(os.environ.get("MB_PULL_ORDER", ""), 1 if P <= 4 else -1)
            needed = [og for og in ((me + sign * t) % P for t in range(1, P)) if og <= max_shard]
        else:
            jobs.append({"q": q, "q_off": me * L,
                         "out_raw": (o.data_ptr(), o.stride(0), o.stride(1), o.stride(2)),
                         "lse_raw": (lse.data_ptr(), lse.stride(0), lse.stride(1))})
            needed = [og for og in self.order[1:] if self._sees_keys_of(og)]

        # ---- transfers: owners nobody here reads are released at once.  Order: the first job's queries, the
        # first K/V shard, the other queries (their job comes after a few waves of the first one), then the
        # remaining K/V shards in consumption order, piece by piece.  The last pull from an owner also tells
        # it that this rank is done with its slot.
        q_owners = {owner for owner, _, _ in q_pulls}
        x.release([og for og in range(P) if og != me and og not in needed and og not in q_owners])
        d, c = self.ring_divide, L // self.ring_divide
        segs: List[tuple] = [(kv[0], kv[1], me * L)]
        shard_bits = {me: 1}                                  # origin -> bit mask of its segments
        kv_pulls: List[List[tuple]] = []                      # per needed shard: its pieces' pull arguments
        for og in needed:
            rkv = self._stage_views(og)[0]
            first = len(segs)
            pieces = []
            for j in range(d):
                flag = x.piece_flag_ptr(og, j)
                pieces.append((og, self._kv_piece_ranges(j) if d > 1 else [(self._off_kv, self._kv_b)], [(flag, e)]))
                rows = slice(j * c, (j + 1) * c)
                segs.append((rkv[0][:, rows], rkv[1][:, rows], og * L + j * c, flag, e))
            kv_pulls.append(pieces)
            shard_bits[og] = ((1 << d) - 1) << first
        q_ops = [(owner, ranges, [(x.aux_ptr(idx), e)]) for owner, ranges, idx in q_pulls]
        first_q = [op_ for op_, (_, _, idx) in zip(q_ops, q_pulls) if idx == 0]
        ops = first_q + (kv_pulls[0] if kv_pulls else []) + [op_ for op_ in q_ops if op_ not in first_q]
        for pieces in kv_pulls[1:]:
            ops += pieces
        last_of = {origin: n for n, (origin, _, _) in enumerate(ops)}
        for n, (origin, ranges, flags) in enumerate(ops):
            x.pull(origin, ranges, raise_after=flags, last=last_of[origin] == n)

        attn_fwd_multi(self._shard_major_jobs(jobs, [me] + needed, shard_bits, e), segs, softmax_scale, self.causal,
                       B, Hq, self.hkv, D, q.device)

        if self.balanced:
            # my own rows: wait for whoever computed them (one launch for both halves)
            ctx.wait_many([(x.res_ptr(me, 0), e), (x.res_ptr(me, 1), e)], main)
            if not self._same(o, self._s_o):
                o.copy_(self._s_o, non_blocking=True)
            if not self._same(lse, self._s_lse):
                lse.copy_(self._s_lse, non_blocking=True)
        self._monitor.post(main)
        self.last_launches = ctx.launch_count - launches0 + 1
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
        self._monitor.poll()
        L = self.seq_local
        me = self.rank
        if self.world == 1:
            stats = bwd_preprocess(dout, o, lse)
            if self.deterministic_backward:
                attn_bwd_dq(q, dout, stats, [(kv[0], kv[1], 0)], softmax_scale, causal=self.causal, q_off=0, dq=dq)
                attn_bwd_dkv(kv[0], kv[1], [(q, dout, stats, 0)], softmax_scale, causal=self.causal, k_off=0,
                             dk=dkv[0], dv=dkv[1])
            else:
                # one sweep: scores computed once, dQ contributions added in fp32 (see attn_bwd_fused)
                if getattr(self, "_dq_accum", None) is None:
                    self._dq_accum = torch.empty((self.batch, self.hq, self.stat_pad, self.head_dim),
                                                 dtype=torch.float32, device=q.device)
                self._dq_accum.zero_()
                attn_bwd_fused(q, dout, stats, kv[0], kv[1], softmax_scale, causal=self.causal, q_off=0, k_off=0,
                               dq=dq, dk=dkv[0], dv=dkv[1], dq_accum=self._dq_accum)
            self._monitor.post(torch.cuda.current_stream())
            return dq, dkv
        if not self.with_backward:
            raise ValueError("construct RingAttention with backward=True to call backward() on more than one rank")

        ctx, P = self.ctx, self.world
        x = self._exchange()
        if self.heads:
            return self._backward_heads(dout, q, kv, o, lse, dq, dkv, softmax_scale)
        launches0 = ctx.launch_count
        main = torch.cuda.current_stream()
        comm = ctx.comm_stream
        e = x.begin(main)
        peers = range(P)
        zero_in = self._same(kv, self._s_kv) and self._same(q, self._s_q) and self._same(dout, self._s_do)
        # always: this call itself rewrites the row statistics inside the slot
        x.wait_slot_free(peers)
        with torch.cuda.stream(comm):
            # statistics of my rows go straight into my slot, the tensors are copied beside them
            stats = bwd_preprocess(dout, o, lse, workspace=self._s_st)
            if not zero_in:
                if not self._same(kv, self._s_kv):
                    self._s_kv.copy_(kv, non_blocking=True)
                if not self._same(q, self._s_q):
                    self._s_q.copy_(q, non_blocking=True)
                if not self._same(dout, self._s_do):
                    self._s_do.copy_(dout, non_blocking=True)
        local_ready = x.publish(peers)

        d, c = self.ring_divide, L // self.ring_divide
        kv_segs = [{"str": kv[0], "str_g": kv[1], "off": me * L}]
        q_segs = [{"str": q, "str_g": dout, "stats": stats, "off": me * L}]
        x.release([og for og in range(P) if og != me and not (self._sees_keys_of(og) or self._seen_by_queries_of(og))])
        for t in range(1, P):
            og = self.order[t]
            need_kv, need_q = self._sees_keys_of(og), self._seen_by_queries_of(og)
            if not (need_kv or need_q):
                continue
            r_kv, r_q, r_do, r_st = self._stage_views(og)
            for j in range(d):
                flag = x.piece_flag_ptr(og, j)
                ranges: List[Tuple[int, int]] = []
                if need_kv:
                    ranges += self._kv_piece_ranges(j) if d > 1 else [(self._off_kv, self._kv_b)]
                if need_q:
                    if d > 1:
                        ranges += self._q_rows_ranges(self._off_q, j * c, (j + 1) * c)
                        ranges += self._q_rows_ranges(self._off_do, j * c, (j + 1) * c)
                        if j == 0:      # the row statistics are small: all of them travel with the first piece
                            ranges.append((self._off_st, self._st_b))
                    else:
                        ranges.append((self._off_q, self._off_st + self._st_b - self._off_q))
                x.pull(og, ranges, raise_after=[(flag, e)], last=(j == d - 1))
                rows = slice(j * c, (j + 1) * c)
                if need_kv:
                    kv_segs.append({"str": r_kv[0][:, rows], "str_g": r_kv[1][:, rows], "off": og * L + j * c,
                                    "flag": flag, "flag_value": e})
                if need_q:
                    st = (RowStats(r_st[0][:, :, j * c:], r_st[1][:, :, j * c:], c, pad=self.stat_pad) if d > 1
                          else RowStats(r_st[0], r_st[1], L))
                    q_segs.append({"str": r_q[:, rows], "str_g": r_do[:, rows], "stats": st, "off": og * L + j * c,
                                   "flag": flag, "flag_value": e})

        main.wait_event(local_ready)   # my own statistics were computed on the transfer stream
        attn_bwd_dq(q, dout, stats, kv_segs, softmax_scale, causal=self.causal, q_off=me * L, dq=dq, hkv=self.hkv)
        attn_bwd_dkv(kv[0], kv[1], q_segs, softmax_scale, causal=self.causal, k_off=me * L, dk=dkv[0], dv=dkv[1],
                     hq=self.hq)
        self._monitor.post(main)
        self.last_launches = ctx.launch_count - launches0 + 3
        return dq, dkv

    def _backward_heads(self, dout, q, kv, o, lse, dq, dkv, softmax_scale):
        """Backward of the heads schedule: this rank computes dq, dk, dv of ALL rows for its head group in one
        sweep (scores once, dq contributions added in fp32: see attn_bwd_fused) -- causal work is the same
        on every rank, and no gradient needs a cross-rank reduction.  It pulls its head group's rectangles of
        k | v (into one [2, B, S, hkv/P, D] buffer: the owner tiles of the launch), q, dout and the row
        statistics (per origin, flagged: the stream segments of the launch) from every peer; dq is converted
        straight into the owners' memory, dk | dv are pushed there by the copy engines, and one flag per
        owner says that this rank's head group is in."""
        ctx, x, P, me = self.ctx, self._x, self.world, self.rank
        B, L, D, S = self.batch, self.seq_local, self.head_dim, self.seq_local * self.world
        Hl, hkl, pad = self.hq // P, self.hkv // P, self.stat_pad
        q_w, kv_w, st_w = Hl * D * 2, hkl * D * 2, Hl * pad * 4
        dev = q.device
        launches0 = ctx.launch_count
        main = torch.cuda.current_stream()
        comm = ctx.comm_stream
        e = x.begin(main)
        peers = range(P)
        if getattr(self, "_bh", None) is None:
            self._bh = {"kv": torch.empty((2, B, S, hkl, D), dtype=torch.bfloat16, device=dev),
                        "dkv": torch.empty((2, B, S, hkl, D), dtype=torch.bfloat16, device=dev),
                        "acc": torch.empty((P, B, Hl, pad, D), dtype=torch.float32, device=dev),
                        "st": torch.empty((2, B, Hl, pad), dtype=torch.float32, device=dev)}
        bh = self._bh
        x.wait_slot_free(peers)      # this call rewrites the row statistics inside the slot
        with torch.cuda.stream(comm):
            bwd_preprocess(dout, o, lse, workspace=self._s_st)
            bh["st"].copy_(self._s_st[:, :, me * Hl:(me + 1) * Hl], non_blocking=True)
            if not self._same(kv, self._s_kv):
                self._s_kv.copy_(kv, non_blocking=True)
            if not self._same(q, self._s_q):
                self._s_q.copy_(q, non_blocking=True)
            if not self._same(dout, self._s_do):
                self._s_do.copy_(dout, non_blocking=True)
        local_ready = x.publish(peers)

        order = [me] + [(me - t) % P for t in range(1, P)]
        row_kv = hkl * D * 2
        # K/V of every origin first (the launch needs all owner tiles), then q | dout | statistics per origin
        for og in order[1:]:
            rects = [(bh["kv"][w, b, og * L].data_ptr(), self._off_kv + (w * B + b) * L * self.hkv * D * 2 + me * kv_w,
                      self.hkv * D * 2, kv_w, L) for w in range(2) for b in range(B)]
            x.pull_rects(og, rects, raise_after=[(x.piece_flag_ptr(og, 0), e)])
        q_rect_b = B * L * q_w
        segs = []
        for og in order:
            if og == me:
                continue
            buf = x.stage(og)
            o_q, o_do, o_st = 0, _align(q_rect_b, 256), 2 * _align(q_rect_b, 256)
            x.pull_rects(og, [(buf.data_ptr() + o_q, self._off_q + me * q_w, self.hq * D * 2, q_w, B * L),
                              (buf.data_ptr() + o_do, self._off_do + me * q_w, self.hq * D * 2, q_w, B * L),
                              (buf.data_ptr() + o_st, self._off_st + me * st_w, self.hq * pad * 4, st_w, 2 * B)],
                         raise_after=[(x.piece_flag_ptr(og, 1), e)], last=True)
        # the local rows: K/V of my head group into the owner buffer; q, dout as strided views; statistics copied
        for w in range(2):
            for b in range(B):
                ctx.copy2d(bh["kv"][w, b, me * L].data_ptr(), kv_w, kv[w, b, 0, me * hkl].data_ptr(), self.hkv * D * 2,
                           kv_w, L, main)
        bh["acc"].zero_()
        for n, og in enumerate(order):
            acc = bh["acc"][n]
            if og == me:
                sg = {"str": q[:, :, me * Hl:(me + 1) * Hl], "str_g": dout[:, :, me * Hl:(me + 1) * Hl],
                      "stats": RowStats(bh["st"][0], bh["st"][1], L), "off": me * L, "dq_accum": acc}
            else:
                buf = x.stage(og)
                rq, _ = _carve(buf, 0, (B, L, Hl, D), torch.bfloat16)
                rdo, _ = _carve(buf, _align(q_rect_b, 256), (B, L, Hl, D), torch.bfloat16)
                rst, _ = _carve(buf, 2 * _align(q_rect_b, 256), (2, B, Hl, pad), torch.float32)
                sg = {"str": rq, "str_g": rdo, "stats": RowStats(rst[0], rst[1], L), "off": og * L, "dq_accum": acc,
                      "flag": x.piece_flag_ptr(og, 1), "flag_value": e}
            segs.append(sg)
        main.wait_event(local_ready)     # my statistics were computed on the transfer stream
        # The owner tiles (K/V of every rank) must be in before the launch; q | dout | statistics are waited for
        # in the kernel, origin by origin.  (With flagged segments the launch uses the kernel instantiation that
        # leaves a few registers free on every SM: the one-warp kernels that raise the flags start beside it.)
        ctx.wait_many([(x.piece_flag_ptr(og, 0), e) for og in order[1:]], main)
        _bwd_launch(_lib.MB_BWD_MODE_FUSED, bh["kv"][0], bh["kv"][1], 0, segs, Hl, hkl, softmax_scale, self.causal,
                    bh["dkv"][0], bh["dkv"][1], False)
        for n, og in enumerate(order):     # dq of owner og's rows, my head group: scaled, converted, stored there
            dq_convert_raw(bh["acc"][n], x.inbox_ptr(og, self._inbox_dq + me * q_w), (L * self.hq * D, self.hq * D, D),
                           B, L, Hl, pad, softmax_scale)
        # dk | dv rows of every owner: pushed by the copy engines once the kernel is done, then the owner's flag
        comm.wait_stream(main)
        for og in order:
            for w in range(2):
                for b in range(B):
                    ctx.copy2d(x.inbox_ptr(og, self._inbox_dkv + (w * B + b) * L * self.hkv * D * 2 + me * kv_w),
                               self.hkv * D * 2, bh["dkv"][w, b, og * L].data_ptr(), row_kv, kv_w, L, comm)
            ctx.signal_many([(x.res_ptr(og, 16 + me), e)], comm)
        ctx.wait_many([(x.res_ptr(me, 16 + p), e) for p in range(P)], main)
        if dq is None:
            dq = self._s_dq
        elif not self._same(dq, self._s_dq):
            dq.copy_(self._s_dq, non_blocking=True)
        if dkv is None:
            dkv = self._s_dkv
        elif not self._same(dkv, self._s_dkv):
            dkv.copy_(self._s_dkv, non_blocking=True)
        self._monitor.post(main)
        self.last_launches = ctx.launch_count - launches0 + 2 + P
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
        Several ranks: the host tensors are copied straight into this rank's symmetric q / kv (once the
        peers have released them), the forward runs without staging copies, and o / lse are read back
        from the symmetric result buffers; with the heads schedule this is done for four (or two) chunks of
        the heads in a pipeline.  Returns after the results are in host memory.
        """
        dev = torch.device("cuda", torch.cuda.current_device()) if self.ctx is None else self.ctx.device
        if softmax_scale is None:
            softmax_scale = self.head_dim ** -0.5
        L = self.seq_local
        main = torch.cuda.current_stream()
        if self.world > 1 and self.heads:
            # Head-group chunks, pipelined: chunk c is one forward over hq / nc of the heads (its own op with its
            # own symmetric buffers); while it runs, chunk c+1 is copied in and chunk c-1 is copied out, so the
            # PCIe transfers in both directions overlap the kernels and the NVLink all-to-all.
            P, B, D = self.world, self.batch, self.head_dim
            want = int(os.environ.get("MB_HOST_CHUNKS", "1"))
            nc = next((n for n in (4, 2) if n <= want and self.hq % (n * P) == 0 and self.hkv % (n * P) == 0), 1)
            if nc > 1:
                if not hasattr(self, "_host_ops"):
                    self._host_ops = ([RingAttention(self.mesh_shape, B, L, self.hq // nc, self.hkv // nc, D,
                                                     causal=self.causal, ctx=self.ctx, schedule="heads") for _ in range(nc)],
                                      torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev))
                ops, s_in, s_out = self._host_ops
                hc, hkc = self.hq // nc, self.hkv // nc
                ctx = self.ctx
                s_in.wait_stream(main)
                arrived = []
                for c, op in enumerate(ops):
                    b = op.symmetric_buffers()
                    with torch.cuda.stream(s_in):
                        op.inputs_writable()
                        ctx.copy2d(b["q"].data_ptr(), hc * D * 2, q_host[0, 0, c * hc].data_ptr(), self.hq * D * 2,
                                   hc * D * 2, B * L, s_in)
                        ctx.copy2d(b["kv"].data_ptr(), hkc * D * 2, kv_host[0, 0, 0, c * hkc].data_ptr(), self.hkv * D * 2,
                                   hkc * D * 2, 2 * B * L, s_in)
                        ev = torch.cuda.Event()
                        ev.record(s_in)
                    arrived.append(ev)
                for c, op in enumerate(ops):
                    b = op.symmetric_buffers()
                    main.wait_event(arrived[c])
                    op.forward(b["q"], b["kv"], b["o"], b["lse"], softmax_scale)
                    ev = torch.cuda.Event()
                    ev.record(main)
                    s_out.wait_event(ev)
                    ctx.copy2d(o_host[0, 0, c * hc].data_ptr(), self.hq * D * 2, b["o"].data_ptr(), hc * D * 2,
                               hc * D * 2, B * L, s_out)
                    ctx.copy2d(lse_host[0, c * hc].data_ptr(), self.hq * L * 4, b["lse"].data_ptr(), hc * L * 4,
                               hc * L * 4, B, s_out)
                s_out.synchronize()
                main.synchronize()
                return
        if self.world > 1:
            bufs = self.symmetric_buffers()
            q, kv, o, lse = bufs["q"], bufs["kv"], bufs["o"], bufs["lse"]
            self.inputs_writable()
            q.copy_(q_host, non_blocking=True)
            kv.copy_(kv_host, non_blocking=True)
            self.forward(q, kv, o, lse, softmax_scale)
            o_host.copy_(o, non_blocking=True)
            lse_host.copy_(lse, non_blocking=True)
            main.synchronize()
            return
        if not hasattr(self, "_host_bufs"):
            self._host_bufs = (torch.empty(self.q_shape, dtype=torch.bfloat16, device=dev),
                               torch.empty(self.kv_shape, dtype=torch.bfloat16, device=dev),
                               torch.empty(self.q_shape, dtype=torch.bfloat16, device=dev),
                               torch.empty((self.batch, self.hq, L), dtype=torch.float32, device=dev),
                               torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev))
        q, kv, o, lse, s_in, s_out = self._host_bufs
        n = max(1, min(chunks, 64))
        pipelined = self.batch == 1 and L % n == 0 and (L // n) % 128 == 0
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

    def _plain_outputs(self, dev):
        if not hasattr(self, "_plain_out"):
            self._plain_out = (torch.empty(self.q_shape, dtype=torch.bfloat16, device=dev),
                               torch.empty(self.lse_shape, dtype=torch.float32, device=dev))
        return self._plain_out

    def memory_bytes(self, backward: Optional[bool] = None) -> dict:
        """Device memory this object allocates per rank for its transfers, by kind (the counterpart of
        the reference's per-card buffer model, mercury/ir/calculate_memory.py:9-66, for a symmetric slot
        and staging instead of the rotating double buffer): `symmetric` is mapped by every peer -- the
        slot [kv | q (| dout | row statistics with backward=True)] plus the flag region; `staging`
        holds pulled shards (world - 1 slots); `inbox` is the symmetric o / lse that results computed
        on other ranks are written into; `state` is the fp32 online-softmax state (and chain words) that
        the forward's per-shard jobs hand on.  `backward` defaults to what the object was built with."""
        if self.world == 1:
            return {"symmetric": 0, "staging": 0, "inbox": 0, "state": 0}
        if backward is not None and bool(backward) != self.with_backward:
            raise ValueError("the slot layout is fixed at construction: pass backward= to RingAttention")
        slot = _align(self._slot_bytes, 1024)
        inbox = _align(self._inbox_bytes, 1024)
        if self.heads:      # one chain per rank's query rows, for this rank's head group
            chunk_rows, heads = [self.seq_local] * self.world, self.hq // self.world
        else:
            chunk_rows, heads = ([self.seq_local // 2] * 2 if self.balanced else [self.seq_local]), self.hq
        state = sum(self.batch * heads * (r * (self.head_dim + 2) + (r + 255) // 256) * 4 for r in chunk_rows)
        return {"symmetric": slot + _FLAG_REGION, "staging": (self.world - 1) * slot, "inbox": inbox, "state": state}

    def check(self) -> None:
        """Synchronise and raise if a device-side wait timed out."""
        if self.ctx is not None:
            self.ctx.check()
        else:
            _lib.raise_on_status(torch.cuda.current_stream().cuda_stream)
