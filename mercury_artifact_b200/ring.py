"""Fused ring / double-ring / GQA attention forward for one rank (public API).

`RingAttention.forward` computes what the generated per-rank loop computes
(mercury/backend/pytorch/codegen.py:443-494 + utils/flash_attn_dsl.py:160-179 of
the reference) with ONE attention launch: the K/V shards of all ranks are the
segments of a single mb_attn_fwd call in the rank's arrival order, so the
online-softmax state stays on chip and no out/LSE merge kernel runs.

Transport.  On an NVSwitch box every peer is one hop away, so a shard is pulled
straight from the rank that owns it instead of being relayed around the ring;
the order in which a rank consumes shards is still the reference's (single ring:
(r - t) mod P; nested rings: mesh.kv_origin_schedule).  The copy engines move
each remote shard over NVLink into a local staging buffer on a side stream and a
per-segment flag is raised behind it; the kernel's loader waits (bounded) on
that flag before its first TMA load of the segment, so compute on the shards
already here overlaps the transfers of the later ones inside one launch.

World size 1 is the unsharded program: one segment, no transport.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

from . import mesh
from .attention import attn_fwd_segments
from .comm import PeerContext, SymmetricBuffer, default_context

_FLAG_REGION = 4096


class RingAttention:
    """Forward attention of one rank of a sequence-sharded job.

    mesh_shape (P,) is the single ring, (n_inner, n_outer) the double ring (inner ring over
    mesh dimension 0, rank = inner + n_inner * outer).  Shard k of the sequence lives on rank k.
    With causal=True a key is visible iff its global position is <= the query's.
    """

    def __init__(self, mesh_shape: Sequence[int], batch: int, seq_local: int, hq: int, hkv: int,
                 head_dim: int = 128, causal: bool = False, ctx: Optional[PeerContext] = None):
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
        self.kv_shape = (2, batch, seq_local, hkv, head_dim)
        self.kv_bytes = 2 * batch * seq_local * hkv * head_dim * 2
        self.epoch = 0
        self.launches_per_forward = 1
        if self.world > 1:
            # symmetric: two epochs of this rank's shard, then flag words:
            #   ready[origin] at +0     raised on every peer once `origin` has published its shard
            #   done[reader]  at +1024  raised on the owner once `reader` has pulled the shard
            self.sym = SymmetricBuffer(self.ctx, 2 * self.kv_bytes + _FLAG_REGION)
            self._flag_off = 2 * self.kv_bytes
            dev = self.ctx.device
            self.staging = [torch.empty(self.kv_shape, dtype=torch.bfloat16, device=dev) for _ in range(self.world - 1)]
            self.seg_flags = torch.zeros(64, dtype=torch.int32, device=dev)
            torch.cuda.synchronize(dev)

    # ------------------------------------------------------------------ addresses
    def _ready_ptr(self, on_rank: int, origin: int) -> int:
        return self.sym.ptr(on_rank, self._flag_off + 4 * origin)

    def _done_ptr(self, on_rank: int, reader: int) -> int:
        return self.sym.ptr(on_rank, self._flag_off + 1024 + 4 * reader)

    def shard_slot(self, epoch: int) -> torch.Tensor:
        """This rank's published K/V slot for `epoch`."""
        return self.sym.local.view((epoch % 2) * self.kv_bytes, self.kv_shape, torch.bfloat16)

    def needed(self, origin: int) -> bool:
        """Whether this rank's queries can see any key of `origin`'s shard."""
        return (not self.causal) or origin <= self.rank

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

        ctx = self.ctx
        main = torch.cuda.current_stream()
        comm = ctx.comm_stream
        self.epoch += 1
        e = self.epoch
        slot = self.shard_slot(e)
        me = self.rank

        # 1. publish my shard.  The slot was last used at epoch e-2: every peer has raised
        #    done >= e-2 on me once it no longer reads it.
        comm.wait_stream(main)
        if e > 2:
            for p in range(self.world):
                if p != me:
                    ctx.wait_flag(self._done_ptr(me, p), e - 2, comm)
        with torch.cuda.stream(comm):
            slot.copy_(kv, non_blocking=True)
        local_ready = torch.cuda.Event()
        local_ready.record(comm)
        for p in range(self.world):
            if p != me:
                ctx.signal(self._ready_ptr(p, me), e, comm)

        # 2. pull the remote shards in arrival order; raise a local flag behind each one
        segs: List[tuple] = [(slot[0], slot[1], me * L)]
        for t in range(1, self.world):
            origin = self.order[t]
            if self.needed(origin):
                ctx.wait_flag(self._ready_ptr(me, origin), e, comm)
                dst = self.staging[t - 1]
                ctx.copy(dst.data_ptr(), self.sym.ptr(origin, (e % 2) * self.kv_bytes), self.kv_bytes, comm)
                ctx.signal(self.seg_flags.data_ptr() + 4 * t, e, comm)
                segs.append((dst[0], dst[1], origin * L, self.seg_flags.data_ptr() + 4 * t, e))
            ctx.signal(self._done_ptr(origin, me), e, comm)

        # 3. one fused launch on the caller's stream once my own shard is in its slot
        main.wait_event(local_ready)
        out = attn_fwd_segments(q, segs, softmax_scale, causal=self.causal, q_off=me * L, out=o, lse=lse)
        # the next forward's first transfer must not overwrite staging this launch still reads
        return out

    def check(self) -> None:
        """Synchronise and raise if a device-side wait timed out."""
        if self.ctx is not None:
            self.ctx.check()
        else:
            from . import _lib

            _lib.raise_on_status(torch.cuda.current_stream().cuda_stream)
