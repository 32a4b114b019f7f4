"""Host logic of the fused ring on CPU, for 2, 4 and 8 ranks: what every rank would enqueue.

RingAttention.forward / backward are run for each rank of a job with the GPU taken away: the peer
context records copies and flag operations instead of launching them, symmetric memory is a CPU
tensor whose peer addresses are made-up bases, and the attention launches are replaced by recorders.
The records of all ranks together must form a consistent protocol: every slot is pulled or released
by every peer exactly once, copies stay inside the slot / staging they belong to, each arrival flag
a kernel waits for is raised behind the copy that fills it (on the same stream), each half-shard of
the balanced causal forward is computed by exactly one rank and lands in its owner's inbox, and the
owner waits for exactly those result flags.
"""
import contextlib
from unittest import mock

import pytest
import torch

from mercury_artifact_b200 import ring

BASE_SHIFT = 44


class FakeStream:
    def __init__(self, name):
        self.name, self.cuda_stream = name, 0

    def wait_stream(self, other):
        pass

    def wait_event(self, ev):
        pass


class FakeEvent:
    def record(self, stream=None):
        pass


class FakeMonitor:
    def poll(self):
        pass

    def post(self, stream):
        pass


class FakeCtx:
    def __init__(self, rank, world):
        self.rank, self.world, self.device = rank, world, torch.device("cpu")
        self.comm_streams = [FakeStream("comm0"), FakeStream("comm1")]
        self.comm_stream = self.comm_streams[0]
        self.monitor = FakeMonitor()
        self.launch_count = 0
        self.ops = []   # (kind, stream name, payload)

    def copy(self, dst, src, nbytes, stream):
        self.ops.append(("copy", stream.name, (dst, src, nbytes)))

    def copy2d(self, dst, dpitch, src, spitch, width, height, stream):
        self.ops.append(("copy2d", stream.name, (dst, dpitch, src, spitch, width, height)))

    def signal(self, ptr, value, stream):
        self.signal_many([(ptr, value)], stream)

    def wait_flag(self, ptr, value, stream, timeout_ns=None):
        self.wait_many([(ptr, value)], stream)

    def signal_many(self, flags, stream):
        self.launch_count += 1
        self.ops.append(("signal", stream.name, list(flags)))

    def wait_many(self, flags, stream, timeout_ns=None):
        self.launch_count += 1
        self.ops.append(("wait", stream.name, list(flags)))


class FakeSym:
    """Symmetric buffer stand-in: a local CPU tensor; rank p's copy 'lives' at (p + 1) << 44."""

    def __init__(self, ctx, nbytes):
        self.ctx, self.nbytes = ctx, ring._align(nbytes)
        self._t = torch.zeros(self.nbytes, dtype=torch.uint8)
        self.local = self

    def bytes(self):
        return self._t

    def ptr(self, rank, offset=0):
        if rank == self.ctx.rank:
            return self._t.data_ptr() + offset
        return ((rank + 1) << BASE_SHIFT) + offset

    def where(self, ptr):
        """(rank, offset) of an address inside some rank's copy of this buffer, else None."""
        lo = self._t.data_ptr()
        if lo <= ptr < lo + self.nbytes:
            return self.ctx.rank, ptr - lo
        r = (ptr >> BASE_SHIFT) - 1
        off = ptr & ((1 << BASE_SHIFT) - 1)
        if 0 <= r < self.ctx.world and off < self.nbytes:
            return r, off
        return None


@contextlib.contextmanager
def _no_gpu(launches):
    main = FakeStream("main")

    def fwd_multi(jobs, segs, scale, causal, b, hq, hkv, d, device):
        launches.append(("fwd", jobs, segs))

    def bwd_dq(q, dout, stats, kv_segs, scale, causal=False, q_off=0, dq=None, accumulate=False, hkv=None):
        launches.append(("dq", kv_segs, q_off))

    def bwd_dkv(k, v, q_segs, scale, causal=False, k_off=0, dk=None, dv=None, accumulate=False, hq=None):
        launches.append(("dkv", q_segs, k_off))

    def pre(dout, o, lse, workspace=None):
        return ring.RowStats(workspace[0], workspace[1], dout.shape[1])

    def bwd_launch(mode, own, own_g, own_off, segments, hq, hkv, scale, causal, out1, out2, accumulate, own_stats=None):
        launches.append(("fused", mode, own, own_off, segments, hq, hkv, out1))

    def convert(acc, ptr, strides, b, sq, hq, pad, scale, out_dtype=torch.bfloat16):
        launches.append(("convert", acc, ptr, strides, (b, sq, hq, pad)))

    with mock.patch.object(ring, "SymmetricBuffer", FakeSym), mock.patch.object(ring, "attn_fwd_multi", fwd_multi), \
            mock.patch.object(ring, "attn_bwd_dq", bwd_dq), mock.patch.object(ring, "attn_bwd_dkv", bwd_dkv), \
            mock.patch.object(ring, "bwd_preprocess", pre), mock.patch.object(torch.cuda, "synchronize", lambda *a: None), \
            mock.patch.object(ring, "_bwd_launch", bwd_launch), mock.patch.object(ring, "dq_convert_raw", convert), \
            mock.patch.object(torch.cuda, "current_stream", lambda *a: main), \
            mock.patch.object(torch.cuda, "stream", lambda s: contextlib.nullcontext()), \
            mock.patch.object(torch.cuda, "Event", FakeEvent):
        yield


def _run_rank(rank, world, mesh, causal, ring_divide, backward, B=1, L=256, H=2, hkv=2, schedule="ring"):
    launches = []
    ctx = FakeCtx(rank, world)
    with _no_gpu(launches):
        op = ring.RingAttention(mesh, B, L, H, hkv, 128, causal=causal, ctx=ctx, ring_divide=ring_divide,
                                backward=backward, schedule=schedule)
        q = torch.zeros(op.q_shape, dtype=torch.bfloat16)
        kv = torch.zeros(op.kv_shape, dtype=torch.bfloat16)
        o, lse = op.forward(q, kv)
        fwd_ops, ctx.ops = ctx.ops, []
        bwd_ops = []
        if backward:
            op.backward(torch.zeros_like(q), q, kv, o, lse)
            bwd_ops = ctx.ops
    return op, launches, fwd_ops, bwd_ops


def _check_transfers(op, ops, epoch, need_done_from_all=True):
    """Per-rank invariants of one epoch's transfer ops; returns {flag address: position} of raised flags."""
    x, me, P = op._x, op.rank, op.world
    sym = x.sym
    stage_lo = x.staging.data_ptr()
    raised = {}
    done_raised = []
    last_copy_on = {}
    for pos, (kind, stream, payload) in enumerate(ops):
        if kind == "copy":
            dst, src, n = payload
            w = sym.where(src)
            assert w is not None and w[0] != me, "a pull reads another rank's symmetric memory"
            origin, off = w
            assert off + n <= x.slot_bytes, "a pull stays inside the owner's slot"
            s_idx = x.stage_index(origin)
            assert stage_lo + s_idx * x.slot_bytes + off == dst, "it lands at the same offset of that origin's staging slot"
            assert stream == x.stream_of(origin).name, "all pulls from one origin share a stream"
            last_copy_on[stream] = pos
        elif kind == "signal":
            for ptr, val in payload:
                assert val == epoch
                raised[ptr] = (pos, stream)
                w = sym.where(ptr)
                if w is not None and w[0] != me and x._flag_off + ring._DONE <= w[1] < x._flag_off + ring._RES:
                    done_raised.append(w[0])
                    assert (w[1] - x._flag_off - ring._DONE) // 4 == me, "done[me] on the owner"
    if need_done_from_all:
        assert sorted(done_raised) == [p for p in range(P) if p != me], "every peer's slot is pulled or released once"
    return raised


@pytest.mark.parametrize("world,mesh", [(2, (2,)), (4, (4,)), (8, (8,))])
@pytest.mark.parametrize("ring_divide", [1, 2])
def test_balanced_causal_forward_plan(world, mesh, ring_divide):
    L, H = 256, 2
    Lh = L // 2
    computed = {}
    waited = {}
    for r in range(world):
        op, launches, ops, _ = _run_rank(r, world, mesh, True, ring_divide, False)
        assert op.balanced and len(launches) == 1
        x = op._x
        raised = _check_transfers(op, ops, 1)
        _, jobs, segs = launches[0]
        assert len(jobs) <= 16 and len(segs) <= 32
        # segments: the local shard first, then remote pieces; every remote piece waits for a flag that is
        # raised behind a copy on the same stream
        assert segs[0][2] == r * L and len(segs[0]) == 3
        for sg in segs:
            if len(sg) > 3:
                assert sg[3] in raised and sg[4] == 1
        shard_of = [sg[2] // L for sg in segs]
        chunks = (2 * world - 1 - r, r)
        # jobs are listed shard by shard in arrival order (local first), each job takes the segments of ONE shard
        arrival = []
        for jb in jobs:
            shards = {shard_of[i] for i in range(len(segs)) if (jb["seg_mask"] >> i) & 1}
            assert len(shards) == 1
            arrival.append(shard_of.index(shards.pop()))
        assert arrival == sorted(arrival)
        for idx, c in enumerate(chunks):
            owner, half = c // 2, c % 2
            mine = [jb for jb in jobs if jb["q_off"] == c * Lh]
            # a chain: the first job starts from nothing, every other continues the state the previous one
            # stored, the last one writes the result into the owner's inbox and raises the owner's flag
            seen_keys = set()
            for p, jb in enumerate(mine):
                assert jb["q"].shape[1] == Lh
                for i in range(len(segs)):
                    if (jb["seg_mask"] >> i) & 1:
                        assert not (seen_keys & set(range(segs[i][2], segs[i][2] + segs[i][0].shape[1])))
                        seen_keys.update(range(segs[i][2], segs[i][2] + segs[i][0].shape[1]))
                last = p == len(mine) - 1
                if len(mine) > 1:
                    assert bool(jb["state_in"]) == (p > 0) and bool(jb["state_out"]) == (not last)
                    assert jb["chain"][1:] == (64 + p, 64 + p + 1) and jb["chain"][0] == mine[0]["chain"][0]
                    assert jb["state"][0].shape == (1, H, Lh, 128) and jb["state"][0] is mine[0]["state"][0]
                else:
                    assert "state" not in jb
                assert ("out_raw" in jb) == last and ("done" in jb) == last
                if owner != r:
                    assert jb["q_flag"][0] in raised, "pulled queries announce themselves"
                else:
                    assert "q_flag" not in jb
            assert seen_keys >= set(range(0, (c + 1) * Lh)), "the chain covers every key the chunk can see"
            job = mine[-1]
            where_o = x.sym.where(job["out_raw"][0])
            assert where_o == (owner, x.slot_bytes + op._inbox_o + half * Lh * H * 128 * 2)
            where_l = x.sym.where(job["lse_raw"][0])
            assert where_l == (owner, x.slot_bytes + op._inbox_lse + half * Lh * 4)
            flag, val, counter = job["done"]
            assert x.sym.where(flag) == (owner, x._flag_off + ring._RES + 4 * half) and val == 1
            assert (owner, half) not in computed, "each half-shard is computed once"
            computed[(owner, half)] = r
        # the owner waits for both of its halves on the main stream, after the launch
        w = [p for k, s, p in ops if k == "wait" and s == "main"]
        assert w and sorted(x.sym.where(ptr)[1] for ptr, _ in w[-1]) == [x._flag_off + ring._RES, x._flag_off + ring._RES + 4]
        waited[r] = True
    assert sorted(computed) == [(o, h) for o in range(world) for h in (0, 1)]
    # the re-assignment balances the work: every rank computes 2P half-shard units
    for r in range(world):
        mine = [oh for oh, who in computed.items() if who == r]
        assert sorted(2 * o + h for o, h in mine) == sorted((r, 2 * world - 1 - r))
        assert sum((2 * o + h) + 0.5 for o, h in mine) == 2 * world


@pytest.mark.parametrize("world,mesh,causal", [(2, (2,), False), (8, (8,), False), (8, (4, 2), False), (8, (8,), True)])
def test_plain_forward_and_backward_plan(world, mesh, causal):
    """balance off: one job on the caller's own tensors; the backward pulls K/V from the ranks whose keys
    it can see and (q, dout, statistics) from the ranks whose queries can see its keys."""
    L = 256
    for r in range(world):
        launches = []
        ctx = FakeCtx(r, world)
        with _no_gpu(launches):
            op = ring.RingAttention(mesh, 1, L, 2, 2, 128, causal=causal, ctx=ctx, balance_causal=False, backward=True,
                                    ring_divide=2)
            q = torch.zeros(op.q_shape, dtype=torch.bfloat16)
            kv = torch.zeros(op.kv_shape, dtype=torch.bfloat16)
            o, lse = op.forward(q, kv)
            raised = _check_transfers(op, ctx.ops, 1)
            ctx.ops = []
            op.backward(torch.zeros_like(q), q, kv, o, lse)
            raised_b = _check_transfers(op, ctx.ops, 2)
        (_, jobs, segs), (_, kv_segs, q_off), (_, q_segs, k_off) = launches
        assert all("done" not in jb and jb["q_off"] == r * L for jb in jobs) and "out_raw" in jobs[-1]
        assert [bool(jb.get("state_in")) for jb in jobs] == [False] + [True] * (len(jobs) - 1)
        order = ring.mesh.kv_origin_schedule(r, mesh)
        want = [og for og in order if (not causal) or og <= r]
        got = []
        for sg in segs:
            og = sg[2] // L
            if og not in got:
                got.append(og)
            if len(sg) > 3:
                assert sg[3] in raised
        assert got == want, "segments follow the reference's consumption order"
        assert q_off == r * L and k_off == r * L
        assert sorted({s["off"] // L for s in kv_segs}) == sorted(og for og in range(world) if (not causal) or og <= r)
        assert sorted({s["off"] // L for s in q_segs}) == sorted(og for og in range(world) if (not causal) or og >= r)
        for s in kv_segs[1:] + q_segs[1:]:
            assert s["flag"] in raised_b and s["flag_value"] == 2


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("causal", [False, True])
def test_heads_schedule_plan(world, causal):
    """Schedule "heads": rank r pulls head group r's rectangle of q and of k | v from every peer exactly once,
    computes every rank's query rows for that head group as one state chain per owner (first job when the
    owner's rows arrive, then one job per later shard), and the last job of each chain stores into the
    owner's o / lse at head group r and raises the owner's flag number r; the owner waits for all P flags."""
    B, L, H, hkv, D = 2, 256, 16, 8, 128
    Hl, hkl = H // world, hkv // world
    q_w, kv_w = Hl * D * 2, hkl * D * 2
    delivered = set()
    for r in range(world):
        op, launches, ops, _ = _run_rank(r, world, (world,), causal, 1, False, B=B, H=H, hkv=hkv, schedule="heads")
        assert op.heads and len(launches) == 1
        x = op._x
        sym = x.sym
        # transfers
        pulled, raised, done_to = {}, {}, []
        for pos, (kind, stream, payload) in enumerate(ops):
            if kind == "copy2d":
                dst, dpitch, src, spitch, width, height = payload
                origin, off = sym.where(src)
                assert origin != r and dpitch == width
                stage_lo = x.staging.data_ptr() + x.stage_index(origin) * x.slot_bytes
                assert stage_lo <= dst and dst + width * height <= stage_lo + x.slot_bytes
                if width == q_w and spitch == H * D * 2 and off == op._off_q + r * q_w:
                    assert height == B * L
                    pulled.setdefault(origin, []).append("q")
                else:
                    assert (width, spitch, off, height) == (kv_w, hkv * D * 2, op._off_kv + r * kv_w, 2 * B * L)
                    pulled.setdefault(origin, []).append("kv")
            elif kind == "signal":
                for ptr, val in payload:
                    assert val == 1
                    raised[ptr] = pos
                    w = sym.where(ptr)
                    if w is not None and w[0] != r and x._flag_off + ring._DONE <= w[1] < x._flag_off + ring._RES:
                        assert w[1] == x._flag_off + ring._DONE + 4 * r
                        done_to.append(w[0])
        assert pulled == {p: ["q", "kv"] for p in range(world) if p != r}
        assert sorted(done_to) == [p for p in range(world) if p != r]
        _, jobs, segs = launches[0]
        assert len(jobs) <= 40 and len(segs) == world
        order = [sg[2] // L for sg in segs]
        assert order[0] == r and sorted(order) == list(range(world))
        for sg in segs[1:]:
            assert sg[3] in raised and sg[4] == 1
        steps = []
        for owner in range(world):
            mine = [(n, jb) for n, jb in enumerate(jobs) if jb["q_off"] == owner * L]
            seen = []
            for p, (n, jb) in enumerate(mine):
                assert jb["q"].shape == (B, L, Hl, D)
                shards = [order[i] for i in range(world) if (jb["seg_mask"] >> i) & 1]
                if p == 0:      # the owner's rows arrive with its shard: everything that is there by then
                    assert set(shards) == {s_ for s_ in order[:order.index(owner) + 1] if (not causal) or s_ <= owner}
                else:
                    assert len(shards) == 1 and order.index(shards[0]) > order.index(owner)
                steps.append((n, max(order.index(s_) for s_ in shards)))
                seen += shards
                last = p == len(mine) - 1
                if len(mine) > 1:
                    assert bool(jb["state_in"]) == (p > 0) and bool(jb["state_out"]) == (not last)
                    assert jb["state"][0].shape == (B, Hl, L, D)
                    # the link before it in the chain is EARLIER in the launch (CTAs are dispatched in job order)
                    # and sets exactly the value this one waits for, on the same words
                    assert jb["chain"][0] == mine[0][1]["chain"][0] and jb["chain"][1:] == (64 + p, 64 + p + 1)
                    assert p == 0 or mine[p - 1][0] < n
                assert ("done" in jb) == last
                assert ("q_flag" in jb) == (owner != r)
            assert sorted(seen) == [s_ for s_ in range(world) if (not causal) or s_ <= owner]
            final = mine[-1][1]
            assert sym.where(final["out_raw"][0]) == (owner, x.slot_bytes + op._inbox_o + r * q_w)
            assert final["out_raw"][1:] == (L * H * D, H * D, D)
            assert sym.where(final["lse_raw"][0]) == (owner, x.slot_bytes + op._inbox_lse + r * Hl * L * 4)
            assert sym.where(final["done"][0]) == (owner, x._flag_off + ring._RES + 4 * r)
            delivered.add((owner, r))
        assert [t for _, t in sorted(steps)] == sorted(t for _, t in steps), "jobs are listed in arrival order"
        w = [p for k, s_, p in ops if k == "wait" and s_ == "main"]
        assert sorted(sym.where(ptr)[1] for ptr, _ in w[-1]) == [x._flag_off + ring._RES + 4 * p for p in range(world)]
    assert delivered == {(o_, r_) for o_ in range(world) for r_ in range(world)}


@pytest.mark.parametrize("world", [2, 4, 8])
def test_heads_backward_plan(world):
    """Heads schedule, backward: rank r pulls its head group's k | v rows of every peer into ONE owner buffer
    (row block of the origin), q | dout | statistics per origin into staging, waits for all K/V before the
    launch, runs one sweep with one flagged stream segment per origin, converts dq of origin j's rows into j's
    memory at head group r, pushes dk | dv rows to their owners and raises flag 16 + r there; every owner
    waits for P such flags."""
    B, L, H, hkv, D = 2, 256, 16, 8, 128
    Hl, hkl = H // world, hkv // world
    q_w, kv_w = Hl * D * 2, hkl * D * 2
    got = set()
    for r in range(world):
        op, launches, fwd_ops, ops = _run_rank(r, world, (world,), True, 1, True, B=B, H=H, hkv=hkv, schedule="heads")
        x, sym = op._x, op._x.sym
        fused = [l for l in launches if l[0] == "fused"]
        conv = [l for l in launches if l[0] == "convert"]
        assert len(fused) == 1 and len(conv) == world
        _, mode, own, own_off, segs, hq_, hkv_, out1 = fused[0]
        assert mode == 2 and own.shape == (B, world * L, hkl, D) and own_off == 0 and (hq_, hkv_) == (Hl, hkl)
        assert out1.shape == own.shape
        kv_lo = op._bh["kv"].data_ptr()
        kv_rows, pushes, flags_to, waits = set(), {}, [], []
        for kind, stream, payload in ops:
            if kind == "copy2d":
                dst, dpitch, src, spitch, width, height = payload
                ws, wd = sym.where(src), sym.where(dst)
                if wd is not None and x.slot_bytes + op._inbox_dkv <= wd[1]:      # a push of dk | dv rows
                    assert (dpitch, width, height) == (hkv * D * 2, kv_w, L)
                    rel = wd[1] - x.slot_bytes - op._inbox_dkv
                    assert rel % (hkv * D * 2) == r * kv_w
                    pushes[wd[0]] = pushes.get(wd[0], 0) + 1
                elif kv_lo <= dst < kv_lo + op._bh["kv"].numel() * 2 and width == kv_w and height == L:
                    row = (dst - kv_lo) // kv_w
                    origin = ws[0] if ws is not None else r
                    assert (row % (world * L)) == origin * L
                    kv_rows.add((origin, row // (world * L)))
            elif kind == "signal":
                for ptr, val in payload:
                    w = sym.where(ptr)
                    if w is not None and w[1] == x._flag_off + ring._RES + 4 * (16 + r):
                        flags_to.append(w[0])
            elif kind == "wait" and stream == "main":
                waits.append(payload)
        assert kv_rows == {(og, wb) for og in range(world) for wb in range(2 * B)}
        assert pushes == {og: 2 * B for og in range(world)} and sorted(flags_to) == list(range(world))
        assert sorted(sg["off"] // L for sg in segs) == list(range(world)) and segs[0]["off"] == r * L
        assert all(("flag" in sg) == (sg["off"] != r * L) and sg["dq_accum"].shape == (B, Hl, op.stat_pad, D) for sg in segs)
        # the K/V arrival flags of all origins are waited for before the launch (they are its owner tiles), the
        # gradient flags after it
        assert len(waits[-2]) == world - 1 and len(waits[-1]) == world
        assert sorted(sym.where(p_)[1] for p_, _ in waits[-1]) == [x._flag_off + ring._RES + 4 * (16 + p_) for p_ in range(world)]
        for (_, acc, ptr, strides, dims), sg in zip(conv, segs):
            owner = sg["off"] // L
            assert sym.where(ptr) == (owner, x.slot_bytes + op._inbox_dq + r * q_w)
            assert strides == (L * H * D, H * D, D) and dims == (B, L, Hl, op.stat_pad) and acc.data_ptr() == sg["dq_accum"].data_ptr()
            got.add((owner, r))
    assert got == {(o_, r_) for o_ in range(world) for r_ in range(world)}


def test_more_shards_than_job_slots_share_jobs():
    """32 ranks, balanced causal ring: two chains of up to 32 shards would need 48 jobs; consecutive shards
    then share a job, the launch stays within its 40 job slots and every chain still covers every key its
    chunk can see, each key once, in arrival order."""
    world, L, Lh = 32, 256, 128
    for r in (0, 13, 31):
        op, launches, ops, _ = _run_rank(r, world, (world,), True, 1, False)
        _, jobs, segs = launches[0]
        assert len(jobs) <= 40 and len(segs) <= 32
        for c in (2 * world - 1 - r, r):
            mine = [jb for jb in jobs if jb["q_off"] == c * Lh]
            keys, last_seg = set(), -1
            for p, jb in enumerate(mine):
                idx = [i for i in range(len(segs)) if (jb["seg_mask"] >> i) & 1]
                assert idx and min(idx) > last_seg
                last_seg = max(idx)
                for i in idx:
                    rng = set(range(segs[i][2], segs[i][2] + segs[i][0].shape[1]))
                    assert not (keys & rng)
                    keys |= rng
                assert bool(jb.get("state_in")) == (p > 0) and ("out_raw" in jb) == (p == len(mine) - 1)
            assert keys >= set(range(0, (c + 1) * Lh))
