"""Flag and copy primitives of the peer transport on one device (no peer needed)."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_flag_wait_times_out_and_context_survives():
    """A wait on a flag nobody raises gives up after its budget, reports through the status
    word, and the device keeps working (failure detection without faulting the GPU)."""
    from mercury_artifact_b200 import _lib
    from mercury_artifact_b200.comm import DeviceBuffer

    buf = DeviceBuffer(256, torch.device("cuda", 0))
    st = torch.cuda.current_stream()
    assert _lib.status_fetch(st.cuda_stream) == 0
    _lib.check(_lib.lib.mb_flag_wait(C.c_void_p(buf.ptr), 1, C.c_uint64(50_000_000), None, C.c_void_p(st.cuda_stream)),
               "mb_flag_wait")
    assert _lib.status_fetch(st.cuda_stream) == 107
    assert _lib.status_fetch(st.cuda_stream) == 0  # cleared by the read
    with pytest.raises(_lib.MercuryB200Error):
        _lib.lib.mb_flag_wait(C.c_void_p(buf.ptr), 1, C.c_uint64(10_000_000), None, C.c_void_p(st.cuda_stream))
        _lib.raise_on_status(st.cuda_stream)
    x = torch.arange(8, device="cuda").sum().item()
    assert x == 28
    buf.free()


def test_signal_then_wait_and_copy():
    from mercury_artifact_b200 import _lib
    from mercury_artifact_b200.comm import DeviceBuffer

    dev = torch.device("cuda", 0)
    buf = DeviceBuffer(4096, dev)
    st = torch.cuda.current_stream()
    src = torch.arange(512, dtype=torch.int32, device=dev)
    _lib.check(_lib.lib.mb_copy_async(C.c_void_p(buf.ptr + 1024), C.c_void_p(src.data_ptr()), 2048, C.c_void_p(st.cuda_stream)), "copy")
    _lib.check(_lib.lib.mb_flag_signal(C.c_void_p(buf.ptr), 7, C.c_void_p(st.cuda_stream)), "signal")
    _lib.check(_lib.lib.mb_flag_wait(C.c_void_p(buf.ptr), 7, C.c_uint64(1_000_000_000), None, C.c_void_p(st.cuda_stream)), "wait")
    assert _lib.status_fetch(st.cuda_stream) == 0
    view = buf.view(1024, (512,), torch.int32)
    assert torch.equal(view, src)
    assert buf.view(0, (1,), torch.int32).item() == 7
    buf.free()


def test_sendrecv_single_rank_self_exchange():
    """world_size 1: a rank that sends to itself gets its own message back through the inbox."""
    from mercury_artifact_b200.comm import PeerContext, SendRecv

    ctx = PeerContext()
    sr = SendRecv(ctx)
    with pytest.raises(RuntimeError, match="wait called before commit"):
        sr.wait()
    x = torch.randn(3, 1000, device="cuda")
    got = sr.send_recv(0, 0, x)
    sr.commit()
    with pytest.raises(RuntimeError, match="commit called twice"):
        sr.commit()
    sr.wait()
    torch.cuda.synchronize()
    assert torch.equal(got, x)
    y = x * 2
    got2 = sr.send_recv(0, 0, y)
    sr.commit()
    sr.wait()
    torch.cuda.synchronize()
    assert torch.equal(got2, y) and torch.equal(got, x)
    ctx.check()


def test_kernel_wait_for_a_shard_that_never_arrives_gives_up():
    """The attention kernels wait inside the launch for the arrival flag of a staged shard.  If the
    flag is never raised the waits run out of their budget (mb_set_peer_wait_ms, shortened here), every other wait of
    the CTA returns at once, the kernel frees its tensor memory and exits, the host reads status 109,
    and the next launch works.  One tiny CTA per launch, so the whole test takes a few seconds."""
    import mercury_artifact_b200 as mb
    from mercury_artifact_b200 import _lib
    from mercury_artifact_b200.comm import DeviceBuffer
    from oracle import block
    from tests.helpers import seeded_qkv

    st = torch.cuda.current_stream()
    assert _lib.status_fetch(st.cuda_stream) == 0
    _lib.set_peer_wait_ms(500)   # the default (30 s) is sized for rank skew in real jobs
    try:
        _kernel_wait_body(mb, _lib, DeviceBuffer, block, seeded_qkv, st)
    finally:
        _lib.set_peer_wait_ms(_lib.PEER_WAIT_MS)


def _kernel_wait_body(mb, _lib, DeviceBuffer, block, seeded_qkv, st):
    flag = DeviceBuffer(256, torch.device("cuda", 0))      # zero-initialised, nobody raises it
    q, k, v, do = seeded_qkv(11, 1, 256, 1, 1, 128, device="cuda")
    # forward: first segment in place, second "still in flight"
    mb.attn_fwd_segments(q, [(k[:, :128], v[:, :128], 0), (k[:, 128:], v[:, 128:], 128, flag.ptr, 1)], 128 ** -0.5)
    assert _lib.status_fetch(st.cuda_stream) == 109
    # the same call with the flag raised completes and is correct
    _lib.check(_lib.lib.mb_flag_signal(C.c_void_p(flag.ptr), 1, C.c_void_p(st.cuda_stream)), "mb_flag_signal")
    o, lse = mb.attn_fwd_segments(q, [(k[:, :128], v[:, :128], 0), (k[:, 128:], v[:, 128:], 128, flag.ptr, 1)],
                                  128 ** -0.5)
    assert _lib.status_fetch(st.cuda_stream) == 0
    ro, rl = block.full_attention(q.cpu(), k.cpu(), v.cpu(), 128 ** -0.5, causal=False)
    assert (o.float().cpu() - ro.float()).abs().max().item() <= 2e-2
    assert (lse.cpu() - rl).abs().max().item() <= 1e-3
    # backward (dQ launch): a K/V shard whose flag stays below the value it waits for
    stats = mb.bwd_preprocess(do, o, lse)
    mb.attn_bwd_dq(q, do, stats, [(k, v, 0, flag.ptr, 2)], 128 ** -0.5)
    assert _lib.status_fetch(st.cuda_stream) == 109
    dq = mb.attn_bwd_dq(q, do, stats, [(k, v, 0, flag.ptr, 1)], 128 ** -0.5)
    assert _lib.status_fetch(st.cuda_stream) == 0
    rdq, _, _ = block.block_attn_bwd(do.cpu(), q.cpu(), k.cpu(), v.cpu(), ro, rl, 128 ** -0.5, causal=False)
    assert (dq.float().cpu() - rdq).abs().max().item() <= 2e-2
    flag.free()


def test_batched_flag_kernels_and_status_monitor():
    """mb_flags_signal / mb_flags_wait handle up to 32 words per launch; a wait that runs out is noticed by
    the StatusMonitor at a later poll(), without the caller synchronising after every call."""
    from mercury_artifact_b200 import _lib
    from mercury_artifact_b200.comm import DeviceBuffer, PeerContext

    ctx = PeerContext()
    buf = DeviceBuffer(1024, torch.device("cuda", 0))
    st = torch.cuda.current_stream()
    flags = [(buf.ptr + 4 * i, 10 + i) for i in range(40)]       # 40 words: two launches
    n0 = ctx.launch_count
    ctx.signal_many(flags, st)
    ctx.wait_many(flags, st)
    assert ctx.launch_count - n0 == 4
    assert _lib.status_fetch(st.cuda_stream) == 0
    assert buf.view(0, (40,), torch.int32).tolist() == [10 + i for i in range(40)]
    # one of the words never reaches its value: the wait gives up, the monitor reports it afterwards
    mon = _lib.StatusMonitor()
    mon.poll()
    ctx.wait_many([(buf.ptr, 10), (buf.ptr + 4, 999)], st, timeout_ns=20_000_000)
    mon.post(st)
    st.synchronize()
    with pytest.raises(_lib.MercuryB200Error, match="earlier call timed out"):
        mon.poll()
    mon.poll()                       # reported once; the device word was cleared
    assert _lib.status_fetch(st.cuda_stream) == 0
    buf.free()


def test_multi_job_forward_flags_and_completion():
    """mb_attn_fwd_multi: two query shards in one launch write where their job says, equal the one-job
    results bit for bit, wait for their queries' arrival flag, and each raises its completion flag once
    all its CTAs have stored (the counter word is back at zero afterwards)."""
    import mercury_artifact_b200 as mb
    from mercury_artifact_b200 import _lib
    from mercury_artifact_b200.attention import attn_fwd_multi
    from mercury_artifact_b200.comm import DeviceBuffer
    from tests.helpers import seeded_qkv

    dev = torch.device("cuda", 0)
    st = torch.cuda.current_stream()
    B, S, H, hkv, D = 2, 1024, 4, 2, 128
    q, k, v, _ = seeded_qkv(21, B, S, H, hkv, D, device="cuda")
    scale = D ** -0.5
    words = DeviceBuffer(256, dev)         # [0] q arrival flag, [1..2] completion flags, [3..4] counters
    segs = [(k[:, 512:], v[:, 512:], 512), (k[:, :512], v[:, :512], 0)]
    # one-job references: rows 768.. (job A) and rows 0..255 (job B), causal on global positions
    ra, la = mb.attn_fwd_segments(q[:, 768:], segs, scale, causal=True, q_off=768)
    rb, lb = mb.attn_fwd_segments(q[:, :256], segs, scale, causal=True, q_off=0)
    o = torch.zeros_like(q)
    lse = torch.zeros(B, H, S, device=dev)

    def job(rows, flag_idx, q_flag=None):
        r0 = rows.start
        j = {"q": q[:, rows], "q_off": r0,
             "out_raw": (o[:, rows].data_ptr(), o.stride(0), o.stride(1), o.stride(2)),
             "lse_raw": (lse[:, :, rows].data_ptr(), lse.stride(0), lse.stride(1)),
             "done": (words.ptr + 4 * flag_idx, 5, words.ptr + 4 * (flag_idx + 2))}
        if q_flag is not None:
            j["q_flag"] = q_flag
        return j

    _lib.check(_lib.lib.mb_flag_signal(C.c_void_p(words.ptr), 3, C.c_void_p(st.cuda_stream)), "signal")
    attn_fwd_multi([job(slice(768, 1024), 1, q_flag=(words.ptr, 3)), job(slice(0, 256), 2)], segs, scale, True,
                   B, H, hkv, D, dev)
    assert _lib.status_fetch(st.cuda_stream) == 0
    assert torch.equal(o[:, 768:], ra) and torch.equal(lse[:, :, 768:], la)
    assert torch.equal(o[:, :256], rb) and torch.equal(lse[:, :, :256], lb)
    assert o[:, 256:768].abs().max().item() == 0          # rows of no job are untouched
    assert words.view(0, (5,), torch.int32).tolist() == [3, 5, 5, 0, 0]
    # queries that never arrive: status 109, the completion flag of that job still gets raised (every CTA
    # counts, so that the counter returns to zero), the other job is complete and correct
    _lib.set_peer_wait_ms(300)
    try:
        o.zero_()
        j0 = job(slice(768, 1024), 1, q_flag=(words.ptr, 4))
        j0["done"] = (words.ptr + 4, 6, words.ptr + 12)
        j1 = job(slice(0, 256), 2)
        j1["done"] = (words.ptr + 8, 6, words.ptr + 16)
        attn_fwd_multi([j0, j1], segs, scale, True, B, H, hkv, D, dev)
        assert _lib.status_fetch(st.cuda_stream) == 109
        assert words.view(0, (5,), torch.int32).tolist() == [3, 6, 6, 0, 0]
        assert torch.equal(o[:, :256], rb)
    finally:
        _lib.set_peer_wait_ms(_lib.PEER_WAIT_MS)
    # and the next launch works
    o2, l2 = mb.attn_fwd_segments(q[:, 768:], segs, scale, causal=True, q_off=768)
    assert _lib.status_fetch(st.cuda_stream) == 0 and torch.equal(o2, ra)
    words.free()


def test_sm_pull_kernel_copies_ranges_waits_and_signals():
    """mb_pull_sm on one device (source and destination local): several ranges of odd sizes arrive bit for
    bit, the kernel waits for the source's flag first, raises the completion flags last, leaves its counter
    at zero, and gives up with a status code when the source's flag never comes."""
    from mercury_artifact_b200 import _lib
    from mercury_artifact_b200.comm import DeviceBuffer, PeerContext

    dev = torch.device("cuda", 0)
    ctx = PeerContext()
    st = torch.cuda.current_stream()
    words = DeviceBuffer(256, dev)    # [0] source flag, [1..2] completion flags, [3] counter
    g = torch.Generator(device="cuda").manual_seed(3)
    src = torch.randint(0, 255, (3 * (1 << 20) + 4096,), dtype=torch.uint8, device=dev, generator=g)
    dst = torch.zeros_like(src)
    # ranges: 1 MiB + 16 bytes, 48 bytes, 8 KiB exactly, 1.5 MiB -- all multiples of 16, none of the chunk size
    spans = [(0, (1 << 20) + 16), (1 << 21, 48), ((1 << 21) + 4096, 8192), ((1 << 21) + 65536, 3 << 19)]
    ranges = [(dst.data_ptr() + o, src.data_ptr() + o, n) for o, n in spans]
    _lib.check(_lib.lib.mb_flag_signal(C.c_void_p(words.ptr), 9, C.c_void_p(st.cuda_stream)), "signal")
    ctx.pull_sm(ranges, (words.ptr, 9), [(words.ptr + 4, 21), (words.ptr + 8, 22)], words.ptr + 12, st)
    assert _lib.status_fetch(st.cuda_stream) == 0
    for o, n in spans:
        assert torch.equal(dst[o:o + n], src[o:o + n])
    touched = torch.zeros_like(src, dtype=torch.bool)
    for o, n in spans:
        touched[o:o + n] = True
    assert int(dst[~touched].max().item()) == 0          # nothing outside the ranges was written
    assert words.view(0, (4,), torch.int32).tolist() == [9, 21, 22, 0]
    # a few CTAs only, and no wait flag
    dst.zero_()
    ctx.pull_sm(ranges[:1], None, [(words.ptr + 4, 23)], words.ptr + 12, st, ctas=3)
    assert _lib.status_fetch(st.cuda_stream) == 0
    assert torch.equal(dst[:spans[0][1]], src[:spans[0][1]]) and words.view(4, (1,), torch.int32).item() == 23
    # the source never publishes: bounded wait, status 107, completion flag still raised so that nothing
    # downstream hangs, counter back at zero
    _lib.set_peer_wait_ms(200)
    try:
        ctx.pull_sm(ranges[:1], (words.ptr, 10), [(words.ptr + 4, 24)], words.ptr + 12, st)
        assert _lib.status_fetch(st.cuda_stream) == 107
    finally:
        _lib.set_peer_wait_ms(_lib.PEER_WAIT_MS)
    assert words.view(0, (4,), torch.int32).tolist() == [9, 24, 22, 0]
    words.free()


def test_copy2d_moves_a_head_group_rectangle():
    """mb_copy2d_async: the rows of one head group of a [batch, seq, heads, d] tensor land densely packed, and
    back again into another tensor's head group; misaligned arguments are refused."""
    from mercury_artifact_b200 import _lib
    from mercury_artifact_b200.comm import PeerContext

    ctx = PeerContext()
    st = torch.cuda.current_stream()
    B, L, H, D, g0, g1 = 2, 96, 8, 128, 2, 5
    g = torch.Generator(device="cuda").manual_seed(11)
    src = torch.randn(B, L, H, D, device="cuda", generator=g).to(torch.bfloat16)
    packed = torch.zeros(B, L, g1 - g0, D, dtype=torch.bfloat16, device="cuda")
    w = (g1 - g0) * D * 2
    ctx.copy2d(packed.data_ptr(), w, src[0, 0, g0].data_ptr(), H * D * 2, w, B * L, st)
    st.synchronize()
    assert torch.equal(packed, src[:, :, g0:g1])
    back = torch.zeros_like(src)
    ctx.copy2d(back[0, 0, g0].data_ptr(), H * D * 2, packed.data_ptr(), w, w, B * L, st)
    st.synchronize()
    assert torch.equal(back[:, :, g0:g1], src[:, :, g0:g1]) and back[:, :, :g0].abs().max().item() == 0
    assert back[:, :, g1:].abs().max().item() == 0
    with pytest.raises(_lib.MercuryB200Error):
        ctx.copy2d(packed.data_ptr() + 2, w, src.data_ptr(), H * D * 2, w, 4, st)      # 16-byte alignment
    with pytest.raises(_lib.MercuryB200Error):
        ctx.copy2d(packed.data_ptr(), w // 2, src.data_ptr(), H * D * 2, w, 4, st)     # pitch below the width
