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
    flag is never raised the waits run out of their (about one second) budget, every other wait of
    the CTA returns at once, the kernel frees its tensor memory and exits, the host reads status 109,
    and the next launch works.  One tiny CTA per launch, so the whole test takes a few seconds."""
    import mercury_artifact_b200 as mb
    from mercury_artifact_b200 import _lib
    from mercury_artifact_b200.comm import DeviceBuffer
    from oracle import block
    from tests.helpers import seeded_qkv

    st = torch.cuda.current_stream()
    assert _lib.status_fetch(st.cuda_stream) == 0
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
