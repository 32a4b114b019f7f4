"""The allocation-free block backward, mb_attn_bwd_block_noalloc, against the regular entry points.

Some callers may not obtain device memory where they run the backward (a fully planned memory
pool, an allocator callback, a serving process with a fixed budget), so they cannot hand the
library the per-row statistics workspace that mb_attn_bwd_preprocess / mb_attn_bwd need.  The
allocation-free entry point keeps that workspace in a fixed array inside the library.  This test
calls it through the C ABI twice in a row, with different inputs, and requires the gradients to
equal those of the regular path (same kernels, same arithmetic: bitwise), which also shows that
the shared array is rewritten, not reused, from one call to the next.  It is collected last so a
run that stops at the first failure has already run every other test.
"""
import ctypes as C

import pytest
import torch

from tests.helpers import seeded_qkv

pytestmark = pytest.mark.gpu


def _noalloc_backward(q, k, v, do, out, lse, scale, causal, q_off, k_off, dtype=torch.bfloat16):
    from mercury_artifact_b200 import _lib

    dq = torch.empty_like(q, dtype=dtype)
    dkv = torch.empty((2,) + tuple(k.shape), dtype=dtype, device=k.device)
    a = _lib.AttnBwdBlockArgs()
    a.dout, a.q, a.out = do.data_ptr(), q.data_ptr(), out.data_ptr()
    assert do.stride() == q.stride() == out.stride()
    a.q_stride_b, a.q_stride_s, a.q_stride_h = q.stride(0), q.stride(1), q.stride(2)
    a.k, a.v = k.data_ptr(), v.data_ptr()
    assert k.stride() == v.stride()
    a.kv_stride_b, a.kv_stride_s, a.kv_stride_h = k.stride(0), k.stride(1), k.stride(2)
    a.lse = lse.data_ptr()
    a.dq = dq.data_ptr()
    a.dq_stride_b, a.dq_stride_s, a.dq_stride_h = dq.stride(0), dq.stride(1), dq.stride(2)
    a.dk, a.dv = dkv[0].data_ptr(), dkv[1].data_ptr()
    a.dkv_stride_b, a.dkv_stride_s, a.dkv_stride_h = dkv[0].stride(0), dkv[0].stride(1), dkv[0].stride(2)
    a.batch, a.sq, a.sk, a.hq, a.hkv, a.head_dim = q.shape[0], q.shape[1], k.shape[1], q.shape[2], k.shape[2], q.shape[3]
    a.q_off, a.k_off, a.causal = q_off, k_off, 1 if causal else 0
    a.out_mode = _lib.MB_OUT_BF16 if dtype == torch.bfloat16 else _lib.MB_OUT_F32
    a.softmax_scale = scale
    a.status = None
    rc = _lib.lib.mb_attn_bwd_block_noalloc(C.byref(a), C.c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc, dq, dkv


def _regular_backward(q, k, v, do, out, lse, scale, causal, q_off, k_off):
    import mercury_artifact_b200 as mb

    st = mb.bwd_preprocess(do, out, lse)
    dq = mb.attn_bwd_dq(q, do, st, [(k, v, k_off)], scale, causal=causal, q_off=q_off)
    dk, dv = mb.attn_bwd_dkv(k, v, [(q, do, st, q_off)], scale, causal=causal, k_off=k_off)
    return dq, dk, dv


def test_noalloc_backward_equals_regular_backward_on_two_calls_in_a_row():
    import mercury_artifact_b200 as mb
    from mercury_artifact_b200 import _lib
    from oracle import block

    scale = 128 ** -0.5
    # two different problems back to back: the second is smaller, causal and GQA, so stale
    # statistics left by the first call would be caught
    problems = [
        dict(seed=41, B=2, Sq=640, Sk=512, Hq=4, Hkv=4, causal=False, q_off=0),
        dict(seed=42, B=1, Sq=300, Sk=391, Hq=8, Hkv=2, causal=True, q_off=91),
    ]
    for p in problems:
        S = max(p["Sq"], p["Sk"])
        q, k, v, do = seeded_qkv(p["seed"], p["B"], S, p["Hq"], p["Hkv"], 128, device="cuda")
        q, do = q[:, :p["Sq"]].contiguous(), do[:, :p["Sq"]].contiguous()
        k, v = k[:, :p["Sk"]].contiguous(), v[:, :p["Sk"]].contiguous()
        out, lse = mb.attn_fwd_segments(q, [(k, v, 0)], scale, causal=p["causal"], q_off=p["q_off"])
        rc, dq, dkv = _noalloc_backward(q, k, v, do, out, lse, scale, p["causal"], p["q_off"], 0)
        assert rc == 0, _lib.ERROR_NAMES.get(rc, rc)
        rdq, rdk, rdv = _regular_backward(q, k, v, do, out, lse, scale, p["causal"], p["q_off"], 0)
        assert _lib.status_fetch(torch.cuda.current_stream().cuda_stream) == 0
        assert torch.equal(dq, rdq) and torch.equal(dkv[0], rdk) and torch.equal(dkv[1], rdv)
        # and both agree with the fp32 oracle within the tolerance the other backward tests use
        ro, rl = block.block_attn_fwd(q.cpu(), k.cpu(), v.cpu(), scale, causal=p["causal"], q_off=p["q_off"], k_off=0)
        gq, gk, gv = block.block_attn_bwd(do.cpu(), q.cpu(), k.cpu(), v.cpu(), ro, rl, scale, causal=p["causal"],
                                          q_off=p["q_off"], k_off=0)
        assert (dq.float().cpu() - gq).abs().max().item() <= 2e-2
        assert (dkv[0].float().cpu() - gk).abs().max().item() <= 2e-2
        assert (dkv[1].float().cpu() - gv).abs().max().item() <= 2e-2


def test_noalloc_backward_rejects_what_does_not_fit():
    from mercury_artifact_b200 import _lib

    # batch 2 x 32 heads x 32768 rows = 2 Mi statistics rows: twice the fixed array
    q = torch.empty(1, 1, 1, 128, dtype=torch.bfloat16, device="cuda")
    a = _lib.AttnBwdBlockArgs()
    for name in ("dout", "q", "out", "k", "v", "lse", "dq", "dk", "dv"):
        setattr(a, name, q.data_ptr())
    a.batch, a.sq, a.sk, a.hq, a.hkv, a.head_dim = 2, 32768, 128, 32, 32, 128
    a.out_mode = _lib.MB_OUT_BF16
    rc = _lib.lib.mb_attn_bwd_block_noalloc(C.byref(a), None)
    assert rc == -6
    with pytest.raises(_lib.MercuryB200Error, match="MB_E_TOO_LARGE"):
        _lib.check(rc, "mb_attn_bwd_block_noalloc")
    # one row past the limit (the row count is padded to 64 first): still refused, nothing launched
    a.batch, a.sq = 1, 32768 + 1
    assert _lib.lib.mb_attn_bwd_block_noalloc(C.byref(a), None) == -6


def test_noalloc_backward_at_exactly_the_limit_allocates_nothing():
    """batch 1 x 32 heads x 32768 query rows = 1 048 576 statistics rows: the last element of each half
    of the fixed array is in use.  The result equals the regular path bit for bit, and the free device
    memory the driver reports is the same before and after the call (a second call, so that one-time
    set-up -- the address look-up, kernel attributes, module load -- is out of the picture)."""
    import mercury_artifact_b200 as mb
    from mercury_artifact_b200 import _lib

    B, Sq, Sk, H = 1, 32768, 256, 32
    scale = 128 ** -0.5
    q, _, _, do = seeded_qkv(43, B, Sq, H, H, 128, device="cuda")
    _, k, v, _ = seeded_qkv(44, B, Sk, H, H, 128, device="cuda")
    out, lse = mb.attn_fwd_segments(q, [(k, v, 0)], scale, causal=False)
    rdq, rdk, rdv = _regular_backward(q, k, v, do, out, lse, scale, False, 0, 0)
    rc, dq, dkv = _noalloc_backward(q, k, v, do, out, lse, scale, False, 0, 0)   # first call: set-up included
    assert rc == 0, _lib.ERROR_NAMES.get(rc, rc)
    torch.cuda.synchronize()
    # outputs for the measured call exist already; nothing else is created between the two readings
    dq2 = torch.empty_like(q)
    dkv2 = torch.empty((2,) + tuple(k.shape), dtype=torch.bfloat16, device="cuda")
    a = _lib.AttnBwdBlockArgs()
    a.dout, a.q, a.out = do.data_ptr(), q.data_ptr(), out.data_ptr()
    a.q_stride_b, a.q_stride_s, a.q_stride_h = q.stride(0), q.stride(1), q.stride(2)
    a.k, a.v = k.data_ptr(), v.data_ptr()
    a.kv_stride_b, a.kv_stride_s, a.kv_stride_h = k.stride(0), k.stride(1), k.stride(2)
    a.lse, a.dq = lse.data_ptr(), dq2.data_ptr()
    a.dq_stride_b, a.dq_stride_s, a.dq_stride_h = dq2.stride(0), dq2.stride(1), dq2.stride(2)
    a.dk, a.dv = dkv2[0].data_ptr(), dkv2[1].data_ptr()
    a.dkv_stride_b, a.dkv_stride_s, a.dkv_stride_h = dkv2[0].stride(0), dkv2[0].stride(1), dkv2[0].stride(2)
    a.batch, a.sq, a.sk, a.hq, a.hkv, a.head_dim = B, Sq, Sk, H, H, 128
    a.out_mode, a.softmax_scale, a.status = _lib.MB_OUT_BF16, scale, None
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    rc = _lib.lib.mb_attn_bwd_block_noalloc(C.byref(a), stream)
    torch.cuda.synchronize()
    free_after = torch.cuda.mem_get_info()[0]
    assert rc == 0, _lib.ERROR_NAMES.get(rc, rc)
    assert free_after == free_before, (free_before, free_after)
    assert _lib.status_fetch(torch.cuda.current_stream().cuda_stream) == 0
    for got in ((dq, dkv), (dq2, dkv2)):
        assert torch.equal(got[0], rdq) and torch.equal(got[1][0], rdk) and torch.equal(got[1][1], rdv)
