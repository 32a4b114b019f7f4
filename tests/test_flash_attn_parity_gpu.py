"""The drop-in block ops against the op they replace: flash-attn's own `_flash_attn_forward` /
`_flash_attn_backward` (flash_attn.flash_attn_interface), which is what the reference's DSL bodies
call (utils/flash_attn_dsl.py:174, utils/attn_bwd_dsl.py:115).  Same seeded bf16 inputs, same
keyword calls; checks the output, the LSE layout ([B, Hq, Sq] fp32, natural log of the scaled
scores), the bottom-right alignment of the causal mask when Sq != Sk, the in-place gradients and
softmax_d.  Skipped when the flash-attn wheel is absent or has no kernel for this GPU.
"""
import pytest
import torch

from tests.helpers import seeded_qkv

pytestmark = pytest.mark.gpu


def _flash_attn_ops():
    try:
        from flash_attn.flash_attn_interface import _flash_attn_backward, _flash_attn_forward
    except Exception as e:  # wheel not installed
        pytest.skip(f"flash-attn not importable: {e}")
    return _flash_attn_forward, _flash_attn_backward


@pytest.mark.parametrize("Sq,Sk,Hq,Hkv,causal", [
    (512, 512, 4, 4, False),
    (384, 640, 4, 4, True),     # bottom-right aligned causal mask, Sq != Sk
    (512, 512, 8, 2, True),     # GQA
    (300, 391, 4, 2, False),    # ragged sizes
])
def test_block_ops_equal_flash_attn(Sq, Sk, Hq, Hkv, causal):
    import mercury_artifact_b200 as mb
    from mercury_artifact_b200 import ops

    fa_fwd, fa_bwd = _flash_attn_ops()
    B, D = 2, 128
    S = max(Sq, Sk)
    q, k, v, do = seeded_qkv(31, B, S, Hq, Hkv, D, device="cuda")
    q, do = q[:, :Sq].contiguous(), do[:, :Sq].contiguous()
    k, v = k[:, :Sk].contiguous(), v[:, :Sk].contiguous()
    scale = D ** -0.5
    kw = dict(dropout_p=0.0, softmax_scale=scale, causal=causal, window_size_left=-1, window_size_right=-1,
              softcap=0.0, alibi_slopes=None)
    try:
        ro, rl, _, _ = fa_fwd(q=q, k=k, v=v, return_softmax=False, **kw)
        torch.cuda.synchronize()
    except Exception as e:
        pytest.skip(f"flash-attn cannot run on this GPU: {type(e).__name__}: {e}")
    o, lse, s_dmask, rng = ops._flash_attn_forward(q=q, k=k, v=v, return_softmax=False, **kw)
    assert s_dmask is None and rng is None
    assert o.shape == ro.shape and o.dtype == ro.dtype
    assert tuple(lse.shape) == tuple(rl.shape) == (B, Hq, Sq) and lse.dtype == rl.dtype == torch.float32
    assert bool(((o.float() - ro.float()).abs() <= 2e-2 + 2.0 ** -7 * ro.float().abs()).all())
    assert (lse - rl).abs().max().item() <= 1e-3

    # backward: both write dq, dk, dv in place and return softmax_d
    rdq, rdk, rdv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    rd = fa_bwd(dout=do, q=q, k=k, v=v, out=ro, softmax_lse=rl, dq=rdq, dk=rdk, dv=rdv, deterministic=False,
                rng_state=None, **kw)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    d = ops._flash_attn_backward(dout=do, q=q, k=k, v=v, out=ro, softmax_lse=rl, dq=dq, dk=dk, dv=dv,
                                 deterministic=False, rng_state=None, **kw)
    # both sides are bf16-rounded: beside the 2e-2 of the fp32 comparison allow one bf16 unit in the last place
    def close(a, b):
        return bool(((a.float() - b.float()).abs() <= 2e-2 + 2.0 ** -7 * b.float().abs()).all())

    assert close(dq, rdq) and close(dk, rdk) and close(dv, rdv)
    # softmax_d = rowsum(dout * out), [B, Hq, rows padded]: compare the Sq real rows
    assert d.shape[:2] == rd.shape[:2] == (B, Hq)
    assert (d[:, :, :Sq] - rd[:, :, :Sq].float()).abs().max().item() <= 2e-2
    from mercury_artifact_b200 import _lib

    assert _lib.status_fetch(torch.cuda.current_stream().cuda_stream) == 0
