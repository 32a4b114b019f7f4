"""The merge kernel against the oracle's restatement of update_out_and_lse."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shape", [(1, 128, 2, 128), (2, 333, 5, 64), (1, 4096, 32, 128)])
def test_running_merge_matches_oracle(dtype, shape):
    import mercury_artifact_b200 as mb
    from oracle import merge

    B, S, H, D = shape
    g = torch.Generator().manual_seed(5)
    parts = [((torch.randn(B, S, H, D, generator=g)).to(dtype), torch.randn(B, H, S, generator=g) * 4) for _ in range(4)]
    out = lse = None
    ro = rl = None
    for po, pl in parts:
        out, lse = mb.update_out_and_lse(out, lse, po.cuda(), pl.cuda())
        ro, rl = merge.update_out_and_lse(ro, rl, po, pl)
    assert out.dtype == torch.float32 and out.shape == (B, S, H, D) and lse.shape == (B, S, H, 1)
    assert (out.cpu() - ro).abs().max().item() <= 1e-5
    assert (lse.cpu() - rl).abs().max().item() <= 1e-5


def test_merge_slice_and_errors():
    import mercury_artifact_b200 as mb
    from oracle import merge

    B, S, H, D = 1, 256, 2, 128
    g = torch.Generator().manual_seed(6)
    o0, l0 = torch.randn(B, S, H, D, generator=g), torch.randn(B, H, S, generator=g)
    o1, l1 = torch.randn(B, 128, H, D, generator=g), torch.randn(B, H, 128, generator=g)
    with pytest.raises(RuntimeError):
        mb.update_out_and_lse(None, None, o0.cuda(), l0.cuda(), slice_=(slice(None), slice(0, 128)))
    sl = (slice(None), slice(128, 256))
    out, lse = mb.update_out_and_lse(None, None, o0.cuda(), l0.cuda())
    out, lse = mb.update_out_and_lse(out, lse, o1.cuda(), l1.cuda(), slice_=sl)
    ro, rl = merge.update_out_and_lse(None, None, o0, l0)
    ro, rl = merge.update_out_and_lse(ro, rl, o1, l1, slice_=sl)
    assert (out.cpu() - ro).abs().max().item() <= 1e-5 and (lse.cpu() - rl).abs().max().item() <= 1e-5


def test_merge_handles_rows_without_keys():
    """-inf block LSE leaves a row untouched; -inf running LSE adopts the block (causal partials)."""
    import mercury_artifact_b200 as mb

    B, S, H, D = 1, 64, 1, 128
    o0, o1 = torch.ones(B, S, H, D), torch.full((B, S, H, D), 3.0)
    l0, l1 = torch.zeros(B, H, S), torch.zeros(B, H, S)
    l1[..., :16] = float("-inf")
    l0[..., 48:] = float("-inf")
    out, lse = mb.update_out_and_lse(None, None, o0.cuda(), l0.cuda())
    out, lse = mb.update_out_and_lse(out, lse, o1.cuda(), l1.cuda())
    out, lse = out.cpu(), lse.cpu().squeeze(-1)
    assert not torch.isnan(out).any() and not torch.isnan(lse).any()
    assert (out[:, :16] == 1).all() and (out[:, 48:] == 3).all()
    assert torch.allclose(out[:, 16:48], torch.full((B, 32, H, D), 2.0))
    assert torch.allclose(lse[:, 16:48], torch.full((B, 32, H), 0.6931472))


@pytest.mark.parametrize("shape", [(1, 128, 2, 129), (2, 333, 5, 65), (1, 2048, 32, 129)])
def test_flash_reduce_matches_oracle(shape):
    import mercury_artifact_b200 as mb
    from oracle import merge

    g = torch.Generator().manual_seed(8)
    parts = [torch.randn(*shape, generator=g) for _ in range(3)]
    for p in parts:
        p[..., -1] *= 4
    acc = parts[0].cuda()
    ref = parts[0]
    for p in parts[1:]:
        acc = mb.flash_reduce(acc, p.cuda())
        ref = merge.flash_reduce(ref, p)
    assert acc.shape == ref.shape and acc.dtype == torch.float32
    assert (acc.cpu() - ref).abs().max().item() <= 1e-5
    with pytest.raises(ValueError):
        mb.flash_reduce(parts[0], parts[1])


@pytest.mark.parametrize("n,shape", [(2, (1, 128, 2, 129)), (8, (2, 100, 3, 65)), (16, (1, 64, 1, 129))])
def test_tree_merge_kernel_matches_oracle(n, shape):
    """mb_tree_merge on one device (all sources local) against the oracle's restatement of
    update_out_and_lse_collective; one source has rows without keys (lse = -inf)."""
    import ctypes as C

    from mercury_artifact_b200 import _lib
    from oracle import merge

    g = torch.Generator().manual_seed(9)
    parts = [torch.randn(*shape, generator=g) for _ in range(n)]
    for p in parts:
        p[..., -1] *= 3
    parts[0][:, :7, :, -1] = float("-inf")
    dev = [p.cuda() for p in parts]
    out = torch.empty_like(dev[0])
    srcs = (C.c_void_p * n)(*[d.data_ptr() for d in dev])
    width = shape[-1]
    rc = _lib.lib.mb_tree_merge(srcs, n, out.data_ptr(), out.numel() // width, width,
                                C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    ref = merge.tree_merge(parts)
    assert not torch.isnan(out).any()
    assert (out.cpu() - ref).abs().max().item() <= 1e-5
    assert _lib.lib.mb_tree_merge(srcs, 17, out.data_ptr(), 1, width, None) == -1
