"""Results at the full benchmark sizes against the fp32 row-sampled checker (oracle/sampled.py).

The full score matrix of these problems does not fit anywhere, so a seeded sample of rows --
always holding the first and last row of the sequence and the rows either side of its middle --
is compared with fp32 attention over ALL keys (forward, dQ) or ALL queries (dK, dV).  The checker
runs on the GPU in fp32 (TF32 off) for 64 rows, and a handful of the same rows are evaluated again
on the CPU so that the GPU-evaluated checker is itself pinned to a CPU evaluation.
Tolerances: bf16 o / dq / dk / dv max-abs <= 2e-2, fp32 lse max-abs <= 1e-3.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

O_TOL, LSE_TOL = 2e-2, 1e-3


def _inputs(B, S, H, hkv, D, seed, with_dout=False):
    g = torch.Generator(device="cuda").manual_seed(seed)
    mk = lambda *shape: (torch.randn(*shape, generator=g, device="cuda") * 0.5).to(torch.bfloat16)
    q, kv = mk(B, S, H, D), mk(2, B, S, hkv, D)
    return (q, kv, mk(B, S, H, D)) if with_dout else (q, kv)


def _status_ok():
    from mercury_artifact_b200 import _lib

    assert _lib.status_fetch(torch.cuda.current_stream().cuda_stream) == 0


@pytest.mark.parametrize("B,S,H,hkv,causal", [
    (1, 32768, 32, 32, True),     # the headline shape
    (1, 131072, 32, 32, True),    # the 131072-token causal forward
    (2, 131072, 32, 8, True),     # GQA, group 4
    (1, 262144, 16, 16, False),   # the double-ring workload's shape (non-causal)
])
def test_forward_at_benchmark_sizes(B, S, H, hkv, causal):
    import mercury_artifact_b200 as mb
    from oracle import sampled

    torch.backends.cuda.matmul.allow_tf32 = False
    q, kv = _inputs(B, S, H, hkv, 128, seed=2024)
    scale = 128 ** -0.5
    o, lse = mb.attn_fwd_segments(q, [(kv[0], kv[1], 0)], scale, causal=causal)
    _status_ok()
    r = sampled.check_forward_shard(q, kv, o, lse, 0, 1, causal, scale, rows=64)
    assert r["rows"] == 64
    assert r["o_max_abs"] <= O_TOL and r["lse_max_abs"] <= LSE_TOL, r
    # the same checker on the CPU for a few of those rows (first, middle, last)
    pos = torch.tensor([0, S // 2 - 1, S // 2, S - 1])
    co, cl = sampled.fwd_rows(q[:, pos].cpu(), pos, kv[0].cpu(), kv[1].cpu(), scale, causal)
    assert (o[:, pos].float().cpu() - co).abs().max().item() <= O_TOL
    assert (lse[:, :, pos].cpu() - cl).abs().max().item() <= LSE_TOL
    del q, kv, o, lse
    torch.cuda.empty_cache()


def test_backward_at_benchmark_size():
    """bf16 B1 S65536 H32 D128 causal: dq, dk, dv of the whole sequence on one GPU."""
    import mercury_artifact_b200 as mb
    from oracle import sampled

    torch.backends.cuda.matmul.allow_tf32 = False
    B, S, H, causal = 1, 65536, 32, True
    q, kv, do = _inputs(B, S, H, H, 128, seed=2025, with_dout=True)
    scale = 128 ** -0.5
    o, lse = mb.attn_fwd_segments(q, [(kv[0], kv[1], 0)], scale, causal=causal)
    st = mb.bwd_preprocess(do, o, lse)
    dq = mb.attn_bwd_dq(q, do, st, [(kv[0], kv[1], 0)], scale, causal=causal, q_off=0)
    dkv = torch.empty_like(kv)
    mb.attn_bwd_dkv(kv[0], kv[1], [(q, do, st, 0)], scale, causal=causal, k_off=0, dk=dkv[0], dv=dkv[1])
    _status_ok()
    r = sampled.check_backward_shard(q, kv, o, lse, do, dq, dkv, 0, 1, causal, scale, rows=48)
    assert max(r["dq_max_abs"], r["dk_max_abs"], r["dv_max_abs"]) <= O_TOL, r
    # CPU evaluation of two query rows and two key rows
    pos = torch.tensor([S // 2, S - 1])
    cq = sampled.dq_rows(q[:, pos].cpu(), do[:, pos].cpu(), o[:, pos].cpu(), lse[:, :, pos].cpu(), pos, kv[0].cpu(),
                         kv[1].cpu(), scale, causal)
    assert (dq[:, pos].float().cpu() - cq).abs().max().item() <= O_TOL
    kp = torch.tensor([0, S // 2 - 1])
    ck, cv = sampled.dkv_rows(kv[0][:, kp].cpu(), kv[1][:, kp].cpu(), kp, q.cpu(), do.cpu(), o.cpu(), lse.cpu(), scale,
                              causal)
    assert (dkv[0][:, kp].float().cpu() - ck).abs().max().item() <= O_TOL
    assert (dkv[1][:, kp].float().cpu() - cv).abs().max().item() <= O_TOL
