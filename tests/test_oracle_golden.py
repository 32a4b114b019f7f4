"""Pin the CPU oracle against vectors produced by the reference's own generated code."""
import pytest
import torch

from oracle import block, merge, ring
from tests.helpers import load_golden, shard_inputs

FWD_CASES = ["ring_p1", "ring_p2", "ring_p4", "gqa_p2", "double_ring_2x2"]


@pytest.mark.parametrize("name", FWD_CASES)
def test_forward_schedules_match_reference_output(name):
    g = load_golden(name)
    t = g["t"]
    qs, kvs = shard_inputs(t["q"], t["k"], t["v"], g["world"])
    outs, lses = ring.simulate_ring_fwd(qs, kvs, g["D"] ** -0.5, g["mesh"])
    for r in range(g["world"]):
        # same fp32 arithmetic in the same order: expect agreement to rounding
        assert torch.allclose(outs[r], t[f"o_rank{r}"], rtol=0, atol=1e-4), name
        assert torch.allclose(lses[r], t[f"lse_rank{r}"], rtol=0, atol=1e-4), name


@pytest.mark.parametrize("name", FWD_CASES)
def test_reference_output_equals_full_attention(name):
    """The reference's own acceptance check (tests/test_ring_attn_codegen.py:120-148): every rank's
    chunk of the ring result equals single-device attention."""
    g = load_golden(name)
    t = g["t"]
    fo, fl = block.full_attention(t["q"], t["k"], t["v"], g["D"] ** -0.5)
    for r in range(g["world"]):
        assert torch.allclose(fo.chunk(g["world"], 1)[r], t[f"o_rank{r}"], atol=1e-4)
        assert torch.allclose(fl.chunk(g["world"], 2)[r], t[f"lse_rank{r}"], atol=1e-4)


@pytest.mark.parametrize("name", ["bwd_p2", "bwd_p4"])
def test_backward_schedule_matches_reference_output(name):
    g = load_golden(name)
    t = g["t"]
    w = g["world"]
    scale = g["D"] ** -0.5
    qs, kvs = shard_inputs(t["q"], t["k"], t["v"], w)
    fo, fl = block.full_attention(t["q"], t["k"], t["v"], scale)
    dq, dkv = ring.simulate_ring_bwd(qs, kvs, list(fo.chunk(w, 1)), list(fl.chunk(w, 2)),
                                     list(t["dout"].chunk(w, 1)), scale, g["mesh"])
    for r in range(w):
        assert torch.allclose(dq[r], t[f"dq_rank{r}"], atol=1e-4)
        assert torch.allclose(dkv[r], t[f"dkv_rank{r}"], atol=1e-4)


def test_backward_matches_autograd():
    torch.manual_seed(3)
    B, S, H, hkv, D = 2, 96, 4, 2, 16
    q = torch.randn(B, S, H, D, requires_grad=True)
    k = torch.randn(B, S, hkv, D, requires_grad=True)
    v = torch.randn(B, S, hkv, D, requires_grad=True)
    do = torch.randn(B, S, H, D)
    for causal in (False, True):
        kk = k.repeat_interleave(H // hkv, 2)
        vv = v.repeat_interleave(H // hkv, 2)
        s = torch.einsum("bqhd,bkhd->bhqk", q, kk) * D ** -0.5
        if causal:
            s = s.masked_fill(~torch.ones(S, S, dtype=torch.bool).tril(), float("-inf"))
        o = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, -1), vv)
        gq, gk, gv = torch.autograd.grad(o, (q, k, v), do)
        fo, fl = block.block_attn_fwd(q.detach(), k.detach(), v.detach(), D ** -0.5, causal=causal)
        assert torch.allclose(fo, o.detach(), atol=1e-4)
        dq, dk, dv = block.block_attn_bwd(do, q.detach(), k.detach(), v.detach(), fo, fl, D ** -0.5, causal=causal)
        assert torch.allclose(dq, gq, atol=1e-4) and torch.allclose(dk, gk, atol=1e-4) and torch.allclose(dv, gv, atol=1e-4)


def test_merge_formula_equals_logsumexp_identity():
    torch.manual_seed(0)
    B, S, H, D = 2, 40, 3, 8
    parts = [(torch.randn(B, S, H, D), torch.randn(B, H, S) * 3) for _ in range(5)]
    out = lse = None
    for po, pl in parts:
        out, lse = merge.update_out_and_lse(out, lse, po, pl)
    eo, el = merge.merge_exact(parts)
    assert torch.allclose(out, eo, atol=1e-4)
    assert torch.allclose(lse.squeeze(-1).transpose(1, 2), el, atol=1e-4)
    packed = [torch.cat([po, pl.transpose(1, 2).unsqueeze(-1)], -1) for po, pl in parts]
    acc = packed[0]
    for p in packed[1:]:
        acc = merge.flash_reduce(acc, p)
    assert torch.allclose(acc[..., :-1], eo, atol=1e-4)


def test_update_out_and_lse_rejects_slice_on_first_call():
    with pytest.raises(RuntimeError):
        merge.update_out_and_lse(None, None, torch.zeros(1, 2, 1, 4), torch.zeros(1, 1, 2), slice_=(slice(None),))


@pytest.mark.parametrize("shape", [(2,), (4,), (8,), (2, 2), (4, 2), (2, 4)])
def test_every_rank_sees_every_shard_once(shape):
    p = 1
    for n in shape:
        p *= n
    for r in range(p):
        sched = ring.kv_origin_schedule(r, shape)
        assert sched[0] == r and sorted(sched) == list(range(p))


def test_double_ring_origin_formula():
    # inner ring over mesh dim 0 (4 ranks), one outer hop over mesh dim 1
    for r in range(8):
        want = [((r % 4 - 3 * o - i) % 4) + 4 * ((r // 4 - o) % 2) for o in range(2) for i in range(4)]
        assert ring.kv_origin_schedule(r, (4, 2)) == want


def test_causal_ring_equals_full_causal_attention():
    """No reference behaviour exists for causal rings (parity unpinned): the build's positional
    rule is checked against single-device causal attention."""
    torch.manual_seed(1)
    B, S, H, D = 1, 256, 2, 32
    q, k, v = (torch.randn(B, S, H, D) for _ in range(3))
    fo, fl = block.full_attention(q, k, v, D ** -0.5, causal=True)
    for shape in [(4,), (2, 2)]:
        qs, kvs = shard_inputs(q, k, v, 4)
        o, l = ring.simulate_ring_fwd(qs, kvs, D ** -0.5, shape, positional_causal=True)
        assert torch.allclose(torch.cat(o, 1), fo, atol=1e-4)
        assert torch.allclose(torch.cat(l, 2), fl, atol=1e-4)


def test_config1_ring_fp32_matches_full_attention():
    """The reference's CPU-runnable case: fp32, B1 S4096 H8 D64, non-causal, 2 contiguous shards."""
    g = torch.Generator().manual_seed(1234)
    B, S, H, D = 1, 4096, 8, 64
    q, k, v = (torch.randn(B, S, H, D, generator=g) for _ in range(3))
    qs, kvs = shard_inputs(q, k, v, 2)
    o, l = ring.simulate_ring_fwd(qs, kvs, D ** -0.5, (2,))
    fo, fl = block.full_attention(q, k, v, D ** -0.5)
    assert (torch.cat(o, 1) - fo).abs().max() < 1e-5
    assert (torch.cat(l, 2) - fl).abs().max() < 1e-5


@pytest.mark.parametrize("name", ["ring_over_q_p2", "ring_over_q_p4"])
def test_ring_over_q_schedule_matches_reference_output(name):
    """K/V stationary, queries and the packed [out | lse] reduce buffer rotate (flash_reduce),
    with the write-back hop: oracle vs the reference's own generated program."""
    g = load_golden(name)
    t = g["t"]
    qs, kvs = shard_inputs(t["q"], t["k"], t["v"], g["world"])
    outs, lses = ring.simulate_ring_over_q(qs, kvs, g["D"] ** -0.5, g["mesh"])
    fo, fl = block.full_attention(t["q"], t["k"], t["v"], g["D"] ** -0.5)
    for r in range(g["world"]):
        assert torch.allclose(outs[r], t[f"o_rank{r}"], atol=1e-4)
        assert torch.allclose(lses[r], t[f"lse_rank{r}"], atol=1e-4)
        assert torch.allclose(fo.chunk(g["world"], 1)[r], t[f"o_rank{r}"], atol=1e-4)


@pytest.mark.parametrize("name", ["tree_p2", "tree_p4"])
def test_tree_merge_matches_reference_output(name):
    """K/V sharded, queries replicated, partial results merged by the all-reduce collective:
    the oracle's one-pass merge equals what the reference's three collectives leave on every rank."""
    g = load_golden(name)
    t = g["t"]
    w = g["world"]
    scale = g["D"] ** -0.5
    parts = []
    for r in range(w):
        k, v = t["k"].chunk(w, 1)[r], t["v"].chunk(w, 1)[r]
        bo, bl = block.block_attn_fwd(t["q"], k, v, scale)
        parts.append(torch.cat([bo.float(), bl.transpose(-2, -1).unsqueeze(-1)], dim=-1))
    res = merge.tree_merge(parts)
    fo, fl = block.full_attention(t["q"], t["k"], t["v"], scale)
    for r in range(w):
        assert torch.allclose(res[..., :-1], t[f"o_rank{r}"], atol=1e-4)
        assert torch.allclose(res[..., -1].transpose(1, 2), t[f"lse_rank{r}"], atol=1e-4)
        assert torch.allclose(fo, t[f"o_rank{r}"], atol=1e-4)
