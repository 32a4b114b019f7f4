"""The row-sampled fp32 checker (oracle/sampled.py) against the full-matrix oracle (oracle/block.py)."""
import pytest
import torch

from oracle import block, sampled
from tests.helpers import seeded_qkv


@pytest.mark.parametrize("causal,hkv", [(False, 4), (True, 4), (True, 2)])
def test_sampled_rows_equal_full_oracle(causal, hkv):
    B, S, H, D = 2, 320, 4, 32
    q, k, v, do = seeded_qkv(5, B, S, H, hkv, D, dtype=torch.float32)
    scale = D ** -0.5
    fo, fl = block.full_attention(q, k, v, scale, causal=causal)
    gq, gk, gv = block.block_attn_bwd(do, q, k, v, fo, fl, scale, causal=causal, q_off=0, k_off=0)
    pos = sampled.sample_positions(S, 24, seed=3, must=(0, S - 1, S // 2 - 1, S // 2))
    assert 0 in pos.tolist() and S - 1 in pos.tolist() and len(set(pos.tolist())) == len(pos) == 24
    o, lse = sampled.fwd_rows(q[:, pos], pos, k, v, scale, causal)
    assert (o - fo[:, pos]).abs().max().item() <= 5e-5
    assert (lse - fl[:, :, pos]).abs().max().item() <= 5e-5
    dq = sampled.dq_rows(q[:, pos], do[:, pos], fo[:, pos], fl[:, :, pos], pos, k, v, scale, causal)
    assert (dq - gq[:, pos]).abs().max().item() <= 5e-5
    dk, dv = sampled.dkv_rows(k[:, pos], v[:, pos], pos, q, do, fo, fl, scale, causal)
    assert (dk - gk[:, pos]).abs().max().item() <= 5e-5
    assert (dv - gv[:, pos]).abs().max().item() <= 5e-5


def test_sampled_rows_with_offsets_match_a_shard_of_the_full_problem():
    """Keys given as a shard (k_off) and queries as a shard (q_off) reproduce the matching slices."""
    B, S, H, D = 1, 256, 2, 32
    q, k, v, do = seeded_qkv(9, B, S, H, H, D, dtype=torch.float32)
    scale = D ** -0.5
    fo, fl = block.full_attention(q, k, v, scale, causal=True)
    pos = torch.tensor([130, 131, 200, 255])
    # forward against the second half of the keys only == block forward of those rows vs that shard
    o, lse = sampled.fwd_rows(q[:, pos], pos, k[:, 128:], v[:, 128:], scale, True, k_off=128)
    bo, bl = block.block_attn_fwd(q[:, pos[0]:], k[:, 128:], v[:, 128:], scale, causal=True, q_off=int(pos[0]), k_off=128)
    assert (o - bo[:, pos - pos[0]]).abs().max().item() <= 5e-5
    assert (lse - bl[:, :, pos - pos[0]]).abs().max().item() <= 5e-5
    # dK/dV of sampled keys against the second half of the queries only
    kp = torch.tensor([0, 100, 128, 250])
    dk, dv = sampled.dkv_rows(k[:, kp], v[:, kp], kp, q[:, 128:], do[:, 128:], fo[:, 128:], fl[:, :, 128:], scale, True,
                              q_off=128)
    _, gk, gv = block.block_attn_bwd(do[:, 128:], q[:, 128:], k, v, fo[:, 128:], fl[:, :, 128:], scale, causal=True,
                                     q_off=128, k_off=0)
    assert (dk - gk[:, kp]).abs().max().item() <= 5e-5
    assert (dv - gv[:, kp]).abs().max().item() <= 5e-5
