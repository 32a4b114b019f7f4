"""Programs emitted by the reference's code generator, run with this package's drop-in ops.

The program text in tests/golden/gpu_*.gen.txt was produced by the unmodified reference
compiler (see tests/golden/make_golden.py).  It is exec'd here exactly as example.py of the
reference does, for P virtual ranks on one device; only the transport is a test double.
"""
import pytest
import torch

from tests.helpers import golden_text, seeded_qkv, shard_inputs
from tests.virtual_ranks import MailboxSendRecv, run_ranks

pytestmark = pytest.mark.gpu

O_TOL, LSE_TOL = 2e-2, 1e-3


def _run_forward(name, fn_name, world, B, S, H, hkv):
    import mercury_artifact_b200 as mb
    from oracle import block

    mb.install_backend(send_recv_cls=MailboxSendRecv, force_stub=True)
    ns = mb.load_generated(golden_text(name))
    fn = ns[fn_name]
    q, k, v, _ = seeded_qkv(1234, B, S, H, hkv, 128)
    qs, kvs = shard_inputs(q, k, v, world)
    scale = 128 ** -0.5

    def rank_body(r):
        lq, lkv = qs[r].cuda(), kvs[r].cuda()
        o = torch.zeros_like(lq)
        lse = torch.zeros(B, H, S // world, device="cuda")
        fn(lq, lkv, o, lse, scale)
        return o.float().cpu(), lse.cpu()

    res = run_ranks(world, rank_body)
    fo, fl = block.full_attention(q, k, v, scale)
    for r in range(world):
        assert (res[r][0] - fo.chunk(world, 1)[r].float()).abs().max().item() <= O_TOL
        assert (res[r][1] - fl.chunk(world, 2)[r]).abs().max().item() <= LSE_TOL
    from mercury_artifact_b200 import _lib

    assert _lib.status_fetch(torch.cuda.current_stream().cuda_stream) == 0


def test_unsharded_program():
    _run_forward("gpu_ring_p1", "flash_attn_pack_kv", 1, 1, 512, 4, 4)


def test_ring_program_two_ranks():
    _run_forward("gpu_ring_p2", "flash_attn_pack_kv", 2, 1, 1024, 4, 4)


def test_ring_program_four_ranks():
    _run_forward("gpu_ring_p4", "flash_attn_pack_kv", 4, 1, 2048, 4, 4)


@pytest.mark.parametrize("name", ["gpu_ring_p2_div2", "gpu_ring_p2_div4"])
def test_ring_divide_programs(name):
    """shift(..., ring_divide=2 | 4): the reference emits an outer loop over K/V sub-blocks with one ring
    round each; the text runs unchanged on the drop-in ops (more, smaller block calls and merges)."""
    _run_forward(name, "flash_attn_pack_kv", 2, 1, 1024, 4, 4)


def test_hybrid_program_ring_by_heads_2x2():
    """Mesh (2, 2): K/V ring along dimension 0, heads split along dimension 1.  The emitter leaves it alone
    (see test_emitter_leaves_hybrid_schedules_unfused) and it runs on the per-step drop-ins: rank
    (i0, i1) holds sequence shard i0 of head group i1."""
    import mercury_artifact_b200 as mb
    from mercury_artifact_b200 import emitter
    from oracle import block

    text = golden_text("gpu_hybrid_ring2_heads2")
    assert emitter.fuse_generated(text) == text
    mb.install_backend(send_recv_cls=MailboxSendRecv, force_stub=True)
    fn = mb.load_generated(text)["flash_attn_pack_kv"]
    B, S, H = 1, 1024, 4
    q, k, v, _ = seeded_qkv(1234, B, S, H, H, 128)
    scale = 128 ** -0.5

    def rank_body(r):
        i0, i1 = r % 2, r // 2
        rows, heads = slice(i0 * 512, (i0 + 1) * 512), slice(i1 * 2, (i1 + 1) * 2)
        lq = q[:, rows, heads].contiguous().cuda()
        lkv = torch.stack([k[:, rows, heads], v[:, rows, heads]]).contiguous().cuda()
        o = torch.zeros_like(lq)
        lse = torch.zeros(B, 2, 512, device="cuda")
        fn(lq, lkv, o, lse, scale)
        return o.float().cpu(), lse.cpu()

    res = run_ranks(4, rank_body)
    fo, fl = block.full_attention(q, k, v, scale)
    for r in range(4):
        i0, i1 = r % 2, r // 2
        rows, heads = slice(i0 * 512, (i0 + 1) * 512), slice(i1 * 2, (i1 + 1) * 2)
        assert (res[r][0] - fo[:, rows, heads].float()).abs().max().item() <= O_TOL
        assert (res[r][1] - fl[:, heads, rows]).abs().max().item() <= LSE_TOL


def test_gqa_ring_program():
    _run_forward("gpu_gqa_p2", "gqa_pack_kv", 2, 2, 1024, 8, 2)


def test_double_ring_program_2x2():
    _run_forward("gpu_double_ring_2x2", "flash_attn_pack_split_kv", 4, 1, 2048, 4, 4)


def test_double_ring_program_4x2():
    _run_forward("gpu_double_ring_4x2", "flash_attn_pack_split_kv", 8, 1, 4096, 2, 2)


def test_ring_over_q_program_two_ranks():
    """Ring-over-Q schedule (K/V stationary, queries + packed reduce buffer rotate, write-back hop)
    with the drop-in block op and the flash_reduce kernel."""
    _run_forward("gpu_ring_over_q_p2", "flash_attn_expose_reduce", 2, 1, 1024, 4, 4)


def test_ring_over_q_program_four_ranks():
    _run_forward("gpu_ring_over_q_p4", "flash_attn_expose_reduce", 4, 2, 1024, 4, 4)


def test_fused_rewrite_of_the_unsharded_program():
    """emitter.fuse_generated: same function name and signature, one fused call instead of the loop."""
    import mercury_artifact_b200 as mb
    from mercury_artifact_b200 import emitter
    from oracle import block

    ns = mb.load_generated(emitter.fuse_generated(golden_text("gpu_ring_p1")))
    q, k, v, _ = seeded_qkv(4321, 1, 512, 4, 4, 128)
    kv = torch.stack([k, v]).cuda()
    for causal in (False, True):
        o = torch.zeros(1, 512, 4, 128, dtype=torch.bfloat16, device="cuda")
        lse = torch.zeros(1, 4, 512, device="cuda")
        ns["flash_attn_pack_kv"](q.cuda(), kv, o, lse, 128 ** -0.5, causal=causal)
        fo, fl = block.full_attention(q, k, v, 128 ** -0.5, causal=causal)
        assert (o.float().cpu() - fo.float()).abs().max().item() <= O_TOL
        assert (lse.cpu() - fl).abs().max().item() <= LSE_TOL
    with pytest.raises(NotImplementedError):
        ns["flash_attn_pack_kv"](q.cuda(), kv, o, lse, 1.0, dropout_p=0.1)
