"""Parity of the sm_100a forward kernel (through the C ABI) against the CPU oracle.

Tolerances are the ones the task states: bf16 O max-abs <= 2e-2 and LSE <= 1e-3
against fp32 attention on the same seeded inputs.
"""
import pytest
import torch

from tests.helpers import seeded_qkv

pytestmark = pytest.mark.gpu

O_TOL = 2e-2
LSE_TOL = 1e-3


def _mb():
    import mercury_artifact_b200 as mb

    return mb


def _check(o, lse, ro, rl):
    o, lse = o.float().cpu(), lse.cpu()
    fin = torch.isfinite(rl)
    assert not torch.isnan(o).any()
    assert (o - ro.float()).abs().max().item() <= O_TOL
    if fin.any():
        assert (lse - rl)[fin].abs().max().item() <= LSE_TOL
    if (~fin).any():
        assert torch.equal(lse[~fin], rl[~fin])  # rows with no visible key: -inf on both sides


def _status_ok():
    from mercury_artifact_b200 import _lib

    assert _lib.status_fetch(torch.cuda.current_stream().cuda_stream) == 0


CASES = [
    # B, Sq, Sk, Hq, Hkv, causal, q_off
    (1, 256, 128, 1, 1, False, 0),
    (1, 256, 1024, 2, 2, False, 0),
    (2, 1024, 2048, 4, 4, False, 0),
    (1, 1024, 1024, 2, 2, True, 0),
    (1, 512, 1024, 2, 2, True, 512),     # bottom-right aligned causal, Sq < Sk
    (1, 1024, 512, 2, 2, True, -512),    # Sq > Sk: the first 512 rows see nothing
    (1, 300, 333, 2, 2, False, 0),       # ragged
    (2, 391, 391, 2, 2, True, 0),        # ragged + causal
    (1, 1, 1, 1, 1, False, 0),           # single query, single key
    (1, 128, 257, 1, 1, True, 129),
    (1, 512, 768, 8, 2, True, 256),      # GQA 4:1
    (2, 640, 640, 32, 8, True, 0),       # GQA, config-3 head layout
]


@pytest.mark.parametrize("B,Sq,Sk,Hq,Hkv,causal,q_off", CASES)
def test_block_forward_matches_oracle(B, Sq, Sk, Hq, Hkv, causal, q_off):
    from oracle import block

    mb = _mb()
    S = max(Sq, Sk)
    q, k, v, _ = seeded_qkv(1234, B, S, Hq, Hkv, 128, device="cuda")
    q, k, v = q[:, :Sq].contiguous(), k[:, :Sk].contiguous(), v[:, :Sk].contiguous()
    scale = 128 ** -0.5
    o, lse = mb.attn_fwd_segments(q, [(k, v, 0)], scale, causal=causal, q_off=q_off)
    _status_ok()
    ro, rl = block.block_attn_fwd(q.cpu(), k.cpu(), v.cpu(), scale, causal=causal, q_off=q_off, k_off=0)
    _check(o, lse, ro, rl)


def test_drop_in_block_call_signature_and_alignment():
    """_flash_attn_forward(**params) as the generated code calls it; causal is bottom-right aligned."""
    from oracle import block

    mb = _mb()
    q, k, v, _ = seeded_qkv(7, 1, 768, 4, 4, 128, device="cuda")
    q = q[:, :256].contiguous()
    params = mb.get_default_args(mb._flash_attn_forward).copy()
    assert params["softcap"] == 0.0 and set(params) >= {"q", "k", "v", "dropout_p", "softmax_scale", "causal"}
    params.update(dict(q=q, k=k, v=v, dropout_p=0, softmax_scale=128 ** -0.5, causal=True, alibi_slopes=None,
                       return_softmax=False, window_size_left=-1, window_size_right=-1))
    outputs = mb._flash_attn_forward(**params)
    assert len(outputs) == 4
    ro, rl = block.block_attn_fwd(q.cpu(), k.cpu(), v.cpu(), 128 ** -0.5, causal=True)
    _check(outputs[0], outputs[1], ro, rl)
    assert outputs[0].dtype == q.dtype and outputs[1].dtype == torch.float32 and outputs[1].shape == (1, 4, 256)


def test_unsupported_options_raise():
    mb = _mb()
    q, k, v, _ = seeded_qkv(7, 1, 128, 1, 1, 128, device="cuda")
    with pytest.raises(NotImplementedError):
        mb._flash_attn_forward(q, k, v, 0.1, 1.0, False)
    with pytest.raises(NotImplementedError):
        mb._flash_attn_forward(q, k, v, 0.0, 1.0, False, 128, 0)
    with pytest.raises(NotImplementedError):
        mb._flash_attn_forward(q, k, v, 0.0, 1.0, False, -1, -1, 30.0)
    with pytest.raises(TypeError):
        mb.attn_fwd_segments(q.float(), [(k, v, 0)], 1.0)
    with pytest.raises(ValueError):
        mb.attn_fwd_segments(q.cpu(), [(k, v, 0)], 1.0)


def test_empty_inputs():
    mb = _mb()
    q, k, v, _ = seeded_qkv(7, 1, 256, 2, 2, 128, device="cuda")
    # no keys at all: o = 0, lse = -inf
    o, lse = mb.attn_fwd_segments(q, [(k[:, :0], v[:, :0], 0)], 1.0)
    _status_ok()
    assert (o == 0).all() and torch.isinf(lse).all() and (lse < 0).all()
    o, lse = mb.attn_fwd_segments(q, [], 1.0)
    assert (o == 0).all() and (lse == float("-inf")).all()
    # no queries: nothing to do
    o, lse = mb.attn_fwd_segments(q[:, :0], [(k, v, 0)], 1.0)
    assert o.shape[1] == 0 and lse.shape[2] == 0


def test_strided_views_of_packed_kv():
    """k = kv[0], v = kv[1] views of the packed [2,B,S,H,D] buffer, as the generated code passes them."""
    from oracle import block

    mb = _mb()
    q, k, v, _ = seeded_qkv(21, 2, 512, 4, 4, 128, device="cuda")
    kv = torch.stack([k, v]).contiguous()
    o, lse = mb.attn_fwd_segments(q, [(kv[0], kv[1], 0)], 128 ** -0.5)
    ro, rl = block.block_attn_fwd(q.cpu(), k.cpu(), v.cpu(), 128 ** -0.5)
    _check(o, lse, ro, rl)
    # sequence-sliced views (ring_divide sub-chunks)
    o2, lse2 = mb.attn_fwd_segments(q, [(kv[0][:, 128:384], kv[1][:, 128:384], 0)], 128 ** -0.5)
    ro2, rl2 = block.block_attn_fwd(q.cpu(), k[:, 128:384].cpu(), v[:, 128:384].cpu(), 128 ** -0.5)
    _check(o2, lse2, ro2, rl2)


@pytest.mark.parametrize("causal", [False, True])
def test_ring_segments_match_full_attention(causal):
    """One rank's whole ring as a single multi-segment call, in arrival order, with global positions."""
    from oracle import block
    from mercury_artifact_b200 import mesh

    mb = _mb()
    P, B, S, H = 4, 1, 2048, 4
    q, k, v, _ = seeded_qkv(99, B, S, H, H, 128, device="cuda")
    fo, fl = block.full_attention(q.cpu(), k.cpu(), v.cpu(), 128 ** -0.5, causal=causal)
    L = S // P
    for shape in [(4,), (2, 2)]:
        for r in range(P):
            order = mesh.kv_origin_schedule(r, shape)
            segs = [(k[:, o * L:(o + 1) * L], v[:, o * L:(o + 1) * L], o * L) for o in order]
            o, lse = mb.attn_fwd_segments(q[:, r * L:(r + 1) * L], segs, 128 ** -0.5, causal=causal, q_off=r * L)
            _check(o, lse, fo[:, r * L:(r + 1) * L], fl[:, :, r * L:(r + 1) * L])
    _status_ok()


@pytest.mark.parametrize("causal", [False, True])
def test_growing_scores_force_the_output_rescale(causal):
    """Keys whose scores grow from tile to tile: the running row max rises by far more than the lazy-rescale
    threshold (2^8 in the exponent), so the accumulated output is rescaled in tensor memory several times; the
    last segment repeats the growth across a segment boundary."""
    from oracle import block

    mb = _mb()
    B, S, H = 1, 1536, 2
    q, k, v, _ = seeded_qkv(5, B, S, H, H, 128, device="cuda")
    ramp = torch.linspace(1.0, 24.0, S, device="cuda").view(1, S, 1, 1)   # |score| grows ~24x along the keys
    k = (k.float() * ramp).bfloat16()
    fo, fl = block.full_attention(q.cpu(), k.cpu(), v.cpu(), 128 ** -0.5, causal=causal)
    o, lse = mb.attn_fwd_segments(q, [(k, v, 0)], 128 ** -0.5, causal=causal)
    _check(o, lse, fo, fl)
    segs = [(k[:, :640], v[:, :640], 0), (k[:, 640:], v[:, 640:], 640)]
    o, lse = mb.attn_fwd_segments(q, segs, 128 ** -0.5, causal=causal)
    _check(o, lse, fo, fl)
    _status_ok()


@pytest.mark.parametrize("causal,chunks", [(True, 4), (True, 16), (False, 4), (True, 3)])
def test_host_buffer_forward_matches_oracle(causal, chunks):
    """forward_host(): pinned host tensors in and out, sequence chunks pipelined over PCIe (chunks=3 does not
    divide into 128-row pieces and takes the plain copy-in / forward / copy-out path)."""
    from oracle import block
    from mercury_artifact_b200.ring import RingAttention

    B, S, H = 1, 2048, 4
    q, k, v, _ = seeded_qkv(7, B, S, H, H, 128, device="cpu")
    fo, fl = block.full_attention(q, k, v, 128 ** -0.5, causal=causal)
    q_host = q.contiguous().pin_memory()
    kv_host = torch.stack([k, v]).contiguous().pin_memory()
    o_host = torch.empty_like(q_host).pin_memory()
    lse_host = torch.empty((B, H, S), dtype=torch.float32).pin_memory()
    op = RingAttention((1,), B, S, H, H, 128, causal=causal)
    for _ in range(2):  # twice: the second call reuses the device buffers and streams
        o_host.zero_()
        lse_host.zero_()
        op.forward_host(q_host, kv_host, o_host, lse_host, chunks=chunks)
        _check(o_host, lse_host, fo, fl)
    _status_ok()


def test_full_size_properties_config2():
    """The headline benchmark shape (bf16 B1 S32768 H32 D128 causal): size-independent properties.

    * splitting K/V into segments at tile boundaries does not change a single bit;
    * query row 0 of a causal run attends to key 0 only: o[0] == v[0], lse[0] == scale * q0.k0;
    * merging the two half-sequence partial results reproduces the one-pass result.
    """
    mb = _mb()
    B, S, H = 1, 32768, 32
    q, k, v, _ = seeded_qkv(1234, B, S, H, H, 128, device="cuda")
    scale = 128 ** -0.5
    o1, l1 = mb.attn_fwd_segments(q, [(k, v, 0)], scale, causal=True)
    h = S // 2
    o2, l2 = mb.attn_fwd_segments(q, [(k[:, :h], v[:, :h], 0), (k[:, h:], v[:, h:], h)], scale, causal=True)
    _status_ok()
    assert torch.equal(o1, o2) and torch.equal(l1, l2)
    assert torch.equal(o1[:, 0], v[:, 0])
    want = (q[:, 0].float() * k[:, 0].float()).sum(-1) * scale
    assert (l1[:, :, 0] - want).abs().max().item() <= LSE_TOL
    # partials over disjoint key halves, merged by the drop-in merge
    pa, la = mb.attn_fwd_segments(q, [(k[:, :h], v[:, :h], 0)], scale, causal=True)
    pb, lb = mb.attn_fwd_segments(q[:, h:], [(k[:, h:], v[:, h:], h)], scale, causal=True, q_off=h)
    out, lse = mb.update_out_and_lse(None, None, pa[:, h:], la[:, :, h:].contiguous())
    out, lse = mb.update_out_and_lse(out, lse, pb, lb)
    assert (out - o1[:, h:].float()).abs().max().item() <= O_TOL
    assert (lse.squeeze(-1).transpose(1, 2) - l1[:, :, h:]).abs().max().item() <= LSE_TOL
    assert torch.equal(pa[:, :h], o1[:, :h])


@pytest.mark.gpu
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("one_launch", [False, True])
def test_carried_state_chain_equals_one_job_bitwise(causal, one_launch):
    """A query shard processed as a chain of jobs, one per K/V shard, each continuing the online-softmax
    state the previous one stored (mb_fwd_job.state_*), gives the bits of one job over all the shards:
    as separate launches of one stream, and as ONE launch whose jobs hand over through chain words.
    Ragged sizes, GQA, a shard that the early query rows cannot see (their state passes through), and a
    first shard that late-positioned keys make invisible to every row of some tiles."""
    import mercury_artifact_b200 as mb
    from mercury_artifact_b200 import _lib
    from mercury_artifact_b200.attention import attn_fwd_multi
    from tests.helpers import seeded_qkv

    dev = torch.device("cuda", 0)
    B, Sq, Sk, H, hkv, D = 2, 1000, 1400, 4, 2, 128
    q, _, _, _ = seeded_qkv(5, B, Sq, H, hkv, D, device="cuda")
    _, k, v, _ = seeded_qkv(6, B, Sk, H, hkv, D, device="cuda")
    scale = D ** -0.5
    q_off = 300
    # K/V shards in "arrival" order: the middle one first (keys 500..899 are invisible to rows < 200 when
    # causal), then the head, then the tail (1 000..1 399: invisible to most rows, ragged)
    cuts = [(500, 900), (0, 500), (900, 1400)]
    segs = [(k[:, a:b], v[:, a:b], a) for a, b in cuts]
    ref_o, ref_l = mb.attn_fwd_segments(q, segs, scale, causal=causal, q_off=q_off)

    o = torch.full_like(q, 7.0)
    lse = torch.full((B, H, Sq), 7.0, device=dev)
    st_o = torch.full((B, H, Sq, D), float("nan"), device=dev)
    st_ml = torch.full((B, H, Sq, 2), float("nan"), device=dev)
    n_pairs = (Sq + 255) // 256
    chain = torch.zeros(B, H, n_pairs, dtype=torch.int32, device=dev)
    jobs = []
    for t in range(len(segs)):
        j = {"q": q, "q_off": q_off, "seg_mask": 1 << t, "state": (st_o, st_ml),
             "state_in": t > 0, "state_out": t < len(segs) - 1}
        if t == len(segs) - 1:
            j["out_raw"] = (o.data_ptr(), o.stride(0), o.stride(1), o.stride(2))
            j["lse_raw"] = (lse.data_ptr(), lse.stride(0), lse.stride(1))
        if one_launch:
            j["chain"] = (chain.data_ptr(), t, t + 1)
        jobs.append(j)
    if one_launch:
        attn_fwd_multi(jobs, segs, scale, causal, B, H, hkv, D, dev)
    else:
        for j in jobs:
            attn_fwd_multi([j], segs, scale, causal, B, H, hkv, D, dev)
    assert _lib.status_fetch(torch.cuda.current_stream().cuda_stream) == 0
    assert torch.equal(o, ref_o)
    assert torch.equal(lse, ref_l)
    if one_launch:
        assert chain.unique().tolist() == [len(segs) - 1]


@pytest.mark.gpu
def test_carried_state_is_the_unnormalised_accumulator():
    """What a state_out job stores: rows o * l with l the sum of exp(scale * (s - m)) and m the stored
    maximum, so that o = state_o / l and lse = scale * m + ln(l) reproduce the one-job result; rows without
    a visible key store (0, -inf, 0).  Two chains in one launch (two query shards) do not disturb each other."""
    import mercury_artifact_b200 as mb
    from mercury_artifact_b200 import _lib
    from mercury_artifact_b200.attention import attn_fwd_multi
    from tests.helpers import seeded_qkv

    dev = torch.device("cuda", 0)
    B, S, H, D = 1, 512, 2, 128
    q, k, v, _ = seeded_qkv(9, B, S, H, H, D, device="cuda")
    scale = D ** -0.5
    segs = [(k[:, 256:], v[:, 256:], 256), (k[:, :256], v[:, :256], 0)]
    ref_o, ref_l = mb.attn_fwd_segments(q, segs, scale, causal=True, q_off=0)
    halves = [slice(0, 256), slice(256, 512)]
    o = torch.zeros_like(q)
    lse = torch.zeros(B, H, S, device=dev)
    states = [(torch.zeros(B, H, 256, D, device=dev), torch.zeros(B, H, 256, 2, device=dev)) for _ in halves]
    chain = torch.zeros(2, B, H, 1, dtype=torch.int32, device=dev)
    jobs = []
    for t in range(2):                      # shard-major order: both chains' first jobs, then their second ones
        for c, rows in enumerate(halves):
            j = {"q": q[:, rows], "q_off": rows.start, "seg_mask": 1 << t, "state": states[c],
                 "state_in": t == 1, "state_out": t == 0, "chain": (chain[c].data_ptr(), t, t + 1)}
            if t == 1:
                j["out_raw"] = (o[:, rows].data_ptr(), o.stride(0), o.stride(1), o.stride(2))
                j["lse_raw"] = (lse[:, :, rows].data_ptr(), lse.stride(0), lse.stride(1))
            jobs.append(j)
    attn_fwd_multi(jobs[:2], segs, scale, True, B, H, H, D, dev)      # first jobs alone: look at the state
    torch.cuda.synchronize()
    so, sml = states[0]                    # rows 0..255 see nothing of keys 256..511
    assert so.abs().max().item() == 0 and torch.isneginf(sml[..., 0]).all() and (sml[..., 1] == 0).all()
    so, sml = states[1]                    # rows 256..511 against keys 256..511, causal
    po, pl = mb.attn_fwd_segments(q[:, 256:], segs[:1], scale, causal=True, q_off=256)
    m, l = sml[..., 0], sml[..., 1]
    assert (l > 0).all()
    assert ((so / l[..., None]).transpose(1, 2) - po.float()).abs().max().item() <= 2e-2
    assert (m * scale + l.log() - pl).abs().max().item() <= 1e-3
    chain.zero_()
    attn_fwd_multi(jobs, segs, scale, True, B, H, H, D, dev)
    assert _lib.status_fetch(torch.cuda.current_stream().cuda_stream) == 0
    assert torch.equal(o, ref_o) and torch.equal(lse, ref_l)


@pytest.mark.gpu
@pytest.mark.parametrize("causal", [False, True])
def test_eight_chains_of_one_launch_like_one_rank_of_eight(causal):
    """The launch one rank of an 8-rank heads schedule issues, with all data local: 8 query chunks x 8 K/V shards
    in an arrival order that starts in the middle, 36 jobs (causal: 24) that share 8 query tensor maps, one
    state chain per chunk -- the first job of a chunk takes every shard that arrived before its queries did.
    Bit-identical to one job per chunk over the same shard order."""
    import mercury_artifact_b200 as mb
    from mercury_artifact_b200 import _lib
    from mercury_artifact_b200.attention import attn_fwd_multi
    from tests.helpers import seeded_qkv

    dev = torch.device("cuda", 0)
    P, B, L, H, hkv, D = 8, 1, 512, 2, 1, 128
    S = P * L
    q, k, v, _ = seeded_qkv(77, B, S, H, hkv, D, device="cuda")
    scale = D ** -0.5
    me = 5
    order = [me] + [(me - t) % P for t in range(1, P)]
    segs = [(k[:, s * L:(s + 1) * L], v[:, s * L:(s + 1) * L], s * L) for s in order]
    o = torch.zeros_like(q)
    lse = torch.zeros(B, H, S, device=dev)
    states = [(torch.empty(B, H, L, D, device=dev), torch.empty(B, H, L, 2, device=dev),
               torch.zeros(B, H, L // 256, dtype=torch.int32, device=dev)) for _ in range(P)]
    plan = []
    for t in range(P):
        for n in range(t + 1):
            j = order[n]
            shards = range(t + 1) if n == t else (t,)
            mask = sum(1 << i for i in shards if (not causal) or order[i] <= j)
            if mask:
                plan.append((n, mask))
    count = [sum(1 for n, _ in plan if n == c) for c in range(P)]
    seen = [0] * P
    jobs = []
    for n, mask in plan:
        j = order[n]
        p, last = seen[n], seen[n] == count[n] - 1
        seen[n] += 1
        jb = {"q": q[:, j * L:(j + 1) * L], "q_off": j * L, "seg_mask": mask}
        if count[n] > 1:
            jb.update(state=states[n][:2], state_in=p > 0, state_out=not last, chain=(states[n][2].data_ptr(), p, p + 1))
        if last:
            jb["out_raw"] = (o[:, j * L:].data_ptr(), o.stride(0), o.stride(1), o.stride(2))
            jb["lse_raw"] = (lse[:, :, j * L:].data_ptr(), lse.stride(0), lse.stride(1))
        jobs.append(jb)
    assert len(jobs) == (24 if causal else 36)      # more than one launch used to take
    attn_fwd_multi(jobs, segs, scale, causal, B, H, hkv, D, dev)
    assert _lib.status_fetch(torch.cuda.current_stream().cuda_stream) == 0
    for j in range(P):
        ro, rl = mb.attn_fwd_segments(q[:, j * L:(j + 1) * L], segs, scale, causal=causal, q_off=j * L)
        assert torch.equal(o[:, j * L:(j + 1) * L], ro), j
        assert torch.equal(lse[:, :, j * L:(j + 1) * L], rl), j
