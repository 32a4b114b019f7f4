"""CPU tests: mesh helpers, schedules, the exported C ABI, the drop-in namespace."""
import ctypes
import os
import re
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
# the reference checkout (needed only by the tests that compare with its own functions):
# MERCURY_REFERENCE, else a directory named "reference" beside this repository
REFERENCE = Path(os.environ.get("MERCURY_REFERENCE") or (ROOT.parent / "reference"))


def test_library_exports_every_declared_symbol():
    from mercury_artifact_b200 import _lib

    header = (ROOT / "include" / "mercury_b200.h").read_text()
    declared = set(re.findall(r"MB_API\s+\w[\w\s\*]*?\b(mb_\w+)\s*\(", header))
    assert {"mb_attn_fwd", "mb_merge_out_lse", "mb_status_fetch", "mb_version", "mb_flag_wait"} <= declared
    lib = ctypes.CDLL(str(_lib.LIB_PATH))
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in mercury_b200.h but not exported"
    out = subprocess.run(["nm", "-D", "--defined-only", str(_lib.LIB_PATH)], capture_output=True, text=True).stdout
    exported = {line.split()[-1] for line in out.splitlines() if " T " in line}
    assert declared <= exported
    assert _lib.lib.mb_version() >= 1000


def test_argument_validation_needs_no_gpu():
    from mercury_artifact_b200 import _lib

    assert _lib.lib.mb_attn_fwd(None, None) == -1
    a = _lib.AttnFwdArgs()
    a.head_dim = 64
    assert _lib.lib.mb_attn_fwd(ctypes.byref(a), None) == -2  # only head_dim 128 is built
    a.head_dim, a.batch, a.hq, a.hkv, a.nseg = 128, 1, 3, 2, 1
    assert _lib.lib.mb_attn_fwd(ctypes.byref(a), None) == -1  # hq not a multiple of hkv
    a.hq, a.nseg = 4, 33
    assert _lib.lib.mb_attn_fwd(ctypes.byref(a), None) == -1  # too many segments
    assert _lib.lib.mb_merge_out_lse(None, None) == -1
    assert _lib.lib.mb_flag_signal(None, 1, None) == -1


def test_mesh_helpers_match_oracle_and_reference_semantics():
    from mercury_artifact_b200 import mesh
    from oracle import ring

    for shape in [(2,), (8,), (2, 2), (4, 2), (2, 4), (2, 2, 2)]:
        p = 1
        for n in shape:
            p *= n
        for r in range(p):
            c = mesh.one_dim_to_n_dim(r, shape)
            assert c == ring.coords_of(r, shape) and mesh.n_dim_to_one_dim(c, shape) == r
            assert mesh.kv_origin_schedule(r, shape) == ring.kv_origin_schedule(r, shape)
            dims = tuple(range(len(shape)))
            assert mesh.get_src_dst_ranks(c, shape, dims) == ring.writeback_src_dst(c, shape, list(dims))
    assert mesh.one_dim_to_n_dim(5, (4, 2)) == (1, 1)
    assert mesh.shift_tuple_element((0, 1), 0, -1, 4) == (3, 1)
    assert mesh.shift_tuple_element((3, 1), 0, 1, 4) == (0, 1)


@pytest.mark.skipif(not (REFERENCE / "mercury").exists(), reason="reference checkout not present (MERCURY_REFERENCE)")
def test_mesh_helpers_equal_reference_functions():
    sys.path.insert(0, str(REFERENCE))
    sys.dont_write_bytecode = True
    try:
        from mercury.backend.pytorch import utils as ref
    finally:
        sys.path.pop(0)
    from mercury_artifact_b200 import mesh

    for shape in [(8,), (4, 2), (2, 2, 2)]:
        p = 1
        for n in shape:
            p *= n
        for r in range(p):
            c = ref.one_dim_to_n_dim(r, shape)
            assert mesh.one_dim_to_n_dim(r, shape) == c
            assert mesh.n_dim_to_one_dim(c, shape) == ref.n_dim_to_one_dim(c, shape)
            for d in range(len(shape)):
                for delta in (-1, 1, -shape[d]):
                    assert mesh.shift_tuple_element(c, d, delta, shape[d]) == ref.shift_tuple_element(c, d, delta, shape[d])
            dims = list(range(len(shape)))
            assert mesh.get_src_dst_ranks(c, shape, tuple(dims)) == ref.get_src_dst_ranks(c, shape, dims)


def test_get_default_args_and_namespace():
    import mercury_artifact_b200 as mb

    d = mb.get_default_args(mb._flash_attn_forward)
    assert list(d)[:6] == ["q", "k", "v", "dropout_p", "softmax_scale", "causal"]
    assert d["softcap"] == 0.0 and d["q"] is None
    ns = mb.namespace()
    assert {"_flash_attn_forward", "get_default_args", "update_out_and_lse"} <= set(ns)
    backend = mb.install_backend(force_stub=True)
    scope = {}
    exec("from mercury.backend import *", scope)
    assert scope["SendRecv"] is backend.SendRecv and scope["one_dim_to_n_dim"](5, (4, 2)) == (1, 1)


def test_cpu_tensors_are_rejected_loudly():
    import mercury_artifact_b200 as mb

    q = torch.zeros(1, 128, 1, 128, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="no CPU path"):
        mb._flash_attn_forward(q, q, q, 0.0, 1.0, False)
    with pytest.raises(ValueError, match="no CPU path"):
        mb.update_out_and_lse(None, None, q, torch.zeros(1, 1, 128))


def test_generated_programs_run_on_virtual_ranks_with_oracle_ops():
    """The virtual-rank harness itself, on CPU: reference-emitted text + oracle ops == golden."""
    import mercury_artifact_b200 as mb
    from oracle import block, merge
    from tests.helpers import golden_text, load_golden, shard_inputs
    from tests.virtual_ranks import MailboxSendRecv, run_ranks

    def fwd(q, k, v, dropout_p, softmax_scale, causal, window_size_left, window_size_right, softcap, alibi_slopes,
            return_softmax):
        o, l = block.block_attn_fwd(q, k, v, softmax_scale, causal=causal)
        return o, l, None, None

    mb.install_backend(send_recv_cls=MailboxSendRecv, force_stub=True)
    for name, fn_name in [("ring_p2", "flash_attn_pack_kv"), ("double_ring_2x2", "flash_attn_pack_split_kv")]:
        g = load_golden(name)
        ns = {"_flash_attn_forward": fwd, "get_default_args": mb.get_default_args,
              "update_out_and_lse": merge.update_out_and_lse}
        exec(golden_text(name), ns)
        qs, kvs = shard_inputs(g["t"]["q"], g["t"]["k"], g["t"]["v"], g["world"])

        def body(r):
            o = torch.zeros_like(qs[r])
            lse = torch.zeros(g["B"], g["H"], g["S"] // g["world"])
            ns[fn_name](qs[r], kvs[r], o, lse, g["D"] ** -0.5)
            return o, lse

        res = run_ranks(g["world"], body)
        for r in range(g["world"]):
            assert torch.allclose(res[r][0], g["t"][f"o_rank{r}"], atol=1e-4)
            assert torch.allclose(res[r][1], g["t"][f"lse_rank{r}"], atol=1e-4)


def test_emitter_recognises_kv_rings_and_leaves_other_programs_alone():
    from mercury_artifact_b200 import emitter
    from tests.helpers import golden_text

    d = emitter.recognise(golden_text("gpu_double_ring_4x2"))
    assert d["mesh"] == (4, 2) and d["name"] == "flash_attn_pack_split_kv" and not d["backward"]
    assert (d["batch"], d["seq_local"], d["hq"], d["hkv"], d["head_dim"]) == (1, 512, 2, 2, 128)
    d = emitter.recognise(golden_text("gpu_gqa_p2"))
    assert (d["hq"], d["hkv"], d["mesh"]) == (8, 2, (2,))
    assert emitter.recognise(golden_text("gpu_bwd_p4"))["backward"] is True
    for name in ("gpu_ring_over_q_p2", "gpu_tree_p2"):   # other schedules: untouched
        text = golden_text(name)
        assert emitter.recognise(text) is None and emitter.fuse_generated(text) == text
    fused = emitter.fuse_generated(golden_text("gpu_ring_p4"))
    assert "def flash_attn_pack_kv(q, kv, o, lse, softmax_scale, dropout_p=0, causal=False" in fused
    assert "for S_kv_ring_idx" not in fused and "RingAttention((4,), 1, 512, 4, 4, 128" in fused
    assert "ring_divide" not in fused
    compile(fused, "<fused>", "exec")
    # shift(..., ring_divide=4): the outer sub-block loop is recognised and carried into the fused call
    assert emitter.recognise(golden_text("gpu_ring_p2_div4"))["ring_divide"] == 4
    fused = emitter.fuse_generated(golden_text("gpu_ring_p2_div4"))
    assert "causal=bool(causal), ring_divide=4)" in fused and "for S_kv" not in fused
    assert "backward=True)" in emitter.fuse_generated(golden_text("gpu_bwd_p4"))
    compile(fused, "<fused>", "exec")


def test_emitter_leaves_hybrid_schedules_unfused(caplog):
    """A K/V ring along mesh dimension 0 with the heads parallelised along dimension 1 (text emitted by the
    reference's compiler for mesh (2, 2)): the ranks along dimension 1 hold other heads, not further K/V
    shards, so a RingAttention over all four ranks would be wrong.  The text must come back unchanged, and
    the log says why."""
    import logging

    from mercury_artifact_b200 import emitter
    from tests.helpers import golden_text

    text = golden_text("gpu_hybrid_ring2_heads2")
    with caplog.at_level(logging.INFO, logger="mercury_artifact_b200.emitter"):
        emitter._reported.clear()
        assert emitter.recognise(text) is None
        assert emitter.fuse_generated(text) == text
        assert emitter.fuse_generated(text) == text           # reported once, not per call
    said = [r.getMessage() for r in caplog.records]
    assert len(said) == 1 and "left as emitted" in said[0] and "hybrid" in said[0]
    # the same for a single-ring text whose mesh gains a second dimension nothing rotates along ...
    widened = golden_text("gpu_ring_p2").replace("(2,))", "(2, 2))")
    assert emitter.recognise(widened) is None and emitter.fuse_generated(widened) == widened
    # ... and for a double ring whose loops are nested the other way round (dimension 1 innermost)
    swapped = golden_text("gpu_double_ring_4x2").replace("shift_tuple_element(indices, 0,", "shift_tuple_element(indices, 9,") \
        .replace("shift_tuple_element(indices, 1,", "shift_tuple_element(indices, 0,") \
        .replace("shift_tuple_element(indices, 9,", "shift_tuple_element(indices, 1,")
    assert emitter.recognise(swapped) is None
    # a recognised program is reported as fused
    with caplog.at_level(logging.INFO, logger="mercury_artifact_b200.emitter"):
        caplog.clear()
        emitter._reported.clear()
        emitter.fuse_generated(golden_text("gpu_double_ring_4x2"))
    assert any("fused into one RingAttention.forward call over mesh (4, 2)" in r.getMessage() for r in caplog.records)


@pytest.mark.skipif(not (REFERENCE / "mercury").exists(), reason="reference checkout not present (MERCURY_REFERENCE)")
def test_search_hooks_fuse_the_program_the_reference_search_would_time():
    """install_search_hooks(): the text bench_program (mercury/search/bench.py) execs is the fused form
    for a ring schedule and the reference's own text for a schedule the emitter does not recognise."""
    import ast
    import textwrap

    sys.path.insert(0, str(REFERENCE))
    sys.dont_write_bytecode = True
    try:
        import mercury.search.bench as ref_bench
        from mercury.frontend.parser import IRBuilder
        from mercury.ir.distributed import DeviceMesh
        from mercury.ir.init_distributed import init_distributed
        from mercury.ir.loop_eliminating import eliminate_loops
        from mercury.ir.primitives import parallelize, shift
        from mercury.ir.utils import collect_axis, collect_loops
        import utils.flash_attn_dsl as dsl
    finally:
        sys.path.pop(0)
    import mercury_artifact_b200 as mb

    def program(kind):
        if kind == "ring":
            src = dsl.flash_attn_pack_kv_template.format(BATCH=1, HEADS=4, SEQ_LEN=2048, HEAD_DIM=128)
        else:
            src = dsl.flash_attn_manage_reduction.format(BATCH=1, HEADS=4, SEQ_LEN=2048, HEAD_DIM=128, RED_DIM=129)
        prog = IRBuilder().visit(ast.parse(textwrap.dedent(src)).body[0])
        axes, loops = prog.visit(collect_axis), prog.visit(collect_loops)
        dm = DeviceMesh(list(range(4)), (4,))
        init_distributed(prog, dm)
        if kind == "ring":
            parallelize(prog, loops[0], axes[2], dm, 0, 1)
            shift(prog, axes[2], dm, 0, 1, 1)
        else:
            parallelize(prog, loops[1], axes[3], dm, 0, 1)
        eliminate_loops(prog)
        return prog

    plain = ref_bench.generate_pytorch_code
    try:
        ns = mb.install_search_hooks()
        assert {"_flash_attn_forward", "update_out_and_lse", "get_default_args"} <= set(ns)
        fused = ref_bench.generate_pytorch_code(program("ring"))
        assert "_RingAttention((4,), 1, 512, 4, 4, 128" in fused and "SendRecv" not in fused
        tree_prog = program("tree")
        assert ref_bench.generate_pytorch_code(tree_prog) == plain(tree_prog)
        mb.install_search_hooks()  # idempotent
        assert ref_bench.generate_pytorch_code._mercury_b200_inner is plain
    finally:
        mb.remove_search_hooks()
    assert ref_bench.generate_pytorch_code is plain


def test_ring_divide_validation_and_memory_model():
    """Constructor checks of ring_divide and the per-rank memory model, without a process group."""
    from mercury_artifact_b200.ring import RingAttention

    class Ctx:
        world, rank, device = 8, 3, None

    op = RingAttention((8,), 1, 4096, 32, 32, 128, causal=True, ctx=Ctx(), schedule="ring")
    kv_b, q_b, lse_b = 2 * 4096 * 32 * 128 * 2, 4096 * 32 * 128 * 2, 32 * 4096 * 4
    st_b = 2 * 32 * 4096 * 4
    # balanced causal forward: one symmetric slot [kv | q], seven staging slots, the o / lse inbox
    state_b = 2 * 32 * (2048 * 130 + 8) * 4          # two half-shards: fp32 rows + (max, sum) + chain words
    assert op.memory_bytes() == {"symmetric": kv_b + q_b + 4096, "staging": 7 * (kv_b + q_b), "inbox": q_b + lse_b,
                                 "state": state_b}
    plain = RingAttention((8,), 1, 4096, 32, 32, 128, causal=False, ctx=Ctx(), schedule="ring")
    assert plain.memory_bytes() == {"symmetric": kv_b + 4096, "staging": 7 * kv_b, "inbox": 0,
                                    "state": 32 * (4096 * 130 + 16) * 4}
    both = RingAttention((8,), 1, 4096, 32, 32, 128, causal=False, ctx=Ctx(), backward=True, schedule="ring")
    # the heads schedule (the default here: 32 heads divide by 8 ranks): slot [kv | q], inbox, and one state
    # chain per rank's query rows for this rank's four heads
    heads = RingAttention((8,), 1, 4096, 32, 32, 128, causal=True, ctx=Ctx())
    assert heads.schedule == "heads" and not heads.balanced
    assert heads.memory_bytes() == {"symmetric": kv_b + q_b + 4096, "staging": 7 * (kv_b + q_b), "inbox": q_b + lse_b,
                                    "state": 8 * 4 * (4096 * 130 + 16) * 4}
    assert RingAttention((8,), 1, 4096, 4, 2, 128, causal=True, ctx=Ctx()).schedule == "ring"
    assert RingAttention((4, 2), 1, 4096, 32, 32, 128, ctx=Ctx()).schedule == "ring"
    with pytest.raises(ValueError, match="divide by the world size"):
        RingAttention((8,), 1, 4096, 4, 2, 128, ctx=Ctx(), schedule="heads")
    assert both.memory_bytes()["staging"] == 7 * (kv_b + 2 * q_b + st_b)
    with pytest.raises(ValueError, match="fixed at construction"):
        plain.memory_bytes(backward=True)
    with pytest.raises(ValueError, match="divide the local sequence"):
        RingAttention((8,), 1, 4096, 32, 32, 128, ctx=Ctx(), ring_divide=3)
    with pytest.raises(ValueError, match="segments exceed"):
        RingAttention((8,), 1, 4096, 32, 32, 128, ctx=Ctx(), ring_divide=8)
    # eight ranks x four pieces = 29 segments fit one launch, also with the balanced causal forward
    assert RingAttention((8,), 1, 4096, 32, 32, 128, causal=True, ctx=Ctx(), ring_divide=4).balanced   # pieces: ring
    with pytest.raises(ValueError, match="multiples of 64 rows"):
        RingAttention((2,), 1, 960, 4, 4, 128, ctx=type("C2", (), dict(world=2, rank=0, device=None))(),
                      ring_divide=2, backward=True)
    Ctx.world, Ctx.rank = 2, 1
    assert RingAttention((2,), 1, 4096, 32, 32, 128, causal=True, ctx=Ctx(), balance_causal=False,
                         ring_divide=7 if 4096 % 7 == 0 else 4).ring_divide == 4
    assert RingAttention((1,), 1, 4096, 32, 32, 128).memory_bytes() == {"symmetric": 0, "staging": 0, "inbox": 0, "state": 0}
