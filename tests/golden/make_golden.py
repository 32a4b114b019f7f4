"""Generate the golden fixtures of tests/golden/ from the UNMODIFIED reference.

Run where the reference checkout is available (it is not needed afterwards):

    python tests/golden/make_golden.py /path/to/mercury_artifact [case ...]

(the path may also come from MERCURY_REFERENCE; default: a directory "reference" beside this repository)

For each schedule the reference's own compiler (frontend parser -> IR passes ->
mercury.backend.generate_pytorch_code) emits the per-rank program, which is then
executed on CPU under torch.distributed/gloo with the reference's own
update_out_and_lse and SendRecv.  Only the CUDA-only flash-attn block op is
replaced, by name, with the fp32 CPU block of oracle/block.py (the block math is
third-party and not part of the reference tree).  Stored per case:

  <case>.npz     seeded inputs (full tensors) and per-rank outputs, fp32
  <case>.gen.txt the program text the reference emitted (exec'd by the GPU tests
                 against this package's drop-in ops; the GPU box has no reference)

The backward program allocates its temporaries on `cuda:{LOCAL_RANK}`
(codegen.py:207-210); for the CPU run that one expression is rewritten to "cpu".
"""
from __future__ import annotations

import ast
import os
import sys
import textwrap
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent
sys.path.insert(0, str(REPO))


def _imports(ref_root: str):
    sys.path.insert(0, ref_root)
    os.environ.setdefault("PYTHONDONTWRITEBYTECODE", "1")
    sys.dont_write_bytecode = True


def generate(ref_root: str, kind: str, world: int, B: int, S: int, H: int, D: int, hkv: int = 0, mesh=None,
             ring_divide: int = 1) -> str:
    """Emit the per-rank program for one schedule with the reference compiler."""
    _imports(ref_root)
    from mercury.backend import generate_pytorch_code
    from mercury.frontend.parser import IRBuilder
    from mercury.ir.distributed import DeviceMesh
    from mercury.ir.init_distributed import init_distributed
    from mercury.ir.loop_eliminating import eliminate_loops
    from mercury.ir.primitives import parallelize, shift
    from mercury.ir.utils import collect_axis, collect_loops
    import utils.flash_attn_dsl as dsl
    from utils.attn_bwd_dsl import attn_backward_template

    if kind in ("ring", "hybrid"):
        src = dsl.flash_attn_pack_kv_template.format(BATCH=B, HEADS=H, SEQ_LEN=S, HEAD_DIM=D)
    elif kind == "gqa":
        src = dsl.gqa_pack_kv_template.format(BATCH=B, HEADS=H, SEQ_LEN=S, HEAD_DIM=D, KV_HEADS=hkv,
                                              HEADS_PER_GROUP=H // hkv)
    elif kind == "double_ring":
        src = dsl.flash_attn_pack_kv_double_ring_template.format(
            BATCH=B, HEADS=H, SEQ_LEN=S, HEAD_DIM=D, SEQ_LEN_IN=S // mesh[1], SEQ_LEN_OUT=mesh[1])
    elif kind == "bwd":
        src = attn_backward_template.format(BATCH=B, HEADS=H, SEQ_LEN=S, HEAD_DIM=D)
    elif kind in ("ring_over_q", "tree"):
        src = dsl.flash_attn_manage_reduction.format(BATCH=B, HEADS=H, SEQ_LEN=S, HEAD_DIM=D, RED_DIM=D + 1)
    else:
        raise ValueError(kind)
    prog = IRBuilder().visit(ast.parse(textwrap.dedent(src)).body[0])
    axes = prog.visit(collect_axis)
    loops = prog.visit(collect_loops)
    shape = tuple(mesh) if mesh else (world,)
    dm = DeviceMesh(list(range(world)), shape)
    init_distributed(prog, dm)
    if world > 1 and kind == "tree":
        # K/V sharded, queries replicated: partial results merged by the all-reduce collective
        parallelize(prog, loops[1], axes[3], dm, 0, len(shape))
    elif kind == "hybrid":
        # mesh (ring, heads): K/V ring over the sequence along mesh dimension 0 only, the heads split
        # along mesh dimension 1 without communication (the shape of tests/test_attn_bwd.py:402-404)
        parallelize(prog, loops[0], axes[2], dm, 0, 1)
        shift(prog, axes[2], dm, 0, 1, 1)
        parallelize(prog, loops[0], axes[1], dm, 1, 2)
    elif world > 1 and kind == "ring_over_q":
        # K/V sharded and stationary; the queries and the packed reduce buffer rotate
        parallelize(prog, loops[1], axes[3], dm, 0, len(shape))
        shift(prog, axes[3], dm, 0, len(shape), 1)
    elif world > 1:
        outer = loops[1] if kind == "bwd" else loops[0]
        parallelize(prog, outer, axes[2], dm, 0, len(shape))
        shift(prog, axes[2], dm, 0, len(shape), ring_divide)
    eliminate_loops(prog)
    return generate_pytorch_code(prog)


def make_inputs(seed: int, B: int, S: int, H: int, hkv: int, D: int, scale: float = 1.0):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, S, H, D, generator=g) * scale
    k = torch.randn(B, S, hkv, D, generator=g) * scale
    v = torch.randn(B, S, hkv, D, generator=g) * scale
    do = torch.randn(B, S, H, D, generator=g) * scale
    return q, k, v, do


def _worker(rank, world, ref_root, code, fn_name, kind, dims, seed, port, ret):
    _imports(ref_root)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    import utils.flash_attn_dsl as dsl
    from oracle import block as ob

    B, S, H, hkv, D = dims
    scale = D ** -0.5

    def _flash_attn_forward(q, k, v, dropout_p, softmax_scale, causal, window_size_left, window_size_right, softcap,
                            alibi_slopes, return_softmax):
        out, lse = ob.block_attn_fwd(q, k, v, softmax_scale, causal=causal)
        return out, lse, None, None

    def _flash_attn_backward(dout, q, k, v, out, softmax_lse, dq, dk, dv, dropout_p, softmax_scale, causal,
                             window_size_left, window_size_right, softcap, alibi_slopes, deterministic,
                             rng_state=None):
        gq, gk, gv = ob.block_attn_bwd(dout, q, k, v, out, softmax_lse, softmax_scale, causal=causal)
        dq.copy_(gq)
        dk.copy_(gk)
        dv.copy_(gv)
        return None

    ns = {
        "get_default_args": dsl.get_default_args,
        "update_out_and_lse": dsl.update_out_and_lse,
        "_flash_attn_forward": _flash_attn_forward,
        "_flash_attn_backward": _flash_attn_backward,
        "flash_reduce": dsl.flash_reduce,
        "update_out_and_lse_collective": dsl.update_out_and_lse_collective,
    }
    if kind in ("bwd", "ring_over_q", "tree"):
        code = code.replace('torch.device(f"cuda:{local_rank}")', 'torch.device("cpu")')
    exec(code, ns)
    fn = ns[fn_name]
    q, k, v, do = make_inputs(seed, B, S, H, hkv, D)
    lq = q.contiguous() if kind == "tree" else q.chunk(world, 1)[rank].contiguous()
    lkv = torch.stack([k.chunk(world, 1)[rank], v.chunk(world, 1)[rank]]).contiguous()
    if kind == "bwd":
        fo, fl = ob.full_attention(q, k, v, scale)
        lo = fo.chunk(world, 1)[rank].contiguous()
        ll = fl.chunk(world, 2)[rank].contiguous()
        ldo = do.chunk(world, 1)[rank].contiguous()
        dq = torch.zeros_like(lq)
        dkv = torch.zeros_like(lkv)
        fn(lq, lkv, lo, ll, ldo, dq, dkv, scale)
        ret[rank] = dict(dq=dq.numpy(), dkv=dkv.numpy())
    else:
        o = torch.zeros_like(lq)
        lse = torch.zeros(B, H, lq.shape[1])
        fn(lq, lkv, o, lse, scale)
        ret[rank] = dict(o=o.numpy(), lse=lse.numpy())
    dist.barrier()
    dist.destroy_process_group()


CASES = [
    # name, kind, fn_name, world, mesh, (B, S, H, hkv, D), seed
    ("ring_p1", "ring", "flash_attn_pack_kv", 1, None, (1, 128, 2, 2, 32), 11),
    ("ring_p2", "ring", "flash_attn_pack_kv", 2, None, (1, 256, 2, 2, 32), 12),
    ("ring_p4", "ring", "flash_attn_pack_kv", 4, None, (2, 256, 2, 2, 32), 13),
    ("gqa_p2", "gqa", "gqa_pack_kv", 2, None, (1, 256, 4, 2, 32), 14),
    ("double_ring_2x2", "double_ring", "flash_attn_pack_split_kv", 4, (2, 2), (1, 256, 2, 2, 32), 15),
    ("bwd_p2", "bwd", "flash_attn_backward", 2, None, (1, 256, 2, 2, 32), 16),
    ("bwd_p4", "bwd", "flash_attn_backward", 4, None, (1, 256, 2, 2, 32), 17),
    ("ring_over_q_p2", "ring_over_q", "flash_attn_expose_reduce", 2, None, (1, 256, 2, 2, 32), 18),
    ("ring_over_q_p4", "ring_over_q", "flash_attn_expose_reduce", 4, None, (1, 256, 2, 2, 32), 19),
    ("tree_p2", "tree", "flash_attn_expose_reduce", 2, None, (1, 256, 2, 2, 32), 20),
    ("tree_p4", "tree", "flash_attn_expose_reduce", 4, None, (1, 256, 2, 2, 32), 21),
]

# Program text only (no vectors): the shapes the GPU tests run through the drop-in ops.
TEXT_ONLY = [
    ("gpu_ring_p1", "ring", 1, None, (1, 512, 4, 4, 128)),
    ("gpu_ring_p2", "ring", 2, None, (1, 1024, 4, 4, 128)),
    ("gpu_ring_p4", "ring", 4, None, (1, 2048, 4, 4, 128)),
    ("gpu_gqa_p2", "gqa", 2, None, (2, 1024, 8, 2, 128)),
    ("gpu_double_ring_2x2", "double_ring", 4, (2, 2), (1, 2048, 4, 4, 128)),
    ("gpu_double_ring_4x2", "double_ring", 8, (4, 2), (1, 4096, 2, 2, 128)),
    ("gpu_bwd_p2", "bwd", 2, None, (1, 1024, 4, 4, 128)),
    ("gpu_bwd_p4", "bwd", 4, None, (1, 2048, 4, 4, 128)),
    ("gpu_ring_over_q_p2", "ring_over_q", 2, None, (1, 1024, 4, 4, 128)),
    ("gpu_ring_over_q_p4", "ring_over_q", 4, None, (2, 1024, 4, 4, 128)),
    ("gpu_tree_p2", "tree", 2, None, (1, 1024, 4, 4, 128)),
    # ring_divide = 2 and 4: the shift primitive halves / quarters the K/V block of a ring round
    ("gpu_ring_p2_div2", "ring", 2, None, (1, 1024, 4, 4, 128), 2),
    ("gpu_ring_p2_div4", "ring", 2, None, (1, 1024, 4, 4, 128), 4),
    # a hybrid schedule: ring over mesh dimension 0, heads parallelised over dimension 1 (must NOT be fused)
    ("gpu_hybrid_ring2_heads2", "hybrid", 4, (2, 2), (1, 1024, 4, 4, 128)),
    # bench.py: the reference's shipped path (flash-attn block + merge + NCCL messages) and this package's
    # per-step drop-ins run these texts at the headline shape (bf16 B1 S32768 H32 D128) on 1/2/4/8 ranks ...
    ("bench_ring_p1", "ring", 1, None, (1, 32768, 32, 32, 128)),
    ("bench_ring_p2", "ring", 2, None, (1, 32768, 32, 32, 128)),
    ("bench_ring_p4", "ring", 4, None, (1, 32768, 32, 32, 128)),
    ("bench_ring_p8", "ring", 8, None, (1, 32768, 32, 32, 128)),
    # ... and its CPU arm runs them as gloo ranks on a shortened sequence (same batch, heads, head_dim)
    ("cpu_ring_p1", "ring", 1, None, (1, 4096, 32, 32, 128)),
    ("cpu_ring_p2", "ring", 2, None, (1, 4096, 32, 32, 128)),
    ("cpu_ring_p4", "ring", 4, None, (1, 4096, 32, 32, 128)),
    ("cpu_ring_p8", "ring", 8, None, (1, 4096, 32, 32, 128)),
]


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("MERCURY_REFERENCE", str(REPO.parent / "reference"))
    only = set(sys.argv[2:])  # optional: regenerate just the named cases
    port = 29611
    for name, kind, fn_name, world, mesh, dims, seed in CASES:
        if only and name not in only:
            continue
        B, S, H, hkv, D = dims
        code = generate(ref_root, kind, world, B, S, H, D, hkv=hkv, mesh=mesh)
        (HERE / f"{name}.gen.txt").write_text(code)
        mgr = mp.Manager()
        ret = mgr.dict()
        port += 1
        mp.spawn(_worker, args=(world, ref_root, code, fn_name, kind, dims, seed, port, ret), nprocs=world, join=True)
        q, k, v, do = make_inputs(seed, B, S, H, hkv, D)
        arrays = dict(q=q.numpy(), k=k.numpy(), v=v.numpy(), dout=do.numpy(),
                      meta=np.array([world, B, S, H, hkv, D, seed] + list(mesh or (world,)), dtype=np.int64))
        for r in range(world):
            for key, val in ret[r].items():
                arrays[f"{key}_rank{r}"] = val
        np.savez_compressed(HERE / f"{name}.npz", **arrays)
        print("wrote", name, {k: v.shape for k, v in arrays.items() if k != "meta"})
    for name, kind, world, mesh, dims, *rest in TEXT_ONLY:
        if only and name not in only:
            continue
        B, S, H, hkv, D = dims
        code = generate(ref_root, kind, world, B, S, H, D, hkv=hkv, mesh=mesh, ring_divide=rest[0] if rest else 1)
        (HERE / f"{name}.gen.txt").write_text(code)
        print("wrote", name)


if __name__ == "__main__":
    main()
