"""Rewrite a program emitted by mercury.backend.generate_pytorch_code into one fused call.

The reference emits a per-rank step loop (post the next transfer, block attention,
merge; mercury/backend/pytorch/codegen.py:264-355, 397-494).  `fuse_generated` recognises the
ring-attention idiom in that text -- forward ring, GQA ring, double ring, and the backward
ring -- reads the shapes from the emitted asserts and the mesh from the emitted
`one_dim_to_n_dim(dist.get_rank(), (...))`, and returns the source of a function with the SAME
name and signature whose body is a single RingAttention.forward / .backward call.  Programs it
does not recognise are returned unchanged, so it is always safe to apply:

    code = generate_pytorch_code(program)
    exec(fuse_generated(code), mb.namespace())

Semantics differ from the step loop in one documented way: with causal=True the reference hands
the flag unchanged to every block (only meaningful for causal=False); the fused call applies the
causal rule on global positions.
"""
from __future__ import annotations

import ast
import re
from typing import Dict, Optional, Tuple

_SHAPE_RE = re.compile(r"assert (\w+)\.shape == \(([^)]*)\)")
_MESH_RE = re.compile(r"one_dim_to_n_dim\(dist\.get_rank\(\), \(([^)]*)\)\)")
# shift(..., ring_divide=d) makes the reference emit an outer loop over K/V sub-blocks around the ring loop
_DIVIDE_RE = re.compile(r"for S_kv in range\(0, (\d+), (\d+)\):\s*\n\s*for S_kv_ring_idx in range")


def _shapes(code: str) -> Dict[str, Tuple[int, ...]]:
    out = {}
    for name, dims in _SHAPE_RE.findall(code):
        out[name] = tuple(int(x) for x in dims.replace(" ", "").split(",") if x)
    return out


def recognise(code: str) -> Optional[dict]:
    """Describe the program if it is a K/V ring (forward or backward), else None."""
    try:
        tree = ast.parse(code)
    except SyntaxError:
        return None
    fns = [n for n in tree.body if isinstance(n, ast.FunctionDef)]
    if len(fns) != 1:
        return None
    fn = fns[0]
    args = [a.arg for a in fn.args.args]
    shapes = _shapes(code)
    mesh_m = _MESH_RE.search(code)
    if mesh_m is None or "q" not in shapes or "kv" not in shapes:
        return None
    mesh = tuple(int(x) for x in mesh_m.group(1).replace(" ", "").split(",") if x)
    world = 1
    for n in mesh:
        world *= n
    q, kv = shapes["q"], shapes["kv"]
    if len(q) != 4 or len(kv) != 5 or kv[0] != 2 or kv[1] != q[0] or kv[4] != q[3]:
        return None
    # K/V must be the rotating buffer (or nothing rotates at world size 1) and the queries stationary
    rotates_kv = "ring_comm_kv" in code
    rotates_q = "ring_comm_q" in code
    if rotates_q or (world > 1 and not rotates_kv) or q[1] != kv[2]:
        return None
    if "update_out_and_lse_collective" in code or "flash_reduce" in code:
        return None
    backward = "_flash_attn_backward(" in code
    forward = "_flash_attn_forward(" in code and "update_out_and_lse(" in code
    if backward == forward:
        return None
    want = ["q", "kv", "o", "lse", "dout", "dq", "dkv", "softmax_scale"] if backward else ["q", "kv", "o", "lse", "softmax_scale"]
    if args[:len(want)] != want:
        return None
    ring_divide = 1
    dm = _DIVIDE_RE.search(code)
    if dm is not None and not backward:
        total, step = int(dm.group(1)), int(dm.group(2))
        if total == kv[2] and step > 0 and total % step == 0:
            ring_divide = total // step
    return dict(name=fn.name, args=args, defaults=fn.args.defaults, mesh=mesh, batch=q[0], seq_local=q[1], hq=q[2],
                ring_divide=ring_divide,
                hkv=kv[3], head_dim=q[3], backward=backward, signature=ast.get_source_segment(code, fn.args))


def fuse_generated(code: str) -> str:
    """Source of the fused equivalent of `code`, or `code` itself if the idiom is not recognised."""
    d = recognise(code)
    if d is None:
        return code
    tree = ast.parse(code)
    fn = [n for n in tree.body if isinstance(n, ast.FunctionDef)][0]
    header = f"def {fn.name}({ast.unparse(fn.args)}):"
    key = (d["mesh"], d["batch"], d["seq_local"], d["hq"], d["hkv"], d["head_dim"])
    world = 1
    for n in d["mesh"]:
        world *= n
    # the program's ring_divide carries over when its pieces fit the eight segments of one launch
    rd = d.get("ring_divide", 1)
    divide = f", ring_divide={rd}, balance_causal=False" if rd > 1 and 1 + (world - 1) * rd <= 8 else ""
    lines = [
        "import torch",
        "from mercury_artifact_b200.ring import RingAttention as _RingAttention",
        "",
        "_fused_ops = {}",
        "",
        header,
        f"    assert q.shape == {tuple(key[1:2] + key[2:4] + key[5:6])!r}, 'Shape mismatch for q'",
        f"    assert kv.shape == {(2, key[1], key[2], key[4], key[5])!r}, 'Shape mismatch for kv'",
        "    if dropout_p or tuple(window_size) != (-1, -1) or alibi_slopes is not None:",
        "        raise NotImplementedError('dropout, sliding window and alibi are not implemented')",
        "    op = _fused_ops.get(bool(causal))",
        "    if op is None:",
        f"        op = _fused_ops[bool(causal)] = _RingAttention({d['mesh']!r}, {d['batch']}, {d['seq_local']}, "
        f"{d['hq']}, {d['hkv']}, {d['head_dim']}, causal=bool(causal){divide})",
    ]
    if d["backward"]:
        lines.append("    op.backward(dout, q, kv, o, lse, dq, dkv, softmax_scale)")
    else:
        lines.append("    op.forward(q, kv, o, lse, softmax_scale)")
    return "\n".join(lines) + "\n"
