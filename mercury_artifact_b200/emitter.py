"""Rewrite a program emitted by mercury.backend.generate_pytorch_code into one fused call.

The reference emits a per-rank step loop (post the next transfer, block attention,
merge; mercury/backend/pytorch/codegen.py:264-355, 397-494).  `fuse_generated` recognises the
ring-attention idiom in that text -- forward ring, GQA ring, double ring, and the backward
ring -- reads the shapes from the emitted asserts and the mesh from the emitted
`one_dim_to_n_dim(dist.get_rank(), (...))`, and returns the source of a function with the SAME
name and signature whose body is a single RingAttention.forward / .backward call.  Programs it
does not recognise are returned unchanged and run on the per-step drop-ins:

    code = generate_pytorch_code(program)
    exec(fuse_generated(code), mb.namespace())

A program is only fused when EVERY mesh dimension (of size > 1) is a dimension along which the K/V
buffer rotates, nested the way RingAttention walks them (mesh dimension 0 innermost).  The
reference also emits hybrid schedules -- a K/V ring along one mesh dimension with heads, batch or
queries parallelised along another (tests/test_gqa.py, tests/test_split.py:220-224,
tests/test_attn_bwd.py:402-403 of the reference) -- in which the ranks along the other dimension
hold different heads or batches, not further K/V shards; those are left as they are.  The logger
"mercury_artifact_b200.emitter" says once per program which way it went, and why.

Semantics differ from the step loop in one documented way: with causal=True the reference hands
the flag unchanged to every block (only meaningful for causal=False); the fused call applies the
causal rule on global positions.
"""
from __future__ import annotations

import ast
import logging
import re
from typing import Dict, List, Optional, Tuple

_log = logging.getLogger(__name__)
_reported = set()

_SHAPE_RE = re.compile(r"assert (\w+)\.shape == \(([^)]*)\)")
_MESH_RE = re.compile(r"one_dim_to_n_dim\(dist\.get_rank\(\), \(([^)]*)\)\)")
# shift(..., ring_divide=d) makes the reference emit an outer loop over K/V sub-blocks around the ring loop
_DIVIDE_RE = re.compile(r"for S_kv in range\(0, (\d+), (\d+)\):\s*\n\s*for S_kv_ring_idx in range")


def _shapes(code: str) -> Dict[str, Tuple[int, ...]]:
    out = {}
    for name, dims in _SHAPE_RE.findall(code):
        out[name] = tuple(int(x) for x in dims.replace(" ", "").split(",") if x)
    return out


def _is_call(node, name: str) -> bool:
    return isinstance(node, ast.Call) and isinstance(node.func, ast.Name) and node.func.id == name


def _kv_ring_dims(fn: ast.FunctionDef) -> Optional[Dict[int, Tuple[int, str]]]:
    """{mesh dim: (ring size, ring-index variable)} of the K/V rotation, read from the emitted
    `if <idx> + 1 != n: ... shift_tuple_element(indices, d, +-1, n) ... ring_comm_kv.send_recv(...)`
    branches (codegen.py:471-491).  None if a branch does not have that form."""
    dims: Dict[int, Tuple[int, str]] = {}
    for node in ast.walk(fn):
        if not isinstance(node, ast.If):
            continue
        sends_kv = any(isinstance(c, ast.Call) and isinstance(c.func, ast.Attribute) and c.func.attr == "send_recv"
                       and isinstance(c.func.value, ast.Name) and c.func.value.id == "ring_comm_kv"
                       for st in node.body for c in ast.walk(st))
        if not sends_kv:
            continue
        t = node.test
        if not (isinstance(t, ast.Compare) and len(t.ops) == 1 and isinstance(t.ops[0], ast.NotEq)
                and isinstance(t.left, ast.BinOp) and isinstance(t.left.op, ast.Add)
                and isinstance(t.left.left, ast.Name) and isinstance(t.comparators[0], ast.Constant)):
            return None
        idx, size = t.left.left.id, int(t.comparators[0].value)
        shifts = [c for st in node.body for c in ast.walk(st) if _is_call(c, "shift_tuple_element")]
        if not shifts:
            return None
        for c in shifts:
            if len(c.args) != 4 or not all(isinstance(a, (ast.Constant, ast.UnaryOp)) for a in c.args[1:]):
                return None
            d, n = int(ast.literal_eval(c.args[1])), int(ast.literal_eval(c.args[3]))
            if n != size or dims.get(d, (n, idx)) != (n, idx):
                return None
            dims[d] = (n, idx)
    return dims


def _ring_loops(fn: ast.FunctionDef) -> List[Tuple[str, int]]:
    """(variable, trip count) of the `for <x>_ring_idx in range(n)` loops, outermost first."""
    out: List[Tuple[str, int]] = []

    def visit(stmts):
        for st in stmts:
            if isinstance(st, ast.For):
                if (isinstance(st.target, ast.Name) and st.target.id.endswith("_ring_idx") and _is_call(st.iter, "range")
                        and len(st.iter.args) == 1 and isinstance(st.iter.args[0], ast.Constant)):
                    out.append((st.target.id, int(st.iter.args[0].value)))
                visit(st.body)
            elif isinstance(st, (ast.If, ast.With)):
                visit(st.body)
                visit(getattr(st, "orelse", []))

    visit(fn.body)
    return out


def analyse(code: str) -> Tuple[Optional[dict], str]:
    """(description, "") if the program is a K/V ring over the whole mesh, else (None, reason)."""
    try:
        tree = ast.parse(code)
    except SyntaxError:
        return None, "not parseable"
    fns = [n for n in tree.body if isinstance(n, ast.FunctionDef)]
    if len(fns) != 1:
        return None, "not exactly one function"
    fn = fns[0]
    args = [a.arg for a in fn.args.args]
    shapes = _shapes(code)
    mesh_m = _MESH_RE.search(code)
    if mesh_m is None or "q" not in shapes or "kv" not in shapes:
        return None, "no mesh line or no q/kv shape asserts"
    mesh = tuple(int(x) for x in mesh_m.group(1).replace(" ", "").split(",") if x)
    world = 1
    for n in mesh:
        world *= n
    q, kv = shapes["q"], shapes["kv"]
    if len(q) != 4 or len(kv) != 5 or kv[0] != 2 or kv[1] != q[0] or kv[4] != q[3]:
        return None, "q/kv are not [B,S,H,D] / [2,B,S,Hkv,D] of one batch and head_dim"
    # K/V must be the rotating buffer (or nothing rotates at world size 1) and the queries stationary
    rotates_kv = "ring_comm_kv" in code
    rotates_q = "ring_comm_q" in code
    if rotates_q or (world > 1 and not rotates_kv) or q[1] != kv[2]:
        return None, "not a K/V ring with stationary queries"
    if "update_out_and_lse_collective" in code or "flash_reduce" in code:
        return None, "uses a reduce collective or a rotating reduce buffer"
    backward = "_flash_attn_backward(" in code
    forward = "_flash_attn_forward(" in code and "update_out_and_lse(" in code
    if backward == forward:
        return None, "neither the forward nor the backward idiom"
    want = ["q", "kv", "o", "lse", "dout", "dq", "dkv", "softmax_scale"] if backward else ["q", "kv", "o", "lse", "softmax_scale"]
    if args[:len(want)] != want:
        return None, "unexpected argument list"
    # Every mesh dimension of size > 1 must carry the K/V rotation, with dimension 0 the innermost
    # ring loop, dimension 1 the next one out, and so on: only then are the ranks of the mesh the
    # shards of one sequence, in RingAttention's order.
    ring_dims = _kv_ring_dims(fn)
    if ring_dims is None:
        return None, "a K/V send branch does not have the emitted `if idx + 1 != n` form"
    loops = [lp for lp in _ring_loops(fn)]
    inner_first = list(reversed(loops))
    real_dims = [d for d, n in enumerate(mesh) if n > 1]
    if sorted(ring_dims) != real_dims:
        return None, (f"K/V rotates along mesh dimension(s) {sorted(ring_dims)} of mesh {mesh}: the other "
                      "dimensions hold different heads, batches or replicas (hybrid schedule)")
    ring_loops = [lp for lp in inner_first if lp[1] > 1 or len(inner_first) == len(real_dims)]
    if len(ring_loops) < len(real_dims):
        return None, "fewer ring loops than ring dimensions"
    for pos, d in enumerate(real_dims):
        n, idx = ring_dims[d]
        if n != mesh[d] or ring_loops[pos] != (idx, n):
            return None, f"ring loop nesting does not put mesh dimension {d} at depth {pos} from the inside"
    ring_divide = 1
    dm = _DIVIDE_RE.search(code)
    if dm is not None and not backward:
        total, step = int(dm.group(1)), int(dm.group(2))
        if total == kv[2] and step > 0 and total % step == 0:
            ring_divide = total // step
    return dict(name=fn.name, args=args, defaults=fn.args.defaults, mesh=mesh, batch=q[0], seq_local=q[1], hq=q[2],
                ring_divide=ring_divide,
                hkv=kv[3], head_dim=q[3], backward=backward, signature=ast.get_source_segment(code, fn.args)), ""


def recognise(code: str) -> Optional[dict]:
    """Describe the program if it is a K/V ring over the whole mesh (forward or backward), else None."""
    return analyse(code)[0]


def _report(key: str, message: str) -> None:
    if key not in _reported:
        _reported.add(key)
        _log.info(message)


def fuse_generated(code: str) -> str:
    """Source of the fused equivalent of `code`, or `code` itself if the idiom is not recognised."""
    d, why = analyse(code)
    if d is None:
        m = re.search(r"def (\w+)\(", code)
        name = m.group(1) if m else "<program>"
        _report(f"{name}:{why}", f"{name}: left as emitted (per-step drop-ins): {why}")
        return code
    _report(f"{d['name']}:{d['mesh']}:{d['backward']}",
            f"{d['name']}: fused into one RingAttention.{'backward' if d['backward'] else 'forward'} call over mesh {d['mesh']}")
    tree = ast.parse(code)
    fn = [n for n in tree.body if isinstance(n, ast.FunctionDef)][0]
    header = f"def {fn.name}({ast.unparse(fn.args)}):"
    key = (d["mesh"], d["batch"], d["seq_local"], d["hq"], d["hkv"], d["head_dim"])
    world = 1
    for n in d["mesh"]:
        world *= n
    # the program's ring_divide carries over when its pieces fit the 32 segments of one launch
    rd = d.get("ring_divide", 1)
    divide = f", ring_divide={rd}" if rd > 1 and 1 + (world - 1) * rd <= 32 else ""
    if d["backward"]:
        divide += ", backward=True"
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
