"""Wiring the drop-in ops into the reference's code generator output.

The generated program finds its ops in two ways (reference: example.py:153-156,
mercury/backend/pytorch/codegen.py:219):
  * free names looked up in the namespace given to exec():
    _flash_attn_forward, _flash_attn_backward, get_default_args, update_out_and_lse
  * `from mercury.backend import *` executed by the generated text itself:
    SendRecv and the mesh index helpers.

`namespace()` serves the first, `install_backend()` the second.  `install_search_hooks()` makes the
reference's schedule search time these ops: its bench_program(program, namespace, ...) takes the exec
namespace as an argument (mercury/search/bench.py:15-45) and emits the text through the module-level name
generate_pytorch_code, which the hook wraps so that a recognised ring loop is replaced by its fused
one-launch form before it is executed.
"""
from __future__ import annotations

import sys
import types
from typing import Dict

from . import mesh, ops


def _collective(tensor, op, group, dst=None):
    from .collective import update_out_and_lse_collective

    return update_out_and_lse_collective(tensor, op, group, dst)


def namespace(extra: Dict[str, object] | None = None) -> Dict[str, object]:
    """Globals for exec(generated_code, ns): every free name the DSL bodies use."""
    ns: Dict[str, object] = {
        "_flash_attn_forward": ops._flash_attn_forward,
        "get_default_args": ops.get_default_args,
        "update_out_and_lse": ops.update_out_and_lse,
        "flash_reduce": ops.flash_reduce,
        "update_out_and_lse_collective": _collective,
    }
    if hasattr(ops, "_flash_attn_backward"):
        ns["_flash_attn_backward"] = ops._flash_attn_backward
    if extra:
        ns.update(extra)
    return ns


_RUNTIME_NAMES = ("one_dim_to_n_dim", "n_dim_to_one_dim", "shift_tuple_element", "get_src_dst_ranks",
                  "get_device_group")


def install_backend(send_recv_cls=None, force_stub: bool = False) -> types.ModuleType:
    """Make `from mercury.backend import *` hand out this package's SendRecv.

    With the reference importable, only SendRecv is replaced (on mercury.backend,
    mercury.backend.pytorch and mercury.backend.pytorch.utils) and everything else is the
    reference's own.  Without it, a stand-in `mercury.backend` module is registered that
    exports SendRecv and the mesh index helpers, which is all the generated text imports.
    """
    if send_recv_cls is None:
        from .comm import SendRecv as send_recv_cls  # noqa: N813
    if not force_stub:
        try:
            import mercury.backend as mb_backend  # type: ignore
            import mercury.backend.pytorch as mb_pt  # type: ignore
            import mercury.backend.pytorch.utils as mb_utils  # type: ignore

            if not getattr(mb_backend, "__mercury_b200_stub__", False):
                for mod in (mb_backend, mb_pt, mb_utils):
                    setattr(mod, "SendRecv", send_recv_cls)
                return mb_backend
        except ImportError:
            pass
    pkg = sys.modules.get("mercury")
    if pkg is None or not getattr(pkg, "__mercury_b200_stub__", False):
        pkg = types.ModuleType("mercury")
        pkg.__path__ = []  # type: ignore[attr-defined]
        pkg.__mercury_b200_stub__ = True  # type: ignore[attr-defined]
        sys.modules["mercury"] = pkg
    backend = types.ModuleType("mercury.backend")
    backend.__mercury_b200_stub__ = True  # type: ignore[attr-defined]
    backend.SendRecv = send_recv_cls  # type: ignore[attr-defined]
    for name in _RUNTIME_NAMES:
        setattr(backend, name, getattr(mesh, name))
    backend.__all__ = ["SendRecv", *_RUNTIME_NAMES]  # type: ignore[attr-defined]
    sys.modules["mercury.backend"] = backend
    pkg.backend = backend  # type: ignore[attr-defined]
    return backend


def load_generated(code: str, extra: Dict[str, object] | None = None) -> Dict[str, object]:
    """exec() a program emitted by mercury.backend.generate_pytorch_code with the drop-in ops."""
    ns = namespace(extra)
    exec(compile(code, "<mercury generated>", "exec"), ns)
    return ns


def install_search_hooks(fuse: bool = True) -> Dict[str, object]:
    """Prepare the reference's schedule search (mercury/search/bench.py: bench_program) for these ops.

    Installs the SendRecv backend, and with fuse=True wraps the name `generate_pytorch_code` that
    bench_program calls so that the emitted text goes through emitter.fuse_generated (a program whose
    idiom is not recognised is returned unchanged and runs on the per-step drop-ins).  Returns the
    namespace to pass as bench_program's second argument.  Needs the reference importable."""
    install_backend()
    import mercury.search.bench as ref_bench  # type: ignore

    if fuse and not getattr(ref_bench.generate_pytorch_code, "_mercury_b200_fusing", False):
        from .emitter import fuse_generated

        inner = ref_bench.generate_pytorch_code

        def generate_pytorch_code(program):
            return fuse_generated(inner(program))

        generate_pytorch_code._mercury_b200_fusing = True  # type: ignore[attr-defined]
        generate_pytorch_code._mercury_b200_inner = inner  # type: ignore[attr-defined]
        ref_bench.generate_pytorch_code = generate_pytorch_code
    return namespace()


def remove_search_hooks() -> None:
    """Undo install_search_hooks(fuse=True)."""
    mod = sys.modules.get("mercury.search.bench")
    fn = getattr(mod, "generate_pytorch_code", None) if mod is not None else None
    if fn is not None and getattr(fn, "_mercury_b200_fusing", False):
        mod.generate_pytorch_code = fn._mercury_b200_inner
