"""Runtime for executing a program emitted by the reference's code generator the way the
reference itself runs it -- torch.distributed point-to-point messages and the running out/LSE
merge -- without the reference checkout (test and baseline infrastructure, never product).

Restates mercury/backend/pytorch/utils.py:9-39 (SendRecv: one isend + one irecv batched with
batch_isend_irecv, waited request by request), the index helpers :41-106 and :171-192 that the
emitted text imports with `from mercury.backend import *` (codegen.py:219), and get_default_args
of utils/flash_attn_dsl.py:14-29.  The merge comes from oracle/merge.py.  The block op is supplied
by the caller: the flash-attn op for the GPU baseline (NCCL), oracle/block.py for CPU/gloo ranks.
"""
from __future__ import annotations

import inspect
import sys
import types
from typing import Callable, Dict, Optional

import torch

from . import merge as _merge
from . import ring as _ring


class SendRecv:
    """mercury/backend/pytorch/utils.py:9-39."""

    def __init__(self):
        self._ops = []
        self._reqs = None

    def send_recv(self, to_rank: int, from_rank: int, send_tensor: torch.Tensor,
                  recv_tensor: Optional[torch.Tensor] = None) -> torch.Tensor:
        import torch.distributed as dist

        res = torch.empty_like(send_tensor) if recv_tensor is None else recv_tensor
        send_tensor = send_tensor.contiguous()
        self._ops.append(dist.P2POp(dist.isend, send_tensor, to_rank))
        self._ops.append(dist.P2POp(dist.irecv, res, from_rank))
        return res

    def commit(self):
        import torch.distributed as dist

        if self._reqs is not None:
            raise RuntimeError("commit called twice")
        self._reqs = dist.batch_isend_irecv(self._ops)

    def wait(self):
        if self._reqs is None:
            raise RuntimeError("wait called before commit")
        for req in self._reqs:
            req.wait()
        self._reqs = None
        self._ops = []


def one_dim_to_n_dim(one_dim_index, dimensions):
    return _ring.coords_of(int(one_dim_index), tuple(dimensions))


def n_dim_to_one_dim(n_dim_index, dimensions):
    return _ring.rank_of(tuple(n_dim_index), tuple(dimensions))


def shift_tuple_element(original_tuple, index, value, modulo):
    return _ring.shift_coord(tuple(original_tuple), index, value, modulo)


def get_src_dst_ranks(indices, mesh_shape, ring_dims):
    return _ring.writeback_src_dst(tuple(indices), tuple(mesh_shape), list(ring_dims))


_NAMES = ("SendRecv", "one_dim_to_n_dim", "n_dim_to_one_dim", "shift_tuple_element", "get_src_dst_ranks")


def install_backend_stub() -> types.ModuleType:
    """Register a stand-in `mercury.backend` that exports the restated runtime above, so that the
    emitted line `from mercury.backend import *` binds it.  Replaces any earlier stand-in."""
    pkg = types.ModuleType("mercury")
    pkg.__path__ = []  # type: ignore[attr-defined]
    backend = types.ModuleType("mercury.backend")
    here = sys.modules[__name__]
    for name in _NAMES:
        setattr(backend, name, getattr(here, name))
    backend.__all__ = list(_NAMES)  # type: ignore[attr-defined]
    pkg.backend = backend  # type: ignore[attr-defined]
    sys.modules["mercury"] = pkg
    sys.modules["mercury.backend"] = backend
    return backend


def get_default_args(func):
    """utils/flash_attn_dsl.py:14-29: argument -> default table (None without default, softcap 0.0);
    custom-op wrappers are looked through via `_init_fn`."""
    fn = func if inspect.isfunction(func) else func._init_fn
    spec = inspect.getfullargspec(fn)
    defaults = spec.defaults or ()
    table = dict(zip(spec.args, (None,) * (len(spec.args) - len(defaults)) + tuple(defaults)))
    if "softcap" in table:
        table["softcap"] = 0.0
    return table


def cpu_block_forward(q, k, v, dropout_p, softmax_scale, causal, window_size_left=-1, window_size_right=-1,
                      softcap=0.0, alibi_slopes=None, return_softmax=False):
    """fp32 CPU stand-in for the CUDA-only flash-attn block op, under its signature."""
    from . import block as _block

    out, lse = _block.block_attn_fwd(q, k, v, softmax_scale, causal=bool(causal))
    return out, lse, None, None


def load_emitted(code: str, block_forward: Callable, extra: Optional[Dict[str, object]] = None) -> Dict[str, object]:
    """exec() an emitted forward program against the restated runtime and the given block op."""
    install_backend_stub()
    ns: Dict[str, object] = {
        "_flash_attn_forward": block_forward,
        "get_default_args": get_default_args,
        "update_out_and_lse": _merge.update_out_and_lse,
        "flash_reduce": _merge.flash_reduce,
    }
    if extra:
        ns.update(extra)
    exec(compile(code, "<reference-emitted program>", "exec"), ns)
    return ns
