"""Run a per-rank program for P virtual ranks on ONE device (test double, not product).

Each rank is a host thread.  `torch.distributed.get_rank` is patched to a thread-local value
and the transport is an in-process mailbox with the SendRecv interface, so a program emitted
by the reference's code generator can be executed for world_size > 1 on a single GPU (or on
the CPU) with only the compute ops under test being real.
"""
from __future__ import annotations

import os
import queue
import threading
from typing import Callable, Dict, List, Tuple

import torch
import torch.distributed as dist

_local = threading.local()
_mailboxes: Dict[Tuple[int, int], "queue.Queue"] = {}
_mail_lock = threading.Lock()


def _box(src: int, dst: int) -> "queue.Queue":
    with _mail_lock:
        return _mailboxes.setdefault((src, dst), queue.Queue())


class MailboxSendRecv:
    """Same interface and error behaviour as the reference's SendRecv."""

    def __init__(self):
        self._ops: List[tuple] = []
        self._committed = None

    def send_recv(self, to_rank, from_rank, send_tensor, recv_tensor=None):
        res = torch.empty_like(send_tensor) if recv_tensor is None else recv_tensor
        self._ops.append((to_rank, from_rank, send_tensor.contiguous(), res))
        return res

    def commit(self):
        if self._committed is not None:
            raise RuntimeError("commit called twice")
        me = _local.rank
        for to_rank, _from, send, _res in self._ops:
            payload = send.clone()
            ev = None
            if payload.is_cuda:
                ev = torch.cuda.Event()
                ev.record(torch.cuda.current_stream())
            _box(me, to_rank).put((payload, ev))
        self._committed = list(self._ops)

    def wait(self):
        if self._committed is None:
            raise RuntimeError("wait called before commit")
        me = _local.rank
        for _to, from_rank, _send, res in self._committed:
            payload, ev = _box(from_rank, me).get(timeout=120)
            if ev is not None:
                torch.cuda.current_stream().wait_event(ev)
            res.copy_(payload)
        self._committed = None
        self._ops = []


def run_ranks(world: int, fn: Callable[[int], object]) -> List[object]:
    """Call fn(rank) on `world` threads with dist.get_rank() answering per thread."""
    _mailboxes.clear()
    results: List[object] = [None] * world
    errors: List[BaseException] = []
    real_get_rank = dist.get_rank
    dist.get_rank = lambda group=None: _local.rank  # type: ignore[assignment]
    os.environ.setdefault("LOCAL_RANK", "0")

    def body(r: int):
        _local.rank = r
        try:
            if torch.cuda.is_available():
                with torch.cuda.stream(torch.cuda.Stream()):
                    results[r] = fn(r)
                    torch.cuda.current_stream().synchronize()
            else:
                results[r] = fn(r)
        except BaseException as e:  # noqa: BLE001
            errors.append(e)

    threads = [threading.Thread(target=body, args=(r,), daemon=True) for r in range(world)]
    try:
        for t in threads:
            t.start()
        for t in threads:
            t.join(timeout=300)
    finally:
        dist.get_rank = real_get_rank  # type: ignore[assignment]
    if errors:
        raise errors[0]
    return results
