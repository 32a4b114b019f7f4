"""Tree (all-reduce) merge of partial attention results over peer memory.

Drop-in for update_out_and_lse_collective (utils/flash_attn_dsl.py:307-324 of the
reference), which the generated code calls when K/V are sharded and the queries
replicated (mercury/backend/pytorch/codegen.py:427-440).  The reference spends
three NCCL collectives (all_reduce MAX of the LSE, all_reduce SUM of the rescaled
outputs and of the weights); here every rank publishes its packed fp32
[..., D+1] = [out | lse] buffer in symmetric memory and one kernel per rank reads
all group members' buffers through the peer mappings (loads over NVLink) and
merges them in a single pass (C ABI: mb_tree_merge).
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, Optional, Tuple

import torch

from . import _lib
from .comm import default_context
from .ring import _Exchange

_exchanges: Dict[Tuple[int, Tuple[int, ...]], _Exchange] = {}


def _members(group) -> Tuple[int, ...]:
    import torch.distributed as dist

    if group is None:
        return tuple(range(dist.get_world_size()))
    if isinstance(group, (tuple, list)):
        return tuple(group)
    return tuple(dist.get_process_group_ranks(group))


def update_out_and_lse_collective(tensor: torch.Tensor, op, group, dst: Optional[int] = None):
    """In-place merge of `tensor` ([..., D+1] fp32, last column the LSE) across `group`.

    op is torch.distributed.all_reduce (every member ends with the merged result) or
    torch.distributed.reduce (only `dst` does); reduce_scatter is unsupported, as in the reference.
    """
    import torch.distributed as dist

    if op not in (dist.all_reduce, dist.reduce):
        raise RuntimeError("Unsupported collective op")
    if not tensor.is_cuda or tensor.dtype != torch.float32 or not tensor.is_contiguous():
        raise ValueError("update_out_and_lse_collective: contiguous fp32 CUDA tensor expected")
    ranks = _members(group)
    if len(ranks) > 16:
        raise ValueError("at most 16 ranks per merge group")
    ctx = default_context()
    me = ctx.rank
    if me not in ranks:
        raise ValueError("the calling rank is not a member of the group")
    width = tensor.shape[-1]
    rows = tensor.numel() // width
    nbytes = tensor.numel() * 4
    if len(ranks) == 1:
        return tensor
    key = (nbytes, ranks)
    x = _exchanges.get(key)
    if x is None:
        # collective: every rank of the job creates it.  No staging: the merge kernel reads peers' slots directly.
        x = _exchanges[key] = _Exchange(ctx, nbytes, 0, staging=False)
    main = torch.cuda.current_stream()
    comm = ctx.comm_stream
    e = x.begin(main)
    x.wait_slot_free(ranks)       # every member has finished reading my buffer of the previous merge
    with torch.cuda.stream(comm):
        x.slot()[:nbytes].view(torch.float32).view(tensor.shape).copy_(tensor, non_blocking=True)
    published = x.publish(ranks)
    main.wait_event(published)
    ctx.wait_many([(x.ready_ptr(me, r), e) for r in ranks if r != me], main)
    if op == dist.all_reduce or dst == me:
        srcs = (C.c_void_p * len(ranks))(*[x.sym.ptr(r, 0) for r in ranks])
        with torch.cuda.device(tensor.device):
            _lib.check(_lib.lib.mb_tree_merge(srcs, len(ranks), tensor.data_ptr(), rows, width,
                                              C.c_void_p(main.cuda_stream)), "mb_tree_merge")
    ctx.signal_many([(x.done_ptr(r, me), e) for r in ranks if r != me], main)
    return tensor
