"""Device-mesh index helpers and ring schedules (host logic).

Same names and meaning as the helpers the generated text imports from
mercury.backend (mercury/backend/pytorch/utils.py:41-106, 171-192): mesh
dimension 0 varies fastest in the rank numbering.
"""
from __future__ import annotations

from functools import lru_cache
from typing import List, Optional, Sequence, Tuple


@lru_cache(maxsize=None)
def one_dim_to_n_dim(one_dim_index: int, dimensions: Tuple[int, ...]) -> Tuple[int, ...]:
    """Rank -> mesh coordinates (coordinate 0 is the fastest-varying one)."""
    coords = []
    rest = int(one_dim_index)
    for n in dimensions:
        coords.append(rest % n)
        rest //= n
    return tuple(coords)


@lru_cache(maxsize=None)
def n_dim_to_one_dim(n_dim_index: Tuple[int, ...], dimensions: Tuple[int, ...]) -> int:
    """Mesh coordinates -> rank."""
    rank, weight = 0, 1
    for c, n in zip(n_dim_index, dimensions):
        rank += c * weight
        weight *= n
    return rank


@lru_cache(maxsize=None)
def shift_tuple_element(original_tuple: tuple, index: int, value: int, modulo: int) -> tuple:
    """Copy of the tuple with element `index` moved by `value` (either sign), wrapped into [0, modulo)."""
    moved = (original_tuple[index] + value) % modulo
    return original_tuple[:index] + (moved,) + original_tuple[index + 1:]


def get_src_dst_ranks(indices: Tuple[int, ...], mesh_shape: Tuple[int, ...], ring_dims: Sequence[int]) -> Tuple[int, int]:
    """(source, destination) rank of the final hop that brings a rotating reduce buffer back
    to the rank owning that shard; ring_dims are walked innermost-last with the step growing
    to the size of the dimension just handled."""
    def walk(sign: int) -> int:
        pos, step = tuple(indices), 1
        for dim in reversed(list(ring_dims)):
            pos = shift_tuple_element(pos, dim, sign * step, mesh_shape[dim])
            step = mesh_shape[dim]
        return n_dim_to_one_dim(pos, tuple(mesh_shape))

    return walk(-1), walk(+1)


def kv_origin_schedule(rank: int, mesh_shape: Sequence[int]) -> List[int]:
    """Origin rank of the K/V shard a rank works on at each step of the generated ring loop.

    Single ring of P ranks: step t uses the shard of rank (r - t) mod P.  Nested rings (mesh
    (n0, n1, ...)): the loop nest runs mesh dim 0 innermost; a step moves the shard one hop
    along the first dimension whose ring index is not at its end, so the coordinate along
    dimension d has moved by -(number of hops taken along d so far).
    """
    shape = tuple(int(n) for n in mesh_shape)
    me = one_dim_to_n_dim(rank, shape)
    total = 1
    for n in shape:
        total *= n
    hops = [0] * len(shape)
    out = []
    idx = [0] * len(shape)
    for _ in range(total):
        origin = tuple((me[d] - hops[d]) % shape[d] for d in range(len(shape)))
        out.append(n_dim_to_one_dim(origin, shape))
        # advance the loop nest (dim 0 innermost) and record which dim the shard moved along
        for d in range(len(shape)):
            if idx[d] + 1 != shape[d]:
                hops[d] += 1
                break
        for d in range(len(shape)):
            idx[d] += 1
            if idx[d] < shape[d]:
                break
            idx[d] = 0
    return out


_group_cache = {}


def group_ranks(indices: Tuple[int, ...], mesh_shape: Tuple[int, ...], dims: Sequence[int]) -> Tuple[int, ...]:
    """Ranks that share every mesh coordinate with `indices` except along `dims` (sorted)."""
    for d in dims:
        if d < 0 or d >= len(mesh_shape):
            raise ValueError(f"Invalid dimension index: {d}, mesh shape: {mesh_shape}")
    ranks = []
    total = 1
    for n in mesh_shape:
        total *= n
    for r in range(total):
        c = one_dim_to_n_dim(r, tuple(mesh_shape))
        if all(c[i] == indices[i] for i in range(len(mesh_shape)) if i not in dims):
            ranks.append(r)
    return tuple(sorted(ranks))


def get_device_group(indices: Tuple[int, ...], mesh_shape: Tuple[int, ...], dims: Tuple[int, ...], debug: bool = False):
    """Communication group of the ranks that differ from `indices` only along `dims`
    (mercury/backend/pytorch/utils.py:114-169).  Every rank of the job must call this in the same
    order, because the groups of ALL ranks are created (torch.distributed.new_group is collective);
    debug=True returns the tuple of ranks instead of a process group."""
    key = (tuple(indices), tuple(mesh_shape), tuple(dims), bool(debug))
    if key in _group_cache:
        return _group_cache[key]
    import torch.distributed as dist

    total = 1
    for n in mesh_shape:
        total *= n
    made = {}
    mine = None
    for r in range(total):
        c = one_dim_to_n_dim(r, tuple(mesh_shape))
        ranks = group_ranks(c, tuple(mesh_shape), tuple(dims))
        if ranks not in made:
            made[ranks] = ranks if debug else dist.new_group(ranks=list(ranks))
        if c == tuple(indices):
            mine = made[ranks]
    _group_cache[key] = mine
    return mine
