"""Shared helpers for the tests: golden loading and seeded inputs."""
from __future__ import annotations

from pathlib import Path

import numpy as np
import torch

GOLDEN = Path(__file__).resolve().parent / "golden"


def load_golden(name: str):
    z = np.load(GOLDEN / f"{name}.npz")
    meta = z["meta"].tolist()
    world, B, S, H, hkv, D, seed = meta[:7]
    mesh = tuple(meta[7:])
    t = {k: torch.from_numpy(z[k]) for k in z.files if k != "meta"}
    return dict(world=world, B=B, S=S, H=H, hkv=hkv, D=D, seed=seed, mesh=mesh, t=t)


def golden_text(name: str) -> str:
    return (GOLDEN / f"{name}.gen.txt").read_text()


def shard_inputs(q, k, v, world):
    qs = [x.contiguous() for x in q.chunk(world, 1)]
    kvs = [torch.stack([k.chunk(world, 1)[r], v.chunk(world, 1)[r]]).contiguous() for r in range(world)]
    return qs, kvs


def seeded_qkv(seed, B, S, H, hkv, D, scale=0.5, dtype=torch.bfloat16, device="cpu"):
    """Q/K/V (and dO) ~ N(0,1)*scale from per-tensor seeds, built on the CPU then moved."""
    out = []
    for i, (heads) in enumerate((H, hkv, hkv, H)):
        g = torch.Generator().manual_seed(seed + i)
        out.append((torch.randn(B, S, heads, D, generator=g) * scale).to(dtype).to(device))
    return out
