"""world_size-2 runs on CPU/gloo: the oracle's per-rank ring, the reference arm of bench.py,
and the rank-dependent host logic of the fused ring (schedules, causal pull sets)."""
import json
import os
import socket
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank_worker(rank, world, port, name, ret):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    from oracle import ring
    from tests.helpers import load_golden, shard_inputs

    g = load_golden(name)
    qs, kvs = shard_inputs(g["t"]["q"], g["t"]["k"], g["t"]["v"], world)
    o, lse = ring.rank_ring_fwd(qs[rank], kvs[rank], g["D"] ** -0.5, g["mesh"])
    ret[rank] = (o, lse)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("name", ["ring_p2", "gqa_p2"])
def test_oracle_rank_ring_over_gloo_matches_reference_vectors(name):
    import torch.multiprocessing as mp
    from tests.helpers import load_golden

    g = load_golden(name)
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_rank_worker, args=(g["world"], _free_port(), name, ret), nprocs=g["world"], join=True)
    for r in range(g["world"]):
        eo = (ret[r][0] - g["t"][f"o_rank{r}"]).abs().max().item()
        el = (ret[r][1] - g["t"][f"lse_rank{r}"]).abs().max().item()
        assert eo <= 1e-4 and el <= 1e-4, (name, r, eo, el)


def _emitted_worker(rank, world, port, name, ret):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    from oracle import refexec
    from tests.helpers import golden_text, load_golden, shard_inputs

    g = load_golden(name)
    qs, kvs = shard_inputs(g["t"]["q"], g["t"]["k"], g["t"]["v"], world)
    ns = refexec.load_emitted(golden_text(name), refexec.cpu_block_forward)
    fn = ns["gqa_pack_kv" if name.startswith("gqa") else "flash_attn_pack_kv"]
    o = torch.zeros_like(qs[rank])
    lse = torch.zeros(g["B"], g["H"], qs[rank].shape[1])
    fn(qs[rank], kvs[rank], o, lse, g["D"] ** -0.5)
    ret[rank] = (o, lse)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("name", ["ring_p2", "gqa_p2"])
def test_emitted_program_on_restated_runtime_matches_reference_vectors(name):
    """The runtime bench.py's CPU arm and GPU baseline use to execute reference-emitted text
    (oracle/refexec.py: restated SendRecv, index helpers, get_default_args, merge) reproduces what
    the reference's own runtime produced for the same text and inputs."""
    import torch.multiprocessing as mp
    from tests.helpers import load_golden

    g = load_golden(name)
    ret = mp.Manager().dict()
    mp.spawn(_emitted_worker, args=(g["world"], _free_port(), name, ret), nprocs=g["world"], join=True)
    for r in range(g["world"]):
        eo = (ret[r][0] - g["t"][f"o_rank{r}"]).abs().max().item()
        el = (ret[r][1] - g["t"][f"lse_rank{r}"]).abs().max().item()
        assert eo <= 1e-4 and el <= 1e-4, (name, r, eo, el)


def test_bench_reference_arm_under_two_ranks():
    """`bench.py --impl reference --gpus 2` as the driver launches it: rank 0 prints one JSON line,
    the other rank exits 0 silently."""
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(_free_port()), WORLD_SIZE="2")
    outs = []
    for rank in (0, 1):
        e = dict(env, RANK=str(rank), LOCAL_RANK=str(rank))
        outs.append(subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "2",
                                    "--steps", "1", "--warmup", "0"], env=e, capture_output=True, text=True, timeout=600))
    assert outs[0].returncode == 0 and outs[1].returncode == 0
    assert outs[1].stdout.strip() == ""
    line = json.loads(outs[0].stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["n_gpus"] == 2 and line["value"] > 0
    assert line["cpu_baseline"]["kind"] == "port" and line["e2e"]["h2d_bytes_per_step"] == 0
    assert line["cpu_baseline"]["cores"] >= 2 and "2 CPU/gloo process(es)" in line["cpu_baseline"]["sample"]
    assert line["unit"] == "TFLOP/s" and line["higher_is_better"] is True


def test_causal_pull_sets_cover_exactly_the_visible_shards():
    """Which shards a rank pulls in the fused ring (forward: keys it can see; backward: also the query
    shards that can see its keys) -- pure host logic, checked for every rank of 2- and 8-rank rings."""
    from mercury_artifact_b200 import mesh

    for shape in [(2,), (8,), (4, 2)]:
        p = 1
        for n in shape:
            p *= n
        for r in range(p):
            order = mesh.kv_origin_schedule(r, shape)
            sees = [o for o in order[1:] if o <= r]
            seen_by = [o for o in order[1:] if o >= r]
            assert sorted(sees + [r]) == list(range(r + 1))
            assert sorted(seen_by + [r]) == list(range(r, p))
            # every unordered pair of ranks exchanges at least one direction under the causal rule
            assert set(sees) | set(seen_by) == set(range(p)) - {r}


def _heads_plan_worker(rank, world, port, ret):
    """One gloo rank: its own heads-schedule plan (forward and backward) against a recording context, then an
    all-gather of who delivers which head group to whom."""
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from mercury_artifact_b200 import ring
    from tests.test_ring_plan_cpu import _run_rank

    L = 256
    op, launches, fwd_ops, bwd_ops = _run_rank(dist.get_rank(), dist.get_world_size(), (world,), True, 1, True,
                                               B=1, L=L, H=4, hkv=2, schedule="heads")
    x = op._x
    fwd = [l for l in launches if l[0] == "fwd"][0]
    delivers = sorted((x.sym.where(jb["out_raw"][0])[0], rank) for jb in fwd[1] if "out_raw" in jb)
    pulls = sorted({x.sym.where(p[2])[0] for k, s, p in fwd_ops if k == "copy2d"})
    grads = sorted({x.sym.where(p[0])[0] for k, s, p in bwd_ops if k == "copy2d" and x.sym.where(p[0]) is not None
                    and x.sym.where(p[0])[1] >= x.slot_bytes + op._inbox_dkv})
    gathered = [None] * world
    dist.all_gather_object(gathered, {"delivers": delivers, "pulls": pulls, "grads": grads})
    ret[rank] = gathered
    dist.barrier()
    dist.destroy_process_group()


def test_heads_schedule_plans_of_two_gloo_ranks_fit_together():
    """world_size 2 over gloo: every (owner, head group) pair of the forward is delivered by exactly one rank,
    every rank pulls from its peer, and the backward pushes dk | dv rows to both owners."""
    import torch.multiprocessing as mp

    world = 2
    ret = mp.Manager().dict()
    mp.spawn(_heads_plan_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    for r in range(world):
        views = ret[r]
        assert sorted(d for v in views for d in v["delivers"]) == [(o, g) for o in range(world) for g in range(world)]
        for p, v in enumerate(views):
            assert v["pulls"] == [q for q in range(world) if q != p]
            assert v["grads"] == list(range(world))
