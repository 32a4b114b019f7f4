#!/usr/bin/env python
"""Headline benchmark: causal ring-attention forward, bf16 B1 S32768 H32 D128, sharded over N GPUs.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

A step is one forward of the whole job (every rank's shard).  `value` is causal-adjusted attention
TFLOP/s summed over all GPUs with inputs resident in HBM; `e2e` is the same metric through the public
API with pinned HOST buffers (host->device copies of q and kv and the device->host read of o and lse
inside the timed region).  Besides the headline the JSON line carries
  parity        row-sampled fp32 check of THIS run's outputs (forward and backward), every rank
  fwd_bwd       forward + backward per step
  sustained     the forward in a >= 2 s back-to-back loop with the SM clock seen (1 GPU)
  extra         the other sequence-parallel workloads (131072-token causal forward, GQA, double ring,
                65536-token causal backward), a few steps each, with their own parity blocks
  gpu_baseline  the reference's shipped path on the same GPUs: the program its compiler emitted for
                this shape, run with the flash-attn block op, its running merge and NCCL messages
  per_step_path the same emitted program on this package's per-step drop-ins, and the merge
                kernels against the HBM roofline
  cpu_baseline  (1 GPU) the CPU restatement on the host cores.

N > 1 is launched by torch.distributed.run, one rank per GPU (NCCL for bootstrap and for gathering
the tensors the parity check needs); timing is CUDA events on the launching stream, max over ranks.
`--impl reference` runs the program the reference's compiler emitted as `--gpus` CPU/gloo ranks on
the host cores (block op replaced by the fp32 CPU restatement), on a shortened sequence.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import socket
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# dram__bytes_read.sum + dram__bytes_write.sum of one attn_fwd_kernel launch, from an ncu capture
# (profiles/attn_fwd_kernel_profile16k.md).  profile_16k was captured directly; the 32768-token case
# at one GPU is that capture scaled by 2 (bytes grow linearly in the sequence length at fixed batch,
# heads and head_dim).
NCU_DRAM_BYTES_PER_LAUNCH = {("profile_16k", 1): 5.23e8, ("cfg2", 1): 1.046e9}

WORKLOADS = {
    # name: (batch, seqlen, hq, hkv, head_dim, causal)
    "cfg2": (1, 32768, 32, 32, 128, True),
    "cfg2_nc": (1, 32768, 32, 32, 128, False),
    "target_131k": (1, 131072, 32, 32, 128, True),
    "cfg3_gqa": (2, 131072, 32, 8, 128, True),
    "cfg4_dring": (1, 262144, 16, 16, 128, False),
    "cfg5_bwd": (1, 65536, 32, 32, 128, True),
    # smaller case of the same kernel for ncu captures: inputs (384 MiB) still exceed L2
    "profile_16k": (1, 16384, 32, 32, 128, True),
}
METRIC = "ring-attn causal-adj TFLOP/s (fwd), whole job"
FALLBACK_PEAK_TFLOPS = 1590.0
FALLBACK_HBM_GBS = 6650.0
O_TOL, LSE_TOL = 2e-2, 1e-3   # bf16 o/dq/dk/dv max-abs, fp32 lse max-abs, against fp32 attention


def flops_fwd(B, S, H, D, causal):
    return 4.0 * B * H * S * S * D * (0.5 if causal else 1.0)


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return (float(d["bf16_tflops"]), float(d.get("bf16_tflops_sustained", 0) or 0),
                    float(d.get("hbm_gbs", 0) or FALLBACK_HBM_GBS), "measured")
        except Exception:
            pass
    return FALLBACK_PEAK_TFLOPS, 1400.0, FALLBACK_HBM_GBS, "fallback"


def mesh_for(workload, world):
    """Single ring, except the double-ring workload: inner ring x outer groups."""
    if workload == "cfg4_dring":
        return {8: (4, 2), 4: (2, 2)}.get(world, (world,))
    return (world,)


def free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 200 ms while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.rows = []
        self.proc = None
        self.gpu_index = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:
            self.proc = None
        return self

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def stop(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        rows = [r for t, r in self.rows if t0 - 0.05 <= t <= t1 + 0.25] or [r for _, r in self.rows]
        sm, mx, reasons = [], [], set()
        for r in rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            except Exception:
                continue
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ----------------------------------------------------------------------------- CPU legs
def _cpu_rank(rank, world, port, threads, seq, steps, warmup, ret):
    """One CPU/gloo rank executing the program the reference's compiler emitted for `world` ranks."""
    import torch
    import torch.distributed as dist

    from oracle import refexec

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(threads)
    torch.set_flush_denormal(True)  # exp() of far-below-max scores is denormal and very slow otherwise
    text = (ROOT / "tests" / "golden" / f"cpu_ring_p{world}.gen.txt").read_text()
    fn = refexec.load_emitted(text, refexec.cpu_block_forward)["flash_attn_pack_kv"]
    B, _, H, hkv, D, _ = WORKLOADS["cfg2"]
    L = seq // world
    g = torch.Generator().manual_seed(1234 + rank)
    q = torch.randn(B, L, H, D, generator=g) * 0.5
    kv = torch.randn(2, B, L, hkv, D, generator=g) * 0.5
    o = torch.empty_like(q)
    lse = torch.empty(B, H, L)
    times = []
    for i in range(warmup + steps):
        dist.barrier()
        t0 = time.perf_counter()
        fn(q, kv, o, lse, D ** -0.5)
        dist.barrier()
        if i >= warmup:
            times.append(time.perf_counter() - t0)
        # stop early, on every rank together, once the timed steps add up to 150 s on the slowest rank
        spent = torch.tensor([sum(times)], dtype=torch.float64)
        dist.all_reduce(spent, op=dist.ReduceOp.MAX)
        if spent.item() > 150:
            break
    if rank == 0:
        ret["times"] = times
    dist.destroy_process_group()


CPU_SAMPLE_SEQ = 4096  # the sequence length of tests/golden/cpu_ring_p*.gen.txt


def cpu_leg(world, steps=1, warmup=1):
    """The reference's emitted ring program as `world` CPU/gloo ranks on this host's cores.

    Bounded sample: batch, heads and head_dim of the headline workload, sequence shortened to 4096, and
    non-causal -- the emitted program hands `causal` unchanged to every block, which is only meaningful
    for causal=False (the FLOP count follows).  Returns (TFLOP/s, cores, description, seconds/step)."""
    import torch.multiprocessing as mp

    B, S, H, hkv, D, _ = WORKLOADS["cfg2"]
    cores = len(os.sched_getaffinity(0))
    threads = max(1, cores // world)
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_cpu_rank, args=(world, free_port(), threads, CPU_SAMPLE_SEQ, steps, warmup, ret), nprocs=world, join=True)
    times = list(ret["times"])
    t = statistics.mean(times)
    tf = flops_fwd(B, CPU_SAMPLE_SEQ, H, D, False) / t / 1e12
    desc = (f"program emitted by the reference's compiler for {world} rank(s), run as {world} CPU/gloo process(es) x "
            f"{threads} thread(s) with the fp32 CPU block stand-in: B{B} H{H}/{hkv} D{D} non-causal at seqlen "
            f"{CPU_SAMPLE_SEQ} ({flops_fwd(B, CPU_SAMPLE_SEQ, H, D, False) / flops_fwd(B, S, H, D, True):.4f} of the "
            f"full workload's FLOPs), {t:.2f} s per step")
    return tf, threads * world, desc, t, len(times)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    tf, cores, desc, t, n = cpu_leg(args.gpus, steps=args.steps, warmup=args.warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": tf, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": n, "warmup": args.warmup, "ms_per_step": 1e3 * t,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(args.workload, args.gpus), "sample": desc},
        "cpu_baseline": {"value": tf, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": desc},
        "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


def bind_host_to_gpu_node(device_index):
    """Run this process on the CPUs of the NUMA node the GPU hangs off, so that the pinned host buffers of the
    host-buffer leg are allocated there (a far node halves the PCIe rate the copies see).  Returns
    (description, previous affinity) -- (None, None) where the node is unknown."""
    try:
        import torch

        pr = torch.cuda.get_device_properties(device_index)
        bdf = f"{pr.pci_domain_id:04x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
        node = int(open(f"/sys/bus/pci/devices/{bdf}/numa_node").read().strip())
        if node < 0:
            return None, None
        cpus = set()
        for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        before = os.sched_getaffinity(0)
        cpus &= before
        if not cpus:
            return None, None
        os.sched_setaffinity(0, cpus)
        return f"GPU {bdf} on NUMA node {node}: process bound to its {len(cpus)} CPUs while the pinned buffers were made", before
    except Exception:
        return None, None


def workload_name(w, n):
    B, S, H, hkv, D, causal = WORKLOADS[w]
    return (f"{w}: ring-attention forward bf16 B{B} S{S} Hq{H} Hkv{hkv} D{D} "
            f"{'causal' if causal else 'non-causal'}, {n} contiguous shard(s)")


# ----------------------------------------------------------------------------- GPU arm
class Job:
    """Process-wide state of the GPU arm: ranks, device, timing and gather helpers."""

    def __init__(self):
        import torch
        import torch.distributed as dist

        self.torch, self.dist = torch, dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(self.local_rank)
        self.dev = torch.device("cuda", self.local_rank)
        torch.backends.cuda.matmul.allow_tf32 = False  # the parity reference is true fp32
        torch.backends.cudnn.allow_tf32 = False
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)
        self.stream = torch.cuda.current_stream()

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, x: float) -> float:
        if self.world == 1:
            return float(x)
        t = self.torch.tensor([x], device=self.dev, dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def timed(self, fn, steps, warmup):
        """W untimed steps, barrier + synchronize, K steps between two events, barrier + synchronize;
        milliseconds per step, max over ranks, plus the wall-clock window for the clock samples."""
        torch = self.torch
        for _ in range(warmup):
            fn()
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.time()
        e0.record(self.stream)
        for _ in range(steps):
            fn()
        e1.record(self.stream)
        self.barrier()
        t1 = time.time()
        return self.max_over_ranks(e0.elapsed_time(e1) / steps), t0, t1

    def inputs_in(self, op, B, L, H, hkv, D, with_dout=False, seed=1234):
        """The same seeded shard, produced inside the op's symmetric buffers (no staging copies when they
        are passed to forward() / backward()), plus its o and lse result tensors."""
        bufs = op.symmetric_buffers()
        q, kv, dout = self.inputs(B, L, H, hkv, D, with_dout=with_dout, seed=seed)
        bufs["q"].copy_(q)
        bufs["kv"].copy_(kv)
        if with_dout:
            bufs["dout"].copy_(dout)
        self.torch.cuda.synchronize()
        return bufs["q"], bufs["kv"], bufs.get("dout"), bufs["o"], bufs["lse"]

    def inputs(self, B, L, H, hkv, D, with_dout=False, seed=1234):
        """Seeded synthetic shard of this rank, generated on the device: q, kv (and dout) ~ N(0,1)*0.5."""
        torch = self.torch
        g = torch.Generator(device=self.dev).manual_seed(seed + self.rank)
        q = (torch.randn(B, L, H, D, generator=g, device=self.dev) * 0.5).to(torch.bfloat16)
        kv = (torch.randn(2, B, L, hkv, D, generator=g, device=self.dev) * 0.5).to(torch.bfloat16)
        dout = (torch.randn(B, L, H, D, generator=g, device=self.dev) * 0.5).to(torch.bfloat16) if with_dout else None
        return q, kv, dout


def parity_forward(job, q, kv, o, lse, causal, scale, rows=64):
    """Row sample of every rank's o/lse against fp32 attention over ALL keys of the job."""
    from oracle import sampled

    r = sampled.check_forward_shard(q, kv, o, lse, job.rank, job.world, causal, scale, rows=rows)
    eo, el = job.max_over_ranks(r["o_max_abs"]), job.max_over_ranks(r["lse_max_abs"])
    fin = math.isfinite(eo) and math.isfinite(el)
    return {"o_max_abs": eo, "lse_max_abs": el, "rows": r["rows"] * job.world,
            "ok": fin and eo <= O_TOL and el <= LSE_TOL}


def parity_backward(job, q, kv, o, lse, dout, dq, dkv, causal, scale, rows=48):
    """Row sample of dq (every rank's queries vs all keys) and of dk/dv (its keys vs all queries)."""
    from oracle import sampled

    r = sampled.check_backward_shard(q, kv, o, lse, dout, dq, dkv, job.rank, job.world, causal, scale, rows=rows)
    eq, ek, ev = (job.max_over_ranks(r[k]) for k in ("dq_max_abs", "dk_max_abs", "dv_max_abs"))
    fin = all(math.isfinite(x) for x in (eq, ek, ev))
    return {"dq_max_abs": eq, "dk_max_abs": ek, "dv_max_abs": ev, "rows": r["rows"] * job.world,
            "ok": fin and max(eq, ek, ev) <= O_TOL}


def run_extra(job, name, peak, sustained, steps=3, warmup=2):
    """One of the other workloads: a few steps, per-GPU rate against both peaks, parity of its outputs."""
    import torch

    import mercury_artifact_b200 as mb
    from mercury_artifact_b200 import _lib
    from mercury_artifact_b200.ring import RingAttention

    B, S, H, hkv, D, causal = WORKLOADS[name]
    world = job.world
    L = S // world
    scale = D ** -0.5
    mesh = mesh_for(name, world)
    backward = name.endswith("_bwd")
    op = RingAttention(mesh, B, L, H, hkv, D, causal=causal, backward=backward)
    q, kv, dout, o, lse = job.inputs_in(op, B, L, H, hkv, D, with_dout=backward, seed=4321)
    fl = flops_fwd(B, S, H, D, causal)
    res = {"workload": workload_name(name, world).replace("forward", "backward" if backward else "forward"),
           "mesh": list(mesh), "schedule": getattr(op, "schedule", "ring") if world > 1 else "one rank",
           "steps": steps, "warmup": warmup}
    if backward:
        op.forward(q, kv, o, lse, scale)
        bufs = op.symmetric_buffers() if world > 1 else {}
        dq, dkv = bufs.get("dq", torch.empty_like(q)), bufs.get("dkv", torch.empty_like(kv))
        ms, _, _ = job.timed(lambda: op.backward(dout, q, kv, o, lse, dq, dkv, scale), steps, warmup)
        fl *= 2.5
        res["note"] = "backward only; FLOPs counted as 2.5 x the forward's"
    else:
        ms, _, _ = job.timed(lambda: op.forward(q, kv, o, lse, scale), steps, warmup)
    status = _lib.status_fetch(job.stream.cuda_stream)
    per_gpu = fl / (ms * 1e-3) / 1e12 / world
    res.update({"ms_per_step": ms, "tflops": per_gpu * world, "tflops_per_gpu": per_gpu,
                "frac_of_burst_peak": per_gpu / peak, "frac_of_sustained_peak": per_gpu / sustained if sustained else None,
                "device_status": int(job.max_over_ranks(status))})
    res["parity"] = parity_forward(job, q, kv, o, lse, causal, scale)
    if backward:
        res["parity"].update(parity_backward(job, q, kv, o, lse, dout, dq, dkv, causal, scale))
        res["parity"]["ok"] = bool(res["parity"]["ok"] and res["parity"]["o_max_abs"] <= O_TOL
                                   and res["parity"]["lse_max_abs"] <= LSE_TOL)
    del op, q, kv, o, lse, dout
    torch.cuda.empty_cache()
    return res


def run_emitted_programs(job, steps=5, warmup=2):
    """The program the reference's compiler emitted for this shape (non-causal: the only mode it computes
    correctly), run (a) as the reference ships it -- flash-attn block op, its running merge, NCCL
    batch_isend_irecv -- and (b) on this package's per-step drop-ins; plus (c) the fused one-launch
    form on the same inputs, and the merge kernels alone against the HBM roofline."""
    import torch
    import torch.distributed as dist

    import mercury_artifact_b200 as mb
    from mercury_artifact_b200.ring import RingAttention

    world = job.world
    B, S, H, hkv, D, _ = WORKLOADS["cfg2_nc"]
    L = S // world
    scale = D ** -0.5
    text_path = ROOT / "tests" / "golden" / f"bench_ring_p{world}.gen.txt"
    out = {"workload": workload_name("cfg2_nc", world), "steps": steps, "warmup": warmup}
    if not text_path.exists():
        return {"unavailable": f"no emitted program for {world} ranks"}, {"unavailable": "no emitted program"}
    text = text_path.read_text()
    os.environ.setdefault("LOCAL_RANK", str(job.local_rank))
    own_group = False
    if not dist.is_initialized():  # the emitted text calls dist.get_rank()
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{free_port()}", rank=0, world_size=1)
        own_group = True
    q, kv, _ = job.inputs(B, L, H, hkv, D, seed=999)
    o = torch.empty_like(q)
    lse = torch.empty(B, H, L, dtype=torch.float32, device=job.dev)
    fl = flops_fwd(B, S, H, D, False)

    def rate(ms):
        return fl / (ms * 1e-3) / 1e12

    # (c) fused form first: its result is the comparison for the other two
    op = RingAttention((world,), B, L, H, hkv, D, causal=False)
    ms_fused, _, _ = job.timed(lambda: op.forward(q, kv, o, lse, scale), steps, warmup)
    o_fused, lse_fused = o.clone(), lse.clone()

    # (a) the reference's shipped path
    base = dict(out)
    try:
        from flash_attn.flash_attn_interface import _flash_attn_forward as fa_forward

        from oracle import refexec

        fn = refexec.load_emitted(text, fa_forward)["flash_attn_pack_kv"]
        ms_ref, _, _ = job.timed(lambda: fn(q, kv, o, lse, scale), steps, warmup)
        base.update({"ms_per_step": ms_ref, "tflops": rate(ms_ref), "kind": "flash-attn block op + running merge + "
                     "NCCL batch_isend_irecv, program emitted by the reference's compiler",
                     "fused_ms_per_step": ms_fused, "fused_tflops": rate(ms_fused),
                     "speedup_fused_over_reference": ms_ref / ms_fused,
                     "o_max_abs_vs_fused": job.max_over_ranks((o.float() - o_fused.float()).abs().max().item()),
                     "lse_max_abs_vs_fused": job.max_over_ranks((lse - lse_fused).abs().max().item())})
    except Exception as e:  # flash-attn wheel missing or not runnable on this GPU
        base = {"unavailable": f"{type(e).__name__}: {e}"[:300]}

    # (b) the same text on the per-step drop-ins
    per = dict(out)
    mb.install_backend(force_stub=True)
    fn2 = mb.load_generated(text)["flash_attn_pack_kv"]
    o.zero_()
    ms_step, _, _ = job.timed(lambda: fn2(q, kv, o, lse, scale), steps, warmup)
    per.update({"ms_per_step": ms_step, "tflops": rate(ms_step), "fused_ms_per_step": ms_fused,
                "o_max_abs_vs_fused": job.max_over_ranks((o.float() - o_fused.float()).abs().max().item()),
                "lse_max_abs_vs_fused": job.max_over_ranks((lse - lse_fused).abs().max().item())})
    if "ms_per_step" in base:
        per["speedup_over_reference_path"] = base["ms_per_step"] / ms_step

    # merge kernels alone, HBM-bound: bytes per output element of one launch
    _, _, hbm, kind = measured_peaks()
    st_o = torch.empty(B, L, H, D, dtype=torch.float32, device=job.dev).normal_()
    st_l = torch.zeros(B, L, H, 1, dtype=torch.float32, device=job.dev)
    blk_l = torch.zeros(B, H, L, dtype=torch.float32, device=job.dev)
    n_el = B * L * H * D
    ms_m, _, _ = job.timed(lambda: mb.update_out_and_lse(st_o, st_l, o, blk_l), 20, 3)
    by_m = n_el * (4 + 2 + 4) + B * L * H * 12   # state read + bf16 block read + state write, + the three lse words
    packed = torch.empty(B, L, H, D + 1, dtype=torch.float32, device=job.dev).normal_()
    ms_r, _, _ = job.timed(lambda: mb.flash_reduce(packed, packed), 20, 3)
    by_r = B * L * H * (D + 1) * 12
    per["merge_kernel"] = {"ms": ms_m, "bytes": by_m, "achieved_gbs": by_m / (ms_m * 1e-3) / 1e9, "peak_gbs": hbm,
                           "frac": by_m / (ms_m * 1e-3) / 1e9 / hbm, "peak_kind": f"hbm_gbs, {kind}", "bound": "hbm"}
    per["flash_reduce_kernel"] = {"ms": ms_r, "bytes": by_r, "achieved_gbs": by_r / (ms_r * 1e-3) / 1e9,
                                  "peak_gbs": hbm, "frac": by_r / (ms_r * 1e-3) / 1e9 / hbm, "bound": "hbm",
                                  "note": "includes the allocation of the result tensor (the op returns a new one)"}
    if own_group:
        dist.destroy_process_group()
    return base, per


def run_ours(args):
    import torch
    import torch.distributed as dist

    world_env = int(os.environ.get("WORLD_SIZE", "1"))
    if world_env != args.gpus and world_env == 1 and args.gpus > 1:
        print(json.dumps({"error": f"--gpus {args.gpus} needs torch.distributed.run with {args.gpus} ranks"}))
        return 2
    job = Job()
    world, rank, dev = job.world, job.rank, job.dev

    import mercury_artifact_b200 as mb
    from mercury_artifact_b200 import _lib
    from mercury_artifact_b200.ring import RingAttention

    B, S, H, hkv, D, causal = WORKLOADS[args.workload]
    L = S // world
    scale = D ** -0.5
    mesh = mesh_for(args.workload, world)

    if world > 1:
        mb.comm.init_p2p()
    op = RingAttention(mesh, B, L, H, hkv, D, causal=causal, backward=True, schedule=args.schedule)
    # resident inputs live in the op's symmetric buffers (its documented zero-copy mode): peers pull
    # q / kv straight from there and results arrive in o / lse without staging copies
    q, kv, dout, o, lse = job.inputs_in(op, B, L, H, hkv, D, with_dout=True)
    schedule_note = None
    if world > 1 and args.schedule is None and op.schedule != "ring":
        # One probing step of the library's default schedule; if a device-side wait runs out on any rank
        # (a status code, never a hang), every rank falls back to the ring schedule and the line says so.
        bad = 0
        try:
            op.forward(q, kv, o, lse, scale)
            op.check()
        except _lib.MercuryB200Error as exc:
            bad = 1
            print(f"[bench] rank {rank}: {op.schedule} schedule failed its probing step: {exc}", file=sys.stderr)
        if job.max_over_ranks(bad) > 0:
            schedule_note = f"the {op.schedule} schedule failed its probing step on some rank; ring schedule used"
            try:
                _lib.status_fetch(job.stream.cuda_stream)      # clears the device word
            except Exception:
                pass
            op = RingAttention(mesh, B, L, H, hkv, D, causal=causal, backward=True, schedule="ring")
            q, kv, dout, o, lse = job.inputs_in(op, B, L, H, hkv, D, with_dout=True)
    numa_note, affinity_before = bind_host_to_gpu_node(job.local_rank)
    q_host, kv_host = q.cpu().pin_memory(), kv.cpu().pin_memory()
    o_host = torch.empty(B, L, H, D, dtype=torch.bfloat16).pin_memory()
    lse_host = torch.empty(B, H, L, dtype=torch.float32).pin_memory()
    if affinity_before is not None:
        os.sched_setaffinity(0, affinity_before)      # the CPU arm and everything else run where they did
    stream = job.stream

    def step_resident():
        op.forward(q, kv, o, lse, scale)

    def step_e2e():
        # public host-buffer entry: pinned host q/kv in, o/lse back in host memory when it returns
        op.forward_host(q_host, kv_host, o_host, lse_host, scale)

    def step_fwd_bwd():
        op.forward(q, kv, o, lse, scale)
        op.backward(dout, q, kv, o, lse, dq, dkv, scale)

    sampler = ClockSampler(job.local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    warm = max(args.warmup, 3)
    ms, t0, t1 = job.timed(step_resident, args.steps, warm)
    clocks = sampler.stop(t0, t1) if rank == 0 else None
    status = _lib.status_fetch(stream.cuda_stream)
    launches_per_step = op.last_launches if world > 1 else 1
    parity = parity_forward(job, q, kv, o, lse, causal, scale)

    # the same forward with ORDINARY tensors in and out: one device-to-device staging copy per tensor
    ms_plain = None
    if world > 1:
        pq, pkv = q.clone(), kv.clone()
        po, pl = torch.empty_like(q), torch.empty_like(lse)
        ms_plain, _, _ = job.timed(lambda: op.forward(pq, pkv, po, pl, scale), max(3, args.steps // 2), 3)
        status |= _lib.status_fetch(stream.cuda_stream)
        parity["plain_tensors_o_max_abs_vs_resident"] = job.max_over_ranks((po.float() - o.float()).abs().max().item())
        parity["ok"] = bool(parity["ok"] and parity["plain_tensors_o_max_abs_vs_resident"] <= O_TOL)
        del pq, pkv, po, pl

    ms_e2e, _, _ = job.timed(step_e2e, max(3, args.steps // 2), 3)
    status |= _lib.status_fetch(stream.cuda_stream)
    e2e_o = (o_host.to(dev).float() - o.float()).abs().max().item()   # the host path must reproduce the resident result
    e2e_l = (lse_host.to(dev) - lse).abs().max().item()
    parity["e2e_o_max_abs_vs_resident"] = job.max_over_ranks(e2e_o)
    parity["e2e_lse_max_abs_vs_resident"] = job.max_over_ranks(e2e_l)
    parity["ok"] = bool(parity["ok"] and parity["e2e_o_max_abs_vs_resident"] <= O_TOL
                        and parity["e2e_lse_max_abs_vs_resident"] <= LSE_TOL)

    # forward + backward (the metric's second figure): bwd counted as 2.5x the forward FLOPs
    gbufs = op.symmetric_buffers() if world > 1 else {}
    dq, dkv = gbufs.get("dq", torch.empty_like(q)), gbufs.get("dkv", torch.empty_like(kv))
    ms_fb, _, _ = job.timed(step_fwd_bwd, max(3, args.steps // 2), 3)
    status |= _lib.status_fetch(stream.cuda_stream)
    parity.update({k: v for k, v in parity_backward(job, q, kv, o, lse, dout, dq, dkv, causal, scale).items()
                   if k not in ("ok", "rows")})
    parity["ok"] = bool(parity["ok"] and max(parity["dq_max_abs"], parity["dk_max_abs"], parity["dv_max_abs"]) <= O_TOL)
    status = int(job.max_over_ranks(status))

    fl_total = flops_fwd(B, S, H, D, causal)
    value = fl_total / (ms * 1e-3) / 1e12
    e2e = fl_total / (ms_e2e * 1e-3) / 1e12
    peak, sustained, hbm, peak_kind = measured_peaks()
    per_gpu = value / world

    sustained_blk = None
    if world == 1 and not args.quick:
        # the same forward back to back for >= 2 s: the SM clock settles under the power cap
        n = max(args.steps, int(math.ceil(2200.0 / ms)))
        s2 = ClockSampler(job.local_rank).start()
        time.sleep(0.2)
        ms_s, a0, a1 = job.timed(step_resident, n, 2)
        c2 = s2.stop(a0, a1)
        tf = fl_total / (ms_s * 1e-3) / 1e12
        sustained_blk = {"value": tf, "unit": "TFLOP/s", "ms_per_step": ms_s, "steps": n, "seconds": n * ms_s * 1e-3,
                         "sm_mhz_median": c2.get("sm_mhz"), "reasons": c2.get("reasons"),
                         "tflops_per_ghz": (tf / (c2["sm_mhz"] / 1e3)) if c2.get("sm_mhz") else None,
                         "frac_of_sustained_peak": tf / sustained if sustained else None}

    extra = []
    if not args.quick and args.workload == "cfg2":
        for name in ("target_131k", "cfg3_gqa", "cfg4_dring", "cfg5_bwd"):
            try:
                extra.append(run_extra(job, name, peak, sustained))
            except Exception as e:
                extra.append({"workload": name, "error": f"{type(e).__name__}: {e}"[:300]})

    gpu_baseline = per_step = None
    if not args.quick and args.workload == "cfg2":
        try:
            gpu_baseline, per_step = run_emitted_programs(job)
        except Exception as e:
            gpu_baseline = {"unavailable": f"{type(e).__name__}: {e}"[:300]}

    rc = 0
    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": warm, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {
                "workload": workload_name(args.workload, world),
                "l2": ("inputs larger than L2: q+k+v %.0f MiB per rank; every step streams all %d shards' K/V "
                       "(%.0f MiB) through this GPU" % (3 * B * L * H * D * 2 / 2 ** 20, world,
                                                       2 * B * S * hkv * D * 2 / 2 ** 20))
                if getattr(op, "schedule", "ring") == "ring" else
                ("q+k+v %.0f MiB per rank; every step pulls this rank's head group of every peer's q, k, v over "
                 "NVLink again (%.0f MiB arrive per step, written by the copy engines), so no step finds its "
                 "inputs in L2 from the one before" % (3 * B * L * H * D * 2 / 2 ** 20,
                                                       (world - 1) * B * L * (H + 2 * hkv) // world * D * 2 / 2 ** 20)),
                "schedule": getattr(op, "schedule", "ring") if world > 1 else "one rank",
                "schedule_note": schedule_note,
                "host_numa": numa_note,
                "per_gpu_tflops": per_gpu,
                "buffers": "q / kv / o / lse in the op's symmetric buffers (zero-copy mode)" if world > 1 else "ordinary tensors",
                "ms_per_step_with_ordinary_tensors": ms_plain,
                "causal_balance": bool(getattr(op, "balanced", False)),
                "frac_of_bf16_peak_per_gpu": per_gpu / peak,
            },
            "e2e": {"value": e2e, "unit": "TFLOP/s", "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": (q_host.numel() + kv_host.numel()) * 2 * world,
                    "d2h_bytes_per_step": (o_host.numel() * 2 + lse_host.numel() * 4) * world},
            "fwd_bwd": {"value": 3.5 * fl_total / (ms_fb * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_fb,
                        "note": "forward + backward per step, FLOPs = 3.5 x forward (backward counted as 2.5 x)"},
            # kernels of this package inside the timed region: per step and rank one attention launch plus, on
            # more than one rank, the one-warp flag kernels of the transfer protocol (copies are copy-engine work)
            "gpu_launches": args.steps * launches_per_step * world,
            # tensor roofline of the attention launch.  At one GPU the launch is the step; at N > 1 the step is
            # one attention launch per rank whose loader waits in-kernel for shards still in flight, so the
            # figure is the per-GPU rate of the whole step (kernel + exposed transfer), not a bare kernel rate.
            "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": peak, "unit": "TFLOP/s",
                         "frac": per_gpu / peak, "traffic": NCU_DRAM_BYTES_PER_LAUNCH.get((args.workload, world)),
                         "kernel": "attn_fwd_kernel" if world == 1 else
                                   "attn_fwd_kernel, whole step per GPU incl. in-kernel waits for shard arrival",
                         "peak_kind": f"bf16_tflops burst, {peak_kind}",
                         "frac_of_sustained": (per_gpu / sustained) if sustained else None},
            "parity": parity,
            "clocks": clocks, "device_status": status,
        }
        if sustained_blk is not None:
            line["sustained"] = sustained_blk
        if extra:
            line["extra"] = extra
        if gpu_baseline is not None:
            line["gpu_baseline"] = gpu_baseline
        if per_step is not None:
            line["per_step_path"] = per_step
        if world == 1 and not args.no_cpu_baseline and not args.quick:
            tf, cores, desc, _, _ = cpu_leg(1, steps=2, warmup=1)
            line["cpu_baseline"] = {"value": tf, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": desc}
        print(json.dumps(line), flush=True)
        bad_extra = [x.get("workload") for x in extra if not x.get("parity", {}).get("ok", False)]
        if not parity["ok"] or status != 0 or bad_extra:
            print(f"bench: PARITY OR DEVICE STATUS FAILURE (headline ok={parity['ok']}, status={status}, "
                  f"failing extras={bad_extra})", file=sys.stderr, flush=True)
            rc = 3
    if world > 1:
        t = torch.tensor([rc], device=dev)
        dist.broadcast(t, 0)
        rc = int(t.item())
        dist.barrier()
        dist.destroy_process_group()
    return rc


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg2", choices=sorted(WORKLOADS))
    ap.add_argument("--schedule", default=None, choices=["ring", "heads"],
                    help="forward schedule on several GPUs (default: the library's choice for the shape)")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU leg")
    ap.add_argument("--quick", action="store_true",
                    help="headline, e2e, fwd+bwd and parity only (profiling runs): no sustained loop, no extra "
                         "workloads, no baselines")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
