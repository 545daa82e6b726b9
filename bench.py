#!/usr/bin/env python
"""Benchmark of the LLSA hot path: llsa_l2 forward + backward, bf16.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config cfg3]

A step is one llsa_l2 forward+backward over one batch of synthetic q, k, v and
upstream gradient: per GPU the shape B=8, H=6, N=16384, D=64, block 16, top-8 at
both levels.  With N GPUs every rank runs its own batch (the (batch, head) axis
is embarrassingly parallel: no collective on the data path), so the whole-job
value is N * per-rank tokens per second, timed on the device (CUDA events) as
the maximum over ranks between two barriers.

Prints one JSON line (rank 0) with
  value      tokens/s with inputs resident in HBM
  e2e        tokens/s through the public API from pinned host buffers, copies included
  roofline   achieved vs measured peak of the kernel with the largest share of the step
  cpu_baseline  the CPU oracle (a port of the reference algorithm) on a bounded sample
`--impl reference` times only the CPU implementation of the reference algorithm.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "llsa_l2 fwd+bwd tokens/sec @N=16384,B*H=48,D=64"


# this library's kernels launched by one llsa_l2 forward + backward (torch's own zero fills are not counted)
KERNELS_PER_STEP = ("pool_pyramid_kernel", "coarse_topk_mma_kernel", "refine_topk_kernel", "attn_fwd_fine8_kernel", "attn_fwd_pooled_tc_kernel",
                    "transpose_kernel", "attn_bwd_pooled_tc_kernel",
                    "attn_dq_fine_kernel", "attn_dkv_fine_ring_kernel", "attn_dkv_finish_ld_kernel")


# DRAM read + write bytes of one launch on 12 (b,h) slices of the config-3 shape, from the ncu capture summarised in
# profiles/attention_kernels_llsa_l2_batch2.md (dram__bytes_read.sum + dram__bytes_write.sum); traffic grows in
# proportion to the slices (every slice is independent), so a full launch is scaled by B*H / 12.
NCU_DRAM_BYTES_12_SLICES = dict(attn_fwd=(49.5 + 2.7 + 54.0 + 0.2) * 1e6, attn_bwd_dq=(100.6 + 11.1) * 1e6,
                                attn_bwd_dkv_pooled=(85.6 + 4.4) * 1e6, attn_bwd_dkv_fine=(89.1 + 14.7 + 15.7 + 0.1) * 1e6)


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="cfg3")
    ap.add_argument("--batch", type=int, default=0, help="override the per-GPU batch (profiling a smaller case)")
    ap.add_argument("--seq-parallel", action="store_true", help="shard the sequence over the ranks even if B*H >= ranks")
    ap.add_argument("--e2e-chunk-batch", type=int, default=1, help="batch elements per chunk of the host-operand pipeline")
    ap.add_argument("--e2e-chunk-heads", type=int, default=0, help="heads per chunk (with --e2e-chunk-batch 1; 0: whole batch elements)")
    ap.add_argument("--e2e-graphs", type=int, default=1, help="1: one CUDA graph per staging slot replays a chunk's fwd+bwd; 0: eager launches")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    return ap.parse_args()


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"], bf16_tflops_sustained=d.get("bf16_tflops_sustained"), src="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, src="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        time.sleep(0.15)
        self.proc.terminate()
        mhz = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = max([int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()] or [0])
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for r in self.rows if len(r) >= 6 for i in range(4) if r[2 + i].lower().startswith("active")})
        return dict(sm_mhz=mhz[len(mhz) // 2] if mhz else None, sm_max_mhz=mx or None, reasons=reasons, samples=len(mhz))


def cpu_reference_sample(cfg, heads):
    """One forward+backward of the CPU oracle on B=1, `heads` heads of the workload; returns seconds."""
    from oracle import llsa_oracle as O
    from llsa_b200 import synth
    q, k, v, do, _ = synth.make_config_inputs(cfg, B=1, H=heads)
    t0 = time.perf_counter()
    O.llsa_l2_fwd_bwd(q, k, v, do)
    return time.perf_counter() - t0, q.shape[2]


def run_reference(args, rank):
    """The reference algorithm on the host cores (the CPU oracle, a port: the reference's own
    kernels are Triton and have no CPU build other than the interpreter)."""
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    heads = 6
    for _ in range(max(args.warmup, 1) if args.warmup < 2 else 1):
        cpu_reference_sample(args.config, heads)
    ts = []
    for _ in range(args.steps):
        dt, N = cpu_reference_sample(args.config, heads)
        ts.append(dt)
    t = sum(ts) / len(ts)
    value = N / t   # tokens = B*N with B = 1 in the sample
    sample = "one step = B=1 (6 of the 48 (b,h) slices) of the workload, fwd+bwd, fp32 math on bf16 inputs"
    print(json.dumps(dict(
        impl="reference", metric=METRIC, value=value, unit="tokens/s", n_gpus=args.gpus, steps=args.steps, warmup=args.warmup,
        ms_per_step=t * 1e3, higher_is_better=True, scaling="weak", vs_baseline=None, dtype="bf16", data="synthetic",
        config=dict(workload="cfg3: llsa_l2 fwd+bwd bf16 B=8 H=6 N=16384 D=64 block=16 topk=8/8", sample=sample),
        cpu_baseline=dict(value=value, unit="tokens/s", cores=cores, kind="port", sample=sample),
        e2e=dict(value=value, unit="tokens/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0))), flush=True)


def main():
    args = parse()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    import torch.distributed as dist
    import llsa_b200
    from llsa_b200 import ops, synth

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    cfg = synth.CONFIGS[args.config]
    B, H, N, D = args.batch or cfg["B"], cfg["H"], cfg["N"], cfg["D"]
    fn = llsa_b200.llsa_l2 if cfg["op"] == "llsa_l2" else llsa_b200.llsa_l1
    call = (lambda q, k, v: fn(q, k, v, 8, 8, 16)) if cfg["op"] == "llsa_l2" else (lambda q, k, v: fn(q, k, v, 8, 16))

    seq_parallel = B * H < world or args.seq_parallel          # too few (b,h) slices to go round: shard the sequence
    if seq_parallel:
        # strong scaling: ONE problem, rank r owns tokens [r*N/W, (r+1)*N/W) of q, k, v (llsa_b200/seqpar.py)
        from llsa_b200 import seqpar
        n_loc = N // world
        full = synth.correlated_qkv(cfg["seed"], B, H, N, D, dtype=cfg["dtype"])
        hq, hk, hv, hdo = [t[:, :, rank * n_loc:(rank + 1) * n_loc].contiguous().pin_memory() for t in full]
        del full
        call = lambda q, k, v: seqpar.llsa_l2_seq_parallel(q, k, v, 8, 8, 16)
    else:
        # every rank owns its own batch (seed offset by rank); host tensors are pinned for the e2e leg
        hq, hk, hv, hdo = [t.pin_memory() for t in synth.correlated_qkv(cfg["seed"] + 100 * rank, B, H, N, D, dtype=cfg["dtype"])]
    q, k, v, do = [t.to(dev) for t in (hq, hk, hv, hdo)]
    q.requires_grad_(True); k.requires_grad_(True); v.requires_grad_(True)

    def step():
        q.grad = k.grad = v.grad = None
        o = call(q, k, v)
        o.backward(do)
        return o

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()

    # ---- timed region: K steps, per-kernel CUDA events on the launching stream
    marks = []

    def hook(name):
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        marks.append((name, ev))

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ops.set_stage_hook(hook)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    ops.set_stage_hook(None)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    clocks = sampler.stop() if rank == 0 else None
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_step = ms / args.steps
    jobs = 1 if seq_parallel else world          # problems of B*N tokens finished per step
    value = jobs * B * N / (ms_step * 1e-3)

    # per-kernel durations from the event marks
    per = {}
    for (name, ev), (_, nxt) in zip(marks[:-1], marks[1:]):
        if name != "end":
            per[name] = per.get(name, 0.0) + ev.elapsed_time(nxt)
    per = {kname: max(tms, 0.0) / args.steps for kname, tms in per.items()}    # a stage moved to a side stream shows ~0 here
    units = B * H * (N // world if seq_parallel else N) * D      # query rows x channels on this rank
    keys = dict(fine=128, p1=128, p2=N // 256 if N // 256 >= 64 else 0)
    ktot = sum(keys.values())
    pooled = keys["p1"] + keys["p2"]
    if N // 256 == 64:      # tcgen05 pooled backward: S, dP, dQ, dPK, dPV of the pooled keys in one kernel; the dQ kernel is fine-only
        flops = dict(attn_fwd=4 * units * ktot, attn_bwd_dq=6 * units * keys["fine"], attn_bwd_dkv_fine=4 * units * keys["fine"],
                     attn_bwd_dkv_pooled=10 * units * pooled)
    else:
        flops = dict(attn_fwd=4 * units * ktot, attn_bwd_dq=6 * units * ktot, attn_bwd_dkv_fine=4 * units * keys["fine"],
                     attn_bwd_dkv_pooled=4 * units * pooled)
    peaks = load_peaks()
    top = max((n for n in per if n in flops), key=lambda n: per[n])
    ach = flops[top] / (per[top] * 1e-3) / 1e12
    peak = peaks["bf16_tflops_sustained"] or peaks["bf16_tflops"]
    traffic = NCU_DRAM_BYTES_12_SLICES[top] * (B * H / 12.0) if (args.config == "cfg3" and not seq_parallel) else None
    roof = dict(kernel=top, bound="tensor", achieved=ach, peak=peak, unit="TFLOP/s", frac=ach / peak, traffic=traffic,
                traffic_source="ncu dram bytes of a 12-slice capture scaled to this launch (profiles/attention_kernels_llsa_l2_batch2.md)",
                peak_source=peaks["src"] + " (sustained bf16 GEMM)", ms_per_launch=per[top],
                algorithmic_flops_per_launch=flops[top])
    total_flops = 14 * units * ktot
    # memory-bound stages: algorithmic bytes per launch (this rank) against the measured copy bandwidth
    T = units * 2                                             # one [B,H,N,D] bf16 tensor
    nq1, n2k = B * H * (N // world if seq_parallel else N) // 16, N // 256
    alg_bytes = dict(pool_pyramid=3 * T + 3 * T * (1 / 16 + 1 / 256),
                     coarse_topk=2 * B * H * n2k * D * 2 + B * H * n2k * 8 * 4,
                     refine_topk=nq1 * D * 2 + (nq1 // 16) * 128 * D * 2 + nq1 * 8 * 4,
                     transpose_indices=nq1 * 8 * 4 * 2 + B * H * (N // 16 + 1) * 4)
    memory_bound = {kname: dict(bytes=int(alg_bytes[kname]), gbs=alg_bytes[kname] / (per[kname] * 1e-3) / 1e9,
                                frac_of_hbm_peak=alg_bytes[kname] / (per[kname] * 1e-3) / 1e9 / peaks["hbm_gbs"])
                    for kname in alg_bytes if per.get(kname, 0.0) > 1e-4}

    out = dict(metric=METRIC, value=value, unit="tokens/s", n_gpus=world, steps=args.steps, warmup=max(args.warmup, 3),
               ms_per_step=ms_step, higher_is_better=True, scaling="strong" if seq_parallel else "weak", vs_baseline=None, dtype="bf16", data="synthetic",
               config=dict(workload="%s: %s fwd+bwd bf16 B=%d H=%d N=%d D=%d block=16 topk=8/8 per GPU" % (args.config, cfg["op"], B, H, N, D),
                           inputs="N(0,1) + 0.5*low-frequency 2-D field, Morton order, seed %d+100*rank" % cfg["seed"],
                           overlap="index transpose on a side stream next to the dQ / pooled backward stages (its kernel_ms entry is ~0)",
                           l2_policy="inputs (4 x %.0f MB per step) exceed the 126 MB L2" % (units * 2 / 1e6),
                           parallelism=("%d rank(s), sequence sharded: all-gather of k, v and pooled levels, reduce-scatter of dk, dv" % world)
                           if seq_parallel else "%d independent rank(s), sharded by (batch, head), no collective" % world),
               effective_tflops=total_flops * world / (ms_step * 1e-3) / 1e12,
               effective_tflops_frac_of_bf16_peak=total_flops / (ms_step * 1e-3) / 1e12 / peak,
               kernel_ms={kname: round(tms, 4) for kname, tms in sorted(per.items())},
               memory_bound_stages=memory_bound, hbm_peak_gbs=peaks["hbm_gbs"],
               roofline=roof, gpu_launches=len(KERNELS_PER_STEP) * args.steps, clocks=clocks)

    # ---- end to end: pinned host buffers -> device -> fwd+bwd -> o, dq, dk, dv back to the host
    if not args.no_e2e and not seq_parallel:
        from llsa_b200.hostpipe import HostPipeline
        ho = torch.empty_like(hq).pin_memory()
        hdq, hdk, hdv = [torch.empty_like(hq).pin_memory() for _ in range(3)]
        pipe = HostPipeline(call, (B, H, N, D), cfg["dtype"], dev, chunk_batch=args.e2e_chunk_batch, chunk_heads=args.e2e_chunk_heads or None,
                            graphs=bool(args.e2e_graphs))

        def e2e_step():
            # the public host-operand call: per batch element copy-in, fwd+bwd and copy-out overlap on three streams
            pipe.fwd_bwd(hq, hk, hv, hdo, ho, hdq, hdk, hdv)

        n_e2e = max(3, min(args.steps, 10))
        for _ in range(2):
            e2e_step()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for _ in range(n_e2e):
            e2e_step()
        s1.record()
        torch.cuda.synchronize()
        ems = s0.elapsed_time(s1)
        if world > 1:
            t = torch.tensor([ems], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ems = float(t.item())
        nbytes = hq.numel() * hq.element_size()
        out["e2e"] = dict(value=jobs * B * N / (ems / n_e2e * 1e-3), unit="tokens/s", h2d_bytes_per_step=4 * nbytes,
                          d2h_bytes_per_step=4 * nbytes, ms_per_step=ems / n_e2e, steps=n_e2e)

    # ---- CPU baseline on rank 0, N = 1 only
    if rank == 0 and world == 1 and not args.no_cpu:
        cores = os.cpu_count() or 1
        torch.set_num_threads(cores)
        cpu_reference_sample(args.config, 2)
        reps = B                   # B samples of B=1: as many (b,h) slices as the whole workload holds
        dt = sum(cpu_reference_sample(args.config, 6)[0] for _ in range(reps))
        out["cpu_baseline"] = dict(value=reps * N / dt, unit="tokens/s", cores=cores, kind="port",
                                   sample="%d x (B=1, H=6) = %d (b,h) slices, fwd+bwd of the CPU oracle, %.1f s in all" % (reps, 6 * reps, dt))
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
