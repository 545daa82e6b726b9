#!/usr/bin/env python
"""Benchmark of the LLSA hot path: llsa_l2 forward + backward, bf16.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config cfg3]
    python bench.py --sweep [--with-reference DIR]      # the reference's own kernel benchmark shapes, one table

A step is one llsa_l2 forward+backward over the workload B=8, H=6, N=16384, D=64, block 16, top-8 at both levels
(q, k, v and the upstream gradient synthetic).  With N GPUs the ONE workload is split along the flattened
(batch, head) axis -- 48 slices, 48/N per rank, no collective on the data path -- so the value is strong scaling:
tokens of the workload / the slowest rank's time, timed on the device (CUDA events) between two barriers.

Timing: W warm-up steps, then windows of exactly K steps each (every window bracketed by CUDA events) are repeated
until at least one second has been timed; the reported ms_per_step is the median window / K.  The timed steps replay
one CUDA graph of the forward + backward (what a training loop that captures its step does); a second pass of K eager
steps with CUDA events around every kernel group gives kernel_ms and the roofline of the largest kernel.

Prints one JSON line (rank 0) with
  value      tokens/s with inputs resident in HBM
  e2e        tokens/s through the public host-operand call, pinned host buffers, copies included
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
KERNELS_PER_STEP = ("pool_pyramid_kernel", "refine_topk_kernel", "attn_fwd_fine8_kernel", "attn_fwd_pooled_tc_kernel",
                    "transpose_kernel", "attn_bwd_pooled_tc_kernel",
                    "attn_dq_fine_kernel", "attn_dkv_fine_ring_kernel", "attn_dkv_finish_ld_kernel")


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="cfg3")
    ap.add_argument("--batch", type=int, default=0, help="override the batch (profiling a smaller case)")
    ap.add_argument("--heads", type=int, default=0, help="override the head count (profiling a smaller case)")
    ap.add_argument("--seq-parallel", action="store_true", help="shard the sequence over the ranks even if B*H >= ranks")
    ap.add_argument("--min-seconds", type=float, default=1.0, help="repeat the K-step window until this much has been timed")
    ap.add_argument("--eager", action="store_true", help="time eager launches instead of replaying a CUDA graph of the step")
    ap.add_argument("--weak", action="store_true", help="also time the weak-scaling form (every rank the whole workload) as an extra key")
    ap.add_argument("--e2e-chunk-batch", type=int, default=1, help="batch elements per chunk of the host-operand pipeline")
    ap.add_argument("--e2e-chunk-heads", type=int, default=0, help="heads per chunk (with --e2e-chunk-batch 1; 0: whole batch elements)")
    ap.add_argument("--e2e-graphs", type=int, default=1, help="1: one CUDA graph per staging slot replays a chunk's fwd+bwd; 0: eager launches")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--sweep", action="store_true", help="the reference benchmark's shapes (test_kernel.py:27-58) as one table")
    ap.add_argument("--with-reference", default=None, help="--sweep: directory holding the reference's `llsa` package (Triton column)")
    ap.add_argument("--sweep-out", default=None, help="--sweep: also write the table to this file")
    return ap.parse_args()


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"], bf16_tflops_sustained=d.get("bf16_tflops_sustained"), src="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, src="fallback")


def load_ncu_traffic():
    """DRAM bytes per launch group from the committed ncu capture (profiles/ncu_dram_bytes.json, written by
    `python -m llsa_b200.ncu_summary`): {group: bytes at `slices` (b,h) slices}.  None when the capture was taken from
    other kernel sources than the ones being timed."""
    p = os.path.join(ROOT, "profiles", "ncu_dram_bytes.json")
    if not os.path.exists(p):
        return None, "no capture committed"
    from llsa_b200.ncu_summary import kernel_source_hash
    d = json.load(open(p))
    if d.get("kernel_source_hash") != kernel_source_hash():
        return None, "capture of other kernel sources (%s)" % d.get("kernel_source_hash")
    return d, "profiles/ncu_dram_bytes.json (ncu dram__bytes_read.sum + dram__bytes_write.sum at %d slices, scaled by slices)" % d["slices"]


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
    for _ in range(min(args.steps, 20)):       # bounded: a step is 0.2 s of CPU work
        dt, N = cpu_reference_sample(args.config, heads)
        ts.append(dt)
    t = sum(ts) / len(ts)
    value = N / t   # tokens = B*N with B = 1 in the sample
    sample = "one step = B=1 (6 of the 48 (b,h) slices) of the workload, fwd+bwd, fp32 math on bf16 inputs; %d steps timed" % len(ts)
    print(json.dumps(dict(
        impl="reference", metric=METRIC, value=value, unit="tokens/s", n_gpus=args.gpus, steps=args.steps, warmup=args.warmup,
        ms_per_step=t * 1e3, higher_is_better=True, scaling="strong", vs_baseline=None, dtype="bf16", data="synthetic",
        config=dict(workload="cfg3: llsa_l2 fwd+bwd bf16 B=8 H=6 N=16384 D=64 block=16 topk=8/8", sample=sample),
        cpu_baseline=dict(value=value, unit="tokens/s", cores=cores, kind="port", sample=sample),
        e2e=dict(value=value, unit="tokens/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0))), flush=True)


def median(xs):
    xs = sorted(xs)
    return xs[len(xs) // 2]


def timed_windows(step_fn, steps, min_seconds, world, dev, max_windows=400):
    """Windows of exactly `steps` calls of step_fn, each between two CUDA events, until min_seconds have been timed on
    this rank (all ranks run the same number of windows: the count is agreed on after the first window).  Returns the
    per-window milliseconds (max over ranks per window)."""
    import torch.distributed as dist

    def one():
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(steps):
            step_fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)

    first = one()
    n = int(min(max_windows, max(3, min_seconds * 1e3 / max(first, 1e-3) + 1)))
    if world > 1:
        t = torch.tensor([n], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        n = int(t.item())
    ms = [first] + [one() for _ in range(n - 1)]
    if world > 1:
        t = torch.tensor(ms, device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = [float(x) for x in t.tolist()]
    return ms


def run_sweep(args):
    """The reference benchmark's sweep (test_kernel.py:27-58) plus the headline shape, with the reference's Triton
    operators on the same GPU when a directory holding them is given, and the CPU oracle as a further column."""
    from llsa_b200 import kernel_sweep, synth
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    reference, why = (None, None)
    if args.with_reference:
        reference, why = kernel_sweep.load_reference(args.with_reference)
    rows = kernel_sweep.sweep([128, 256, 512], 20, dev, reference)
    # the headline shape (BASELINE config 3) with its correlated inputs
    cfg = synth.CONFIGS["cfg3"]
    rows += [dict(r, config="cfg3") for r in kernel_sweep.sweep(
        [128], 20, dev, reference, shapes={128: (cfg["B"], cfg["H"])},
        make_inputs=lambda size, B, H, n: synth.correlated_qkv(cfg["seed"], B, H, n, 64, dtype=torch.bfloat16)) if r["op"] == "llsa_l2"]
    if not args.no_cpu:
        from oracle import llsa_oracle as O
        cores = os.cpu_count() or 1
        torch.set_num_threads(cores)
        cache = {}
        for r in rows:
            if r["mode"] != "fwd+bwd" or r["size"] > 128:
                continue                                  # bounded: the CPU column is filled at 128 x 128 tokens only
            key = (r["op"], r["size"])
            if key not in cache:
                q, k, v, do = synth.gaussian_qkv(r["size"], 1, 2, r["tokens"], 64, dtype=torch.bfloat16)
                fn = O.llsa_l1_fwd_bwd if r["op"] == "llsa_l1" else O.llsa_l2_fwd_bwd
                fn(q[:, :1], k[:, :1], v[:, :1], do[:, :1])
                t0 = time.perf_counter()
                fn(q, k, v, do)
                cache[key] = r["tokens"] * 2 / (time.perf_counter() - t0) / r["H"]       # tokens/s of a B x H problem: per-slice rate / H
            r["cpu_tokens_per_s"], r["cpu_cores"] = cache[key], cores
    text = kernel_sweep.format_rows(rows)
    if args.with_reference and reference is None:
        text = "reference Triton operators unavailable on this box: %s\n" % why + text
    print(text)
    if args.sweep_out:
        with open(args.sweep_out, "w") as f:
            f.write(text + "\n")
            f.write(json.dumps(rows) + "\n")


def main():
    args = parse()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.sweep:
        if rank == 0:
            run_sweep(args)
        return
    import torch.distributed as dist
    import llsa_b200
    from llsa_b200 import ops, shard, synth

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    cfg = synth.CONFIGS[args.config]
    B, H, N, D = args.batch or cfg["B"], args.heads or cfg["H"], cfg["N"], cfg["D"]
    fn = llsa_b200.llsa_l2 if cfg["op"] == "llsa_l2" else llsa_b200.llsa_l1
    call = (lambda q, k, v: fn(q, k, v, 8, 8, 16)) if cfg["op"] == "llsa_l2" else (lambda q, k, v: fn(q, k, v, 8, 16))
    if cfg["rope"]:      # the model's 2-D RoPE on q and k, fused into the pooling pass (rope_dit_transformer_2d.py:232-241)
        import math
        table = synth.rope_table_2d(int(round(math.sqrt(N))), dtype=cfg["dtype"]).to(dev)
        call = lambda q, k, v: llsa_b200.llsa_l1_rope(q, k, v, table, 8, 16)

    # Default: (b,h) slices over the ranks, no collective -- also when they do not go round (6 slices on 4 ranks run 2-2-1-1, on 8
    # ranks two ranks idle: measured faster than sharding the sequence, whose exchange costs more than the imbalance).
    # --seq-parallel: groups of ranks share slices and shard the sequence inside a group (llsa_b200/seqpar.py).
    seq_parallel = args.seq_parallel
    full = synth.correlated_qkv(cfg["seed"], B, H, N, D, dtype=cfg["dtype"])          # the ONE workload, the same on every rank
    idle = False
    if seq_parallel:
        # rank r owns tokens [r*N/W, (r+1)*N/W) of q, k, v (llsa_b200/seqpar.py)
        # (b,h) slices are split over groups of ranks first; inside a group rank r owns tokens [r*N/R, (r+1)*N/R)
        from llsa_b200 import seqpar
        grp, rpg, sr, pg = seqpar.make_head_group(B * H, world, rank)
        n_grp = B * H // (world // rpg)
        n_loc = N // rpg
        hq, hk, hv, hdo = [t.reshape(1, B * H, N, D)[:, grp * n_grp:(grp + 1) * n_grp, sr * n_loc:(sr + 1) * n_loc].contiguous().pin_memory()
                           for t in full]
        sp_group = pg if rpg > 1 else seqpar._ALONE
        call = lambda q, k, v: seqpar.llsa_l2_seq_parallel(q, k, v, 8, 8, 16, group=sp_group)
        n_slices = n_grp
        seq_ranks = rpg
    else:
        # rank r owns a contiguous range of the flattened (batch, head) axis: [1, slices, N, D] (llsa_b200/shard.py)
        hq, hk, hv, hdo = [shard.take_slices(t, world, rank).contiguous().pin_memory() for t in full]
        n_slices = hq.shape[1]
    idle = n_slices == 0                     # more ranks than slices: this rank only keeps the barriers company
    del full
    q, k, v, do = [t.to(dev) for t in (hq, hk, hv, hdo)]
    q.requires_grad_(True); k.requires_grad_(True); v.requires_grad_(True)

    def eager_step():
        if idle:
            return None
        q.grad = k.grad = v.grad = None
        o = call(q, k, v)
        o.backward(do)
        return o

    for _ in range(max(args.warmup, 3)):
        eager_step()
    torch.cuda.synchronize()
    use_graph = not args.eager and not seq_parallel and not idle            # collectives stay eager
    if use_graph:
        graph, _outs = llsa_b200.capture_fwd_bwd(call, q.detach(), k.detach(), v.detach(), do)
        step = graph.replay
        for _ in range(3):
            step()
        torch.cuda.synchronize()
    else:
        step = eager_step

    # ---- timed region: windows of exactly K steps until min_seconds are covered; the median window is reported
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    windows = timed_windows(step, args.steps, args.min_seconds, world, dev)
    clocks = sampler.stop() if rank == 0 else None
    ms_step = median(windows) / args.steps
    value = B * N / (ms_step * 1e-3)                           # the ONE workload's tokens over the slowest rank's time
    if idle:                                                   # the e2e leg's barrier and reduction, then out
        if not args.no_e2e and not seq_parallel:
            dist.barrier()
            dist.all_reduce(torch.zeros(1, device=dev), op=dist.ReduceOp.MAX)
        dist.destroy_process_group()
        return

    # ---- per-kernel CUDA events: K eager steps with an event in front of every kernel group (on the launching stream)
    marks = []

    def hook(name):
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        marks.append((name, ev))

    torch.cuda.synchronize()
    ops.set_stage_hook(hook)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        eager_step()
    e1.record()
    ops.set_stage_hook(None)
    torch.cuda.synchronize()
    eager_ms_step = e0.elapsed_time(e1) / args.steps
    # One more step with the device checks on (every operator then reads the kernels' status word back and raises if a
    # bounded wait ran out or a block index was out of range): a kernel that gave up a wait ends early, and a step
    # timed that way would be a wrong number that looks fast or slow, not an error.
    ops.set_device_checks(True)
    try:
        eager_step()
        torch.cuda.synchronize()
    finally:
        ops.set_device_checks(False)
    per = {}
    for (name, ev), (_, nxt) in zip(marks[:-1], marks[1:]):
        if name != "end":
            per[name] = per.get(name, 0.0) + ev.elapsed_time(nxt)
    per = {kname: max(tms, 0.0) / args.steps for kname, tms in per.items()}
    if not seq_parallel:
        seq_ranks = 1
    units = n_slices * (N // seq_ranks) * D      # query rows x channels on this rank
    if cfg["op"] == "llsa_l2":
        keys = dict(fine=128, p1=128, p2=N // 256 if N // 256 >= 64 else 0)
    else:
        keys = dict(fine=128, p1=N // 16 if N // 16 >= 64 else 0, p2=0)
    ktot = sum(keys.values())
    pooled = keys["p1"] + keys["p2"]
    if cfg["op"] == "llsa_l2" and N // 256 == 64:      # tcgen05 pooled backward: S, dP, dQ, dPK, dPV of the pooled keys in one kernel; the dQ kernel is fine-only
        flops = dict(attn_fwd=4 * units * ktot, attn_bwd_dq=6 * units * keys["fine"], attn_bwd_dkv_fine=4 * units * keys["fine"],
                     attn_bwd_dkv_pooled=10 * units * pooled)
    else:
        flops = dict(attn_fwd=4 * units * ktot, attn_bwd_dq=6 * units * ktot, attn_bwd_dkv_fine=4 * units * keys["fine"],
                     attn_bwd_dkv_pooled=4 * units * pooled)
    peaks = load_peaks()
    top = max((n for n in per if n in flops), key=lambda n: per[n])
    ach = flops[top] / (per[top] * 1e-3) / 1e12
    peak = peaks["bf16_tflops_sustained"] or peaks["bf16_tflops"]
    ncu, traffic_src = load_ncu_traffic()
    traffic = None
    if ncu is not None and args.config == "cfg3" and not seq_parallel and top in ncu["groups"]:
        traffic = ncu["groups"][top] * (n_slices / float(ncu["slices"]))
    roof = dict(kernel=top, bound="tensor", achieved=ach, peak=peak, unit="TFLOP/s", frac=ach / peak, traffic=traffic,
                traffic_source=traffic_src, peak_source=peaks["src"] + " (sustained bf16 GEMM)", ms_per_launch=per[top],
                algorithmic_flops_per_launch=flops[top])
    total_flops = 14 * B * H * N * D * ktot                    # the whole workload
    # memory-bound stages: algorithmic bytes per launch (this rank) against the measured copy bandwidth
    T = units * 2                                             # one [slices, N, D] bf16 tensor
    nq1, n2k = n_slices * (N // seq_ranks) // 16, N // 256
    alg_bytes = dict(pool_pyramid=3 * T + 3 * T * (1 / 16 + 1 / 256),
                     coarse_topk=2 * n_slices * n2k * D * 2 + n_slices * n2k * 8 * 4,
                     refine_topk=nq1 * D * 2 + (nq1 // 16) * 128 * D * 2 + nq1 * 8 * 4,
                     select_two_level=2 * n_slices * n2k * D * 2 + n_slices * n2k * 8 * 4 + nq1 * D * 2 + (nq1 // 16) * 128 * D * 2 + nq1 * 8 * 4,
                     transpose_indices=nq1 * 8 * 4 * 2 + n_slices * (N // 16 + 1) * 4)
    memory_bound = {kname: dict(bytes=int(alg_bytes[kname]), gbs=alg_bytes[kname] / (per[kname] * 1e-3) / 1e9,
                                frac_of_hbm_peak=alg_bytes[kname] / (per[kname] * 1e-3) / 1e9 / peaks["hbm_gbs"])
                    for kname in alg_bytes if per.get(kname, 0.0) > 1e-4}

    out = dict(metric=METRIC if args.config == "cfg3" else "%s fwd+bwd tokens/sec (%s)" % (cfg["op"], args.config), value=value, unit="tokens/s", n_gpus=world, steps=args.steps, warmup=max(args.warmup, 3),
               ms_per_step=ms_step, higher_is_better=True, scaling="strong", vs_baseline=None, dtype="bf16", data="synthetic",
               config=dict(workload="%s: %s fwd+bwd bf16 B=%d H=%d N=%d D=%d block=16 topk=8, ONE problem split over %d GPU(s)" % (
                               args.config, cfg["op"], B, H, N, D, world),
                           inputs="N(0,1) + 0.5*low-frequency 2-D field, Morton order, seed %d" % cfg["seed"],
                           slices_per_gpu=n_slices,
                           step_launch="one CUDA graph replay per step (forward + backward captured once)" if use_graph else "eager launches",
                           timing="median of %d windows of %d steps (%.2f s timed); min %.4f / max %.4f ms per step" % (
                               len(windows), args.steps, sum(windows) * 1e-3, min(windows) / args.steps, max(windows) / args.steps),
                           overlap="index transpose on a side stream next to the dQ / pooled backward stages (kernel_ms times it alone, on the main stream)",
                           l2_policy="no flush: a step streams %.0f MB per GPU (q, k, v, do in, o, dq, dk, dv out: 8 x %.1f MB; P / dS scratch %.0f MB), "
                                     "%s the 126 MB L2" % (8 * units * 2 / 1e6 + nq1 * 8 * 1024 / 1e6, units * 2 / 1e6, nq1 * 8 * 1024 / 1e6,
                                                           "more than" if 8 * units * 2 + nq1 * 8 * 1024 > 126e6 else "LESS than (reads may hit L2)"),
                           parallelism=("%d rank(s): %d group(s) of (b,h) slices x %d rank(s) sharding the sequence (all-gather of k, v and pooled "
                                        "levels, reduce-scatter of dk, dv inside a group)" % (world, world // seq_ranks, seq_ranks))
                           if seq_parallel else "%d rank(s), the %d (batch, head) slices split contiguously%s, no collective"
                           % (world, B * H, " (%d rank(s) without a slice)" % (world - B * H) if world > B * H else "")),
               windows=len(windows), eager_ms_per_step=eager_ms_step,
               effective_tflops=total_flops / (ms_step * 1e-3) / 1e12,
               effective_tflops_frac_of_bf16_peak=total_flops / (ms_step * 1e-3) / 1e12 / (peak * world),
               kernel_ms={kname: round(tms, 4) for kname, tms in sorted(per.items())},
               memory_bound_stages=memory_bound, hbm_peak_gbs=peaks["hbm_gbs"],
               roofline=roof, gpu_launches=len(KERNELS_PER_STEP) * args.steps, clocks=clocks,
               device_checks="one eager step with the kernels' status word read back after every operator: clean")

    # ---- weak-scaling form as an extra key: every rank the whole workload (what data-parallel training does)
    if args.weak and world > 1 and not seq_parallel and world <= B * H:
        wq, wk, wv, wdo = [t.to(dev) for t in synth.correlated_qkv(cfg["seed"] + 100 * rank, B, H, N, D, dtype=cfg["dtype"])]
        wgraph, _w = llsa_b200.capture_fwd_bwd(call, wq, wk, wv, wdo)
        for _ in range(3):
            wgraph.replay()
        wms = median(timed_windows(wgraph.replay, args.steps, args.min_seconds, world, dev)) / args.steps
        out["weak_scaling"] = dict(value=world * B * N / (wms * 1e-3), unit="tokens/s", ms_per_step=wms,
                                   note="every rank its own B=%d batch; N x per-rank tokens / slowest rank" % B)
        del wq, wk, wv, wdo, wgraph, _w

    # ---- end to end: pinned host buffers -> device -> fwd+bwd -> o, dq, dk, dv back to the host
    if not args.no_e2e and not seq_parallel:
        from llsa_b200.hostpipe import HostPipeline
        ho = torch.empty_like(hq).pin_memory()
        hdq, hdk, hdv = [torch.empty_like(hq).pin_memory() for _ in range(3)]
        sb, sh = hq.shape[0], hq.shape[1]
        chunk_heads = args.e2e_chunk_heads or (6 if (sb == 1 and sh % 6 == 0) else None)
        pipe = HostPipeline(call, (sb, sh, N, D), cfg["dtype"], dev, chunk_batch=args.e2e_chunk_batch, chunk_heads=chunk_heads,
                            graphs=bool(args.e2e_graphs))

        def e2e_step():
            # the public host-operand call: per chunk copy-in, fwd+bwd and copy-out overlap on three streams
            pipe.fwd_bwd(hq, hk, hv, hdo, ho, hdq, hdk, hdv)

        n_e2e = max(50, min(args.steps, 100))
        for _ in range(3):
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
        out["e2e"] = dict(value=B * N / (ems / n_e2e * 1e-3), unit="tokens/s", h2d_bytes_per_step=4 * nbytes,
                          d2h_bytes_per_step=4 * nbytes, ms_per_step=ems / n_e2e, steps=n_e2e,
                          note="bytes are per rank; every rank copies its own slices in and out")

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
