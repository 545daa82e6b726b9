"""Kernel benchmark over image sizes -- the counterpart of the reference's test_kernel.py:27-58.

Same sweep (size x size tokens for size in 128, 256, 512; B=2, H=4, D=64, bf16, N(0,1) inputs;
llsa_l1 and llsa_l2 with block 16, top-8), forward only and forward + backward, median / 20 % / 80 %
quantiles of CUDA-event times like triton.testing.do_bench, plus tokens/s and the effective TFLOP/s
(4 FLOP per query row, attended key and channel forward, 14 forward + backward).

    python -m llsa_b200.kernel_sweep [--sizes 128 256 512] [--reps 30] [--json]
    python -m llsa_b200.kernel_sweep --mma-rate      # issue rate of mma.sync.m16n8k16, the ceiling of the fine-block kernels
"""
import argparse
import json

import torch

from . import llsa_l1, llsa_l2


def attended_keys(op: str, n: int) -> int:
    """Keys per query row: 8 fine blocks + pooled stages (a stage with fewer than 64 keys is skipped)."""
    n1, n2 = n // 16, n // 256
    if op == "l1":
        return 128 + (n1 if n1 >= 64 else 0)
    return 128 + 128 + (n2 if n2 >= 64 else 0)


def time_call(fn, reps: int, flush: torch.Tensor):
    for _ in range(3):
        fn()
    ts = []
    for _ in range(reps):
        flush.zero_()                                   # 256 MB write: nothing of the last run stays in the 126 MB L2
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    q = lambda f: ts[min(len(ts) - 1, int(f * len(ts)))]
    return q(0.5), q(0.2), q(0.8)


def mma_rate(dev) -> list:
    """Cycles per mma.sync.m16n8k16 (bf16) per SM sub-partition for 1..32 warps per SM and 1..8 independent chains, and the
    whole-GPU rate that the best of them implies at the current SM clock."""
    import ctypes as C

    from . import _lib
    props = torch.cuda.get_device_properties(dev)
    sms = props.multi_processor_count
    sink = torch.empty(sms * 1024, dtype=torch.float32, device=dev)
    cyc = torch.zeros(1, dtype=torch.int64, device=dev)
    iters, rows = 2000, []
    stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    for warps in (1, 4, 8, 12, 16, 32):
        for ilp in (1, 2, 4, 8):
            for _ in range(2):
                _lib.check(_lib.lib().llsa_probe_mma_rate(warps, ilp, iters, sms, C.c_void_p(sink.data_ptr()), C.c_void_p(cyc.data_ptr()), stream),
                           "probe_mma_rate")
            torch.cuda.synchronize(dev)
            per_smsp = float(cyc.item()) / (iters * ilp * max(warps, 4) / 4)
            rows.append(dict(warps_per_sm=warps, ilp=ilp, cycles_per_mma_per_subpartition=per_smsp))
    best = min(r["cycles_per_mma_per_subpartition"] for r in rows)
    try:
        mhz = int(torch.cuda.clock_rate(dev))           # current SM clock (NVML); 0 if it cannot be read
    except Exception:
        mhz = 0
    for r in rows:
        r["gpu_tflops_at_sm_clock"] = sms * 4 * (2 * 16 * 8 * 16) / r["cycles_per_mma_per_subpartition"] * mhz * 1e6 / 1e12 if mhz else None
    rows.append(dict(best_cycles=best, sms=sms, sm_mhz=mhz))
    return rows


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mma-rate", action="store_true", help="measure the issue rate of mma.sync.m16n8k16 instead of the operator sweep")
    ap.add_argument("--sizes", type=int, nargs="+", default=[128, 256, 512])
    ap.add_argument("--reps", type=int, default=30)
    ap.add_argument("--json", action="store_true")
    args = ap.parse_args()
    dev = torch.device("cuda", torch.cuda.current_device())
    if args.mma_rate:
        for r in mma_rate(dev):
            print(json.dumps(r))
        return
    B, H, D = 2, 4, 64
    flush = torch.empty(64 * 1024 * 1024, dtype=torch.float32, device=dev)
    rows = []
    for size in args.sizes:
        n = size * size
        g = torch.Generator(device="cpu").manual_seed(size)
        q, k, v, do = [torch.randn(B, H, n, D, generator=g).to(torch.bfloat16).to(dev) for _ in range(4)]
        for op, fn in (("l1", lambda a, b, c: llsa_l1(a, b, c, 8, 16)), ("l2", lambda a, b, c: llsa_l2(a, b, c, 8, 8, 16))):
            keys = attended_keys(op, n)
            for mode in ("fwd", "fwd+bwd"):
                if mode == "fwd":
                    def run():
                        with torch.no_grad():
                            fn(q, k, v)
                else:
                    qg, kg, vg = [t.detach().requires_grad_(True) for t in (q, k, v)]

                    def run():
                        qg.grad = kg.grad = vg.grad = None
                        fn(qg, kg, vg).backward(do)
                ms, lo, hi = time_call(run, args.reps, flush)
                flops = (4 if mode == "fwd" else 14) * B * H * n * keys * D
                rows.append(dict(size=size, tokens=n, op="llsa_" + op, mode=mode, ms=ms, ms_q20=lo, ms_q80=hi,
                                 tokens_per_s=B * n / (ms * 1e-3), tflops=flops / (ms * 1e-3) / 1e12, keys_per_row=keys))
    if args.json:
        print(json.dumps(rows))
        return
    print("%5s %8s %8s %8s %9s %9s %9s %12s %8s" % ("size", "tokens", "op", "mode", "ms", "q20", "q80", "tokens/s", "TFLOP/s"))
    for r in rows:
        print("%5d %8d %8s %8s %9.3f %9.3f %9.3f %12.3e %8.1f" % (r["size"], r["tokens"], r["op"], r["mode"], r["ms"], r["ms_q20"], r["ms_q80"],
                                                                   r["tokens_per_s"], r["tflops"]))


if __name__ == "__main__":
    main()
