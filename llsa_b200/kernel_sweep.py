"""Kernel benchmark over image sizes -- the counterpart of the reference's test_kernel.py:27-58.

Same sweep (size x size tokens for size in 128, 256, 512; B=2, H=4, D=64, bf16, N(0,1) inputs;
llsa_l1 and llsa_l2 with block 16, top-8), forward only and forward + backward, median / 20 % / 80 %
quantiles of CUDA-event times like triton.testing.do_bench, plus tokens/s and the effective TFLOP/s
(4 FLOP per query row, attended key and channel forward, 14 forward + backward).

    python -m llsa_b200.kernel_sweep [--sizes 128 256 512] [--reps 30] [--json]
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes", type=int, nargs="+", default=[128, 256, 512])
    ap.add_argument("--reps", type=int, default=30)
    ap.add_argument("--json", action="store_true")
    args = ap.parse_args()
    dev = torch.device("cuda", torch.cuda.current_device())
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
