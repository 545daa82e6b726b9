"""Kernel benchmark over image sizes -- the counterpart of the reference's test_kernel.py:27-58.

Same sweep (size x size tokens for size in 128, 256, 512; B=2, H=4, D=64, bf16, N(0,1) inputs;
llsa_l1 and llsa_l2 with block 16, top-8), forward only and forward + backward, median / 20 % / 80 %
quantiles of CUDA-event times like triton.testing.do_bench, plus tokens/s, the effective TFLOP/s
(4 FLOP per query row, attended key and channel forward, 14 forward + backward) and the GB/s of the
call's compulsory HBM traffic (q, k, v read and o written forward: 4 tensors; 12 forward + backward).

    python -m llsa_b200.kernel_sweep [--sizes 128 256 512] [--reps 30] [--json]
    python -m llsa_b200.kernel_sweep --with-reference DIR   # DIR holds the reference's `llsa` package

With --with-reference the reference's own Triton operators (torch_op/flash_sparse_attention_res_{1,2}.py:41-59)
are imported from DIR, timed on the same tensors in the same process, and their outputs and gradients are
compared with this library's (bf16 parity on the GPU).  If Triton cannot compile them on the device the
column reads "unavailable" with the error.  A `cpu` column is added by `bench.py --sweep`, which owns the
CPU baseline.
"""
import argparse
import json
import sys

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


def load_reference(path: str):
    """The reference's llsa_l1 / llsa_l2 from a directory that holds its `llsa` package; (fns, None) or (None, why)."""
    try:
        sys.path.insert(0, path)
        from llsa.kernel.torch_op.flash_sparse_attention_res_1 import llsa_l1 as r1
        from llsa.kernel.torch_op.flash_sparse_attention_res_2 import llsa_l2 as r2
        return dict(l1=lambda a, b, c: r1(a, b, c, 8, 16), l2=lambda a, b, c: r2(a, b, c, 8, 8, 16)), None
    except Exception as e:  # noqa: BLE001 - any import problem makes the column unavailable
        return None, "%s: %s" % (type(e).__name__, str(e).splitlines()[0] if str(e) else "")
    finally:
        if sys.path and sys.path[0] == path:
            sys.path.pop(0)


def _rel(a: torch.Tensor, b: torch.Tensor) -> float:
    return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-30))


def sweep(sizes, reps, dev, reference=None, shapes=None, make_inputs=None):
    """Rows of the table.  `shapes` maps a size to (B, H); `make_inputs(size, B, H, n)` returns q, k, v, do on the host."""
    flush = torch.empty(64 * 1024 * 1024, dtype=torch.float32, device=dev)
    ours = dict(l1=lambda a, b, c: llsa_l1(a, b, c, 8, 16), l2=lambda a, b, c: llsa_l2(a, b, c, 8, 8, 16))
    rows = []
    for size in sizes:
        n = size * size
        B, H = (shapes or {}).get(size, (2, 4))
        D = 64
        if make_inputs is not None:
            q, k, v, do = [t.to(dev) for t in make_inputs(size, B, H, n)]
        else:
            g = torch.Generator(device="cpu").manual_seed(size)
            q, k, v, do = [torch.randn(B, H, n, D, generator=g).to(torch.bfloat16).to(dev) for _ in range(4)]
        T = B * H * n * D * 2
        for op in ("l1", "l2"):
            keys = attended_keys(op, n)
            for mode in ("fwd", "fwd+bwd"):
                def make_run(fn):
                    if mode == "fwd":
                        def run():
                            with torch.no_grad():
                                return fn(q, k, v)
                        return run, None
                    qg, kg, vg = [t.detach().clone().requires_grad_(True) for t in (q, k, v)]

                    def run():
                        qg.grad = kg.grad = vg.grad = None
                        o = fn(qg, kg, vg)
                        o.backward(do)
                        return o
                    return run, (qg, kg, vg)

                run, leaves = make_run(ours[op])
                ms, lo, hi = time_call(run, reps, flush)
                flops = (4 if mode == "fwd" else 14) * B * H * n * keys * D
                nbytes = (4 if mode == "fwd" else 12) * T
                row = dict(size=size, tokens=n, B=B, H=H, op="llsa_" + op, mode=mode, ms=ms, ms_q20=lo, ms_q80=hi,
                           tokens_per_s=B * n / (ms * 1e-3), tflops=flops / (ms * 1e-3) / 1e12, gbs=nbytes / (ms * 1e-3) / 1e9,
                           keys_per_row=keys)
                if reference is not None:
                    try:
                        rrun, rleaves = make_run(reference[op])
                        rms, rlo, rhi = time_call(rrun, max(5, reps // 3), flush)
                        row.update(ref_ms=rms, ref_ms_q20=rlo, ref_ms_q80=rhi, speedup=rms / ms)
                        o_ref, o_our = rrun(), run()
                        torch.cuda.synchronize()
                        row["o_rel_l2_vs_ref"] = _rel(o_our, o_ref)
                        if leaves is not None:
                            for name, a, b in zip(("dq", "dk", "dv"), leaves, rleaves):
                                row[name + "_rel_l2_vs_ref"] = _rel(a.grad, b.grad)
                    except Exception as e:  # noqa: BLE001 - Triton failing to compile / run on this device
                        row["ref_unavailable"] = "%s: %s" % (type(e).__name__, (str(e).splitlines() or [""])[0][:200])
                rows.append(row)
    return rows


def format_rows(rows) -> str:
    has_ref = any("ref_ms" in r or "ref_unavailable" in r for r in rows)
    has_cpu = any("cpu_tokens_per_s" in r for r in rows)
    head = "%5s %8s %3s %2s %8s %8s %9s %9s %9s %12s %8s %8s" % ("size", "tokens", "B", "H", "op", "mode", "ms", "q20", "q80", "tokens/s", "TFLOP/s", "GB/s")
    if has_ref:
        head += " %10s %8s %10s %10s" % ("ref ms", "ref/ours", "o relL2", "dk relL2")
    if has_cpu:
        head += " %12s %6s" % ("cpu tok/s", "cores")
    out = [head]
    for r in rows:
        line = "%5d %8d %3d %2d %8s %8s %9.3f %9.3f %9.3f %12.3e %8.1f %8.1f" % (
            r["size"], r["tokens"], r["B"], r["H"], r["op"], r["mode"], r["ms"], r["ms_q20"], r["ms_q80"], r["tokens_per_s"], r["tflops"], r["gbs"])
        if has_ref:
            if "ref_ms" in r:
                line += " %10.3f %8.2f %10.2e %10s" % (r["ref_ms"], r["speedup"], r.get("o_rel_l2_vs_ref", float("nan")),
                                                       ("%.2e" % r["dk_rel_l2_vs_ref"]) if "dk_rel_l2_vs_ref" in r else "-")
            else:
                line += "  unavailable: %s" % r.get("ref_unavailable", "")
        if has_cpu:
            line += " %12s %6s" % (("%.3e" % r["cpu_tokens_per_s"]) if "cpu_tokens_per_s" in r else "-", r.get("cpu_cores", "-"))
        out.append(line)
    return "\n".join(out)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes", type=int, nargs="+", default=[128, 256, 512])
    ap.add_argument("--reps", type=int, default=30)
    ap.add_argument("--with-reference", default=None, help="directory that holds the reference's `llsa` package")
    ap.add_argument("--json", action="store_true")
    args = ap.parse_args()
    dev = torch.device("cuda", torch.cuda.current_device())
    reference, why = (None, None)
    if args.with_reference:
        reference, why = load_reference(args.with_reference)
        if reference is None:
            print("reference unavailable: %s" % why)
    rows = sweep(args.sizes, args.reps, dev, reference)
    print(json.dumps(rows) if args.json else format_rows(rows))


if __name__ == "__main__":
    main()
