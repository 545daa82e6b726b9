"""Turns an ncu report of the benchmark's kernels into the figures the repository keeps.

    ncu -i REPORT.ncu-rep --page raw --csv > raw.csv
    python -m llsa_b200.ncu_summary raw.csv --slices 12 [--json profiles/ncu_dram_bytes.json] [--table]

--json writes, per kernel group of bench.py (attn_fwd, attn_bwd_dq, attn_bwd_dkv_pooled, attn_bwd_dkv_fine, ...),
the DRAM bytes of one launch (dram__bytes_read.sum + dram__bytes_write.sum, mean over the captured launches) at the
captured number of (b,h) slices, together with a hash of the kernel sources the capture was taken from; bench.py
scales them to its launch and prints `traffic: null` when the sources have changed since.
--table prints the per-kernel table (time, DRAM bytes, tensor pipe, L1/TEX, L2, warps, issue, registers) as markdown.
"""
import argparse
import csv
import hashlib
import json
import os

GROUPS = {
    "attn_fwd": ("attn_fwd_fine8_kernel", "attn_fwd_fine_kernel", "attn_fwd_pooled_tc_kernel", "attn_fwd_pooled_loop_tc_kernel", "attn_fwd_mma_kernel"),
    "attn_bwd_dq": ("attn_dq_fine_kernel", "attn_dq_mma_kernel"),
    "attn_bwd_dkv_pooled": ("attn_bwd_pooled_tc_kernel", "attn_dkv_pooled_kernel", "attn_dq_pooled_loop_tc_kernel", "attn_dkv_pooled_loop_tc_kernel"),
    "attn_bwd_dkv_fine": ("attn_dkv_fine_ring_kernel", "attn_dkv_finish_ld_kernel"),
    "pool_pyramid": ("pool_pyramid_kernel",),
    "coarse_topk": ("coarse_topk_mma_kernel", "coarse_topk_kernel"),
    "refine_topk": ("refine_topk_kernel",),
    "transpose_indices": ("transpose_kernel",),
}
UNIT = {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9, "Tbyte": 1e12, "ns": 1e-3, "us": 1.0, "ms": 1e3, "s": 1e6}
COLS = [("time us", "gpu__time_duration.sum"), ("dram rd MB", "dram__bytes_read.sum"), ("dram wr MB", "dram__bytes_write.sum"),
        ("tensor pipe %", "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active"),
        ("L1/TEX %", "l1tex__throughput.avg.pct_of_peak_sustained_active"), ("L2 %", "lts__throughput.avg.pct_of_peak_sustained_elapsed"),
        ("warps active %", "sm__warps_active.avg.pct_of_peak_sustained_active"), ("issue active %", "sm__inst_issued.avg.pct_of_peak_sustained_active"),
        ("regs", "launch__registers_per_thread")]


def kernel_source_hash() -> str:
    h = hashlib.sha256()
    d = os.path.join(os.path.dirname(os.path.abspath(__file__)), "csrc")
    for name in sorted(os.listdir(d)):
        if name.endswith((".cu", ".cuh")):
            h.update(name.encode())
            h.update(open(os.path.join(d, name), "rb").read())
    return h.hexdigest()[:16]


def read_raw(path):
    rows = list(csv.reader(open(path)))
    hdr, units, body = rows[0], rows[1], rows[2:]
    col = {name: i for i, name in enumerate(hdr)}

    def val(r, name):
        if name not in col or r[col[name]] in ("", "n/a"):
            return None
        x = float(r[col[name]].replace(",", ""))
        return x * UNIT.get(units[col[name]], 1.0)

    out = []
    for r in body:
        short = r[col["Kernel Name"]].split("(")[0].split("<")[0].split("::")[-1].split()[-1]
        out.append(dict(name=short, full=r[col["Kernel Name"]], get=lambda n, r=r: val(r, n)))
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("raw_csv")
    ap.add_argument("--slices", type=int, required=True, help="(b,h) slices of the captured launch")
    ap.add_argument("--json", default=None)
    ap.add_argument("--table", action="store_true")
    args = ap.parse_args()
    launches = read_raw(args.raw_csv)
    per = {}
    for k in launches:
        per.setdefault(k["name"], []).append(k)
    if args.table:
        print("| kernel | launches | " + " | ".join(c for c, _ in COLS) + " |")
        print("|---|---|" + "---|" * len(COLS))
        for name, ks in per.items():
            cells = []
            for label, metric in COLS:
                xs = [k["get"](metric) for k in ks if k["get"](metric) is not None]
                if not xs:
                    cells.append("-")
                    continue
                m = sum(xs) / len(xs)
                cells.append("%.1f" % (m / 1e6 if "MB" in label else m))
            print("| %s | %d | %s |" % (name, len(ks), " | ".join(cells)))
    if args.json:
        groups = {}
        for g, names in GROUPS.items():
            tot = 0.0
            for name in names:
                ks = per.get(name, [])
                if ks:
                    tot += sum((k["get"]("dram__bytes_read.sum") or 0.0) + (k["get"]("dram__bytes_write.sum") or 0.0) for k in ks) / len(ks)
            if tot:
                groups[g] = tot
        with open(args.json, "w") as f:
            json.dump(dict(slices=args.slices, kernel_source_hash=kernel_source_hash(), groups=groups,
                           kernels={n: len(ks) for n, ks in per.items()},
                           how="mean per launch of dram__bytes_read.sum + dram__bytes_write.sum, summed over the kernels of a group"), f, indent=1)
            f.write("\n")
        print("wrote %s" % args.json)


if __name__ == "__main__":
    main()
