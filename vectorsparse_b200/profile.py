"""Command-line harness that runs (and optionally profiles) one benchmark through this package's drivers with the
reference harness's options and CSV naming, so that its plotting scripts can read CSVs of these kernels next to
CSVs of the reference's kernels.

    python -m vectorsparse_b200.profile --bm <file.smtx | synthetic:...> -k 256 -v 8 --kernel wmma --sort \
        --job spmm --precision half [--func] [--prof [--mem]] [--ncu /path/to/ncu]

What it keeps from the reference harness (ncu_profile.py:8-122, file_name_server.py:6-45):
  * the options and their meaning; kernel -> driver selector (wmma 0, cuda 1, sputnik 2, cusparse 3; dense and
    bell through the `sparse` argument), precision -> `mixed`, sddmm_alg -> `alg`;
  * the positional driver command lines (spmm: bm k v kernel sort func sparse mixed; sddmm: bm k v kernel alg sort
    func sparse mixed);
  * the name of the CSV a profiled run writes:
        ./csv[/mem]/<job>/<bm without dataset prefix and .smtx><_kernel><_precision>[_sort][_<sddmm_alg>]_k<K>_v<V>.csv
  * the profiler flags --csv --cache-control all --profile-from-start 0 (the drivers bracket the one API call with
    cudaProfilerStart/Stop).
What differs: the profiler is always told not to touch the GPU's clocks, the drivers are the ones built in this
package, and selectors for kernels that are not built here (sputnik, cusparse, dense, bell) are passed through to
the drivers, which say so and exit.
"""
from __future__ import annotations

import argparse
import csv
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DATASET_PREFIX = "/raid/datasets/"     # the prefix the reference harness strips from benchmark paths

KERNELS = {   # name -> (driver selector, `sparse` argument, CSV suffix)
    "wmma": (0, 1, "_wmma"),
    "cuda": (1, 1, "_cuda"),
    "sputnik": (2, 1, "_sputnik"),
    "cusparse": (3, 1, "_cusparse"),
    "bell": (0, 2, "_blocked_ell"),
    "dense": (0, 0, "_dense"),
}
SDDMM_ALGS = {"wmma": 0, "mma_reg": 1, "mma_shfl": 2, "mma_arch": 3}


def _bm_stem(bm: str) -> str:
    stem = bm.replace(DATASET_PREFIX, "")
    if stem.endswith(".smtx"):
        stem = stem[:-5]
    # a synthetic pattern spec is not a path: make it one file name
    return stem.replace(":", "_").replace("=", "") if stem.startswith("synthetic:") else stem


def csv_name(bm, dimK, dimV, kernel, sort, job, sddmm_alg="mma_reg", precision="half", mem=False, root="./csv"):
    """Path of the CSV of one profiled run; same layout as file_name_server.py:6-45 of the reference."""
    suffix = KERNELS.get(kernel, KERNELS["dense"])[2]
    suffix += "_half" if precision == "half" else "_single"
    if sort:
        suffix += "_sort"
    if job != "spmm" and kernel == "wmma":
        suffix += "_%s" % sddmm_alg
    sub = os.path.join("mem", job) if mem else job
    return "%s/%s/%s_k%d_v%d.csv" % (root, sub, _bm_stem(bm) + suffix, dimK, dimV)


def driver_command(bm, dimK, dimV, kernel, sort, func, job, sddmm_alg="mma_reg", precision="half", driver_dir=None):
    """argv of the driver for one run (positional contract of spmm_benchmark.cpp:480-509, sddmm_benchmark.cpp:399-432)."""
    ker, sparse, _ = KERNELS.get(kernel, KERNELS["dense"])
    mixed = 1 if precision == "half" else 0
    d = driver_dir or os.path.join(HERE, "drivers")
    if job == "spmm":
        return [os.path.join(d, "spmm_benchmark"), bm, str(dimK), str(dimV), str(ker), str(int(bool(sort))),
                str(int(bool(func))), str(sparse), str(mixed)]
    alg = SDDMM_ALGS.get(sddmm_alg, 1)
    return [os.path.join(d, "sddmm_benchmark"), bm, str(dimK), str(dimV), str(ker), str(alg), str(int(bool(sort))),
            str(int(bool(func))), str(sparse), str(mixed)]


def profile_command(ncu, output_file, driver_argv, mem=False):
    """argv of the profiler around a driver run.  `mem` adds the L1 read-traffic counter the reference's memory
    profiles use (ncu_profile.py:85-86)."""
    cmd = [ncu, "-f", "--csv", "--clock-control", "none", "--cache-control", "all", "--profile-from-start", "0",
           "--log-file", output_file]
    if mem:
        cmd += ["--metrics", "l1tex__m_xbar2l1tex_read_bytes_mem_lg_op_ld.sum"]
    return cmd + list(driver_argv)


_TO_MS = {"second": 1e3, "msecond": 1.0, "usecond": 1e-3, "nsecond": 1e-6, "s": 1e3, "ms": 1.0, "us": 1e-3, "ns": 1e-6}


def duration_ms(csv_file):
    """Sum of the kernels' "Duration" rows of a profiler CSV, in milliseconds; None when the file has none.  (One
    benchmark run may launch several kernels — here a tensor-core SpMM is a plan kernel, the multiplying kernel and
    a fallback that returns at once — and the reference's collector adds them up the same way,
    file_name_server.py:58-82.)"""
    total, seen = 0.0, False
    with open(csv_file, newline="") as f:
        rows = [r for r in csv.reader(f) if r and not r[0].startswith("==")]
    if not rows:
        return None
    header = rows[0]
    try:
        i_name, i_unit, i_val = header.index("Metric Name"), header.index("Metric Unit"), header.index("Metric Value")
    except ValueError:
        return None
    for r in rows[1:]:
        if len(r) <= max(i_name, i_unit, i_val) or "Duration" not in r[i_name]:
            continue
        scale = _TO_MS.get(r[i_unit])
        if scale is None:
            continue
        total += float(r[i_val].replace(",", "")) * scale
        seen = True
    return total if seen else None


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="run or profile one SpMM / SDDMM benchmark")
    ap.add_argument("--ncu", default=os.environ.get("NCU_PATH", "ncu"), help="path of the profiler")
    ap.add_argument("--bm", required=True, help=".smtx pattern file or synthetic:<kind>:<m_vec>x<n>:s=<sparsity>")
    ap.add_argument("--dimK", "-k", type=int, default=256, help="width of the dense operand (SpMM) / contraction length (SDDMM)")
    ap.add_argument("--dimV", "-v", type=int, default=1, help="vector length")
    ap.add_argument("--kernel", choices=sorted(KERNELS), default="wmma")
    ap.add_argument("--sort", action="store_true", help="process vector-rows by decreasing length")
    ap.add_argument("--prof", action="store_true", help="run under the profiler and write the CSV")
    ap.add_argument("--func", action="store_true", help="compare the result with the host loop")
    ap.add_argument("--job", choices=["spmm", "sddmm"], default="spmm")
    ap.add_argument("--sddmm_alg", choices=sorted(SDDMM_ALGS), default="mma_reg")
    ap.add_argument("--precision", choices=["half", "single"], default="half")
    ap.add_argument("--mem", action="store_true", help="memory profile (L1 read traffic) instead of durations")
    ap.add_argument("--print", action="store_true", dest="show", help="print the summed kernel time of the CSV")
    ap.add_argument("--dry", action="store_true", help="print the command and do not run it")
    a = ap.parse_args(argv)

    drv = driver_command(a.bm, a.dimK, a.dimV, a.kernel, a.sort, a.func, a.job, a.sddmm_alg, a.precision)
    out = None
    cmd = drv
    if a.prof:
        out = csv_name(a.bm, a.dimK, a.dimV, a.kernel, a.sort, a.job, a.sddmm_alg, a.precision, a.mem)
        os.makedirs(os.path.dirname(out), exist_ok=True)
        cmd = profile_command(a.ncu, out, drv, a.mem)
    print(" ".join(cmd), flush=True)
    if a.dry:
        return 0
    rc = subprocess.call(cmd)
    if rc == 0 and out and a.show:
        print("%s: %s ms" % (out, duration_ms(out)))
    return rc


if __name__ == "__main__":
    sys.exit(main())
