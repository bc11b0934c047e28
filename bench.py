#!/usr/bin/env python
"""Benchmark of the column-vector sparse SpMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference|dense-library|blocked-ell] [--workload NAME]

Default workload `spmm_v8_s90`: the tensor-core SpMM (wmmaSpmm entry point) on the pruned ResNet-50 layer shape
the target is quoted on — A 2048 x 512 in CVSE with V = 8 at 90 % sparsity (Beta(2,2)-skewed rows), fp16 values
N(0, 0.02), dense B 512 x 256 fp16 N(0,1), fp32 accumulate, fp16 C.  One such product is ~54 MFLOP / 1.6 MB,
far below launch latency, so a STEP is a stream of 256 independent instances (distinct values, B and C buffers
sharing one sparsity structure, 384 MB in all, three times the L2) issued as ONE batched launch.  At N GPUs
every rank runs its own stream (weak scaling, no collective on the data path).

Metric: effective TFLOP/s = 2 * nnz * N / time, nnz = nnz_vec * V, summed over all ranks.
`roofline`: algorithmic HBM bytes per launch / CUDA-event time per launch against the measured copy bandwidth.
`e2e`: the same step through the public Python API with operands in pinned HOST memory: H2D of values and B,
the launch, D2H of C, all inside the timed region.
`--impl reference`: the reference's own CPU path (its sequential host loop) timed on this box's host cores on a
bounded sample of the same stream.
`--impl dense-library`: context only, one GPU, SpMM workloads: the sparse matrices expanded to dense fp16 once,
outside the timed region, and multiplied by the vendor library's batched GEMM (torch.bmm); answers "what would
ignoring the sparsity cost on this part".  Not a product path and not part of any other number.
`--impl blocked-ell`: context only: the reference's other comparator, the vendor library's Blocked-ELL SpMM on V x V
blocks of the same shape and sparsity (spmm_benchmark.cpp:246-323).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (op, M, K, V, sparsity, N or k, instances, pattern kind)
    "spmm_v8_s90": dict(op="spmm", M=2048, K=512, V=8, s=0.9, N=256, inst=256, kind="beta"),
    "spmm_v8_s50": dict(op="spmm", M=2048, K=512, V=8, s=0.5, N=256, inst=256, kind="beta"),
    "spmm_v8_s90_n128": dict(op="spmm", M=2048, K=512, V=8, s=0.9, N=128, inst=256, kind="beta"),
    "spmm_v8_s90_n64": dict(op="spmm", M=2048, K=512, V=8, s=0.9, N=64, inst=256, kind="beta"),
    # the sparsity sweep of configs 2 and 3 at V = 8 (0.5 and 0.9 are above and below)
    "spmm_v8_s70": dict(op="spmm", M=2048, K=512, V=8, s=0.7, N=256, inst=256, kind="beta"),
    "spmm_v8_s80": dict(op="spmm", M=2048, K=512, V=8, s=0.8, N=256, inst=256, kind="beta"),
    "spmm_v8_s95": dict(op="spmm", M=2048, K=512, V=8, s=0.95, N=256, inst=256, kind="beta"),
    "spmm_v8_s98": dict(op="spmm", M=2048, K=512, V=8, s=0.98, N=256, inst=256, kind="beta"),
    "sddmm_v8_s50": dict(op="sddmm", M=2048, K=512, V=8, s=0.5, N=256, inst=256, kind="beta"),
    "sddmm_v8_s70": dict(op="sddmm", M=2048, K=512, V=8, s=0.7, N=256, inst=256, kind="beta"),
    "sddmm_v8_s80": dict(op="sddmm", M=2048, K=512, V=8, s=0.8, N=256, inst=256, kind="beta"),
    "sddmm_v8_s95": dict(op="sddmm", M=2048, K=512, V=8, s=0.95, N=256, inst=256, kind="beta"),
    "sddmm_v8_s98": dict(op="sddmm", M=2048, K=512, V=8, s=0.98, N=256, inst=256, kind="beta"),
    "sddmm_v4_s90": dict(op="sddmm", M=2048, K=512, V=4, s=0.9, N=256, inst=256, kind="beta"),
    "sddmm_v2_s90": dict(op="sddmm", M=2048, K=512, V=2, s=0.9, N=256, inst=256, kind="beta"),
    "spmm_v4_s90": dict(op="spmm", M=2048, K=512, V=4, s=0.9, N=256, inst=256, kind="beta"),
    "spmm_v2_s90": dict(op="spmm", M=2048, K=512, V=2, s=0.9, N=256, inst=256, kind="beta"),
    "sddmm_v8_s90": dict(op="sddmm", M=2048, K=512, V=8, s=0.9, N=256, inst=256, kind="beta"),
    # product with the transposed sparse matrix (vs_spmm_t): out [K x N] = A^T . rhs, rhs [M x N]
    "spmm_t_v8_s90": dict(op="spmm_t", M=2048, K=512, V=8, s=0.9, N=256, inst=256, kind="beta"),
    # config 5: fixed-mask sparse attention, batch 8 x 16 heads = 128 problems sharing one band + strided mask,
    # sequence 4096, head dimension 64 (N), V = 8, 90 % sparse; forward (SDDMM -> softmax -> SpMM) and backward
    "attention_cfg5": dict(op="attention", M=4096, K=4096, V=8, s=0.9, N=64, inst=128, kind="band", band=256),
    "attention_bwd_cfg5": dict(op="attention_bwd", M=4096, K=4096, V=8, s=0.9, N=64, inst=128, kind="band", band=256),
    "spmm_cc_v8_s90": dict(op="spmm", M=2048, K=512, V=8, s=0.9, N=256, inst=256, kind="beta", path=1),
    "sddmm_cc_v8_s90": dict(op="sddmm", M=2048, K=512, V=8, s=0.9, N=256, inst=256, kind="beta", path=1),
    # fp32 CUDA-core SpMM (the cudaSpmm entry point), M = K = 4096, uniform random positions, values and B U(-1,1)
    "spmm_f32_v4_s90_n1024": dict(op="spmm", M=4096, K=4096, V=4, s=0.9, N=1024, inst=8, kind="uniform", path=1, dtype="f32"),
    "spmm_f32_v1_s90_n1024": dict(op="spmm", M=4096, K=4096, V=1, s=0.9, N=1024, inst=8, kind="uniform", path=1, dtype="f32"),
    "spmm_f32_v4_s80_n8192": dict(op="spmm", M=4096, K=4096, V=4, s=0.8, N=8192, inst=2, kind="uniform", path=1, dtype="f32"),
    "spmm_f32_v1_s80_n8192": dict(op="spmm", M=4096, K=4096, V=1, s=0.8, N=8192, inst=2, kind="uniform", path=1, dtype="f32"),
}

# The partitioned configurations, measured by every `--gpus N` run next to the headline number (the `sharded` object
# of the JSON line): fp32 CUDA-core SpMM split by columns of the dense operand, fixed-mask attention split by
# batch x head.  One instance each (the configuration itself, not a stream of copies).
SHARDED = ("spmm_f32_v4_s80_n8192", "spmm_f32_v1_s80_n8192", "attention_cfg5")

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from an ncu capture of this
# command (profiles/ holds the summary it comes from); None until one has been taken for the workload.
NCU_TRAFFIC_BYTES = {
    "spmm_v8_s90": 335.7e6,    # profiles/spmm_pair_kernel__spmm_v8_s90.md
    "sddmm_v8_s90": 400.8e6,   # profiles/sddmm_pair_kernel__sddmm_v8_s90.md
}


def kernels_per_step(w, a=None):
    """Names of the library's kernels one step launches (the count is what `gpu_launches` reports)."""
    tensor = w.get("path") != 1
    # the densified product runs on pairs of CTAs for dense widths that are multiples of 128, on single CTAs otherwise
    pair = w["N"] % 128 == 0 and os.environ.get("VSPARSE_B200_SPMM_PAIR") != "0"
    dense = "spmm_pair_kernel" if pair else "spmm_dense_kernel"
    if w["op"] == "attention":
        return ["sddmm_tma_kernel", "softmax_cvse_kernel", "dense_plan_kernel", dense,
                "spmm_tma_kernel (returns at once unless the plan kernel chose it)"]
    if w["op"] == "attention_bwd":
        plan3 = ["dense_plan_kernel", dense,
                 "fallback kernel (returns at once unless the plan kernel chose it)"]
        return ["sddmm_tma_kernel", "softmax_cvse_kernel"] + plan3 + ["sddmm_tma_kernel", "softmax_cvse_backward_kernel"] + plan3 + plan3
    if w["op"] == "spmm_t":
        if os.environ.get("VSPARSE_B200_SPMM_T") == "gather":
            return ["spmm_t_kernel"]
        return ["dense_plan_kernel<transposed>", dense + "<transposed>",
                "spmm_t_kernel (returns at once unless the plan kernel chose it)"]
    if w["op"] == "spmm" and tensor:
        if os.environ.get("VSPARSE_B200_SPMM") == "gather":
            return ["spmm_tma_kernel"]
        return ["dense_plan_kernel", dense,
                "spmm_tma_kernel (returns at once unless the plan kernel chose it)"]
    if w["op"] == "spmm":
        return ["spmm_cc_kernel"]
    if not tensor:
        # a group of lanes per vector-row while the contraction length fits 32 chunks of 16 bytes, per mask entry beyond
        by_row = w["N"] // 8 <= 32 and os.environ.get("VSPARSE_B200_SDDMM_CC") != "entry"
        return ["sddmm_cc_row_kernel" if by_row else "sddmm_cc_kernel"]
    from vectorsparse_b200 import _lib
    dense = a is not None and _lib.lib().vs_sddmm_formulation(a.m_vec, w["N"], w["K"], a.nnz_vec, w["V"]) == 1
    if not dense:
        return ["sddmm_tma_kernel"]
    if os.environ.get("VSPARSE_B200_SDDMM_PAIR") == "0":
        return ["sddmm_plan_kernel", "sddmm_dense_kernel"]
    return ["sddmm_cell_plan_kernel", "sddmm_pair_kernel", "sddmm_twin_kernel (returns at once unless a vector-row names a column twice)"]


def config_of(name, w, a):
    """The workload as both arms (this library, the reference's CPU path) print it: identical dictionaries."""
    return {"workload": name, "op": w["op"], "M": w["M"], "K": w["K"], "V": w["V"], "sparsity": w["s"],
            "dense_width_or_k": w["N"], "nnz_vec": a.nnz_vec, "instances_per_step": w["inst"]}


def metric_name(w):
    return {"sddmm": "SDDMM effective TFLOP/s (2*nnz*k)",
            "attention": "sparse attention effective TFLOP/s (2 products: 4*nnz*d)",
            "attention_bwd": "sparse attention backward effective TFLOP/s (5 products: 10*nnz*d)",
            }.get(w["op"], "SpMM effective TFLOP/s (2*nnz*N)")


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def measured_tensor_peaks():
    """(burst, sustained) dense 16-bit GEMM TFLOP/s of the library GEMM on this pool, and where they come from."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["bf16_tflops"]), float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "measured"
    return 1590.0, 1400.0, "fallback"


def tensor_pipe_view(w, avg_launch_s):
    """The densifying SpMM kernels multiply whole 128- or 256-row tiles of A, zeros included, so the tensor pipe
    executes 2*M*K*N flops per instance whatever the sparsity.  That dense-equivalent rate against the measured
    GEMM peak is the second ceiling of these kernels (the first is HBM, `roofline`): at 90 % sparsity and K = 512
    it is the higher of the two floors."""
    dense_flops = 2.0 * w["M"] * w["K"] * w["N"] * w["inst"]
    burst, sustained, kind = measured_tensor_peaks()
    tfl = dense_flops / avg_launch_s / 1e12
    return {"dense_equivalent_tflops": tfl, "peak_burst": burst, "peak_sustained": sustained, "peak_source": f"of {kind}",
            "frac_of_burst": tfl / burst, "frac_of_sustained": tfl / sustained,
            "floor_ms_at_burst": dense_flops / (burst * 1e12) * 1e3}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def build_problem(w, seed=2026):
    from vectorsparse_b200 import cvse
    kind = {"beta": cvse.GEN_BETA, "fixed": cvse.GEN_FIXED, "uniform": cvse.GEN_UNIFORM, "band": cvse.GEN_BAND}[w["kind"]]
    a = cvse.generate(kind, seed, w["M"] // w["V"], w["K"], w["V"], w["s"], w.get("band", 0))
    return a


def algorithmic(w, a):
    """(flops, HBM bytes) of ONE launch = `inst` instances sharing the structure arrays."""
    nnz_vec, V, inst = a.nnz_vec, w["V"], w["inst"]
    structure = nnz_vec * 4 + (2 * a.m_vec + 1) * 4
    es = 4 if w.get("dtype") == "f32" else 2
    if w["op"] == "spmm":
        k_touched = int(np.unique(a.col_indices).size)
        per = nnz_vec * V * es + k_touched * w["N"] * es + w["M"] * w["N"] * es
        flops = 2.0 * nnz_vec * V * w["N"]
    elif w["op"] in ("attention", "attention_bwd"):
        # unfused pipeline: the dense operands once each, the score / probability arrays once per pass over them
        d, n, nnz = w["N"], w["K"], nnz_vec * V
        if w["op"] == "attention":   # q, k, v in, o out; scores written, read + written by the softmax, read by the SpMM
            per = 4 * n * d * 2 + 4 * nnz * 2
            flops = 2 * 2.0 * nnz * d
        else:                        # q, k, v, dO in, dq, dk, dv out; P: w, r, w, r, r; dP / dS: w, r, w, r, r
            per = 7 * n * d * 2 + 10 * nnz * 2
            flops = 5 * 2.0 * nnz * d
    elif w["op"] == "spmm_t":  # rhs M x N (the rows of nonempty vector-rows), out K x N
        rows_touched = int(np.count_nonzero(np.diff(a.row_offsets))) * V
        per = nnz_vec * V * es + rows_touched * w["N"] * es + w["K"] * w["N"] * es
        flops = 2.0 * nnz_vec * V * w["N"]
        structure = nnz_vec * 8 + (w["K"] + 1) * 4   # t_rows, t_src, t_offsets
    else:  # sddmm: lhs M x k, rhs K x k, out nnz
        k = w["N"]
        n_touched = int(np.unique(a.col_indices).size)
        per = w["M"] * k * 2 + n_touched * k * 2 + nnz_vec * V * 2
        flops = 2.0 * nnz_vec * V * k
    return flops * inst, float(structure + per * inst)


def run_ours(args):
    import torch
    import torch.distributed as dist

    from vectorsparse_b200 import VS_PATH_CUDA_CORE, VS_PATH_TENSOR, cvse, ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    w = WORKLOADS[args.workload]
    path = VS_PATH_CUDA_CORE if w.get("path") == 1 else VS_PATH_TENSOR
    a = build_problem(w)
    inst, V, M, K, N = w["inst"], w["V"], w["M"], w["K"], w["N"]
    ri, ro, ci = a.to_device(dev)
    flops, alg_bytes = algorithmic(w, a)

    # operands of this rank's stream, in pinned host memory (for the end-to-end leg) and on the device
    seed = 100 + rank
    f32 = w.get("dtype") == "f32"
    if w["op"] == "spmm":
        row = (a.nnz_vec * V + 7) // 8 * 8  # per-instance stride kept 16-byte aligned for every V
        npdt, tdt = (np.float32, torch.float32) if f32 else (np.float16, torch.float16)
        dist_a, dist_b, sig = (cvse.DIST_UNIFORM, cvse.DIST_UNIFORM, 1.0) if f32 else (cvse.DIST_NORMAL, cvse.DIST_NORMAL, 0.02)
        h_a = torch.from_numpy(cvse.fill_random((inst, row), npdt, dist_a, seed, sig)).pin_memory()
        h_b = torch.from_numpy(cvse.fill_random((inst, K, N), npdt, dist_b, seed + 1, 1.0)).pin_memory()
        h_out = torch.empty((inst, M, N), dtype=tdt).pin_memory()
        d_out = torch.empty((inst, M, N), dtype=tdt, device=dev)

        def launch(d_a, d_b, out):
            ops.spmm_batched(path, a.m_vec, V, N, K, ri, ro, ci, d_a, d_b, out)
    elif w["op"] in ("attention", "attention_bwd"):
        # inputs stacked in one pinned array (q, k, v and, for the backward pass, dO), outputs in another
        bwd = w["op"] == "attention_bwd"
        n, d = K, N
        h_a = torch.from_numpy(cvse.fill_random((4 if bwd else 3, inst, n, d), np.float16, cvse.DIST_NORMAL, seed, 1.0)).pin_memory()
        h_b = torch.zeros(8, dtype=torch.float16).pin_memory()   # the second input slot of the harness: unused here
        h_out = torch.empty((3 if bwd else 1, inst, n, d), dtype=torch.float16).pin_memory()
        d_out = torch.empty((3 if bwd else 1, inst, n, d), dtype=torch.float16, device=dev)
        ws_p = torch.empty((inst, a.nnz_vec * V), dtype=torch.float16, device=dev)
        ws_g = torch.empty((inst, a.nnz_vec * V), dtype=torch.float16, device=dev) if bwd else None
        if bwd:
            t_off, t_rows, t_src = (torch.from_numpy(x).to(dev) for x in cvse.transpose(a))

        def launch(d_a, d_b, out):
            if bwd:
                ops.attention_cvse_backward(path, a.m_vec, V, n, d, a.nnz_vec, ri, ro, ci, t_off, t_rows, t_src, d_a[0], d_a[1],
                                            d_a[2], d_a[3], out[0], out[1], out[2], ws_p, ws_g, 0.125)
            else:
                ops.attention_cvse(path, a.m_vec, V, n, d, a.nnz_vec, ri, ro, ci, d_a[0], d_a[1], d_a[2], out[0], ws_p, 0.125)
    elif w["op"] == "spmm_t":
        row = (a.nnz_vec * V + 7) // 8 * 8
        t_off, t_rows, t_src = (torch.from_numpy(x).to(dev) for x in cvse.transpose(a))
        h_a = torch.from_numpy(cvse.fill_random((inst, row), np.float16, cvse.DIST_NORMAL, seed, 0.02)).pin_memory()
        h_b = torch.from_numpy(cvse.fill_random((inst, M, N), np.float16, cvse.DIST_NORMAL, seed + 1, 1.0)).pin_memory()
        h_out = torch.empty((inst, K, N), dtype=torch.float16).pin_memory()
        d_out = torch.empty((inst, K, N), dtype=torch.float16, device=dev)

        def launch(d_a, d_b, out):
            ops.spmm_t(a.m_vec, V, N, K, t_off, t_rows, t_src, d_a, d_b, out)
    else:
        k = N
        h_a = torch.from_numpy(cvse.fill_random((inst, M, k), np.float16, cvse.DIST_NORMAL, seed, 1.0)).pin_memory()
        h_b = torch.from_numpy(cvse.fill_random((inst, K, k), np.float16, cvse.DIST_NORMAL, seed + 1, 1.0)).pin_memory()
        row = (a.nnz_vec * V + 7) // 8 * 8  # per-instance stride kept 16-byte aligned for every V
        h_out = torch.empty((inst, row), dtype=torch.float16).pin_memory()
        d_out = torch.empty((inst, row), dtype=torch.float16, device=dev)

        def launch(d_a, d_b, out):
            # through the C ABI directly: the Python wrapper takes contiguous [B, nnz] outputs only
            from vectorsparse_b200 import _lib
            with torch.cuda.device(dev):
                rc = _lib.lib().vs_sddmm_batched(path, 0, 0, a.m_vec, k, K, a.nnz_vec, ri.data_ptr(), ro.data_ptr(), ci.data_ptr(),
                                                 d_a.data_ptr(), d_b.data_ptr(), out.data_ptr(), V, inst, M * k, K * k, row,
                                                 torch.cuda.current_stream().cuda_stream, 1)
            _lib.check(rc, "vs_sddmm_batched")
    d_a = h_a.to(dev)
    d_b = h_b.to(dev)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident leg: `value` and the roofline ------------------------------------------------------
    # clocks are sampled from here to the end of the end-to-end leg: the timed region alone (a few ms) is shorter
    # than nvidia-smi's sampling period
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for _ in range(max(args.warmup, 3)):
        launch(d_a, d_b, d_out)
    barrier()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    ev[0].record()
    for s in range(args.steps):
        launch(d_a, d_b, d_out)
        ev[s + 1].record()
    barrier()
    per_launch_ms = [ev[s].elapsed_time(ev[s + 1]) for s in range(args.steps)]
    total_ms = ev[0].elapsed_time(ev[args.steps])
    assert ops.device_status() == 0, "a kernel gave up on a bounded wait"

    # ---- the dominant kernel alone (outside the timed region above): the library brackets its multiplying kernel
    # with CUDA events on the launching stream, which also stops it from overlapping the plan kernel before it and
    # the fallback kernel behind it; the same steps again, so the device is as warm as in the timed region
    kernel_alone = None
    if rank == 0 and kernels_per_step(w, a)[0] in ("dense_plan_kernel", "dense_plan_kernel<transposed>", "sddmm_cell_plan_kernel") \
            and w["op"] in ("spmm", "spmm_t", "sddmm"):
        ops.kernel_timing(True)
        for _ in range(args.steps):
            launch(d_a, d_b, d_out)
        k_ms, k_n = ops.kernel_timing(False)
        if k_n > 0:
            kernel_alone = {"name": kernels_per_step(w, a)[1], "launches": k_n, "ms_per_launch": k_ms / k_n}
    barrier()

    # ---- end-to-end leg: host buffers, copies inside the timed region --------------------------------------
    # Every step copies its inputs from pinned host memory, runs the public API call and copies the result back.
    # The three stages run on three streams over two sets of device buffers, so that step s+1's upload and step
    # s-1's download overlap step s's kernels (PCIe is full duplex); the time is that of the whole sequence.
    e2e_steps = 0 if args.kernel_only else max(4, min(args.steps, 10))
    if e2e_steps:
        s_in, s_run, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
        bufs = [(torch.empty_like(d_a), torch.empty_like(d_b), torch.empty_like(d_out)) for _ in range(2)]
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_run = [torch.cuda.Event() for _ in range(2)]
        ev_out = [torch.cuda.Event() for _ in range(2)]

    def e2e_sequence(n):
        for st in (s_in, s_run, s_out):
            st.wait_stream(torch.cuda.current_stream())
        for s in range(n):
            i = s & 1
            da, db, dout = bufs[i]
            with torch.cuda.stream(s_in):
                if s >= 2:
                    s_in.wait_event(ev_run[i])     # step s-2 has consumed this set of inputs
                da.copy_(h_a, non_blocking=True)
                db.copy_(h_b, non_blocking=True)
                ev_in[i].record(s_in)
            with torch.cuda.stream(s_run):
                s_run.wait_event(ev_in[i])
                if s >= 2:
                    s_run.wait_event(ev_out[i])    # step s-2's result has left this output buffer
                launch(da, db, dout)
                ev_run[i].record(s_run)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_run[i])
                h_out.copy_(dout, non_blocking=True)
                ev_out[i].record(s_out)
        for st in (s_in, s_run, s_out):
            torch.cuda.current_stream().wait_stream(st)

    if e2e_steps:
        e2e_sequence(2)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    if e2e_steps:
        e2e_sequence(e2e_steps)
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1) if e2e_steps else float("nan")
    if rank == 0 and args.steps * 0.3 < 500:   # keep the GPU under the same load until ~0.5 s of samples exist
        t_end = time.time() + 0.5
        while time.time() < t_end:
            launch(d_a, d_b, d_out)
            torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None

    # ---- single-launch latency of ONE instance (the reference API's granularity), L2-hot ----------------------
    lat_us = None
    if w["op"] == "spmm" and not args.kernel_only:
        for _ in range(5):
            ops.spmm.wmmaSpmm(a.m_vec, V, N, K, ri, ro, ci, d_a[0], d_b[0], d_out[0]) if path == VS_PATH_TENSOR else \
                ops.spmm.cudaSpmm(a.m_vec, V, N, K, ri, ro, ci, d_a[0], d_b[0], d_out[0])
        torch.cuda.synchronize()
        l0, l1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0.record()
        for _ in range(50):
            ops.spmm.wmmaSpmm(a.m_vec, V, N, K, ri, ro, ci, d_a[0], d_b[0], d_out[0]) if path == VS_PATH_TENSOR else \
                ops.spmm.cudaSpmm(a.m_vec, V, N, K, ri, ro, ci, d_a[0], d_b[0], d_out[0])
        l1.record()
        torch.cuda.synchronize()
        lat_us = l0.elapsed_time(l1) * 1000.0 / 50

    # context: the reference's own kernels, recompiled for this part, on the same stream of instances
    ref_kernels = None
    if rank == 0 and world == 1 and not args.kernel_only and w["op"] in ("spmm", "sddmm") and path == VS_PATH_TENSOR:
        ref_kernels = reference_kernels_leg(w, a, dev, d_a, d_b, flops)

    # the partitioned configurations: every rank takes part (timings are reduced inside)
    h2d = h_a.numel() * h_a.element_size() + h_b.numel() * h_b.element_size()
    d2h = h_out.numel() * h_out.element_size()
    sharded = None
    if not args.kernel_only and not args.no_sharded:
        del d_a, d_b, d_out, h_a, h_b, h_out
        if e2e_steps:
            del bufs
        torch.cuda.empty_cache()
        sharded = sharded_leg(world, rank, dev)

    # max over ranks
    t = torch.tensor([total_ms, e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, e2e_ms = float(t[0]), float(t[1])

    if rank == 0:
        peak, peak_kind = measured_peaks()
        avg_launch_s = float(np.mean(per_launch_ms)) * 1e-3
        achieved = alg_bytes / avg_launch_s / 1e9
        if f32 and w["op"] == "spmm":
            # M = K = 4096 in fp32 is bound by fp32 FMA issue, not by memory (50 to 190 flop per byte): the denominator
            # is the FMA throughput measured in this run by a register-only probe kernel
            fma_peak = ops.measure_fp32_fma()
            tfl = flops / avg_launch_s / 1e12
            roofline = {"bound": "fp32_fma", "achieved": tfl, "peak": fma_peak, "unit": "TFLOP/s", "frac": tfl / fma_peak,
                        "peak_source": "fp32 FMA probe kernel, measured in this run", "traffic": NCU_TRAFFIC_BYTES.get(args.workload),
                        "algorithmic_bytes_per_launch": alg_bytes, "hbm_gbs_achieved": achieved}
        else:
            roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                        "peak_source": f"of {peak_kind}", "frac_of_nominal_8tbs": achieved / 8000.0,
                        "traffic": NCU_TRAFFIC_BYTES.get(args.workload), "algorithmic_bytes_per_launch": alg_bytes}
            if w["op"] in ("spmm", "spmm_t") and path != VS_PATH_CUDA_CORE:
                roofline["tensor_pipe"] = tensor_pipe_view(w, avg_launch_s)
            if kernel_alone:
                # `achieved` / `frac` above are those of the whole call (plan kernel, multiplying kernel and the kernel
                # that returns at once behind it); these are the multiplying kernel's own
                k_gbs = alg_bytes / (kernel_alone["ms_per_launch"] * 1e-3) / 1e9
                roofline["dominant_kernel"] = dict(kernel_alone, achieved=k_gbs, frac=k_gbs / peak,
                                                   how="CUDA events recorded by the library around this kernel on its stream, "
                                                       "the same steps run once more after the timed region")
        line = {
            "metric": metric_name(w),
            "value": flops * args.steps * world / (total_ms * 1e-3) / 1e12,
            "unit": "TFLOP/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": max(args.warmup, 3),
            "ms_per_step": total_ms / args.steps,
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": "f32" if f32 else "f16 (fp32 accumulate)",
            "data": "synthetic",
            "config": config_of(args.workload, w, a),
            "run": {"path": "cuda-core" if path == VS_PATH_CUDA_CORE else "tensor (tcgen05)",
                    "l2": "working set larger than L2 (distinct operands per instance), no flush needed",
                    "parallelism": f"independent streams x{world}"},
            "roofline": roofline,
            "e2e": {"value": flops * e2e_steps * world / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps},
            "gpu_launches": args.steps * len(kernels_per_step(w, a)),
            "kernels_per_step": kernels_per_step(w, a),
            "single_launch_latency_us": lat_us,
            "clocks": clocks,
        }
        if ref_kernels is not None:
            line["reference_kernels_context"] = ref_kernels
        if sharded is not None:
            line["sharded"] = sharded
        if world == 1 and not args.no_cpu and not args.kernel_only:
            line["cpu_baseline"] = cpu_leg(w, a, budget_s=12.0)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def reference_kernels_leg(w, a, dev, d_a, d_b, flops, steps=3):
    """CONTEXT, not a target and not part of any other number: the reference's own tensor-core kernels
    (spmm::wmmaSpmm, src/wmma_spmm.cu:13-116; sddmm::wmmaSddmm algorithm 1, src/wmma_sddmm.cu:250-504), compiled
    unmodified for sm_100a into baseline/_ref/, on this workload's stream: one launch per instance, as the reference
    API works.  For SpMM every vector-row is padded to a positive multiple of 32 vectors with zero values (see
    baseline/refk.py); the padded product equals the original one.  A small problem is checked first with the
    reference's own criterion (abs error <= 0.5); nothing is timed if that fails."""
    import torch

    from baseline import refk
    from vectorsparse_b200 import cvse, ops

    L = refk.lib()
    if L is None:
        return {"unavailable": "baseline/_ref/libvsref_kernels.so is not built (no reference checkout at build time)"}
    V, M, K, N, inst = w["V"], w["M"], w["K"], w["N"], w["inst"]
    # the reference's entry points print "V=8" at every call (src/wmma_spmm.cu:341): keep that off this program's stdout
    sys.stdout.flush()
    saved_fd = os.dup(1)
    devnull = os.open(os.devnull, os.O_WRONLY)
    os.dup2(devnull, 1)
    try:
        return _reference_kernels_timed(L, refk, w, a, dev, d_a, d_b, flops, steps)
    finally:
        os.dup2(saved_fd, 1)
        os.close(saved_fd)
        os.close(devnull)


def _reference_kernels_timed(L, refk, w, a, dev, d_a, d_b, flops, steps):
    import torch

    from vectorsparse_b200 import cvse, ops
    V, M, K, N, inst = w["V"], w["M"], w["K"], w["N"], w["inst"]

    def spmm_call(p_struct, m_vec, vals, B, out):
        ri, ro, ci = p_struct
        return L.refk_wmma_spmm(m_vec, V, N, K, ri.data_ptr(), ro.data_ptr(), ci.data_ptr(), vals.data_ptr(), B.data_ptr(), out.data_ptr(), 0)

    alg = [1]   # the reference harness's default algorithm first; the WMMA-based one if that fails the small check

    def sddmm_call(p_struct, m_vec, nnz_vec, lhs, rhs, out):
        ri, ro, ci = p_struct
        return L.refk_wmma_sddmm(m_vec, N, K, nnz_vec, ri.data_ptr(), ro.data_ptr(), ci.data_ptr(), lhs.data_ptr(), rhs.data_ptr(),
                                 out.data_ptr(), V, alg[0], 0)

    # ---- a small problem first, against this library's result -------------------------------------------------
    t = cvse.generate(cvse.GEN_BETA, 3, 128 // V, K, V, 0.8)
    if w["op"] == "spmm":
        ro, ci, src = refk.pad_rows(t.row_offsets, t.col_indices, K)
        tp = cvse.CVSE(t.m_vec, K, V, ro, ci, cvse.row_swizzle(ro))
        st = tp.to_device(dev)
        tv = torch.from_numpy(refk.pad_values(cvse.fill_random((t.nnz_vec * V,), np.float16, cvse.DIST_NORMAL, 1, 0.5), src, V)).to(dev)
        tb = d_b[0]
        got, want = (torch.zeros((t.m, N), dtype=torch.float16, device=dev) for _ in range(2))
        rc = spmm_call(st, tp.m_vec, tv, tb, got)
        ops.spmm.wmmaSpmm(tp.m_vec, V, N, K, *st, tv, tb, want)
    else:
        st = t.to_device(dev)
        lhs = d_a[0][:t.m].contiguous()
        got, want = (torch.zeros(t.nnz_vec * V, dtype=torch.float16, device=dev) for _ in range(2))
        ops.sddmm.wmmaSddmm(t.m_vec, N, K, t.nnz_vec, *st, lhs, d_b[0], want, V)
        for alg[0] in (1, 0):
            got.zero_()
            rc = sddmm_call(st, t.m_vec, t.nnz_vec, lhs, d_b[0], got)
            torch.cuda.synchronize()
            if rc == 0 and float((got.float() - want.float()).abs().max()) <= 0.5:
                break
    torch.cuda.synchronize()
    worst = float((got.float() - want.float()).abs().max())
    if rc != 0 or not (worst <= 0.5):
        return {"unavailable": f"small check failed (rc {rc}, max abs difference {worst}): not timed"}

    # ---- the stream of the step: one launch per instance --------------------------------------------------------
    if w["op"] == "spmm":
        ro, ci, src = refk.pad_rows(a.row_offsets, a.col_indices, K)
        ap = cvse.CVSE(a.m_vec, K, V, ro, ci, cvse.row_swizzle(ro))
        st = ap.to_device(dev)
        keep = torch.from_numpy(np.nonzero(src >= 0)[0]).to(dev)
        srck = torch.from_numpy(src[src >= 0]).to(dev)
        vals = torch.zeros((inst, len(src), V), dtype=torch.float16, device=dev)
        vals[:, keep] = d_a[:, :a.nnz_vec * V].reshape(inst, a.nnz_vec, V)[:, srck]
        out = torch.empty((inst, M, N), dtype=torch.float16, device=dev)

        def step():
            for b in range(inst):
                spmm_call(st, ap.m_vec, vals[b], d_b[b], out[b])
        note = f"rows padded to multiples of 32 vectors with zero values ({a.nnz_vec} -> {len(src)} vectors)"
    else:
        st = a.to_device(dev)
        out = torch.empty((inst, a.nnz_vec * V), dtype=torch.float16, device=dev)

        def step():
            for b in range(inst):
                sddmm_call(st, a.m_vec, a.nnz_vec, d_a[b], d_b[b], out[b])
        note = "the workload's own mask"
    step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    return {"kernel": "spmm::wmmaSpmm (src/wmma_spmm.cu:13-116)" if w["op"] == "spmm" else
            f"sddmm::wmmaSddmm, algorithm {alg[0]} (src/wmma_sddmm.cu:{'250-504' if alg[0] == 1 else '23-243'})",
            "built": "the reference's sources, unmodified, nvcc -gencode arch=compute_100a,code=sm_100a (it ships -arch=sm_70)",
            "ms_per_step": ms, "tflops": flops / (ms * 1e-3) / 1e12, "launches_per_step": inst, "input": note,
            "small_check_max_abs_difference": worst, "role": "context only"}


def sharded_leg(world, rank, dev, steps=10, warmup=3):
    """The two partitions of the operators over the GPUs of one box, each rank computing its shard with no collective
    on the data path: fp32 CUDA-core SpMM (M = K = 4096, N = 8192) split by COLUMNS of the dense operand, and
    fixed-mask attention (128 batch x head problems) split by batch x head.  Per configuration: ms per pass of the
    sharded run (max over ranks), TFLOP/s over all ranks, the same pass on ONE GPU in the same run (rank 0 computing
    the whole problem) and the strong-scaling efficiency t(1) / (N t(N)); the optional all-gather of the result is
    timed on its own and is not part of either time.  Rank 0 returns the dictionary, the others None."""
    import torch
    import torch.distributed as dist

    from vectorsparse_b200 import VS_PATH_TENSOR, cvse, ops, shard

    def timed(fn):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    def max_over_ranks(ms):
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    def once(fn):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)

    out = {}
    for name in SHARDED:
        w = WORKLOADS[name]
        a = build_problem(w)
        V, M, K, N = w["V"], w["M"], w["K"], w["N"]
        ri, ro, ci = a.to_device(dev)
        entry = {"n_gpus": world}
        gather_ms, t_one = None, None
        if w["op"] == "spmm":      # columns of the dense operand; every rank holds the whole sparse matrix
            flops = 2.0 * a.nnz_vec * V * N
            vals = torch.from_numpy(cvse.fill_random((a.nnz_vec * V,), np.float32, cvse.DIST_UNIFORM, 7)).to(dev)
            B = cvse.fill_random((K, N), np.float32, cvse.DIST_UNIFORM, 8, 1.0)
            c0, wd = shard.column_shards(N, world, 64)[rank]
            B_local = torch.from_numpy(np.ascontiguousarray(B[:, c0:c0 + wd])).to(dev)
            C_local = torch.empty((M, wd), dtype=torch.float32, device=dev)
            t_shard = max_over_ranks(timed(lambda: shard.spmm_column_sharded(ops.spmm.cudaSpmm, a.m_vec, V, N, K, (ri, ro, ci), vals,
                                                                            B_local, C_local)))
            entry["partition"] = f"columns of the dense operand: {N} -> {wd} per GPU"
            if world > 1:
                shard.gather_columns(C_local, N, 64)   # first collective of the run: communicator set-up is not timed
                gather_ms = max_over_ranks(once(lambda: shard.gather_columns(C_local, N, 64)))
            if rank == 0 and world > 1:
                B_full = torch.from_numpy(B).to(dev)
                C_full = torch.empty((M, N), dtype=torch.float32, device=dev)
                t_one = _timed_local(lambda: ops.spmm.cudaSpmm(a.m_vec, V, N, K, ri, ro, ci, vals, B_full, C_full), steps, warmup)
                del B_full, C_full
            del B_local, C_local, vals
        else:                      # batch x head: every rank holds the mask and its own heads
            heads, n, d = w["inst"], K, N
            flops = 2 * 2.0 * a.nnz_vec * V * d * heads
            h0, cnt = shard.batch_shards(heads, world)[rank]
            q, k, v = (torch.from_numpy(cvse.fill_random((cnt, n, d), np.float16, cvse.DIST_NORMAL, 11 + 3 * h0 + i, 1.0)).to(dev)
                       for i in range(3))
            o = torch.empty((cnt, n, d), dtype=torch.float16, device=dev)
            ws = torch.empty((cnt, a.nnz_vec * V), dtype=torch.float16, device=dev)
            t_shard = max_over_ranks(timed(lambda: ops.attention_cvse(VS_PATH_TENSOR, a.m_vec, V, n, d, a.nnz_vec, ri, ro, ci, q, k, v,
                                                                      o, ws, 0.125)))
            entry["partition"] = f"batch x head: {heads} -> {cnt} per GPU"
            if world > 1:
                shard.gather_batch(o, heads)
                gather_ms = max_over_ranks(once(lambda: shard.gather_batch(o, heads)))
            del q, k, v, o, ws
            if rank == 0 and world > 1:
                q, k, v = (torch.from_numpy(cvse.fill_random((heads, n, d), np.float16, cvse.DIST_NORMAL, 11 + i, 1.0)).to(dev)
                           for i in range(3))
                o = torch.empty((heads, n, d), dtype=torch.float16, device=dev)
                ws = torch.empty((heads, a.nnz_vec * V), dtype=torch.float16, device=dev)
                t_one = _timed_local(lambda: ops.attention_cvse(VS_PATH_TENSOR, a.m_vec, V, n, d, a.nnz_vec, ri, ro, ci, q, k, v, o,
                                                                ws, 0.125), steps, warmup)
                del q, k, v, o, ws
        torch.cuda.empty_cache()
        if world > 1:
            dist.barrier()   # the other ranks wait while rank 0 times the whole problem on one GPU
        if rank == 0:
            if world == 1:
                t_one = t_shard
            entry.update({"ms": t_shard, "tflops": flops / (t_shard * 1e-3) / 1e12, "ms_on_one_gpu": t_one,
                          "strong_scaling_efficiency": t_one / (world * t_shard), "all_gather_ms": gather_ms})
            out[name] = entry
    return out if rank == 0 else None


def _timed_local(fn, steps, warmup):
    """CUDA-event time per call on this rank alone (no barrier: the other ranks are idle)."""
    import torch
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def cpu_leg(w, a, budget_s, threads=None):
    """The reference's CPU path on a bounded sample of the stream: its sequential host loop — the compiled
    reference code where that library exists, else the oracle's restatement — one instance per host thread."""
    import concurrent.futures as cf

    import oracle
    from vectorsparse_b200 import cvse

    cores = threads or (os.cpu_count() or 1)
    use_ref = oracle.ref() is not None
    V, M, K, N = w["V"], w["M"], w["K"], w["N"]
    if w["op"] == "spmm":
        if w.get("dtype") == "f32":
            x = cvse.fill_random((a.nnz_vec * V,), np.float32, cvse.DIST_UNIFORM, 1)
            y = cvse.fill_random((K, N), np.float32, cvse.DIST_UNIFORM, 2)
        else:
            x = cvse.fill_random((a.nnz_vec * V,), np.float16, cvse.DIST_NORMAL, 1, 0.02)
            y = cvse.fill_random((K, N), np.float16, cvse.DIST_NORMAL, 2, 1.0)
        flops = 2.0 * a.nnz_vec * V * N

        def one(_):
            if use_ref:
                return oracle.ref_spmm(a.m_vec, V, N, a.row_offsets, a.col_indices, x, y)
            return oracle.spmm(a.m_vec, V, N, a.row_offsets, a.col_indices, x, y, acc="f32", threads=1)
    elif w["op"] in ("attention", "attention_bwd"):   # no reference code: the oracle's fp64 pipeline, one head per call
        use_ref = False
        n, d = K, N
        q, kk, vv, go = (cvse.fill_random((n, d), np.float16, cvse.DIST_NORMAL, 1 + i, 1.0).astype(np.float32) for i in range(4))
        flops = (5 if w["op"] == "attention_bwd" else 2) * 2.0 * a.nnz_vec * V * d

        if w["op"] == "attention_bwd":
            cores = 1   # the backward oracle is numpy / scipy code that holds the interpreter lock: threads would not add up

        def one(_):
            if w["op"] == "attention_bwd":
                return oracle.attention_backward(a.m_vec, V, d, a.row_offsets, a.col_indices, q, kk, vv, go, 0.125)
            return oracle.attention(a.m_vec, V, d, d, a.row_offsets, a.col_indices, q, kk, vv, 0.125)
    elif w["op"] == "spmm_t":   # no reference code for this product: the oracle's loop is the CPU path
        use_ref = False
        x = cvse.fill_random((a.nnz_vec * V,), np.float16, cvse.DIST_NORMAL, 1, 0.02).astype(np.float32)
        y = cvse.fill_random((M, N), np.float16, cvse.DIST_NORMAL, 2, 1.0).astype(np.float32)
        flops = 2.0 * a.nnz_vec * V * N

        def one(_):
            return oracle.spmm_t(a.m_vec, V, N, K, a.row_offsets, a.col_indices, x, y)
    else:
        k = N
        x = cvse.fill_random((M, k), np.float16, cvse.DIST_NORMAL, 1, 1.0)
        y = cvse.fill_random((K, k), np.float16, cvse.DIST_NORMAL, 2, 1.0)
        flops = 2.0 * a.nnz_vec * V * k

        def one(_):
            if use_ref:
                return oracle.ref_sddmm(a.m_vec, k, V, a.row_offsets, a.col_indices, x, y)
            return oracle.sddmm(a.m_vec, k, V, a.row_offsets, a.col_indices, x, y, acc="f32", threads=1)
    t0 = time.perf_counter()
    one(0)
    t_one = time.perf_counter() - t0
    count = int(cores * max(1, int(budget_s / max(t_one, 1e-4))))   # ~budget_s of wall time on every core
    t0 = time.perf_counter()
    with cf.ThreadPoolExecutor(cores) as ex:
        list(ex.map(one, range(count)))
    dt = time.perf_counter() - t0
    return {"value": flops * count / dt / 1e12, "unit": "TFLOP/s", "cores": cores,
            "kind": "reference" if use_ref else "port",
            "sample": f"{count} instances of the step's problem (the step has {w['inst']}), one instance per host thread, "
                      f"{dt:.1f} s; single instance on one core {t_one * 1e3:.1f} ms"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    w = WORKLOADS[args.workload]
    a = build_problem(w)
    steps = max(1, args.steps)
    budget = min(20.0, 120.0 / (steps + args.warmup))
    vals = []
    base = None
    for i in range(args.warmup + steps):
        base = cpu_leg(w, a, budget_s=budget)
        if i >= args.warmup:
            vals.append(base["value"])
    v = float(np.mean(vals))
    base["value"] = v
    # the time one whole step of this workload (all its instances) takes at the measured rate
    per_instance = {"attention": 4.0, "attention_bwd": 10.0}.get(w["op"], 2.0) * a.nnz_vec * w["V"] * w["N"]
    step_ms = per_instance * w["inst"] / (v * 1e12) * 1e3 if v > 0 else None
    line = {
        "impl": "reference",
        "metric": metric_name(w),
        "value": v, "unit": "TFLOP/s", "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": steps,
        "warmup": args.warmup, "ms_per_step": step_ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16 (fp32 accumulate)", "data": "synthetic",
        "config": config_of(args.workload, w, a),
        "run": {"path": "host loop (spmm_benchmark.cpp:66-86)" if w["op"] == "spmm" else
                "host loop (include/bm_test_utils.h:171-193)" if w["op"] == "sddmm" else
                "host loops of the oracle (the reference has no such operator)"},
        "cpu_baseline": base,
        "e2e": {"value": v, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_dense_library(args):
    """The densified problem through the library's batched GEMM: a comparator, not a product path."""
    import torch

    from vectorsparse_b200 import cvse
    w = WORKLOADS[args.workload]
    assert w["op"] == "spmm" and w.get("dtype") != "f32", "dense-library comparator: fp16 SpMM workloads only"
    dev = "cuda:0"
    a = build_problem(w)
    inst, V, M, K, N = w["inst"], w["V"], w["M"], w["K"], w["N"]
    flops, alg_bytes = algorithmic(w, a)
    vals = torch.from_numpy(cvse.fill_random((inst, a.nnz_vec * V), np.float16, cvse.DIST_NORMAL, 100, 0.02)).to(dev)
    B = torch.from_numpy(cvse.fill_random((inst, K, N), np.float16, cvse.DIST_NORMAL, 101, 1.0)).to(dev)
    # dense A[inst, M, K]: values[j*V+v] -> row (row of j)*V+v, column col_indices[j]
    row_of = np.repeat(np.arange(a.m_vec), np.diff(a.row_offsets)).astype(np.int64)
    rows = torch.from_numpy((row_of[:, None] * V + np.arange(V)[None, :]).reshape(-1)).to(dev)
    cols = torch.from_numpy(np.repeat(a.col_indices.astype(np.int64), V)).to(dev)
    A = torch.zeros((inst, M, K), dtype=torch.float16, device=dev)
    A[:, rows, cols] = vals
    C = torch.empty((inst, M, N), dtype=torch.float16, device=dev)
    for _ in range(max(args.warmup, 3)):
        torch.bmm(A, B, out=C)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        torch.bmm(A, B, out=C)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    print(json.dumps({
        "impl": "dense-library", "metric": "SpMM effective TFLOP/s (2*nnz*N)", "value": flops / (ms * 1e-3) / 1e12,
        "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms,
        "higher_is_better": True, "dtype": "f16 (fp32 accumulate)", "data": "synthetic",
        "dense_tflops": 2.0 * inst * M * K * N / (ms * 1e-3) / 1e12,
        "config": {"workload": args.workload, "note": "A expanded to dense outside the timed region; torch.bmm (cuBLAS)"},
    }), flush=True)


def run_blocked_ell(args):
    """The reference's Blocked-ELL comparator (spmm_benchmark.cpp:246-323, its `sparse = 2` branch): the vendor
    library's Blocked-ELL SpMM (cusparseSpMM, CUSPARSE_SPMM_BLOCKED_ELL_ALG1) on a matrix of V x V blocks with the
    workload's shape and sparsity — the same number of nonzero blocks in every block-row at uniformly drawn block
    columns, as GenerateUniformBlockedELLIndex makes them — one library call per instance.  A comparator, not a
    product path: the library is reached through ctypes here and nowhere else."""
    import ctypes as C

    import torch
    w = WORKLOADS[args.workload]
    assert w["op"] == "spmm" and w.get("dtype") != "f32", "Blocked-ELL comparator: fp16 SpMM workloads only"
    dev = "cuda:0"
    inst, V, M, K, N = w["inst"], w["V"], w["M"], w["K"], w["N"]
    L = None
    for name in ("libcusparse.so.12", "libcusparse.so"):
        try:
            L = C.CDLL(name)
            break
        except OSError:
            continue
    if L is None:
        print(json.dumps({"impl": "blocked-ell", "unavailable": "libcusparse could not be loaded"}), flush=True)
        return
    vp, i64 = C.c_void_p, C.c_int64
    rows_b, cols_b = M // V, (K + V - 1) // V
    nz_b = int(cols_b * (1.0 - w["s"])) + 1                 # blocks per block-row, as the reference sizes it
    ell_cols = nz_b * V
    rng = np.random.default_rng(7)
    colind = np.stack([np.sort(rng.choice(cols_b, nz_b, replace=False)) for _ in range(rows_b)]).astype(np.int32)
    d_col = torch.from_numpy(colind).to(dev)
    vals = torch.randn((inst, M, ell_cols), dtype=torch.float16, device=dev) * 0.02
    B = torch.randn((inst, cols_b * V, N), dtype=torch.float16, device=dev)
    Cmat = torch.empty((inst, M, N), dtype=torch.float16, device=dev)
    handle = vp()
    assert L.cusparseCreate(C.byref(handle)) == 0
    L.cusparseSetStream(handle, vp(torch.cuda.current_stream().cuda_stream))
    alpha, beta = C.c_float(1.0), C.c_float(0.0)
    R16F, R32F, ROW, I32, BASE0, NT, ALG = 2, 0, 2, 2, 0, 0, 13
    descs = []
    buf_bytes = C.c_size_t(0)
    for b in range(inst):
        a_d, b_d, c_d = vp(), vp(), vp()
        assert L.cusparseCreateBlockedEll(C.byref(a_d), i64(M), i64(cols_b * V), i64(V), i64(ell_cols), vp(d_col.data_ptr()),
                                          vp(vals[b].data_ptr()), I32, BASE0, R16F) == 0
        assert L.cusparseCreateDnMat(C.byref(b_d), i64(cols_b * V), i64(N), i64(N), vp(B[b].data_ptr()), R16F, ROW) == 0
        assert L.cusparseCreateDnMat(C.byref(c_d), i64(M), i64(N), i64(N), vp(Cmat[b].data_ptr()), R16F, ROW) == 0
        descs.append((a_d, b_d, c_d))
    a_d, b_d, c_d = descs[0]
    rc = L.cusparseSpMM_bufferSize(handle, NT, NT, C.byref(alpha), a_d, b_d, C.byref(beta), c_d, R32F, ALG, C.byref(buf_bytes))
    if rc != 0:
        print(json.dumps({"impl": "blocked-ell", "unavailable": f"cusparseSpMM_bufferSize returned {rc} (block size {V})"}), flush=True)
        return
    work = torch.empty(max(int(buf_bytes.value), 16), dtype=torch.uint8, device=dev)

    def step():
        for a_d, b_d, c_d in descs:
            rc = L.cusparseSpMM(handle, NT, NT, C.byref(alpha), a_d, b_d, C.byref(beta), c_d, R32F, ALG, vp(work.data_ptr()))
            assert rc == 0, rc
    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    nnz = rows_b * nz_b * V * V
    print(json.dumps({
        "impl": "blocked-ell", "metric": "SpMM effective TFLOP/s (2*nnz*N)", "value": 2.0 * nnz * N * inst / (ms * 1e-3) / 1e12,
        "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms,
        "higher_is_better": True, "dtype": "f16 (fp32 accumulate)", "data": "synthetic",
        "config": {"workload": args.workload, "note": f"{V} x {V} blocks, {nz_b} per block-row of {cols_b}, one cusparseSpMM "
                   f"(CUSPARSE_SPMM_BLOCKED_ELL_ALG1) per instance, {inst} instances per step"},
    }), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "dense-library", "blocked-ell"])
    ap.add_argument("--workload", default="spmm_v8_s90", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-sharded", action="store_true", help="skip the partitioned configurations (`sharded` in the JSON line)")
    ap.add_argument("--kernel-only", action="store_true",
                    help="device-resident leg only (for profiler captures): no end-to-end, latency or CPU legs")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.impl == "dense-library":
        run_dense_library(args)
    elif args.impl == "blocked-ell":
        run_blocked_ell(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
