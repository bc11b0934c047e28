"""The C++ benchmark drivers, the source-compatibility header and the profiling harness, run as programs on the GPU.

The drivers keep the reference's positional command lines and stdout lines (spmm_benchmark.cpp:480-509 and :124-223,
sddmm_benchmark.cpp:399-432 and :252-300): `Using WMMA` / `Using CUDA`, `V=<n>`, `Results verified: they agree.`,
`Unsupported Vector Length!`.  They are built against include/vsparse_compat.h, so every run below goes through the
reference-named overloads (spmm::wmmaSpmm, spmm::cudaSpmm, sddmm::wmmaSddmm, sddmm::cudaSddmm); compat_check calls all
twelve.  Patterns are synthetic (the DLMC files the reference reads are not available)."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DRIVERS = os.path.join(ROOT, "vectorsparse_b200", "drivers")
BM = "synthetic:beta:64x320:s=0.8:seed=3"


@pytest.fixture(scope="module", autouse=True)
def built_drivers():
    """The programs are built by `python -m vectorsparse_b200.build` (and by __graft_entry__.build()); only a
    checkout that has none yet builds them here."""
    if not all(os.path.exists(os.path.join(DRIVERS, exe)) for exe in ("spmm_benchmark", "sddmm_benchmark", "compat_check")):
        from vectorsparse_b200 import build
        build.build_library()
        build.build_drivers()


def run(exe, *args, timeout=300):
    p = subprocess.run([os.path.join(DRIVERS, exe), *map(str, args)], capture_output=True, text=True, timeout=timeout)
    assert p.returncode == 0, f"{exe} {args}: rc {p.returncode}\n{p.stdout}\n{p.stderr}"
    return p.stdout


@pytest.mark.parametrize("kernel,V", [(0, 2), (0, 4), (0, 8), (1, 1), (1, 2), (1, 4), (1, 8)])
@pytest.mark.parametrize("mixed", [1, 0])
def test_spmm_benchmark_verifies(kernel, V, mixed):
    """bm k v kernel sort function sparse mixed; function = 1 compares with the sequential host product."""
    out = run("spmm_benchmark", BM, 128, V, kernel, 1, 1, 1, mixed)
    assert ("Using WMMA" if kernel == 0 else "Using CUDA") in out
    if kernel == 0 and mixed == 0:   # the float tensor-core overload computes nothing, in the reference and here
        assert "wmmaSpmm doesn't support float input." in out
        assert "does not agree" in out
        return
    assert f"V={V}" in out
    assert "Results verified: they agree." in out, out


@pytest.mark.parametrize("kernel,V,alg", [(0, 2, 0), (0, 4, 1), (0, 8, 0), (0, 8, 1), (0, 8, 2), (0, 8, 3), (1, 1, 0), (1, 2, 0),
                                          (1, 4, 0), (1, 8, 0)])
def test_sddmm_benchmark_verifies(kernel, V, alg):
    """bm k v kernel alg sort function sparse mixed."""
    out = run("sddmm_benchmark", BM, 128, V, kernel, alg, 1, 1, 1, 1)
    assert ("Using WMMA" if kernel == 0 else "Using CUDA") in out
    assert "Results verified: they agree." in out, out


def test_sddmm_benchmark_single_precision_says_unsupported():
    for kernel, name in ((0, "wmmaSddmm"), (1, "cudaSddmm")):
        out = run("sddmm_benchmark", BM, 64, 8, kernel, 1, 1, 0, 1, 0)
        assert f"{name} doesn't support float input." in out


def test_selectors_that_are_not_built_say_so():
    assert "not built here" in run("spmm_benchmark", BM, 128, 8, 2, 1, 0, 1, 1)      # sputnik
    assert "not built here" in run("spmm_benchmark", BM, 128, 8, 3, 1, 0, 1, 1)      # cuSPARSE
    assert "not built here" in run("spmm_benchmark", BM, 128, 8, 0, 1, 0, 0, 1)      # dense cuBLAS
    assert "not built here" in run("sddmm_benchmark", BM, 128, 8, 2, 1, 1, 0, 1, 1)
    assert "not built here" in run("sddmm_benchmark", BM, 128, 8, 0, 1, 1, 0, 0, 1)


def test_unsupported_vector_length_is_announced_like_the_reference():
    for kernel in (0, 1):
        out = run("spmm_benchmark", BM, 128, 3, kernel, 1, 0, 1, 1)
        assert "Unsupported Vector Length!" in out
    assert "Unsupported Vector Length!" in run("spmm_benchmark", BM, 128, 1, 0, 1, 0, 1, 1)   # V = 1 has no tensor-core kernel


def test_smtx_pattern_file(tmp_path):
    """A pattern file in the reference's .smtx format (rows = vector rows) instead of a synthetic spec."""
    from vectorsparse_b200 import cvse
    a = cvse.generate(cvse.GEN_BETA, 5, 48, 256, 8, 0.85)
    path = str(tmp_path / "layer.smtx")
    cvse.to_smtx(path, a)
    out = run("spmm_benchmark", path, 256, 8, 0, 1, 1, 1, 1)
    assert "Results verified: they agree." in out
    out = run("sddmm_benchmark", path, 64, 8, 0, 1, 1, 1, 1, 1)
    assert "Results verified: they agree." in out


@pytest.mark.parametrize("V", [2, 4, 8])
def test_all_twelve_overloads_of_the_compat_header(V):
    out = run("compat_check", V)
    assert "all 12 overloads agree" in out, out
    assert out.count(" ok ") == 12


@pytest.mark.parametrize("job,kernel,V", [("spmm", "wmma", 8), ("spmm", "cuda", 4), ("sddmm", "wmma", 8), ("sddmm", "cuda", 2)])
def test_profile_harness_runs_the_driver(job, kernel, V):
    """python -m vectorsparse_b200.profile with the reference harness's options (ncu_profile.py:8-25), --func and no
    --prof: the driver is run directly and verifies its result."""
    cmd = [sys.executable, "-m", "vectorsparse_b200.profile", "--bm", BM, "-k", "128", "-v", str(V), "--kernel", kernel, "--sort",
           "--job", job, "--precision", "half", "--func"]
    p = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stdout + p.stderr
    assert ("spmm_benchmark" if job == "spmm" else "sddmm_benchmark") in p.stdout.splitlines()[0]
    assert "Results verified: they agree." in p.stdout, p.stdout
