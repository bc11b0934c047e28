"""The shared library loads and exports every function include/vsparse_b200.h declares; argument validation
rejects bad calls before anything touches a GPU."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from vectorsparse_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "vsparse_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(vs_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    names = declared_functions()
    assert len(names) >= 20
    handle = C.CDLL(_lib.LIB_PATH)
    for n in names:
        assert hasattr(handle, n), f"{n} declared in the header but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"
    assert set(_lib.SIGNATURES) == set(names)


def test_compat_header_names_the_reference_overloads():
    text = open(os.path.join(ROOT, "include", "vsparse_compat.h")).read()
    for ns, fn in (("spmm", "wmmaSpmm"), ("spmm", "cudaSpmm"), ("sddmm", "wmmaSddmm"), ("sddmm", "cudaSddmm")):
        assert f"namespace {ns}" in text
        assert len(re.findall(rf"\b{fn}\s*\(", text)) >= 3, fn  # three overloads each


def test_version_and_error_strings():
    L = _lib.lib()
    assert L.vs_version().decode().startswith("vsparse_b200")
    assert L.vs_error_string(0) == b"ok"
    assert L.vs_error_string(-1) == b"Unsupported Vector Length!"  # the reference's message (wmma_spmm.cu:346)
    for code in range(-9, 0):
        assert L.vs_error_string(code) not in (b"", b"unknown error")


def test_validation_happens_before_any_launch():
    """All of these return a negative code from the host-side checks (no CUDA device is needed)."""
    L = _lib.lib()
    buf = np.zeros(64, np.int32)
    p = buf.ctypes.data_as(C.c_void_p)
    T, CC, H, F = _lib.VS_PATH_TENSOR, _lib.VS_PATH_CUDA_CORE, _lib.VS_F16, _lib.VS_F32

    def spmm(path, i, o, m_vec, V, k, n, ptr=p):
        return L.vs_spmm(path, i, o, m_vec, V, k, n, ptr, ptr, ptr, ptr, ptr, ptr, None)

    assert spmm(T, H, H, 4, 3, 64, 8) == -1          # V = 3
    assert spmm(T, H, H, 4, 1, 64, 8) == -1          # tensor path has no V = 1 (wmmaSpmmEx switch)
    assert spmm(CC, H, H, 4, 16, 64, 8) == -1
    assert spmm(T, F, F, 4, 8, 64, 8) == -2          # float wmmaSpmm: unsupported in the reference too
    assert spmm(CC, F, H, 4, 8, 64, 8) == -2
    assert spmm(T, H, H, 4, 8, 96, 8) == -3          # tensor path needs k % 64 == 0
    assert spmm(CC, H, H, 4, 8, 12, 8) == -3
    assert spmm(CC, F, F, 4, 8, 6, 8) == -3
    assert spmm(CC, H, H, -1, 8, 64, 8) == -3
    assert spmm(CC, H, H, 4, 8, 64, 8, None) == -4
    assert spmm(7, H, H, 4, 8, 64, 8) == -8
    assert spmm(CC, H, H, 0, 8, 64, 8, None) == 0    # nothing to do is not an error
    odd = C.c_void_p(buf.ctypes.data + 4)
    assert L.vs_spmm(CC, H, H, 4, 8, 64, 8, p, p, p, odd, p, p, None) == -5

    def sddmm(path, i, o, V, k, alg=0, ptr=p, nnz=4):
        return L.vs_sddmm(path, i, o, 4, k, 8, nnz, ptr, ptr, ptr, ptr, ptr, ptr, V, None, alg)

    assert sddmm(T, H, H, 1, 64) == -1
    assert sddmm(T, F, F, 8, 64) == -2               # fp32 SDDMM: "doesn't support" in the reference
    assert sddmm(CC, F, F, 8, 64) == -2
    assert sddmm(T, H, H, 8, 32) == -3
    assert sddmm(T, H, H, 8, 64, alg=4) == -8
    assert sddmm(CC, H, F, 8, 12) == -3
    assert sddmm(CC, H, F, 8, 64, ptr=None) == -4
    assert sddmm(CC, H, F, 8, 64, ptr=None, nnz=0) == 0

    assert L.vs_spmm_batched(CC, H, H, 4, 8, 64, 8, p, p, p, p, p, p, 0, 0, 0, 0, None) == -8
    assert L.vs_spmm_batched(CC, H, H, 4, 8, 64, 8, p, p, p, p, p, p, 2, 0, 0, 0, None) == -8   # stride_out 0
    assert L.vs_spmm_batched(CC, H, H, 4, 8, 64, 8, p, p, p, p, p, p, 2, 4, 0, 64, None) == -5  # 8-byte stride
    assert L.vs_softmax_cvse(H, 4, 3, p, p, p, p, 1.0, 1, 0, None) == -1
    assert L.vs_softmax_cvse(5, 4, 8, p, p, p, p, 1.0, 1, 0, None) == -2
    assert L.vs_row_swizzle(2, 4, p, p) == -8
    assert L.vs_cvse_generate(9, 0, 4, 4, 8, 0.5, 0, p, None) == -8
    assert L.vs_cvse_generate(0, 0, 4, 4, 3, 0.5, 0, p, None) == -1
    assert L.vs_fill_random(7, 0, 0, 1.0, 4, p) == -2


def test_host_forms_validate_structure_first():
    L = _lib.lib()
    ro = np.array([0, 2, 1], np.int32)  # not monotone
    ci = np.array([0, 1], np.int32)
    z = np.zeros(256, np.float32)
    pv = lambda a: a.ctypes.data_as(C.c_void_p)
    rc = L.vs_spmm_host(_lib.VS_PATH_CUDA_CORE, _lib.VS_F32, _lib.VS_F32, 2, 1, 4, 4, pv(ro), pv(ro), pv(ci), pv(z), pv(z), pv(z))
    assert rc == -6


def test_sddmm_formulation_choice(monkeypatch):
    """Host-side choice between the dense and the gather tensor-core SDDMM: needs no device."""
    f = _lib.lib().vs_sddmm_formulation
    monkeypatch.delenv("VSPARSE_B200_SDDMM", raising=False)
    assert f(256, 256, 512, 12685, 8) == 1        # 90 % sparse, k = 256: dense tiles
    assert f(256, 256, 512, 600, 8) == 1          # 99.5 % sparse, narrow mask: the gather kernel's cost per vector-row still exceeds 16 dense tiles
    assert f(256, 256, 8192, 256 * 82, 8) == 0    # 99 % sparse and 8192 columns wide: 256 dense tiles for 21 K entries: gather
    assert f(512, 64, 4096, 209920, 8) == 0       # attention, head dimension 64: the sampling pass would dominate
    assert f(256, 256, 512, 12685, 1) == 0        # no tensor path at V = 1
    assert f(0, 256, 512, 0, 8) == 0
    monkeypatch.setenv("VSPARSE_B200_SDDMM", "dense")
    assert f(512, 64, 4096, 209920, 8) == 1
    monkeypatch.setenv("VSPARSE_B200_SDDMM", "gather")
    assert f(256, 256, 512, 12685, 8) == 0


def test_workspace_queries_and_setter():
    """Sizing a caller-owned plan scratch and handing it over need no device."""
    L = _lib.lib()
    b1 = L.vs_spmm_workspace_bytes(256, 8, 512, 1, 0)
    assert b1 >= 256 * 512 * 8                      # one entry per possible (vector-row, column)
    b256 = L.vs_spmm_workspace_bytes(256, 8, 512, 256, 12685 * 8)
    assert 12685 * 8 <= b256 < b1                   # a batch stride bounds the number of nonzero vectors
    assert L.vs_spmm_workspace_bytes(256, 1, 512, 1, 0) == 0      # no tensor path at V = 1
    assert L.vs_spmm_workspace_bytes(1 << 20, 8, 1 << 20, 1, 0) == 0   # beyond the 512 MB cap: gather kernels
    assert L.vs_sddmm_workspace_bytes(256, 512, 12685) >= 12685 * 8
    assert L.vs_sddmm_workspace_bytes(0, 512, 12685) == 0
    assert L.vs_set_workspace(None, 0) == 0
    assert L.vs_set_workspace(None, 64) == -8       # a size without a buffer
    assert L.vs_set_workspace(C.c_void_p(0x1008), 64) == -5      # not 16-byte aligned
    assert L.vs_set_workspace(C.c_void_p(0x1000), -1) == -8
    assert L.vs_set_workspace(None, 0) == 0
