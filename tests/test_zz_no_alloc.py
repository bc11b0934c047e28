"""vs_attention_cvse_static: fixed-mask attention for callers that cannot allocate device memory (a runtime that
pre-plans every buffer, a loop that must stay clear of cudaMalloc's device-wide synchronisation).  Its scratch
is an array inside the library, so the test checks, through the C ABI, that it gives exactly what
vs_attention_cvse gives with a caller workspace — on two calls in a row, the second on a different problem, since
the array keeps the first call's contents — and that an oversized request is refused before anything runs.

Collected last on purpose: a failure here must not hide the other tests from a run that stops at the first failure."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from conftest import assert_close
from vectorsparse_b200 import VS_PATH_CUDA_CORE, VS_PATH_TENSOR, _lib, cvse, ops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def attention_pair(path, seed, heads, n, band, sparsity, check_oracle=False):
    """Runs both entry points on one seeded problem; returns (with caller workspace, with built-in scratch)."""
    V, d = 8, 64
    a = cvse.generate(cvse.GEN_BAND, seed, n // V, n, V, sparsity, band=band)
    ri, ro, ci = a.to_device(DEV)
    q, k, v = (torch.from_numpy(cvse.fill_random((heads, n, d), np.float16, cvse.DIST_NORMAL, seed + i, 1.0)).to(DEV)
               for i in range(3))
    want = torch.full((heads, n, d), float("nan"), dtype=torch.float16, device=DEV)
    got = torch.full_like(want, float("nan"))
    ws = torch.empty((heads, a.nnz_vec * V), dtype=torch.float16, device=DEV)
    L = _lib.lib()
    stream = torch.cuda.current_stream().cuda_stream
    args = (path, a.m_vec, V, n, d, a.nnz_vec, ri.data_ptr(), ro.data_ptr(), ci.data_ptr(), q.data_ptr(),
            k.data_ptr(), v.data_ptr())
    assert L.vs_attention_cvse(*args, want.data_ptr(), ws.data_ptr(), C.c_float(0.125), heads, stream) == 0
    assert L.vs_attention_cvse_static(*args, got.data_ptr(), C.c_float(0.125), heads, stream) == 0
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    if check_oracle:   # the entry point against the fp64 oracle itself, not only against its sibling
        for h in range(heads):
            ref = oracle.attention(a.m_vec, V, d, d, a.row_offsets, a.col_indices, q[h].float().cpu().numpy(),
                                   k[h].float().cpu().numpy(), v[h].float().cpu().numpy(), 0.125)
            assert_close(got[h].float().cpu().numpy(), ref, f"static scratch, head {h}")
    return want, got


@pytest.mark.parametrize("path", [VS_PATH_TENSOR, VS_PATH_CUDA_CORE])
def test_two_calls_in_a_row_match_the_workspace_form(path, monkeypatch):
    # The no-allocation form always runs the row-gather tensor kernels (the dense formulations keep plan scratch);
    # the workspace form is pinned to the same ones here, so that the comparison can be bit for bit.
    monkeypatch.setenv("VSPARSE_B200_SPMM", "gather")
    monkeypatch.setenv("VSPARSE_B200_SDDMM", "gather")
    want, got = attention_pair(path, seed=31, heads=3, n=512, band=64, sparsity=0.8, check_oracle=True)
    assert not torch.isnan(got).any()
    assert torch.equal(got, want)          # same kernels in the same order: the results are bit-identical
    # second call: a smaller, different problem over the scratch the first call left behind
    want2, got2 = attention_pair(path, seed=77, heads=2, n=256, band=32, sparsity=0.7, check_oracle=True)
    assert not torch.isnan(got2).any()
    assert torch.equal(got2, want2)


def test_matches_the_default_formulations_within_tolerance(monkeypatch):
    """Left to choose, the workspace form may run the dense formulations: same values up to fp16 rounding."""
    monkeypatch.delenv("VSPARSE_B200_SPMM", raising=False)
    monkeypatch.delenv("VSPARSE_B200_SDDMM", raising=False)
    want, got = attention_pair(VS_PATH_TENSOR, seed=5, heads=2, n=512, band=64, sparsity=0.8)
    assert not torch.isnan(got).any()
    assert torch.allclose(got.float(), want.float(), rtol=0, atol=2e-2)


def test_requests_beyond_the_built_in_scratch_are_refused():
    L = _lib.lib()
    z = torch.zeros(64, dtype=torch.int32, device=DEV)
    p = z.data_ptr()
    # 64 heads x 100000 vectors x 8 values x 2 bytes = 102 MB > 8 MiB: rejected on the host, nothing launched
    rc = L.vs_attention_cvse_static(VS_PATH_TENSOR, 512, 8, 4096, 64, 100000, p, p, p, p, p, p, p, C.c_float(1.0), 64, None)
    assert rc == -3
    torch.cuda.synchronize()


def test_a_request_of_exactly_the_built_in_size_runs_and_one_vector_more_is_refused(monkeypatch):
    """4 heads x 131072 vectors x 8 values x 2 bytes = 8 388 608 bytes: the whole array, accepted and correct; one
    vector more per head is refused on the host."""
    monkeypatch.setenv("VSPARSE_B200_SPMM", "gather")
    monkeypatch.setenv("VSPARSE_B200_SDDMM", "gather")
    V, n, heads = 8, 2048, 4
    a = cvse.generate(cvse.GEN_BAND, 9, n // V, n, V, 0.75, band=128)
    assert heads * a.nnz_vec * V * 2 == 8 * 1024 * 1024, "the generator no longer gives 512 vectors per row"
    want, got = attention_pair(VS_PATH_TENSOR, seed=9, heads=heads, n=n, band=128, sparsity=0.75, check_oracle=True)
    assert torch.equal(got, want)
    z = torch.zeros(64, dtype=torch.int32, device=DEV)
    p = z.data_ptr()
    rc = _lib.lib().vs_attention_cvse_static(VS_PATH_TENSOR, n // V, V, n, 64, a.nnz_vec + 1, p, p, p, p, p, p, p, C.c_float(1.0),
                                             heads, None)
    assert rc == -3


def test_a_batch_whose_entries_would_be_misaligned_is_refused():
    """Probabilities of consecutive heads lie nonzeros_vec * V * 2 bytes apart in the scratch; when that is not a
    multiple of 16 bytes and there is more than one head, the call is refused (VS_ERR_ALIGN) before any launch."""
    z = torch.zeros(64, dtype=torch.int32, device=DEV)
    p = z.data_ptr()
    rc = _lib.lib().vs_attention_cvse_static(VS_PATH_TENSOR, 4, 2, 8, 64, 3, p, p, p, p, p, p, p, C.c_float(1.0), 2, None)
    assert rc == -5
    torch.cuda.synchronize()
    assert ops.device_status() == 0
