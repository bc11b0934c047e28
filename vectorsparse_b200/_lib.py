"""ctypes binding of libvsparse_b200.so — the only way this package reaches its kernels.

There is no CPU or PyTorch fallback: if the library is missing the import fails with the build command.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# VSPARSE_B200_LIB selects another build of the same library (an instrumented one, for instance)
LIB_PATH = os.environ.get("VSPARSE_B200_LIB") or os.path.join(_HERE, "libvsparse_b200.so")

VS_F16, VS_F32 = 0, 1
VS_PATH_TENSOR, VS_PATH_CUDA_CORE = 0, 1

ERRORS = {
    -1: "VS_ERR_VEC_LENGTH", -2: "VS_ERR_DTYPE", -3: "VS_ERR_SHAPE", -4: "VS_ERR_NULL", -5: "VS_ERR_ALIGN",
    -6: "VS_ERR_STRUCTURE", -7: "VS_ERR_IO", -8: "VS_ERR_ARG", -9: "VS_ERR_DEVICE",
}


class VsError(RuntimeError):
    def __init__(self, code: int, where: str):
        self.code = code
        msg = lib().vs_error_string(code).decode()
        super().__init__(f"{where}: {ERRORS.get(code, 'cudaError ' + str(code))} ({msg})")


_I32P = C.POINTER(C.c_int32)
_vp, _i, _i64, _f = C.c_void_p, C.c_int, C.c_int64, C.c_float

# name -> (restype, argtypes); every symbol include/vsparse_b200.h declares
SIGNATURES = {
    "vs_error_string": (C.c_char_p, [_i]),
    "vs_version": (C.c_char_p, []),
    "vs_spmm": (_i, [_i, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "vs_spmm_batched": (_i, [_i, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i64, _i64, _i64, _vp]),
    "vs_spmm_t": (_i, [_i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "vs_spmm_t_batched": (_i, [_i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i64, _i64, _i64, _vp]),
    "vs_sddmm": (_i, [_i, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _vp, _i]),
    "vs_sddmm_batched": (_i, [_i, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i64, _i64, _i64, _vp, _i]),
    "vs_softmax_cvse": (_i, [_i, _i, _i, _vp, _vp, _vp, _vp, _f, _i, _i64, _vp]),
    "vs_attention_cvse": (_i, [_i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _f, _i, _vp]),
    "vs_softmax_cvse_backward": (_i, [_i, _i, _i, _vp, _vp, _vp, _vp, _f, _i, _i64, _vp]),
    "vs_attention_cvse_backward": (_i, [_i, _i, _i, _i, _i, _i] + [_vp] * 15 + [_f, _i, _vp]),
    "vs_attention_cvse_static": (_i, [_i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _f, _i, _vp]),
    "vs_spmm_host": (_i, [_i, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp]),
    "vs_sddmm_host": (_i, [_i, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i]),
    "vs_device_status": (_i, [_i, C.POINTER(C.c_uint32)]),
    "vs_measure_fp32_fma": (_i, [C.POINTER(C.c_double)]),
    "vs_kernel_timing": (_i, [_i, C.POINTER(C.c_double), C.POINTER(C.c_int)]),
    "vs_sddmm_formulation": (_i, [_i, _i, _i, _i, _i]),
    "vs_spmm_workspace_bytes": (_i64, [_i, _i, _i, _i, _i64]),
    "vs_sddmm_workspace_bytes": (_i64, [_i, _i, _i]),
    "vs_spmm_t_workspace_bytes": (_i64, [_i, _i, _i, _i, _i64]),
    "vs_set_workspace": (_i, [_vp, _i64]),
    "vs_release_scratch": (_i, [_vp, _i]),
    "vs_selftest_mma": (_i, [_vp, _i, _vp, _i, C.c_uint32, _i, _f, _vp, _vp]),
    "vs_selftest_mma_pair": (_i, [_vp, _vp, _i, _vp, _i, C.c_uint32, _i, _f, _vp, _vp]),
    "vs_selftest_gather4": (_i, [_vp, _i, _i, _vp, _i, _i, _vp, _vp]),
    "vs_cvse_validate": (_i, [_i, _i, _i, _vp, _vp]),
    "vs_row_swizzle": (_i, [_i, _i, _vp, _vp]),
    "vs_smtx_read_header": (_i, [C.c_char_p, C.POINTER(_i), C.POINTER(_i), C.POINTER(_i)]),
    "vs_smtx_read": (_i, [C.c_char_p, _i, _i, _vp, _vp]),
    "vs_smtx_write": (_i, [C.c_char_p, _i, _i, _i, _vp, _vp]),
    "vs_cvse_from_dense_mask": (_i, [_i, _i, _vp, _vp, _vp]),
    "vs_cvse_transpose": (_i, [_i, _i, _i, _vp, _vp, _vp, _vp, _vp]),
    "vs_cvse_prune_dense": (_i, [_i, _i, _i, _vp, C.c_double, _i, _vp, _vp, _vp]),
    "vs_cvse_generate": (_i, [_i, C.c_uint64, _i, _i, _i, C.c_double, _i, _vp, _vp]),
    "vs_fill_random": (_i, [_i, _i, C.c_uint64, C.c_double, _i64, _vp]),
}

_LIB = None


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m vectorsparse_b200.build` "
                "(needs nvcc; targets sm_100a). There is no fallback implementation.")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError here = the library is older than the header
            fn.restype = res
            fn.argtypes = args
        _LIB = handle
    return _LIB


def check(code: int, where: str) -> None:
    if code != 0:
        raise VsError(code, where)
