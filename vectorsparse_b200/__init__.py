"""vectorsparse_b200 — column-vector sparse SpMM / SDDMM for NVIDIA B200 (sm_100a).

Host side of libvsparse_b200.so: the CVSE builder (`cvse`), the operators named as in the vectorSparse
reference (`spmm.wmmaSpmm`, `spmm.cudaSpmm`, `sddmm.wmmaSddmm`, `sddmm.cudaSddmm`), batched forms, the masked
row softmax, fixed-mask sparse attention, and sharding helpers for several GPUs (`shard`).
"""
from . import _lib, cvse  # noqa: F401
from ._lib import VS_F16, VS_F32, VS_PATH_CUDA_CORE, VS_PATH_TENSOR, VsError  # noqa: F401

__all__ = ["cvse", "VsError", "VS_F16", "VS_F32", "VS_PATH_TENSOR", "VS_PATH_CUDA_CORE"]


def __getattr__(name):
    # torch-dependent parts are imported on first use so that the host-only builder works without CUDA
    if name in ("ops", "shard"):
        import importlib
        return importlib.import_module("." + name, __name__)
    if name in ("spmm", "sddmm", "spmm_batched", "sddmm_batched", "softmax_cvse", "attention_cvse", "device_status"):
        from . import ops
        return getattr(ops, name)
    raise AttributeError(name)
