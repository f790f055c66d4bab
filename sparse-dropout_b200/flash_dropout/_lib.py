"""ctypes binding of libsparsedrop.so (the C ABI declared in include/sparsedrop.h).

The library is built in-tree by ``csrc/build.sh`` into ``lib/libsparsedrop.so`` next to this
package.  There is no fallback: if the library is missing, or no CUDA device is present when a
kernel is requested, the call raises.
"""
from __future__ import annotations

import ctypes as C
import os
from functools import lru_cache

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(os.path.dirname(_HERE), "lib", "libsparsedrop.so")

SD_F16, SD_BF16, SD_F32 = 0, 1, 2
SD_PLAN_ROWS, SD_PLAN_COLS = 0, 1

#: every symbol include/sparsedrop.h declares
EXPORTS = (
    "sd_version", "sd_last_error", "sd_plan_bytes", "sd_plan_offsets", "sd_plan_from_seed", "sd_plan_from_seed_counter",
    "sd_plan_from_mask", "sd_workspace_bytes", "sd_workspace_init", "sd_gemm", "sd_gemm_dsd", "sd_gemm_sdd", "sd_gemm_sdd_kept", "sd_gemm_sdd_kept_t",
    "sd_gemm_dsd_static_scratch", "sd_im2col_kept", "sd_col2im_kept", "sd_im2col_kept_panels", "sd_col2im_kept_panels",
    "sd_gemm_dsd_panels", "sd_gemm_sdd_kept_t_panels", "sd_selftest_bounded_wait", "sd_check_status",
    "sd_conv_fused_supported", "sd_conv_dsd_fwd", "sd_conv_dsd_dw",
    "sd_gemm_dsd_relu", "sd_gemm_dsd_f32", "sd_gemm_sdd_relu_mask",
    "sd_plan_batch_desc_bytes", "sd_plan_batch_describe", "sd_plan_batch_launch", "sd_set_sm_margin",
    "sd_layernorm_fwd", "sd_layernorm_bwd_workspace_bytes", "sd_layernorm_bwd",
)


class PlanLayout(C.Structure):
    _fields_ = [(n, C.c_int64) for n in (
        "header", "row_ptr", "col_idx", "col_ptr", "row_idx", "kept_pairs", "drop_pairs",
        "row_order", "col_order", "sdd_items", "mask", "total_bytes")]


class SparseDropError(RuntimeError):
    pass


@lru_cache(maxsize=None)
def lib() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise SparseDropError(
            f"{LIB_PATH} not found: build it with sparse-dropout_b200/csrc/build.sh "
            "(there is no CPU or PyTorch fallback for the SparseDrop kernels)")
    L = C.CDLL(LIB_PATH)
    i64, i32, vp, f32, u64 = C.c_int64, C.c_int, C.c_void_p, C.c_float, C.c_uint64
    L.sd_version.restype = i32
    L.sd_last_error.restype = C.c_char_p
    L.sd_plan_bytes.restype = C.c_size_t
    L.sd_plan_bytes.argtypes = [i32, i32]
    L.sd_plan_offsets.restype = i32
    L.sd_plan_offsets.argtypes = [i32, i32, C.POINTER(PlanLayout)]
    L.sd_plan_from_seed.restype = i32
    L.sd_plan_from_seed.argtypes = [vp, i32, i32, i32, i32, u64, u64, f32, vp, vp]
    L.sd_plan_from_seed_counter.restype = i32
    L.sd_plan_from_seed_counter.argtypes = [vp, i32, i32, i32, i32, u64, u64, vp, f32, vp, vp]
    L.sd_plan_batch_desc_bytes.restype = C.c_size_t
    L.sd_plan_batch_desc_bytes.argtypes = [i32]
    L.sd_plan_batch_describe.restype = i32
    L.sd_plan_batch_describe.argtypes = [vp, vp, i32, i32, vp, i32, i32, i32, i32, u64, u64, vp, f32, vp]
    L.sd_plan_batch_launch.restype = i32
    L.sd_plan_batch_launch.argtypes = [vp, i32, vp]
    L.sd_plan_from_mask.restype = i32
    L.sd_plan_from_mask.argtypes = [vp, i32, i32, i32, i32, vp, i64, i64, vp]
    mat = [vp, i64, i64]
    L.sd_gemm.restype = i32
    L.sd_gemm.argtypes = mat * 3 + [i32, i32, i32, f32, i32, vp, vp, vp]
    L.sd_gemm_dsd.restype = i32
    L.sd_gemm_dsd.argtypes = mat * 3 + [i32, i32, i32, vp, i32, f32, i32, vp, vp, vp]
    L.sd_gemm_sdd.restype = i32
    L.sd_gemm_sdd.argtypes = mat * 3 + [i32, i32, i32, vp, f32, i32, vp, vp, vp]
    L.sd_gemm_sdd_kept.restype = i32
    L.sd_gemm_sdd_kept.argtypes = L.sd_gemm_sdd.argtypes
    L.sd_gemm_sdd_kept_t.restype = i32
    L.sd_gemm_sdd_kept_t.argtypes = L.sd_gemm_sdd.argtypes
    L.sd_gemm_dsd_static_scratch.restype = i32
    L.sd_gemm_dsd_static_scratch.argtypes = mat * 3 + [i32, i32, i32, vp, i32, f32, i32, vp, vp]
    L.sd_im2col_kept.restype = i32
    L.sd_im2col_kept.argtypes = [vp] + [i32] * 12 + [vp, i64, i32, vp, vp]
    L.sd_col2im_kept.restype = i32
    L.sd_col2im_kept.argtypes = [vp, i64, i32] + [i32] * 12 + [vp, vp, i32, vp]
    L.sd_im2col_kept_panels.restype = i32
    L.sd_im2col_kept_panels.argtypes = [vp] + [i32] * 12 + [vp, i32, vp, vp]
    L.sd_col2im_kept_panels.restype = i32
    L.sd_col2im_kept_panels.argtypes = [vp, i32] + [i32] * 12 + [vp, vp, i32, vp]
    L.sd_gemm_dsd_panels.restype = i32
    L.sd_gemm_dsd_panels.argtypes = [vp, i32, i32] + mat * 2 + [i32, vp, i32, f32, i32, vp, vp, vp]
    L.sd_gemm_sdd_kept_t_panels.restype = i32
    L.sd_gemm_sdd_kept_t_panels.argtypes = mat * 2 + [vp, i32, i32, i32, vp, f32, i32, vp, vp, vp]
    L.sd_gemm_dsd_relu.restype = i32
    L.sd_gemm_dsd_relu.argtypes = L.sd_gemm_dsd.argtypes
    L.sd_gemm_dsd_f32.restype = i32
    L.sd_gemm_dsd_f32.argtypes = mat * 3 + [i32, i32, i32, vp, i32, f32, i32, i32, vp, vp, vp]
    L.sd_gemm_sdd_relu_mask.restype = i32
    L.sd_gemm_sdd_relu_mask.argtypes = mat * 3 + [i32, i32, i32, vp, vp, i64, f32, i32, vp, vp, vp]
    L.sd_conv_fused_supported.restype = i32
    L.sd_conv_fused_supported.argtypes = [i32] * 12
    L.sd_conv_dsd_fwd.restype = i32
    L.sd_conv_dsd_fwd.argtypes = [vp] + [i32] * 12 + mat * 2 + [i32, vp, f32, i32, vp, vp, vp]
    L.sd_conv_dsd_dw.restype = i32
    L.sd_conv_dsd_dw.argtypes = [vp] + [i32] * 12 + mat * 2 + [i32, vp, f32, i32, vp, vp, vp]
    L.sd_selftest_bounded_wait.restype = i32
    L.sd_selftest_bounded_wait.argtypes = [vp, u64, vp]
    L.sd_workspace_bytes.restype = C.c_size_t
    L.sd_workspace_bytes.argtypes = []
    L.sd_workspace_init.restype = i32
    L.sd_workspace_init.argtypes = [vp, vp]
    L.sd_check_status.restype = i32
    L.sd_check_status.argtypes = [vp, vp]
    L.sd_set_sm_margin.restype = i32
    L.sd_set_sm_margin.argtypes = [i32]
    L.sd_layernorm_fwd.restype = i32
    L.sd_layernorm_fwd.argtypes = [vp, i32, i32, vp, vp, f32, vp, i32, vp, vp, vp]
    L.sd_layernorm_bwd_workspace_bytes.restype = C.c_size_t
    L.sd_layernorm_bwd_workspace_bytes.argtypes = [i32, i32]
    L.sd_layernorm_bwd.restype = i32
    L.sd_layernorm_bwd.argtypes = [vp, vp, i32, vp, vp, vp, i32, i32, vp, vp, vp, i32, vp, vp]
    return L


def check(rc: int) -> None:
    if rc != 0:
        raise SparseDropError(f"libsparsedrop error {rc}: {lib().sd_last_error().decode()}")


def require_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise SparseDropError(f"{name} must be CUDA")


def stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float16:
        return SD_F16
    if dt == torch.bfloat16:
        return SD_BF16
    raise SparseDropError(f"operands must be half or bfloat16, got {dt}")


def plan_layout(R: int, Cc: int) -> PlanLayout:
    out = PlanLayout()
    check(lib().sd_plan_offsets(R, Cc, C.byref(out)))
    return out
