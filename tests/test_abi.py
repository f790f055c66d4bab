"""The C-ABI shared library: loads, exports every symbol the header declares, validates arguments.
No kernel is launched here (there is no GPU on the CPU test box)."""
import ctypes as C
import os
import re

from conftest import REPO


def _declared_symbols():
    text = open(os.path.join(REPO, "include", "sparsedrop.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(sd_[a-z_0-9]+)\s*\(", text)))


def test_exports_match_header(built_lib):
    from flash_dropout import _lib
    declared = _declared_symbols()
    assert declared, "no declarations parsed"
    for name in declared:
        assert hasattr(built_lib, name), f"{name} declared in include/sparsedrop.h but not exported"
    assert sorted(_lib.EXPORTS) == declared


def test_version_and_error_text(built_lib):
    assert built_lib.sd_version() >= 100
    assert isinstance(built_lib.sd_last_error(), bytes)


def test_plan_layout_is_consistent(built_lib):
    from flash_dropout import _lib
    for R, Cc in [(1, 1), (8, 8), (32, 32), (2048, 5), (3, 5), (128, 12)]:
        L = _lib.plan_layout(R, Cc)
        assert built_lib.sd_plan_bytes(R, Cc) == L.total_bytes
        offs = [L.header, L.row_ptr, L.col_idx, L.col_ptr, L.row_idx, L.kept_pairs, L.drop_pairs, L.row_order,
                L.col_order, L.sdd_items, L.mask, L.total_bytes]
        assert offs == sorted(offs) and all(o % 16 == 0 for o in offs)
        assert L.row_ptr - L.header >= 64
        assert L.col_idx - L.row_ptr >= 4 * (R + 1)
        assert L.kept_pairs - L.row_idx >= 4 * R * Cc
        assert L.total_bytes - L.mask >= R * Cc
    assert built_lib.sd_plan_bytes(0, 4) == 0


def test_argument_validation_without_a_gpu(built_lib):
    SD_ERR_INVALID_ARG, SD_ERR_LAYOUT = -1, -2
    buf = C.create_string_buffer(1 << 16)
    # p outside [0, 1): the reference asserts this in Python (blockwise_dropout_matmul_cuda.py:17)
    assert built_lib.sd_plan_from_seed(buf, 4, 4, 1, 1, 0, 0, 1.0, None, None) == SD_ERR_INVALID_ARG
    assert b"[0, 1)" in built_lib.sd_last_error()
    assert built_lib.sd_plan_from_seed(buf, 4, 4, 1, 1, 0, 0, -0.1, None, None) == SD_ERR_INVALID_ARG
    assert built_lib.sd_plan_from_mask(buf, 4, 4, 1, 1, None, 4, 1, None) == SD_ERR_INVALID_ARG
    # GEMM entry points reject bad sizes / dtypes / layouts before touching the device
    a = C.cast(buf, C.c_void_p)
    assert built_lib.sd_gemm(a, 128, 1, a, 128, 1, a, 128, 1, 0, 128, 128, 1.0, 0, None, None, None) == SD_ERR_INVALID_ARG
    assert built_lib.sd_gemm(a, 128, 1, a, 128, 1, a, 128, 1, 128, 128, 128, 1.0, 7, None, None, None) == SD_ERR_INVALID_ARG
    assert built_lib.sd_gemm(a, 128, 1, a, 128, 1, a, 128, 2, 128, 128, 128, 1.0, 0, None, None, None) == SD_ERR_LAYOUT
    assert built_lib.sd_gemm(a, 128, 2, a, 128, 1, a, 128, 1, 128, 128, 128, 1.0, 0, None, None, None) == SD_ERR_LAYOUT
    assert b"row or column major" in built_lib.sd_last_error()
    assert built_lib.sd_gemm(a, 100, 1, a, 128, 1, a, 128, 1, 128, 128, 128, 1.0, 0, None, None, None) == SD_ERR_LAYOUT
    assert built_lib.sd_gemm_dsd(a, 128, 1, a, 128, 1, a, 128, 1, 128, 128, 128, None, 0, 1.0, 0, None, None, None) \
        == SD_ERR_INVALID_ARG
    assert built_lib.sd_gemm_dsd(a, 128, 1, a, 128, 1, a, 128, 1, 128, 128, 128, a, 5, 1.0, 0, None, None, None) \
        == SD_ERR_INVALID_ARG
    assert built_lib.sd_gemm_sdd(a, 128, 1, a, 128, 1, None, 128, 1, 128, 128, 128, a, 1.0, 0, None, None, None) \
        == SD_ERR_INVALID_ARG
    # panel forms: the k extent of the panel matrix must be a multiple of 64
    assert built_lib.sd_gemm_dsd_panels(a, 256, 100, a, 128, 1, a, 128, 1, 128, a, 0, 1.0, 0, None, None, None) \
        == SD_ERR_LAYOUT
    assert b"multiple of 64" in built_lib.sd_last_error()
    assert built_lib.sd_gemm_dsd_panels(a, 256, 128, a, 128, 1, a, 128, 1, 128, a, 3, 1.0, 0, None, None, None) \
        == SD_ERR_INVALID_ARG
    assert built_lib.sd_gemm_sdd_kept_t_panels(a, 1, 136, a, 128, 1, a, 136, 256, 128, a, 1.0, 0, None, None, None) \
        == SD_ERR_LAYOUT
    assert built_lib.sd_im2col_kept_panels(None, 1, 1, 8, 8, 3, 3, 1, 1, 1, 1, 1, 1, a, 64, None, None) == SD_ERR_INVALID_ARG
    assert built_lib.sd_check_status(None, None) == SD_ERR_INVALID_ARG
    assert built_lib.sd_workspace_init(None, None) == SD_ERR_INVALID_ARG
    # SM margin: a process-wide setting, returns the previous value
    assert built_lib.sd_set_sm_margin(-1) == SD_ERR_INVALID_ARG
    prev = built_lib.sd_set_sm_margin(24)
    assert prev >= 0 and built_lib.sd_set_sm_margin(prev) == 24
