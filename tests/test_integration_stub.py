"""The ctypes stub INTEGRATION.md shows a maintainer of the reference (a replacement for the reference's
flash_dropout/cuda/binding_gemm.py:7-47) is executed as written, so it cannot rot: the code block is cut out of
the document, pointed at the built library, and its GEMM facade is checked against the oracle."""
import os
import re

import pytest
import torch

from oracle import masked_dense as md
from oracle import philox_mask as pm

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _stub_namespace(built_lib):
    from flash_dropout import _lib
    text = open(os.path.join(REPO, "INTEGRATION.md")).read()
    blocks = re.findall(r"```python\n(.*?)```", text, flags=re.S)
    stub = next(b for b in blocks if "class GEMM" in b)
    assert "/path/to/libsparsedrop.so" in stub
    ns = {}
    exec(compile(stub.replace("/path/to/libsparsedrop.so", _lib.LIB_PATH), "INTEGRATION.md", "exec"), ns)
    return ns


def test_stub_loads_and_binds_every_symbol_it_names(built_lib):
    ns = _stub_namespace(built_lib)
    assert {"gemm", "gemm_dsd", "gemm_sdd"} <= set(dir(ns["GEMM"]))
    for name in ("sd_plan_bytes", "sd_plan_from_mask", "sd_gemm", "sd_gemm_dsd", "sd_gemm_sdd", "sd_last_error"):
        assert getattr(ns["_L"], name)
    assert ns["_L"].sd_plan_bytes(32, 32) > 0


@pytest.mark.gpu
def test_stub_products_match_the_oracle(built_lib):
    """The three calls the reference's autograd function makes (blockwise_dropout_matmul_cuda.py:21-26, 44-51)."""
    ext = _stub_namespace(built_lib)["GEMM"]()
    dev = torch.device("cuda:0")
    M, N, K, p = 512, 384, 640, 0.5
    g = torch.Generator().manual_seed(3)
    x = (torch.randn(M, K, generator=g) * K ** -0.25).half()
    w = (torch.randn(N, K, generator=g) * K ** -0.25).half()
    dy = (torch.randn(M, N, generator=g) * N ** -0.25).half()
    mask_np = pm.block_mask(M, K, 128, p, seed=4)
    y_ref, dx_ref, dw_ref = md.forward_backward(x, mask_np, 128, p, w, dy)
    mask = torch.from_numpy(mask_np).to(dev)
    A, B, dC = x.to(dev), w.to(dev), dy.to(dev)
    s = 1 / (1 - p)
    tol = dict(rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(ext.gemm(A, B).float().cpu(), x.float() @ w.float().T, **tol)
    torch.testing.assert_close(ext.gemm_dsd(A, B, mask, 128, s).float().cpu(), y_ref, **tol)
    torch.testing.assert_close(ext.gemm_sdd(dC, B.T, mask, 128, s).float().cpu(), dx_ref, **tol)
    torch.testing.assert_close(ext.gemm_dsd(A.T, dC.T, mask.T, 128, s).T.float().cpu(), dw_ref, **tol)
