"""sd_gemm_dsd_static_scratch: the DSD product for callers that cannot give the library device memory.

Some hosts own every byte of device memory themselves (a serving process with a fixed pool, a loop that must
not pay the device-wide synchronisation of an allocation, a bare C caller), so they cannot allocate the
workspace sd_gemm_dsd() uses to spread a small product over the SMs.  This entry point uses scratch that is
compiled into the library instead.  The test calls it through the C ABI, twice in a row, and checks both
results against the regular entry point on the same inputs and plan.

Collected last on purpose (file name): a run that stops at the first failure has then already run everything else.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
RTOL = ATOL = 1e-2          # the GEMM tolerance of tests/test_gpu_gemm.py
SD_ERR_TOO_LARGE = -5


def _mat(t):
    return (t.data_ptr(), t.stride(0), t.stride(1))


@pytest.mark.parametrize("M,N,K,p,side", [(512, 512, 2048, 0.5, 0), (1024, 2048, 1024, 0.3, 0), (640, 384, 4096, 0.5, 1)])
def test_static_scratch_matches_regular_entry_point(built_lib, M, N, K, p, side):
    from flash_dropout import _lib
    from flash_dropout.cuda.binding_gemm import BlockPlan, dsd
    g = torch.Generator().manual_seed(M + N + K)
    a = (torch.randn(M, K, generator=g) * K ** -0.25).half().to(DEV)
    b = (torch.randn(N, K, generator=g) * K ** -0.25).half().to(DEV)
    if side == 0:     # forward: plan rows are A's row blocks
        plan = BlockPlan.from_seed(M, K, 128, p, 21, 0, DEV)
    else:             # dW form: A = x^T, plan columns are A's row blocks
        plan = BlockPlan.from_seed(K, M, 128, p, 21, 0, DEV)
    scale = 1.0 / (1.0 - p)
    want = dsd(a, b, plan, side, scale)                       # regular entry point, caller-allocated workspace
    stream = torch.cuda.current_stream(DEV).cuda_stream
    outs = []
    for _ in range(2):                                        # two calls in a row share the built-in array
        out = torch.full((M, N), float("nan"), device=DEV, dtype=torch.float16)
        rc = built_lib.sd_gemm_dsd_static_scratch(*_mat(a), *_mat(b), *_mat(out), M, N, K, plan.buf.data_ptr(), side,
                                                  scale, _lib.SD_F16, None, stream)
        assert rc == 0, built_lib.sd_last_error().decode()
        outs.append(out)
    torch.cuda.synchronize()
    for out in outs:
        assert not torch.isnan(out).any()
        torch.testing.assert_close(out.float(), want.float(), rtol=RTOL, atol=ATOL)
    assert torch.equal(outs[0], outs[1])


def test_static_scratch_rejects_products_beyond_its_limit(built_lib):
    from flash_dropout import _lib
    from flash_dropout.cuda.binding_gemm import BlockPlan
    M, N, K = 4096, 4096, 256                                 # 32 x 16 = 512 output tiles > 64
    a = torch.zeros(M, K, device=DEV, dtype=torch.float16)
    b = torch.zeros(N, K, device=DEV, dtype=torch.float16)
    out = torch.zeros(M, N, device=DEV, dtype=torch.float16)
    plan = BlockPlan.from_seed(M, K, 128, 0.5, 1, 0, DEV)
    rc = built_lib.sd_gemm_dsd_static_scratch(*_mat(a), *_mat(b), *_mat(out), M, N, K, plan.buf.data_ptr(), 0, 2.0,
                                              _lib.SD_F16, None, torch.cuda.current_stream(DEV).cuda_stream)
    assert rc == SD_ERR_TOO_LARGE
    assert b"exceed" in built_lib.sd_last_error()
    torch.cuda.synchronize()
