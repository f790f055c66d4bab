"""sd_gemm_dsd_static_scratch: the DSD product for callers that cannot give the library device memory.

Some hosts own every byte of device memory themselves (a serving process with a fixed pool, a loop that must
not pay the device-wide synchronisation of an allocation, a bare C caller), so they cannot allocate the
workspace sd_gemm_dsd() uses to spread a small product over the SMs.  This entry point uses scratch that is
compiled into the library instead.  The test calls it through the C ABI, twice in a row, and checks both
results against the CPU oracle, against the regular entry point on the same inputs and plan, and that the
device's free memory did not change across the calls.  Every case is small enough (at most 32 output tiles, a
reduction of 16+ K tiles) that the kernel really takes the split schedule and parks partial tiles in the array.

Collected last on purpose (file name): a run that stops at the first failure has then already run everything else.
"""
import pytest
import torch

from oracle import masked_dense as md
from oracle import philox_mask as pm

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
TOL = {torch.float16: dict(rtol=1e-2, atol=1e-2),      # the GEMM tolerances of tests/test_gpu_gemm.py
       torch.bfloat16: dict(rtol=2e-2, atol=4e-2)}
SD_ERR_TOO_LARGE = -5


def _mat(t):
    return (t.data_ptr(), t.stride(0), t.stride(1))


@pytest.mark.parametrize("M,N,K,p,side,dtype", [
    (512, 512, 2048, 0.5, 0, torch.float16),
    (512, 1024, 4096, 0.3, 0, torch.float16),
    (640, 384, 4096, 0.5, 1, torch.float16),
    (500, 520, 2048, 0.5, 0, torch.bfloat16),           # ragged rows and columns
])
def test_static_scratch_matches_oracle_and_regular_entry_point(built_lib, M, N, K, p, side, dtype):
    from flash_dropout import _lib
    from flash_dropout.cuda.binding_gemm import BlockPlan, dsd
    assert -(-M // 128) * -(-N // 256) * 2 <= 64 and K >= 16 * 128      # the shape takes the split schedule
    g = torch.Generator().manual_seed(M + N + K)
    a_host = (torch.randn(M, K, generator=g) * K ** -0.25).to(dtype)
    b_host = (torch.randn(N, K, generator=g) * K ** -0.25).to(dtype)
    a, b = a_host.to(DEV), b_host.to(DEV)
    scale = 1.0 / (1.0 - p)
    if side == 0:     # forward: plan rows are A's row blocks; oracle = masked-dense forward
        mask_np = pm.block_mask(M, K, 128, p, seed=21, offset=0)
        oracle = md.forward(a_host, mask_np, 128, p, b_host)
    else:             # dW form: A = x^T for a layer input x (K x M); plan columns are A's row blocks
        mask_np = pm.block_mask(K, M, 128, p, seed=21, offset=0)
        # out = (keep o x)^T . b^T / (1-p) = dW^T for the upstream gradient dy = b^T
        _, dw = md.backward(a_host.T, mask_np, 128, p, torch.zeros(N, M), b_host.T)
        oracle = dw.T
    plan = BlockPlan.from_mask(torch.from_numpy(mask_np).to(DEV), *((M, K) if side == 0 else (K, M)), 128)
    regular = dsd(a, b, plan, side, scale)                    # regular entry point, caller-allocated workspace
    stream = torch.cuda.current_stream(DEV).cuda_stream
    code = _lib.dtype_code(dtype)
    outs = [torch.full((M, N), float("nan"), device=DEV, dtype=dtype) for _ in range(3)]

    def call(out):
        rc = built_lib.sd_gemm_dsd_static_scratch(*_mat(a), *_mat(b), *_mat(out), M, N, K, plan.buf.data_ptr(), side,
                                                  scale, code, None, stream)
        assert rc == 0, built_lib.sd_last_error().decode()

    call(outs[0])                                             # first call on the device: one-time address look-up
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info(DEV)
    torch_before = torch.cuda.memory_allocated(DEV)
    for out in outs[1:]:                                      # two calls in a row share the built-in array
        call(out)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info(DEV)
    assert free_after == free_before and torch.cuda.memory_allocated(DEV) == torch_before   # nothing was allocated
    for out in outs:
        assert not torch.isnan(out).any()
        torch.testing.assert_close(out.float().cpu(), oracle, **TOL[dtype])
        torch.testing.assert_close(out.float(), regular.float(), **TOL[dtype])
    assert torch.equal(outs[1], outs[2]) and torch.equal(outs[0], outs[1])


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
