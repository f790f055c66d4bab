"""Failure detection without a GPU fault: device-side waits are bounded and report through a status word.

The waits of the GEMM kernel (mbarrier waits between its roles, the arrival counter of the split schedule) all go
through two helpers that give up after a time limit, record a code and let the kernel finish normally.  The self-test
kernel runs exactly those helpers against a barrier nobody arrives on and a counter nobody increments, with a 20 ms
limit; afterwards the context must still run kernels."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
SD_ERR_TIMEOUT = -4


def test_bounded_waits_give_up_and_context_survives(built_lib):
    from flash_dropout.cuda.binding_gemm import dense
    words = torch.full((4,), -1, dtype=torch.int32, device=DEV)
    stream = torch.cuda.current_stream(DEV).cuda_stream
    assert built_lib.sd_selftest_bounded_wait(words.data_ptr(), 20_000_000, stream) == 0
    rc = built_lib.sd_check_status(words.data_ptr(), stream)           # synchronises and reads the status word
    assert rc == SD_ERR_TIMEOUT
    assert b"code 101" in built_lib.sd_last_error()
    status, counter, flags, elapsed_us = words.cpu().tolist()
    assert status == 101 and counter == 0
    assert flags == 4 | 8                                              # neither wait succeeded, both raised their flag
    assert 2 * 20_000 <= elapsed_us < 2_000_000                        # two waits of >= 20 ms each, far below a hang
    # the kernel returned normally: the same context keeps working
    a = torch.randn(256, 256, device=DEV, dtype=torch.float16)
    torch.testing.assert_close(dense(a, a).float(), a.float() @ a.float().T, rtol=1e-2, atol=1e-1)
    # a clean status word reports OK
    ok = torch.zeros(1, dtype=torch.int32, device=DEV)
    assert built_lib.sd_check_status(ok.data_ptr(), stream) == 0


def test_selftest_rejects_long_limits(built_lib):
    words = torch.zeros(4, dtype=torch.int32, device=DEV)
    assert built_lib.sd_selftest_bounded_wait(words.data_ptr(), 5_000_000_000, None) == -1
    assert built_lib.sd_selftest_bounded_wait(None, 1000, None) == -1


def test_operator_api_reports_a_timeout_and_recovers(built_lib):
    """Every launch of the operator API carries the device's status word.  A time-out recorded in that word (made
    here by the self-test kernel, whose waits nobody satisfies, run against the very same word) is raised by
    flash_dropout.check_status(), which also re-arms the split-schedule workspace; the next layer call works."""
    import flash_dropout
    import flash_dropout.functional as F
    from flash_dropout import _lib
    from flash_dropout.cuda import binding_gemm as bg
    from oracle import masked_dense as md
    from oracle import philox_mask as pm
    M, N, K, p = 256, 256, 4096, 0.5                          # 2 output tiles, 32 K tiles: the split schedule
    g = torch.Generator().manual_seed(0)
    x = (torch.randn(M, K, generator=g) * K ** -0.25).half()
    w = (torch.randn(N, K, generator=g) * K ** -0.25).half()
    mask_np = pm.block_mask(M, K, 128, p, seed=1)
    plan = bg.BlockPlan.from_mask(torch.from_numpy(mask_np).to(DEV), M, K, 128)
    want = md.forward(x, mask_np, 128, p, w)
    y = bg.dsd(x.to(DEV), w.to(DEV), plan, _lib.SD_PLAN_ROWS, 2.0)
    flash_dropout.check_status(DEV)                           # healthy: returns quietly
    torch.testing.assert_close(y.float().cpu(), want, rtol=1e-2, atol=1e-2)
    words = bg.status_word(DEV)
    stream = torch.cuda.current_stream(DEV).cuda_stream
    assert built_lib.sd_selftest_bounded_wait(words.data_ptr(), 5_000_000, stream) == 0
    ws = bg.workspace(DEV)
    ws[:8].fill_(1)                                           # what a launch that gave up may leave: dirty counters
    with pytest.raises(_lib.SparseDropError, match="bounded wait expired"):
        flash_dropout.check_status(DEV)
    assert words[0].item() == 0 and int(ws[:8].sum().item()) == 0     # word reset, workspace counters cleared
    flash_dropout.check_status(DEV)                           # and quiet again
    y2 = bg.dsd(x.to(DEV), w.to(DEV), plan, _lib.SD_PLAN_ROWS, 2.0)
    torch.testing.assert_close(y2.float().cpu(), want, rtol=1e-2, atol=1e-2)
    xa, wa = x.to(DEV).requires_grad_(), w.to(DEV).requires_grad_()
    F.cuda_blockwise_dropout_matmul(xa, wa, 128, p).sum().backward()  # the autograd op still runs
    flash_dropout.check_status(DEV)
