"""DSD / SDD / dense kernels through the C ABI vs the CPU oracle.

Structure follows the reference's test/test_cuda.py:13-57 — one mask handed to both implementations,
forward + dX + dW in one test, its (m, n, k) x p grid including the degenerate ends — with the tolerance
of this build's contract: rtol 1e-2 / atol 1e-2 for 16-bit inputs with fp32 accumulation (the reference
accepts atol 0.2 on unscaled inputs).  Inputs are N(0, K^-1/2) so outputs are O(1).
"""
from itertools import product

import numpy as np
import pytest
import torch

from oracle import masked_dense as md
from oracle import philox_mask as pm

pytestmark = pytest.mark.gpu

RTOL = ATOL = 1e-2
DEV = torch.device("cuda:0")


def _inputs(M, N, K, seed, dtype=torch.float16):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(M, K, generator=g) * K ** -0.25).to(dtype)
    w = (torch.randn(N, K, generator=g) * K ** -0.25).to(dtype)
    dy = (torch.randn(M, N, generator=g) * N ** -0.25).to(dtype)
    return x, w, dy


def _close(got, want, what):
    torch.testing.assert_close(got.float().cpu(), want, rtol=RTOL, atol=ATOL, msg=lambda m: f"{what}: {m}")


mnks = [(128, 128, 128), (512, 512, 512), (1024, 1024, 1024), (2048, 2048, 2048)]
ps = [0.0, 0.1, 0.2, 0.5, 0.9, 0.99, 0.999]


@pytest.mark.parametrize("mnk,p", list(product(mnks, ps)))
def test_blockwise_dropout_matmul_reference_grid(built_lib, mnk, p):
    """Through the reference-shaped GEMM facade (split schedule with the cached workspace)."""
    from flash_dropout.cuda.binding_gemm import GEMM
    M, N, K = mnk
    x, w, dy = _inputs(M, N, K, seed=0)
    mask_np = pm.block_mask(M, K, 128, p, seed=0, offset=int(p * 1000))
    y_ref, dx_ref, dw_ref = md.forward_backward(x, mask_np, 128, p, w, dy)
    ext = GEMM()
    mask = torch.from_numpy(mask_np).to(DEV)
    A, B, dC = x.to(DEV), w.to(DEV), dy.to(DEV)
    s = 1 / (1 - p)
    C = ext.gemm_dsd(A, B, mask, 128, s)
    dA = ext.gemm_sdd(dC, B.T, mask, 128, s)
    dB = ext.gemm_dsd(A.T, dC.T, mask.T, 128, s).T
    _close(C, y_ref, "C")
    _close(dB, dw_ref, "dB")
    _close(dA, dx_ref, "dA")
    # dropped blocks of dA are exact zeros (matmul_sdd.cuh:64-65 writes them too)
    keep = md._keep_matrix(mask_np, M, K, 128)
    assert (dA.float().cpu()[keep == 0] == 0).all()


def test_golden_cases_from_the_reference(built_lib, golden):
    """fp16 kernels on the very inputs the reference saw, against the reference's own fp32 outputs."""
    from flash_dropout.cuda.binding_gemm import GEMM
    ext = GEMM()
    ran = 0
    for i in range(int(golden["mm_count"])):
        M, N, K, bs, _ = (int(v) for v in golden[f"mm{i}_cfg"])
        if bs % 128:
            continue
        p = float(golden[f"mm{i}_p"])
        x, w, dy = (torch.from_numpy(golden[f"mm{i}_{n}"]).to(DEV) for n in ("x", "w", "dy"))
        mask = torch.from_numpy(golden[f"mm{i}_mask"]).to(DEV)
        s = 1 / (1 - p)
        _close(ext.gemm_dsd(x, w, mask, bs, s), torch.from_numpy(golden[f"mm{i}_y"]), f"y[{i}]")
        _close(ext.gemm_sdd(dy, w.T, mask, bs, s), torch.from_numpy(golden[f"mm{i}_dx"]), f"dx[{i}]")
        _close(ext.gemm_dsd(x.T, dy.T, mask.T, bs, s).T, torch.from_numpy(golden[f"mm{i}_dw"]), f"dw[{i}]")
        ran += 1
    assert ran >= 3


@pytest.mark.parametrize("la,lb", list(product(("row", "col"), repeat=2)))
def test_all_operand_layouts(built_lib, la, lb):
    """The 4 (row|col)-major operand combinations of flash_dropout/cuda/binding_gemm.py:98-133 (2048^3, p=0.2)."""
    from flash_dropout.cuda.binding_gemm import GEMM
    M = N = K = 2048
    p = 0.2
    x, w, _ = _inputs(M, N, K, seed=1)
    A, B = x.to(DEV), w.to(DEV)
    if la == "col":
        A = A.T.contiguous().T
    if lb == "col":
        B = B.T.contiguous().T
    ext = GEMM()
    _close(ext.gemm(A, B), x.float() @ w.float().T, "gemm")
    mk = pm.block_mask(M, K, 128, p, seed=2)
    _close(ext.gemm_dsd(A, B, torch.from_numpy(mk).to(DEV), 128, 1 / (1 - p)), md.forward(x, mk, 128, p, w), "dsd")
    mn = pm.block_mask(M, N, 128, p, seed=3)
    want = (x.float() @ w.float().T) * md._keep_matrix(mn, M, N, 128) / (1 - p)
    _close(ext.gemm_sdd(A, B, torch.from_numpy(mn).to(DEV), 128, 1 / (1 - p)), want, "sdd")


@pytest.mark.parametrize("M,N,K,p", [(300, 264, 392, 0.4), (512, 1024, 784, 0.5), (129, 8, 136, 0.3),
                                      (1000, 136, 576, 0.5), (64, 64, 64, 0.0), (2048, 128, 640, 0.5)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_ragged_shapes_and_bf16(built_lib, M, N, K, p, dtype):
    """Shapes that are not multiples of 128 (the reference asserts divisibility, matmul_dsd.cuh:87-95)."""
    from flash_dropout import _lib
    from flash_dropout.cuda.binding_gemm import BlockPlan, dsd, sdd, sdd_kept_t
    x, w, dy = _inputs(M, N, K, seed=5, dtype=dtype)
    mask_np = pm.block_mask(M, K, 128, p, seed=6)
    y_ref, dx_ref, dw_ref = md.forward_backward(x, mask_np, 128, p, w, dy)
    plan = BlockPlan.from_mask(torch.from_numpy(mask_np).to(DEV), M, K, 128)
    A, B, dC = x.to(DEV), w.to(DEV), dy.to(DEV)
    s = 1 / (1 - p)
    tol = dict(rtol=RTOL, atol=ATOL) if dtype == torch.float16 else dict(rtol=2e-2, atol=4e-2)   # bf16: 8-bit mantissa
    torch.testing.assert_close(dsd(A, B, plan, _lib.SD_PLAN_ROWS, s).float().cpu(), y_ref, **tol)
    torch.testing.assert_close(sdd(dC, B.T, plan, s).float().cpu(), dx_ref, **tol)
    dW = torch.full((N, K), float("nan"), device=DEV, dtype=dtype)
    dsd(A.T, dC.T, plan, _lib.SD_PLAN_COLS, s, out=dW.T)          # transposed store straight into dW[N, K]
    torch.testing.assert_close(dW.float().cpu(), dw_ref, **tol)
    dXT = torch.zeros((K, M), device=DEV, dtype=dtype)            # dX^T = W^T . dY^T from the plan of the M x K mask
    sdd_kept_t(B.T, dC, plan, s, out=dXT)
    torch.testing.assert_close(dXT.T.float().cpu(), dx_ref, **tol)


def test_block_size_larger_than_tile(built_lib):
    from flash_dropout.cuda.binding_gemm import GEMM
    M, N, K, bs, p = 1024, 256, 1536, 256, 0.5
    x, w, dy = _inputs(M, N, K, seed=7)
    mask_np = pm.block_mask(M, K, bs, p, seed=8)
    y_ref, dx_ref, dw_ref = md.forward_backward(x, mask_np, bs, p, w, dy)
    mask = torch.from_numpy(mask_np).to(DEV)
    ext = GEMM()
    _close(ext.gemm_dsd(x.to(DEV), w.to(DEV), mask, bs, 2.0), y_ref, "y")
    _close(ext.gemm_sdd(dy.to(DEV), w.to(DEV).T, mask, bs, 2.0), dx_ref, "dx")
    _close(ext.gemm_dsd(x.to(DEV).T, dy.to(DEV).T, mask.T, bs, 2.0).T, dw_ref, "dw")


def test_full_size_properties_4096(built_lib):
    """The headline GEMM size (4096^3, p = 0.5): size-independent properties instead of a CPU oracle pass.

    With whole-tile shares (no workspace) every output element is one sequential fp32 accumulation over its
    kept K tiles, so:
    * skipping a dropped tile == multiplying by an explicitly zeroed tile, bit for bit (zeros add nothing
      to an fp32 accumulator), for all three products;
    * p = 0 plan == the dense kernel, bit for bit;
    * dropped tiles of dx are exact zeros; linearity in the scale.
    """
    from flash_dropout import _lib
    from flash_dropout.cuda import binding_gemm as bg
    from flash_dropout.cuda.binding_gemm import BlockPlan
    dense = lambda *a, **k: bg.dense(*a, ws=None, **k)
    dsd = lambda *a, **k: bg.dsd(*a, ws=None, **k)
    sdd = lambda *a, **k: bg.sdd(*a, ws=None, **k)
    M = N = K = 4096
    p = 0.5
    x, w, dy = (t.to(DEV) for t in _inputs(M, N, K, seed=9))
    plan = BlockPlan.from_seed(M, K, 128, p, 0, 0, DEV)
    assert np.array_equal(plan.mask.cpu().numpy(), pm.block_mask(M, K, 128, p, 0, 0))
    keep = (~plan.mask).repeat_interleave(128, 0).repeat_interleave(128, 1)
    xz = x * keep
    s = 1 / (1 - p)
    y = dsd(x, w, plan, _lib.SD_PLAN_ROWS, s)
    assert torch.equal(y, dense(xz, w, scale=s))
    dx = sdd(dy, w.T, plan, s)
    assert torch.equal(dx, dense(dy, w.T, scale=s) * keep)
    dw = torch.empty(N, K, device=DEV, dtype=torch.float16)
    dsd(x.T, dy.T, plan, _lib.SD_PLAN_COLS, s, out=dw.T)
    assert torch.equal(dw.T, dense(xz.T, dy.T, scale=s))
    full = BlockPlan.from_seed(M, K, 128, 0.0, 0, 0, DEV)
    assert torch.equal(dsd(x, w, full, _lib.SD_PLAN_ROWS, 1.0), dense(x, w))
    assert torch.equal(sdd(dy, w.T, full, 1.0), dense(dy, w.T))
    # all three products against fp32 matmuls of the masked operands (fp32 accumulate both sides)
    torch.testing.assert_close(y.float(), s * (xz.float() @ w.float().T), rtol=RTOL, atol=ATOL)
    torch.testing.assert_close(dx.float(), s * (dy.float() @ w.float()) * keep, rtol=RTOL, atol=ATOL)
    torch.testing.assert_close(dw.float(), s * (dy.float().T @ xz.float()), rtol=RTOL, atol=ATOL)
    torch.testing.assert_close(dsd(x, w, plan, _lib.SD_PLAN_ROWS, 2 * s).float(), 2 * y.float(), rtol=2e-3, atol=2e-3)


@pytest.mark.parametrize("la,lb", list(product(("row", "col"), repeat=2)))
def test_dense_variants_4096_against_fp32(built_lib, la, lb):
    """Every operand-major variant of the kernel at the full 4096^3 size against an fp32 matmul: descriptors, K
    walks and stores beyond 2048 rows and columns, for K-major and MN-major operands alike."""
    from flash_dropout.cuda import binding_gemm as bg
    M = N = K = 4096
    x, w, _ = (t.to(DEV) for t in _inputs(M, N, K, seed=13))
    A = x.T.contiguous().T if la == "col" else x
    B = w.T.contiguous().T if lb == "col" else w
    want = x.float() @ w.float().T
    torch.testing.assert_close(bg.dense(A, B, ws=None).float(), want, rtol=RTOL, atol=ATOL)
    torch.testing.assert_close(bg.dense(A, B).float(), want, rtol=RTOL, atol=ATOL)


# GEMM shapes (M, N, K, p) of the two training-step workloads, in the dtype those steps run in: the hidden layers
# of the 784-1024-1024-1024-10 MLP at batch 512, and the attention projections, c_fc and c_proj of the 6-layer
# d=384 char-GPT at 64 x 256 tokens.
TRAIN_SHAPES = [(512, 1024, 1024, 0.5), (512, 128, 1024, 0.5), (16384, 384, 384, 0.2), (16384, 1536, 384, 0.2),
                (16384, 384, 1536, 0.2)]


@pytest.mark.parametrize("M,N,K,p", TRAIN_SHAPES)
@pytest.mark.parametrize("use_ws", [True, False])
def test_training_step_shapes_bf16(built_lib, M, N, K, p, use_ws):
    """bf16 forward, dX and dW at the exact layer shapes of the MLP and GPT steps, with the workspace (dW of the
    16384-row layers takes the split schedule) and without it (whole tiles), against the oracle."""
    from flash_dropout import _lib
    from flash_dropout.cuda import binding_gemm as bg
    from flash_dropout.cuda.binding_gemm import BlockPlan
    ws = "auto" if use_ws else None
    x, w, dy = _inputs(M, N, K, seed=31, dtype=torch.bfloat16)
    mask_np = pm.block_mask(M, K, 128, p, seed=32, offset=M + K)
    y_ref, dx_ref, dw_ref = md.forward_backward(x, mask_np, 128, p, w, dy)
    plan = BlockPlan.from_mask(torch.from_numpy(mask_np).to(DEV), M, K, 128)
    A, B, dC = x.to(DEV), w.to(DEV), dy.to(DEV)
    s = 1 / (1 - p)
    tol = dict(rtol=2e-2, atol=4e-2)                              # bf16: 8-bit mantissa
    torch.testing.assert_close(bg.dsd(A, B, plan, _lib.SD_PLAN_ROWS, s, ws=ws).float().cpu(), y_ref, **tol)
    dX = bg.sdd(dC, B.T, plan, s, ws=ws)
    torch.testing.assert_close(dX.float().cpu(), dx_ref, **tol)
    assert (dX.float().cpu()[md._keep_matrix(mask_np, M, K, 128) == 0] == 0).all()
    dW = torch.full((N, K), float("nan"), device=DEV, dtype=torch.bfloat16)
    bg.dsd(A.T, dC.T, plan, _lib.SD_PLAN_COLS, s, out=dW.T, ws=ws)
    torch.testing.assert_close(dW.float().cpu(), dw_ref, **tol)


def test_equal_share_schedule_4096(built_lib):
    """Same workload with the workspace: shares are cut inside tiles and partial accumulators are added up in
    CTA order.  The regrouped fp32 sums may differ from the sequential ones by an fp16 rounding step, never
    more; results are reproducible run to run; dropped dx tiles stay exact zeros."""
    from flash_dropout import _lib
    from flash_dropout.cuda.binding_gemm import BlockPlan, dense, dsd, sdd
    M = N = K = 4096
    x, w, dy = (t.to(DEV) for t in _inputs(M, N, K, seed=9))
    for p in (0.0, 0.5, 0.9):
        plan = BlockPlan.from_seed(M, K, 128, p, 0, 0, DEV)
        keep = (~plan.mask).repeat_interleave(128, 0).repeat_interleave(128, 1)
        s = 1 / (1 - p)
        dw_a, dw_b = (torch.empty(N, K, device=DEV, dtype=torch.float16) for _ in range(2))
        pairs = [
            (dsd(x, w, plan, _lib.SD_PLAN_ROWS, s), dsd(x, w, plan, _lib.SD_PLAN_ROWS, s, ws=None)),
            (sdd(dy, w.T, plan, s), sdd(dy, w.T, plan, s, ws=None)),
            (dsd(x.T, dy.T, plan, _lib.SD_PLAN_COLS, s, out=dw_a.T).T, dsd(x.T, dy.T, plan, _lib.SD_PLAN_COLS, s, out=dw_b.T, ws=None).T),
        ]
        for split, whole in pairs:
            torch.testing.assert_close(split.float(), whole.float(), rtol=2e-3, atol=2e-3)
        assert (pairs[1][0][~keep] == 0).all()
        assert torch.equal(pairs[0][0], dsd(x, w, plan, _lib.SD_PLAN_ROWS, s))          # deterministic
        assert torch.equal(pairs[1][0], sdd(dy, w.T, plan, s))
    torch.testing.assert_close(dense(x, w).float(), x.float() @ w.float().T, rtol=RTOL, atol=ATOL)


@pytest.mark.parametrize("M,N,K", [(128, 256, 8192), (128, 128, 16384), (256, 512, 4096), (640, 384, 2048)])
def test_many_ctas_per_tile(built_lib, M, N, K):
    """Fewer output tiles than SMs: one tile is shared by many CTAs and its owner adds up many partials."""
    from flash_dropout import _lib
    from flash_dropout.cuda.binding_gemm import BlockPlan, dense, dsd, sdd
    x, w, dy = _inputs(M, N, K, seed=11)
    A, B, dC = x.to(DEV), w.to(DEV), dy.to(DEV)
    _close(dense(A, B), x.float() @ w.float().T, "dense")
    p = 0.5
    mask_np = pm.block_mask(M, K, 128, p, seed=12)
    y_ref, dx_ref, dw_ref = md.forward_backward(x, mask_np, 128, p, w, dy)
    plan = BlockPlan.from_mask(torch.from_numpy(mask_np).to(DEV), M, K, 128)
    _close(dsd(A, B, plan, _lib.SD_PLAN_ROWS, 2.0), y_ref, "y")
    _close(sdd(dC, B.T, plan, 2.0), dx_ref, "dx")
    _close(dsd(A.T, dC.T, plan, _lib.SD_PLAN_COLS, 2.0).T, dw_ref, "dw")
    for _ in range(3):      # flags are left cleared: back-to-back launches reuse the workspace
        _close(dsd(A.T, dC.T, plan, _lib.SD_PLAN_COLS, 2.0).T, dw_ref, "dw again")


@pytest.mark.parametrize("panels", [False, True])
def test_sdd_kept_t_with_many_tiles(built_lib, panels):
    """Transposed-plan SDD on a grid of hundreds of tiles (several tiles per CTA), flat and panel results."""
    from flash_dropout.cuda.binding_gemm import BlockPlan, sdd_kept_t, sdd_kept_t_panels
    M, N, K, p = 16384 + 64, 200, 640, 0.5                       # plan grid 129 x 5; ragged pixel count
    x, w, dy = _inputs(M, N, K, seed=21)
    mask_np = pm.block_mask(M, K, 128, p, seed=22)
    _, dx_ref, _ = md.forward_backward(x, mask_np, 128, p, w, dy)
    plan = BlockPlan.from_mask(torch.from_numpy(mask_np).to(DEV), M, K, 128)
    B, dC = w.to(DEV), dy.to(DEV)
    Mp = (M + 127) // 128 * 128
    if panels:
        out = torch.zeros((Mp // 128, K, 128), device=DEV, dtype=torch.float16)
        sdd_kept_t_panels(B.T, dC, plan, 2.0, out=out)
        dxT = out.permute(1, 0, 2).reshape(K, Mp)[:, :M]
    else:
        dxT = torch.zeros((K, M), device=DEV, dtype=torch.float16)
        sdd_kept_t(B.T, dC, plan, 2.0, out=dxT)
    _close(dxT.T, dx_ref, "dx^T")


def test_errors_mirror_the_reference(built_lib):
    """gemm_binding.cu:18-22,49-50,87-89 raise RuntimeError for device / rank / stride / dtype problems."""
    from flash_dropout.cuda.binding_gemm import GEMM
    ext = GEMM()
    a = torch.zeros(256, 256, device=DEV, dtype=torch.float16)
    mask = torch.zeros(2, 2, device=DEV, dtype=torch.bool)
    with pytest.raises(RuntimeError, match="CUDA"):
        ext.gemm_dsd(a.cpu(), a, mask, 128, 1.0)
    with pytest.raises(RuntimeError, match="2D"):
        ext.gemm_dsd(a[None], a, mask, 128, 1.0)
    with pytest.raises(RuntimeError, match="row or column major"):
        ext.gemm_dsd(a[:, ::2], a[:, ::2], mask[:, :1], 128, 1.0)
    with pytest.raises(RuntimeError, match="half"):
        ext.gemm_dsd(a.float(), a.float(), mask, 128, 1.0)
    with pytest.raises(RuntimeError, match="bool"):
        ext.gemm_dsd(a, a, mask.to(torch.uint8), 128, 1.0)
    with pytest.raises(RuntimeError, match="mask shape"):
        ext.gemm_dsd(a, a, mask[:1], 128, 1.0)
    with pytest.raises(ValueError, match="multiple of 128"):
        ext.gemm_dsd(a, a, mask, 64, 1.0)
    assert ext.gemm(a, a).abs().sum().item() == 0     # the context is still healthy


@pytest.mark.parametrize("M,N,K,p", [(512, 1024, 1024, 0.5), (384, 264, 640, 0.3), (2048, 2048, 2048, 0.5), (16384, 384, 1536, 0.2)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_fused_epilogues_against_oracle(built_lib, M, N, K, p, dtype):
    """The elementwise neighbours fused into the epilogues, each against fp32 PyTorch of the same composition on the
    oracle's products: ReLU after the forward, the ReLU-derivative mask on dX, and dW written / accumulated in fp32."""
    from flash_dropout import _lib
    from flash_dropout.cuda import binding_gemm as bg
    x, w, dy = _inputs(M, N, K, seed=41, dtype=dtype)
    x = torch.relu(x)                                             # the layer's input is the output of a ReLU
    mask_np = pm.block_mask(M, K, 128, p, seed=42, offset=N)
    y_ref, dx_ref, dw_ref = md.forward_backward(x, mask_np, 128, p, w, dy)
    plan = bg.BlockPlan.from_mask(torch.from_numpy(mask_np).to(DEV), M, K, 128)
    A, B, dC = x.to(DEV), w.to(DEV), dy.to(DEV)
    s = 1 / (1 - p)
    tol = dict(rtol=RTOL, atol=ATOL) if dtype == torch.float16 else dict(rtol=2e-2, atol=4e-2)
    y = bg.dsd(A, B, plan, _lib.SD_PLAN_ROWS, s, relu=True)
    torch.testing.assert_close(y.float().cpu(), torch.relu(y_ref), **tol)
    assert (y >= 0).all()
    dX = bg.sdd(dC, B.T, plan, s, relu_mask=A)
    torch.testing.assert_close(dX.float().cpu(), dx_ref * (x.float() > 0), **tol)
    assert (dX.float().cpu()[x.float() <= 0] == 0).all()
    # fp32 weight gradient: written, then accumulated on top
    dW = torch.full((N, K), float("nan"), device=DEV, dtype=torch.float32)
    bg.dsd(A.T, dC.T, plan, _lib.SD_PLAN_COLS, s, out=dW.T)
    tol32 = dict(rtol=5e-3, atol=5e-3 * max(1.0, M ** 0.5 / 16))  # fp32 store: only the 16-bit inputs round
    torch.testing.assert_close(dW.cpu(), dw_ref, **tol32)
    bg.dsd(A.T, dC.T, plan, _lib.SD_PLAN_COLS, s, out=dW.T, accumulate=True)
    torch.testing.assert_close(dW.cpu(), 2 * dw_ref, **tol32)
    dW2 = torch.zeros((N, K), device=DEV, dtype=torch.float32)
    bg.dsd(A.T, dC.T, plan, _lib.SD_PLAN_COLS, s, out=dW2.T, ws=None)      # whole tiles, no workspace
    torch.testing.assert_close(dW2.cpu(), dw_ref, **tol32)


@pytest.mark.parametrize("bs", [(128, 384), (256, 128), (512, 256)])
def test_rectangular_block_sizes(built_lib, bs):
    """block_size given as an (m, k) pair with m != k (eval/mlp/config.py:23-27 passes pairs): mask drawn on the
    device bit-exact vs the oracle, and the three products of the layer against the masked-dense oracle."""
    import flash_dropout.functional as F
    from flash_dropout import random as sd_random
    from flash_dropout.cuda.binding_gemm import BlockPlan
    M, N, K, p = 1024, 384, 1152, 0.5
    x, w, dy = _inputs(M, N, K, seed=51)
    sd_random.manual_seed(61, subsequence=0)
    plan = BlockPlan.draw(M, K, bs, p, DEV)
    mask_np = pm.block_mask(M, K, bs, p, seed=61, offset=0)
    assert np.array_equal(plan.mask.cpu().numpy(), mask_np)
    assert np.array_equal(plan.tile_mask.cpu().numpy().astype(bool), pm.expand_to_tiles(mask_np, M, K, bs))
    sd_random.manual_seed(61, subsequence=0)
    xa, wa = x.to(DEV).requires_grad_(), w.to(DEV).requires_grad_()
    y = F.cuda_blockwise_dropout_matmul(xa, wa, bs, p)
    y.backward(dy.to(DEV))
    y_ref, dx_ref, dw_ref = md.forward_backward(x, mask_np, bs, p, w, dy)
    _close(y, y_ref, "y")
    _close(xa.grad, dx_ref, "dx")
    _close(wa.grad, dw_ref, "dw")
    sd_random.follow_torch_seed()


def test_sm_margin_changes_only_the_grid(built_lib):
    """With SMs left free for a kernel running beside the products (flash_dropout.set_sm_margin) the three
    products of a full-grid layer give bit-identical results: the margin only changes how many CTAs share the tiles."""
    import flash_dropout
    from flash_dropout import _lib
    from flash_dropout.cuda.binding_gemm import BlockPlan, dsd, sdd
    M = N = K = 2048
    x, w, dy = _inputs(M, N, K, seed=71)
    xd, wd, dyd = x.to(DEV), w.to(DEV), dy.to(DEV)
    plan = BlockPlan.from_seed(M, K, 128, 0.5, 9, 0, DEV)

    def products():
        return (dsd(xd, wd, plan, _lib.SD_PLAN_ROWS, 2.0), sdd(dyd, wd.T, plan, 2.0),
                dsd(xd.T, dyd.T, plan, _lib.SD_PLAN_COLS, 2.0))
    base = products()
    prev = flash_dropout.set_sm_margin(24)
    try:
        assert prev == 0
        with_margin = products()
    finally:
        assert flash_dropout.set_sm_margin(prev) == 24
    torch.cuda.synchronize()
    for a, b, name in zip(base, with_margin, ("y", "dx", "dw")):
        assert torch.equal(a, b), name
    mask_np = pm.block_mask(M, K, 128, 0.5, seed=9, offset=0)
    y_ref, dx_ref, dw_ref = md.forward_backward(x, mask_np, 128, 0.5, w, dy)
    _close(with_margin[0], y_ref, "y")
    _close(with_margin[1], dx_ref, "dx")
    _close(with_margin[2].T, dw_ref, "dw")           # the third product is dW^T (K x N)
