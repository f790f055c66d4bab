"""im2col / col2im stages (kept blocks only) and the SparseDrop convolution vs the CPU oracle."""
import numpy as np
import pytest
import torch
import torch.nn.functional as TF

from oracle import masked_dense as md
from oracle import philox_mask as pm

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")

GEOMS = [  # N, C, H, W, R, S, padding, stride, dilation
    (2, 16, 16, 16, 3, 3, (1, 1), (1, 1), (1, 1)),
    (3, 5, 9, 7, 3, 2, (0, 1), (2, 1), (1, 1)),
    (2, 8, 10, 10, 3, 3, (2, 2), (1, 2), (2, 2)),
    (1, 64, 32, 32, 3, 3, (1, 1), (1, 1), (1, 1)),
    (4, 3, 13, 11, 5, 5, (2, 2), (2, 2), (1, 1)),
    (3, 6, 12, 8, 2, 3, (0, 1), (1, 1), (2, 1)),      # 3-wide filter fast paths: 8-pixel rows, M = 240, R = 2, dilated rows
    (1, 20, 6, 64, 3, 3, (1, 1), (2, 1), (1, 1)),     # 64-pixel rows, vertical stride 2, K = 180 splits a tap triple
]


@pytest.mark.parametrize("geom", GEOMS)
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("panels", [False, True])
def test_im2col_and_col2im_against_unfold_fold(built_lib, geom, dtype, panels):
    """Bit-exact data movement: every kept block equals the unfold matrix, dropped blocks are left alone;
    col2im equals fold of the masked matrix (fp32 sum of at most R*S 16-bit values, rounded once)."""
    from flash_dropout.cuda.binding_gemm import BlockPlan
    from flash_dropout.functional.blockwise_dropout_conv2d import col2im_kept, im2col_kept
    N, C, H, W, R, S, pad, stride, dil = geom
    g = torch.Generator().manual_seed(N * 100 + C)
    x = torch.randn(N, C, H, W, generator=g).to(dtype)
    cols = TF.unfold(x.float(), (R, S), padding=pad, stride=stride, dilation=dil)      # (N, K, PQ)
    K, PQ = cols.shape[1], cols.shape[2]
    M = N * PQ
    want = cols.permute(1, 0, 2).reshape(K, M)                                           # colT
    Kg = (K + 63) & ~63 if panels else (K + 7) & ~7
    Mp = (M + 127) // 128 * 128 if panels else (M + 7) & ~7                              # columns that exist
    flat = (lambda t: t.permute(1, 0, 2).reshape(Kg, Mp)) if panels else (lambda t: t)  # panels -> colT[k][m]
    to_layout = (lambda t: t.view(Kg, Mp // 128, 128).permute(1, 0, 2).contiguous()) if panels else (lambda t: t)
    for p in (0.0, 0.5):
        mask = pm.block_mask(M, Kg, 128, p, seed=5)
        plan = BlockPlan.from_mask(torch.from_numpy(mask).to(DEV), M, Kg, 128)
        colT = torch.full((Kg, (M + 7) & ~7), 7.0, dtype=dtype, device=DEV)              # sentinel in dropped blocks
        got = flat(im2col_kept(x.to(DEV), (R, S), pad, stride, dil, plan, Kg, panels=panels))
        keep = md._keep_matrix(mask, M, Kg, 128).T.bool()[:K]                            # (K, M)
        assert torch.equal(got[:K, :M].float().cpu()[keep], want[keep])
        if Kg > K:
            assert (got[K:] == 0).all()
        # adjoint on a random cotangent
        dcol = torch.randn(Kg, Mp, generator=g).to(dtype)
        dcol_masked = dcol[:K, :M].float() * keep
        want_dx = TF.fold(dcol_masked.view(K, N, PQ).permute(1, 0, 2), (H, W), (R, S), padding=pad, stride=stride,
                          dilation=dil)
        got_dx = col2im_kept(to_layout(dcol.to(DEV)), (N, C, H, W), (R, S), pad, stride, dil, plan)
        torch.testing.assert_close(got_dx.float().cpu(), want_dx.to(dtype).float(), rtol=2e-2, atol=2e-2)
    dense = flat(im2col_kept(x.to(DEV), (R, S), pad, stride, dil, None, Kg, panels=panels))
    assert torch.equal(dense[:K, :M].float().cpu(), want)


FUSED_GEOMS = [  # geometries the fused im2col + DSD kernels serve (3-wide filter, unit horizontal stride, pad_w 1)
    (2, 16, 16, 16, 3, 3, (1, 1), (1, 1), (1, 1)),       # K = 144: a ragged second K block
    (1, 64, 32, 32, 3, 3, (1, 1), (1, 1), (1, 1)),       # the benchmark layer's shape for one image
    (3, 6, 12, 8, 2, 3, (0, 1), (1, 1), (2, 1)),         # 8-pixel rows, M = 240 (ragged last pixel block), R = 2, dilated rows
    (1, 20, 6, 64, 3, 3, (1, 1), (2, 1), (1, 1)),        # 64-pixel rows, vertical stride 2, K = 180
    (5, 24, 8, 8, 3, 3, (1, 1), (1, 1), (1, 1)),         # 8x8 images: a pixel block spans two images; K = 216
    (2, 43, 16, 32, 1, 3, (0, 1), (1, 1), (1, 1)),       # R = 1, K = 129: one k-row in the second block
]


@pytest.mark.parametrize("geom", FUSED_GEOMS)
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("Ko", [128, 40, 264])
def test_fused_conv_products_against_oracle(built_lib, geom, dtype, Ko):
    """sd_conv_dsd_fwd / sd_conv_dsd_dw (im2col gathered inside the GEMM kernel) against the masked-dense oracle on the
    unfold matrix, for p = 0 and p = 0.5, with and without the workspace."""
    from flash_dropout.cuda import binding_gemm as bg
    N, C, H, W, R, S, pad, stride, dil = geom
    assert bg.conv_fused_supported((N, C, H, W), (R, S), pad, stride, dil)
    g = torch.Generator().manual_seed(N * 100 + C + Ko)
    x = torch.randn(N, C, H, W, generator=g).to(dtype)
    cols = md.im2col_matrix(x, R, S, pad, stride, dil)                               # (M, K) fp32, unfold order
    M, K = cols.shape
    Kp, Kop = (K + 7) & ~7, (Ko + 7) & ~7
    w = (torch.randn(Ko, K, generator=g) * K ** -0.5).to(dtype)
    dy = (torch.randn(M, Ko, generator=g) * 0.5).to(dtype)
    w2d = torch.zeros(Kop, Kp, dtype=dtype)
    w2d[:Ko, :K] = w
    dy2d = torch.zeros(M, Kop, dtype=dtype)
    dy2d[:, :Ko] = dy
    tol = dict(rtol=1e-2, atol=1e-2) if dtype == torch.float16 else dict(rtol=2e-2, atol=4e-2)
    xd, w2dd, dy2dd = x.to(DEV), w2d.to(DEV), dy2d.to(DEV)
    for p, ws in ((0.5, "auto"), (0.0, "auto"), (0.5, None)):
        mask = pm.block_mask(M, K, 128, p, seed=17, offset=Ko)
        plan = bg.BlockPlan.from_mask(torch.from_numpy(mask).to(DEV), M, K, 128)
        s = 1 / (1 - p)
        y_ref, _, dw_ref = md.forward_backward(cols, mask, 128, p, w, dy)
        y2d = bg.conv_dsd_fwd(xd, w2dd, plan, (R, S), pad, stride, dil, s, ws=ws)
        torch.testing.assert_close(y2d[:, :Ko].float().cpu(), y_ref, **tol)
        assert (y2d[:, Ko:] == 0).all()
        dw2d = torch.full((Kop, Kp), float("nan"), dtype=dtype, device=DEV)
        bg.conv_dsd_dw(xd, dy2dd, plan, (R, S), pad, stride, dil, s, out=dw2d, ws=ws)
        scale = max(1.0, float(M) ** 0.5 / 8)                                        # |dW| grows with sqrt(M)
        torch.testing.assert_close(dw2d[:Ko, :K].float().cpu() / scale, dw_ref / scale, **tol)
    assert not bg.conv_fused_supported((N, C, H, W), (R, 2), pad, stride, dil)
    assert not bg.conv_fused_supported((N, C, H, W), (R, S), pad, (1, 2), dil)


@pytest.mark.parametrize("recompute,fused", [(False, True), (False, False), (True, False)])
@pytest.mark.parametrize("geom,Ko", [(GEOMS[0], 128), (GEOMS[1], 24), (GEOMS[2], 40), (GEOMS[4], 10), (GEOMS[5], 24),
                                     (GEOMS[6], 136)])
def test_conv_op_against_oracle(built_lib, geom, Ko, recompute, fused):
    import flash_dropout.functional as F
    from flash_dropout import random as sd_random
    N, C, H, W, R, S, pad, stride, dil = geom
    p = 0.5
    g = torch.Generator().manual_seed(Ko)
    x = torch.randn(N, C, H, W, generator=g).half()
    k = (torch.randn(Ko, C, R, S, generator=g) / (C * R * S) ** 0.5).half()
    xa, ka = x.to(DEV).requires_grad_(), k.to(DEV).requires_grad_()
    sd_random.manual_seed(31, subsequence=0)
    y = F.cuda_blockwise_dropout_conv2d(xa, ka, 128, p, padding=pad, stride=stride, dilation=dil,
                                        recompute_cols=recompute, fused=fused)
    P, Q = y.shape[2:]
    dy = (torch.randn(N, Ko, P, Q, generator=g) * 0.25).half()
    y.backward(dy.to(DEV))
    M, K = N * P * Q, C * R * S
    mask = pm.block_mask(M, K, 128, p, seed=31, offset=0)
    y_ref = md.conv_forward(x, k, mask, 128, p, pad, stride, dil)
    dx_ref, dk_ref = md.conv_backward(x, k, mask, 128, p, dy, pad, stride, dil)
    torch.testing.assert_close(y.float().cpu(), y_ref, rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(ka.grad.float().cpu(), dk_ref, rtol=1e-2, atol=2e-2)
    torch.testing.assert_close(xa.grad.float().cpu(), dx_ref, rtol=1e-2, atol=2e-2)
    sd_random.follow_torch_seed()


def test_conv_baseline_config_shapes(built_lib):
    """The benchmark conv layer at a reduced batch (N=16 of 256): 64 -> 128 channels, 32x32, 3x3, pad 1, p=0.5;
    mask grid (N*1024/128) x 5 with a ragged last K block (576 = 4.5 blocks)."""
    import flash_dropout.functional as F
    from flash_dropout import random as sd_random
    N = 16
    g = torch.Generator().manual_seed(0)
    x = torch.randn(N, 64, 32, 32, generator=g).half()
    k = (torch.randn(128, 64, 3, 3, generator=g) / 24).half()
    dy = torch.randn(N, 128, 32, 32, generator=g).half()
    xa, ka = x.to(DEV).requires_grad_(), k.to(DEV).requires_grad_()
    sd_random.manual_seed(1, subsequence=0)
    y = F.cuda_blockwise_dropout_conv2d(xa, ka, 128, 0.5, padding=(1, 1))
    y.backward(dy.to(DEV))
    mask = pm.block_mask(N * 1024, 576, 128, 0.5, seed=1, offset=0)
    assert mask.shape == (N * 8, 5)
    y_ref = md.conv_forward(x, k, mask, 128, 0.5, (1, 1))
    dx_ref, dk_ref = md.conv_backward(x, k, mask, 128, 0.5, dy, (1, 1))
    torch.testing.assert_close(y.float().cpu(), y_ref, rtol=1e-2, atol=1e-2)
    # dW sums 16384 products per element (sigma ~ 128): compare relative to that scale
    torch.testing.assert_close(ka.grad.float().cpu() / 128, dk_ref / 128, rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(xa.grad.float().cpu(), dx_ref, rtol=1e-2, atol=2e-2)
    sd_random.follow_torch_seed()


def test_conv_full_size_properties(built_lib):
    """The benchmark conv layer at its full size (256 x 64 x 32 x 32, 64 -> 128, 3x3, pad 1): size-independent properties.

    * p = 0 (nothing dropped): forward, dW and dx agree with cuDNN's dense convolution;
    * p = 0.5: the op equals the dense convolution machinery applied to an explicitly masked im2col matrix, checked
      through linearity — conv(x; mask) + conv(x; ~mask) == 2 * dense conv(x) / 1 (each scaled by 1/(1-p) = 2).
    """
    import flash_dropout.functional as F
    from flash_dropout.cuda.binding_gemm import BlockPlan
    torch.manual_seed(0)
    x = torch.randn(256, 64, 32, 32, device=DEV, dtype=torch.float16, requires_grad=True)
    k = (torch.randn(128, 64, 3, 3, device=DEV, dtype=torch.float16) / 24).requires_grad_()
    dy = torch.randn(256, 128, 32, 32, device=DEV, dtype=torch.float16).contiguous(memory_format=torch.channels_last)
    y = F.cuda_blockwise_dropout_conv2d(x, k, 128, 0.0, padding=(1, 1))
    y.backward(dy)
    gx, gk = x.grad.clone(), k.grad.clone()
    x.grad = k.grad = None
    yd = torch.nn.functional.conv2d(x, k, padding=1)
    yd.backward(dy)
    torch.testing.assert_close(y.float(), yd.float(), rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(gx.float(), x.grad.float(), rtol=1e-2, atol=2e-2)
    # dW sums 262144 products per element: compare on the scale of its magnitude
    scale = x.grad.new_tensor(512.0)
    torch.testing.assert_close(gk.float() / scale, k.grad.float() / scale, rtol=1e-2, atol=1e-2)
    # complementary masks add up to the dense result
    M, Kg = 256 * 1024, 576
    plan = BlockPlan.from_seed(M, Kg, 128, 0.5, 7, 0, DEV)
    anti = BlockPlan.from_mask(~plan.mask, M, Kg, 128)
    with torch.no_grad():
        ya = F.cuda_blockwise_dropout_conv2d(x, k, 128, 0.5, padding=(1, 1), plan=plan)
        yb = F.cuda_blockwise_dropout_conv2d(x, k, 128, 0.5, padding=(1, 1), plan=anti)
    torch.testing.assert_close((ya.float() + yb.float()) / 2, yd.float(), rtol=1e-2, atol=2e-2)
