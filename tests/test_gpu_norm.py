"""Fused LayerNorm kernels against torch's fp32 LayerNorm: forward, dx, dgamma, dbeta; fp32 and 16-bit results."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")

SHAPES = [  # (leading shape, n, bias)
    ((64, 256), 384, False),          # the char-GPT rows: (batch, context, n_embed), no bias (eval/llm/model.py:72)
    ((1000,), 512, True),
    ((64,), 1024, True),              # widest row the kernels take
    ((33,), 4, True),                 # narrowest
    ((7, 5), 132, False),             # not a multiple of 128: the last vector of a lane is partly out of range
    ((3,), 768, True),
]


@pytest.mark.parametrize("lead,n,bias", SHAPES)
def test_layernorm_matches_torch_fp32(built_lib, lead, n, bias):
    from flash_dropout.layers.norm import LayerNorm
    g = torch.Generator().manual_seed(n + len(lead))
    x = (torch.randn(*lead, n, generator=g) * 2 + 0.5).to(DEV)
    dy = torch.randn(*lead, n, generator=g).to(DEV)
    ours = LayerNorm(n, bias=bias).to(DEV)
    ref = torch.nn.LayerNorm(n, bias=bias).to(DEV)
    with torch.no_grad():
        ours.weight.copy_(torch.randn(n, generator=g) * 0.5 + 1)
        if bias:
            ours.bias.copy_(torch.randn(n, generator=g))
    ref.load_state_dict(ours.state_dict())
    xa, xb = x.clone().requires_grad_(), x.clone().requires_grad_()
    ya, yb = ours(xa), ref(xb)
    assert ya.dtype == torch.float32 and ya.shape == yb.shape
    torch.testing.assert_close(ya, yb, rtol=1e-5, atol=1e-5)
    ya.backward(dy)
    yb.backward(dy)
    torch.testing.assert_close(xa.grad, xb.grad, rtol=1e-4, atol=1e-5)
    rows = x.numel() // n
    torch.testing.assert_close(ours.weight.grad, ref.weight.grad, rtol=1e-4, atol=1e-5 * rows ** 0.5)
    if bias:
        torch.testing.assert_close(ours.bias.grad, ref.bias.grad, rtol=1e-4, atol=1e-5 * rows ** 0.5)


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_layernorm_under_autocast_writes_the_consumer_dtype(built_lib, dt):
    """Under autocast the result comes out in the autocast dtype (what the Linear / DropoutMM behind it would cast it
    to), the gradient arrives in that dtype, and dx / dgamma equal torch's fp32 LayerNorm fed the same rounded tensors."""
    from flash_dropout.layers.norm import LayerNorm
    n, rows = 384, 4096
    g = torch.Generator().manual_seed(5)
    x = torch.randn(rows, n, generator=g).to(DEV)
    dy16 = torch.randn(rows, n, generator=g).to(DEV).to(dt)
    ours = LayerNorm(n, bias=False).to(DEV)
    with torch.no_grad():
        ours.weight.copy_(torch.rand(n, generator=g) + 0.5)
    xa = x.clone().requires_grad_()
    with torch.autocast("cuda", dtype=dt):
        ya = ours(xa)
    assert ya.dtype == dt
    xb = x.clone().requires_grad_()
    wb = ours.weight.detach().clone().requires_grad_()
    yb = F.layer_norm(xb, (n,), wb, None, ours.eps)
    torch.testing.assert_close(ya.float(), yb.to(dt).float(), rtol=0, atol=2 ** -6 if dt == torch.bfloat16 else 2 ** -9)
    ya.backward(dy16)
    yb.backward(dy16.float())
    torch.testing.assert_close(xa.grad, xb.grad, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(ours.weight.grad, wb.grad, rtol=1e-4, atol=1e-3)


def test_layernorm_falls_back_where_the_kernels_do_not_apply(built_lib):
    from flash_dropout.layers.norm import LayerNorm
    for n, dtype in ((1028, torch.float32), (386, torch.float32), (384, torch.bfloat16)):
        m = LayerNorm(n).to(DEV).to(dtype)
        x = torch.randn(8, n, device=DEV, dtype=dtype, requires_grad=True)
        y = m(x)
        torch.testing.assert_close(y, F.layer_norm(x, (n,), m.weight, m.bias, m.eps))
        y.sum().backward()
        assert x.grad is not None
