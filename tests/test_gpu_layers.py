"""Autograd op and modules on the GPU vs the CPU oracle (forward, dX, dW), plus the conv composition."""
import numpy as np
import pytest
import torch

from oracle import masked_dense as md
from oracle import philox_mask as pm

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
RTOL = ATOL = 1e-2


def test_autograd_op_matches_oracle(built_lib):
    import flash_dropout.functional as F
    from flash_dropout import random as sd_random
    M, N, K, p = 512, 384, 1024, 0.5
    g = torch.Generator().manual_seed(0)
    x = (torch.randn(M, K, generator=g) * K ** -0.25).half()
    w = (torch.randn(N, K, generator=g) * K ** -0.25).half()
    dy = (torch.randn(M, N, generator=g) * N ** -0.25).half()
    sd_random.manual_seed(77, subsequence=0)
    xa, wa = x.to(DEV).requires_grad_(), w.to(DEV).requires_grad_()
    y = F.cuda_blockwise_dropout_matmul(xa, wa, 128, p)
    y.backward(dy.to(DEV))
    mask = pm.block_mask(M, K, 128, p, seed=77, offset=0)        # first mask after manual_seed(77)
    y_ref, dx_ref, dw_ref = md.forward_backward(x, mask, 128, p, w, dy)
    torch.testing.assert_close(y.float().cpu(), y_ref, rtol=RTOL, atol=ATOL)
    torch.testing.assert_close(xa.grad.float().cpu(), dx_ref, rtol=RTOL, atol=ATOL)
    torch.testing.assert_close(wa.grad.float().cpu(), dw_ref, rtol=RTOL, atol=ATOL)
    assert wa.grad.is_contiguous() and xa.grad.dtype == torch.float16
    # the next call draws the next mask of the stream
    y2 = F.cuda_blockwise_dropout_matmul(xa, wa, 128, p)
    mask2 = pm.block_mask(M, K, 128, p, seed=77, offset=1)
    torch.testing.assert_close(y2.float().cpu(), md.forward(x, mask2, 128, p, w), rtol=RTOL, atol=ATOL)
    with pytest.raises(AssertionError):
        F.cuda_blockwise_dropout_matmul(xa, wa, 128, 1.0)
    with pytest.raises(RuntimeError):
        F.cuda_blockwise_dropout_matmul(xa.float(), wa, 128, 0.5)
    sd_random.follow_torch_seed()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_dropout_mm_under_autocast(built_lib, dtype):
    from flash_dropout import random as sd_random
    from flash_dropout.layers import DropoutMM
    torch.manual_seed(0)
    layer = DropoutMM(768, 256, p=0.5, variant="blockwise[cuda]", block_size=(128, 128)).to(DEV)
    x = torch.randn(4, 96, 768, device=DEV, requires_grad=True)
    sd_random.manual_seed(5, subsequence=1)
    with torch.autocast("cuda", dtype=dtype):
        y = layer(x)
    assert y.dtype == dtype and tuple(y.shape) == (4, 96, 256)
    dy = torch.randn_like(y)
    y.backward(dy)
    assert layer.weight.grad.dtype == torch.float32 and x.grad.dtype == torch.float32
    mask = pm.block_mask(384, 768, 128, 0.5, seed=5, offset=(1 << 40))
    xq, wq, dyq = x.detach().to(dtype).cpu().view(384, 768), layer.weight.detach().to(dtype).cpu(), dy.cpu().view(384, 256)
    y_ref, dx_ref, dw_ref = md.forward_backward(xq, mask, 128, 0.5, wq, dyq)
    tol = dict(rtol=1e-2, atol=1e-2) if dtype == torch.float16 else dict(rtol=2e-2, atol=4e-2)
    torch.testing.assert_close(y.float().cpu().view(384, 256), y_ref, **tol)
    torch.testing.assert_close(x.grad.cpu().view(384, 768), dx_ref, **tol)
    torch.testing.assert_close(layer.weight.grad.cpu(), dw_ref, **tol)
    layer.eval()
    torch.testing.assert_close(layer(x), torch.nn.functional.linear(x, layer.weight))
    sd_random.follow_torch_seed()


def test_dropout_conv2d_blockwise(built_lib):
    """Blockwise dropout on the im2col matrix: forward, dX (through fold) and dW vs the oracle."""
    from flash_dropout import random as sd_random
    from flash_dropout.layers import DropoutConv2d
    torch.manual_seed(1)
    N, C, H, W, Ko, p = 8, 64, 16, 16, 128, 0.5
    conv = DropoutConv2d(C, Ko, (3, 3), padding=(1, 1), p=p, variant="blockwise[cuda]", block_size=128).to(DEV).half()
    x = torch.randn(N, C, H, W, device=DEV, dtype=torch.float16, requires_grad=True)
    sd_random.manual_seed(9, subsequence=0)
    y = conv(x)
    assert tuple(y.shape) == (N, Ko, H, W)
    dy = (torch.randn_like(y) * 0.1)
    y.backward(dy)
    M, K = N * H * W, C * 9
    mask = pm.block_mask(M, K, 128, p, seed=9, offset=0)
    assert mask.shape == (16, 5)
    xc, kc = x.detach().cpu(), conv.weight.detach().cpu()
    y_ref = md.conv_forward(xc, kc, mask, 128, p, padding=(1, 1))
    dx_ref, dw_ref = md.conv_backward(xc, kc, mask, 128, p, dy.cpu(), padding=(1, 1))
    torch.testing.assert_close(y.float().cpu(), y_ref, rtol=RTOL, atol=ATOL)
    torch.testing.assert_close(conv.weight.grad.float().cpu(), dw_ref, rtol=RTOL, atol=2e-2)
    torch.testing.assert_close(x.grad.float().cpu(), dx_ref, rtol=RTOL, atol=2e-2)
    sd_random.follow_torch_seed()


def test_non_contiguous_grad_output(built_lib):
    import flash_dropout.functional as F
    x = torch.randn(256, 256, device=DEV, dtype=torch.float16, requires_grad=True)
    w = torch.randn(256, 256, device=DEV, dtype=torch.float16, requires_grad=True)
    y = F.cuda_blockwise_dropout_matmul(x, w, 128, 0.0)
    y.sum().backward()                                   # expanded (stride-0) upstream gradient
    torch.testing.assert_close(x.grad.float(), w.float().sum(0).expand(256, 256), rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("kind", ["mlp", "gpt"])
def test_training_step_consumers(built_lib, kind):
    """The two models of the training-step workloads run a few optimizer steps on the SparseDrop kernels."""
    from flash_dropout import random as sd_random
    from flash_dropout.train import GPT, BasicNet, FlatGradDataParallel, train_step
    torch.manual_seed(0)
    sd_random.manual_seed(3, subsequence=0)
    drop = dict(p=0.5 if kind == "mlp" else 0.2, variant="blockwise[cuda]", block_size=(128, 128))
    if kind == "mlp":
        model = BasicNet(784, 2, 1024, 10, drop).to(DEV)
        x, y = torch.rand(512, 28, 28, device=DEV), torch.randint(0, 10, (512,), device=DEV)
        loss_fn = lambda m: torch.nn.functional.cross_entropy(m(x).float(), y)
        opt = torch.optim.AdamW(model.parameters(), lr=1e-3, fused=True)
    else:
        model = GPT(65, 256, 2, 6, 384, drop).to(DEV)
        idx = torch.randint(0, 65, (16, 256), device=DEV)
        loss_fn = lambda m: m(idx)[1]
        opt = model.configure_optimizers(0.1, 1e-3)
    dp = FlatGradDataParallel(model)

    def eval_loss():
        model.eval()
        with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
            v = loss_fn(model).item()
        model.train()
        return v

    before = eval_loss()
    losses = [train_step(model, dp, opt, loss_fn, autocast_dtype=torch.bfloat16).item() for _ in range(30)]
    assert dp.grads_are_views()
    assert all(torch.isfinite(torch.tensor(losses)))
    assert eval_loss() < before                              # it learns the fixed batch
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in model.parameters())
    sd_random.follow_torch_seed()


def test_graphed_train_step_draws_fresh_masks(built_lib):
    """The captured step replays with new masks (device-side offset counter) and keeps learning."""
    from flash_dropout import random as sd_random
    from flash_dropout.train import BasicNet, FlatGradDataParallel, GraphedTrainStep
    torch.manual_seed(0)
    sd_random.manual_seed(11, subsequence=0)
    model = BasicNet(784, 2, 1024, 10, dict(p=0.5, variant="blockwise[cuda]", block_size=128)).to(DEV)
    x, y = torch.rand(512, 28, 28, device=DEV), torch.randint(0, 10, (512,), device=DEV)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3, fused=True)
    dp = FlatGradDataParallel(model)
    step = GraphedTrainStep(model, dp, opt, lambda m, a, b: torch.nn.functional.cross_entropy(m(a).float(), b),
                            (x, y), autocast_dtype=torch.bfloat16)
    counter = sd_random.device_counter(DEV)
    c0 = counter.item()
    losses = [step().item() for _ in range(20)]
    assert counter.item() == c0 + 20 * 4                      # four DropoutMM layers, one mask each per replay
    assert len(set(losses)) > 10 and all(np.isfinite(losses))
    assert dp.grads_are_views()
    model.eval()
    with torch.no_grad():
        final = torch.nn.functional.cross_entropy(model(x).float(), y).item()
    assert final < 2.30
    sd_random.disable_device_counter()
    sd_random.follow_torch_seed()


def test_fused_mlp_matches_unfused_composition(built_lib):
    """BasicNet on the CUDA variant fuses every ReLU into the neighbouring kernels and (under the data-parallel wrapper
    with fuse_wgrad) writes fp32 weight gradients straight into the flat buffer.  Same masks, same inputs: loss and
    all gradients must equal those of the plain composition (separate ReLU ops, autograd-accumulated gradients)."""
    from flash_dropout import random as sd_random
    from flash_dropout.train import BasicNet, FlatGradDataParallel
    torch.manual_seed(0)
    drop = dict(p=0.5, variant="blockwise[cuda]", block_size=(128, 128))
    fused = BasicNet(784, 2, 512, 10, drop).to(DEV)
    plain = BasicNet(784, 2, 512, 10, drop).to(DEV)
    plain.load_state_dict(fused.state_dict())
    x, y = torch.rand(256, 28, 28, device=DEV), torch.randint(0, 10, (256,), device=DEV)

    def plain_forward(m, inp):                                # the reference's forward, op by op
        h = torch.relu(m.in_proj(inp.flatten(1)))
        for layer in m.layers:
            h = torch.relu(layer(h))
        return m.out_proj(h)[..., : m.output_dim]

    dp = FlatGradDataParallel(fused, fuse_wgrad=True)
    assert all(hasattr(m.weight, "_sd_wgrad") for m in (fused.in_proj, fused.out_proj, *fused.layers))
    losses = []
    for model, fwd in ((fused, lambda m, a: m(a)), (plain, plain_forward)):
        sd_random.manual_seed(21, subsequence=0)              # both draw the same four masks
        if model is fused:
            dp.zero_grad()
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = torch.nn.functional.cross_entropy(fwd(model, x).float(), y)
        loss.backward()
        losses.append(loss.item())
    assert abs(losses[0] - losses[1]) < 1e-3
    assert dp.grads_are_views()
    for (n, a), (_, b) in zip(fused.named_parameters(), plain.named_parameters()):
        # identical products; the fused path rounds dW once less (fp32 store instead of bf16), hence a loose bound
        torch.testing.assert_close(a.grad, b.grad, rtol=2e-2, atol=2e-3, msg=lambda m, n=n: f"{n}: {m}")
    sd_random.follow_torch_seed()


def test_vit_consumer_trains_on_the_cuda_variant(built_lib):
    """The reference's third consumer (eval/vit/model.py): fused qkv DropoutMM, GELU feed-forward, on the SparseDrop
    kernels under bf16 autocast; a few optimizer steps on a fixed batch lower its loss."""
    from flash_dropout import random as sd_random
    from flash_dropout.train import ViT
    torch.manual_seed(0)
    sd_random.manual_seed(5, subsequence=0)
    x, y = torch.rand(32, 1, 32, 32, device=DEV), torch.randint(0, 10, (32,), device=DEV)
    model = ViT((x, y), 10, (2, 2), (8, 8), 256, 8, 2, dict(p=0.2, variant="blockwise[cuda]", block_size=(128, 128))).to(DEV)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3)
    losses = []
    for _ in range(25):
        opt.zero_grad()
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = torch.nn.functional.cross_entropy(model(x).float(), y)
        loss.backward()
        opt.step()
        losses.append(loss.item())
    assert all(np.isfinite(losses)) and min(losses[-5:]) < losses[0]
    sd_random.follow_torch_seed()


def test_convergence_smoke_on_synthetic_data(built_lib):
    """SparseDrop does not stop a model from learning: the MLP with p = 0.5, trained for 300 graph-replayed steps on
    a synthetic 10-class problem (ten fixed prototypes in pixel space plus heavy noise), classifies fresh samples
    of it, on the CUDA kernels as with the masked-dense path and with ordinary dropout."""
    from flash_dropout import random as sd_random
    from flash_dropout.train import BasicNet, FlatGradDataParallel, GraphedTrainStep
    torch.manual_seed(0)
    protos = torch.rand(10, 784, device=DEV)
    def batch(n, seed):
        g = torch.Generator(device=DEV).manual_seed(seed)
        ys = torch.randint(0, 10, (n,), device=DEV, generator=g)
        return (protos[ys] + 0.5 * torch.randn(n, 784, device=DEV, generator=g)).clamp_(0, 1), ys
    acc, first, last = {}, {}, {}
    for variant in ("blockwise[cuda]", "blockwise[naive]", "vanilla"):
        torch.manual_seed(1)
        sd_random.manual_seed(13, subsequence=0)
        model = BasicNet(784, 2, 512, 10, dict(p=0.5, variant=variant, block_size=128)).to(DEV)
        opt = torch.optim.AdamW(model.parameters(), lr=2e-3, fused=True)
        dp = FlatGradDataParallel(model, fuse_wgrad=True)
        xb, yb = batch(512, 0)
        step = GraphedTrainStep(model, dp, opt, lambda m, a, b: torch.nn.functional.cross_entropy(m(a).float(), b),
                                (xb, yb), autocast_dtype=torch.bfloat16)
        losses = []
        for i in range(300):
            xs, ys = batch(512, 100 + i)
            xb.copy_(xs); yb.copy_(ys)
            losses.append(step().clone())
        losses = torch.stack(losses).tolist()
        first[variant], last[variant] = sum(losses[:10]) / 10, sum(losses[-50:]) / 50
        model.eval()
        xt, yt = batch(4096, 7)
        with torch.no_grad():
            acc[variant] = (model(xt).argmax(1) == yt).float().mean().item()
        model.train()
        sd_random.disable_device_counter()
    sd_random.follow_torch_seed()
    assert all(a > 0.95 for a in acc.values()), acc
    assert all(last[v] < 0.5 * first[v] for v in acc), (first, last)
    # both SparseDrop paths draw the same mask stream, fresh on every replay: with whole 128-sample blocks dropped
    # their training loss stays noisy where a mask frozen into the graph would let it collapse to ~0
    assert last["blockwise[naive]"] > 0.05 and last["blockwise[cuda]"] > 0.05, last


def test_recompute_plan_gives_the_same_gradients(built_lib):
    """With ``recompute_plan`` the layer keeps only (seed, offset) of its mask and draws the plan again in backward:
    output and gradients are bit-identical to keeping the plan, and the autograd node holds no plan."""
    from flash_dropout import random as sd_random
    from flash_dropout.layers import DropoutMM
    sd_random.disable_device_counter()         # host-side offsets: the mode in which a plan can be drawn again
    torch.manual_seed(3)
    x = torch.randn(640, 1024, device=DEV, dtype=torch.float16)
    dy = torch.randn(640, 768, device=DEV, dtype=torch.float16)
    outs = []
    for recompute in (False, True):
        sd_random.manual_seed(77, subsequence=0)
        torch.manual_seed(4)
        layer = DropoutMM(1024, 768, p=0.5, variant="blockwise[cuda]", block_size=128, recompute_plan=recompute).to(DEV).half()
        xa = x.clone().requires_grad_()
        y = layer(xa)
        node = y.grad_fn
        while node is not None and not hasattr(node, "plan"):
            node = node.next_functions[0][0] if node.next_functions else None
        assert node is not None and (node.plan is None) == recompute
        if recompute:
            assert node.origin[4:] == (77, 0) and node.origin[:2] == (640, 1024)
        y.backward(dy)
        outs.append((y.detach(), xa.grad, layer.weight.grad))
    sd_random.follow_torch_seed()
    for a, b, name in zip(outs[0], outs[1], ("y", "dx", "dw")):
        assert torch.equal(a, b), name


def test_weight_shadows_equal_per_layer_casts_and_are_ignored_when_stale(built_lib):
    """One multi-tensor cast of all SparseDrop weights per step (``refresh_weight_shadows``) trains exactly like a
    cast per layer, and a layer whose weight changed after the copy was made goes back to casting for itself."""
    from flash_dropout import random as sd_random
    from flash_dropout.train import BasicNet, FlatGradDataParallel
    from flash_dropout.train.dp import train_step
    sd_random.disable_device_counter()
    g = torch.Generator().manual_seed(12)
    x = torch.rand(512, 784, generator=g).to(DEV)
    y = torch.randint(0, 10, (512,), generator=g).to(DEV)
    models = []
    for use_shadows in (False, True):
        torch.manual_seed(21)
        sd_random.manual_seed(31, subsequence=0)
        model = BasicNet(784, 2, 512, 10, dict(p=0.5, variant="blockwise[cuda]", block_size=128)).to(DEV)
        opt = torch.optim.AdamW(model.parameters(), lr=1e-3)
        dp = FlatGradDataParallel(model, fuse_wgrad=True)
        dp.shadow_min_layers = 1 if use_shadows else 10 ** 6      # the MLP has fewer layers than the default threshold
        for _ in range(3):
            train_step(model, dp, opt, lambda m: torch.nn.functional.cross_entropy(m(x).float(), y),
                       autocast_dtype=torch.bfloat16)
        models.append(model)
    for (na, pa), (nb, pb) in zip(models[0].named_parameters(), models[1].named_parameters()):
        assert torch.equal(pa, pb), na
    # the optimizer's last update made every copy stale: the layers must not use them
    stale = [p for p in models[1].parameters() if hasattr(p, "_sd_w16")]
    assert stale and all(p._sd_w16[1] != p._version for p in stale)
    outs = []
    for model in models:
        sd_random.manual_seed(41, subsequence=0)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            outs.append(model(x))
    assert torch.equal(outs[0], outs[1])
    sd_random.follow_torch_seed()
