"""Host-side mirror of the reference's operator / module API, on the CPU (no kernels)."""
import numpy as np
import pytest
import torch

import flash_dropout.functional as F
from flash_dropout import random as sd_random
from flash_dropout.functional.naive import blockwise_dropout_matmul_mask
from flash_dropout.functional.utils import blockwise_dropout_mask, mask_to_increment_table
from flash_dropout.layers import DropoutConv2d, DropoutMM


def test_functional_names_match_reference():
    # flash_dropout/functional/__init__.py:1-9
    for name in ("cuda_blockwise_dropout_matmul", "triton_blockwise_dropout_matmul", "im2col_conv2d",
                 "naive_blockwise_dropout_matmul", "vanilla_dropout_matmul"):
        assert callable(getattr(F, name))


def test_naive_matmul_against_reference(golden):
    for i in range(int(golden["mm_count"])):
        M, N, K, bs, _ = (int(v) for v in golden[f"mm{i}_cfg"])
        p = float(golden[f"mm{i}_p"])
        x = torch.from_numpy(golden[f"mm{i}_x"].astype(np.float32)).requires_grad_()
        w = torch.from_numpy(golden[f"mm{i}_w"].astype(np.float32)).requires_grad_()
        dy = torch.from_numpy(golden[f"mm{i}_dy"].astype(np.float32))
        y = blockwise_dropout_matmul_mask(x, torch.from_numpy(golden[f"mm{i}_mask"]), bs, p, w)
        y.backward(dy)
        torch.testing.assert_close(y.detach(), torch.from_numpy(golden[f"mm{i}_y"]), rtol=1e-5, atol=1e-5)
        torch.testing.assert_close(x.grad, torch.from_numpy(golden[f"mm{i}_dx"]), rtol=1e-5, atol=1e-5)
        torch.testing.assert_close(w.grad, torch.from_numpy(golden[f"mm{i}_dw"]), rtol=1e-5, atol=1e-5)


def test_naive_rejects_p_of_one():
    with pytest.raises(AssertionError):
        blockwise_dropout_matmul_mask(torch.zeros(128, 128), torch.zeros(1, 1, dtype=torch.bool), 128, 1.0,
                                      torch.zeros(8, 128))


def test_im2col_conv2d_against_reference(golden):
    for i in range(int(golden["conv_count"])):
        N, C, H, W, Ko, R, S, p0, p1, s0, s1, d0, d1 = (int(v) for v in golden[f"conv{i}_cfg"])
        y = F.im2col_conv2d(torch.from_numpy(golden[f"conv{i}_x"]), torch.from_numpy(golden[f"conv{i}_k"]),
                            padding=(p0, p1), stride=(s0, s1), dilation=(d0, d1))
        torch.testing.assert_close(y, torch.from_numpy(golden[f"conv{i}_y"]), rtol=1e-5, atol=1e-5)


def test_increment_table_against_reference(golden):
    for i in range(int(golden["inc_count"])):
        mask = torch.from_numpy(golden[f"inc{i}_mask"])
        table, row_indices, row_widths = mask_to_increment_table(mask, int(golden[f"inc{i}_block_k"]))
        assert np.array_equal(table.numpy(), golden[f"inc{i}_table"])
        assert np.array_equal(row_indices.numpy(), golden[f"inc{i}_row_indices"])
        assert np.array_equal(row_widths.numpy(), golden[f"inc{i}_row_widths"])


def test_cpu_mask_shape(golden):
    for M, K, bs, R, C, _, _ in golden["mask_shape_cases"]:
        m = blockwise_dropout_mask(torch.empty(int(M), int(K)), int(bs), 0.5)
        assert tuple(m.shape) == (R, C) and m.dtype == torch.bool
    assert tuple(blockwise_dropout_mask(torch.empty(2, 3, 256, 384), 128, 0.5).shape) == (2, 3, 2, 3)


def test_dropout_mm_variants_on_cpu():
    torch.manual_seed(0)
    x = torch.randn(4, 32, 256)
    for variant in ("none", "vanilla", "blockwise[naive]"):
        m = DropoutMM(256, 128, p=0.5, variant=variant, block_size=(128, 128))
        assert tuple(m.weight.shape) == (128, 256) and not hasattr(m, "bias")
        y = m(x)
        assert tuple(y.shape) == (4, 32, 128)
        y.sum().backward()
        assert m.weight.grad is not None
        m.eval()
        torch.testing.assert_close(m(x), torch.nn.functional.linear(x, m.weight))
    with pytest.raises(ValueError):
        DropoutMM(256, 128, variant="bogus")(x)
    rect = DropoutMM(256, 128, p=0.5, variant="blockwise[naive]", block_size=(64, 128))   # an (m, k) pair, m != k
    assert tuple(rect(x).shape) == (4, 32, 128)
    with pytest.raises(ValueError):
        DropoutMM(256, 128, variant="blockwise[naive]", block_size=(128, 64, 1))(x)
    none = DropoutMM(256, 128, p=0.9, variant="none")
    torch.testing.assert_close(none(x), torch.nn.functional.linear(x, none.weight))


def test_dropout_conv_variants_on_cpu():
    torch.manual_seed(0)
    x = torch.randn(2, 16, 8, 8)
    for variant in ("none", "im2col", "vanilla", "vanilla_2d", "blockwise[naive]"):
        c = DropoutConv2d(16, 32, (3, 3), padding=(1, 1), p=0.5, variant=variant, block_size=128)
        y = c(x)
        assert tuple(y.shape) == (2, 32, 8, 8)
        c.eval()
        torch.testing.assert_close(c(x), torch.nn.functional.conv2d(x, c.weight, padding=1))
    c = DropoutConv2d(16, 32, (3, 3), padding=(1, 1), variant="im2col")
    torch.testing.assert_close(c(x), torch.nn.functional.conv2d(x, c.weight, padding=1), rtol=1e-4, atol=1e-5)
    with pytest.raises(ValueError):
        DropoutConv2d(16, 32, (3, 3), variant="bogus")(x)


def test_mask_rng_state():
    sd_random.manual_seed(7, subsequence=0)
    a = [sd_random.next_seed_offset() for _ in range(3)]
    assert a == [(7, 0), (7, 1), (7, 2)]
    sd_random.manual_seed(7, subsequence=3)
    assert sd_random.next_seed_offset() == (7, 3 << 40)
    st = sd_random.get_state()
    b = sd_random.next_seed_offset()
    sd_random.set_state(st)
    assert sd_random.next_seed_offset() == b          # a resumed run replays its masks
    sd_random.follow_torch_seed()
    sd_random.set_subsequence(0)
    torch.manual_seed(123)
    assert sd_random.next_seed_offset() == (123, 0)
    assert sd_random.next_seed_offset() == (123, 1)
    torch.manual_seed(124)
    assert sd_random.next_seed_offset() == (124, 0)


def test_cuda_op_fails_loudly_without_cuda():
    if torch.cuda.is_available():
        pytest.skip("CUDA present")
    with pytest.raises(RuntimeError):
        F.cuda_blockwise_dropout_matmul(torch.zeros(128, 128, dtype=torch.float16),
                                        torch.zeros(128, 128, dtype=torch.float16), 128, 0.5)


def test_autocast_cast_cache_never_outlives_its_tensor():
    """The shared q/k/v input cast must hit only for the very same tensor, and must miss for a new tensor that the
    allocator happens to place at the address of a freed one (same shape, version 0)."""
    from flash_dropout.functional.blockwise_dropout_matmul_cuda import _autocast_input
    for _ in range(20):
        x1 = torch.randn(64, 32)
        kept = _autocast_input(x1, torch.float16)            # stays alive, as autograd would keep it for backward
        addr = x1.data_ptr()
        del x1
        x2 = torch.randn(64, 32)
        got = _autocast_input(x2, torch.float16)
        assert torch.equal(got, x2.half()), f"stale cast returned (same address reused: {x2.data_ptr() == addr})"
        assert kept is not got
    # the three projections of an attention block: fresh 2-D views of one 3-D activation share one cast
    x = torch.randn(2, 8, 32)
    a = _autocast_input(x.reshape(-1, 32), torch.float16)
    b = _autocast_input(x.reshape(-1, 32), torch.float16)
    assert a is b
    x.add_(1.0)                                              # an in-place update invalidates the entry
    c = _autocast_input(x.reshape(-1, 32), torch.float16)
    assert c is not a and torch.equal(c, x.reshape(-1, 32).half())
    # a different window of the same owner is a different tensor
    d = _autocast_input(x[0], torch.float16)
    e = _autocast_input(x[1], torch.float16)
    assert torch.equal(d, x[0].half()) and torch.equal(e, x[1].half())


def _load_reference_params(model, golden, prefix):
    names = [str(n) for n in golden[f"{prefix}_param_names"]]
    assert list(model.state_dict().keys()) == names          # same names in the same order as the reference's
    sd = {n: torch.from_numpy(golden[f"{prefix}_param/{n}"]) for n in names}
    for n, v in model.state_dict().items():
        assert tuple(v.shape) == tuple(sd[n].shape), n
    model.load_state_dict(sd, strict=True)


def test_models_load_reference_checkpoints(golden):
    """The restated MLP and char-GPT take the reference models' state_dict unchanged and reproduce their logits
    (eval/mlp/model.py:8-40, eval/llm/model.py:83-155; fixtures from the reference's own classes)."""
    from flash_dropout.train import GPT, BasicNet
    din, layers, hidden, dout = (int(v) for v in golden["mlp_cfg"])
    x = torch.from_numpy(golden["mlp_x"])
    for first_arg in (din, x):                               # width, or a sample batch as the reference passes
        mlp = BasicNet(first_arg, layers, hidden, dout, dict(p=0.5, variant="none", block_size=(128, 128))).train()
        _load_reference_params(mlp, golden, "mlp")
        torch.testing.assert_close(mlp(x), torch.from_numpy(golden["mlp_logits"]), rtol=1e-5, atol=1e-5)
    vocab, ctx, n_layer, n_head, n_embed = (int(v) for v in golden["gpt_cfg"])
    gpt = GPT(vocab, ctx, n_layer, n_head, n_embed, dict(p=0.2, variant="none", block_size=(128, 128))).train()
    _load_reference_params(gpt, golden, "gpt")
    logits, loss = gpt(torch.from_numpy(golden["gpt_idx"]))
    torch.testing.assert_close(logits, torch.from_numpy(golden["gpt_logits"]), rtol=1e-4, atol=1e-5)
    assert abs(loss.item() - float(golden["gpt_loss"])) < 1e-4
    opt = gpt.configure_optimizers(weight_decay=0.1, lr=1e-3, fused=False)
    decayed = {id(q) for q in opt.param_groups[0]["params"]}
    want = {str(n) for n in golden["gpt_decay_names"]}
    assert {n for n, q in gpt.named_parameters() if id(q) in decayed} == want
    assert opt.param_groups[0]["weight_decay"] == 0.1 and opt.param_groups[1]["weight_decay"] == 0.0


def test_vit_loads_reference_checkpoint(golden):
    """The restated ViT (eval/vit/model.py:73-124) takes the reference model's state_dict and reproduces its logits,
    including the block-grouped patch order of its einops rearrangement."""
    from flash_dropout.train import ViT
    classes, p1, p2, b1, b2, n_embed, n_head, n_layers = (int(v) for v in golden["vit_cfg"])
    x = torch.from_numpy(golden["vit_x"])
    vit = ViT((x, None), classes, (p1, p2), (b1, b2), n_embed, n_head, n_layers,
              dict(p=0.2, variant="none", block_size=(128, 128))).train()
    _load_reference_params(vit, golden, "vit")
    torch.testing.assert_close(vit(x), torch.from_numpy(golden["vit_logits"]), rtol=1e-4, atol=1e-5)


def test_layernorm_module_is_torch_layernorm_on_cpu():
    """The fused LayerNorm is nn.LayerNorm with another CUDA path: same parameters, same result on the CPU."""
    import torch
    from flash_dropout.layers.norm import LayerNorm
    torch.manual_seed(0)
    ours, ref = LayerNorm(48, bias=False), torch.nn.LayerNorm(48, bias=False)
    assert isinstance(ours, torch.nn.LayerNorm) and list(ours.state_dict()) == list(ref.state_dict())
    ref.load_state_dict(ours.state_dict())
    x = torch.randn(5, 7, 48)
    assert torch.equal(ours(x), ref(x))
