"""Generates tests/golden/reference_golden.npz by running andylolu2/sparse-dropout's OWN functions on the CPU.

Run once, in a container that has the reference checked out (it is not needed at test time):

    python tests/golden/make_golden.py /path/to/sparse-dropout

Imported from the reference (paths relative to its root):
    flash_dropout/functional/utils.py     blockwise_dropout_mask, mask_to_increment_table
    flash_dropout/functional/naive.py     blockwise_dropout_matmul_mask  (+ autograd for dx, dW)
    flash_dropout/functional/im2col_conv2d.py   im2col_conv2d
    eval/mlp/model.py                     BasicNet   (variant "none", reduced width)
    eval/llm/model.py                     GPT        (variant "none", reduced width)
    eval/vit/model.py                     ViT        (variant "none", reduced width)
Masks fed to the reference are drawn by oracle/philox_mask.py (the reference's tests also draw one mask
and hand it to both implementations, test/test_cuda.py:34); inputs are stored in the file so the
fixture does not depend on any RNG version.
"""
import os
import sys

import numpy as np
import torch

REPO = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    sys.path.insert(1, REPO)
    from flash_dropout.functional.im2col_conv2d import im2col_conv2d
    from flash_dropout.functional.naive import blockwise_dropout_matmul_mask
    from flash_dropout.functional.utils import blockwise_dropout_mask, mask_to_increment_table
    import flash_dropout.functional.naive as ref_naive
    assert os.path.realpath(ref_naive.__file__).startswith(os.path.realpath(ref_root)), ref_naive.__file__

    from oracle import philox_mask as pm

    out = {}
    torch.manual_seed(0)

    # ---- 1. mask shape / dtype / polarity of blockwise_dropout_mask (utils.py:11-16)
    shapes = [(1024, 1024, 128), (300, 392, 128), (512, 1024, 256), (5, 7, 3)]
    rec = []
    for (M, K, bs) in shapes:
        m0 = blockwise_dropout_mask(torch.empty(M, K), bs, 0.0)
        m1 = blockwise_dropout_mask(torch.empty(M, K), bs, 1.0)
        assert m0.dtype == torch.bool
        rec.append([M, K, bs, m0.shape[0], m0.shape[1], int(m0.any()), int(m1.all())])
    out["mask_shape_cases"] = np.array(rec, dtype=np.int64)   # p=0 -> nothing dropped, p=1 -> all dropped

    # ---- 2. mask_to_increment_table (utils.py:19-69): docstring example + seeded masks
    doc = np.array([[0, 1, 1, 0, 1], [1, 0, 0, 1, 0], [0, 1, 0, 1, 1]], dtype=bool)
    cases = [(doc, 16)]
    for i, (R, C, p, bk) in enumerate([(8, 8, 0.5, 128), (32, 32, 0.5, 128), (4, 12, 0.9, 64), (7, 3, 0.2, 32),
                                       (6, 6, 0.7, 128)]):
        cases.append((pm.block_mask(R * 128, C * 128, 128, p, seed=100 + i, offset=i), bk))
    last_row_dropped = np.array([[0, 1, 0], [1, 0, 0], [1, 1, 1]], dtype=bool)   # the reference's edge case
    cases.append((last_row_dropped, 16))
    for i, (m, bk) in enumerate(cases):
        table, row_indices, row_widths = mask_to_increment_table(torch.from_numpy(m), bk)
        out[f"inc{i}_mask"] = m
        out[f"inc{i}_block_k"] = np.int64(bk)
        out[f"inc{i}_table"] = table.numpy()
        out[f"inc{i}_row_indices"] = row_indices.numpy()
        out[f"inc{i}_row_widths"] = row_widths.numpy()
        out[f"inc{i}_nonzero"] = torch.nonzero(~torch.from_numpy(m), as_tuple=False).numpy()
    out["inc_count"] = np.int64(len(cases))

    # ---- 3. masked-dense forward + autograd backward (naive.py:8-25)
    mm_cases = [  # (M, N, K, bs, p, seed)
        (48, 24, 80, 16, 0.5, 1), (64, 40, 64, 16, 0.3, 2), (32, 16, 96, 32, 0.9, 3),
        (256, 128, 384, 128, 0.5, 4), (128, 128, 128, 128, 0.0, 5), (256, 128, 256, 128, 0.99, 6),
    ]
    for i, (M, N, K, bs, p, seed) in enumerate(mm_cases):
        g = torch.Generator().manual_seed(seed)
        # inputs are rounded to fp16-representable values and stored as fp16, so the fp16 kernels can be
        # fed exactly what the reference saw
        x = (torch.randn(M, K, generator=g) * K ** -0.25).half().float()
        w = (torch.randn(N, K, generator=g) * K ** -0.25).half().float()
        dy = (torch.randn(M, N, generator=g) * N ** -0.25).half().float()
        mask = pm.block_mask(M, K, bs, p, seed=seed, offset=0)
        xa, wa = x.clone().requires_grad_(), w.clone().requires_grad_()
        y = blockwise_dropout_matmul_mask(xa, torch.from_numpy(mask), bs, p, wa)
        y.backward(dy)
        out[f"mm{i}_cfg"] = np.array([M, N, K, bs, seed], dtype=np.int64)
        out[f"mm{i}_p"] = np.float64(p)
        for name, t in (("x", x), ("w", w), ("dy", dy)):
            out[f"mm{i}_{name}"] = t.numpy().astype(np.float16)
        for name, t in (("y", y.detach()), ("dx", xa.grad), ("dw", wa.grad)):
            out[f"mm{i}_{name}"] = t.numpy().astype(np.float32)
        out[f"mm{i}_mask"] = mask
    out["mm_count"] = np.int64(len(mm_cases))

    # ---- 4. im2col_conv2d (im2col_conv2d.py:5-27)
    conv_cases = [  # (N, C, H, W, Ko, R, S, pad, stride, dil)
        (2, 3, 8, 8, 4, 3, 3, (1, 1), (1, 1), (1, 1)),
        (1, 4, 9, 7, 5, 3, 2, (0, 1), (2, 1), (1, 1)),
        (2, 2, 10, 10, 3, 3, 3, (2, 2), (1, 2), (2, 2)),
    ]
    for i, (N, Cc, H, W, Ko, R, S, pad, stride, dil) in enumerate(conv_cases):
        g = torch.Generator().manual_seed(50 + i)
        x = torch.randn(N, Cc, H, W, generator=g)
        k = torch.randn(Ko, Cc, R, S, generator=g) / (Cc * R * S) ** 0.5
        y = im2col_conv2d(x, k, padding=pad, stride=stride, dilation=dil)
        out[f"conv{i}_cfg"] = np.array([N, Cc, H, W, Ko, R, S, *pad, *stride, *dil], dtype=np.int64)
        out[f"conv{i}_x"] = x.numpy()
        out[f"conv{i}_k"] = k.numpy()
        out[f"conv{i}_y"] = y.numpy()
    out["conv_count"] = np.int64(len(conv_cases))

    # ---- 5. the two consumer models (eval/mlp/model.py:8-40, eval/llm/model.py:83-155) at reduced width, built by the
    # reference's own classes with variant "none" (no randomness in forward): parameter names, shapes and values,
    # logits (and the GPT loss) for a stored input.  eval/utils.py imports wandb, which is not needed for the
    # models: an empty stand-in module satisfies the import.
    import types
    for name in ("wandb", "wandb.apis", "wandb.apis.public"):
        sys.modules.setdefault(name, types.ModuleType(name))
    sys.modules["wandb.apis.public"].Run = object
    from eval.llm.model import GPT as RefGPT
    from eval.mlp.model import BasicNet as RefBasicNet
    torch.manual_seed(1234)
    xs = torch.rand(16, 28, 28)
    mlp = RefBasicNet(xs, 2, 128, 10, dict(p=0.5, variant="none", block_size=(128, 128))).train()
    out["mlp_cfg"] = np.array([784, 2, 128, 10], dtype=np.int64)
    out["mlp_x"] = xs.numpy()
    out["mlp_logits"] = mlp(xs).detach().numpy()
    out["mlp_param_names"] = np.array(list(mlp.state_dict().keys()))
    for k, v in mlp.state_dict().items():
        out["mlp_param/" + k] = v.numpy()
    gpt = RefGPT(65, 32, 2, 4, 64, dict(p=0.2, variant="none", block_size=(128, 128))).train()
    idx = torch.randint(0, 65, (4, 32))
    logits, loss = gpt(idx)
    out["gpt_cfg"] = np.array([65, 32, 2, 4, 64], dtype=np.int64)
    out["gpt_idx"] = idx.numpy()
    out["gpt_logits"] = logits.detach().numpy()
    out["gpt_loss"] = np.float32(loss.item())
    out["gpt_param_names"] = np.array(list(gpt.state_dict().keys()))
    for k, v in gpt.state_dict().items():
        out["gpt_param/" + k] = v.numpy()
    from eval.vit.model import ViT as RefViT
    imgs = torch.rand(4, 1, 16, 16)
    vit = RefViT((imgs, torch.zeros(4, dtype=torch.long)), num_classes=10, patch_size=(2, 2), block_size=(2, 2),
                 n_embed=64, n_head=4, n_layers=2, dropout=dict(p=0.2, variant="none", block_size=(128, 128))).train()
    out["vit_cfg"] = np.array([10, 2, 2, 2, 2, 64, 4, 2], dtype=np.int64)
    out["vit_x"] = imgs.numpy()
    out["vit_logits"] = vit(imgs).detach().numpy()
    out["vit_param_names"] = np.array(list(vit.state_dict().keys()))
    for k, v in vit.state_dict().items():
        out["vit_param/" + k] = v.numpy()
    # which parameters AdamW decays (eval/llm/model.py:157-173): every tensor with 2 or more dimensions
    out["gpt_decay_names"] = np.array([n for n, q in gpt.named_parameters() if q.dim() >= 2])

    path = os.path.join(REPO, "tests", "golden", "reference_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes;", "torch", torch.__version__)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/sparse-dropout")
    main(sys.argv[1])
