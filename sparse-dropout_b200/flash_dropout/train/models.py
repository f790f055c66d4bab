"""The models the reference trains with DropoutMM, restated (architecture, parameter names and
initialisation follow the reference so checkpoints stay interchangeable):

  BasicNet — eval/mlp/model.py:8-40: in_proj, `num_layers` hidden DropoutMM layers, out_proj whose width is
             padded to a multiple of 128 and sliced back, ReLU in between.
  GPT      — eval/llm/model.py:8-173: nanoGPT-style decoder; q/k/v/out projections and both MLP linears are
             DropoutMM, LayerNorm without bias, causal SDPA, untied lm_head, AdamW with decay on >=2-D params.
  ViT      — eval/vit/model.py:8-124: patches grouped into blocks of neighbouring patches, fused qkv DropoutMM,
             pre-norm feed-forward with GELU, mean pooling, linear head.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import nn

from flash_dropout.layers import DropoutMM
from flash_dropout.layers.norm import LayerNorm


def next_multiple(x: int, base: int) -> int:
    return -(-x // base) * base


class BasicNet(nn.Module):
    """``input_dim`` may be the flattened input width or, as in the reference (eval/mlp/model.py:10-21), a sample
    batch whose first element has that many entries."""

    def __init__(self, input_dim: int | torch.Tensor, num_layers: int, hidden_dim: int, output_dim: int, dropout: dict):
        super().__init__()
        assert num_layers >= 0
        self.output_dim = output_dim
        if isinstance(input_dim, torch.Tensor):
            input_dim = input_dim[0].numel()
        self.in_proj = DropoutMM(input_dim, hidden_dim, **dropout)
        self.out_proj = DropoutMM(hidden_dim, next_multiple(output_dim, 128), **dropout)
        self.layers = nn.ModuleList(DropoutMM(hidden_dim, hidden_dim, **dropout) for _ in range(num_layers))
        self.act = nn.ReLU()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        # Every ReLU sits between two DropoutMM layers and feeds only the next one, so on the CUDA variant it is fused:
        # forward into the producing layer's epilogue, its derivative into the consuming layer's dX epilogue.
        x = self.in_proj(x.flatten(1), activation="relu", grad_premasked=True)
        for layer in self.layers:
            x = layer(x, activation="relu", input_relu=True, grad_premasked=True)
        return self.out_proj(x, input_relu=True)[..., : self.output_dim]


class CausalSelfAttention(nn.Module):
    def __init__(self, n_embed: int, n_head: int, dropout: dict):
        super().__init__()
        assert n_embed % n_head == 0
        self.n_head = n_head
        self.q_proj = DropoutMM(n_embed, n_embed, **dropout)
        self.k_proj = DropoutMM(n_embed, n_embed, **dropout)
        self.v_proj = DropoutMM(n_embed, n_embed, **dropout)
        self.out_proj = DropoutMM(n_embed, n_embed, **dropout)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        b, s, d = x.shape
        heads = lambda t: t.view(b, s, self.n_head, d // self.n_head).transpose(1, 2)
        y = F.scaled_dot_product_attention(heads(self.q_proj(x)), heads(self.k_proj(x)), heads(self.v_proj(x)),
                                           is_causal=True)
        return self.out_proj(y.transpose(1, 2).reshape(b, s, d))


class MLP(nn.Module):
    def __init__(self, n_embed: int, dropout: dict):
        super().__init__()
        self.c_fc = DropoutMM(n_embed, 4 * n_embed, **dropout)
        self.gelu = nn.GELU()
        self.c_proj = DropoutMM(4 * n_embed, n_embed, **dropout)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.c_proj(self.gelu(self.c_fc(x)))


class Block(nn.Module):
    def __init__(self, n_embed: int, n_head: int, dropout: dict):
        super().__init__()
        self.ln_1 = LayerNorm(n_embed, bias=False)
        self.attn = CausalSelfAttention(n_embed, n_head, dropout)
        self.ln_2 = LayerNorm(n_embed, bias=False)
        self.mlp = MLP(n_embed, dropout)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x = x + self.attn(self.ln_1(x))
        return x + self.mlp(self.ln_2(x))


class GPT(nn.Module):
    def __init__(self, vocab_size: int, context_length: int, n_layer: int, n_head: int, n_embed: int, dropout: dict):
        super().__init__()
        self.vocab_size, self.context_length = vocab_size, context_length
        self.transformer = nn.ModuleDict(dict(
            wte=nn.Embedding(vocab_size, n_embed),
            wpe=nn.Embedding(context_length, n_embed),
            h=nn.ModuleList(Block(n_embed, n_head, dropout) for _ in range(n_layer)),
            ln_f=LayerNorm(n_embed, bias=False),
        ))
        self.lm_head = nn.Linear(n_embed, vocab_size, bias=False)

    def forward(self, idx: torch.Tensor, calc_loss: bool = True):
        b, s = idx.shape
        assert s <= self.context_length
        pos = torch.arange(s, device=idx.device)
        x = self.transformer.wte(idx) + self.transformer.wpe(pos)[None]
        for block in self.transformer.h:
            x = block(x)
        logits = self.lm_head(self.transformer.ln_f(x))[:, :-1, :].contiguous()
        loss = None
        if calc_loss:   # next-token prediction
            loss = F.cross_entropy(logits.view(-1, self.vocab_size).float(), idx[:, 1:].reshape(-1))
        return logits, loss

    def configure_optimizers(self, weight_decay: float, lr: float, fused: bool | None = None):
        params = [p for p in self.parameters() if p.requires_grad]
        groups = [{"params": [p for p in params if p.dim() >= 2], "weight_decay": weight_decay},
                  {"params": [p for p in params if p.dim() < 2], "weight_decay": 0.0}]
        if fused is None:
            fused = all(p.is_cuda for p in params)
        return torch.optim.AdamW(groups, lr=lr, fused=fused)


class _BlockedPatches(nn.Module):
    """Image -> sequence of flattened patches, ordered so that the patches of one (b1 x b2) block of neighbouring
    patches are consecutive: the einops pattern "b c (h b1 p1) (w b2 p2) -> b (h w b1 b2) (p1 p2 c)" of
    eval/vit/model.py:97-103, written with view / permute.  No parameters (it holds index 0 of the embedding
    Sequential, as the reference's Rearrange layer does)."""

    def __init__(self, block: tuple[int, int], patch: tuple[int, int]):
        super().__init__()
        self.block, self.patch = block, patch

    def forward(self, img: torch.Tensor) -> torch.Tensor:
        b, c, H, W = img.shape
        (b1, b2), (p1, p2) = self.block, self.patch
        h, w = H // (b1 * p1), W // (b2 * p2)
        x = img.view(b, c, h, b1, p1, w, b2, p2)
        x = x.permute(0, 2, 5, 3, 6, 4, 7, 1)                    # b h w b1 b2 p1 p2 c
        return x.reshape(b, h * w * b1 * b2, p1 * p2 * c)


class ViTSelfAttention(nn.Module):
    def __init__(self, n_embed: int, n_head: int, dropout: dict):
        super().__init__()
        assert n_embed % n_head == 0
        self.n_head, self.n_embed = n_head, n_embed
        self.qkv_proj = DropoutMM(n_embed, 3 * n_embed, **dropout)
        self.out_proj = DropoutMM(n_embed, n_embed, **dropout)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        q, k, v = self.qkv_proj(x).split(self.n_embed, dim=2)
        b, s, d = q.shape
        heads = lambda t: t.view(b, s, self.n_head, d // self.n_head).transpose(1, 2)
        # the reference passes is_causal=True here as well (eval/vit/model.py:41)
        y = F.scaled_dot_product_attention(heads(q), heads(k), heads(v), is_causal=True)
        return self.out_proj(y.transpose(1, 2).reshape(b, s, d))


class ViTTransformer(nn.Module):
    def __init__(self, n_embed: int, n_layers: int, n_head: int, dropout: dict):
        super().__init__()
        self.norm = LayerNorm(n_embed)
        self.layers = nn.ModuleList(
            nn.ModuleList([
                ViTSelfAttention(n_embed, n_head, dropout),
                nn.Sequential(LayerNorm(n_embed), DropoutMM(n_embed, 4 * n_embed, **dropout), nn.GELU(),
                              DropoutMM(4 * n_embed, n_embed, **dropout)),
            ]) for _ in range(n_layers))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        for attn, ff in self.layers:
            x = attn(x) + x
            x = ff(x) + x
        return self.norm(x)


class ViT(nn.Module):
    """``sample`` is an (images, labels) pair as in the reference (only the image shape is used), or the image shape."""

    def __init__(self, sample, num_classes: int, patch_size: tuple[int, int], block_size: tuple[int, int],
                 n_embed: int, n_head: int, n_layers: int, dropout: dict):
        super().__init__()
        shape = sample[0].shape if isinstance(sample, (tuple, list)) and torch.is_tensor(sample[0]) else tuple(sample)
        _, c, h, w = shape
        (ph, pw), (bh, bw) = patch_size, block_size
        assert h % (bh * ph) == 0 and w % (bw * pw) == 0, "Image dimensions must be divisible by the patch size."
        num_patches, patch_dim = (h // ph) * (w // pw), c * ph * pw
        self.to_patch_embedding = nn.Sequential(_BlockedPatches((bh, bw), (ph, pw)), LayerNorm(patch_dim),
                                                nn.Linear(patch_dim, n_embed), LayerNorm(n_embed))
        self.pos_embedding = nn.Parameter(torch.randn(1, num_patches, n_embed))
        self.transformer = ViTTransformer(n_embed, n_layers, n_head, dropout)
        self.out = nn.Linear(n_embed, num_classes)

    def forward(self, img: torch.Tensor) -> torch.Tensor:
        x = self.to_patch_embedding(img) + self.pos_embedding
        return self.out(self.transformer(x).mean(dim=1))
