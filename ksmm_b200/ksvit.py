"""KS-ViT-B/16 timing harness: a SimpleViT-B/16 whose MLP projections are
``KSLinear`` layers with ``algo='kernel'``.

This is benchmark scaffolding, not part of the KSMM hot path: attention,
LayerNorm, GELU, residuals and the patch embedding are stock PyTorch, exactly
as in the reference's timing script, where a SimpleViT is built and its
FeedForward projections ``net[1]`` / ``net[3]`` are swapped for KSLinear
(src/ksmm_py/model/vit.py:416-431, 770-800; get_vit.py:81-100;
benchmark/ksvit_time.py:167-229).  Architecture: 224x224 images, 16x16 patches
(196 tokens), width 768, 12 layers, 12 heads of 64, MLP 3072, mean pooling,
1000 classes, random initialisation.

    fc1 = KSLinear([(4,192,192,1), (1,768,192,4)])   768 -> 3072
    fc2 = KSLinear([(1,192,768,4), (4,192,192,1)])   3072 -> 768
"""
from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import nn

from .interface import KSLinear

FC1_PATTERNS = [(4, 192, 192, 1), (1, 768, 192, 4)]
FC2_PATTERNS = [(1, 192, 768, 4), (4, 192, 192, 1)]


def posemb_sincos_2d(h, w, dim, temperature=10000.0):
    y, x = torch.meshgrid(torch.arange(h), torch.arange(w), indexing="ij")
    omega = torch.arange(dim // 4) / (dim // 4 - 1)
    omega = 1.0 / (temperature ** omega)
    y = y.flatten()[:, None] * omega[None, :]
    x = x.flatten()[:, None] * omega[None, :]
    return torch.cat((x.sin(), x.cos(), y.sin(), y.cos()), dim=1)


class KSFeedForward(nn.Module):
    """LayerNorm -> fc1 -> GELU -> fc2.  `layout_plan` (default) keeps the 3072-feature activations
    between the two KSLinear layers batch-last: fc1 reads batch-first tokens and returns
    (3072, tokens), fc2 reads that and returns (tokens, 768).  Their d = 1 factors change the
    layout inside the kernel, so the d = 4 factors run in their fast batch-last form and nothing
    is transposed; the GELU is element-wise and does not care.  `fuse_gelu` applies it in the
    epilogue of fc1's last factor instead of as a separate PyTorch kernel (model/vit.py:416-431)."""

    def __init__(self, dim, dtype, device, dense=False, fuse_gelu=True, layout_plan=True):
        super().__init__()
        self.norm = nn.LayerNorm(dim)
        self.dense = dense
        self.fuse_gelu = fuse_gelu and not dense
        self.layout_plan = layout_plan and not dense
        if dense:  # same shapes with nn.Linear, for an accuracy / speed comparison
            self.fc1 = nn.Linear(dim, 4 * dim)
            self.fc2 = nn.Linear(4 * dim, dim)
        else:
            mid_last = True if self.layout_plan else False
            self.fc1 = KSLinear(FC1_PATTERNS, bias=True, algo="kernel", dtype=dtype, bs_last=False,
                                device=device, activation="gelu" if self.fuse_gelu else None,
                                out_bs_last=mid_last)
            self.fc2 = KSLinear(FC2_PATTERNS, bias=True, algo="kernel", dtype=dtype, bs_last=mid_last,
                                device=device, out_bs_last=False)

    def forward(self, x, add_residual=False):
        """With add_residual the block's `x + ff(x)` is formed inside fc2's last kernel."""
        h = self.fc1(self.norm(x))
        if not self.fuse_gelu:
            h = F.gelu(h)
        if add_residual and not self.dense:
            y = self.fc2(h, residual=x)
        else:
            y = self.fc2(h)
            if add_residual:
                y = y.view(x.shape) + x
        return y.view(x.shape) if self.layout_plan else y


class Attention(nn.Module):
    def __init__(self, dim, heads=12, dim_head=64):
        super().__init__()
        self.heads = heads
        self.norm = nn.LayerNorm(dim)
        self.to_qkv = nn.Linear(dim, heads * dim_head * 3, bias=False)
        self.to_out = nn.Linear(heads * dim_head, dim, bias=False)

    def forward(self, x):
        b, n, _ = x.shape
        q, k, v = self.to_qkv(self.norm(x)).view(b, n, 3, self.heads, -1).permute(2, 0, 3, 1, 4)
        out = F.scaled_dot_product_attention(q, k, v)
        return self.to_out(out.transpose(1, 2).reshape(b, n, -1))


class KSViTB(nn.Module):
    def __init__(self, dtype=torch.float16, device="cuda", depth=12, dim=768, num_classes=1000,
                 dense_mlp=False, fuse_gelu=True, layout_plan=True, fuse_residual=False):
        super().__init__()
        self.patch = 16
        patch_dim = 3 * 16 * 16
        self.embed = nn.Sequential(nn.LayerNorm(patch_dim), nn.Linear(patch_dim, dim), nn.LayerNorm(dim))
        self.register_buffer("pos", posemb_sincos_2d(14, 14, dim), persistent=False)
        self.layers = nn.ModuleList(
            [nn.ModuleList([Attention(dim), KSFeedForward(dim, dtype, device, dense_mlp, fuse_gelu, layout_plan)])
             for _ in range(depth)])
        self.norm = nn.LayerNorm(dim)
        self.head = nn.Linear(dim, num_classes)
        self.fuse_residual = fuse_residual
        # stock layers to the requested dtype / device; KSLinear parameters were created there
        for m in self.modules():
            if isinstance(m, (nn.Linear, nn.LayerNorm)):
                m.to(device=device, dtype=dtype)
        self.pos = self.pos.to(device=device, dtype=dtype)

    def forward(self, img):
        b, c, h, w = img.shape
        p = self.patch
        x = img.view(b, c, h // p, p, w // p, p).permute(0, 2, 4, 3, 5, 1).reshape(b, -1, p * p * c)
        x = self.embed(x) + self.pos
        for attn, ff in self.layers:
            x = attn(x) + x
            x = ff(x, add_residual=True) if self.fuse_residual else ff(x) + x
        return self.head(self.norm(x).mean(dim=1))
