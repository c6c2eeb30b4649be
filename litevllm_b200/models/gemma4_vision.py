"""Vision towers (PyTorch): a ViT encoder over patch embeddings with learned 2-D position tables and
a projector into the text model's hidden size.  Shared by Gemma4 (patchified images with explicit
(row, col) position ids, average-pooled to a fixed number of soft tokens per image) and by the
Qwen2-VL style model (2x2 patch merge).  Reference: vllm/model_executor/models/gemma4/vision.py
(405 lines, tower + projector) and vllm/model_executor/models/qwen2_vl.py:16-251 (HF tower)."""
from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import nn


class VisionBlock(nn.Module):
    def __init__(self, dim: int, heads: int, mlp: int, dtype):
        super().__init__()
        self.heads = heads
        self.ln1 = nn.LayerNorm(dim, dtype=dtype)
        self.qkv = nn.Linear(dim, 3 * dim, dtype=dtype)
        self.proj = nn.Linear(dim, dim, dtype=dtype)
        self.ln2 = nn.LayerNorm(dim, dtype=dtype)
        self.fc1 = nn.Linear(dim, mlp, dtype=dtype)
        self.fc2 = nn.Linear(mlp, dim, dtype=dtype)

    def forward(self, x, mask=None):
        n, d = x.shape
        q, k, v = self.qkv(self.ln1(x)).view(n, 3, self.heads, d // self.heads).permute(1, 2, 0, 3)
        a = F.scaled_dot_product_attention(q[None], k[None], v[None], attn_mask=mask)[0]
        x = x + self.proj(a.permute(1, 0, 2).reshape(n, d))
        return x + self.fc2(F.gelu(self.fc1(self.ln2(x)), approximate="tanh"))


class Gemma4VisionTower(nn.Module):
    def __init__(self, arch, dtype):
        super().__init__()
        v = arch.vision or {}
        self.patch = int(v.get("patch_size", 16))
        self.dim = int(v.get("hidden_size", 256))
        self.max_side = int(v.get("position_embedding_size", 64))
        self.tokens_per_image = int(v.get("mm_tokens_per_image", v.get("tokens_per_image", 16)))
        depth, heads = int(v.get("num_hidden_layers", 2)), int(v.get("num_attention_heads", 4))
        self.patch_embed = nn.Linear(3 * self.patch * self.patch, self.dim, dtype=dtype)
        self.pos_row = nn.Embedding(self.max_side, self.dim, dtype=dtype)
        self.pos_col = nn.Embedding(self.max_side, self.dim, dtype=dtype)
        self.blocks = nn.ModuleList([VisionBlock(self.dim, heads, int(v.get("intermediate_size", 4 * self.dim)), dtype)
                                     for _ in range(depth)])
        self.post_ln = nn.LayerNorm(self.dim, dtype=dtype)
        self.projector = nn.Linear(self.dim, arch.hidden_size, dtype=dtype)
        for p in self.parameters():
            p.requires_grad_(False)
        with torch.no_grad():
            g = torch.Generator().manual_seed(1234)
            for p in self.parameters():
                if p.dim() > 1:      # deterministic default init; real checkpoints overwrite it
                    p.copy_((torch.randn(p.shape, generator=g, device="cpu") * 0.02).to(p.dtype))

    def forward(self, pixel_patches: torch.Tensor, position_ids: torch.Tensor, patches_per_image: list[int]):
        """pixel_patches [P, 3*patch*patch] in [-1, 1]; position_ids [P, 2] (row, col);
        returns [n_images * tokens_per_image, text hidden]."""
        dev, dt = self.patch_embed.weight.device, self.patch_embed.weight.dtype
        x = self.patch_embed(pixel_patches.to(dev, dt))
        x = x + self.pos_row(position_ids[:, 0].to(dev)) + self.pos_col(position_ids[:, 1].to(dev))
        outs, off = [], 0
        for n in patches_per_image:
            h = x[off:off + n]
            for blk in self.blocks:
                h = blk(h)
            h = self.post_ln(h)
            # pool the patch sequence to a fixed number of soft tokens
            pooled = F.adaptive_avg_pool1d(h.t()[None].float(), self.tokens_per_image)[0].t().to(dt)
            outs.append(self.projector(pooled))
            off += n
        return torch.cat(outs, 0)
