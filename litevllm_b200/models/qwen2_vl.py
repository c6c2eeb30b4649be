"""Qwen2-VL: the Llama/Qwen2 text decoder of this engine plus the Qwen2 vision transformer.

Vision tower (``Qwen2VisionTransformer``; weights ``visual.*`` of the HF checkpoint):
  patch embedding = the 3-D convolution over (2 frames x 14 x 14) patches written as one linear map
  over flattened patches; blocks of LayerNorm -> attention (fused qkv with bias, 2-D rotary embedding
  over the patch's (row, col), attention confined to one image) -> LayerNorm -> MLP with QuickGELU;
  ``PatchMerger``: LayerNorm, 2x2 neighbouring patches concatenated, two-layer MLP into the text width.
Image processor (``Qwen2VLImageProcessor``): resize so that both sides are multiples of 28 inside a
pixel budget, CLIP mean/std normalisation, the still image repeated over the two temporal frames,
patches emitted in merge order (the four patches of a 2x2 group are adjacent), grid (1, gh, gw);
an image becomes ``gh * gw / 4`` placeholder tokens.
Rotary positions are multimodal: three streams (t, h, w).  Text tokens advance all three together;
the tokens of an image share one t and walk the merged grid in h and w; text after an image continues
at the largest position used so far + 1, so a request decodes at ``position = index + delta`` with a
per-request ``delta <= 0``.  ``mrope_section`` says how many rotary frequencies read each stream.
Reference: vllm/model_executor/models/qwen2_vl.py:16-251 (HF tower instantiated from transformers,
mRoPE index computation, placeholder merge), vllm/engine/multimodal_processor.py:343-360 (HF image
processor call).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import nn

from .llama import LlamaForCausalLM

CLIP_MEAN = (0.48145466, 0.4578275, 0.40821073)
CLIP_STD = (0.26862954, 0.26130258, 0.27577711)


# ---------------------------------------------------------------------------- image processor
def smart_resize(height: int, width: int, factor: int = 28, min_pixels: int = 56 * 56,
                 max_pixels: int = 14 * 14 * 4 * 1280) -> tuple[int, int]:
    """Both sides rounded to multiples of ``factor``, the area kept inside [min_pixels, max_pixels],
    the aspect ratio kept as far as the rounding allows."""
    if max(height, width) / max(1, min(height, width)) > 200:
        raise ValueError("aspect ratio above 200 is not supported")
    h = max(factor, round(height / factor) * factor)
    w = max(factor, round(width / factor) * factor)
    if h * w > max_pixels:
        beta = math.sqrt(height * width / max_pixels)
        h = max(factor, math.floor(height / beta / factor) * factor)
        w = max(factor, math.floor(width / beta / factor) * factor)
    elif h * w < min_pixels:
        beta = math.sqrt(min_pixels / (height * width))
        h = math.ceil(height * beta / factor) * factor
        w = math.ceil(width * beta / factor) * factor
    return h, w


class Qwen2VLImageProcessor:
    def __init__(self, patch_size: int = 14, merge_size: int = 2, temporal_patch_size: int = 2,
                 min_pixels: int = 56 * 56, max_pixels: int = 14 * 14 * 4 * 1280):
        self.patch, self.merge, self.tps = patch_size, merge_size, temporal_patch_size
        self.min_pixels, self.max_pixels = min_pixels, max_pixels

    def __call__(self, img) -> tuple[torch.Tensor, tuple[int, int, int]]:
        """PIL RGB image -> (patches float32 [gh * gw, 3 * tps * patch * patch], grid (1, gh, gw))."""
        import numpy as np
        w0, h0 = img.size
        f = self.patch * self.merge
        h, w = smart_resize(h0, w0, f, self.min_pixels, self.max_pixels)
        img = img.resize((w, h), resample=3)                     # bicubic
        a = torch.from_numpy(np.asarray(img, dtype=np.float32) / 255.0)          # [H, W, 3]
        a = (a - torch.tensor(CLIP_MEAN)) / torch.tensor(CLIP_STD)
        a = a.permute(2, 0, 1)                                                   # [3, H, W]
        frames = a[None].repeat(self.tps, 1, 1, 1)                               # the still image fills every frame
        gh, gw, m, p = h // self.patch, w // self.patch, self.merge, self.patch
        x = frames.reshape(1, self.tps, 3, gh // m, m, p, gw // m, m, p)
        x = x.permute(0, 3, 6, 4, 7, 2, 1, 5, 8)                                 # [t, gh/m, gw/m, m, m, C, tps, p, p]
        return x.reshape(gh * gw, 3 * self.tps * p * p).contiguous(), (1, gh, gw)

    def num_tokens(self, grid) -> int:
        return grid[0] * grid[1] * grid[2] // (self.merge * self.merge)


def mrope_positions(token_ids: list[int], image_token_id: int, grids: list[tuple[int, int, int]],
                    merge: int = 2) -> tuple[torch.Tensor, int]:
    """-> (positions int64 [3, L], delta) for a prompt whose image placeholders are already expanded;
    decode step ``n`` (0-based token index L + n) uses position ``L + n + delta`` on all streams."""
    L = len(token_ids)
    pos = torch.zeros(3, L, dtype=torch.int64)
    nxt, i, img = 0, 0, 0
    while i < L:
        if token_ids[i] == image_token_id and img < len(grids):
            t, gh, gw = grids[img]
            mh, mw = gh // merge, gw // merge
            n = t * mh * mw
            if token_ids[i:i + n] != [image_token_id] * n:
                raise ValueError("image placeholder run is shorter than the image's token count")
            tt = torch.arange(t).view(t, 1, 1).expand(t, mh, mw).reshape(-1)
            hh = torch.arange(mh).view(1, mh, 1).expand(t, mh, mw).reshape(-1)
            ww = torch.arange(mw).view(1, 1, mw).expand(t, mh, mw).reshape(-1)
            pos[0, i:i + n], pos[1, i:i + n], pos[2, i:i + n] = nxt + tt, nxt + hh, nxt + ww
            nxt = nxt + max(t, mh, mw)
            i += n
            img += 1
        else:
            pos[:, i] = nxt
            nxt += 1
            i += 1
    return pos, int(nxt - L)


# ---------------------------------------------------------------------------- vision tower
def _rot_half(x):
    a, b = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
    return torch.cat([-b, a], dim=-1)


class VisionAttention(nn.Module):
    def __init__(self, dim: int, heads: int, dtype):
        super().__init__()
        self.heads = heads
        self.qkv = nn.Linear(dim, 3 * dim, dtype=dtype)
        self.proj = nn.Linear(dim, dim, dtype=dtype)

    def forward(self, x, cos, sin, seqlens: list[int]):
        n, d = x.shape
        hd = d // self.heads
        q, k, v = self.qkv(x).view(n, 3, self.heads, hd).unbind(1)
        q = (q.float() * cos + _rot_half(q.float()) * sin).to(x.dtype)
        k = (k.float() * cos + _rot_half(k.float()) * sin).to(x.dtype)
        outs, off = [], 0
        for L in seqlens:                                  # attention never crosses an image boundary
            qq, kk, vv = (t[off:off + L].transpose(0, 1)[None] for t in (q, k, v))
            outs.append(F.scaled_dot_product_attention(qq, kk, vv)[0].transpose(0, 1).reshape(L, d))
            off += L
        return self.proj(torch.cat(outs, 0))


class VisionBlock(nn.Module):
    def __init__(self, dim: int, heads: int, mlp_dim: int, dtype):
        super().__init__()
        self.norm1 = nn.LayerNorm(dim, eps=1e-6, dtype=dtype)
        self.norm2 = nn.LayerNorm(dim, eps=1e-6, dtype=dtype)
        self.attn = VisionAttention(dim, heads, dtype)
        self.fc1 = nn.Linear(dim, mlp_dim, dtype=dtype)
        self.fc2 = nn.Linear(mlp_dim, dim, dtype=dtype)

    def forward(self, x, cos, sin, seqlens):
        x = x + self.attn(self.norm1(x), cos, sin, seqlens)
        h = self.fc1(self.norm2(x))
        return x + self.fc2(h * torch.sigmoid(1.702 * h))       # QuickGELU


class PatchMerger(nn.Module):
    def __init__(self, out_dim: int, context_dim: int, merge: int, dtype):
        super().__init__()
        self.hidden = context_dim * merge * merge
        self.ln_q = nn.LayerNorm(context_dim, eps=1e-6, dtype=dtype)
        self.mlp0 = nn.Linear(self.hidden, self.hidden, dtype=dtype)
        self.mlp2 = nn.Linear(self.hidden, out_dim, dtype=dtype)

    def forward(self, x):
        return self.mlp2(F.gelu(self.mlp0(self.ln_q(x).view(-1, self.hidden))))


class Qwen2VisionTransformer(nn.Module):
    def __init__(self, vcfg: dict, text_hidden: int, dtype):
        super().__init__()
        self.patch = int(vcfg.get("patch_size", 14))
        self.tps = int(vcfg.get("temporal_patch_size", 2))
        self.merge = int(vcfg.get("spatial_merge_size", 2))
        self.dim = int(vcfg.get("embed_dim", vcfg.get("hidden_size", 1280)))
        depth = int(vcfg.get("depth", vcfg.get("num_hidden_layers", 32)))
        self.heads = int(vcfg.get("num_heads", vcfg.get("num_attention_heads", 16)))
        mlp_dim = int(self.dim * float(vcfg.get("mlp_ratio", 4)))
        self.in_features = 3 * self.tps * self.patch * self.patch
        self.patch_embed = nn.Linear(self.in_features, self.dim, bias=False, dtype=dtype)
        self.blocks = nn.ModuleList([VisionBlock(self.dim, self.heads, mlp_dim, dtype) for _ in range(depth)])
        self.merger = PatchMerger(text_hidden, self.dim, self.merge, dtype)
        self.rot_dim = self.dim // self.heads // 2
        for p in self.parameters():
            p.requires_grad_(False)
        with torch.no_grad():
            g = torch.Generator().manual_seed(4321)
            for p in self.parameters():
                if p.dim() > 1:      # deterministic default init; a real checkpoint overwrites it
                    p.copy_((torch.randn(p.shape, generator=g, device="cpu") * 0.02).to(p.dtype))

    def rot_pos_emb(self, grids, device):
        """(cos, sin) fp32 [P, 1, head_dim]: half of the rotary pairs turn with the patch row, half with the column,
        patches listed in merge order."""
        inv = 1.0 / (10000.0 ** (torch.arange(0, self.rot_dim, 2, dtype=torch.float32, device=device) / self.rot_dim))
        parts = []
        m = self.merge
        for t, gh, gw in grids:
            hp = torch.arange(gh, device=device).view(gh, 1).expand(gh, gw)
            wp = torch.arange(gw, device=device).view(1, gw).expand(gh, gw)
            order = lambda z: z.reshape(gh // m, m, gw // m, m).permute(0, 2, 1, 3).reshape(-1)
            hw = torch.stack([order(hp), order(wp)], dim=-1).repeat(t, 1)            # [P, 2]
            parts.append(hw)
        hw = torch.cat(parts, 0).float()
        freqs = (hw[:, :, None] * inv[None, None, :]).reshape(hw.shape[0], -1)       # [P, rot_dim]
        emb = torch.cat([freqs, freqs], dim=-1)                                      # [P, head_dim]
        return emb.cos()[:, None, :], emb.sin()[:, None, :]

    def forward(self, pixel_values: torch.Tensor, grid_thw: list[tuple[int, int, int]]) -> torch.Tensor:
        """pixel_values [P, 3 * tps * patch * patch] (merge order) -> [P / merge^2, text hidden]."""
        w = self.patch_embed.weight
        x = self.patch_embed(pixel_values.to(w.device, w.dtype))
        cos, sin = self.rot_pos_emb(grid_thw, w.device)
        seqlens = [t * gh * gw for t, gh, gw in grid_thw]
        for blk in self.blocks:
            x = blk(x, cos, sin, seqlens)
        return self.merger(x)

    def load_weights(self, weights) -> set[str]:
        """HF names below ``visual.``: the conv patch embedding is flattened, ``mlp.fc1/fc2`` and
        ``merger.mlp.0/2`` are renamed."""
        params = dict(self.named_parameters())
        used = set()
        for name, t in weights:
            if not name.startswith("visual."):
                continue
            key = name[len("visual."):]
            key = key.replace("patch_embed.proj.weight", "patch_embed.weight")
            key = key.replace(".mlp.fc1.", ".fc1.").replace(".mlp.fc2.", ".fc2.")
            key = key.replace("merger.mlp.0.", "merger.mlp0.").replace("merger.mlp.2.", "merger.mlp2.")
            p = params.get(key)
            if p is None:
                continue
            p.data.copy_(t.reshape(p.shape).to(p.dtype))
            used.add(name)
        return used


# ---------------------------------------------------------------------------- model
class Qwen2VLForConditionalGeneration(LlamaForCausalLM):
    supports_multimodal = True
    supports_lora = False

    def __init__(self, vllm_config):
        super().__init__(vllm_config)
        arch = vllm_config.model_config.arch
        vcfg = dict(arch.vision or {})
        self.vision_tower = Qwen2VisionTransformer(vcfg, arch.hidden_size, vllm_config.model_config.dtype)
        self.visual = self.vision_tower
        self.image_processor = Qwen2VLImageProcessor(
            self.vision_tower.patch, self.vision_tower.merge, self.vision_tower.tps,
            int(vcfg.get("min_pixels", 56 * 56)), int(vcfg.get("max_pixels", 14 * 14 * 4 * 1280)))
        half = (arch.rotary_dim or arch.head_dim) // 2
        sec = arch.extra.get("mrope_section") or [half - 2 * (half * 3 // 8), half * 3 // 8, half * 3 // 8]
        if sum(sec) != half:
            raise ValueError(f"mrope_section {sec} must sum to half the rotary dimension ({half})")
        self.mrope_section = list(sec)
        self._freq_stream = None

    def freq_stream(self, device) -> torch.Tensor:
        """int32 [rotary_dim / 2]: which position stream (0 t, 1 h, 2 w) every rotary frequency reads."""
        if self._freq_stream is None or self._freq_stream.device != device:
            fs = torch.cat([torch.full((n,), i, dtype=torch.int32) for i, n in enumerate(self.mrope_section)])
            self._freq_stream = fs.to(device)
        return self._freq_stream

    def get_multimodal_embeddings(self, **mm_inputs):
        return self.vision_tower(mm_inputs["pixel_values"], mm_inputs["image_grid_thw"])

    def prepare_prefill(self, batch, items, states) -> None:
        """Swap the 1-D positions of a prefill batch for the three multimodal streams when any request
        of the batch carries images (text-only batches keep the fused 1-D path)."""
        if not any(states[it.request_id].multimodal_inputs for it in items):
            return
        cols = []
        for it in items:
            st = states[it.request_id]
            mp = (st.multimodal_inputs or {}).get("mrope_positions")
            if mp is None:
                cols.append(torch.arange(it.start, it.end).expand(3, -1))
            else:
                cols.append(mp[:, it.start:it.end])
        pos3 = torch.cat(cols, dim=1).to(device=batch.positions.device, dtype=torch.int32).contiguous()
        batch.positions = pos3
        batch.extras["freq_stream"] = self.freq_stream(pos3.device)

    def load_weights(self, weights):
        weights = list(weights)
        loaded = super().load_weights((n, t) for n, t in weights if not n.startswith("visual."))
        return set(loaded) | self.vision_tower.load_weights(weights)
