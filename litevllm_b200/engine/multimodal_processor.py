"""Image input for multimodal models.

Accepted image sources are bounded on purpose: only ``data:image/{png,jpeg,webp};base64,...`` URLs
(or PIL images passed in process), at most 8 MiB of encoded bytes and 16 megapixels.  An image is
resized (aspect preserved) to a whole number of patches, cut into ``patch x patch`` tiles with their
(row, col) grid positions, and the prompt's ``<image>`` marker is expanded into the model's number of
placeholder tokens; at prefill the placeholder embeddings are replaced by the vision tower's output.
Reference: vllm/engine/multimodal_processor.py:17-538.
"""
from __future__ import annotations

import base64
import binascii
import io
import re

import torch

from .errors import InvalidRequestError

MAX_IMAGE_BYTES = 8 * 1024 * 1024
MAX_IMAGE_PIXELS = 16 * 1000 * 1000
_DATA_URL = re.compile(r"^data:image/(png|jpeg|jpg|webp);base64,(.*)$", re.S)
IMAGE_MARKER = "<image>"


def decode_image(src):
    from PIL import Image
    if hasattr(src, "size") and hasattr(src, "convert"):
        img = src
    else:
        if not isinstance(src, str):
            raise InvalidRequestError("image must be a data URL or a PIL image")
        m = _DATA_URL.match(src.strip())
        if m is None:
            raise InvalidRequestError("only data:image/{png,jpeg,webp};base64 URLs are accepted")
        payload = m.group(2)
        if len(payload) * 3 // 4 > MAX_IMAGE_BYTES:
            raise InvalidRequestError(f"image larger than {MAX_IMAGE_BYTES} bytes")
        try:
            raw = base64.b64decode(payload, validate=True)
        except (binascii.Error, ValueError):
            raise InvalidRequestError("image payload is not valid base64") from None
        if len(raw) > MAX_IMAGE_BYTES:
            raise InvalidRequestError(f"image larger than {MAX_IMAGE_BYTES} bytes")
        try:
            img = Image.open(io.BytesIO(raw))
            img.load()
        except Exception:
            raise InvalidRequestError("cannot decode image") from None
    if img.size[0] * img.size[1] > MAX_IMAGE_PIXELS:
        raise InvalidRequestError(f"image exceeds {MAX_IMAGE_PIXELS} pixels")
    return img.convert("RGB")


def patchify(img, patch: int, max_patches: int, max_side: int):
    """-> (patches float32 [P, 3*patch*patch] in [-1, 1], position ids int64 [P, 2])."""
    import numpy as np
    w, h = img.size
    scale = min(1.0, (max_patches * patch * patch / float(w * h)) ** 0.5)
    gw = max(1, min(max_side, int(round(w * scale / patch))))
    gh = max(1, min(max_side, int(round(h * scale / patch))))
    while gw * gh > max_patches:
        if gw >= gh:
            gw -= 1
        else:
            gh -= 1
    img = img.resize((gw * patch, gh * patch))
    a = torch.from_numpy(np.asarray(img, dtype=np.float32) / 127.5 - 1.0)          # [H, W, 3]
    tiles = a.view(gh, patch, gw, patch, 3).permute(0, 2, 4, 1, 3).reshape(gh * gw, 3 * patch * patch)
    rows = torch.arange(gh).repeat_interleave(gw)
    cols = torch.arange(gw).repeat(gh)
    return tiles.contiguous(), torch.stack([rows, cols], 1)


class MultimodalProcessor:
    def __init__(self, arch, model, image_token_id: int | None = None, max_patches: int = 1024):
        self.arch, self.model = arch, model
        tower = getattr(model, "vision_tower", None)
        self.patch = getattr(tower, "patch", 16)
        self.max_side = getattr(tower, "max_side", 64)
        self.tokens_per_image = getattr(tower, "tokens_per_image", 16)
        self.max_patches = max_patches
        self.image_token_id = image_token_id if image_token_id is not None else arch.vocab_size - 1
        # a model that brings its own image processor (Qwen2-VL: resize to multiples of 28, CLIP normalisation,
        # merge-ordered patches, a token count that depends on the image size) is used instead of patchify()
        self.image_processor = getattr(model, "image_processor", None)
        self.images_seen = 0
        self.patches_seen = 0

    def expand_prompt(self, text, ids, mm: dict, tokenizer):
        """Returns (text, token ids with placeholders expanded, multimodal inputs dict)."""
        srcs = mm.get("image") or mm.get("images") or []
        if not isinstance(srcs, (list, tuple)):
            srcs = [srcs]
        if not srcs:
            return text, ids, None
        images = [decode_image(s) for s in srcs]
        if self.image_processor is not None:
            return self._expand_with_image_processor(text, ids, images, tokenizer)
        tiles, pos, counts = [], [], []
        for im in images:
            t, p = patchify(im, self.patch, self.max_patches, self.max_side)
            tiles.append(t); pos.append(p); counts.append(t.shape[0])
        if ids is None:
            if text is None or tokenizer is None:
                raise InvalidRequestError("image prompts need text and a tokenizer, or token ids with placeholders")
            parts = text.split(IMAGE_MARKER)
            if len(parts) - 1 != len(images):
                raise InvalidRequestError(f"{len(images)} image(s) given but {len(parts) - 1} {IMAGE_MARKER} marker(s) in the prompt")
            ids = []
            for i, part in enumerate(parts):
                if part:
                    ids.extend(tokenizer.encode(part) if i == 0 else _encode_plain(tokenizer, part))
                if i < len(images):
                    ids.extend([self.image_token_id] * self.tokens_per_image)
        else:
            n_ph = sum(1 for t in ids if t == self.image_token_id)
            if n_ph == len(images):      # one placeholder per image: expand
                out = []
                for t in ids:
                    out.extend([t] * self.tokens_per_image if t == self.image_token_id else [t])
                ids = out
            elif n_ph != len(images) * self.tokens_per_image:
                raise InvalidRequestError("placeholder token count does not match the images")
        self.images_seen += len(images)
        self.patches_seen += sum(counts)
        return text, ids, {"pixel_patches": torch.cat(tiles), "position_ids": torch.cat(pos),
                           "patches_per_image": counts}

    def _expand_with_image_processor(self, text, ids, images, tokenizer):
        from ..models.qwen2_vl import mrope_positions
        ip = self.image_processor
        pix, grids = [], []
        for im in images:
            pv, grid = ip(im)
            pix.append(pv)
            grids.append(grid)
        counts = [ip.num_tokens(g) for g in grids]
        if ids is None:
            if text is None or tokenizer is None:
                raise InvalidRequestError("image prompts need text and a tokenizer, or token ids with placeholders")
            parts = text.split(IMAGE_MARKER)
            if len(parts) - 1 != len(images):
                raise InvalidRequestError(f"{len(images)} image(s) given but {len(parts) - 1} {IMAGE_MARKER} marker(s) in the prompt")
            ids = []
            for i, part in enumerate(parts):
                if part:
                    ids.extend(tokenizer.encode(part) if i == 0 else _encode_plain(tokenizer, part))
                if i < len(images):
                    ids.extend([self.image_token_id] * counts[i])
        else:
            n_ph = sum(1 for t in ids if t == self.image_token_id)
            if n_ph == len(images):                      # one placeholder per image: expand each to its own count
                out, k = [], 0
                for t in ids:
                    if t == self.image_token_id:
                        out.extend([t] * counts[k])
                        k += 1
                    else:
                        out.append(t)
                ids = out
            elif n_ph != sum(counts):
                raise InvalidRequestError("placeholder token count does not match the images")
        try:
            pos3, delta = mrope_positions(list(ids), self.image_token_id, grids, ip.merge)
        except ValueError as e:
            raise InvalidRequestError(str(e)) from None
        self.images_seen += len(images)
        self.patches_seen += sum(p.shape[0] for p in pix)
        return text, ids, {"pixel_values": torch.cat(pix), "image_grid_thw": grids, "mrope_positions": pos3,
                           "rope_delta": delta}

    def embed_for_prefill(self, model, batch, items, states):
        """Token embeddings of the batch with image soft tokens merged in (None for text-only batches)."""
        if not any(states[it.request_id].multimodal_inputs for it in items):
            return None
        from .. import ops
        embeds = ops.embedding(batch.input_ids, model.embed_tokens, getattr(model.arch, "embed_scale", 1.0))
        off = 0
        for it in items:
            st = states[it.request_id]
            n = it.chunk_len
            if st.multimodal_inputs:
                cached = st.multimodal_inputs.get("_embeds")
                if cached is None:
                    cached = model.get_multimodal_embeddings(**{
                        k: v for k, v in st.multimodal_inputs.items()
                        if not k.startswith("_") and k not in ("mrope_positions", "rope_delta")})
                    st.multimodal_inputs["_embeds"] = cached
                ids = torch.tensor(st.prompt_token_ids, device=embeds.device)
                ph = torch.nonzero(ids == self.image_token_id).flatten()          # positions in the prompt
                sel = (ph >= it.start) & (ph < it.end)
                if bool(sel.any()):
                    embeds[off + ph[sel] - it.start] = cached[torch.nonzero(sel).flatten()].to(embeds.dtype)
            off += n
        return embeds

    def stats(self) -> dict:
        return {"images": self.images_seen, "patches": self.patches_seen, "tokens_per_image": self.tokens_per_image}


def _encode_plain(tokenizer, text):
    try:
        return list(tokenizer.encode(text, add_special_tokens=False))
    except TypeError:
        return list(tokenizer.encode(text))
