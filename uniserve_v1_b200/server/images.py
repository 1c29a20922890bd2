"""Image inputs of chat requests: decode, resize, normalise and cut into the patch rows the
vision tower reads.

``image_url`` content parts carry ``data:`` URLs (base64) or ``file://`` paths; remote URLs
are refused (a serving process does not fetch from the network on a client's behalf).
Preprocessing follows the Qwen-VL image processor: both sides become multiples of
``patch * merge`` with the pixel count clamped to [min_pixels, max_pixels] at (nearly)
the same aspect ratio, values are scaled to [0, 1] and normalised with mean = std = 0.5,
a still image is repeated ``temporal_patch`` times, and patches leave in merge-block order
as rows of ``C * T * P * P`` values - the layout ``Qwen3VLVisionTower.forward`` expects.

Reference behaviour: crates/processing (image and frame preparation, reference project
path).
"""
from __future__ import annotations

import base64
import io
import math

import numpy as np
import torch


def load_image(url: str) -> np.ndarray:
    """-> uint8 [H, W, 3] (RGB)."""
    from PIL import Image
    if url.startswith("data:"):
        head, _, payload = url.partition(",")
        if not head.endswith(";base64"):
            raise ValueError("data URLs must be base64-encoded")
        raw = base64.b64decode(payload, validate=True)
    elif url.startswith("file://"):
        with open(url[7:], "rb") as f:
            raw = f.read()
    else:
        raise ValueError("image URLs must be data: or file:// URLs; remote URLs are not fetched")
    try:
        img = Image.open(io.BytesIO(raw)).convert("RGB")
    except Exception as e:
        raise ValueError(f"cannot decode the image: {e}")
    return np.asarray(img)


def smart_resize(height: int, width: int, factor: int, min_pixels: int, max_pixels: int):
    if max(height, width) / max(1, min(height, width)) > 200:
        raise ValueError("the aspect ratio of an image must be below 200")
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


def patch_rows(frames: torch.Tensor, patch: int, temporal_patch: int, merge: int):
    """frames [F, C, H, W] (normalised) -> (rows [t * h * w, C * T * P * P], (t, h, w))."""
    F_, C, H, W = frames.shape
    if F_ % temporal_patch:
        frames = torch.cat([frames, frames[-1:].repeat(temporal_patch - F_ % temporal_patch, 1, 1, 1)])
    t, gh, gw = frames.shape[0] // temporal_patch, H // patch, W // patch
    x = frames.view(t, temporal_patch, C, gh // merge, merge, patch, gw // merge, merge, patch)
    x = x.permute(0, 3, 6, 4, 7, 2, 1, 5, 8)
    return x.reshape(t * gh * gw, C * temporal_patch * patch * patch).contiguous(), (t, gh, gw)


def preprocess(image: np.ndarray, patch: int = 16, temporal_patch: int = 2, merge: int = 2,
               min_pixels: int = 64 * 64, max_pixels: int = 1280 * 28 * 28):
    """uint8 [H, W, 3] -> (rows float32, grid (t, h, w))."""
    from PIL import Image
    H, W = image.shape[:2]
    h, w = smart_resize(H, W, patch * merge, min_pixels, max_pixels)
    if (h, w) != (H, W):
        image = np.asarray(Image.fromarray(image).resize((w, h), Image.BICUBIC))
    x = torch.from_numpy(image.copy()).permute(2, 0, 1).float() / 255.0
    x = (x - 0.5) / 0.5
    return patch_rows(x[None], patch, temporal_patch, merge)


def expand_placeholders(ids: list, image_token_id: int, grids: list, merge: int) -> list:
    """Every single placeholder token becomes as many tokens as its image has merged rows."""
    out, g = [], iter(grids)
    for t in ids:
        if t == image_token_id:
            gt, gh, gw = next(g)
            out.extend([image_token_id] * (gt * (gh // merge) * (gw // merge)))
        else:
            out.append(t)
    if next(g, None) is not None:
        raise ValueError("more images than placeholder tokens in the prompt")
    return out


def collect(messages: list) -> list:
    """The image URLs of a chat request, in prompt order."""
    urls = []
    for m in messages:
        c = m.get("content")
        if isinstance(c, list):
            for part in c:
                if part.get("type") == "image_url":
                    u = part.get("image_url")
                    urls.append(u.get("url") if isinstance(u, dict) else u)
    return urls
