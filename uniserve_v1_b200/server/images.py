"""Image and video inputs of chat requests: decode, resize, normalise and cut into the patch
rows the vision tower reads.

``image_url`` content parts carry ``data:`` URLs (base64) or ``file://`` paths; remote URLs
are refused (a serving process does not fetch from the network on a client's behalf).
``file://`` is read only below the deployment's media directory
(``media_config.directory``): the URL names an absolute path without a host part, the
canonical path (symbolic links resolved) must lie under the canonical directory, and with
no directory configured every ``file://`` URL is refused (api/input/media.rs of the
reference project reads local media under the same rule).
Preprocessing follows the Qwen-VL image processor: both sides become multiples of
``patch * merge`` with the pixel count clamped to [min_pixels, max_pixels] at (nearly)
the same aspect ratio, values are scaled to [0, 1] and normalised with mean = std = 0.5,
a still image is repeated ``temporal_patch`` times, and patches leave in merge-block order
as rows of ``C * T * P * P`` values - the layout ``Qwen3VLVisionTower.forward`` expects.
A video is sampled at a fixed rate; every temporal patch (two frames) becomes one image-like
group of rows that the prompt introduces with its time ("<1.2 seconds>").

Reference behaviour: crates/processing (image and frame preparation, reference project
path).
"""
from __future__ import annotations

import base64
import io
import math
import os
from typing import Optional

import numpy as np
import torch


_MEDIA_DIRECTORY = None          # canonical path, or None: file:// URLs are refused


def set_media_directory(path) -> None:
    """The one directory ``file://`` media may be read from (None closes ``file://``)."""
    global _MEDIA_DIRECTORY
    _MEDIA_DIRECTORY = os.path.realpath(str(path)) if path else None


def media_directory():
    return _MEDIA_DIRECTORY


_MEDIA_LIMIT = 256 << 20         # bytes one medium of a request may have


def set_media_limit(nbytes) -> None:
    """The size one medium (an image, a video: a file or a decoded ``data:`` URL) may have
    (``media_config.max_request_bytes``)."""
    global _MEDIA_LIMIT
    _MEDIA_LIMIT = max(1, int(nbytes)) if nbytes else 256 << 20


def _decode_data_url(payload: str) -> bytes:
    if (len(payload) // 4) * 3 > _MEDIA_LIMIT + 3:              # before anything is decoded
        raise ValueError("the medium is larger than the deployment accepts")
    return base64.b64decode(payload, validate=True)


def resolve_file_url(url: str) -> str:
    """``file:///abs/path`` -> the canonical path, if it lies below the media directory.
    Raises ValueError otherwise (no directory configured, a host part, a relative path,
    ``..`` or a symbolic link that leaves the directory)."""
    from urllib.parse import unquote, urlparse
    if _MEDIA_DIRECTORY is None:
        raise ValueError("file:// URLs are not served: the deployment sets no "
                         "media_config.directory")
    u = urlparse(url)
    if u.scheme != "file" or u.netloc not in ("", "localhost") or u.query or u.fragment:
        raise ValueError("file:// URLs name a local absolute path and nothing else")
    path = unquote(u.path)
    if not path.startswith("/") or "\x00" in path:
        raise ValueError("file:// URLs name an absolute path")
    real = os.path.realpath(path)
    if os.path.commonpath([real, _MEDIA_DIRECTORY]) != _MEDIA_DIRECTORY:
        raise ValueError("the file lies outside the deployment's media directory")
    return real


def read_file_url(url: str, limit: Optional[int] = None) -> bytes:
    """Bytes of a ``file://`` medium (``resolve_file_url`` rules; I/O errors become
    ValueError so that a request naming a missing file is an input error)."""
    real = resolve_file_url(url)
    try:
        if os.path.getsize(real) > (limit if limit is not None else _MEDIA_LIMIT):
            raise ValueError("the file is larger than the deployment accepts")
        with open(real, "rb") as f:
            return f.read()
    except OSError as e:
        raise ValueError(f"cannot read the file: {e.strerror or e}")


def load_image(url: str) -> np.ndarray:
    """-> uint8 [H, W, 3] (RGB)."""
    from PIL import Image
    if url.startswith("data:"):
        head, _, payload = url.partition(",")
        if not head.endswith(";base64"):
            raise ValueError("data URLs must be base64-encoded")
        raw = _decode_data_url(payload)
    elif url.startswith("file://"):
        raw = read_file_url(url)
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
    return [u for kind, u in collect_media(messages) if kind == "image"]


def collect_media(messages: list) -> list:
    """(kind, url) of every ``image_url`` / ``video_url`` part, in prompt order."""
    out = []
    for m in messages:
        c = m.get("content")
        if isinstance(c, list):
            for part in c:
                t = part.get("type")
                if t in ("image_url", "video_url"):
                    u = part.get(t)
                    out.append((t[:5], u.get("url") if isinstance(u, dict) else u))
    return out


def load_video(url: str, fps: float = 2.0, max_frames: int = 64):
    """Decodes a ``file://`` (or base64 ``data:``) video and samples it at ``fps``: returns
    (frames uint8 [F, H, W, 3] with F even, seconds of each sampled frame)."""
    import tempfile

    import cv2
    tmp = None
    if url.startswith("data:"):
        head, _, payload = url.partition(",")
        if not head.endswith(";base64"):
            raise ValueError("data URLs must be base64-encoded")
        fd, tmp = tempfile.mkstemp(suffix=".mp4")
        with os.fdopen(fd, "wb") as f:
            f.write(_decode_data_url(payload))
        path = tmp
    elif url.startswith("file://"):
        path = resolve_file_url(url)
        if not os.path.isfile(path):
            raise ValueError("cannot read the file: no such file")
        if os.path.getsize(path) > _MEDIA_LIMIT:
            raise ValueError("the file is larger than the deployment accepts")
    else:
        raise ValueError("video URLs must be data: or file:// URLs; remote URLs are not fetched")
    try:
        cap = cv2.VideoCapture(path)
        native = cap.get(cv2.CAP_PROP_FPS) or 0.0
        frames = []
        while True:
            ok, f = cap.read()
            if not ok:
                break
            frames.append(cv2.cvtColor(f, cv2.COLOR_BGR2RGB))
        cap.release()
    finally:
        if tmp:
            os.unlink(tmp)
    if not frames:
        raise ValueError("cannot decode the video")
    native = native if native > 0 else 24.0
    step = max(1.0, native / fps)
    idx = [int(round(i * step)) for i in range(int(len(frames) / step) or 1)]
    idx = [i for i in idx if i < len(frames)][:max_frames]
    if len(idx) % 2:
        idx.append(idx[-1])                    # whole temporal patches of two frames
    return np.stack([frames[i] for i in idx]), [i / native for i in idx]


def preprocess_video(frames: np.ndarray, patch: int = 16, temporal_patch: int = 2, merge: int = 2,
                     min_pixels: int = 64 * 64, max_pixels: int = 256 * 28 * 28):
    """uint8 [F, H, W, 3] -> (rows float32 [t * h * w, C * T * P * P], grid (t, h, w)); every
    frame gets the size ``smart_resize`` picks for the first one."""
    from PIL import Image
    H, W = frames.shape[1:3]
    h, w = smart_resize(H, W, patch * merge, min_pixels, max_pixels)
    out = []
    for f in frames:
        if (h, w) != (H, W):
            f = np.asarray(Image.fromarray(f).resize((w, h), Image.BICUBIC))
        out.append(torch.from_numpy(f.copy()).permute(2, 0, 1).float() / 255.0)
    x = (torch.stack(out) - 0.5) / 0.5
    return patch_rows(x, patch, temporal_patch, merge)


def video_prompt(seconds: list, temporal_patch: int = 2) -> str:
    """The text that stands for a video: one timestamped, delimited placeholder per temporal
    patch (the language model sees every pair of frames as an image at its time)."""
    groups = [sum(seconds[i:i + temporal_patch]) / temporal_patch
              for i in range(0, len(seconds), temporal_patch)]
    return "".join(f"<{t:.1f} seconds><|vision_start|><|image_pad|><|vision_end|>" for t in groups)
