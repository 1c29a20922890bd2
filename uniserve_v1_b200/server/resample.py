"""Host resampling with the arithmetic of the libraries the models were trained behind.

* ``lanczos_resize``      Pillow's 8-bit LANCZOS resize of an RGB image: one separable filter
                          per axis, 22-bit fixed-point weights, horizontal pass then vertical,
                          each clipped back to 8 bits.
* ``sinc_resample``       torchaudio's band-limited sinc resampling with its defaults
                          (filter width 6, roll-off 0.99, Hann window).
* ``bicubic_antialias``   torch's antialiased bicubic resize (a = -0.5) of planar images:
                          float32, or 8-bit with 16-bit fixed-point weights and an 8-bit image
                          between the two passes.

Each restates its library's published algorithm on numpy arrays; the tests compare them with
Pillow, torchaudio and torch themselves.  Preprocessing of request media runs on the host
before anything is copied to the GPU, like the reference's media crate
(crates/media/src/resample/{lanczos,sinc,bicubic}.rs, reference project paths).
"""
from __future__ import annotations

import math

import numpy as np

_PRECISION_BITS = 22            # 32 - 8 bits of result - 2 of sign and overflow


def _sinc(x: np.ndarray) -> np.ndarray:
    y = x * math.pi
    with np.errstate(invalid="ignore", divide="ignore"):
        return np.where(x == 0.0, 1.0, np.sin(y) / y)


def _lanczos(x: np.ndarray) -> np.ndarray:
    return np.where((x >= -3.0) & (x < 3.0), _sinc(x) * _sinc(x / 3.0), 0.0)


def _coefficients(n_in: int, n_out: int, kernel, support: float):
    """For every output position the first input position it reads, how many it reads, and
    the normalised weights (float64, zero padded to a common width)."""
    scale = n_in / n_out
    fscale = max(scale, 1.0)
    sup = support * fscale
    ksize = int(math.ceil(sup)) * 2 + 1
    centers = (np.arange(n_out, dtype=np.float64) + 0.5) * scale
    xmin = np.maximum((centers - sup + 0.5).astype(np.int64), 0)        # C truncation
    xmax = np.minimum((centers + sup + 0.5).astype(np.int64), n_in)
    count = xmax - xmin
    j = np.arange(ksize, dtype=np.float64)[None, :]
    w = kernel((j + xmin[:, None] - centers[:, None] + 0.5) / fscale)
    w = np.where(j < count[:, None], w, 0.0)
    total = w.sum(1, keepdims=True)
    w = np.where(total != 0.0, w / np.where(total == 0.0, 1.0, total), w)
    return xmin, count, w


def _pass_8bit(img: np.ndarray, n_out: int, axis: int) -> np.ndarray:
    """One Pillow pass along ``axis`` of an [H, W, C] uint8 image."""
    n_in = img.shape[axis]
    xmin, count, w = _coefficients(n_in, n_out, _lanczos, 3.0)
    scaled = w * float(1 << _PRECISION_BITS)
    kk = np.where(w < 0, (scaled - 0.5).astype(np.int64), (scaled + 0.5).astype(np.int64))
    src = np.moveaxis(img, axis, 0).astype(np.int64)                     # [n_in, ...]
    idx = np.minimum(xmin[:, None] + np.arange(kk.shape[1])[None, :], n_in - 1)   # weights there are 0
    acc = np.full((n_out,) + src.shape[1:], 1 << (_PRECISION_BITS - 1), dtype=np.int64)
    for t in range(kk.shape[1]):
        acc += src[idx[:, t]] * kk[:, t].reshape((-1,) + (1,) * (src.ndim - 1))
    out = np.clip(acc >> _PRECISION_BITS, 0, 255).astype(np.uint8)
    return np.moveaxis(out, 0, axis)


def lanczos_resize(image: np.ndarray, out_height: int, out_width: int) -> np.ndarray:
    """``image`` [H, W, 3] uint8 -> [out_height, out_width, 3] uint8."""
    if image.ndim != 3 or image.dtype != np.uint8 or min(image.shape[:2]) < 1 \
            or out_height < 1 or out_width < 1:
        raise ValueError("an [H, W, C] uint8 image and positive sizes")
    out = image
    if out_width != image.shape[1]:
        out = _pass_8bit(out, out_width, 1)
    if out_height != image.shape[0]:
        out = _pass_8bit(out, out_height, 0)
    return np.ascontiguousarray(out)


def sinc_resample(audio: np.ndarray, orig_freq: int, new_freq: int, width: int = 6,
                  rolloff: float = 0.99) -> np.ndarray:
    """``audio`` [channels, length] float32 -> [channels, ceil(new * length / orig)]."""
    if orig_freq <= 0 or new_freq <= 0 or audio.ndim != 2:
        raise ValueError("positive rates and a [channels, length] array")
    g = math.gcd(int(orig_freq), int(new_freq))
    orig, new = int(orig_freq) // g, int(new_freq) // g
    length = audio.shape[1]
    if orig == new:
        return audio.astype(np.float32, copy=True)
    base = min(orig, new) * rolloff
    half = int(math.ceil(width * orig / base))
    idx = np.arange(-half, half + orig, dtype=np.float64)[None, :] / orig
    t = (np.arange(0, -new, -1, dtype=np.float64)[:, None] / new + idx) * base
    t = np.clip(t, -width, width)
    window = np.cos(t * math.pi / width / 2) ** 2
    t = t * math.pi
    with np.errstate(invalid="ignore", divide="ignore"):
        kernels = np.where(t == 0, 1.0, np.sin(t) / t)
    kernels = (kernels * window * (base / orig)).astype(np.float32)       # [new, 2 half + orig]
    x = np.pad(audio.astype(np.float32), ((0, 0), (half, half + orig)))
    frames = (x.shape[1] - kernels.shape[1]) // orig + 1
    win = np.lib.stride_tricks.sliding_window_view(x, kernels.shape[1], axis=1)[:, ::orig][:, :frames]
    out = np.einsum("cfk,nk->cfn", win, kernels, dtype=np.float32).reshape(audio.shape[0], -1)
    target = int(math.ceil(new * length / orig))
    return np.ascontiguousarray(out[:, :target])


def _cubic(x: np.ndarray, a: float = -0.5) -> np.ndarray:
    x = np.abs(x)
    return np.where(x < 1.0, ((a + 2.0) * x - (a + 3.0)) * x * x + 1.0,
                    np.where(x < 2.0, (((x - 5.0) * x + 8.0) * x - 4.0) * a, 0.0))


def _pass_float(img: np.ndarray, n_out: int, axis: int) -> np.ndarray:
    n_in = img.shape[axis]
    xmin, count, w = _coefficients(n_in, n_out, _cubic, 2.0)
    w = w.astype(np.float32)
    src = np.moveaxis(img, axis, 0)
    idx = np.minimum(xmin[:, None] + np.arange(w.shape[1])[None, :], n_in - 1)
    acc = np.zeros((n_out,) + src.shape[1:], dtype=np.float32)
    for t in range(w.shape[1]):
        acc += src[idx[:, t]] * w[:, t].reshape((-1,) + (1,) * (src.ndim - 1))
    return np.moveaxis(acc, 0, axis)


def _pass_u8_int16(img: np.ndarray, n_out: int, axis: int) -> np.ndarray:
    """One pass of torch's 8-bit antialiased resize: 16-bit fixed-point weights whose precision
    is the largest that keeps the greatest weight below 2^15, the result clipped to 8 bits."""
    n_in = img.shape[axis]
    xmin, count, w = _coefficients(n_in, n_out, _cubic, 2.0)
    top = float(w.max())
    prec = 0
    while prec < 22 and int(0.5 + top * (1 << (prec + 1))) < (1 << 15):
        prec += 1
    scaled = w * float(1 << prec)
    kk = np.where(w < 0, (scaled - 0.5).astype(np.int64), (scaled + 0.5).astype(np.int64))
    src = np.moveaxis(img, axis, 0).astype(np.int64)
    idx = np.minimum(xmin[:, None] + np.arange(kk.shape[1])[None, :], n_in - 1)
    acc = np.full((n_out,) + src.shape[1:], 1 << (prec - 1), dtype=np.int64)
    for t in range(kk.shape[1]):
        acc += src[idx[:, t]] * kk[:, t].reshape((-1,) + (1,) * (src.ndim - 1))
    return np.moveaxis(np.clip(acc >> prec, 0, 255).astype(np.uint8), 0, axis)


def bicubic_antialias(planes: np.ndarray, out_height: int, out_width: int) -> np.ndarray:
    """``planes`` [channels, H, W] float32 or uint8 -> [channels, out_height, out_width] of the
    same type.  The 8-bit form runs two fixed-point passes (width, then height) with an 8-bit
    image between them, as torch's does."""
    if planes.ndim != 3 or out_height < 1 or out_width < 1:
        raise ValueError("a [channels, H, W] array and positive sizes")
    if planes.dtype == np.uint8:
        x = planes
        if out_width != planes.shape[2]:
            x = _pass_u8_int16(x, out_width, 2)
        if out_height != planes.shape[1]:
            x = _pass_u8_int16(x, out_height, 1)
        return np.ascontiguousarray(x)
    x = planes.astype(np.float32)
    if out_width != planes.shape[2]:
        x = _pass_float(x, out_width, 2)
    if out_height != planes.shape[1]:
        x = _pass_float(x, out_height, 1)
    return np.ascontiguousarray(x)
