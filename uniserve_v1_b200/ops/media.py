"""Media operators: colour conversion, PCM packing, tile stitching, cross-fade,
1-D convolutions of the audio VAE, and the host MP4 / WAV writers."""
from __future__ import annotations

import ctypes
import os
import tempfile

import numpy as np
import torch
import torch.nn.functional as TF

from . import native as N

N.register_signatures({
    "us_rgb_to_yuv420": (N.I, [N.P, N.P, N.P, N.P, N.I, N.I, N.I, N.P]),
    "us_rgb_bytes": (N.I, [N.P, N.P, N.I, N.I, N.I, N.P]),
    "us_pcm_interleave": (N.I, [N.P, N.P, N.I, N.L, N.P]),
    "us_tile_stitch": (N.I, [N.P, N.P, N.P, N.I, N.I, N.I, N.I, N.I, N.I, N.I, N.I, N.P]),
    "us_tile_normalise": (N.I, [N.P, N.P, N.I, N.I, N.I, N.P]),
    "us_cross_fade": (N.I, [N.P, N.P, N.P, N.I, N.L, N.P]),
    "us_frame_moments": (N.I, [N.P, N.P, N.P, N.I, N.L, N.F, N.P]),
    "us_frame_norm_pad": (N.I, [N.P, N.P, N.P, N.P, N.P, N.P, N.I, N.I, N.I, N.I, N.I, N.I, N.P]),
    "us_conv1d": (N.I, [N.P, N.P, N.P, N.P, N.I, N.I, N.I, N.I, N.I, N.I, N.I, N.I, N.P]),
    "us_conv_transpose1d": (N.I, [N.P, N.P, N.P, N.P, N.I, N.I, N.I, N.I, N.I, N.I, N.I, N.P]),
    "us_snake": (N.I, [N.P, N.P, N.P, N.P, N.I, N.I, N.L, N.P]),
    "us_activation1d": (N.I, [N.P, N.P, N.P, N.P, N.P, N.I, N.I, N.I, N.I, N.P]),
})


def rgb_to_yuv420(frames: torch.Tensor):
    """[F, 3, H, W] in [-1, 1] -> (Y [F,H,W], U [F,H/2,W/2], V) uint8, BT.709 limited range."""
    Fn, _, H, W = frames.shape
    if not frames.is_cuda:
        x = (frames.float() * 0.5 + 0.5).clamp(0, 1)
        r, g, b = x[:, 0], x[:, 1], x[:, 2]
        yy = 0.2126 * r + 0.7152 * g + 0.0722 * b
        cb = TF.avg_pool2d(((b - yy) / 1.8556)[:, None], 2)[:, 0]
        cr = TF.avg_pool2d(((r - yy) / 1.5748)[:, None], 2)[:, 0]
        q = lambda t: t.round().clamp(0, 255).to(torch.uint8)
        return q(16 + 219 * yy), q(128 + 224 * cb), q(128 + 224 * cr)
    frames = frames.float().contiguous()
    y = torch.empty(Fn, H, W, dtype=torch.uint8, device=frames.device)
    u = torch.empty(Fn, H // 2, W // 2, dtype=torch.uint8, device=frames.device)
    v = torch.empty_like(u)
    N.call("us_rgb_to_yuv420", N.ptr(frames), N.ptr(y), N.ptr(u), N.ptr(v), Fn, H, W, N.stream())
    return y, u, v


def rgb_bytes(frames: torch.Tensor) -> torch.Tensor:
    """[F, 3, H, W] in [-1, 1] -> [F, H, W, 3] uint8."""
    Fn, _, H, W = frames.shape
    if not frames.is_cuda:
        x = ((frames.float() * 0.5 + 0.5).clamp(0, 1) * 255).round().to(torch.uint8)
        return x.permute(0, 2, 3, 1).contiguous()
    out = torch.empty(Fn, H, W, 3, dtype=torch.uint8, device=frames.device)
    N.call("us_rgb_bytes", N.ptr(frames.float().contiguous()), N.ptr(out), Fn, H, W, N.stream())
    return out


def pcm_interleave(audio: torch.Tensor) -> torch.Tensor:
    """[channels, samples] fp32 -> [samples, channels] int16 (clamped)."""
    C, S = audio.shape
    if not audio.is_cuda:
        return (audio.float().clamp(-1, 1) * 32767).round().to(torch.int16).t().contiguous()
    out = torch.empty(S, C, dtype=torch.int16, device=audio.device)
    N.call("us_pcm_interleave", N.ptr(audio.float().contiguous()), N.ptr(out), C, S, N.stream())
    return out


def _ramp(n, overlap, lo_edge, hi_edge, device):
    w = torch.ones(n, device=device)
    if overlap > 0:
        i = torch.arange(n, device=device, dtype=torch.float32)
        if not lo_edge:
            w = torch.minimum(w, torch.where(i < overlap, (i + 1) / (overlap + 1), torch.ones_like(i)))
        if not hi_edge:
            w = torch.minimum(w, torch.where(i >= n - overlap, (n - i) / (overlap + 1), torch.ones_like(i)))
    return w


def tile_stitch_(canvas, weight, tile, y0, x0, overlap):
    """Accumulates ``tile [F, C, th, tw]`` into ``canvas [F, C, H, W]`` with linear
    cross-fade weights over the overlap; ``weight [H, W]`` collects the weights."""
    Fn, C, H, W = canvas.shape
    th, tw = tile.shape[-2:]
    if not canvas.is_cuda:
        wy = _ramp(th, overlap, y0 == 0, y0 + th >= H, canvas.device)
        wx = _ramp(tw, overlap, x0 == 0, x0 + tw >= W, canvas.device)
        w2 = wy[:, None] * wx[None, :]
        hh, ww = min(th, H - y0), min(tw, W - x0)
        canvas[:, :, y0:y0 + hh, x0:x0 + ww] += tile[:, :, :hh, :ww] * w2[:hh, :ww]
        weight[y0:y0 + hh, x0:x0 + ww] += w2[:hh, :ww]
        return
    N.call("us_tile_stitch", N.ptr(tile.float().contiguous()), N.ptr(canvas), N.ptr(weight),
           Fn * C, H, W, th, tw, y0, x0, overlap, N.stream())


def tile_normalise_(canvas, weight):
    Fn, C, H, W = canvas.shape
    if not canvas.is_cuda:
        canvas /= weight.clamp_min(1e-12)
        return canvas
    N.call("us_tile_normalise", N.ptr(canvas), N.ptr(weight), Fn * C, H, W, N.stream())
    return canvas


def cross_fade(a, b):
    """Blend along dim 0: out[i] = a[i] (1 - i/n) + b[i] (i/n)."""
    n = a.shape[0]
    if not a.is_cuda:
        t = (torch.arange(n, dtype=torch.float32) / n).view(n, *([1] * (a.dim() - 1)))
        return a * (1 - t) + b * t
    out = torch.empty_like(a, dtype=torch.float32)
    N.call("us_cross_fade", N.ptr(a.float().contiguous()), N.ptr(b.float().contiguous()),
           N.ptr(out), n, a[0].numel(), N.stream())
    return out


# ------------------------------------------------------------- audio convs --
def conv1d(x, w, bias=None, stride=1, padding=0, dilation=1):
    if not x.is_cuda:
        return TF.conv1d(x.float(), w.float(), None if bias is None else bias.float(), stride,
                         padding, dilation)
    B, Cin, L = x.shape
    Cout, _, K = w.shape
    Lout = (L + 2 * padding - dilation * (K - 1) - 1) // stride + 1
    out = torch.empty(B, Cout, Lout, dtype=torch.float32, device=x.device)
    N.call("us_conv1d", N.ptr(x.float().contiguous()), N.ptr(w.float().contiguous()), N.ptr(bias),
           N.ptr(out), B, Cin, Cout, L, K, stride, padding, dilation, N.stream())
    return out


def conv_transpose1d(x, w, bias=None, stride=1, padding=0):
    """w: [Cin, Cout, K] (PyTorch layout)."""
    if not x.is_cuda:
        return TF.conv_transpose1d(x.float(), w.float(), None if bias is None else bias.float(),
                                   stride, padding)
    B, Cin, L = x.shape
    _, Cout, K = w.shape
    Lout = (L - 1) * stride - 2 * padding + K
    out = torch.empty(B, Cout, Lout, dtype=torch.float32, device=x.device)
    N.call("us_conv_transpose1d", N.ptr(x.float().contiguous()), N.ptr(w.float().contiguous()),
           N.ptr(bias), N.ptr(out), B, Cin, Cout, L, K, stride, padding, N.stream())
    return out


def snake_ref(x, log_alpha, log_beta):
    a = log_alpha.exp()[None, :, None]
    b = log_beta.exp()[None, :, None]
    return x + torch.sin(a * x) ** 2 / (b + 1e-9)


def kaiser_sinc_taps(n: int = 12, cutoff: float = 0.25) -> torch.Tensor:
    """Low-pass FIR of the anti-aliased activation (unit DC gain)."""
    half = n / 2
    t = torch.arange(n, dtype=torch.float64) - half + 0.5
    win = torch.kaiser_window(n, periodic=False, beta=6.0, dtype=torch.float64)
    h = 2 * cutoff * win * torch.sinc(2 * cutoff * t)
    return (h / h.sum()).float()


def activation1d_ref(x, taps, log_alpha, log_beta):
    """2x upsample (zero stuffing + FIR, gain 2) -> snake -> FIR -> keep every 2nd."""
    B, C, L = x.shape
    n = taps.numel()
    half = n // 2
    up = torch.zeros(B, C, 2 * L, dtype=torch.float32, device=x.device)
    # replicate padding in the sample domain, as the kernel does
    idx = torch.arange(-n, L + n, device=x.device).clamp(0, L - 1)
    xp = x.float()[:, :, idx]                       # [B, C, L + 2n]
    stuffed = torch.zeros(B, C, 2 * xp.shape[-1], device=x.device)
    stuffed[:, :, 0::2] = xp
    k = (2 * taps).view(1, 1, n).to(x.device)
    lp = TF.conv1d(stuffed.view(B * C, 1, -1), k).view(B, C, -1)
    # lp[j] = sum_k 2 taps[k] stuffed[j + k]; up-rate index u = j + half - 2n
    u0 = 2 * n - half
    up_full = lp[:, :, :]                           # index j <-> u = j - u0 ... (see below)
    act = snake_ref(up_full, log_alpha, log_beta)
    k2 = taps.view(1, 1, n).to(x.device)
    dn = TF.conv1d(act.view(B * C, 1, -1), k2).view(B, C, -1)
    # dn[m] = sum_j taps[j] act[m + j], act index m + j <-> u = m + j - u0
    # kernel: out[t] = sum_j taps[j] act_u[2t - half + j]  =>  m = 2t - half + u0
    start = u0 - half
    return dn[:, :, start:start + 2 * L:2]


def activation1d(x, taps, log_alpha, log_beta):
    if not x.is_cuda:
        return activation1d_ref(x, taps, log_alpha, log_beta)
    B, C, L = x.shape
    out = torch.empty(B, C, L, dtype=torch.float32, device=x.device)
    N.call("us_activation1d", N.ptr(x.float().contiguous()), N.ptr(taps.float().contiguous()),
           N.ptr(log_alpha), N.ptr(log_beta), N.ptr(out), B, C, L, taps.numel(), N.stream())
    return out


# ------------------------------------------------------------- host writers --
_bound = False


def _host():
    global _bound
    lib = N.host()
    if not _bound:
        vp, ll, ci = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int
        lib.us_mp4_write.restype = ll
        lib.us_mp4_write.argtypes = [ctypes.c_char_p, ci, ci, ci, ci, vp, vp, vp, vp, ll, ci, ci]
        lib.us_mp4_build.restype = vp
        lib.us_mp4_build.argtypes = [ci, ci, ci, ci, vp, vp, vp, vp, ll, ci, ci,
                                     ctypes.POINTER(ll)]
        lib.us_mp4_take.restype = ll
        lib.us_mp4_take.argtypes = [vp, vp]
        lib.us_h264_encode_annexb.restype = ll
        lib.us_h264_encode_annexb.argtypes = [ctypes.c_char_p, ci, ci, ci, vp, vp, vp]
        lib.us_wav_write.restype = ll
        lib.us_wav_write.argtypes = [ctypes.c_char_p, vp, ll, ci, ci]
        _bound = True
    return lib


def write_mp4(y, u, v, fps: int, pcm=None, sample_rate: int = 32000, path=None) -> bytes:
    """Planes as uint8 tensors [F,H,W] / [F,H/2,W/2] (any device); pcm int16
    [samples, channels].  Returns the MP4 bytes (H.264 video, 16-bit PCM audio)."""
    lib = _host()
    yn = np.ascontiguousarray(y.cpu().numpy())
    un = np.ascontiguousarray(u.cpu().numpy())
    vn = np.ascontiguousarray(v.cpu().numpy())
    Fn, H, W = yn.shape
    pn, frames, ch = None, 0, 0
    if pcm is not None and pcm.numel():
        pn = np.ascontiguousarray(pcm.cpu().numpy())
        frames, ch = pn.shape
    if path is None:
        # built in memory: the pictures are encoded in parallel, then copied straight into a
        # bytes object of the exact size (created uninitialised through the C API, filled
        # before anything else can see it) - no file round trip, no zeroed scratch, no copy
        size = ctypes.c_longlong(0)
        handle = lib.us_mp4_build(W, H, fps, Fn, yn.ctypes.data, un.ctypes.data, vn.ctypes.data,
                                  pn.ctypes.data if pn is not None else None, frames, ch,
                                  sample_rate, ctypes.byref(size))
        if not handle:
            raise RuntimeError("MP4 writer failed")
        api = ctypes.pythonapi
        api.PyBytes_FromStringAndSize.restype = ctypes.py_object
        api.PyBytes_FromStringAndSize.argtypes = [ctypes.c_char_p, ctypes.c_ssize_t]
        api.PyBytes_AsString.restype = ctypes.c_void_p
        api.PyBytes_AsString.argtypes = [ctypes.py_object]
        out = api.PyBytes_FromStringAndSize(None, size.value)
        lib.us_mp4_take(handle, api.PyBytes_AsString(out))
        return out
    n = lib.us_mp4_write(str(path).encode(), W, H, fps, Fn, yn.ctypes.data, un.ctypes.data,
                         vn.ctypes.data, pn.ctypes.data if pn is not None else None, frames, ch,
                         sample_rate)
    if n < 0:
        raise RuntimeError("MP4 writer failed")
    return b""
