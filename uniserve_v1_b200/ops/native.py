"""ctypes binding of the in-tree native libraries.

``libus_kernels.so`` holds every CUDA kernel (sm_100a) behind plain C entry
points ``int us_*(…, void* stream)``; ``libus_host.so`` holds the host-side C++
runtime (block manager, batch assembly, media writers).  An op called on a
CUDA tensor without the kernel library present raises: there is no silent
fallback on a GPU.

The calling convention mirrors the reference's native kernel entry
``int32_t entry(const Call*, void* stream)`` (crates/ops/src/kernel.rs:19-31,
reference project path) without the generated call structs.
"""
from __future__ import annotations

import ctypes
import os
import threading
from ctypes import c_char_p, c_float, c_int, c_longlong, c_ulonglong, c_void_p, c_size_t, POINTER
from pathlib import Path

import torch

_LIB_DIR = Path(__file__).resolve().parent.parent / "_lib"
_lock = threading.Lock()
_kernels = None
_host = None

# Number of kernel launches issued through this module (bench.py reports it).
launch_count = 0

P = c_void_p
I = c_int
L = c_longlong
F = c_float

_SIGNATURES = {
    "us_last_error": (c_char_p, []),
    "us_status_read": (I, [P]),
    "us_device_info": (I, [P, P, P, P]),
    "us_gemm_wx": (I, [P, P, P, I, I, I, I, I, L, L, L, I, I, I, I, P, I, P, P, P, P, P, P, I, I, P]),
    "us_gemm_wx_hint": (I, [I]),
    "us_linear_decode": (I, [P, P, P, P, I, I, I, L, L, L, I, I, P]),
    "us_kv_write_scaled": (I, [P, P, L, L, P, P, P, P, P, I, I, I, I, P]),
    "us_kv_gather": (I, [P, P, P, P, P, I, P, P, I, I, I, I, I, P, P, L, I, P]),
    "us_paged_decode_attention_fp8": (I, [P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I,
                                          F, L, L, P]),
    "us_causal_conv1d": (I, [P, L, P, P, P, L, P, P, I, I, I, I, I, I, P]),
    "us_gated_delta_rule": (I, [P, P, P, L, L, L, I, I, I, I, P, P, P, P, L, P, P, P, P, P, P,
                                I, I, I, I, I, F, P]),
    "us_rmsnorm_gated": (I, [P, P, P, L, I, P, I, I, I, F, I, P]),
    "us_rmsnorm": (I, [P, P, P, I, I, L, L, F, P]),
    "us_add_rmsnorm": (I, [P, P, P, P, I, I, F, I, P]),
    "us_modulated_rmsnorm": (I, [P, P, P, P, I, I, I, P, I, I, F, P]),
    "us_gated_residual": (I, [P, P, P, P, I, I, I, I, P]),
    "us_layer_norm": (I, [P, P, P, P, I, I, F, P]),
    "us_qk_norm_rope_kv": (I, [P, P, P, P, P, P, P, P, I, I, I, I, I, I, F, P]),
    "us_qk_norm_rope3": (I, [P, P, P, P, P, P, I, I, I, I, I, L, L, F, P]),
    "us_qk_norm_rope3_table": (I, [P, P, P, P, P, I, I, I, I, I, L, L, F, P]),
    "us_paged_decode_scratch_bytes": (L, [I, I, I, I]),
    "us_paged_decode_persist_scratch_bytes": (L, []),
    "us_paged_decode_attention_persist": (I, [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, F, L, L, P]),
    "us_paged_decode_attention": (I, [P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, L, L, P]),
    "us_paged_decode_attention_tc": (I, [P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, F, L, L, P]),
    "us_paged_decode_attention_tc_merged": (I, [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, F,
                                            L, L, P]),
    "us_unpermute_add_rmsnorm": (I, [P, P, P, I, I, I, P, P, P, F, I, P]),
    "us_route_sort_gather": (I, [P, P, P, I, I, I, I, P, I, I, I, I, P, P, P, P, P, P, P, P, I, P,
                                 P, P]),
    "us_topk_softmax": (I, [P, P, P, I, I, I, I, P, P, P, P]),
    "us_moe_sort": (I, [P, I, I, I, I, I, P, P, P, P, P, P, P, P]),
    "us_route_sort": (I, [P, P, P, I, I, I, I, P, I, I, I, I, P, P, P, P, P, P, P, P]),
    "us_moe_gather": (I, [P, P, P, I, I, I, P, P]),
    "us_moe_unpermute": (I, [P, P, P, I, I, I, P, P]),
    "us_argmax": (I, [P, I, I, L, P, P]),
    "us_logits_shape": (I, [P, I, I, L, P, P, P, P, P, P, P, P, P, P, P]),
    "us_sample_from_logits": (I, [P, I, I, L, P, P, P, P, P, P, P]),
    "us_logprob_stats": (I, [P, I, I, L, P, P, P, P, P]),
    "us_embedding": (I, [P, P, I, I, I, I, P, P]),
    "us_gather_rows": (I, [P, P, I, I, L, P, P]),
    "us_decode_advance": (I, [P, P, P, P, P, P, I, I, I, P, P, I, I, P, P]),
    "us_cast": (I, [P, P, L, I, P]),
}


class NativeMissing(RuntimeError):
    pass


def kernels_path() -> Path:
    return _LIB_DIR / "libus_kernels.so"


def host_path() -> Path:
    return _LIB_DIR / "libus_host.so"


def _bind(lib, table, strict=False):
    for name, (res, args) in table.items():
        try:
            fn = getattr(lib, name)
        except AttributeError:
            if strict:
                raise
            continue
        fn.restype = res
        fn.argtypes = args


def register_signatures(table: dict) -> None:
    """Lets other op modules add the entry points they own."""
    _SIGNATURES.update(table)
    if _kernels is not None:
        _bind(_kernels, table)


def kernels():
    """The CUDA kernel library (loaded once)."""
    global _kernels
    if _kernels is not None:
        return _kernels
    with _lock:
        if _kernels is None:
            path = kernels_path()
            if not path.exists():
                raise NativeMissing(
                    f"{path} is missing: run `python -m uniserve_v1_b200.build` (needs nvcc)")
            lib = ctypes.CDLL(str(path), mode=ctypes.RTLD_GLOBAL)
            _bind(lib, _SIGNATURES)
            _kernels = lib
    return _kernels


def host():
    """The host C++ runtime library (loaded once)."""
    global _host
    if _host is not None:
        return _host
    with _lock:
        if _host is None:
            path = host_path()
            if not path.exists():
                raise NativeMissing(
                    f"{path} is missing: run `python -m uniserve_v1_b200.build` (needs g++)")
            _host = ctypes.CDLL(str(path))
    return _host


def have_kernels() -> bool:
    return kernels_path().exists()


def ptr(t):
    """Device (or host) address of a tensor as a void pointer; None passes NULL."""
    if t is None:
        return None
    return c_void_p(t.data_ptr())


def stream():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def check(rc: int, what: str = "") -> None:
    if rc != 0:
        msg = kernels().us_last_error()
        raise RuntimeError(f"{what or 'native call'} failed with status {rc}: "
                           f"{msg.decode() if msg else ''}")


def call(name: str, *args, launches: int = 1) -> None:
    """Calls an ``int us_*`` entry point and raises on a non-zero status."""
    global launch_count
    fn = getattr(kernels(), name)
    rc = fn(*args)
    if rc != 0:
        check(rc, name)
    launch_count += launches


def read_status() -> int:
    """Reads and clears the device status word (synchronises the device)."""
    out = ctypes.c_uint(0)
    check(kernels().us_status_read(ctypes.byref(out)), "us_status_read")
    return out.value


STATUS_NAMES = {
    0: "ok",
    0x100: "timeout waiting for a TMA stage",
    0x200: "timeout waiting for a free stage",
    0x300: "timeout waiting for the accumulator",
    0x400: "timeout waiting for a peer flag",
    0x500: "index outside its table",
    0x600: "timeout waiting for another CTA of the grid",
}


def raise_on_device_error() -> None:
    code = read_status()
    if code:
        raise RuntimeError(f"device status {code:#x}: {STATUS_NAMES.get(code, 'unknown')}")
