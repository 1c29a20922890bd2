"""Quantized checkpoints expanded while they are read.

``DequantizingLoader`` wraps any loader (``get`` / ``has`` / ``names``) and returns the
high-precision value of every quantized ``*.weight``; the companion scale tensors
disappear from ``names()``.  Recognised layouts:

* **NVFP4** (ModelOpt): ``weight`` uint8 [M, K / 2], ``weight_scale`` E4M3 [M, K / 16],
  ``weight_scale_2`` FP32 scalar;
* **per-tensor FP8** (ModelOpt static / dynamic): ``weight`` E4M3, ``weight_scale`` scalar;
* **block-scaled FP8**: ``weight`` E4M3, ``weight_scale_inv`` [M / 128, K / 128].

A model that keeps some weights quantized on the device (the experts' block-scaled FP8
path, the FP8 feed-forward of the video transformer) re-quantizes from these values, so
every family can be served from every such export.  ``input_scale`` tensors (static
activation scales) stay readable under their own names.

Reference behaviour: crates/nn/src/quantization/{modelopt,nvfp4,dynamic}.rs,
crates/nn/src/quantization.rs:26-31 (reference project paths).
"""
from __future__ import annotations

import torch

from ..ops import nvfp4

_COMPANIONS = ("_scale", "_scale_2", "_scale_inv")


class DequantizingLoader:
    def __init__(self, loader, dtype=torch.bfloat16):
        self.loader, self.dtype = loader, dtype
        self.config = getattr(loader, "config", {})
        self.expanded = {"nvfp4": 0, "fp8_tensor": 0, "fp8_block": 0}

    def has(self, name: str) -> bool:
        return self.loader.has(name)

    def names(self):
        return {n for n in self.loader.names()
                if not any(n.endswith("weight" + c) for c in _COMPANIONS)}

    def kind(self, name: str):
        if not name.endswith("weight"):
            return None
        L = self.loader
        if L.has(name + "_scale_inv"):
            return "fp8_block"
        if L.has(name + "_scale") and L.has(name + "_scale_2"):
            return "nvfp4"
        if L.has(name + "_scale"):
            return "fp8_tensor"
        return None

    def get(self, name: str) -> torch.Tensor:
        kind = self.kind(name)
        w = self.loader.get(name)
        if kind is None:
            return w
        self.expanded[kind] += 1
        if kind == "nvfp4":
            return nvfp4.dequantize(w.view(torch.uint8), self.loader.get(name + "_scale"),
                                    self.loader.get(name + "_scale_2").float().reshape(-1)[0],
                                    self.dtype)
        if w.dtype == torch.uint8:
            w = w.view(torch.float8_e4m3fn)
        if kind == "fp8_tensor":
            s = self.loader.get(name + "_scale").float()
            return (w.float() * (s if s.numel() == 1 else s.reshape(-1, 1))).to(self.dtype)
        s = self.loader.get(name + "_scale_inv").float()           # [M / 128, K / 128] (ceil)
        M, K = w.shape
        full = s.repeat_interleave(128, 0)[:M].repeat_interleave(128, 1)[:, :K]
        return (w.float() * full).to(self.dtype)


def open_checkpoint(directory, dtype=torch.bfloat16):
    """A ``CheckpointLoader`` for ``directory``, wrapped when its config declares a
    quantization (``quantization_config`` or ModelOpt's ``hf_quant_config.json``)."""
    from pathlib import Path

    from .safetensors_io import CheckpointLoader
    loader = CheckpointLoader(directory)
    declared = loader.quantization() or (Path(directory) / "hf_quant_config.json").exists()
    if not declared:
        # undeclared exports still carry their scale tensors
        declared = any(n.endswith(("weight_scale", "weight_scale_inv")) for n in loader.names())
    return DequantizingLoader(loader, dtype) if declared else loader
