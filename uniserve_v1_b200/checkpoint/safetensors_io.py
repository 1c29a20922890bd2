"""Hugging Face safetensors checkpoints: memory-mapped shards, sharded index,
hub-cache resolution and family resolution.

A safetensors file is an 8-byte little-endian header length, a JSON header
``{name: {dtype, shape, data_offsets}}`` and the raw tensor bytes.  Shards are
mapped read-only; a tensor is a zero-copy view until it is moved to the device.
File identity (size, mtime, inode) keys retained weights.

Reference behaviour: crates/nn/src/checkpoint.rs:1-30 (mmap shards, index, file
identity), crates/daemon/src/api/model/assets/hub.rs (hub cache layout),
crates/processing/src/lib.rs ``Registry::resolve`` (family by ``architectures[0]`` /
``_class_name``) — reference project paths.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from pathlib import Path
from typing import Optional

import torch

_DTYPES = {"F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
           "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
           "U8": torch.uint8, "BOOL": torch.bool, "F64": torch.float64,
           "F8_E4M3": torch.float8_e4m3fn, "F8_E5M2": torch.float8_e5m2}
_NAMES = {v: k for k, v in _DTYPES.items()}


class Shard:
    def __init__(self, path: Path):
        self.path = Path(path)
        self.f = open(self.path, "rb")
        st = os.fstat(self.f.fileno())
        self.identity = (st.st_size, int(st.st_mtime_ns), st.st_ino)
        (n,) = struct.unpack("<Q", self.f.read(8))
        if n > st.st_size or n > (100 << 20):
            raise ValueError(f"{path}: implausible safetensors header length {n}")
        self.header = json.loads(self.f.read(n))
        self.metadata = self.header.pop("__metadata__", {})
        self.base = 8 + n
        self.mm = mmap.mmap(self.f.fileno(), 0, access=mmap.ACCESS_READ)

    def names(self):
        return self.header.keys()

    def get(self, name: str) -> torch.Tensor:
        e = self.header[name]
        lo, hi = e["data_offsets"]
        dt = _DTYPES[e["dtype"]]
        buf = memoryview(self.mm)[self.base + lo:self.base + hi]
        if hi == lo:
            return torch.empty(e["shape"], dtype=dt)
        t = torch.frombuffer(buf, dtype=dt)
        return t.view(e["shape"])


def save_file(tensors: dict, path, metadata: Optional[dict] = None) -> None:
    """Writes one safetensors file (used by tests and tools; tensors on CPU)."""
    header, off, blobs = {}, 0, []
    if metadata:
        header["__metadata__"] = {k: str(v) for k, v in metadata.items()}
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


class CheckpointLoader:
    """All shards of a checkpoint directory behind ``get`` / ``has``."""

    def __init__(self, directory):
        self.dir = Path(directory)
        self.shards: dict = {}
        self.where: dict = {}
        idx = self.dir / "model.safetensors.index.json"
        if idx.exists():
            wm = json.loads(idx.read_text())["weight_map"]
            for name, fn in wm.items():
                self.where[name] = fn
        else:
            files = sorted(self.dir.glob("*.safetensors"))
            if not files:
                raise FileNotFoundError(f"{self.dir}: no safetensors files")
            for fp in files:
                sh = self._shard(fp.name)
                for name in sh.names():
                    self.where[name] = fp.name
        cfg = self.dir / "config.json"
        self.config = json.loads(cfg.read_text()) if cfg.exists() else {}

    def _shard(self, fn: str) -> Shard:
        sh = self.shards.get(fn)
        if sh is None:
            sh = Shard(self.dir / fn)
            self.shards[fn] = sh
        return sh

    def has(self, name: str) -> bool:
        return name in self.where

    def get(self, name: str) -> torch.Tensor:
        if name not in self.where:
            raise KeyError(f"{self.dir}: no tensor {name!r}")
        return self._shard(self.where[name]).get(name)

    def names(self):
        return self.where.keys()

    def identity(self) -> tuple:
        """What retained weights are keyed by: every file's identity."""
        return tuple(sorted((fn, self._shard(fn).identity) for fn in set(self.where.values())))

    def quantization(self) -> Optional[dict]:
        """The checkpoint's own quantization declaration.  Block-scaled FP8
        (``weight_block_size``) is served here (128x128 weight blocks)."""
        return self.config.get("quantization_config")


# ------------------------------------------------------------------ hub cache --
def parse_model_id(spec: str):
    """``<owner>/<name>[@<revision>][/<folder>]`` -> (repo, revision, folder)."""
    rev, folder = None, None
    parts = spec.split("/")
    if len(parts) < 2:
        raise ValueError(f"not a repository id: {spec!r}")
    owner, name = parts[0], parts[1]
    if "@" in name:
        name, rev = name.split("@", 1)
    if len(parts) > 2:
        folder = "/".join(parts[2:])
    return f"{owner}/{name}", rev, folder


def resolve_hub(spec: str, cache_dir: Optional[str] = None) -> Path:
    """Finds a checkpoint in the local Hugging Face hub cache (no download: the
    deployment host is offline; ``HF_HUB_OFFLINE`` semantics)."""
    repo, rev, folder = parse_model_id(spec)
    root = Path(cache_dir or os.environ.get("HF_HUB_CACHE")
                or Path(os.environ.get("HF_HOME", Path.home() / ".cache/huggingface")) / "hub")
    d = root / ("models--" + repo.replace("/", "--"))
    if not d.exists():
        raise FileNotFoundError(f"{spec}: not in the hub cache at {root} (offline)")
    if rev is None:
        ref = d / "refs" / "main"
        rev = ref.read_text().strip() if ref.exists() else None
    snaps = d / "snapshots"
    if rev and (snaps / rev).exists():
        snap = snaps / rev
    else:
        ref = d / "refs" / (rev or "main")
        if ref.exists():
            snap = snaps / ref.read_text().strip()
        else:
            cands = sorted(snaps.iterdir())
            if not cands:
                raise FileNotFoundError(f"{spec}: no snapshot in {d}")
            snap = cands[-1]
    return snap / folder if folder else snap


# ------------------------------------------------------------ family registry --
FAMILIES = {
    "Qwen3MoeForCausalLM": "qwen3_moe", "Qwen3ForCausalLM": "qwen3_moe",
    "Qwen3_5MoeForConditionalGeneration": "qwen3_5_moe", "Qwen3_5MoeForCausalLM": "qwen3_5_moe",
    "Qwen3NextForCausalLM": "qwen3_5_moe", "Qwen3_5ForCausalLM": "qwen3_5_moe",
    "Qwen3_5ForConditionalGeneration": "qwen3_5_moe", "Qwen3VLForConditionalGeneration": "qwen3_vl",
    "Qwen3VLMoeForConditionalGeneration": "qwen3_vl",
    "Qwen4ExpForConditionalGeneration": "qwen4_exp", "Qwen4ExpForCausalLM": "qwen4_exp",
    "MiniMaxH3Pipeline": "minimax_h3", "FastH3Pipeline": "minimax_h3",
    "MiniMaxH3Transformer3DModel": "minimax_h3",
}


def resolve_family(directory) -> str:
    """Family of a checkpoint: transformers ``config.json`` -> ``architectures[0]``;
    diffusers ``model_index.json`` / ``modular_model_index.json`` -> ``_class_name``."""
    d = Path(directory)
    for fn, key in (("config.json", "architectures"), ("model_index.json", "_class_name"),
                    ("modular_model_index.json", "_class_name")):
        p = d / fn
        if p.exists():
            v = json.loads(p.read_text()).get(key)
            name = v[0] if isinstance(v, list) and v else v
            if name in FAMILIES:
                return FAMILIES[name]
            if name:
                raise ValueError(f"{d}: no family serves {name!r}")
    raise ValueError(f"{d}: neither config.json nor a pipeline index names a family")
