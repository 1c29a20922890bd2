"""Weight adapters: a safetensors file of edits fused into a checkpoint at the
loading boundary.

Roles of an adapter tensor, by the suffix of its name (the ``fastvideo-lora-v2``
container of the FastH3 students)::

    <param>.lora_A   [rank, in]     down projection   }  contributes  up @ down
    <param>.lora_B   [out, rank]    up projection     }  (unscaled: alpha is folded in)
    <param>.diff     like <param>   added as it is
    <param>.diff_b   like the bias  added to ``<module>.bias``
    <param>.set_weight              a parameter the base does not hold, assigned

``<param>`` names the module (``blocks.3.attn.to_q``); the edited tensor is
``<param>.weight`` (or ``.bias`` for ``diff_b``).  For one element of an edited
parameter ``fused = round((up @ down + diff) + base)``: the delta is evaluated in
FP32 from the stored values, added to the widened base and rounded once into the
base tensor's own type.  ``AdaptedLoader`` wraps a ``CheckpointLoader`` so that
every ``get`` of an edited tensor returns the fused value and everything else is
read from its shard as without an adapter.

Reference: crates/nn/src/adapter.rs:1-45 (roles, fusion rule), docs/minimax_h3/minimax_h3.md:43-45
(container); reference project paths.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Optional

import torch

from .safetensors_io import Shard

SUFFIXES = (".lora_A", ".lora_B", ".diff", ".diff_b", ".set_weight")


class Adapter:
    def __init__(self, path):
        p = Path(path)
        if p.is_dir():
            p = p / "adapter_model.safetensors"
        self.path = p
        self.shard = Shard(p)
        self.edits: dict = {}          # module -> {role: tensor name}
        for name in self.shard.names():
            for suf in SUFFIXES:
                if name.endswith(suf):
                    self.edits.setdefault(name[:-len(suf)], {})[suf[1:]] = name
                    break
            else:
                raise ValueError(f"{p}: tensor {name!r} has no adapter role")
        for mod, roles in self.edits.items():
            if ("lora_A" in roles) != ("lora_B" in roles):
                raise ValueError(f"{p}: {mod} carries one low-rank factor without the other")
        contract = p.parent / "fastvideo_inference.json"
        self.contract = json.loads(contract.read_text()) if contract.exists() else {}

    def contents(self) -> dict:
        c = {"low_rank": 0, "diff": 0, "assign": 0}
        for roles in self.edits.values():
            c["low_rank"] += 2 * ("lora_A" in roles)
            c["diff"] += ("diff" in roles) + ("diff_b" in roles)
            c["assign"] += "set_weight" in roles
        return c

    def edits_tensor(self, name: str) -> bool:
        mod, _, leaf = name.rpartition(".")
        roles = self.edits.get(mod)
        if not roles:
            return False
        if leaf == "weight":
            return bool({"lora_A", "diff", "set_weight"} & roles.keys())
        return leaf == "bias" and "diff_b" in roles

    def assigned(self):
        """Names of the parameters the adapter adds (the base does not hold them)."""
        return [m + ".weight" for m, r in self.edits.items() if "set_weight" in r]

    def fuse(self, name: str, base: Optional[torch.Tensor]) -> torch.Tensor:
        mod, _, leaf = name.rpartition(".")
        roles = self.edits[mod]
        get = lambda role: self.shard.get(roles[role]).float()
        if leaf == "bias":
            return (get("diff_b") + base.float()).to(base.dtype)
        if "set_weight" in roles:
            return self.shard.get(roles["set_weight"])
        delta = None
        if "lora_A" in roles:
            down, up = get("lora_A"), get("lora_B")
            if up.shape[1] != down.shape[0]:
                raise ValueError(f"{mod}: factor ranks {tuple(up.shape)} x {tuple(down.shape)}")
            delta = up @ down
        if "diff" in roles:
            d = get("diff")
            delta = d if delta is None else delta + d
        if tuple(delta.shape) != tuple(base.shape):
            raise ValueError(f"{name}: edit of shape {tuple(delta.shape)} on a parameter of "
                             f"shape {tuple(base.shape)}")
        return (delta + base.float()).to(base.dtype)


class AdaptedLoader:
    """A checkpoint with an adapter attached: same ``get`` / ``has`` / ``names``."""

    def __init__(self, loader, adapter: Adapter):
        self.loader, self.adapter = loader, adapter
        self.config = loader.config
        self._extra = set(adapter.assigned())
        missing = [m for m, r in adapter.edits.items()
                   if "set_weight" not in r and not loader.has(m + ".weight")]
        if missing:
            raise KeyError(f"adapter edits parameters the checkpoint does not hold: {missing[:3]}")

    def has(self, name: str) -> bool:
        return name in self._extra or self.loader.has(name)

    def names(self):
        return set(self.loader.names()) | self._extra

    def get(self, name: str) -> torch.Tensor:
        if not self.adapter.edits_tensor(name):
            return self.loader.get(name)
        base = self.loader.get(name) if self.loader.has(name) else None
        return self.adapter.fuse(name, base)
