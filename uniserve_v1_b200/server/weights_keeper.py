"""Retained weights: a keeper process holds a model's weight tensors so that a serving process
that starts (or restarts) maps them instead of reading a checkpoint again.

    python -m uniserve_v1_b200 keep PACKAGE_DIR --socket /run/uniserve/weights.sock
    python -m uniserve_v1_b200 serve PACKAGE_DIR --weights-socket /run/uniserve/weights.sock

The keeper loads the package's model once and answers ``manifest`` requests on a unix socket
with one record per weight tensor: a key (``m.embed``, ``l3.w13`` ...), its
shape, dtype and where it lives.  On a GPU the tensor stays in the keeper's device memory and
the record carries a CUDA IPC handle: the serving process opens it and its model's tensors
ARE the keeper's memory (no copy, no second 57 GB).  On CPU ranks the tensors live in files
under ``/dev/shm`` that both processes map.  The serving process builds its model object
without weights and fills it from the records; everything else (KV cache, graphs, scheduler)
is its own, so it can fail, restart, hot-restart or be replaced by a standby without the
weights moving.  The keeper is the only writer; consumers treat the tensors as read-only.

A keeper is tied to one weights identity (model, dtype, parallel layout, rank): a consumer
that asks with another identity is refused and loads the checkpoint itself.

Reference behaviour: crates/storage-server (weights retained by the Storage Server across
engine generations; reference project path).  The keeper retains weights only; the content-keyed
KV pages travel between generations as a file (``engine/prefix_store.py``).
"""
from __future__ import annotations

import base64
import json
import os
import socket
import struct
import threading
from dataclasses import fields
from typing import Optional

import torch

_DTYPES = {str(d): d for d in (torch.bfloat16, torch.float16, torch.float32, torch.uint8,
                               torch.int32, torch.int64, torch.float8_e4m3fn)}


def weight_records(model):
    """(key, holder, attribute, tensor) of every weight tensor of a model, with keys that are
    the same in every process that builds the same model."""
    def walk(prefix, holder):
        items = holder.items() if isinstance(holder, dict) else vars(holder).items()
        for name, v in sorted(items, key=lambda kv: str(kv[0])):
            if torch.is_tensor(v) and v.dim() > 0:
                yield f"{prefix}.{name}", holder, name, v
    yield from walk("m", model)
    for i, lw in enumerate(getattr(model, "layers", None) or []):
        if lw is None:
            continue
        yield from walk(f"l{i}", lw)


def identity_of(model) -> dict:
    c = model.cfg
    return {"family": type(model).__name__, "hidden": c.hidden_size, "layers": c.num_hidden_layers,
            "experts": getattr(c, "num_experts", 0), "vocab": c.vocab_size,
            "dtype": str(model.dtype), "tp": model.ctx.tp_size, "tp_rank": model.ctx.tp_rank,
            "ep": model.ctx.ep_size, "layer_lo": model.layer_lo, "layer_hi": model.layer_hi,
            "expert_quant": model.expert_quant}


def _plain_fields(record) -> dict:
    """The non-tensor fields of a per-layer weight record (flags such as ``dense``)."""
    return {f.name: getattr(record, f.name) for f in fields(record)
            if isinstance(getattr(record, f.name), (bool, int, float, str))}


def _handle_to_json(handle) -> str:
    """A CUDA IPC storage handle (a flat tuple of integers, booleans and byte strings) as
    text: byte strings become ``{"b": base64}``.  Nothing but those three kinds is accepted,
    so reading a record never constructs an object of the sender's choosing."""
    out = []
    for x in handle:
        if isinstance(x, (bytes, bytearray)):
            out.append({"b": base64.b64encode(bytes(x)).decode()})
        elif isinstance(x, (bool, int)):
            out.append(x)
        else:
            raise TypeError(f"unexpected field of kind {type(x).__name__} in an IPC handle")
    return json.dumps(out, separators=(",", ":"))


def _handle_from_json(text: str) -> tuple:
    fields_ = json.loads(text)
    if not isinstance(fields_, list) or len(fields_) > 16:
        raise ValueError("not an IPC handle record")
    out = []
    for x in fields_:
        if isinstance(x, dict) and set(x) == {"b"} and isinstance(x["b"], str):
            out.append(base64.b64decode(x["b"], validate=True))
        elif isinstance(x, (bool, int)):
            out.append(x)
        else:
            raise ValueError("not an IPC handle record")
    return tuple(out)


def _send(sock, obj) -> None:
    data = json.dumps(obj).encode()
    sock.sendall(struct.pack(">Q", len(data)) + data)


def _recv(sock):
    head = b""
    while len(head) < 8:
        chunk = sock.recv(8 - len(head))
        if not chunk:
            return None
        head += chunk
    n = struct.unpack(">Q", head)[0]
    buf = bytearray()
    while len(buf) < n:
        chunk = sock.recv(min(1 << 20, n - len(buf)))
        if not chunk:
            return None
        buf += chunk
    return json.loads(bytes(buf))


class WeightsKeeper:
    def __init__(self, model, socket_path: str, shm_prefix: Optional[str] = None):
        if getattr(model, "expert_quant", None):
            raise ValueError("quantised expert records are not retained; keep the bf16 weights")
        self.model, self.path = model, socket_path
        self.identity = identity_of(model)
        self.shm_prefix = shm_prefix or f"/dev/shm/uniserve-weights-{os.getpid()}"
        self.records, self.files = [], []
        self._alive = []                           # tensors whose memory the records name
        seen = {}
        for key, _holder, _name, t in weight_records(model):
            if id(t) in seen:                      # tied weights: one memory, two keys
                self.records.append(dict(seen[id(t)], key=key))
                continue
            rec = {"key": key, "shape": list(t.shape), "dtype": str(t.dtype),
                   "stride": list(t.stride()), "device": t.device.type}
            if t.is_cuda:
                st = t.untyped_storage()
                handle = st._share_cuda_()
                rec["cuda"] = _handle_to_json(handle)
                rec["offset"] = t.storage_offset()
                self._alive.append(t)
            else:
                fn = f"{self.shm_prefix}-{len(self.files)}"
                nbytes = t.numel() * t.element_size()
                shared = torch.from_file(fn, shared=True, size=max(1, nbytes), dtype=torch.uint8)
                shared[:nbytes].copy_(t.contiguous().view(-1).view(torch.uint8))
                rec["file"], rec["nbytes"] = fn, nbytes
                rec["stride"] = list(t.contiguous().stride())
                self.files.append(fn)
                self._alive.append(shared)
            seen[id(t)] = rec
            self.records.append(rec)
        self.meta = [None if lw is None else _plain_fields(lw) for lw in model.layers]
        self.model_meta = {k: getattr(model, k) for k in ("vocab_lo", "vocab_hi")
                           if hasattr(model, k)}
        self.served = 0
        self._stop = threading.Event()
        self.sock: Optional[socket.socket] = None

    def serve_forever(self, ready=None) -> None:
        if os.path.exists(self.path):
            os.unlink(self.path)
        self.sock = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        self.sock.bind(self.path)
        self.sock.listen(16)
        self.sock.settimeout(0.25)
        if ready is not None:
            ready()
        try:
            while not self._stop.is_set():
                try:
                    conn, _ = self.sock.accept()
                except socket.timeout:
                    continue
                with conn:
                    req = _recv(conn)
                    if not req:
                        continue
                    if req.get("op") == "stop":
                        _send(conn, {"ok": True})
                        break
                    if req.get("identity") != self.identity:
                        _send(conn, {"ok": False, "error": "another weights identity",
                                     "identity": self.identity})
                        continue
                    _send(conn, {"ok": True, "identity": self.identity, "records": self.records,
                                 "layers": self.meta, "model": self.model_meta,
                                 "pid": os.getpid()})
                    self.served += 1
        finally:
            self.close()

    def stop(self) -> None:
        self._stop.set()

    def close(self) -> None:
        if self.sock is not None:
            self.sock.close()
            self.sock = None
        if os.path.exists(self.path):
            os.unlink(self.path)
        for fn in self.files:
            try:
                os.unlink(fn)
            except OSError:
                pass
        self.files = []


def _open(rec: dict, device) -> torch.Tensor:
    dtype = _DTYPES[rec["dtype"]]
    if "cuda" in rec:
        handle = _handle_from_json(rec["cuda"])
        storage = torch.UntypedStorage._new_shared_cuda(*handle)
        t = torch.empty(0, dtype=dtype, device=storage.device)
        return t.set_(storage, rec["offset"], rec["shape"], rec["stride"])
    raw = torch.from_file(rec["file"], shared=True, size=max(1, rec["nbytes"]), dtype=torch.uint8)
    return raw[:rec["nbytes"]].view(dtype).as_strided(rec["shape"], rec["stride"])


def attach(model, socket_path: str, timeout: float = 10.0) -> bool:
    """Fills a weight-less ``model`` from the keeper behind ``socket_path``.  False when no
    keeper answers or it keeps another identity (the caller then loads the checkpoint)."""
    from ..models.qwen3_moe import LayerWeights
    try:
        s = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        s.settimeout(timeout)
        s.connect(socket_path)
    except OSError:
        return False
    with s:
        _send(s, {"op": "manifest", "identity": identity_of(model)})
        ans = _recv(s)
    if not ans or not ans.get("ok"):
        return False
    model.layers = []
    names = {f.name for f in fields(LayerWeights)}
    for meta in ans["layers"]:
        if meta is None:
            model.layers.append(None)
            continue
        kw = {n: None for n in names}
        kw.update({k: v for k, v in meta.items() if k in names})
        model.layers.append(LayerWeights(**kw))
    opened = {}
    for rec in ans["records"]:
        ident = rec.get("cuda") or rec.get("file")
        if ident not in opened:
            opened[ident] = _open(rec, model.device)
        t = opened[ident]
        parts = rec["key"].split(".")
        if parts[0] == "m":
            setattr(model, parts[1], t)
        elif len(parts) == 2:
            setattr(model.layers[int(parts[0][1:])], parts[1], t)
    for k, v in (ans.get("model") or {}).items():
        setattr(model, k, v)
    model.weights_from = {"keeper_pid": ans.get("pid"), "tensors": len(opened)}
    return True


def stop_keeper(socket_path: str) -> bool:
    try:
        s = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        s.settimeout(5.0)
        s.connect(socket_path)
    except OSError:
        return False
    with s:
        _send(s, {"op": "stop"})
        return bool(_recv(s))
