"""The prefix cache outlives the process that filled it.

A serving process that hands over to a successor (hot restart, a promoted standby, a restart
by hand) writes the content-keyed pages of its KV cache to a file - their chained keys and,
per layer, the page contents of both planes (with the page scales of E4M3 planes) - and the
successor reads them into its own cache before it serves, so the conversations and system
prompts that were cached stay cached.  Keys carry the weights identity and the isolation salt
(``BlockManager.page_keys``), so a file only matches the model that wrote it; the header's
page size, layer shapes and dtypes must equal the reader's.  Pages are written oldest first and
the newest ``max_bytes`` worth are kept; a page whose predecessors in its chain were dropped
is harmless (a look-up stops at the first missing page of a run).

File: ``MAGIC | u32 header length | JSON header | keys (n x 2 u64) | per layer: K pages, V
pages [, K scales, V scales]`` in host byte order.  Nothing in it is executable.

Reference behaviour: the Storage Server retains KV segments across engine generations
(crates/storage-server/src/restart.rs, crates/engine/src/memory/cache; reference project
paths); here the retention is a file between two generations of one deployment.
"""
from __future__ import annotations

import json
import os
import struct
from typing import Optional

import numpy as np
import torch

MAGIC = b"USPC\x01"
_DTYPES = {str(d): d for d in (torch.bfloat16, torch.float16, torch.float32, torch.uint8)}


def _layers(runner):
    return [(i, pair) for i, pair in enumerate(runner.kv_caches)
            if pair is not None and pair[0] is not None]


def _describe(engine) -> dict:
    runner = engine.runner
    layers = []
    for i, (k, v) in _layers(runner):
        layers.append({"layer": i, "shape": list(k.shape[1:]), "dtype": str(k.dtype),
                       "scaled": getattr(k, "page_scale", None) is not None})
    return {"identity": engine.blocks.identity, "page_size": engine.blocks.page_size,
            "layers": layers}


def _page_bytes(desc: dict) -> int:
    total = 0
    for lay in desc["layers"]:
        n = 1
        for x in lay["shape"]:
            n *= x
        total += 2 * n * _DTYPES[lay["dtype"]].itemsize + (8 if lay["scaled"] else 0)
    return total


def save_prefix_cache(engine, path: str, max_bytes: int = 1 << 30) -> dict:
    """Writes the engine's content-keyed pages to ``path`` (atomically: a temporary file is
    renamed).  Call on the engine's thread, between two steps."""
    blocks, runner = engine.blocks, engine.runner
    desc = _describe(engine)
    keys, pages = blocks.committed()
    per = max(1, _page_bytes(desc))
    n = int(min(len(pages), max(0, max_bytes // per)))
    keys, pages = keys[len(keys) - n:], pages[len(pages) - n:]
    desc["pages"] = n
    head = json.dumps(desc, separators=(",", ":")).encode()
    tmp = f"{path}.{os.getpid()}.tmp"
    idx = torch.as_tensor(pages.astype(np.int64), device=runner.device)
    with open(tmp, "wb") as f:
        f.write(MAGIC + struct.pack("<I", len(head)) + head)
        f.write(np.ascontiguousarray(keys, dtype=np.uint64).tobytes())
        for _, pair in _layers(runner):
            for plane in pair:
                sel = plane.index_select(0, idx).contiguous().cpu()
                f.write(sel.view(torch.uint8).numpy().tobytes() if n else b"")
            if getattr(pair[0], "page_scale", None) is not None:
                for plane in pair:
                    f.write(plane.page_scale.index_select(0, idx).float().cpu().numpy().tobytes())
    os.replace(tmp, path)
    return {"pages": n, "bytes": os.path.getsize(path), "path": path}


def load_prefix_cache(engine, path: str, remove: bool = True) -> dict:
    """Reads a file of ``save_prefix_cache`` into the engine's cache: pages are allocated,
    filled, committed under their keys and released (they stay as cached pages).  A file of
    another model, page size or cache layout is refused with the reason; pages that do not fit
    the free pool are dropped (oldest first)."""
    blocks, runner = engine.blocks, engine.runner
    try:
        with open(path, "rb") as f:
            data = f.read()
    except OSError as e:
        return {"pages": 0, "refused": str(e)}
    finally:
        if remove:
            try:
                os.unlink(path)
            except OSError:
                pass
    if len(data) < len(MAGIC) + 4 or data[:len(MAGIC)] != MAGIC:
        return {"pages": 0, "refused": "not a prefix-cache file"}
    (hl,) = struct.unpack_from("<I", data, len(MAGIC))
    off = len(MAGIC) + 4
    try:
        desc = json.loads(data[off:off + hl].decode())
        n = int(desc["pages"])
    except (ValueError, KeyError, UnicodeDecodeError):
        return {"pages": 0, "refused": "unreadable header"}
    off += hl
    mine = _describe(engine)
    for field in ("identity", "page_size", "layers"):
        if desc.get(field) != mine[field]:
            return {"pages": 0, "refused": f"{field} differs from this engine's"}
    if n <= 0:
        return {"pages": 0}
    if len(data) != off + 16 * n + n * _page_bytes(mine):
        return {"pages": 0, "refused": "file length does not match its header"}
    keys = np.frombuffer(data, dtype=np.uint64, count=2 * n, offset=off).reshape(n, 2)
    off += 16 * n
    take = min(n, max(0, blocks.num_free - 1))
    pages = blocks.allocate(take) if take > 0 else None
    if not pages:
        return {"pages": 0, "refused": "no free pages"}
    first = n - take                                    # the newest pages are at the end
    idx = torch.as_tensor(pages, dtype=torch.long, device=runner.device)
    for _, pair in _layers(runner):
        shape = list(pair[0].shape[1:])
        numel = int(np.prod(shape))
        for plane in pair:
            nbytes = n * numel * plane.element_size()
            raw = torch.frombuffer(bytearray(data[off:off + nbytes]), dtype=torch.uint8)
            off += nbytes
            sel = raw.view(plane.dtype).view(n, *shape)[first:]
            plane.index_copy_(0, idx, sel.to(runner.device))
        if getattr(pair[0], "page_scale", None) is not None:
            for plane in pair:
                sc = torch.frombuffer(bytearray(data[off:off + 4 * n]), dtype=torch.float32)
                off += 4 * n
                plane.page_scale.index_copy_(0, idx, sc[first:].to(runner.device))
    kept = 0
    for page, key in zip(pages, keys[first:]):
        kept += int(blocks.commit(page, (int(key[0]), int(key[1]))) == page)
    blocks.release(pages)
    return {"pages": kept, "read": n, "dropped": n - take}


def default_path(state_dir: Optional[str], generation: int = 0) -> str:
    base = state_dir or ("/dev/shm" if os.path.isdir("/dev/shm") else "/tmp")
    return os.path.join(base, f"uniserve-prefix-{os.getpid()}-{generation}.kv")
