"""Tokenizers and incremental detokenisation.

``HFTokenizer`` wraps a Hugging Face ``tokenizer.json`` (the ``tokenizers``
library); ``ByteTokenizer`` serves random-init models that ship no tokenizer
files (byte b <-> id b + 3).  ``IncrementalDecoder`` emits only text that can no
longer change: it decodes a short window of recent ids and holds back output
while the tail is an incomplete UTF-8 sequence (stable-prefix decode).

Reference behaviour: crates/daemon/src/api/tokenizer/{hf,incremental}.rs
(reference project paths).
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Optional


class ByteTokenizer:
    """UTF-8 bytes shifted past three specials: 0 pad, 1 bos, 2 eos."""

    def __init__(self, vocab_size: int = 259, eos_token_id: int = 2):
        self.vocab_size = max(vocab_size, 259)
        self.eos_token_id = eos_token_id
        self.bos_token_id = 1
        self.chat_template = None
        self.specials = {"<|im_start|>": None, "<|im_end|>": None}

    def encode(self, text: str, add_special_tokens: bool = False) -> list:
        return [b + 3 for b in text.encode("utf-8")]

    def decode(self, ids, skip_special_tokens: bool = True) -> str:
        return bytes((i - 3) & 0xFF for i in ids if 3 <= i < 259).decode("utf-8", errors="replace")

    def id_to_token(self, i: int) -> str:
        return self.decode([i])


class HFTokenizer:
    def __init__(self, directory):
        from tokenizers import Tokenizer
        d = Path(directory)
        self.tk = Tokenizer.from_file(str(d / "tokenizer.json"))
        self.vocab_size = self.tk.get_vocab_size()
        cfg = {}
        if (d / "tokenizer_config.json").exists():
            cfg = json.loads((d / "tokenizer_config.json").read_text())
        self.chat_template = cfg.get("chat_template")
        if self.chat_template is None and (d / "chat_template.jinja").exists():
            self.chat_template = (d / "chat_template.jinja").read_text()
        eos = cfg.get("eos_token")
        if isinstance(eos, dict):
            eos = eos.get("content")
        self.eos_token = eos
        self.eos_token_id = self.tk.token_to_id(eos) if eos else None
        bos = cfg.get("bos_token")
        if isinstance(bos, dict):
            bos = bos.get("content")
        self.bos_token = bos
        self.bos_token_id = self.tk.token_to_id(bos) if bos else None
        gen = d / "generation_config.json"
        self.generation_config = json.loads(gen.read_text()) if gen.exists() else {}

    def encode(self, text: str, add_special_tokens: bool = False) -> list:
        return self.tk.encode(text, add_special_tokens=add_special_tokens).ids

    def decode(self, ids, skip_special_tokens: bool = True) -> str:
        return self.tk.decode(list(ids), skip_special_tokens=skip_special_tokens)

    def id_to_token(self, i: int) -> str:
        return self.tk.id_to_token(i) or ""


def load_tokenizer(directory: Optional[str], vocab_size: int, eos_token_id: Optional[int]):
    if directory and (Path(directory) / "tokenizer.json").exists():
        return HFTokenizer(directory)
    return ByteTokenizer(vocab_size, eos_token_id if eos_token_id is not None else 2)


class IncrementalDecoder:
    """Stable-prefix incremental decode of one request's output ids."""

    WINDOW = 6

    def __init__(self, tokenizer, skip_special_tokens: bool = True):
        self.tk = tokenizer
        self.skip = skip_special_tokens
        self.ids: list = []
        self.prefix_offset = 0     # ids[prefix_offset:read_offset] decode to already-emitted text
        self.read_offset = 0

    def push(self, new_ids) -> str:
        self.ids.extend(new_ids)
        prefix = self.tk.decode(self.ids[self.prefix_offset:self.read_offset], self.skip)
        full = self.tk.decode(self.ids[self.prefix_offset:], self.skip)
        if len(full) > len(prefix) and not full.endswith("\ufffd"):
            out = full[len(prefix):]
            self.prefix_offset = max(self.read_offset - self.WINDOW, self.prefix_offset) \
                if self.read_offset else 0
            self.prefix_offset = max(0, len(self.ids) - self.WINDOW)
            self.read_offset = len(self.ids)
            return out
        return ""

    def flush(self) -> str:
        prefix = self.tk.decode(self.ids[self.prefix_offset:self.read_offset], self.skip)
        full = self.tk.decode(self.ids[self.prefix_offset:], self.skip)
        self.read_offset = len(self.ids)
        return full[len(prefix):] if len(full) > len(prefix) else ""
