"""Speculative decoding: drafters and the acceptance rule.

A drafter proposes up to ``k`` next tokens for a decoding request; the target
model verifies them in one call over ``k + 1`` positions (the last accepted token
plus the drafts) and keeps the longest prefix it agrees with plus one token of
its own, so the output is exactly what step-by-step decoding produces while a
step can advance several tokens.  Verification batches run eagerly (variable
row counts), as in the reference; rejected positions leave stale KV entries
behind ``num_computed`` that the next call overwrites.

``NgramDrafter`` needs no extra weights: it continues the most recent earlier
occurrence of the context's last ``n`` tokens (prompt-lookup drafting).  The
multi-token-prediction head (``models/qwen3_mtp.py``) is a drafter with state
(``needs_hidden``): the engine calls ``propose_for(request)`` and hands it the target's
hidden states of the verified positions through ``observe``.

Reference behaviour: docs/configuration.md:418-431,
crates/engine/src/runner/causal_lm/speculation.rs (reference project paths).
"""
from __future__ import annotations

from typing import Sequence


class Drafter:
    k: int = 4

    def propose(self, token_ids: Sequence[int]) -> list:
        raise NotImplementedError


class NgramDrafter(Drafter):
    def __init__(self, n: int = 3, k: int = 4, window: int = 4096):
        self.n, self.k, self.window = n, k, window

    def propose(self, token_ids: Sequence[int]) -> list:
        ids = list(token_ids[-self.window:])
        for n in range(min(self.n, len(ids) - 1), 0, -1):
            tail = ids[-n:]
            for start in range(len(ids) - n - 1, -1, -1):      # most recent match first
                if ids[start:start + n] == tail:
                    cont = ids[start + n:start + n + self.k]
                    if cont:
                        return cont
        return []


def accept(drafts: Sequence[int], target: Sequence[int]) -> list:
    """Greedy acceptance: ``target[i]`` is the model's token after the context extended by
    ``drafts[:i]``.  Returns the tokens to emit: the agreed drafts, then one model token."""
    out = []
    for i, d in enumerate(drafts):
        if int(d) != int(target[i]):
            break
        out.append(int(d))
    out.append(int(target[len(out)]))
    return out
