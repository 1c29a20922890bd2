"""Plain-data request types shared by the scheduler, the runner and the API layer.

Field names follow the reference's ``SamplingParams`` and error taxonomy
(crates/proto/src/request/sampling.rs:20-64, crates/engine/src/batch.rs:264-309,
reference project paths).
"""
from __future__ import annotations

import enum
import time
from dataclasses import dataclass, field
from typing import Optional


@dataclass
class SamplingParams:
    temperature: float = 1.0
    top_k: int = 0                  # 0 / negative = whole row
    top_p: float = 1.0
    min_p: float = 0.0
    repetition_penalty: float = 1.0
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    logit_bias: Optional[dict] = None          # token id -> bias
    allowed_token_ids: Optional[list] = None
    bad_words_ids: Optional[list] = None       # list of single-token bans / sequences
    min_tokens: int = 0
    max_tokens: int = 16
    ignore_eos: bool = False
    seed: Optional[int] = None
    stop_token_ids: tuple = ()
    logprobs: bool = False
    top_logprobs: int = 0
    forced_token_ids: Optional[list] = None

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0 or self.top_k == 1

    @property
    def needs_shaping(self) -> bool:
        return (self.repetition_penalty != 1.0 or self.frequency_penalty != 0.0
                or self.presence_penalty != 0.0 or bool(self.logit_bias)
                or bool(self.allowed_token_ids) or bool(self.bad_words_ids)
                or self.min_tokens > 0)


class RequestState(enum.Enum):
    WAITING = "waiting"
    RUNNING = "running"
    PREEMPTED = "preempted"
    FINISHED = "finished"


class FinishReason(enum.Enum):
    STOP = "stop"
    LENGTH = "length"
    ABORT = "abort"
    ERROR = "error"


class ErrorClass(enum.Enum):
    """input_error rejects the request; numerical_fault fails rows;
    invariant_violation / fatal_worker_failure stop the engine."""
    INPUT_ERROR = "input_error"
    NUMERICAL_FAULT = "numerical_fault"
    INVARIANT_VIOLATION = "invariant_violation"
    FATAL_WORKER_FAILURE = "fatal_worker_failure"


@dataclass(eq=False)      # requests are compared and hashed by identity
class Request:
    request_id: str
    prompt_ids: list
    params: SamplingParams
    arrival: float = field(default_factory=time.monotonic)
    priority: int = 0
    cache_salt: Optional[str] = None
    state: RequestState = RequestState.WAITING
    output_ids: list = field(default_factory=list)
    logprobs: list = field(default_factory=list)     # per output token: (logprob, rank, top list)
    num_computed: int = 0        # tokens whose K/V are in the cache
    num_cached: int = 0          # prompt tokens served from the prefix cache
    pages: list = field(default_factory=list)
    slot: int = -1               # device slot row while running
    finish_reason: Optional[FinishReason] = None
    error: Optional[str] = None
    first_token_time: Optional[float] = None
    finish_time: Optional[float] = None
    migrations: int = 0
    preemptions: int = 0
    committed_pages: int = 0

    @property
    def seed(self) -> int:
        """Lineage seed: the request's own seed or a hash of its id."""
        if self.params.seed is not None:
            return self.params.seed & 0xFFFFFFFFFFFFFFFF
        import zlib
        return zlib.crc32(self.request_id.encode()) | (len(self.prompt_ids) << 32)

    @property
    def all_ids(self) -> list:
        return self.prompt_ids + self.output_ids

    @property
    def num_tokens(self) -> int:
        return len(self.prompt_ids) + len(self.output_ids)

    def token_slice(self, lo: int, hi: int) -> list:
        """Tokens [lo, hi) of prompt + outputs without building the whole list."""
        n = len(self.prompt_ids)
        if hi <= n:
            return self.prompt_ids[lo:hi]
        if lo >= n:
            return self.output_ids[lo - n:hi - n]
        return self.prompt_ids[lo:] + self.output_ids[:hi - n]

    @property
    def finished(self) -> bool:
        return self.state == RequestState.FINISHED

    def migratable_facts(self) -> dict:
        """(prompt, generated tokens, seed): enough to resume anywhere
        (crates/daemon/src/migration.rs:12-25, reference path)."""
        return {"request_id": self.request_id, "prompt_ids": list(self.prompt_ids),
                "output_ids": list(self.output_ids), "seed": self.seed,
                "params": self.params, "migrations": self.migrations}


@dataclass
class StepOutput:
    request_id: str
    new_token_ids: list
    finished: bool
    finish_reason: Optional[FinishReason] = None
    logprobs: Optional[list] = None
    num_cached_tokens: int = 0
    error: Optional[str] = None
    handoff: Optional[bytes] = None      # the request left this engine: its framed state
