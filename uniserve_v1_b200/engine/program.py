"""Scheduling programs: user code that makes the scheduler's decisions under a budget.

A policy package may carry ``programs/<name>.py`` and name it in ``[programs.<name>]``.
The program defines any of the six decisions - ``init(config)``, ``observe(event,
request, facts)``, ``dispatch(waiting, room)``, ``preempt(running)``, ``place(request,
groups)``, ``limits()`` - as plain functions over read-only request facts (dicts), plus
optionally ``save_state()`` / ``restore_state(state)`` returning / taking JSON values so
that what it learned survives an engine restart.

The host (``ProgramHost``) runs the source in its own namespace with a small set of
builtins and meters every call: each executed line of the program costs one unit of
fuel, and a call that exceeds ``scheduler_config.policy_budget.call_fuel`` is cut
(``FuelExhausted``).  ``ProgramPolicy`` adapts a host to the scheduler's ``Policy``
interface: a decision the program does not define, cuts short, or answers with
something malformed falls back to the default ``arrival`` decision and is counted in
``faults``, so a bad program degrades scheduling order, never the engine.

Reference behaviour: crates/program/src/lib.rs:1-36 (wasmtime host, fuel budgets,
save / restore), crates/scheduling (the six decisions), docs/configuration.md
(``policy_budget``) - reference project paths.  The sandbox here is a metered Python
namespace, not a WebAssembly machine.
"""
from __future__ import annotations

import json
import sys
from pathlib import Path
from typing import Optional

from .scheduler import Policy
from .types import Request


class FuelExhausted(RuntimeError):
    pass


_BUILTINS = {n: __builtins__[n] if isinstance(__builtins__, dict) else getattr(__builtins__, n)
             for n in ("abs", "all", "any", "bool", "dict", "enumerate", "filter", "float", "int",
                       "len", "list", "map", "max", "min", "range", "reversed", "round", "set",
                       "sorted", "str", "sum", "tuple", "zip", "isinstance", "ValueError",
                       "KeyError", "Exception", "True", "False", "None")
             if (n in __builtins__ if isinstance(__builtins__, dict) else hasattr(__builtins__, n))}


class ProgramHost:
    def __init__(self, source: str, name: str = "program", call_fuel: int = 10_000_000,
                 args: Optional[dict] = None):
        self.name, self.call_fuel = name, int(call_fuel)
        self.fuel_used = 0
        self.calls = 0
        self.ns = {"__builtins__": dict(_BUILTINS), "ARGS": dict(args or {})}
        self.filename = f"<program {name}>"
        self._metered(lambda: exec(compile(source, self.filename, "exec"), self.ns))

    @classmethod
    def load(cls, package, name: str) -> "ProgramHost":
        prog = package.programs[name]
        path = Path(prog.source)
        if not path.is_absolute() and package.source_dir is not None:
            path = Path(package.source_dir) / prog.source
        budget = package.scheduler_config.policy_budget.call_fuel
        return cls(path.read_text(), name, budget, prog.args)

    def has(self, fn: str) -> bool:
        return callable(self.ns.get(fn))

    def _metered(self, thunk):
        left = [self.call_fuel]
        fname = self.filename

        def tracer(frame, event, arg):
            if frame.f_code.co_filename != fname:
                return None
            if event == "line":
                left[0] -= 1
                if left[0] < 0:
                    raise FuelExhausted(f"{self.name}: call budget of {self.call_fuel} spent")
            return tracer
        old = sys.gettrace()
        sys.settrace(tracer)
        try:
            return thunk()
        finally:
            sys.settrace(old)
            self.fuel_used += self.call_fuel - max(left[0], 0)
            self.calls += 1

    def call(self, fn: str, *args):
        f = self.ns[fn]
        return self._metered(lambda: f(*args))

    # state that outlives the engine
    def save_state(self) -> str:
        return json.dumps(self.call("save_state") if self.has("save_state") else None)

    def restore_state(self, blob: str) -> None:
        state = json.loads(blob)
        if state is not None and self.has("restore_state"):
            self.call("restore_state", state)


def _facts(r: Request) -> dict:
    return {"id": r.request_id, "prompt_tokens": len(r.prompt_ids),
            "output_tokens": len(r.output_ids), "priority": r.priority, "arrival": r.arrival,
            "max_tokens": r.params.max_tokens, "computed": r.num_computed,
            "preemptions": r.preemptions}


class ProgramPolicy(Policy):
    """The scheduler's policy object backed by a program; see the module docstring."""

    def __init__(self, host: ProgramHost):
        self.host = host
        self.name = host.name
        self.faults = 0

    def _try(self, fn: str, default, *args):
        if not self.host.has(fn):
            return default
        try:
            return self.host.call(fn, *args)
        except Exception:                     # FuelExhausted included
            self.faults += 1
            return default

    def init(self, config) -> None:
        self.config = config
        self._try("init", None, {"max_num_seqs": config.max_num_seqs,
                                 "max_num_batched_tokens": config.max_num_batched_tokens,
                                 "page_size": config.page_size,
                                 "max_model_len": config.max_model_len})

    def observe(self, event: str, request: Optional[Request] = None, **facts) -> None:
        self._try("observe", None, event, _facts(request) if request is not None else None, facts)

    def dispatch(self, waiting: list, room: dict) -> list:
        default = super().dispatch(waiting, room)
        order = self._try("dispatch", None, [_facts(r) for r in waiting], dict(room))
        if order is None:
            return default
        by_id = {r.request_id: r for r in waiting}
        try:
            picked = [by_id[i] for i in order]
        except (KeyError, TypeError):
            self.faults += 1
            return default
        if len(set(id(r) for r in picked)) != len(picked):
            self.faults += 1
            return default
        return picked                          # a subset defers the rest to a later step

    def preempt(self, running: list) -> Optional[Request]:
        default = super().preempt(running)
        rid = self._try("preempt", None, [_facts(r) for r in running])
        return next((r for r in running if r.request_id == rid), default)

    def place(self, request: Request, groups: list) -> int:
        g = self._try("place", 0, _facts(request), list(groups))
        return g if isinstance(g, int) and 0 <= g < max(1, len(groups)) else 0

    def limits(self) -> dict:
        lim = self._try("limits", {})
        return lim if isinstance(lim, dict) else {}
