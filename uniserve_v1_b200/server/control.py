"""Control programs: periodic programs that read the observation store and write options.

A package's ``[programs.<name>]`` with a ``period`` is a control program: every period the
host gathers the *readings* the program's kind needs from the observation store (p99 of
``uniserve_ttft_seconds`` / ``uniserve_tpot_seconds`` by replica, tokens per expert, the
decode step's median device time, ...), calls ``step(readings, now)`` in the metered
program host and applies the returned ``{option path: value}`` as one configuration change
through the same path as ``PUT /admin/policy``.  A change that is refused or rolled back
calls the program's ``rolled_back(now)`` (it then holds back for its ``pause``); a program
that faults or runs past its fuel is ended and the configuration stays as it is.  Program
state (``save_state`` / ``restore_state``) is kept across restarts under the deployment's
``program-state/<name>.state``.

Reference behaviour: docs/configuration.md:100-215 (programs, readings, effects),
crates/daemon/src/programs/{host,control}.rs (reference project paths).
"""
from __future__ import annotations

import json
import time
from pathlib import Path
from typing import Callable, Optional

from ..engine.program import ProgramHost
from ..programs import NAMES, source_of

_UNITS = {"ms": 1e-3, "s": 1.0, "m": 60.0, "h": 3600.0}


def seconds(v, default: float) -> float:
    """``"10s"`` / ``"15m"`` / ``"50ms"`` / a number -> seconds."""
    if v is None:
        return default
    if isinstance(v, (int, float)):
        return float(v)
    s = str(v).strip()
    for unit in ("ms", "s", "m", "h"):
        if s.endswith(unit) and s[:-len(unit)].replace(".", "", 1).isdigit():
            return float(s[:-len(unit)]) * _UNITS[unit]
    return float(s)


_DURATION_ARGS = ("tpot", "ttft", "window", "pause", "baseline", "probe", "interval", "rate_span")


def load_program(package, name: str) -> ProgramHost:
    """A package's program: ``uniserve:<name>`` resolves to the released source, anything
    else to a file of the package.  Duration arguments arrive in seconds."""
    prog = package.programs[name]
    args = dict(prog.args or {})
    for k in _DURATION_ARGS:
        if k in args:
            args[k] = seconds(args[k], 0.0)
    budget = package.scheduler_config.policy_budget.call_fuel
    if str(prog.source).startswith("uniserve:"):
        return ProgramHost(source_of(prog.source), name, budget, args)
    path = Path(prog.source)
    if not path.is_absolute() and package.source_dir is not None:
        path = Path(package.source_dir) / prog.source
    return ProgramHost(path.read_text(), name, budget, args)


def _quantile(values: list, q: float) -> Optional[float]:
    if not values:
        return None
    s = sorted(values)
    return s[min(len(s) - 1, int(q * len(s)))]


class Readings:
    """What the released control programs read, computed from the observation store."""

    def __init__(self, obs, package_ref: Callable[[], object]):
        self.obs, self.package = obs, package_ref

    def _stat(self, name: str, since: float) -> list:
        rows = self.obs.query(f"select labels, value from stats where name = '{name}' and "
                              f"ts >= {since!r}")["rows"]
        return [(json.loads(l or "{}"), v) for l, v in rows]

    def quantile_by(self, name: str, label: str, q: float, window: float, now: float) -> dict:
        by: dict = {}
        for labels, v in self._stat(name, now - window):
            by.setdefault(labels.get(label, ""), []).append(v)
        return {k: _quantile(v, q) for k, v in by.items()}

    def flat_config(self) -> dict:
        pkg = self.package()
        out = {}
        for table, obj in pkg.tables.items():
            for k, v in vars(obj).items():
                out[f"{table}.{k}"] = v if isinstance(v, (int, float, str, bool, list, type(None))) \
                    else str(v)
        out.update({k: v for k, v in pkg.top.items()
                    if isinstance(v, (int, float, str, bool, type(None)))})
        return out

    def for_program(self, kind: str, args: dict, now: float) -> dict:
        pkg = self.package()
        w = float(args.get("window", 10.0) or 10.0)
        if kind == "chunk":
            return {"ttft_p99": self.quantile_by("uniserve_ttft_seconds", "replica", 0.99, w, now),
                    "tpot_p99": self.quantile_by("uniserve_tpot_seconds", "replica", 0.99, w, now),
                    "chunk": pkg.scheduler_config.chunked_prefill_size,
                    "max_num_batched_tokens": pkg.max_num_batched_tokens}
        if kind == "expert_order":
            tokens: dict = {}
            for labels, v in self._stat("uniserve_expert_tokens_total", now - w):
                row = tokens.setdefault(str(labels.get("layer", "0")), {})
                e = int(labels.get("expert", 0))
                row[e] = max(row.get(e, 0.0), v)
            return {"tokens": {l: [row.get(e, 0.0) for e in range(max(row) + 1)]
                               for l, row in tokens.items() if row},
                    "order": dict(pkg.moe_config.expert_order or {})
                    if isinstance(pkg.moe_config.expert_order, dict) else {}}
        if kind == "role":
            def whole(name):
                vals = [v for _, v in self._stat(name, now - w)]
                return _quantile(vals, 0.99)
            run = {}
            for labels, v in self._stat("uniserve_scheduler_running_requests", now - w):
                run[labels.get("replica", "")] = v
            return {"ttft_p99": whole("uniserve_ttft_seconds"),
                    "tpot_p99": whole("uniserve_tpot_seconds"), "running": run,
                    "roles": {k: r.role for k, r in pkg.replicas.items()}}
        if kind == "layout":
            run = [v for _, v in self._stat("uniserve_scheduler_running_requests", now - w)]
            span = float(args.get("rate_span", 60.0) or 60.0)
            toks = [v for _, v in self._stat("uniserve_generation_tokens_total", now - span)]
            rate = (max(toks) - min(toks)) / span if len(toks) > 1 else 0.0
            return {"running_mean": sum(run) / len(run) if run else 0.0, "token_rate": rate,
                    "config": self.flat_config(), "served_window": len(run) > 0}
        if kind == "backend":
            def p50(span):
                vals = [v for l, v in self._stat("uniserve_step_device_seconds", now - span)
                        if l.get("phase") == "decode"]
                return _quantile(vals, 0.5)
            return {"decode_p50_window": p50(w),
                    "decode_p50_baseline": p50(float(args.get("baseline", 3600.0) or 3600.0)),
                    "config": self.flat_config(), "probe": None}
        return {}


class ControlLoop:
    """Runs a package's control programs.  ``apply(changes) -> bool`` applies one change set
    (False: refused or rolled back)."""

    def __init__(self, package_ref: Callable[[], object], obs, apply: Callable[[dict], bool],
                 state_dir: Optional[str] = None, clock: Callable[[], float] = time.time):
        self.package, self.obs, self.apply, self.clock = package_ref, obs, apply, clock
        self.readings = Readings(obs, package_ref)
        self.state_dir = Path(state_dir) if state_dir else None
        self.hosts: dict = {}
        self.next_run: dict = {}
        self.ended: dict = {}
        self.applied: list = []
        pkg = package_ref()
        for name, prog in pkg.programs.items():
            kind = str(prog.source).split(":", 1)[-1].replace("-", "_")
            if prog.period is None or name in ("scheduling", "routing"):
                continue
            try:
                host = load_program(pkg, name)
            except Exception as e:
                self.ended[name] = f"load: {e}"
                continue
            if not host.has("step"):
                continue
            host.kind = kind if kind in NAMES else name.replace("-", "_")
            self._restore(name, host)
            self.hosts[name] = host
            self.next_run[name] = self.clock() + seconds(prog.period, 10.0)

    def _state_path(self, name: str) -> Optional[Path]:
        return self.state_dir / f"{name}.state" if self.state_dir else None

    def _restore(self, name: str, host: ProgramHost) -> None:
        p = self._state_path(name)
        if p is not None and p.exists():
            try:
                saved = json.loads(p.read_text())
                if saved.get("args") == host.ns["ARGS"]:
                    host.restore_state(json.dumps(saved.get("state")))
            except Exception:
                pass

    def _save(self, name: str, host: ProgramHost) -> None:
        p = self._state_path(name)
        if p is None:
            return
        try:
            p.parent.mkdir(parents=True, exist_ok=True)
            p.write_text(json.dumps({"args": host.ns["ARGS"],
                                     "state": json.loads(host.save_state())}))
        except Exception:
            pass

    def tick(self) -> list:
        """Runs every program whose period has passed; returns the change sets applied."""
        now = self.clock()
        done = []
        pkg = self.package()
        for name, host in list(self.hosts.items()):
            if now < self.next_run[name]:
                continue
            self.next_run[name] = now + seconds(pkg.programs[name].period, 10.0)
            try:
                readings = self.readings.for_program(host.kind, host.ns["ARGS"], now)
                change = host.call("step", readings, now)
            except Exception as e:           # fault or fuel: the program is ended
                self.ended[name] = str(e)
                del self.hosts[name]
                self.obs.event("log", "", writer=name, level="error", message=f"ended: {e}")
                continue
            if change:
                if not isinstance(change, dict):
                    self.obs.event("log", "", writer=name, level="error",
                                   message="refused output: not a table of options")
                elif self.apply(dict(change)):
                    done.append((name, change))
                    self.applied.append((now, name, change))
                    self.obs.event("revision", "", writer=name, changes=sorted(change))
                elif host.has("rolled_back"):
                    try:
                        host.call("rolled_back", now)
                    except Exception:
                        pass
            self._save(name, host)
        return done
