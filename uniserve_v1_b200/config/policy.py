"""Policy package: the single TOML tree a deployment is configured by.

A package is a directory with ``config.toml`` (and optionally ``programs/``).
Parsing is strict: an unknown key is refused with its path, durations
(``"30s"``, ``"10m"``, ``"250ms"``) and byte sizes (``"64MiB"``) are typed
literals, and every option declares the *effect* a change of it has
(``step | order | program | generation | storage | epoch | daemon``), which the
admin API uses to decide what can be applied to a running deployment.

Reference behaviour: docs/configuration.md:1-37, :215-229, :270-681, :711-787;
crates/proto/src/config/{mod,block,worker_group}.rs (reference project paths).
The reference's example deployments (configs/qwen3_moe/tp4, configs/afd/qwen3_moe,
configs/minimax_h3/*) parse verbatim.
"""
from __future__ import annotations

import dataclasses
import os
import re
import shutil
import json
import tomllib
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Optional


class ConfigError(ValueError):
    def __init__(self, path: str, message: str):
        super().__init__(f"{path}: {message}")
        self.path = path


# ---------------------------------------------------------------- literals --
_DUR = {"us": 1e-6, "ms": 1e-3, "s": 1.0, "m": 60.0, "h": 3600.0, "d": 86400.0}
_BYTES = {"B": 1, "KB": 10**3, "MB": 10**6, "GB": 10**9, "TB": 10**12,
          "KiB": 2**10, "MiB": 2**20, "GiB": 2**30, "TiB": 2**40}


def parse_duration(v, path="") -> float:
    """Seconds from "250ms" / "30s" / "10m" (a bare number is seconds)."""
    if isinstance(v, (int, float)) and not isinstance(v, bool):
        return float(v)
    m = re.fullmatch(r"\s*([0-9]*\.?[0-9]+)\s*(us|ms|s|m|h|d)\s*", str(v))
    if not m:
        raise ConfigError(path, f"not a duration: {v!r} (expected e.g. \"30s\", \"250ms\")")
    return float(m.group(1)) * _DUR[m.group(2)]


def parse_bytes(v, path="") -> int:
    if isinstance(v, int) and not isinstance(v, bool):
        return v
    m = re.fullmatch(r"\s*([0-9]*\.?[0-9]+)\s*([KMGT]i?B|B)\s*", str(v))
    if not m:
        raise ConfigError(path, f"not a byte size: {v!r} (expected e.g. \"64MiB\")")
    return int(float(m.group(1)) * _BYTES[m.group(2)])


class Duration(float):
    pass


class ByteSize(int):
    pass


# ------------------------------------------------------------------ tables --
def opt(default, effect: str, doc: str = ""):
    return field(default=default, metadata={"effect": effect, "doc": doc})


def optf(factory, effect: str, doc: str = ""):
    return field(default_factory=factory, metadata={"effect": effect, "doc": doc})


@dataclass
class ServerConfig:
    api_key: Optional[str] = opt(None, "daemon", "Bearer token every route but /health requires")
    request_timeout: Optional[Duration] = opt(None, "daemon")
    max_concurrent_requests: Optional[int] = opt(None, "daemon")
    shutdown_timeout: Duration = opt(Duration(30.0), "daemon")
    request_id_headers: bool = opt(False, "daemon")
    max_request_head: ByteSize = opt(ByteSize(64 << 10), "daemon")
    max_request_body: ByteSize = opt(ByteSize(64 << 20), "daemon")
    stream_keep_alive: Duration = opt(Duration(15.0), "daemon")
    max_request_id: int = opt(128, "daemon")
    retry_after: Duration = opt(Duration(1.0), "daemon")


@dataclass
class AdminConfig:
    host: str = opt("127.0.0.1", "daemon")
    port: int = opt(0, "daemon")
    uds: Optional[str] = opt(None, "daemon")
    join: int = opt(29700, "daemon")


@dataclass
class KvCacheConfig:
    max_tokens: Optional[int] = opt(None, "epoch")
    block_size: int = opt(64, "epoch", "tokens per page (16, 32 or 64)")
    dtype: Optional[str] = opt(None, "epoch")
    prefix_caching: bool = opt(True, "step")
    host_tier: bool = opt(True, "step")
    host_ratio: float = opt(2.0, "storage")
    host_gib: Optional[float] = opt(None, "storage")
    mooncake: Optional[dict] = opt(None, "storage")
    boundary_interval: int = opt(64, "epoch")
    state_interval: int = opt(256, "epoch")
    state_ratio: float = opt(1.0, "epoch")
    prefetch_timeout_base: Duration = opt(Duration(1.0), "step")
    prefetch_timeout_per_ki_token: Duration = opt(Duration(0.25), "step")
    lease: Duration = opt(Duration(30.0), "step")


@dataclass
class PolicyBudget:
    call_fuel: int = opt(10_000_000, "program")
    message_fuel_per_byte: int = opt(200, "program")
    max_timeout: Duration = opt(Duration(30.0), "program")
    min_prefetch_tokens: int = opt(256, "program")


@dataclass
class SchedulerConfigTable:
    max_queued_requests: Optional[int] = opt(None, "step")
    chunked_prefill_size: int = opt(8192, "step")
    max_batch: int = opt(128, "step")
    policy_budget: PolicyBudget = optf(PolicyBudget, "program")


@dataclass
class SpeculativeConfig:
    num_draft_tokens: int = opt(0, "generation")
    expected_speedup: Optional[float] = opt(None, "program")
    refill_token_cost: Optional[float] = opt(None, "program")


@dataclass
class MigrationConfig:
    max_migrations: int = opt(3, "daemon")


@dataclass
class Rollback:
    failure_rate: Optional[float] = opt(None, "daemon")
    step_time_regression: Optional[float] = opt(None, "daemon")
    throughput_regression: Optional[float] = opt(None, "daemon")
    window: Optional[Duration] = opt(None, "daemon")


@dataclass
class UpdateConfig:
    trial: Duration = opt(Duration(30.0), "daemon")
    in_flight: str = opt("keep", "daemon")
    previous_epoch: str = opt("parked", "daemon")
    drain_s: float = opt(5.0, "daemon")
    transfer_slowdown: Optional[float] = opt(None, "daemon")
    baseline: float = opt(60.0, "daemon")
    baseline_batches: int = opt(20, "daemon")
    rollback: Rollback = optf(Rollback, "daemon")


@dataclass
class MoeConfig:
    expert_parallel: bool = opt(False, "epoch")
    microbatches: int = opt(1, "epoch", "attention/expert hand-off micro-batches (AFD layout)")
    exchange: Optional[str] = opt(None, "generation", "expert exchange transport")
    expert_order: Optional[list] = opt(None, "step")


@dataclass
class LoadConfig:
    weights: Optional[str] = opt(None, "epoch")


@dataclass
class StorageConfig:
    tcp: Optional[str] = opt(None, "storage")
    host_reserve_gib: float = opt(10.0, "step")
    transfer_calibration: Optional[str] = opt(None, "storage")
    transfer_chunk_us: int = opt(1000, "step")
    transfer_progress_ms: int = opt(100, "step")
    nixl_transports: str = opt("selected", "storage")
    child_restart_s: float = opt(5.0, "step")
    child_restart_max_s: float = opt(300.0, "step")
    transfer_deadline_s: float = opt(60.0, "step")
    put_deadline_s: float = opt(60.0, "step")
    shoot_down_s: float = opt(60.0, "step")
    buffer_pool_trace: Optional[str] = opt(None, "storage")
    directory: Optional[str] = opt(None, "storage")
    directory_period_ms: int = opt(1000, "step")
    handoff_transports: list = optf(lambda: ["nixl"], "step")


@dataclass
class ProfilingSession:
    collectors: list = optf(list, "step")
    duration: Optional[Duration] = opt(None, "step")
    output: Optional[str] = opt(None, "step")


@dataclass
class ProfilingConfig:
    fence_probes: int = opt(2, "generation")
    kernel_probes: bool = opt(False, "generation")
    expert_load: bool = opt(True, "generation")
    pc_sampling: bool = opt(False, "epoch")
    watchdog_timeout: Duration = opt(Duration(150.0), "step")
    standby: bool = opt(False, "daemon", "keep a parked standby process beside the serving one")
    standby_storage: str = opt("auto", "daemon", "resident | suspended | auto")
    standby_snapshot: Duration = opt(Duration(0.0), "daemon",
                                     "period of the prefix-cache snapshots a standby starts from (0: none)")
    session: ProfilingSession = optf(ProfilingSession, "step")


@dataclass
class LoggingConfig:
    level: str = opt("info", "daemon")
    http_level: Optional[str] = opt(None, "daemon")
    format: str = opt("text", "daemon")


@dataclass
class MediaConfig:
    max_request_bytes: ByteSize = opt(ByteSize(256 << 20), "daemon")
    allow_private: bool = opt(False, "daemon", "allow media URLs on private networks")
    directory: Optional[str] = opt(None, "daemon", "the only directory file:// media are read "
                                                   "from; unset refuses file:// URLs")
    fetch_timeout: Duration = opt(Duration(30.0), "daemon")
    max_redirects: int = opt(5, "daemon")
    job_retention: Duration = opt(Duration(3600.0), "daemon")
    job_store_bytes: ByteSize = opt(ByteSize(1 << 30), "daemon")


@dataclass
class ObservationConfig:
    otlp_endpoint: Optional[str] = opt(None, "daemon")
    fine_bucket: Duration = opt(Duration(1.0), "daemon")
    coarse_bucket: Duration = opt(Duration(60.0), "daemon")
    kv_events: Optional[str] = opt(None, "daemon", "ZMQ endpoint for KV events")


@dataclass
class Program:
    source: str = ""
    period: Optional[Duration] = None
    args: dict = field(default_factory=dict)


@dataclass
class SequenceParallel:
    kind: str = "ulysses"               # ulysses | allgather | hybrid
    ulysses_degree: int = 1
    allgather_degree: int = 1
    projection: str = "exchange"        # exchange | gather
    projection_rows: Optional[int] = None


@dataclass
class Block:
    name: str = ""
    ranks: Optional[list] = None
    tensor_parallel_size: int = 1
    pipeline_parallel_size: int = 1
    sequence_parallel: Optional[SequenceParallel] = None
    distribution: Optional[str] = None   # "temporal_units"
    units_per_rank: Optional[int] = None
    weights: Optional[str] = None        # "device" | "host"


@dataclass
class Rank:
    host: Optional[str]
    device: str      # "cuda"
    index: int

    def __str__(self):
        return (f"{self.host}/" if self.host else "") + f"{self.device}:{self.index}"


@dataclass
class WorkerGroup:
    id: str = ""
    role: str = "model"                  # model | experts
    copies: int = 1
    ranks: list = field(default_factory=list)      # expanded Rank list
    queue_depth: int = 2
    mem_fraction_static: Optional[float] = None
    blocks: dict = field(default_factory=dict)


@dataclass
class Replica:
    role: str = "mixed"                  # prefill | decode | mixed


TABLES = {
    "server_config": ServerConfig, "admin_config": AdminConfig, "kv_cache_config": KvCacheConfig,
    "scheduler_config": SchedulerConfigTable, "speculative_config": SpeculativeConfig,
    "migration_config": MigrationConfig, "update_config": UpdateConfig, "moe_config": MoeConfig,
    "load_config": LoadConfig, "storage_config": StorageConfig,
    "profiling_config": ProfilingConfig, "logging_config": LoggingConfig,
    "media_config": MediaConfig, "observation_config": ObservationConfig,
}

TOP_LEVEL = {
    # name: (type, default, effect)
    "model": (str, None, "epoch"), "model_dir": (str, None, "epoch"),
    "served_model_name": (str, None, "step"), "max_model_len": (int, None, "epoch"),
    "lora": (str, None, "epoch"), "lora_dir": (str, None, "epoch"),
    "dtype": (str, "bfloat16", "epoch"), "quantization": (dict, {}, "epoch"),
    "mm_processor_kwargs": (dict, {}, "daemon"), "kernels": (dict, {}, "generation"),
    "max_running_requests": (int, 128, "epoch"), "max_logprobs": (int, 20, "generation"),
    "max_num_batched_tokens": (int, 8192, "program"),
    "mem_fraction_static": (float, 0.7, "epoch"),
    "tensor_parallel_size": (int, 1, "epoch"), "data_parallel_size": (int, 1, "epoch"),
    "pipeline_parallel_size": (int, 1, "epoch"),
    "hosts": (list, [], "epoch"), "engine_host": (str, None, "epoch"),
    "paused": (bool, False, "step"), "asleep": (bool, False, "step"), "flush": (int, 0, "step"),
    "retire": (bool, False, "step"), "adapters": (dict, {}, "step"),
}

_RANK_RE = re.compile(r"^(?:(?P<host>[^/]+)/)?(?P<dev>cuda|cpu):(?P<lo>\d+)(?:-(?P<hi>\d+))?$")


def _toml_value(v) -> str:
    if isinstance(v, bool):
        return "true" if v else "false"
    if isinstance(v, (int, float)):
        return repr(v)
    if isinstance(v, str):
        return json.dumps(v)
    if isinstance(v, (list, tuple)):
        return "[" + ", ".join(_toml_value(x) for x in v) + "]"
    if isinstance(v, dict):
        return "{ " + ", ".join(f"{json.dumps(str(k))} = {_toml_value(x)}" for k, x in v.items()) + " }"
    raise ConfigError("", f"cannot write {type(v).__name__} as TOML")


def dump_toml(data: dict) -> str:
    """Writes a parsed package back as TOML text (scalars and arrays first, then tables;
    tables inside arrays as inline tables)."""
    lines = []

    def emit(table: dict, prefix: str) -> None:
        subs = []
        for k, v in table.items():
            if isinstance(v, dict):
                subs.append((k, v))
            else:
                lines.append(f"{json.dumps(str(k)) if not str(k).replace('_', 'a').replace('-', 'a').isalnum() else k} = {_toml_value(v)}")
        for k, v in subs:
            key = k if str(k).replace("_", "a").replace("-", "a").isalnum() else json.dumps(str(k))
            name = f"{prefix}.{key}" if prefix else key
            lines.append("")
            lines.append(f"[{name}]")
            emit(v, name)
    emit(data, "")
    return "\n".join(lines) + "\n"


def parse_ranks(items, path: str) -> list:
    """``["cuda:0-3"]`` / ``["rank-1/cuda:0-1"]`` -> expanded Rank list."""
    out = []
    if not isinstance(items, list):
        raise ConfigError(path, "expected a list of rank ranges")
    for i, it in enumerate(items):
        m = _RANK_RE.match(str(it))
        if not m:
            raise ConfigError(f"{path}[{i}]", f"not a rank range: {it!r} (e.g. \"cuda:0-3\")")
        lo = int(m["lo"])
        hi = int(m["hi"]) if m["hi"] is not None else lo
        if hi < lo:
            raise ConfigError(f"{path}[{i}]", "descending rank range")
        if m["dev"] == "cpu":
            raise ConfigError(f"{path}[{i}]", "a main process serves CUDA devices only")
        out += [Rank(m["host"], m["dev"], k) for k in range(lo, hi + 1)]
    return out


def _coerce(tp, v, path):
    origin = getattr(tp, "__origin__", None)
    args = getattr(tp, "__args__", ())
    if origin is not None and type(None) in args:          # Optional[T]
        if v is None:
            return None
        inner = [a for a in args if a is not type(None)][0]
        return _coerce(inner, v, path)
    if tp is Duration:
        return Duration(parse_duration(v, path))
    if tp is ByteSize:
        return ByteSize(parse_bytes(v, path))
    if tp is bool:
        if not isinstance(v, bool):
            raise ConfigError(path, f"expected true or false, got {v!r}")
        return v
    if tp is int:
        if isinstance(v, bool) or not isinstance(v, int):
            raise ConfigError(path, f"expected an integer, got {v!r}")
        return v
    if tp is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(path, f"expected a number, got {v!r}")
        return float(v)
    if tp is str:
        if not isinstance(v, str):
            raise ConfigError(path, f"expected a string, got {v!r}")
        return v
    if tp in (list, dict):
        if not isinstance(v, tp):
            raise ConfigError(path, f"expected a {tp.__name__}")
        return v
    if dataclasses.is_dataclass(tp):
        return _parse_table(tp, v, path)
    return v


def _parse_table(cls, data, path):
    if not isinstance(data, dict):
        raise ConfigError(path, "expected a table")
    hints = {f.name: f for f in dataclasses.fields(cls)}
    import typing
    types = typing.get_type_hints(cls)
    kw = {}
    for k, v in data.items():
        if k not in hints:
            raise ConfigError(f"{path}.{k}" if path else k,
                              f"unknown option (known: {', '.join(sorted(hints))})")
        kw[k] = _coerce(types[k], v, f"{path}.{k}" if path else k)
    return cls(**kw)


@dataclass
class Package:
    """A parsed policy package."""
    top: dict = field(default_factory=dict)
    tables: dict = field(default_factory=dict)
    worker_groups: list = field(default_factory=list)
    programs: dict = field(default_factory=dict)
    replicas: dict = field(default_factory=dict)
    source_dir: Optional[Path] = None
    raw: dict = field(default_factory=dict)

    def __getattr__(self, name):
        top = self.__dict__.get("top", {})
        if name in top:
            return top[name]
        tables = self.__dict__.get("tables", {})
        if name in tables:
            return tables[name]
        raise AttributeError(name)

    # ------------------------------------------------------------- changes --
    def with_options(self, changes: dict) -> "Package":
        """A new package with ``{option path: value}`` written over this one's
        (``scheduler_config.chunked_prefill_size``, ``replicas.a.role``, ``kernels.<op>`` ...);
        the result is parsed and validated like a package read from a file."""
        import copy
        data = copy.deepcopy(self.raw)
        for path, value in changes.items():
            node = data
            parts = path.split(".")
            for part in parts[:-1]:
                node = node.setdefault(part, {})
                if not isinstance(node, dict):
                    raise ConfigError(path, "not a table")
            if value is None:
                node.pop(parts[-1], None)
            else:
                node[parts[-1]] = value
        return Package.parse(dump_toml(data), self.source_dir)

    # ---------------------------------------------------------------- load --
    @classmethod
    def parse(cls, text: str, source_dir: Optional[Path] = None) -> "Package":
        try:
            data = tomllib.loads(text)
        except tomllib.TOMLDecodeError as e:
            raise ConfigError("config.toml", str(e))
        pkg = cls(source_dir=source_dir, raw=data)
        for k, (tp, default, _) in TOP_LEVEL.items():
            pkg.top[k] = default if not isinstance(default, (dict, list)) else type(default)(default)
        for name, tcls in TABLES.items():
            pkg.tables[name] = tcls()
        for k, v in data.items():
            if k in TOP_LEVEL:
                pkg.top[k] = _coerce(TOP_LEVEL[k][0], v, k)
            elif k in TABLES:
                pkg.tables[k] = _parse_table(TABLES[k], v, k)
            elif k == "worker_groups":
                pkg.worker_groups = cls._parse_groups(v)
            elif k == "programs":
                for name, p in v.items():
                    prog = _parse_table(Program, {kk: vv for kk, vv in p.items()},
                                        f"programs.{name}")
                    if prog.period is not None:
                        prog.period = Duration(parse_duration(prog.period, f"programs.{name}.period"))
                    pkg.programs[name] = prog
            elif k == "replicas":
                for rid, r in v.items():
                    rep = _parse_table(Replica, r, f"replicas.{rid}")
                    if rep.role not in ("prefill", "decode", "mixed"):
                        raise ConfigError(f"replicas.{rid}.role", f"unknown role {rep.role!r}")
                    pkg.replicas[rid] = rep
            elif k == "quantization_config":
                raise ConfigError(k, "retired option: state it as `quantization`")
            else:
                raise ConfigError(k, "unknown option")
        pkg.validate()
        return pkg

    @classmethod
    def load(cls, path) -> "Package":
        p = Path(path)
        cfg = p / "config.toml" if p.is_dir() else p
        if not cfg.exists():
            raise ConfigError(str(cfg), "policy package has no config.toml")
        return cls.parse(cfg.read_text(), cfg.parent)

    @staticmethod
    def _parse_groups(items) -> list:
        if not isinstance(items, list):
            raise ConfigError("worker_groups", "expected [[worker_groups]] tables")
        groups = []
        for gi, g in enumerate(items):
            path = f"worker_groups[{gi}]"
            known = {"id", "role", "copies", "ranks", "queue_depth", "mem_fraction_static", "blocks"}
            for k in g:
                if k not in known:
                    raise ConfigError(f"{path}.{k}", "unknown option")
            wg = WorkerGroup(id=str(g.get("id", f"group{gi}")), role=g.get("role", "model"),
                             copies=int(g.get("copies", 1)),
                             ranks=parse_ranks(g.get("ranks", []), f"{path}.ranks"),
                             queue_depth=int(g.get("queue_depth", 2)),
                             mem_fraction_static=g.get("mem_fraction_static"))
            if wg.role not in ("model", "experts"):
                raise ConfigError(f"{path}.role", f"unknown role {wg.role!r}")
            if not wg.ranks:
                raise ConfigError(f"{path}.ranks", "a worker group needs ranks")
            for bname, b in (g.get("blocks") or {}).items():
                bpath = f"{path}.blocks.{bname}"
                blk = _parse_table(Block, {k: v for k, v in b.items() if k != "sequence_parallel"},
                                   bpath)
                blk.name = bname
                if "sequence_parallel" in b:
                    sp = _parse_table(SequenceParallel, b["sequence_parallel"],
                                      f"{bpath}.sequence_parallel")
                    if sp.kind not in ("ulysses", "allgather", "hybrid"):
                        raise ConfigError(f"{bpath}.sequence_parallel.kind", f"unknown kind {sp.kind!r}")
                    if sp.projection not in ("exchange", "gather"):
                        raise ConfigError(f"{bpath}.sequence_parallel.projection",
                                          f"unknown projection {sp.projection!r}")
                    blk.sequence_parallel = sp
                if blk.distribution not in (None, "temporal_units"):
                    raise ConfigError(f"{bpath}.distribution", f"unknown distribution {blk.distribution!r}")
                if blk.weights not in (None, "device", "host"):
                    raise ConfigError(f"{bpath}.weights", f"unknown weights placement {blk.weights!r}")
                wg.blocks[bname] = blk
            groups.append(wg)
        ids = [g.id for g in groups]
        if len(set(ids)) != len(ids):
            raise ConfigError("worker_groups", "duplicate group id")
        return groups

    # ------------------------------------------------------------ validate --
    def validate(self) -> None:
        t = self.top
        if t["model"] and t["model_dir"]:
            raise ConfigError("model", "state `model` or `model_dir`, not both")
        if not (0.0 < t["mem_fraction_static"] <= 1.0):
            raise ConfigError("mem_fraction_static", "must be in (0, 1]")
        if t["dtype"] not in ("bfloat16", "float16", "float32"):
            raise ConfigError("dtype", f"unknown dtype {t['dtype']!r}")
        kv = self.tables["kv_cache_config"]
        if kv.block_size not in (16, 32, 64):
            raise ConfigError("kv_cache_config.block_size", "pages of 16, 32 or 64 tokens are served")
        hosts = set(t["hosts"])
        for g in self.worker_groups:
            per = len(g.ranks)
            if per % g.copies:
                raise ConfigError(f"worker_groups.{g.id}.copies", "ranks do not divide into copies")
            per //= g.copies
            for r in g.ranks:
                if r.host and hosts and r.host not in hosts:
                    raise ConfigError(f"worker_groups.{g.id}.ranks", f"host {r.host!r} is not in `hosts`")
            for b in g.blocks.values():
                n = b.tensor_parallel_size * b.pipeline_parallel_size
                if b.sequence_parallel:
                    n *= b.sequence_parallel.ulysses_degree * b.sequence_parallel.allgather_degree
                if b.ranks is None and n > per:
                    raise ConfigError(f"worker_groups.{g.id}.blocks.{b.name}",
                                      f"needs {n} ranks, a copy of the group has {per}")
        if any(g.role == "experts" for g in self.worker_groups) and \
                not self.tables["moe_config"].expert_parallel:
            raise ConfigError("moe_config.expert_parallel", "an experts group needs expert_parallel = true")

    # --------------------------------------------------------------- layout --
    def layout(self) -> dict:
        """Resolved device layout: what each group runs where."""
        if not self.worker_groups:
            tp = self.top["tensor_parallel_size"]
            return {"groups": [{"id": "model", "role": "model", "copies": 1,
                                "ranks": [f"cuda:{i}" for i in range(tp)],
                                "blocks": {"model": {"tensor_parallel_size": tp}}}],
                    "data_parallel_size": self.top["data_parallel_size"]}
        return {"groups": [{"id": g.id, "role": g.role, "copies": g.copies,
                            "ranks": [str(r) for r in g.ranks], "queue_depth": g.queue_depth,
                            "blocks": {n: {k: v for k, v in dataclasses.asdict(b).items()
                                           if v not in (None, "", 1) or k.endswith("size")}
                                       for n, b in g.blocks.items()}}
                           for g in self.worker_groups],
                "data_parallel_size": self.top["data_parallel_size"]}

    # --------------------------------------------------------------- effects --
    def flat(self) -> dict:
        out = dict(self.top)
        for name, tab in self.tables.items():
            for f in dataclasses.fields(tab):
                v = getattr(tab, f.name)
                if dataclasses.is_dataclass(v):
                    for ff in dataclasses.fields(v):
                        out[f"{name}.{f.name}.{ff.name}"] = getattr(v, ff.name)
                else:
                    out[f"{name}.{f.name}"] = v
        out["worker_groups"] = repr(self.layout())
        out["programs"] = repr({k: dataclasses.asdict(v) for k, v in self.programs.items()})
        out["replicas"] = repr({k: dataclasses.asdict(v) for k, v in self.replicas.items()})
        return out

    @staticmethod
    def effect_of(option: str) -> str:
        if option in TOP_LEVEL:
            return TOP_LEVEL[option][2]
        if option in ("worker_groups", "replicas"):
            return "epoch"
        if option == "programs":
            return "program"
        parts = option.split(".")
        cls = TABLES.get(parts[0])
        for p in parts[1:]:
            if cls is None:
                break
            f = {x.name: x for x in dataclasses.fields(cls)}.get(p)
            if f is None:
                break
            eff = f.metadata.get("effect", "epoch")
            import typing
            tp = typing.get_type_hints(cls)[p]
            cls = tp if dataclasses.is_dataclass(tp) else None
            if cls is None:
                return eff
        return "epoch"

    def diff(self, other: "Package") -> list:
        """[(option, old, new, effect)] of what changes from self to other."""
        a, b = self.flat(), other.flat()
        return [(k, a.get(k), b.get(k), self.effect_of(k)) for k in sorted(set(a) | set(b))
                if a.get(k) != b.get(k)]


ORDER = ["step", "order", "program", "generation", "storage", "epoch", "daemon"]


def strongest_effect(changes: list) -> Optional[str]:
    effs = [c[3] for c in changes]
    return max(effs, key=ORDER.index) if effs else None


# ----------------------------------------------------------- revision store --
class RevisionStore:
    """Persisted packages: ``<state>/deployments/<name>/revisions/N`` with a
    ``current`` symlink; the newest 64 are kept (docs/configuration.md:53-68)."""

    KEEP = 64

    def __init__(self, name: str, state_home: Optional[str] = None):
        root = Path(state_home or os.environ.get("XDG_STATE_HOME") or Path.home() / ".local/state")
        self.dir = root / "uniserve" / "deployments" / name / "revisions"
        self.dir.mkdir(parents=True, exist_ok=True)

    def revisions(self) -> list:
        return sorted(int(p.name) for p in self.dir.iterdir() if p.name.isdigit())

    def commit(self, config_text: str) -> int:
        Package.parse(config_text)                 # never store what does not parse
        n = (self.revisions() or [0])[-1] + 1
        d = self.dir / str(n)
        d.mkdir()
        (d / "config.toml").write_text(config_text)
        (d / "lock.toml").write_text(f"revision = {n}\n")
        cur = self.dir / "current"
        tmp = self.dir / ".current.tmp"
        if tmp.is_symlink() or tmp.exists():
            tmp.unlink()
        tmp.symlink_to(str(n))
        tmp.replace(cur)
        for old in self.revisions()[:-self.KEEP]:
            shutil.rmtree(self.dir / str(old), ignore_errors=True)
        return n

    def current(self) -> Optional[Package]:
        cur = self.dir / "current"
        return Package.load(cur) if cur.exists() else None
