"""Profile sessions -> Perfetto / Chrome trace JSON.

    python -m uniserve_v1_b200.tools.profile trace session_rank0.sqlite [more ...] -o trace.json
    python -m uniserve_v1_b200.tools.profile summary session_rank0.sqlite
    python -m uniserve_v1_b200.tools.profile timeline session_rank0.sqlite --limit 100

``trace`` merges the per-rank session files: host spans become complete events
on one track per (rank, thread), fence-probe pairs (``X.begin`` / ``X.end`` with
the same tag) become complete events on a "device" track per rank, counters
become counter events, kernel and copy records of the ``timeline`` collector events on a
track per stream.  ``summary`` prints per-name totals (host spans, device ranges, the heaviest
kernels), ``timeline`` the records of every track in time order as text.

Reference: tools/profile/src/{perfetto,session,timeline}.rs (reference project paths).
"""
from __future__ import annotations

import argparse
import json
import sqlite3
import sys
from collections import defaultdict


def load(path: str) -> dict:
    db = sqlite3.connect(path)
    out = {"spans": db.execute("SELECT rank, thread, name, start_ns, end_ns, step FROM spans")
           .fetchall(),
           "probes": db.execute("SELECT rank, name, timer_ns, sm_clock, tag FROM probes "
                                "ORDER BY timer_ns").fetchall(),
           "counters": db.execute("SELECT rank, name, step, value FROM counters").fetchall(),
           "meta": dict(db.execute("SELECT key, value FROM meta").fetchall())}
    try:        # sessions with the ``timeline`` collector
        out["kernels"] = db.execute("SELECT rank, name, kind, stream, start_ns, dur_ns FROM kernels "
                                    "ORDER BY start_ns").fetchall()
    except sqlite3.OperationalError:
        out["kernels"] = []
    db.close()
    return out


def device_ranges(probes) -> list:
    """Pairs ``X.begin`` / ``X.end`` probes of one rank by (X, tag)."""
    open_, out = {}, []
    for rank, name, t, clk, tag in probes:
        base, _, edge = name.rpartition(".")
        key = (rank, base, tag)
        if edge == "begin":
            open_[key] = (t, clk)
        elif edge == "end" and key in open_:
            t0, c0 = open_.pop(key)
            out.append((rank, base, tag, t0, t, clk - c0))
    return out


def to_trace(sessions: list) -> dict:
    events = []
    for s in sessions:
        for rank, thread, name, t0, t1, step in s["spans"]:
            events.append({"name": name, "ph": "X", "ts": t0 / 1e3, "dur": (t1 - t0) / 1e3,
                           "pid": rank, "tid": f"host:{thread}", "args": {"step": step}})
        for rank, base, tag, t0, t1, cycles in device_ranges(s["probes"]):
            events.append({"name": base, "ph": "X", "ts": t0 / 1e3, "dur": (t1 - t0) / 1e3,
                           "pid": rank, "tid": "device", "args": {"tag": tag, "sm_cycles": cycles}})
        for rank, name, step, value in s["counters"]:
            events.append({"name": name, "ph": "C", "ts": float(step), "pid": rank,
                           "args": {name: value}})
        for rank, name, kind, stream, t0, dur in s.get("kernels", []):
            events.append({"name": name, "ph": "X", "ts": t0 / 1e3, "dur": dur / 1e3, "pid": rank,
                           "tid": f"{kind}s:stream {stream}", "args": {}})
    return {"traceEvents": events, "displayTimeUnit": "ns"}


def summary(sessions: list) -> dict:
    host, dev = defaultdict(lambda: [0, 0.0]), defaultdict(lambda: [0, 0.0])
    for s in sessions:
        for _, _, name, t0, t1, _ in s["spans"]:
            host[name][0] += 1
            host[name][1] += (t1 - t0) / 1e6
        for _, base, _, t0, t1, _ in device_ranges(s["probes"]):
            dev[base][0] += 1
            dev[base][1] += (t1 - t0) / 1e6
    kern = defaultdict(lambda: [0, 0.0])
    for s in sessions:
        for _, name, kind, _, _, dur in s.get("kernels", []):
            key = name if kind != "host_op" else "host:" + name
            kern[key][0] += 1
            kern[key][1] += dur / 1e6
    fmt = lambda d: {k: {"count": c, "total_ms": round(ms, 3), "mean_ms": round(ms / c, 4)}
                     for k, (c, ms) in sorted(d.items())}
    top = dict(sorted(fmt(kern).items(), key=lambda kv: -kv[1]["total_ms"])[:40])
    return {"host_spans": fmt(host), "device_ranges": fmt(dev), "kernels": top}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="uniserve-profile")
    sub = ap.add_subparsers(dest="cmd", required=True)
    t = sub.add_parser("trace")
    t.add_argument("sessions", nargs="+")
    t.add_argument("-o", "--out", required=True)
    s = sub.add_parser("summary")
    s.add_argument("sessions", nargs="+")
    tl = sub.add_parser("timeline", help="records in time order, as text")
    tl.add_argument("sessions", nargs="+")
    tl.add_argument("--limit", type=int, default=200)
    args = ap.parse_args(argv)
    sessions = [load(p) for p in args.sessions]
    if args.cmd == "timeline":
        rows = []
        for ses in sessions:
            for rank, thread, name, t0, t1, step in ses["spans"]:
                rows.append((t0, rank, f"host:{thread}", name, (t1 - t0) / 1e3))
            for rank, base, tag, t0, t1, _ in device_ranges(ses["probes"]):
                rows.append((t0, rank, "device", f"{base} [{tag}]", (t1 - t0) / 1e3))
            for rank, name, kind, stream, t0, dur in ses.get("kernels", []):
                rows.append((t0, rank, f"{kind}:{stream}", name, dur / 1e3))
        # host spans and probes use the host's monotonic / the device's timer, kernel records
        # the profiler's clock: each track is ordered in itself
        rows.sort(key=lambda r: (r[2].split(":")[0], r[0]))
        for t0, rank, track, name, us in rows[:args.limit]:
            print(f"{t0 / 1e6:14.3f} ms  rank {rank}  {track:<18} {us:10.1f} us  {name[:90]}")
        if len(rows) > args.limit:
            print(f"... {len(rows) - args.limit} more")
        return 0
    if args.cmd == "trace":
        with open(args.out, "w") as f:
            json.dump(to_trace(sessions), f)
        print(f"{args.out}: {sum(len(x['spans']) + len(x['probes']) + len(x.get('kernels', [])) for x in sessions)} records")
    else:
        print(json.dumps(summary(sessions), indent=1))
    return 0


if __name__ == "__main__":
    sys.exit(main())
