# backend: deepens observation when the decode step slows and moves the attention kernels to
# the faster backend.
# readings: {"decode_p50_window": s, "decode_p50_baseline": s, "config": {...},
#            "probe": None | {"modules": {class: p50 s}, "keys": [descriptor], "backend": name}}
# ARGS: slowdown 0.1, probe 30, interval 600, modules ["*"], attention ["*.Attention"],
#       op "paged_attention", backends [...], margin 0.05, weight 0.3, pause
STATE = {"held_until": 0.0, "probe_until": None, "last_probe": -1e18, "saved": None,
         "class_records": {}, "backend_records": {}}


def _match(pattern, name):
    if pattern == "*":
        return True
    if pattern.startswith("*"):
        return name.endswith(pattern[1:])
    return name == pattern


def step(readings, now):
    slow = float(ARGS.get("slowdown", 0.1))
    if STATE["probe_until"] is None:
        w, b = readings.get("decode_p50_window"), readings.get("decode_p50_baseline")
        if now < STATE["held_until"] or w is None or b is None or b <= 0:
            return {}
        if w > b * (1 + slow) and now - STATE["last_probe"] >= float(ARGS.get("interval", 600.0)):
            cfg = readings.get("config", {})
            STATE["saved"] = {k: cfg.get(k) for k in ("profiling_config.fence_modules",
                                                      "profiling_config.fence_probes",
                                                      "profiling_config.fence_probes_off")}
            STATE["probe_until"] = now + float(ARGS.get("probe", 30.0))
            STATE["last_probe"] = now
            return {"profiling_config.fence_modules": list(ARGS.get("modules", ["*"])),
                    "profiling_config.fence_probes": True,
                    "profiling_config.fence_probes_off": []}
        return {}
    if now < STATE["probe_until"]:
        return {}
    # the probe ends: its options go back (never held back), and what it measured is read
    change = dict(STATE["saved"] or {})
    STATE["probe_until"], STATE["saved"] = None, None
    probe = readings.get("probe") or {}
    w = float(ARGS.get("weight", 0.3))
    slowed = []
    attn_time = 0.0
    for cls, t in (probe.get("modules") or {}).items():
        rec = STATE["class_records"].get(cls)
        if rec is not None and t > rec * (1 + slow):
            slowed.append(cls)
        STATE["class_records"][cls] = t if rec is None else (1 - w) * rec + w * t
        if any(_match(p, cls) for p in ARGS.get("attention", ["*.Attention"])):
            attn_time += t
    backends = list(ARGS.get("backends", ["tcgen05", "simt"]))
    on = probe.get("backend") or backends[0]
    if attn_time > 0:
        rec = STATE["backend_records"].get(on)
        STATE["backend_records"][on] = attn_time if rec is None else (1 - w) * rec + w * attn_time
    if on in backends and backends.index(on) + 1 < len(backends):
        nxt = backends[backends.index(on) + 1]
        rec = STATE["backend_records"].get(nxt)
        attn_slowed = any(any(_match(p, c) for p in ARGS.get("attention", ["*.Attention"]))
                          for c in slowed)
        faster = rec is not None and rec < attn_time * (1 - float(ARGS.get("margin", 0.05)))
        if faster or (rec is None and attn_slowed):
            pins = {key: nxt + "@latest" for key in probe.get("keys", [])}
            if pins:
                change["kernels." + ARGS.get("op", "paged_attention")] = pins
    return change


def rolled_back(now):
    STATE["held_until"] = now + float(ARGS.get("pause", 3600.0))


def save_state():
    return dict(STATE)


def restore_state(state):
    for k in STATE:
        if k in state:
            STATE[k] = state[k]
