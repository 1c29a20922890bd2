# role: plans the replicas' roles in place.
# readings: {"ttft_p99": s, "tpot_p99": s, "running": {replica: n}, "roles": {replica: role}}
# ARGS: ttft, tpot, room 0.2, interval 300, keep 1, pause
STATE = {"held_until": 0.0, "last_change": -1e18}


def step(readings, now):
    if now < STATE["held_until"] or now - STATE["last_change"] < float(ARGS.get("interval", 300.0)):
        return {}
    ttft, tpot = readings.get("ttft_p99"), readings.get("tpot_p99")
    if ttft is None or tpot is None:
        return {}
    room, keep = float(ARGS.get("room", 0.2)), int(ARGS.get("keep", 1))
    roles, running = readings.get("roles", {}), readings.get("running", {})
    pre = sorted(r for r, v in roles.items() if v == "prefill")
    dec = sorted(r for r, v in roles.items() if v == "decode")
    fewest = lambda rs: min(rs, key=lambda r: (running.get(r, 0), r))
    if ttft > float(ARGS["ttft"]) and tpot < (1 - room) * float(ARGS["tpot"]) and len(dec) > keep:
        STATE["last_change"] = now
        return {"replicas." + fewest(dec) + ".role": "prefill"}
    if tpot > float(ARGS["tpot"]) and ttft < (1 - room) * float(ARGS["ttft"]) and len(pre) > keep:
        STATE["last_change"] = now
        return {"replicas." + fewest(pre) + ".role": "decode"}
    return {}


def rolled_back(now):
    STATE["held_until"] = now + float(ARGS.get("pause", 3600.0))


def save_state():
    return dict(STATE)


def restore_state(state):
    for k in STATE:
        if k in state:
            STATE[k] = float(state[k])
