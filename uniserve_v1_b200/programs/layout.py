# layout: chooses the parallel layout by concurrency among the layouts its arguments name.
# readings: {"running_mean": x, "token_rate": tokens/s, "config": {option path: value},
#            "served_window": bool (the serving layout served a whole window)}
# ARGS: layouts {name: {path: value}}, bounds [..], margin 0.05, samples 3, weight 0.2, pause
STATE = {"held_until": 0.0, "records": {}}      # records[name][range] = [mean rate, samples]


def _serving(config):
    for name, options in ARGS["layouts"].items():
        if all(config.get(path) == value for path, value in options.items()):
            return name
    return None


def _range_of(running):
    i = 0
    for b in ARGS["bounds"]:
        if running >= b:
            i += 1
    return str(i)


def step(readings, now):
    cur = _serving(readings.get("config", {}))
    if cur is None or now < STATE["held_until"]:
        return {}
    rng = _range_of(readings.get("running_mean", 0.0))
    w = float(ARGS.get("weight", 0.2))
    if readings.get("served_window"):
        rec = STATE["records"].setdefault(cur, {}).setdefault(rng, [0.0, 0])
        rate = float(readings.get("token_rate", 0.0))
        rec[0] = rate if rec[1] == 0 else (1 - w) * rec[0] + w * rate
        rec[1] += 1
    mine = STATE["records"].get(cur, {}).get(rng)
    if not mine or mine[1] < int(ARGS.get("samples", 3)):
        return {}
    best, best_rate = None, mine[0] * (1 + float(ARGS.get("margin", 0.05)))
    for name in ARGS["layouts"]:
        rec = STATE["records"].get(name, {}).get(rng)
        if name != cur and rec and rec[1] >= int(ARGS.get("samples", 3)) and rec[0] > best_rate:
            best, best_rate = name, rec[0]
    return dict(ARGS["layouts"][best]) if best else {}


def rolled_back(now):
    STATE["held_until"] = now + float(ARGS.get("pause", 3600.0))


def save_state():
    return {"held_until": STATE["held_until"], "records": STATE["records"]}


def restore_state(state):
    STATE["held_until"] = float(state.get("held_until", 0.0))
    STATE["records"] = dict(state.get("records", {}))
