# expert-order: balances each routed layer's expert ranks.
# readings: {"tokens": {layer: [tokens of logical expert e]}, "order": {layer: [expert in slot]}}
# ARGS: ranks, imbalance (default 1.1), pause
STATE = {"held_until": 0.0}


def _rank_loads(order, tokens, ranks):
    per = len(order) // ranks
    return [sum(tokens[e] for e in order[r * per:(r + 1) * per]) for r in range(ranks)]


def _rebalance(order, tokens, ranks):
    per = len(order) // ranks
    home = {e: i // per for i, e in enumerate(order)}
    slot_of = {e: i for i, e in enumerate(order)}
    loads = [0] * ranks
    members = [[] for _ in range(ranks)]
    for e in sorted(range(len(order)), key=lambda e: (-tokens[e], e)):
        open_ranks = [r for r in range(ranks) if len(members[r]) < per]
        r = min(open_ranks, key=lambda r: (loads[r], r))
        members[r].append(e)
        loads[r] += tokens[e]
    new = [None] * len(order)
    for r in range(ranks):
        free = [i for i in range(r * per, (r + 1) * per)]
        stay = [e for e in members[r] if home[e] == r]
        for e in stay:                       # an expert that stays on its rank keeps its slot
            new[slot_of[e]] = e
            free.remove(slot_of[e])
        for e in members[r]:
            if home[e] != r:
                new[free.pop(0)] = e
    return new


def step(readings, now):
    if now < STATE["held_until"]:
        return {}
    ranks = int(ARGS["ranks"])
    limit = float(ARGS.get("imbalance", 1.1))
    out = dict(readings.get("order") or {})
    changed = False
    for layer, tokens in readings.get("tokens", {}).items():
        n = len(tokens)
        if n % ranks or sum(tokens) == 0:
            continue
        order = list(out.get(layer) or range(n))
        loads = _rank_loads(order, tokens, ranks)
        mean = sum(loads) / ranks
        if max(loads) <= limit * mean:
            continue
        new = _rebalance(order, tokens, ranks)
        if max(_rank_loads(new, tokens, ranks)) < max(loads):
            out[layer] = new
            changed = True
    return {"moe_config.expert_order": out} if changed else {}


def rolled_back(now):
    STATE["held_until"] = now + float(ARGS.get("pause", 3600.0))


def save_state():
    return dict(STATE)


def restore_state(state):
    STATE["held_until"] = float(state.get("held_until", 0.0))
