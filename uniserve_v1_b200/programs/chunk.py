# chunk: trades time to first token against time per output token through the prefill chunk.
# readings: {"ttft_p99": {replica: s}, "tpot_p99": {replica: s}, "chunk": tokens or None,
#            "max_num_batched_tokens": tokens or None}
# ARGS: tpot, ttft (seconds), low, high (tokens), pause (seconds, default 3600)
STATE = {"held_until": 0.0}


def step(readings, now):
    if now < STATE["held_until"]:
        return {}
    low, high = int(ARGS["low"]), int(ARGS["high"])
    chunk = readings.get("chunk")
    if chunk is None:
        chunk = readings.get("max_num_batched_tokens") or high
    tpot = [v for v in readings.get("tpot_p99", {}).values() if v is not None]
    ttft = [v for v in readings.get("ttft_p99", {}).values() if v is not None]
    new = chunk
    if any(v > float(ARGS["tpot"]) for v in tpot):
        new = max(low, chunk // 2)
    elif any(v > float(ARGS["ttft"]) for v in ttft):
        new = min(high, chunk * 2)
    if new == chunk:
        return {}
    return {"scheduler_config.chunked_prefill_size": new}


def rolled_back(now):
    STATE["held_until"] = now + float(ARGS.get("pause", 3600.0))


def save_state():
    return dict(STATE)


def restore_state(state):
    STATE["held_until"] = float(state.get("held_until", 0.0))
