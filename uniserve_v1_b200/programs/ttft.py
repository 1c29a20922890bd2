# ttft: routes each request to the prefill replica predicted to give its first token soonest.
# request: {"prompt_tokens": n, "hits": {replica: cached prompt tokens}}
# replicas: [{"id", "role", "remaining" (s of the running batch), "queued_prefill_tokens",
#             "running", "reservable_pages"}]
# ARGS: rate (prefill tokens / s), page (tokens of a KV page)
# returns {"prefill": id, "decode": id} (None where the deployment has no replica of a role)


def route(request, replicas):
    rate, page = float(ARGS["rate"]), int(ARGS["page"])
    can_prefill = [r for r in replicas if r["role"] in ("prefill", "mixed")]
    if not can_prefill:
        return {"prefill": None, "decode": None, "why": "no replica computes prompts"}

    def eta(r):
        missing = request["prompt_tokens"] - request.get("hits", {}).get(r["id"], 0)
        return r.get("remaining", 0.0) + (r.get("queued_prefill_tokens", 0) + max(missing, 0)) / rate
    order = sorted(range(len(can_prefill)),
                   key=lambda i: (eta(can_prefill[i]), can_prefill[i].get("running", 0), i))
    p = can_prefill[order[0]]
    if p["role"] == "mixed":
        return {"prefill": p["id"], "decode": p["id"]}
    dec = [r for r in replicas if r["role"] in ("decode", "mixed")]
    if not dec:
        return {"prefill": p["id"], "decode": None, "why": "no replica decodes"}
    need = (request["prompt_tokens"] + page - 1) // page
    fits = [r for r in dec if r.get("reservable_pages", 0) >= need] or dec
    d = min(fits, key=lambda r: (r.get("running", 0), r["id"]))
    return {"prefill": p["id"], "decode": d["id"]}
