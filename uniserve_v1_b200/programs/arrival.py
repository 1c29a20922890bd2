# The default scheduling program: admit by (priority, arrival), preempt the latest arrival of
# the lowest priority, place on the first group.  Reads its scheduler's queue, writes the batch.


def dispatch(waiting, room):
    order = sorted(waiting, key=lambda r: (-r["priority"], r["arrival"]))
    return [r["id"] for r in order]


def preempt(running):
    if not running:
        return None
    victim = max(running, key=lambda r: (-r["priority"], r["arrival"]))
    return victim["id"]


def place(request, groups):
    return 0


def limits():
    return {}
