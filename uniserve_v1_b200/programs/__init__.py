"""The release's programs: sources that a policy package names as ``uniserve:<name>``.

Each file is a *program*: plain functions run by ``engine.program.ProgramHost`` in a
metered namespace, like a package's own programs.  ``arrival`` is the default scheduling
program; ``chunk``, ``expert_order``, ``layout``, ``backend`` and ``role`` are control
programs (``step(readings, now) -> {option path: value}``); ``ttft`` is a routing program
(``route(request, replicas)``).  The rules are those the reference documents for its
programs of the same names (docs/configuration.md:100-215, reference project path).
"""
from pathlib import Path

NAMES = ("arrival", "chunk", "expert_order", "layout", "backend", "role", "ttft")


def source_of(name: str) -> str:
    """Source text of ``uniserve:<name>`` (``expert-order`` and ``expert_order`` both work)."""
    key = name.split(":", 1)[-1].replace("-", "_")
    if key not in NAMES:
        raise KeyError(f"no released program {name!r}; there are {', '.join(NAMES)}")
    return (Path(__file__).parent / f"{key}.py").read_text()
