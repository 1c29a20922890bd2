"""Test doubles: a deterministic fake executor so the real scheduler, block manager
and engine loop can be exercised without a model or a GPU (the reference's
``FakeExecutor`` / ``InProcessPool`` idea, crates/testkit/src/lib.rs:1-22,
reference project path)."""
from .fakes import FakeEngine, FakeRunner  # noqa: F401
