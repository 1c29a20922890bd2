"""Request-side rules of the MiniMax-H3 / FastH3 family: task derivation, served
sizes, the frame rule and the canvas rule.

Reference behaviour: crates/processing/src/minimax_h3/{mod,rules,frames}.rs:41-160,
docs/minimax_h3/minimax_h3.md:218-278 (reference project paths).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

SIZES = ["1536x672", "1344x768", "1024x768", "768x768", "768x1024", "768x1344"]
FPS = 24
MIN_SECONDS, MAX_SECONDS = 4, 15
MAX_REFS = {"image": 9, "video": 3, "audio": 3, "total": 12}


class VideoRuleError(ValueError):
    def __init__(self, param: str, message: str):
        super().__init__(message)
        self.param = param


def frames_for_seconds(seconds: float) -> int:
    """seconds x 24 rounded half to even, extended to the next 17n + 5."""
    raw = round(float(seconds) * FPS)           # Python rounds half to even
    n = max(0, -(-(raw - 5) // 17))
    return 17 * n + 5


def is_rule_count(frames: int) -> bool:
    return frames >= 5 and (frames - 5) % 17 == 0


def canvas_for(width: int, height: int):
    """768-pixel short edge, area <= 768 x 1344, sides multiples of 32."""
    short, long_ = min(width, height), max(width, height)
    scale = 768.0 / short
    l2 = int(long_ * scale) // 32 * 32
    l2 = min(l2, 1344 if True else l2)
    w, h = (l2, 768) if width >= height else (768, l2)
    return w, h


@dataclass
class VideoPlan:
    task: str                 # t2va | fl2va | ref2va
    width: int
    height: int
    num_frames: int
    fps: int
    seed: int
    steps: int
    keyframes: list = field(default_factory=list)     # (frame_index, reference)
    references: list = field(default_factory=list)

    @property
    def seconds(self) -> float:
        return self.num_frames / self.fps


def plan_request(req, served_sizes=None, max_seconds: int = MAX_SECONDS, schedule_steps: int = 8,
                 served_tasks=("t2va", "fl2va", "ref2va"), rng=None) -> VideoPlan:
    """Validates a video request against the family rules and lowers it."""
    import random
    served_sizes = served_sizes or SIZES
    if req.negative_prompt is not None:
        raise VideoRuleError("negative_prompt", "the schedule runs without classifier-free guidance")
    if req.guidance_scale is not None:
        raise VideoRuleError("guidance_scale", "the schedule runs without classifier-free guidance")
    if req.extra_params:
        raise VideoRuleError("extra_params", "the model defines no extra parameter")
    if req.fps is not None and req.fps != FPS:
        raise VideoRuleError("fps", f"the model generates {FPS} frames per second")
    if req.num_inference_steps is not None and req.num_inference_steps != schedule_steps:
        raise VideoRuleError("num_inference_steps",
                             f"the served schedule has {schedule_steps} denoiser evaluations")
    refs = req.input_references or []
    keyframes = [(r.frame_index, r) for r in refs if r.frame_index is not None]
    plain = [r for r in refs if r.frame_index is None]
    if not refs:
        task = "t2va"
    elif plain:
        task = "ref2va"
        if len(keyframes) > 2:
            raise VideoRuleError("input_references", "ref2va takes up to two keyframes")
    else:
        task = "fl2va"
        idx = [k for k, _ in keyframes]
        if any(r.type != "image" for _, r in keyframes) or idx not in ([0], [-1], [0, -1]):
            raise VideoRuleError("input_references",
                                 "keyframes are images at frame_index 0, -1 or both in that order")
    if task not in served_tasks:
        raise VideoRuleError("input_references", f"the deployment does not serve {task}")
    counts = {"image": 0, "video": 0, "audio": 0}
    for r in plain:
        counts[r.type] += 1
    for k in ("image", "video", "audio"):
        if counts[k] > MAX_REFS[k]:
            raise VideoRuleError("input_references", f"at most {MAX_REFS[k]} {k} references")
    if sum(counts.values()) > MAX_REFS["total"]:
        raise VideoRuleError("input_references", f"at most {MAX_REFS['total']} references")
    size = req.size or served_sizes[0]
    if size not in served_sizes:
        raise VideoRuleError("size", f"served sizes: {', '.join(served_sizes)}")
    w, h = (int(x) for x in size.split("x"))
    lo, hi = frames_for_seconds(MIN_SECONDS), frames_for_seconds(max_seconds)
    if req.num_frames is not None:
        if not is_rule_count(req.num_frames) or not lo <= req.num_frames <= hi:
            raise VideoRuleError("num_frames", f"a count 17n + 5 between {lo} and {hi}")
        frames = req.num_frames
    else:
        try:
            secs = float(req.seconds) if req.seconds is not None else 5.0
        except ValueError:
            raise VideoRuleError("seconds", "a number or a numeric string")
        if not MIN_SECONDS <= secs <= max_seconds:
            raise VideoRuleError("seconds", f"{MIN_SECONDS} to {max_seconds}")
        frames = frames_for_seconds(secs)
    seed = req.seed if req.seed is not None else (rng or random).randrange(1 << 31)
    return VideoPlan(task, w, h, frames, FPS, seed, schedule_steps, keyframes, plain)


def capabilities(served_sizes=None, max_seconds: int = MAX_SECONDS, steps: int = 8) -> dict:
    return {"tasks": ["t2va", "fl2va", "ref2va"], "sizes": served_sizes or SIZES,
            "seconds": {"min": MIN_SECONDS, "max": max_seconds},
            "frame_rule": "17n + 5", "fps": FPS,
            "frames": {"min": frames_for_seconds(MIN_SECONDS), "max": frames_for_seconds(max_seconds)},
            "schedule": {"num_inference_steps": steps, "guidance": False},
            "references": MAX_REFS,
            "request_fields": ["model", "prompt", "size", "seconds", "num_frames", "fps", "seed",
                               "num_inference_steps", "input_references"],
            "media": {"schemes": ["data", "file", "http", "https"]},
            "jobs": {"retention_seconds": 3600, "store_bytes": 1 << 30}}
