"""Strict request schemas of the HTTP API (unknown fields are refused by name).

Reference behaviour: crates/daemon/src/api/protocol.rs:483-586 (chat),
crates/daemon/src/api/protocol/video.rs:36-80 (video) — reference project paths.
"""
from __future__ import annotations

from typing import Any, Literal, Optional, Union

from pydantic import BaseModel, ConfigDict, Field, field_validator, model_validator


class Strict(BaseModel):
    model_config = ConfigDict(extra="forbid")


class FunctionDef(Strict):
    name: str
    description: Optional[str] = None
    parameters: Optional[dict] = None
    strict: Optional[bool] = None


class Tool(Strict):
    type: Literal["function"] = "function"
    function: FunctionDef


class ToolCallFunction(Strict):
    name: str
    arguments: Union[str, dict]


class ToolCall(Strict):
    id: Optional[str] = None
    type: Literal["function"] = "function"
    function: ToolCallFunction
    index: Optional[int] = None


class Message(Strict):
    role: Literal["system", "developer", "user", "assistant", "tool"]
    content: Optional[Union[str, list]] = None
    name: Optional[str] = None
    tool_calls: Optional[list[ToolCall]] = None
    tool_call_id: Optional[str] = None
    reasoning: Optional[str] = None
    reasoning_content: Optional[str] = None


class StreamOptions(Strict):
    include_usage: Optional[bool] = None


class ChatCompletionRequest(Strict):
    model: str
    messages: list[Message]
    stream: bool = False
    stream_options: Optional[StreamOptions] = None
    max_tokens: Optional[int] = Field(None, ge=1)
    max_completion_tokens: Optional[int] = Field(None, ge=1)
    temperature: Optional[float] = Field(None, ge=0)
    top_p: Optional[float] = Field(None, gt=0, le=1)
    top_k: Optional[int] = None
    min_p: Optional[float] = Field(None, ge=0, le=1)
    n: int = Field(1, ge=1, le=1)
    seed: Optional[int] = None
    stop: Optional[Union[str, list[str]]] = None
    stop_token_ids: Optional[list[int]] = None
    presence_penalty: Optional[float] = Field(None, ge=-2, le=2)
    frequency_penalty: Optional[float] = Field(None, ge=-2, le=2)
    repetition_penalty: Optional[float] = Field(None, gt=0)
    logit_bias: Optional[dict[str, float]] = None
    logprobs: Optional[bool] = None
    top_logprobs: Optional[int] = Field(None, ge=0)
    tools: Optional[list[Tool]] = None
    tool_choice: Optional[Union[Literal["auto", "none", "required"], dict]] = None
    parallel_tool_calls: Optional[bool] = None
    response_format: Optional[dict] = None
    user: Optional[str] = None
    # extensions
    allowed_token_ids: Optional[list[int]] = None
    bad_words: Optional[list[str]] = None
    min_tokens: Optional[int] = Field(None, ge=0)
    ignore_eos: Optional[bool] = None
    priority: Optional[int] = None
    cache_salt: Optional[str] = None
    prompt_cache_key: Optional[str] = None
    chat_template_kwargs: Optional[dict] = None
    skip_special_tokens: Optional[bool] = None
    include_reasoning: Optional[bool] = None

    @field_validator("messages")
    @classmethod
    def _nonempty(cls, v):
        if not v:
            raise ValueError("messages must not be empty")
        return v


class InputReference(Strict):
    type: Literal["image", "video", "audio"]
    url: str
    frame_index: Optional[int] = None
    start_time_seconds: Optional[float] = None


class VideoGenerationRequest(Strict):
    model: str
    prompt: str
    negative_prompt: Optional[str] = None
    size: Optional[str] = None
    seconds: Optional[Union[float, str]] = None
    num_frames: Optional[int] = None
    fps: Optional[int] = None
    seed: Optional[int] = None
    num_inference_steps: Optional[int] = None
    guidance_scale: Optional[float] = None
    input_references: Optional[list[InputReference]] = None
    extra_params: Optional[dict] = None

    @model_validator(mode="after")
    def _exclusive(self):
        if self.seconds is not None and self.num_frames is not None:
            raise ValueError("state `seconds` or `num_frames`, not both")
        return self


def openai_error(message: str, type_: str = "invalid_request_error", code=None, param=None):
    return {"error": {"message": message, "type": type_, "param": param, "code": code}}
