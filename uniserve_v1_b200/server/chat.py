"""Chat templating, reasoning split and tool-call parsing.

Templates are Jinja (the checkpoint's ``chat_template``); without one the ChatML
form of the Qwen family is used.  Output parsing is incremental so streamed
deltas carry ``reasoning`` / ``content`` / ``tool_calls`` separately:

* reasoning: text between ``<think>`` and ``</think>``;
* tool calls, JSON form: ``<tool_call>{"name": ..., "arguments": {...}}</tool_call>``;
* tool calls, XML form: ``<tool_call><function=NAME><parameter=KEY>VALUE</parameter>
  ...</function></tool_call>`` with parameter values typed by the tool's JSON Schema.

Reference behaviour: crates/daemon/src/api/input/chat/*, output/reasoning/*,
output/tools/{json,xml}/* (reference project paths).
"""
from __future__ import annotations

import json
import re
import uuid
from typing import Optional

import jinja2

CHATML = (
    "{%- if tools %}{{- '<|im_start|>system\\n' }}"
    "{%- if messages[0].role == 'system' %}{{- messages[0].content + '\\n\\n' }}{%- endif %}"
    "{{- '# Tools\\n\\nYou may call one or more functions to assist with the user query.\\n\\n"
    "You are provided with function signatures within <tools></tools> XML tags:\\n<tools>' }}"
    "{%- for tool in tools %}{{- '\\n' }}{{- tool | tojson }}{%- endfor %}"
    "{{- '\\n</tools>\\n\\nFor each function call, return a json object with function name and "
    "arguments within <tool_call></tool_call> XML tags:\\n<tool_call>\\n{\\\"name\\\": <function-name>, "
    "\\\"arguments\\\": <args-json-object>}\\n</tool_call><|im_end|>\\n' }}"
    "{%- elif messages[0].role == 'system' %}"
    "{{- '<|im_start|>system\\n' + messages[0].content + '<|im_end|>\\n' }}{%- endif %}"
    "{%- for m in messages %}"
    "{%- if m.role == 'system' and loop.first %}{%- elif m.role == 'tool' %}"
    "{{- '<|im_start|>user\\n<tool_response>\\n' + m.content + '\\n</tool_response><|im_end|>\\n' }}"
    "{%- elif m.role == 'assistant' %}{{- '<|im_start|>assistant\\n' + (m.content or '') }}"
    "{%- for tc in m.tool_calls or [] %}{{- '\\n<tool_call>\\n{\\\"name\\\": \\\"' + tc.function.name + "
    "'\\\", \\\"arguments\\\": ' + (tc.function.arguments if tc.function.arguments is string else "
    "tc.function.arguments | tojson) + '}\\n</tool_call>' }}{%- endfor %}{{- '<|im_end|>\\n' }}"
    "{%- else %}{{- '<|im_start|>' + m.role + '\\n' + m.content + '<|im_end|>\\n' }}{%- endif %}"
    "{%- endfor %}"
    "{%- if add_generation_prompt %}{{- '<|im_start|>assistant\\n' }}"
    "{%- if enable_thinking is defined and enable_thinking is false %}"
    "{{- '<think>\\n\\n</think>\\n\\n' }}{%- endif %}{%- endif %}"
)


def _flatten_content(content):
    """OpenAI content parts -> text (image parts are kept as placeholders)."""
    if content is None or isinstance(content, str):
        return content or ""
    out = []
    for part in content:
        t = part.get("type")
        if t == "text":
            out.append(part.get("text", ""))
        elif t == "image_url":
            out.append("<|vision_start|><|image_pad|><|vision_end|>")
        elif t == "video_url":
            out.append("<|vision_start|><|video_pad|><|vision_end|>")
        else:
            raise ValueError(f"unsupported content part type {t!r}")
    return "".join(out)


class ChatTemplate:
    def __init__(self, template: Optional[str] = None):
        env = jinja2.Environment(trim_blocks=True, lstrip_blocks=True,
                                 extensions=["jinja2.ext.loopcontrols"])
        env.filters["tojson"] = lambda v, **kw: json.dumps(v, ensure_ascii=False)
        env.globals["raise_exception"] = self._raise
        env.globals["strftime_now"] = lambda fmt: __import__("datetime").datetime.now().strftime(fmt)
        self.template = env.from_string(template or CHATML)

    @staticmethod
    def _raise(msg):
        raise jinja2.TemplateError(msg)

    def render(self, messages: list, tools: Optional[list] = None,
               add_generation_prompt: bool = True, **kwargs) -> str:
        msgs = []
        for m in messages:
            mm = dict(m)
            mm["content"] = _flatten_content(m.get("content"))
            msgs.append(mm)
        return self.template.render(messages=msgs, tools=tools or None,
                                    add_generation_prompt=add_generation_prompt, **kwargs)


# ------------------------------------------------------------ output parsing --
class ReasoningSplitter:
    """Routes streamed text into reasoning (inside <think>…</think>) and content."""

    OPEN, CLOSE = "<think>", "</think>"

    def __init__(self, starts_in_reasoning: bool = False):
        self.in_reasoning = starts_in_reasoning
        self.buf = ""

    def push(self, text: str):
        """Returns (reasoning_delta, content_delta)."""
        self.buf += text
        r_out, c_out = [], []
        while self.buf:
            tag = self.CLOSE if self.in_reasoning else self.OPEN
            i = self.buf.find(tag)
            if i >= 0:
                (r_out if self.in_reasoning else c_out).append(self.buf[:i])
                self.buf = self.buf[i + len(tag):]
                self.in_reasoning = not self.in_reasoning
                continue
            # hold back a tail that could be the start of the tag
            keep = 0
            for k in range(min(len(tag) - 1, len(self.buf)), 0, -1):
                if tag.startswith(self.buf[-k:]):
                    keep = k
                    break
            emit = self.buf[:len(self.buf) - keep]
            (r_out if self.in_reasoning else c_out).append(emit)
            self.buf = self.buf[len(self.buf) - keep:]
            break
        return "".join(r_out), "".join(c_out)

    def flush(self):
        out, self.buf = self.buf, ""
        return (out, "") if self.in_reasoning else ("", out)


_XML_FN = re.compile(r"<function=([^>\s]+)>(.*?)</function>", re.S)
_XML_PARAM = re.compile(r"<parameter=([^>\s]+)>(.*?)</parameter>", re.S)


def _typed(value: str, schema: Optional[dict]):
    """Types an XML parameter value by the tool's JSON Schema."""
    v = value.strip("\n")
    t = (schema or {}).get("type")
    try:
        if t == "integer":
            return int(v)
        if t == "number":
            return float(v)
        if t == "boolean":
            return v.strip().lower() == "true"
        if t in ("object", "array"):
            return json.loads(v)
        if t == "null":
            return None
    except (ValueError, json.JSONDecodeError):
        return v
    return v


class ToolCallParser:
    """Extracts ``<tool_call>…</tool_call>`` blocks from streamed content.  Text
    outside the blocks passes through; a block is released once it is closed."""

    OPEN, CLOSE = "<tool_call>", "</tool_call>"

    def __init__(self, tools: Optional[list] = None):
        self.buf = ""
        self.inside = False
        self.calls: list = []
        self.schemas = {}
        for t in tools or []:
            fn = t.get("function", {})
            self.schemas[fn.get("name")] = (fn.get("parameters") or {}).get("properties", {})

    def _parse_block(self, body: str) -> Optional[dict]:
        body = body.strip()
        m = _XML_FN.search(body)
        if m:
            name = m.group(1)
            props = self.schemas.get(name, {})
            args = {k: _typed(v, props.get(k)) for k, v in _XML_PARAM.findall(m.group(2))}
        else:
            try:
                obj = json.loads(body)
            except json.JSONDecodeError:
                return None
            name, args = obj.get("name"), obj.get("arguments", {})
            if isinstance(args, str):
                try:
                    args = json.loads(args)
                except json.JSONDecodeError:
                    pass
        if not name:
            return None
        return {"id": "call_" + uuid.uuid4().hex[:24], "type": "function",
                "function": {"name": name, "arguments": json.dumps(args, ensure_ascii=False)}}

    def push(self, text: str):
        """Returns (content_delta, [new tool calls])."""
        self.buf += text
        content, new = [], []
        while self.buf:
            if self.inside:
                j = self.buf.find(self.CLOSE)
                if j < 0:
                    break
                call = self._parse_block(self.buf[:j])
                if call:
                    call["index"] = len(self.calls)
                    self.calls.append(call)
                    new.append(call)
                else:      # not a call after all: give the text back
                    content.append(self.OPEN + self.buf[:j] + self.CLOSE)
                self.buf = self.buf[j + len(self.CLOSE):]
                self.inside = False
                continue
            i = self.buf.find(self.OPEN)
            if i >= 0:
                content.append(self.buf[:i])
                self.buf = self.buf[i + len(self.OPEN):]
                self.inside = True
                continue
            keep = 0
            for k in range(min(len(self.OPEN) - 1, len(self.buf)), 0, -1):
                if self.OPEN.startswith(self.buf[-k:]):
                    keep = k
                    break
            content.append(self.buf[:len(self.buf) - keep])
            self.buf = self.buf[len(self.buf) - keep:]
            break
        return "".join(content), new

    def flush(self):
        out = (self.OPEN if self.inside else "") + self.buf
        self.buf, self.inside = "", False
        return out


class StopStrings:
    """Stop-string matcher over streamed text: holds back text that could still
    become a stop string; ``push`` returns (text_to_emit, stopped)."""

    def __init__(self, stops):
        self.stops = [s for s in (stops or []) if s]
        self.buf = ""

    def push(self, text: str):
        if not self.stops:
            return text, False
        self.buf += text
        hit = min((i for i in (self.buf.find(s) for s in self.stops) if i >= 0), default=-1)
        if hit >= 0:
            out, self.buf = self.buf[:hit], ""
            return out, True
        keep = 0
        for s in self.stops:
            for k in range(min(len(s) - 1, len(self.buf)), 0, -1):
                if s.startswith(self.buf[-k:]):
                    keep = max(keep, k)
                    break
        out = self.buf[:len(self.buf) - keep]
        self.buf = self.buf[len(self.buf) - keep:]
        return out, False

    def flush(self):
        out, self.buf = self.buf, ""
        return out
