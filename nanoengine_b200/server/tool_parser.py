"""Tool-call extraction from model text, whole or streamed.

Formats:
  hermes      <tool_call>{"name": ..., "arguments": {...}}</tool_call>
  qwen3_xml   <tool_call><function=NAME><parameter=KEY>VALUE</parameter>...</function></tool_call>
  glm_xml     <tool_call>NAME<arg_key>K</arg_key><arg_value>V</arg_value>...</tool_call>
  kimi        <|tool_calls_section_begin|><|tool_call_begin|>functions.NAME:IDX<|tool_call_argument_begin|>{json}<|tool_call_end|>...

`parse` handles a finished completion; `StreamingToolParser` consumes deltas and emits content text as soon as it is
certain not to belong to a tool call, holding back only a possible prefix of an opening tag.

Parity: reference server/tool_parser.py (Hermes / Qwen3-XML / GLM-XML) and server/kimi_k3_parser.py; tests/test_tool_parser.py.
"""
from __future__ import annotations

import json
import re
import uuid
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


@dataclass
class ToolCall:
    name: str
    arguments: Dict[str, Any]
    id: str = field(default_factory=lambda: "call_" + uuid.uuid4().hex[:24])

    def to_openai(self, index: int = 0) -> Dict[str, Any]:
        return {"index": index, "id": self.id, "type": "function",
                "function": {"name": self.name, "arguments": json.dumps(self.arguments, ensure_ascii=False)}}


def _coerce(value: str, schema_type: Optional[str] = None) -> Any:
    v = value.strip()
    if schema_type == "string":
        return value.strip("\n")
    try:
        return json.loads(v)
    except Exception:
        return value.strip("\n")


def _param_types(tools: Optional[List[dict]], name: str) -> Dict[str, str]:
    for t in tools or []:
        fn = t.get("function", t)
        if fn.get("name") == name:
            props = (fn.get("parameters") or fn.get("input_schema") or {}).get("properties", {})
            return {k: v.get("type") for k, v in props.items() if isinstance(v, dict)}
    return {}


_HERMES = re.compile(r"<tool_call>\s*(\{.*?\})\s*</tool_call>", re.S)
_QWEN_BLOCK = re.compile(r"<tool_call>\s*<function=([^>\s]+)>(.*?)</function>\s*</tool_call>", re.S)
_QWEN_PARAM = re.compile(r"<parameter=([^>\s]+)>(.*?)</parameter>", re.S)
_GLM_BLOCK = re.compile(r"<tool_call>\s*([^\s<]+)\s*(.*?)</tool_call>", re.S)
_GLM_ARG = re.compile(r"<arg_key>(.*?)</arg_key>\s*<arg_value>(.*?)</arg_value>", re.S)
_KIMI_CALL = re.compile(r"<\|tool_call_begin\|>\s*(?:functions\.)?([\w\-.]+?)(?::(\d+))?\s*<\|tool_call_argument_begin\|>(.*?)<\|tool_call_end\|>", re.S)
_KIMI_SECTION = re.compile(r"<\|tool_calls_section_begin\|>.*?(?:<\|tool_calls_section_end\|>|$)", re.S)

OPEN_TAGS = {"hermes": "<tool_call>", "qwen3_xml": "<tool_call>", "glm_xml": "<tool_call>", "kimi": "<|tool_calls_section_begin|>"}
CLOSE_TAGS = {"hermes": "</tool_call>", "qwen3_xml": "</tool_call>", "glm_xml": "</tool_call>", "kimi": "<|tool_calls_section_end|>"}


def detect_format(text: str) -> str:
    if "<|tool_call_begin|>" in text:
        return "kimi"
    if "<function=" in text:
        return "qwen3_xml"
    if "<arg_key>" in text:
        return "glm_xml"
    return "hermes"


def parse(text: str, fmt: str = "auto", tools: Optional[List[dict]] = None) -> Tuple[str, List[ToolCall]]:
    """Returns (content without the tool-call markup, tool calls in order).  Malformed calls stay in the content."""
    if fmt == "auto":
        fmt = detect_format(text)
    calls: List[ToolCall] = []
    content = text
    if fmt == "hermes":
        def sub(m):
            try:
                d = json.loads(m.group(1))
                args = d.get("arguments", d.get("parameters", {}))
                if isinstance(args, str):
                    args = json.loads(args)
                calls.append(ToolCall(d["name"], args))
                return ""
            except Exception:
                return m.group(0)
        content = _HERMES.sub(sub, text)
    elif fmt == "qwen3_xml":
        def sub(m):
            name = m.group(1)
            types = _param_types(tools, name)
            args = {k: _coerce(v, types.get(k)) for k, v in _QWEN_PARAM.findall(m.group(2))}
            calls.append(ToolCall(name, args))
            return ""
        content = _QWEN_BLOCK.sub(sub, text)
    elif fmt == "glm_xml":
        def sub(m):
            name = m.group(1)
            types = _param_types(tools, name)
            args = {k.strip(): _coerce(v, types.get(k.strip())) for k, v in _GLM_ARG.findall(m.group(2))}
            calls.append(ToolCall(name, args))
            return ""
        content = _GLM_BLOCK.sub(sub, text)
    elif fmt == "kimi":
        for name, idx, raw in _KIMI_CALL.findall(text):
            try:
                calls.append(ToolCall(name, json.loads(raw) if raw.strip() else {}))
            except Exception:
                calls.append(ToolCall(name, {"_raw": raw}))
        content = _KIMI_SECTION.sub("", text)
    else:
        raise ValueError(f"unknown tool-call format {fmt}")
    return content.strip() if calls else text, calls


class StreamingToolParser:
    """Feed text deltas; get back (content_delta, finished tool calls).  Text inside an open tool-call block is buffered
    until the block closes; a trailing fragment that could be the start of an opening tag is held back one step."""

    def __init__(self, fmt: str = "hermes", tools: Optional[List[dict]] = None):
        self.fmt, self.tools = fmt, tools
        self.open_tag, self.close_tag = OPEN_TAGS[fmt], CLOSE_TAGS[fmt]
        self.buf = ""
        self.in_block = False
        self.n_calls = 0

    def feed(self, delta: str) -> Tuple[str, List[ToolCall]]:
        self.buf += delta
        out, calls = "", []
        while True:
            if self.in_block:
                j = self.buf.find(self.close_tag)
                if j < 0:
                    break
                block = self.buf[: j + len(self.close_tag)]
                self.buf = self.buf[j + len(self.close_tag):]
                self.in_block = False
                rest, got = parse(block, self.fmt, self.tools)
                if got:
                    calls.extend(got)
                else:
                    out += block
            else:
                i = self.buf.find(self.open_tag)
                if i >= 0:
                    out += self.buf[:i]
                    self.buf = self.buf[i:]
                    self.in_block = True
                    continue
                # hold back a possible partial opening tag at the end
                keep = 0
                for k in range(min(len(self.open_tag) - 1, len(self.buf)), 0, -1):
                    if self.open_tag.startswith(self.buf[-k:]):
                        keep = k
                        break
                out += self.buf[: len(self.buf) - keep]
                self.buf = self.buf[len(self.buf) - keep:]
                break
        self.n_calls += len(calls)
        return out, calls

    def flush(self) -> Tuple[str, List[ToolCall]]:
        """End of stream: an unterminated block is parsed leniently, else returned as content."""
        rest, self.buf = self.buf, ""
        if self.in_block:
            self.in_block = False
            content, calls = parse(rest + self.close_tag, self.fmt, self.tools)
            if calls:
                return "", calls
        return rest, []
