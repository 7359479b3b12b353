"""HTTP surface on a CPU engine: OpenAI chat/completions (plain and streamed), Anthropic messages, metrics, health,
profiler guard, tool-call extraction, and the engine-process watchdog."""
import asyncio
import json
import os
import time

import pytest

from nanoengine_b200 import Config
from nanoengine_b200.server import tool_parser as tp
from nanoengine_b200.server.tokenizer import ByteTokenizer


def _cfg(**kw):
    base = dict(model="tiny-deepseek-v3", dtype="float32", device="cpu", kvcache_block_size=16, max_num_seqs=8, num_kvcache_blocks=128)
    base.update(kw)
    return Config(**base)


@pytest.fixture(scope="module")
def served():
    from starlette.testclient import TestClient
    from nanoengine_b200.server.engine_server import EngineClient, spawn_backend
    from nanoengine_b200.server.openai_server import create_app
    cfg = _cfg()
    proc, endpoint = spawn_backend(cfg)
    client = EngineClient(endpoint, proc)
    app = create_app(client, ByteTokenizer(1024), "tiny", tool_format="hermes")
    with TestClient(app) as tc:
        yield tc, proc
    client.destroy()
    if proc.is_alive():
        proc.terminate()
    proc.join(timeout=10)


def test_health_models_metrics(served):
    tc, _ = served
    assert tc.get("/health").json()["status"] == "ok"
    assert tc.get("/v1/models").json()["data"][0]["id"] == "tiny"
    r = tc.post("/v1/completions", json={"prompt": "hello", "max_tokens": 4, "temperature": 0, "ignore_eos": True})
    assert r.status_code == 200 and r.json()["usage"]["completion_tokens"] == 4
    assert "dlengine_requests" in tc.get("/metrics").text


def test_chat_completion_and_streaming_agree(served):
    tc, _ = served
    body = {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 6, "temperature": 0, "ignore_eos": True}
    full = tc.post("/v1/chat/completions", json=body).json()
    assert full["choices"][0]["finish_reason"] == "length"
    text = ""
    with tc.stream("POST", "/v1/chat/completions", json={**body, "stream": True, "stream_options": {"include_usage": True}}) as r:
        lines = [l for l in r.iter_lines() if l.startswith("data: ")]
    assert lines[-1] == "data: [DONE]"
    usage = None
    for l in lines[:-1]:
        d = json.loads(l[6:])
        for c in d.get("choices", []):
            text += (c.get("delta") or {}).get("content") or ""
        usage = d.get("usage") or usage
    assert text == full["choices"][0]["message"]["content"]
    assert usage["completion_tokens"] == 6


def test_anthropic_messages(served):
    tc, _ = served
    body = {"model": "tiny", "max_tokens": 5, "temperature": 0, "system": "be brief", "messages": [{"role": "user", "content": [{"type": "text", "text": "hi"}]}]}
    r = tc.post("/v1/messages", json=body).json()
    assert r["type"] == "message" and r["usage"]["output_tokens"] <= 5 and r["stop_reason"] in ("max_tokens", "end_turn")
    n = tc.post("/v1/messages/count_tokens", json=body).json()["input_tokens"]
    assert n == r["usage"]["input_tokens"]
    with tc.stream("POST", "/v1/messages", json={**body, "stream": True}) as resp:
        events = [l for l in resp.iter_lines() if l.startswith("event: ")]
    assert events[0] == "event: message_start" and events[-1] == "event: message_stop"


def test_profiler_endpoints_guard_the_trace_name(served):
    tc, _ = served
    assert tc.post("/start_profiler", json={"trace_name": "../x"}).status_code == 400
    assert tc.post("/start_profiler", json={"trace_name": "ok"}).json() == {"started": False}   # no profiler_dir configured


def test_backend_death_is_noticed(served):
    tc, proc = served
    proc.terminate()
    proc.join(timeout=10)
    time.sleep(1.2)
    assert tc.get("/health").status_code == 503
    r = tc.post("/v1/completions", json={"prompt": "x", "max_tokens": 2})
    assert r.status_code == 503


# ---- tool parsers (no engine needed) ------------------------------------------------------------
def test_hermes_tool_call_roundtrip():
    text = 'Sure.<tool_call>{"name": "get_weather", "arguments": {"city": "Paris", "days": 2}}</tool_call>'
    content, calls = tp.parse(text, "hermes")
    assert content == "Sure." and calls[0].name == "get_weather" and calls[0].arguments == {"city": "Paris", "days": 2}
    assert json.loads(calls[0].to_openai()["function"]["arguments"])["days"] == 2
    same, none = tp.parse("no tools here", "hermes")
    assert same == "no tools here" and none == []
    bad, none = tp.parse("<tool_call>{oops}</tool_call>", "hermes")
    assert none == [] and "oops" in bad


def test_qwen3_xml_and_glm_xml_use_schema_types():
    tools = [{"type": "function", "function": {"name": "f", "parameters": {"properties": {"q": {"type": "string"}, "n": {"type": "integer"}}}}}]
    q = "<tool_call>\n<function=f>\n<parameter=q>\n42\n</parameter>\n<parameter=n>\n7\n</parameter>\n</function>\n</tool_call>"
    _, calls = tp.parse(q, "auto", tools)
    assert calls[0].arguments == {"q": "42", "n": 7}
    g = "<tool_call>f\n<arg_key>q</arg_key>\n<arg_value>hello</arg_value>\n<arg_key>n</arg_key>\n<arg_value>3</arg_value>\n</tool_call>"
    _, calls = tp.parse(g, "auto", tools)
    assert calls[0].name == "f" and calls[0].arguments == {"q": "hello", "n": 3}


def test_kimi_format():
    t = "ok<|tool_calls_section_begin|><|tool_call_begin|>functions.search:0<|tool_call_argument_begin|>{\"q\": \"x\"}<|tool_call_end|><|tool_calls_section_end|>"
    content, calls = tp.parse(t)
    assert content == "ok" and calls[0].name == "search" and calls[0].arguments == {"q": "x"}


def test_streaming_parser_holds_back_partial_tags():
    p = tp.StreamingToolParser("hermes")
    out, calls = [], []
    for piece in ["Hello <to", "ol_call>{\"name\": \"f\", \"argu", "ments\": {\"a\": 1}}</tool", "_call> bye <", "b>"]:
        o, c = p.feed(piece)
        out.append(o); calls.extend(c)
    o, c = p.flush()
    out.append(o); calls.extend(c)
    assert "".join(out) == "Hello  bye <b>" and len(calls) == 1 and calls[0].arguments == {"a": 1}
    assert out[0] == "Hello "     # the possible tag prefix was held back
