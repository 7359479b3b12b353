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


class LetterTokenizer(ByteTokenizer):
    """Printable bytes as themselves, every other id as a letter: a random-weight model then answers in visible text."""

    def decode(self, ids):
        return "".join(chr(i) if 32 <= i < 127 else chr(97 + i % 26) for i in ids)


@pytest.fixture(scope="module")
def served():
    from starlette.testclient import TestClient
    from nanoengine_b200.server.engine_server import EngineClient, spawn_backend
    from nanoengine_b200.server.openai_server import create_app
    cfg = _cfg()
    proc, endpoint = spawn_backend(cfg)
    client = EngineClient(endpoint, proc)
    app = create_app(client, LetterTokenizer(1024), "tiny", tool_format="hermes")
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


def test_unknown_model_is_404_and_names_are_case_insensitive(served):
    tc, _ = served
    body = {"prompt": "hello", "max_tokens": 2, "temperature": 0, "ignore_eos": True}
    assert tc.post("/v1/completions", json={**body, "model": "TINY"}).status_code == 200
    r = tc.post("/v1/completions", json={**body, "model": "someone-else"})
    assert r.status_code == 404 and r.json()["error"]["code"] == "model_not_found"
    assert tc.post("/v1/chat/completions", json={"model": "nope", "messages": [{"role": "user", "content": "x"}]}).status_code == 404
    assert tc.post("/v1/messages", json={"model": "nope", "max_tokens": 2, "messages": [{"role": "user", "content": "x"}]}).status_code == 404


def test_stop_strings_cut_the_answer_plain_and_streamed(served):
    tc, _ = served
    body = {"prompt": "stop strings", "max_tokens": 24, "temperature": 0, "ignore_eos": True}
    full = tc.post("/v1/completions", json=body).json()["choices"][0]["text"]
    assert len(full) >= 12
    stop = full[8:11]
    want = full[: full.find(stop)]
    r = tc.post("/v1/completions", json={**body, "stop": [stop, "\x00never"]}).json()
    assert r["choices"][0]["text"] == want and r["choices"][0]["finish_reason"] == "stop" and r["usage"]["completion_tokens"] < 24
    text, finish = "", None
    with tc.stream("POST", "/v1/completions", json={**body, "stop": stop, "stream": True}) as resp:
        for l in resp.iter_lines():
            if l.startswith("data: ") and l != "data: [DONE]":
                for c in json.loads(l[6:]).get("choices", []):
                    text += c.get("text") or ""
                    finish = c.get("finish_reason") or finish
    assert text == want and finish == "stop"
    # the engine is free again: the aborted requests left nothing behind
    assert tc.post("/v1/completions", json=body).json()["choices"][0]["text"] == full


def test_reasoning_goes_to_its_own_field_when_the_prompt_opens_the_block(served):
    tc, _ = served
    body = {"messages": [{"role": "user", "content": "solve <think>"}], "max_tokens": 6, "temperature": 0, "ignore_eos": True}
    msg = tc.post("/v1/chat/completions", json=body).json()["choices"][0]["message"]
    assert msg["content"] == "" and len(msg["reasoning_content"]) > 0
    thought = ""
    with tc.stream("POST", "/v1/chat/completions", json={**body, "stream": True}) as resp:
        for l in resp.iter_lines():
            if l.startswith("data: ") and l != "data: [DONE]":
                for c in json.loads(l[6:]).get("choices", []):
                    d = c.get("delta") or {}
                    assert not d.get("content")
                    thought += d.get("reasoning_content") or ""
    assert thought == msg["reasoning_content"]
    plain = tc.post("/v1/chat/completions", json={**body, "messages": [{"role": "user", "content": "solve"}]}).json()["choices"][0]["message"]
    assert "reasoning_content" not in plain and len(plain["content"]) > 0


def test_anthropic_stop_sequences_and_thinking_blocks(served):
    tc, _ = served
    body = {"model": "tiny", "max_tokens": 24, "temperature": 0, "ignore_eos": True, "messages": [{"role": "user", "content": "stop here"}]}
    full = tc.post("/v1/messages", json=body).json()
    text = full["content"][0]["text"]
    assert full["stop_reason"] == "max_tokens" and len(text) >= 12
    stop = text[8:11]
    r = tc.post("/v1/messages", json={**body, "stop_sequences": [stop]}).json()
    assert r["stop_reason"] == "stop_sequence" and r["stop_sequence"] == stop and r["usage"]["output_tokens"] < 24
    assert "".join(b["text"] for b in r["content"] if b["type"] == "text") == text[: text.find(stop)]
    got, reason = "", None
    with tc.stream("POST", "/v1/messages", json={**body, "stop_sequences": [stop], "stream": True}) as resp:
        for l in resp.iter_lines():
            if l.startswith("data: "):
                d = json.loads(l[6:])
                if d["type"] == "content_block_delta":
                    got += d["delta"].get("text", "")
                if d["type"] == "message_delta":
                    reason = (d["delta"]["stop_reason"], d["delta"]["stop_sequence"])
    assert got == text[: text.find(stop)] and reason == ("stop_sequence", stop)
    # a prompt that leaves a thinking block open: the answer is a thinking block, plain and streamed
    think = {**body, "max_tokens": 6, "messages": [{"role": "user", "content": "solve <think>"}]}
    r = tc.post("/v1/messages", json=think).json()
    assert [b["type"] for b in r["content"]] == ["thinking"] and len(r["content"][0]["thinking"]) > 0
    kinds, thought = [], ""
    with tc.stream("POST", "/v1/messages", json={**think, "stream": True}) as resp:
        for l in resp.iter_lines():
            if l.startswith("data: "):
                d = json.loads(l[6:])
                if d["type"] == "content_block_start":
                    kinds.append((d["index"], d["content_block"]["type"]))
                if d["type"] == "content_block_delta":
                    thought += d["delta"].get("thinking", "")
    assert kinds == [(0, "thinking")] and thought == r["content"][0]["thinking"]


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


# ---- model names, stop strings, reasoning blocks ------------------------------------------------------------------------------
def test_text_filters():
    from nanoengine_b200.server.text_stream import (ReasoningStream, StopStream, cut_at_stop, model_aliases, parse_stop,
                                                     prompt_opens_thinking, resolve_request_model, split_reasoning)
    assert parse_stop({"stop": "x"}) == ["x"] and parse_stop({"stop": ["a", "", 3, "b"]}) == ["a", "b"] and parse_stop({}) == [] and parse_stop({"stop": 5}) == []
    assert cut_at_stop("one two three", ["three", "two"]) == ("one ", True) and cut_at_stop("abc", ["x"]) == ("abc", False)
    # streamed in any split, the stop filter gives the text before the first stop string and nothing of a half-seen one
    text, stops = "alpha beta END gamma\n\ndelta", ["END", "\n\n"]
    for cuts in ([3, 11, 12, 13, 20], list(range(1, len(text))), []):
        s, out, hit = StopStream(stops), "", False
        for a, b in zip([0] + cuts, cuts + [len(text)]):
            piece, hit = s.feed(text[a:b])
            out += piece
            if hit:
                break
        assert out + s.flush() == "alpha beta " and hit
    s = StopStream(["END"])
    assert s.feed("the E")[0] == "the " and s.flush() == "E"               # a half-seen stop string is text after all
    assert prompt_opens_thinking("...<|assistant|>\n<think>\n") and not prompt_opens_thinking("<think>\n\n</think>\n\n") and not prompt_opens_thinking("hi")
    assert split_reasoning("<think>why</think>\n\nanswer", False) == ("why", "answer")
    assert split_reasoning("why</think>answer", True) == ("why", "answer") and split_reasoning("<think>why</think>answer", True) == ("why", "answer")
    assert split_reasoning("no block", False) == (None, "no block") and split_reasoning("never closed", True) == ("never closed", "")
    full = "  <think>step 1\nstep 2</think>\nfinal <b>text</b>"
    for n in (1, 2, 3, 7):
        r, th, co = ReasoningStream(False), "", ""
        for i in range(0, len(full), n):
            a, b = r.feed(full[i: i + n])
            th, co = th + a, co + b
        a, b = r.flush()
        assert (th + a, co + b) == ("step 1\nstep 2", "final <b>text</b>")
    al = model_aliases("GLM-5.2-NVFP4", "/models/GLM-5.2-NVFP4/")
    assert {"GLM-5.2-NVFP4", "/models/GLM-5.2-NVFP4"} <= al
    assert resolve_request_model("glm-5.2-nvfp4", "GLM-5.2-NVFP4", al) == "GLM-5.2-NVFP4"
    assert resolve_request_model("/models/glm-5.2-nvfp4", "GLM-5.2-NVFP4", al) == "GLM-5.2-NVFP4"
    assert resolve_request_model("other", "GLM-5.2-NVFP4", al) is None and resolve_request_model(None, "x", al) is None
