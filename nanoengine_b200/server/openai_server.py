"""OpenAI- and Anthropic-compatible HTTP server in front of one engine process.

Endpoints: GET /health, /metrics, /v1/models; POST /v1/chat/completions, /v1/completions, /v1/messages,
/v1/messages/count_tokens, /start_profiler, /stop_profiler, /pd/free.  Streaming uses server-sent events.  Prefill/decode
disaggregation: a request carrying ``kv_transfer_params.do_remote_decode`` runs the prompt only and answers with
``kv_transfer_params = {migration, seq_id, first_token}``; a request carrying ``kv_transfer_params.migration`` resumes
that sequence on this (decode) engine and emits the prefill's first token before the decode tokens.

Parity: reference server/openai_server.py - /health :879, /metrics :883, profiler :912/:938, /v1/models :991,
chat :1007, messages :1373/:1406, completions :1436, /pd/free :1686, sampling params :360-375, submit :435,
submit_migrated :482-532, ctrl registration :1748-1810; server/anthropic_api.py.
"""
from __future__ import annotations

import asyncio
import json
import time
import uuid
from typing import Any, Dict, List, Optional

from fastapi import FastAPI, Request
from fastapi.responses import JSONResponse, PlainTextResponse, StreamingResponse

from .._native import _core as C
from .tokenizer import load_tokenizer
from .text_stream import ReasoningStream, StopStream, cut_at_stop, model_aliases, parse_stop, prompt_opens_thinking, resolve_request_model, split_reasoning
from .tool_parser import StreamingToolParser, parse as parse_tools


def build_sampling_params(body: Dict[str, Any], default_max: int = 256):
    temperature = body.get("temperature")
    temperature = 1.0 if temperature is None else float(temperature)
    max_tokens = body.get("max_completion_tokens") or body.get("max_tokens") or default_max
    return C.SamplingParams(temperature=max(0.0, temperature), max_tokens=max(1, int(max_tokens)),
                            ignore_eos=bool(body.get("ignore_eos", False)),
                            return_completion_logprobs=bool(body.get("logprobs", False)))


def affinity_key(body: Dict[str, Any]) -> int:
    """Requests of one session go to the attention-DP rank that already caches their prefix."""
    key = body.get("session_id") or body.get("user")
    if not key:
        return 0
    import zlib
    return zlib.crc32(str(key).encode()) or 1


def anthropic_to_chat(body: Dict[str, Any]) -> Dict[str, Any]:
    """Anthropic /v1/messages request -> chat-completions request."""
    msgs: List[Dict[str, Any]] = []
    system = body.get("system")
    if system:
        if isinstance(system, list):
            system = "".join(b.get("text", "") for b in system if b.get("type") == "text")
        msgs.append({"role": "system", "content": system})
    for m in body.get("messages", []):
        c = m.get("content")
        if isinstance(c, list):
            text, calls, results = [], [], []
            for b in c:
                t = b.get("type")
                if t == "text":
                    text.append(b.get("text", ""))
                elif t == "tool_use":
                    calls.append({"id": b.get("id"), "type": "function", "function": {"name": b.get("name"), "arguments": json.dumps(b.get("input", {}))}})
                elif t == "tool_result":
                    rc = b.get("content")
                    if isinstance(rc, list):
                        rc = "".join(x.get("text", "") for x in rc if x.get("type") == "text")
                    results.append({"role": "tool", "tool_call_id": b.get("tool_use_id"), "content": rc or ""})
            msgs.extend(results)
            if text or calls:
                mm = {"role": m["role"], "content": "".join(text)}
                if calls:
                    mm["tool_calls"] = calls
                msgs.append(mm)
        else:
            msgs.append({"role": m["role"], "content": c or ""})
    out = {"messages": msgs, "max_tokens": body.get("max_tokens", 1024), "temperature": body.get("temperature"),
           "stream": body.get("stream", False), "model": body.get("model")}
    if body.get("tools"):
        out["tools"] = [{"type": "function", "function": {"name": t["name"], "description": t.get("description", ""),
                                                         "parameters": t.get("input_schema", {})}} for t in body["tools"]]
    return out


def create_app(client, tokenizer, model_name: str, tool_format: str = "hermes", mode: str = "hybrid", default_max_tokens: int = 256,
               model_path: Optional[str] = None, reasoning: bool = True):
    """`model_path`: the checkpoint path, accepted as a request's `model` next to `model_name` (a request that names another
    model gets 404; one that names none is served).  `reasoning`: route `<think>` blocks of chat answers to
    `reasoning_content`."""
    app = FastAPI(title="nanoengine_b200")
    t_start = time.time()
    aliases = model_aliases(model_name, model_path or model_name)

    def _unknown_model(body: Dict[str, Any]):
        req_model = body.get("model")
        if req_model and resolve_request_model(req_model, model_name, aliases) is None:
            return JSONResponse({"error": {"message": f"Model '{req_model}' not found. Use one of: {sorted(aliases)}",
                                           "type": "invalid_request_error", "code": "model_not_found"}}, status_code=404)
        return None

    @app.on_event("startup")
    async def _startup():
        client.start()

    @app.get("/health")
    async def health():
        if client.dead:
            return JSONResponse({"status": "engine backend down"}, status_code=503)
        return {"status": "ok", "uptime_s": time.time() - t_start}

    @app.get("/metrics")
    async def metrics():
        return PlainTextResponse(await client.metrics())

    @app.post("/start_profiler")
    async def start_profiler(req: Request):
        body = await _json(req)
        name = body.get("trace_name", "trace")
        if not name or "/" in name or ".." in name:
            return JSONResponse({"error": "trace_name must be a plain file stem"}, status_code=400)
        return {"started": await client.start_profiler(name)}

    @app.post("/stop_profiler")
    async def stop_profiler():
        return {"traces": await client.stop_profiler()}

    @app.get("/v1/models")
    async def models():
        return {"object": "list", "data": [{"id": model_name, "object": "model", "owned_by": "nanoengine_b200", "created": int(t_start)}]}

    @app.post("/pd/free")
    async def pd_free(req: Request):
        body = await _json(req)
        ids = body.get("seq_ids") or ([body["seq_id"]] if "seq_id" in body else [])
        await client.free([int(i) for i in ids])
        return {"freed": len(ids)}

    async def _json(req: Request) -> Dict[str, Any]:
        try:
            b = await req.json()
            return b if isinstance(b, dict) else {}
        except Exception:
            return {}

    def _prompt_ids(body: Dict[str, Any], chat: bool) -> List[int]:
        if chat:
            return tokenizer.apply_chat_template(body.get("messages", []), tools=body.get("tools"))
        p = body.get("prompt", "")
        if isinstance(p, list) and p and isinstance(p[0], int):
            return list(p)
        if isinstance(p, list):
            p = p[0] if p else ""
        return tokenizer.encode(p)

    async def _start(body: Dict[str, Any], prompt_ids: List[int]):
        """Returns (seq_id, tokens to emit before the engine's own)."""
        kv = body.get("kv_transfer_params") or {}
        if kv.get("migration"):
            sid = await client.submit_migrated(bytes.fromhex(kv["migration"]))
            first = kv.get("first_token")
            return sid, ([int(first)] if first is not None else [])
        sp = build_sampling_params(body, default_max_tokens)
        sid = await client.submit(prompt_ids, sp, affinity_key(body))
        return sid, []

    async def _collect(sid: int, pre: List[int], stops: Optional[List[str]] = None):
        """All tokens of the request.  With stop strings the text is decoded as it arrives and the request is aborted at the
        first one (status FINISHED, the text is cut by the caller)."""
        toks, lps, status = list(pre), [], C.RUNNING
        dec, text = (tokenizer.incremental_decoder(), "") if stops else (None, "")
        if dec is not None:
            for t in pre:
                text += dec.add(t)
        async for o in client.stream(sid):
            toks.extend(o.token_ids)
            lps.extend(o.logprobs)
            status = o.status
            if dec is not None:
                for t in o.token_ids:
                    text += dec.add(t)
                if cut_at_stop(text, stops)[1]:
                    await client.abort(sid)
                    return toks, lps, C.FINISHED
        return toks, lps, status

    def _finish_reason(status: int, n: int, sp_max: int, has_calls: bool) -> str:
        if has_calls:
            return "tool_calls"
        return "length" if n >= sp_max else "stop"

    async def _pd_prefill_reply(sid: int, toks: List[int], prompt_len: int, rid: str, obj: str):
        info = await client.info(export=True)
        blob = None
        for hx in info.get("migrations", []):
            m = C.RequestMigrate.from_bytes(bytes.fromhex(hx))
            if m.seq_id == sid:
                blob = hx
        return {"id": rid, "object": obj, "model": model_name, "choices": [],
                "kv_transfer_params": {"migration": blob, "seq_id": sid, "first_token": toks[-1] if toks else None,
                                       "engine_id": info.get("id")},
                "usage": {"prompt_tokens": prompt_len, "completion_tokens": len(toks), "total_tokens": prompt_len + len(toks)}}

    async def _chat_or_completion(body: Dict[str, Any], chat: bool):
        rid = ("chatcmpl-" if chat else "cmpl-") + uuid.uuid4().hex[:24]
        obj = "chat.completion" if chat else "text_completion"
        bad = _unknown_model(body)
        if bad is not None:
            return bad
        try:
            prompt_ids = _prompt_ids(body, chat)
        except Exception as e:
            return JSONResponse({"error": {"message": f"bad request: {e}", "type": "invalid_request_error"}}, status_code=400)
        if not prompt_ids:
            return JSONResponse({"error": {"message": "empty prompt", "type": "invalid_request_error"}}, status_code=400)
        sp = build_sampling_params(body, default_max_tokens)
        kv = body.get("kv_transfer_params") or {}
        try:
            sid, pre = await _start(body, prompt_ids)
        except Exception as e:
            return JSONResponse({"error": {"message": str(e), "type": "server_error"}}, status_code=503)
        tools = body.get("tools") if body.get("tool_choice") != "none" else None
        stops = parse_stop(body)
        think = chat and reasoning
        think_open = think and prompt_opens_thinking(tokenizer.decode(prompt_ids[-64:]))
        created = int(time.time())

        if kv.get("do_remote_decode") and mode == "prefill":
            toks, _, status = await _collect(sid, pre)
            if status == C.TO_BE_MIGRATED:
                return await _pd_prefill_reply(sid, toks, len(prompt_ids), rid, obj)
            text = tokenizer.decode(toks)      # finished inside prefill (EOS or max_tokens = 1): answer directly
            msg = {"role": "assistant", "content": text}
            return {"id": rid, "object": obj, "created": created, "model": model_name,
                    "choices": [{"index": 0, "message": msg, "finish_reason": "stop"} if chat else {"index": 0, "text": text, "finish_reason": "stop"}],
                    "usage": {"prompt_tokens": len(prompt_ids), "completion_tokens": len(toks), "total_tokens": len(prompt_ids) + len(toks)}}

        if not body.get("stream"):
            try:
                toks, lps, status = await _collect(sid, pre, stops)
            except Exception as e:
                return JSONResponse({"error": {"message": str(e), "type": "server_error"}}, status_code=503)
            text, stopped = cut_at_stop(tokenizer.decode(toks), stops)
            thought = None
            if think:
                thought, text = split_reasoning(text, think_open)
            calls = []
            if chat and tools:
                text, calls = parse_tools(text, tool_format, tools)
            choice: Dict[str, Any] = {"index": 0, "finish_reason": "stop" if stopped and not calls else _finish_reason(status, len(toks), sp.max_tokens, bool(calls))}
            if chat:
                msg: Dict[str, Any] = {"role": "assistant", "content": text or None if calls else text}
                if thought is not None:
                    msg["reasoning_content"] = thought
                if calls:
                    msg["tool_calls"] = [c.to_openai(i) for i, c in enumerate(calls)]
                choice["message"] = msg
            else:
                choice["text"] = text
            if lps:
                choice["logprobs"] = {"token_logprobs": lps, "tokens": [tokenizer.decode([t]) for t in toks[len(pre):]]}
            return {"id": rid, "object": obj, "created": created, "model": model_name, "choices": [choice],
                    "usage": {"prompt_tokens": len(prompt_ids), "completion_tokens": len(toks), "total_tokens": len(prompt_ids) + len(toks)}}

        include_usage = bool((body.get("stream_options") or {}).get("include_usage"))

        async def gen():
            dec = tokenizer.incremental_decoder()
            tp = StreamingToolParser(tool_format, tools) if (chat and tools) else None
            ss = StopStream(stops) if stops else None
            rs = ReasoningStream(think_open) if think else None
            n, ncalls = 0, 0
            chunk_obj = "chat.completion.chunk" if chat else "text_completion"

            def chunk(delta=None, text=None, finish=None):
                ch: Dict[str, Any] = {"index": 0, "finish_reason": finish}
                if chat:
                    ch["delta"] = delta if delta is not None else {}
                else:
                    ch["text"] = text or ""
                return "data: " + json.dumps({"id": rid, "object": chunk_obj, "created": created, "model": model_name, "choices": [ch]}) + "\n\n"

            if chat:
                yield chunk({"role": "assistant", "content": ""})

            def emit(piece: str, last: bool = False):
                """decoded text -> stop strings -> reasoning / content -> tool calls -> chunks"""
                nonlocal ncalls
                outs = []
                if ss is not None:
                    piece = ss.feed(piece)[0] + (ss.flush() if last else "")
                if rs is not None:
                    thought, piece = rs.feed(piece)
                    if last:
                        t2, p2 = rs.flush()
                        thought, piece = thought + t2, piece + p2
                    if thought:
                        outs.append(chunk({"reasoning_content": thought}))
                if tp is not None:
                    piece, calls = tp.feed(piece)
                    for c in calls:
                        outs.append(chunk({"tool_calls": [c.to_openai(ncalls)]}))
                        ncalls += 1
                if piece:
                    outs.append(chunk({"content": piece}) if chat else chunk(text=piece))
                return outs

            try:
                for t in pre:
                    n += 1
                    for s in emit(dec.add(t)):
                        yield s
                async for o in client.stream(sid):
                    for t in o.token_ids:
                        if ss is not None and ss.hit:
                            break
                        n += 1
                        for s in emit(dec.add(t)):
                            yield s
                    if ss is not None and ss.hit:
                        await client.abort(sid)
                        break
                for s in emit(dec.flush() or "", last=True):
                    yield s
                tail = ""
                if tp is not None:
                    rest, calls = tp.flush()
                    tail = (tail or "") + rest if not calls else tail
                    for c in calls:
                        yield chunk({"tool_calls": [c.to_openai(ncalls)]})
                        ncalls += 1
                if tail:
                    yield chunk({"content": tail}) if chat else chunk(text=tail)
                yield chunk(finish="stop" if (ss is not None and ss.hit and not ncalls) else _finish_reason(C.FINISHED, n, sp.max_tokens, ncalls > 0))
                if include_usage:
                    yield "data: " + json.dumps({"id": rid, "object": chunk_obj, "created": created, "model": model_name, "choices": [],
                                                 "usage": {"prompt_tokens": len(prompt_ids), "completion_tokens": n, "total_tokens": len(prompt_ids) + n}}) + "\n\n"
            except asyncio.CancelledError:
                await client.abort(sid)      # client went away: stop generating for it
                raise
            except Exception as e:
                yield "data: " + json.dumps({"error": {"message": str(e), "type": "server_error"}}) + "\n\n"
            yield "data: [DONE]\n\n"

        return StreamingResponse(gen(), media_type="text/event-stream")

    @app.post("/v1/chat/completions")
    async def chat_completions(req: Request):
        return await _chat_or_completion(await _json(req), True)

    @app.post("/v1/completions")
    async def completions(req: Request):
        return await _chat_or_completion(await _json(req), False)

    @app.post("/v1/messages/count_tokens")
    async def count_tokens(req: Request):
        body = anthropic_to_chat(await _json(req))
        return {"input_tokens": len(tokenizer.apply_chat_template(body["messages"], tools=body.get("tools")))}

    @app.post("/v1/messages")
    async def messages(req: Request):
        raw = await _json(req)
        bad = _unknown_model(raw)
        if bad is not None:
            return bad
        body = anthropic_to_chat(raw)
        mid = "msg_" + uuid.uuid4().hex[:24]
        prompt_ids = tokenizer.apply_chat_template(body["messages"], tools=body.get("tools"))
        sp = build_sampling_params(body, 1024)
        sid = await client.submit(prompt_ids, sp, affinity_key(raw))
        tools = body.get("tools")
        stops = parse_stop({"stop": raw.get("stop_sequences")})
        think_open = reasoning and prompt_opens_thinking(tokenizer.decode(prompt_ids[-64:]))

        def which_stop(text: str):
            """The stop sequence that ends `text` first, if any."""
            hits = [(text.find(s_), s_) for s_ in stops if s_ in text]
            return min(hits)[1] if hits else None

        if not body.get("stream"):
            toks, _, status = await _collect(sid, [], stops)
            full = tokenizer.decode(toks)
            matched = which_stop(full)
            text = cut_at_stop(full, stops)[0]
            thought = None
            if reasoning:
                thought, text = split_reasoning(text, think_open)
            calls = []
            if tools:
                text, calls = parse_tools(text, tool_format, tools)
            content: List[Dict[str, Any]] = []
            if thought:
                content.append({"type": "thinking", "thinking": thought, "signature": ""})
            if text:
                content.append({"type": "text", "text": text})
            for c in calls:
                content.append({"type": "tool_use", "id": c.id.replace("call_", "toolu_"), "name": c.name, "input": c.arguments})
            stop = "tool_use" if calls else "stop_sequence" if matched else ("max_tokens" if len(toks) >= sp.max_tokens else "end_turn")
            return {"id": mid, "type": "message", "role": "assistant", "model": model_name, "content": content, "stop_reason": stop,
                    "stop_sequence": matched if stop == "stop_sequence" else None,
                    "usage": {"input_tokens": len(prompt_ids), "output_tokens": len(toks)}}

        async def gen():
            def ev(name, data):
                return f"event: {name}\ndata: {json.dumps(data)}\n\n"
            yield ev("message_start", {"type": "message_start", "message": {"id": mid, "type": "message", "role": "assistant", "model": model_name,
                                                                           "content": [], "stop_reason": None,
                                                                           "usage": {"input_tokens": len(prompt_ids), "output_tokens": 0}}})
            dec = tokenizer.incremental_decoder()
            tp = StreamingToolParser(tool_format, tools) if tools else None
            ss = StopStream(stops) if stops else None
            rs = ReasoningStream(think_open) if reasoning else None
            n, calls_all, seen = 0, [], ""
            block = {"index": -1, "kind": None}          # the content block that is open

            def to_block(kind: str):
                """Events that close the open block (if it is of another kind) and open one of `kind`."""
                out = []
                if block["kind"] == kind:
                    return out
                if block["kind"] is not None:
                    out.append(ev("content_block_stop", {"type": "content_block_stop", "index": block["index"]}))
                block["index"] += 1
                block["kind"] = kind
                start = {"type": "thinking", "thinking": ""} if kind == "thinking" else {"type": "text", "text": ""}
                out.append(ev("content_block_start", {"type": "content_block_start", "index": block["index"], "content_block": start}))
                return out

            def emit(piece: str, last: bool = False):
                nonlocal seen
                outs = []
                seen += piece
                if ss is not None:
                    piece = ss.feed(piece)[0] + (ss.flush() if last else "")
                thought = ""
                if rs is not None:
                    thought, piece = rs.feed(piece)
                    if last:
                        t2, p2 = rs.flush()
                        thought, piece = thought + t2, piece + p2
                if thought:
                    outs += to_block("thinking")
                    outs.append(ev("content_block_delta", {"type": "content_block_delta", "index": block["index"],
                                                           "delta": {"type": "thinking_delta", "thinking": thought}}))
                if tp is not None:
                    piece, calls = tp.feed(piece)
                    calls_all.extend(calls)
                    if last:
                        rest, calls = tp.flush()
                        calls_all.extend(calls)
                        piece += "" if calls else rest
                if piece:
                    outs += to_block("text")
                    outs.append(ev("content_block_delta", {"type": "content_block_delta", "index": block["index"], "delta": {"type": "text_delta", "text": piece}}))
                return outs

            try:
                async for o in client.stream(sid):
                    for t in o.token_ids:
                        if ss is not None and ss.hit:
                            break
                        n += 1
                        for e in emit(dec.add(t)):
                            yield e
                    if ss is not None and ss.hit:
                        await client.abort(sid)
                        break
            except asyncio.CancelledError:
                await client.abort(sid)
                raise
            for e in emit(dec.flush() or "", last=True):
                yield e
            if block["kind"] is None:                     # an answer without any text still carries one (empty) text block
                for e in to_block("text"):
                    yield e
            yield ev("content_block_stop", {"type": "content_block_stop", "index": block["index"]})
            base = block["index"] + 1
            for i, c in enumerate(calls_all):
                yield ev("content_block_start", {"type": "content_block_start", "index": base + i,
                                                 "content_block": {"type": "tool_use", "id": c.id.replace("call_", "toolu_"), "name": c.name, "input": {}}})
                yield ev("content_block_delta", {"type": "content_block_delta", "index": base + i,
                                                 "delta": {"type": "input_json_delta", "partial_json": json.dumps(c.arguments)}})
                yield ev("content_block_stop", {"type": "content_block_stop", "index": base + i})
            matched = which_stop(seen) if (ss is not None and ss.hit) else None
            if matched and not calls_all:
                yield ev("message_delta", {"type": "message_delta", "delta": {"stop_reason": "stop_sequence", "stop_sequence": matched}, "usage": {"output_tokens": n}})
                yield ev("message_stop", {"type": "message_stop"})
                return
            stop = "tool_use" if calls_all else ("max_tokens" if n >= sp.max_tokens else "end_turn")
            yield ev("message_delta", {"type": "message_delta", "delta": {"stop_reason": stop, "stop_sequence": None}, "usage": {"output_tokens": n}})
            yield ev("message_stop", {"type": "message_stop"})

        return StreamingResponse(gen(), media_type="text/event-stream")

    return app


def run_server(config, host: Optional[str] = None, port: Optional[int] = None, tool_format: str = "hermes"):
    """Spawn the engine process, then serve HTTP in this one."""
    import uvicorn
    from .engine_server import EngineClient, spawn_backend
    proc, endpoint = spawn_backend(config, endpoint=getattr(config, "engine_endpoint", None))
    client = EngineClient(endpoint, proc)
    tok = load_tokenizer(config.model, config.model_config.vocab_size)
    import os
    name = getattr(config, "served_model_name", None) or os.path.basename(str(config.model).rstrip("/")) or str(config.model)
    app = create_app(client, tok, model_name=name, tool_format=tool_format, mode=config.mode, model_path=str(config.model),
                     reasoning=os.environ.get("NANOENGINE_REASONING", "1") != "0")
    ctrl = None
    if config.ctrl_address:
        from .ctrl import register_with_ctrl
        ctrl = register_with_ctrl(config, host or config.host, port or config.port, name)
        if ctrl is None:
            print(f"control plane {config.ctrl_address} unreachable: this engine will not be discovered", flush=True)
    try:
        uvicorn.run(app, host=host or config.host, port=port or config.port, log_level=config.log_level.lower())
    finally:
        if ctrl is not None:
            ctrl.stop()
        if proc.is_alive():
            proc.terminate()
