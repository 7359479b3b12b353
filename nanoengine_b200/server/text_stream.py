"""Serving-layer text filters: stop strings, reasoning ("thinking") blocks, and the `model` names a server answers to.

The engine stops on token ids only; stop STRINGS are cut here, on the decoded text, and the request is aborted once one is
seen.  Reasoning models open their answer with a `<think>` block (or the chat template opens it for them): that text goes to
`reasoning_content`, the rest to `content`.

Parity: reference server/openai_server.py - model aliases :198-234, `_prompt_opens_thinking` :299-318, `_parse_stop` :377-393,
the hold-back logic of `stream_text` :662-800.
"""
from __future__ import annotations

import os
from typing import Iterable, List, Optional, Set, Tuple

THINK_PAIRS = (("<think>", "</think>"), ("<|open|>think<|sep|>", "<|close|>think<|sep|>"))


def parse_stop(body: dict) -> List[str]:
    raw = body.get("stop")
    if isinstance(raw, str):
        raw = [raw]
    return [s for s in raw if isinstance(s, str) and s] if isinstance(raw, list) else []


def cut_at_stop(text: str, stops: Iterable[str]) -> Tuple[str, bool]:
    """Text before the earliest stop string, and whether one was found."""
    at = min((i for i in (text.find(s) for s in stops) if i >= 0), default=-1)
    return (text[:at], True) if at >= 0 else (text, False)


def _held_suffix(text: str, markers: Iterable[str]) -> int:
    """Length of the longest suffix of `text` that is a proper prefix of one of `markers` (text that may yet become one)."""
    best = 0
    for m in markers:
        for k in range(min(len(m) - 1, len(text)), best, -1):
            if text.endswith(m[:k]):
                best = k
                break
    return best


class StopStream:
    """Incremental `cut_at_stop`: feed decoded pieces, get the text that can no longer be part of a stop string."""

    def __init__(self, stops: List[str]):
        self.stops, self.buf, self.hit = list(stops), "", False

    def feed(self, piece: str) -> Tuple[str, bool]:
        if self.hit or not self.stops:
            return ("" if self.hit else piece), self.hit
        self.buf += piece
        out, self.hit = cut_at_stop(self.buf, self.stops)
        if self.hit:
            self.buf = ""
            return out, True
        keep = _held_suffix(self.buf, self.stops)
        out, self.buf = self.buf[: len(self.buf) - keep], self.buf[len(self.buf) - keep:]
        return out, False

    def flush(self) -> str:
        out, self.buf = ("" if self.hit else self.buf), ""
        return out


def prompt_opens_thinking(prompt_tail: str) -> bool:
    """True when the rendered prompt ends inside a thinking block (an opener with no closer after it)."""
    for opener, closer in THINK_PAIRS:
        i = prompt_tail.rfind(opener)
        if i >= 0 and prompt_tail.rfind(closer) < i:
            return True
    return False


def split_reasoning(text: str, opened: bool) -> Tuple[Optional[str], str]:
    """(reasoning, content) of a finished answer.  `opened`: the prompt already opened the block."""
    r = ReasoningStream(opened)
    a, b = r.feed(text)
    a2, b2 = r.flush()
    reasoning, content = a + a2, b + b2
    return (reasoning if (reasoning or r.saw_block) else None), content


class ReasoningStream:
    """Routes streamed text to (reasoning, content).  Before the first visible character it decides whether the answer opens
    a thinking block; inside one it holds back whatever may be the start of the closing marker."""

    def __init__(self, opened: bool):
        self.opened = opened
        self.state = "think" if opened else "start"        # start -> think | content ; think -> content
        self.closer = THINK_PAIRS[0][1]
        self.buf = ""
        self.saw_block = opened
        self.after_close = False

    def feed(self, piece: str) -> Tuple[str, str]:
        self.buf += piece
        reasoning = content = ""
        while True:
            if self.state == "start":
                t = self.buf.lstrip()
                hit = next(((o, c) for o, c in THINK_PAIRS if t.startswith(o)), None)
                if hit:
                    self.state, self.closer, self.saw_block = "think", hit[1], True
                    self.buf = t[len(hit[0]):]
                    continue
                if t and not any(o.startswith(t) for o, _ in THINK_PAIRS):
                    self.state = "content"
                    continue
                return reasoning, content                    # nothing visible yet, or a possible opener: wait
            if self.state == "think":
                if self.opened:                              # a model that repeats the opener the template already wrote
                    t = self.buf.lstrip()
                    rep = next((o for o, _ in THINK_PAIRS if t.startswith(o)), None)
                    if rep:
                        self.buf = t[len(rep):]
                    elif t and any(o.startswith(t) for o, _ in THINK_PAIRS):
                        return reasoning, content
                    self.opened = False
                closers = [c for _, c in THINK_PAIRS]
                at = min((i for i in (self.buf.find(c) for c in closers) if i >= 0), default=-1)
                if at >= 0:
                    c = next(c for c in closers if self.buf.startswith(c, at))
                    reasoning += self.buf[:at]
                    self.buf = self.buf[at + len(c):]
                    self.state, self.after_close = "content", True
                    continue
                keep = _held_suffix(self.buf, closers)
                reasoning += self.buf[: len(self.buf) - keep]
                self.buf = self.buf[len(self.buf) - keep:]
                return reasoning, content
            if self.after_close:                              # the line breaks between the block and the answer belong to neither
                self.buf = self.buf.lstrip("\n")
                self.after_close = not self.buf
            content += self.buf
            self.buf = ""
            return reasoning, content

    def flush(self) -> Tuple[str, str]:
        out, self.buf = self.buf, ""
        return (out, "") if self.state == "think" else ("", out)


def model_aliases(served_name: str, model_path: str) -> Set[str]:
    """Every `model` value a request may carry for this server: the served name, the checkpoint path as given, expanded and
    resolved, and its last component."""
    path = str(model_path).rstrip("/")
    out = {served_name}
    for raw in (path, os.path.expanduser(path)):
        if raw:
            out.add(raw.rstrip("/"))
            try:
                out.add(os.path.realpath(raw).rstrip("/"))
            except OSError:
                pass
    if path.split("/")[-1]:
        out.add(path.split("/")[-1])
    return out


def resolve_request_model(requested: Optional[str], served_name: str, aliases: Set[str]) -> Optional[str]:
    """The served name when `requested` is one of the aliases (case-insensitively, also after ~ expansion and symlink
    resolution), else None."""
    if not requested:
        return None
    lower = {a.lower() for a in aliases}
    key = str(requested).strip().rstrip("/")
    cands = [key, os.path.expanduser(key).rstrip("/")]
    try:
        cands.append(os.path.realpath(os.path.expanduser(key)).rstrip("/"))
    except OSError:
        pass
    return served_name if any(c in aliases or c.lower() in lower for c in cands) else None
