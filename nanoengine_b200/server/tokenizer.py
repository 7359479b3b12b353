"""Tokenizer access for the servers: the checkpoint's HF tokenizer when there is one, a byte-level stand-in otherwise
(synthetic-weight runs and tests have no vocabulary files).  Both expose encode / decode / apply_chat_template and an
incremental decoder that never emits half a UTF-8 character.  Parity: reference models/trait.py:173-178."""
from __future__ import annotations

import json
import os
from typing import Any, Dict, List, Optional


class IncrementalDecoder:
    def __init__(self, tok):
        self.tok = tok
        self.ids: List[int] = []
        self.sent = 0

    def add(self, token_id: int) -> str:
        self.ids.append(int(token_id))
        text = self.tok.decode(self.ids)
        if text.endswith("�"):          # incomplete multi-byte character: wait for the rest
            return ""
        out = text[self.sent:]
        self.sent = len(text)
        if len(self.ids) > 64:               # keep the re-decoded window short
            self.ids = self.ids[-8:]
            self.sent = len(self.tok.decode(self.ids))
        return out

    def flush(self) -> str:
        text = self.tok.decode(self.ids)
        out = text[self.sent:]
        self.sent = len(text)
        return out.replace("�", "")


class ByteTokenizer:
    """ids 0..255 are bytes; 256 = BOS, 257 = EOS, 258.. role markers.  Ids beyond the byte range decode to nothing."""

    def __init__(self, vocab_size: int = 1024):
        self.vocab_size = vocab_size
        self.bos_token_id, self.eos_token_id = 256, 257

    def encode(self, text: str) -> List[int]:
        return list(text.encode("utf-8"))

    def decode(self, ids: List[int]) -> str:
        return bytes(i for i in ids if 0 <= i < 256).decode("utf-8", errors="replace")

    def apply_chat_template(self, messages: List[Dict[str, Any]], tools: Optional[List[dict]] = None) -> List[int]:
        parts = []
        if tools:
            parts.append("<tools>" + json.dumps(tools) + "</tools>\n")
        for m in messages:
            c = m.get("content")
            if isinstance(c, list):
                c = "".join(b.get("text", "") for b in c if isinstance(b, dict))
            parts.append(f"<|{m.get('role', 'user')}|>{c or ''}\n")
        parts.append("<|assistant|>")
        return self.encode("".join(parts))

    def incremental_decoder(self) -> IncrementalDecoder:
        return IncrementalDecoder(self)


class HFTokenizer:
    def __init__(self, path: str):
        from transformers import AutoTokenizer
        self.tok = AutoTokenizer.from_pretrained(path, trust_remote_code=False)
        self.eos_token_id = self.tok.eos_token_id
        self.vocab_size = len(self.tok)

    def encode(self, text: str) -> List[int]:
        return self.tok.encode(text, add_special_tokens=False)

    def decode(self, ids: List[int]) -> str:
        return self.tok.decode(ids, skip_special_tokens=True)

    def apply_chat_template(self, messages, tools=None) -> List[int]:
        out = self.tok.apply_chat_template(messages, tools=tools, add_generation_prompt=True, tokenize=True)
        return list(out["input_ids"] if isinstance(out, dict) else out)

    def incremental_decoder(self) -> IncrementalDecoder:
        return IncrementalDecoder(self)


def load_tokenizer(model: str, vocab_size: int = 1024):
    if os.path.isdir(model) and any(os.path.exists(os.path.join(model, f)) for f in ("tokenizer.json", "tokenizer_config.json", "tokenizer.model")):
        return HFTokenizer(model)
    return ByteTokenizer(vocab_size)
