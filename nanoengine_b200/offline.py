"""Offline generation loop: drive ``engine.step()`` until every request has finished and yield each
sequence's output as it completes.  Parity: reference offline/generate.py:8-112."""
from __future__ import annotations

from typing import Dict, Iterator, List

from ._native import _core as C


def generate(llm, max_steps: int = 1 << 30) -> Iterator[Dict]:
    acc: Dict[int, List[int]] = {}
    lps: Dict[int, List[float]] = {}
    steps = 0
    while not llm.is_finished() and steps < max_steps:
        steps += 1
        for so in llm.step():
            acc.setdefault(so.seq_id, []).extend(so.token_ids)
            if so.logprobs:
                lps.setdefault(so.seq_id, []).extend(so.logprobs)
            if so.status in (C.FINISHED, C.TO_BE_MIGRATED):
                out = {"seq_id": so.seq_id, "token_ids": acc.pop(so.seq_id, []), "status": so.status}
                if so.seq_id in lps:
                    out["logprobs"] = lps.pop(so.seq_id)
                yield out
