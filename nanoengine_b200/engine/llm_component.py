"""User-facing engine handles.

``LLM`` is the offline API (add requests, drive steps, collect outputs); ``LLMComponent`` adds what serving
and PD disaggregation need: engine info for peers, control-plane registration with heartbeat, and
"free" notifications back to the prefill engine.

Parity: reference engine/llm_component.py (LLM / LLMComponent, as_remote :20-29, engine info :155-233,
send_free_sequences :355-423, control-plane registration + heartbeat :449-573) and examples/disagg.py:85-160.
"""
from __future__ import annotations

import json
import threading
import time
import urllib.request
from typing import Dict, Iterable, Iterator, List, Optional

from .._native import _core as C
from ..config import Config
from .llm_engine import LLMEngine


class LLM:
    def __init__(self, config: Optional[Config] = None, **kwargs):
        self.config = config if config is not None else Config(**kwargs)
        self.engine = LLMEngine(self.config)

    # -- reference-compatible surface
    def add_request_payload(self, payload: bytes) -> int:
        return self.engine.add_request_payload(payload)

    def add_request(self, prompt_token_ids: List[int], sampling_params=None, seq_id=None, affinity_key: int = 0) -> int:
        return self.engine.add_request(prompt_token_ids, sampling_params, seq_id, affinity_key)

    def step(self):
        return self.engine.step()

    def is_finished(self) -> bool:
        return self.engine.is_finished()

    def abort(self, seq_id: int) -> bool:
        return self.engine.abort(seq_id)

    def generate(self, prompts: Optional[List[List[int]]] = None, sampling_params=None, return_serialized: bool = False):
        """Run everything queued (plus `prompts`) to completion.

        Hybrid / decode engines return ``[{"seq_id", "token_ids", ...}]`` in completion order.  A prefill engine
        with ``return_serialized=True`` returns the RequestMigrate blobs to feed a decode engine.
        """
        from ..offline import generate as _generate
        if prompts is not None:
            sps = sampling_params if isinstance(sampling_params, (list, tuple)) else [sampling_params] * len(prompts)
            for p, sp in zip(prompts, sps):
                self.add_request(p, sp)
        outs = list(_generate(self))
        if return_serialized:
            return [m.to_bytes() for m in self.engine.export_to_be_migrated()]
        return outs

    def free_to_be_migrated_ids(self, ids: Iterable[int]) -> int:
        return self.engine.free_to_be_migrated_ids(ids)

    def start_profiler(self, trace_name="trace"):
        return self.engine.start_profiler(trace_name)

    def stop_profiler(self):
        return self.engine.stop_profiler()

    def update_weights(self, src):
        return self.engine.update_weights(src)

    def export_weights(self, direct: bool = False):
        return self.engine.export_weights(direct)

    def pull_weights(self, per_worker):
        return self.engine.pull_weights(per_worker)

    def metrics(self) -> str:
        return self.engine.metrics_prometheus()

    def shutdown(self):
        self.engine.shutdown()

    @classmethod
    def as_remote(cls, config: Config):
        """A handle whose engine lives in a child process (so a prefill and a decode engine can coexist)."""
        from .remote import RemoteLLM
        return RemoteLLM(config, cls.__name__)


class LLMComponent(LLM):
    """LLM + peer-facing duties (engine info, registration / heartbeat, PD free notifications)."""

    def __init__(self, config: Optional[Config] = None, **kwargs):
        super().__init__(config, **kwargs)
        self._hb_thread = None
        self._hb_stop = threading.Event()
        self.registered = False
        if self.config.ctrl_address:
            self.register_with_ctrl()

    def engine_info(self) -> Dict:
        return self.engine.engine_info()

    # -- control plane: POST {ctrl}/register_entity every few seconds; a ctrl that lost state gets a fresh registration
    def _post(self, path: str, body: Dict, timeout=2.0) -> Optional[Dict]:
        url = self.config.ctrl_address.rstrip("/") + path
        req = urllib.request.Request(url, json.dumps(body).encode(), {"Content-Type": "application/json"})
        try:
            with urllib.request.urlopen(req, timeout=timeout) as r:
                return json.loads(r.read() or b"{}")
        except Exception:
            return None

    def register_with_ctrl(self, interval_s: float = 2.0) -> None:
        info = self.engine_info()
        self.registered = self._post("/register_entity", info) is not None

        def beat():
            while not self._hb_stop.wait(interval_s):
                r = self._post("/heartbeat", {"id": info["id"], "ts": time.time()})
                if r is None or r.get("unknown"):
                    self.registered = self._post("/register_entity", info) is not None
                else:
                    self.registered = True

        self._hb_thread = threading.Thread(target=beat, daemon=True)
        self._hb_thread.start()

    def send_free_sequences(self, prefill_url: str, seq_ids: List[int]) -> bool:
        req = urllib.request.Request(prefill_url.rstrip("/") + "/pd/free", json.dumps({"seq_ids": list(seq_ids)}).encode(),
                                     {"Content-Type": "application/json"})
        try:
            with urllib.request.urlopen(req, timeout=5.0):
                return True
        except Exception:
            return False

    def shutdown(self):
        self._hb_stop.set()
        super().shutdown()
