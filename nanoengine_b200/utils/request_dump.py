"""Optional request log for offline replay and debugging: JSON lines appended to a file, or pushed to a Redis stream when
``NANOENGINE_DUMP_REQUESTS_REDIS`` names a server and the `redis` package is importable.
Parity: reference dlengine/metrics/dump.py (env DLENGINE_DUMP_REQUESTS_{REDIS,STREAM,MAXLEN})."""
from __future__ import annotations

import json
import os
import threading
import time
from typing import Any, Dict, Optional


class RequestDumper:
    def __init__(self, path: Optional[str] = None, redis_url: Optional[str] = None, stream: str = "nanoengine:requests", maxlen: int = 100000):
        self.path = path or os.environ.get("NANOENGINE_DUMP_REQUESTS_FILE")
        self.redis_url = redis_url or os.environ.get("NANOENGINE_DUMP_REQUESTS_REDIS") or os.environ.get("DLENGINE_DUMP_REQUESTS_REDIS")
        self.stream = os.environ.get("NANOENGINE_DUMP_REQUESTS_STREAM", stream)
        self.maxlen = int(os.environ.get("NANOENGINE_DUMP_REQUESTS_MAXLEN", maxlen))
        self._lock = threading.Lock()
        self._redis = None
        if self.redis_url:
            try:
                import redis  # type: ignore
                self._redis = redis.Redis.from_url(self.redis_url)
            except Exception:
                self._redis = None

    @property
    def enabled(self) -> bool:
        return bool(self.path) or self._redis is not None

    def dump(self, record: Dict[str, Any]) -> None:
        if not self.enabled:
            return
        rec = dict(record, ts=time.time())
        line = json.dumps(rec, ensure_ascii=False)
        if self._redis is not None:
            try:
                self._redis.xadd(self.stream, {"json": line}, maxlen=self.maxlen, approximate=True)
            except Exception:
                pass
        if self.path:
            with self._lock, open(self.path, "a") as f:
                f.write(line + "\n")
