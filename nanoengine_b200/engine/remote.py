"""An LLM whose engine lives in a child process, driven over a pipe.  Lets a prefill engine and a decode engine (each with
its own workers and process groups) coexist under one controlling script.  Parity: reference engine/llm_component.py:20-29
(`as_remote` turns the component into a Ray actor); here the actor is a spawned process."""
from __future__ import annotations

import multiprocessing as mp
import traceback
from typing import Any


def _serve(config_dict, cls_name, conn):
    try:
        from ..config import Config
        from . import llm_component
        obj = getattr(llm_component, cls_name)(Config.from_dict(config_dict))
        conn.send(("ready", None))
        while True:
            msg = conn.recv()
            if msg is None:
                break
            name, args, kw = msg
            try:
                conn.send(("ok", getattr(obj, name)(*args, **kw)))
            except Exception as e:
                conn.send(("err", f"{type(e).__name__}: {e}\n{traceback.format_exc()}"))
        obj.shutdown()
    except Exception as e:
        conn.send(("err", f"remote engine failed to start: {e}\n{traceback.format_exc()}"))


class RemoteLLM:
    def __init__(self, config, cls_name: str = "LLM"):
        ctx = mp.get_context("spawn")
        self._conn, child = ctx.Pipe()
        self._proc = ctx.Process(target=_serve, args=(config.to_dict(), cls_name, child), daemon=True)
        self._proc.start()
        status, val = self._conn.recv()
        if status != "ready":
            raise RuntimeError(val)

    def __getattr__(self, name: str):
        if name.startswith("_"):
            raise AttributeError(name)

        def call(*args, **kw) -> Any:
            if not self._proc.is_alive():
                raise RuntimeError(f"remote engine process exited with code {self._proc.exitcode}")
            self._conn.send((name, args, kw))
            status, val = self._conn.recv()
            if status == "err":
                raise RuntimeError(val)
            return val

        return call

    def shutdown(self):
        try:
            if self._proc.is_alive():
                self._conn.send(None)
            self._proc.join(timeout=20)
        finally:
            if self._proc.is_alive():
                self._proc.terminate()
