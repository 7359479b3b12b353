"""Command line: ``python -m nanoengine_b200.server.cli serve <model> [--flag value ...] [--config file.yaml]``,
``... monitor --targets host:port,... --out DIR``, ``... router --port P ...`` (the C++ gateway) and ``... ctrl --port P`` (the control
plane engines register with and the gateway discovers them from).

Every Config field is a flag (``--attention_dp 8 --ffn_ep 8 --num_speculative_tokens 2``); nested per-role overrides for PD
launches use ``--prefill.<field>`` / ``--decode.<field>``.
Parity: reference server/cli.py:51-104 (`dlengine serve`, `dlengine monitor`), dlengine/router.py, examples/disagg.py:28-83."""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
from dataclasses import fields
from typing import Any, Dict, List, Tuple

from ..config import Config


def _coerce(v: str, typ) -> Any:
    t = str(typ)
    if "bool" in t:
        return v.lower() in ("1", "true", "yes", "on")
    if "int" in t and "Dict" not in t:
        return None if v.lower() == "none" else int(v)
    if "float" in t:
        return float(v)
    if "Dict" in t:
        return json.loads(v)
    return None if v.lower() == "none" else v


def parse_config_args(argv: List[str]) -> Tuple[Dict[str, Any], Dict[str, Dict[str, Any]]]:
    """Returns (common overrides, {"prefill": {...}, "decode": {...}})."""
    types = {f.name: f.type for f in fields(Config)}
    common: Dict[str, Any] = {}
    roles: Dict[str, Dict[str, Any]] = {"prefill": {}, "decode": {}}
    i = 0
    while i < len(argv):
        a = argv[i]
        if not a.startswith("--"):
            raise SystemExit(f"unexpected argument {a}")
        key = a[2:].replace("-", "_")
        val = argv[i + 1] if i + 1 < len(argv) and not argv[i + 1].startswith("--") else "true"
        i += 2 if val is not argv[i] and i + 1 < len(argv) and not argv[i + 1].startswith("--") else 1
        target = common
        if "." in key:
            role, key = key.split(".", 1)
            if role not in roles:
                raise SystemExit(f"unknown role prefix {role}")
            target = roles[role]
        if key == "config":
            import yaml
            with open(val) as f:
                target.update(yaml.safe_load(f) or {})
            continue
        if key not in types:
            raise SystemExit(f"unknown flag --{key}")
        target[key] = _coerce(val, types[key])
    return common, roles


def gateway_binary() -> str:
    return os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "_native", "ne-gateway")


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] in ("-h", "--help"):
        print(__doc__)
        return 0
    cmd, rest = argv[0], argv[1:]
    if cmd == "serve":
        if not rest or rest[0].startswith("--"):
            raise SystemExit("usage: serve <model> [--flag value ...]")
        common, _ = parse_config_args(rest[1:])
        tool_format = os.environ.get("NANOENGINE_TOOL_FORMAT", "hermes")
        cfg = Config(model=rest[0], **common)
        from .openai_server import run_server
        run_server(cfg, tool_format=tool_format)
        return 0
    if cmd == "ctrl":
        ap = argparse.ArgumentParser(prog="ctrl", description="control plane: registry of engines for dynamic discovery by the gateway")
        ap.add_argument("--host", default="0.0.0.0")
        ap.add_argument("--port", type=int, default=4479)
        ap.add_argument("--ttl", type=float, default=15.0, help="seconds after the last heartbeat before an engine is dropped")
        a = ap.parse_args(rest)
        from .ctrl import run_ctrl
        run_ctrl(a.host, a.port, a.ttl)
        return 0
    if cmd == "monitor":
        ap = argparse.ArgumentParser(prog="monitor")
        ap.add_argument("--targets", required=True)
        ap.add_argument("--out", default="./monitor")
        ap.add_argument("--prometheus-port", type=int, default=9090)
        ap.add_argument("--grafana-port", type=int, default=3000)
        a = ap.parse_args(rest)
        from ..utils.monitor import write_monitor_stack
        for p in write_monitor_stack(a.out, a.targets.split(","), a.prometheus_port, a.grafana_port):
            print(p)
        return 0
    if cmd == "router":
        from ..build_native import build_gateway
        build_gateway()
        return subprocess.call([gateway_binary(), *rest])
    if cmd == "serve-encoder":
        ap = argparse.ArgumentParser(prog="serve-encoder", description="vision encoder engine: ZMQ service and HTTP front")
        ap.add_argument("--model", default="", help="checkpoint directory with vision_config and visual.* tensors ('' = random weights)")
        ap.add_argument("--device", default="cuda")
        ap.add_argument("--dtype", default="bfloat16")
        ap.add_argument("--num-slots", type=int, default=64)
        ap.add_argument("--max-tokens-per-slot", type=int, default=4096)
        ap.add_argument("--endpoint", default="", help="ZMQ endpoint for the language-model engines, e.g. ipc:///tmp/encoder.sock")
        ap.add_argument("--engine-id", default="encoder-0")
        ap.add_argument("--host", default="0.0.0.0")
        ap.add_argument("--port", type=int, default=8100)
        a = ap.parse_args(rest)
        from ..vl import EncoderConfig
        from .vl_server import serve
        serve(EncoderConfig(model=a.model, device=a.device, dtype=a.dtype, num_slots=a.num_slots, max_tokens_per_slot=a.max_tokens_per_slot,
                            endpoint=a.endpoint, engine_id=a.engine_id), a.host, a.port)
        return 0
    raise SystemExit(f"unknown command {cmd}; expected serve | serve-encoder | monitor | router")


if __name__ == "__main__":
    sys.exit(main())
