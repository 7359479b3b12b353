"""HTTP front of a vision encoder engine: POST /encode (patches as base64 + grids) -> slot descriptor, POST /free, GET /info,
GET /health.  Parity: reference vl/server/vl_engine_server.py:75-177."""
from __future__ import annotations

import base64

import torch


def build_app(engine):
    from fastapi import FastAPI, HTTPException
    from dataclasses import asdict
    app = FastAPI(title="nanoengine-b200 vision encoder")

    @app.get("/health")
    def health():
        return {"status": "ok", "available_slots": engine.pool.available_slots}

    @app.get("/info")
    def info():
        i = engine.engine_info()
        return dict(i, pool=dict(i["pool"], tensor=i["pool"]["tensor"] if isinstance(i["pool"]["tensor"], dict) else None))

    @app.post("/encode")
    def encode(body: dict):
        try:
            dt = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}[body.get("dtype", "float32")]
            raw = bytearray(base64.b64decode(body["patches"]))
            patches = torch.frombuffer(raw, dtype=dt).view(-1, engine.vision_config.patch_dim)
            return asdict(engine.encode(patches, body["grid_thw"]))
        except (KeyError, ValueError, RuntimeError) as e:
            raise HTTPException(status_code=400, detail=f"{type(e).__name__}: {e}")

    @app.post("/free")
    def free(body: dict):
        return {"freed": engine.free_slots(list(body.get("slots", [])))}

    return app


def serve(cfg, host: str = "0.0.0.0", port: int = 8100):
    import uvicorn
    from ..vl import EncoderEngine
    engine = EncoderEngine(cfg)
    try:
        uvicorn.run(build_app(engine), host=host, port=port, log_level="warning")
    finally:
        engine.shutdown()
