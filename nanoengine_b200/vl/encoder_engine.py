"""The vision encoder as a service of its own: it owns a GPU (or a share of one), the vision transformer and the embedding pool,
answers "encode these images" with slot descriptors, and frees slots when the language model is done with them.

Wire: one ZMQ ROUTER socket, JSON packets {"action": "encode" | "free" | "info", ...} with pixel patches as raw bytes in a
second frame; the language-model engine (or the HTTP front end) is the client.  `VisionSlot` is what travels on with the
request (`RequestIn.vision_slots` carries the slot numbers, the engine keeps the descriptors).

Parity: reference vl/encoder/encoder_engine.py:62-537 (encode :136-167, free :169-179, ZMQ service :280-349, slot metadata
:39-60), vl/server/vl_engine_server.py:75-177 (HTTP wrapper), vl/encoder/encoder_config.py.
"""
from __future__ import annotations

import json
import threading
from dataclasses import asdict, dataclass
from typing import List, Optional

import torch

from .embedding_pool import EmbeddingPool
from .vision import VisionConfig, VisionModel, random_vision_weights


@dataclass
class EncoderConfig:
    model: str = ""                          # checkpoint directory (config.json with vision_config + safetensors); "" = random weights
    vision_config: Optional[VisionConfig] = None
    device: str = "cuda"
    dtype: str = "bfloat16"
    num_slots: int = 64
    max_tokens_per_slot: int = 4096
    max_patches_per_batch: int = 16384       # images are encoded in groups of at most this many patches
    engine_id: str = "encoder-0"
    endpoint: str = ""                       # ZMQ endpoint to serve on ("" = no service thread)
    seed: int = 0


@dataclass
class VisionSlot:
    encoder_engine_id: str
    slot: int
    num_tokens: int
    hidden_size: int
    grid_thw: List[List[int]]


class EncoderEngine:
    def __init__(self, cfg: EncoderConfig):
        self.cfg = cfg
        dt = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}[cfg.dtype]
        vc = cfg.vision_config or (VisionConfig.from_pretrained(cfg.model) if cfg.model else VisionConfig())
        self.vision_config = vc
        self.model = VisionModel(vc, dt, cfg.device)
        if cfg.model:
            from ..models.weights import iterate_safetensors
            n = self.model.load_weights(iterate_safetensors(cfg.model, keep=lambda name: "visual." in name))
            if n == 0:
                raise ValueError(f"no vision tensors (visual.*) under {cfg.model!r}")
        else:
            self.model.load_weights(random_vision_weights(vc, cfg.seed))
        self.pool = EmbeddingPool(cfg.num_slots, cfg.max_tokens_per_slot, vc.out_hidden_size, cfg.device, dt)
        self._lock = threading.Lock()
        self._thread = None
        self._stop = threading.Event()
        self.encoded_images = 0
        if cfg.endpoint:
            self._start_service()

    # ---- direct API ----------------------------------------------------------------------------
    def encode(self, patches: torch.Tensor, grid_thw) -> VisionSlot:
        """patches [T, patch_dim] of one request's images (in order), grid_thw one (frames, height, width) per image.  The
        embeddings of all images go into one slot, image after image."""
        grids = [[int(v) for v in g] for g in (grid_thw.tolist() if isinstance(grid_thw, torch.Tensor) else grid_thw)]
        m2 = self.vision_config.spatial_merge_size ** 2
        counts = [t * h * w for t, h, w in grids]
        if sum(counts) != patches.shape[0]:
            raise ValueError(f"{patches.shape[0]} patches do not match the grids {grids}")
        with self._lock:
            slot = self.pool.allocate(sum(counts) // m2)
            try:
                outs, lo, group, gp = [], 0, [], 0
                for g, c in list(zip(grids, counts)) + [(None, 0)]:
                    if g is None or (group and gp + c > self.cfg.max_patches_per_batch):
                        n = sum(t * h * w for t, h, w in group)
                        outs.append(self.model(patches[lo: lo + n], group))
                        lo, group, gp = lo + n, [], 0
                    if g is not None:
                        group.append(tuple(g)); gp += c
                self.pool.write(slot, torch.cat(outs))
            except Exception:
                self.pool.free(slot)
                raise
            self.encoded_images += len(grids)
        return VisionSlot(self.cfg.engine_id, slot, self.pool.num_tokens(slot), self.vision_config.out_hidden_size, grids)

    def free_slots(self, slots) -> int:
        with self._lock:
            return self.pool.free(slots)

    def engine_info(self, direct: bool = False) -> dict:
        return {"id": self.cfg.engine_id, "kind": "vision_encoder", "pool": self.pool.export(direct), "available_slots": self.pool.available_slots,
                "patch_dim": self.vision_config.patch_dim, "merge": self.vision_config.spatial_merge_size}

    # ---- ZMQ service ----------------------------------------------------------------------------
    def handle_packet(self, header: bytes, payload: bytes = b"") -> bytes:
        try:
            msg = json.loads(header)
            act = msg.get("action")
            if act == "encode":
                dt = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}[msg.get("dtype", "float32")]
                patches = torch.frombuffer(bytearray(payload), dtype=dt).view(-1, self.vision_config.patch_dim)
                return json.dumps({"ok": True, "slot": asdict(self.encode(patches, msg["grid_thw"]))}).encode()
            if act == "free":
                return json.dumps({"ok": True, "freed": self.free_slots(list(msg["slots"]))}).encode()
            if act == "info":
                info = self.engine_info()
                pool = dict(info["pool"])
                t = pool["tensor"]
                pool["tensor"] = t if isinstance(t, dict) else None        # a CPU pool cannot be mapped by another process
                return json.dumps({"ok": True, "info": dict(info, pool=pool)}).encode()
            return json.dumps({"ok": False, "error": f"unknown action {act!r}"}).encode()
        except Exception as e:                      # a bad request must not take the service down
            return json.dumps({"ok": False, "error": f"{type(e).__name__}: {e}"}).encode()

    def _start_service(self) -> None:
        import zmq
        ctx = zmq.Context.instance()
        sock = ctx.socket(zmq.ROUTER)
        sock.bind(self.cfg.endpoint)

        def loop():
            poller = zmq.Poller()
            poller.register(sock, zmq.POLLIN)
            while not self._stop.is_set():
                if not dict(poller.poll(100)):
                    continue
                frames = sock.recv_multipart()
                ident, header = frames[0], frames[1]
                reply = self.handle_packet(header, frames[2] if len(frames) > 2 else b"")
                sock.send_multipart([ident, reply])
            sock.close(0)

        self._thread = threading.Thread(target=loop, daemon=True)
        self._thread.start()

    def shutdown(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)


class EncoderClient:
    """ZMQ client of an `EncoderEngine` service."""

    def __init__(self, endpoint: str, timeout_ms: int = 30000):
        import zmq
        self.sock = zmq.Context.instance().socket(zmq.DEALER)
        self.sock.setsockopt(zmq.RCVTIMEO, timeout_ms)
        self.sock.setsockopt(zmq.LINGER, 0)
        self.sock.connect(endpoint)

    def _call(self, header: dict, payload: bytes = b"") -> dict:
        self.sock.send_multipart([json.dumps(header).encode()] + ([payload] if payload else []))
        rep = json.loads(self.sock.recv_multipart()[-1])
        if not rep.get("ok"):
            raise RuntimeError(rep.get("error", "encoder error"))
        return rep

    def encode(self, patches: torch.Tensor, grid_thw) -> VisionSlot:
        p = patches.contiguous().cpu()
        dt = str(p.dtype).replace("torch.", "")
        raw = p.view(torch.uint8).numpy().tobytes() if p.dtype != torch.bfloat16 else p.view(torch.int16).numpy().tobytes()
        grids = grid_thw.tolist() if isinstance(grid_thw, torch.Tensor) else [list(g) for g in grid_thw]
        return VisionSlot(**self._call({"action": "encode", "grid_thw": grids, "dtype": dt}, raw)["slot"])

    def free(self, slots) -> int:
        return self._call({"action": "free", "slots": list(slots)})["freed"]

    def info(self) -> dict:
        return self._call({"action": "info"})["info"]

    def close(self):
        self.sock.close(0)
