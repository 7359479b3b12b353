"""Vision-language side: the vision transformer, the embedding pool it fills and the encoder engine that serves them.
Parity: reference dlengine/vl/ (vision/encoder.py, encoder/encoder_engine.py, server/vl_engine_server.py) and
runtime/context/cache/emb.py."""
from .embedding_pool import EmbeddingPool
from .encoder_engine import EncoderConfig, EncoderEngine
from .vision import VisionConfig, VisionModel

__all__ = ["EmbeddingPool", "EncoderConfig", "EncoderEngine", "VisionConfig", "VisionModel"]
