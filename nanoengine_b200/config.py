"""Engine configuration: one object, consumed as Python kwargs, from a YAML/JSON file, or from CLI flags.

Parity: reference dlengine/config.py:17-271 (fields) and :273-884 (validator: architecture detection, MLA
forces block size 64 and attention_tp == 1, MTP / PP / HiSparse constraints), :886-897 (world sizes).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, fields
from typing import Any, Dict, Optional

from .models.config import PRESETS, ModelConfig
from .parallel.dist import ParallelSpec


@dataclass
class Config:
    model: str = "tiny-deepseek-v3"          # checkpoint directory, or a preset name with dummy_weight
    hf_overrides: Dict[str, Any] = field(default_factory=dict)
    model_config: Optional[ModelConfig] = None
    dtype: str = "bfloat16"
    device: str = "auto"                     # "auto" | "cuda" | "cpu"
    seed: int = 0
    dummy_weight: bool = False               # random-init weights in the HF layout
    dummy_prefill: bool = False              # decode engines only: prompts arrive as if migrated, their cache rows are whatever the cache holds (no prefill peer)
    # scheduling
    max_num_batched_tokens: int = 16384
    max_num_seqs: int = 16
    max_model_len: Optional[int] = None
    enable_prefix_caching: bool = True
    enable_chunked_prefill: bool = True
    routing_strategy: str = "round_robin"    # round_robin | least_batch | least_cache | affinity
    mode: str = "hybrid"                     # hybrid | prefill | decode
    # parallel layout
    attention_dp: int = 1
    attention_sp: int = 1
    attention_tp: int = 1
    ffn_dp: int = 1
    ffn_ep: int = 1
    ffn_tp: int = 1
    pp: int = 1
    # fp8 block scales: auto (what the checkpoint's quantization_config.scale_fmt says) | fp32 | ue8m0.  ue8m0 rounds every
    # activation scale up to a power of two (and re-quantises weights whose scales are not) so that the tensor cores apply
    # the scales themselves; one setting per process.
    fp8_scale_format: str = "auto"
    # cache
    kv_cache_dtype: str = "auto"             # auto | bfloat16 | fp8
    kvcache_block_size: int = 256
    num_kvcache_blocks: Optional[int] = None  # None = size from free memory
    gpu_memory_utilization: float = 0.9
    num_host_kvcache_blocks: int = 0
    l3_dir: Optional[str] = None
    l3_capacity_blocks: int = 0
    # speculative decoding
    num_speculative_tokens: int = 0
    # sparse attention
    disable_nsa: bool = False
    enable_hisparse: bool = False            # DSA decode engines: latent cache in pinned host memory, top-k rows staged into a hot device buffer
    hisparse_device_buffer_size: int = 4096  # hot rows per sequence and layer (a multiple of 64, at least index_topk + 64)
    hisparse_host_gb: float = 16.0           # pinned host memory for the cold tier when num_kvcache_blocks is not given
    # execution
    enforce_eager: bool = False
    cuda_graph_max_bs: int = 256
    executor_backend: str = "auto"           # auto | inproc | mp | spmd (one engine per torchrun rank)
    use_fused_comm: bool = True              # fused compute+collective kernels when peers are reachable
    peer_timeout_s: float = 120.0            # SPMD: how long the per-step host rendezvous waits for a silent peer
    kernel_status_every: int = 1             # worker: read the kernels' status words every this many steps (0 = never)
    dummy_eplb: bool = False                 # routers deal expert ids evenly over the EP ranks (capacity runs with random-init routers)
    eplb_redundant_experts: int = 0          # extra physical expert slots (whole model); hot experts get replicas in them
    eplb_load_path: Optional[str] = None     # torch file with the expert load [layers, experts] the plan balances (default: uniform)
    # observability
    log_level: str = "INFO"
    status_log_interval_s: float = 10.0      # the engine logs one status line (requests, cache occupancy, throughput) this often; 0 = never
    step_timing: bool = False
    profiler_dir: Optional[str] = None
    # serving / PD
    engine_id: str = "engine-0"
    engine_endpoint: Optional[str] = None    # ZMQ endpoint of the engine process behind the HTTP server (default: a fresh ipc:// path); what a decode engine's pd_peers names
    ctrl_address: Optional[str] = None       # control plane the HTTP server registers with (`nanoengine ctrl`); the gateway discovers engines there
    ctrl_scope: Optional[str] = None         # only gateways started with the same scope take this engine
    served_model_name: Optional[str] = None  # model id in /v1/models and for routing (default: the last component of `model`)
    host: str = "127.0.0.1"
    port: int = 8000
    pd_peers: Dict[str, str] = field(default_factory=dict)   # decode engines: prefill engine id -> ZMQ endpoint of its engine process

    def __post_init__(self):
        self.validate()

    # ---- validation ------------------------------------------------------------------------
    def validate(self) -> None:
        if self.model_config is None:
            if self.model in PRESETS:
                self.model_config = PRESETS[self.model]()
                self.dummy_weight = True
            elif os.path.isdir(self.model):
                self.model_config = ModelConfig.from_pretrained(self.model)
            else:
                raise ValueError(f"model '{self.model}' is neither a checkpoint directory nor a preset {sorted(PRESETS)}")
        elif not os.path.isdir(self.model):
            self.dummy_weight = True          # a model_config without a checkpoint directory can only be random-init
        for k, v in self.hf_overrides.items():
            if not hasattr(self.model_config, k):
                raise ValueError(f"unknown model field in hf_overrides: {k}")
            setattr(self.model_config, k, v)
        mc = self.model_config
        if self.mode not in ("hybrid", "prefill", "decode"):
            raise ValueError("mode must be hybrid, prefill or decode")
        # the reference's spellings (RoundRobin, LeastBatch, LeastCache, Affinity) are taken too
        import re as _re
        self.routing_strategy = _re.sub(r"(?<=[a-z])(?=[A-Z])", "_", str(self.routing_strategy)).lower().replace("-", "_")
        if self.routing_strategy not in ("round_robin", "least_batch", "least_cache", "affinity"):
            raise ValueError(f"unknown routing_strategy {self.routing_strategy}")
        if self.fp8_scale_format not in ("auto", "fp32", "ue8m0"):
            raise ValueError("fp8_scale_format must be auto, fp32 or ue8m0")
        if self.kv_cache_dtype not in ("auto", "bfloat16", "float32", "fp8"):
            raise ValueError("kv_cache_dtype must be auto, bfloat16, float32 or fp8")
        if self.dtype not in ("bfloat16", "float16", "float32"):
            raise ValueError("dtype must be bfloat16, float16 or float32")
        if mc.is_mla:
            # the latent-cache kernels page in units of 64 rows; latent KV is shared by all heads, so head-sharding it buys nothing
            if self.kvcache_block_size == 256:
                self.kvcache_block_size = 64
            if self.attention_tp != 1:
                raise ValueError("MLA architectures run attention data-parallel: attention_tp must be 1")
        elif self.kvcache_block_size == 256:
            self.kvcache_block_size = 64
        if self.attention_sp != 1:
            raise ValueError("attention_sp > 1 is not supported by the runner")
        spec = self.parallel_spec()
        spec.validate()
        if mc.n_routed_experts and mc.n_routed_experts % self.ffn_ep:
            raise ValueError("n_routed_experts must be divisible by ffn_ep")
        if not mc.is_mla and mc.num_key_value_heads % self.attention_tp and self.attention_tp % mc.num_key_value_heads:
            raise ValueError("attention_tp must divide (or be a multiple of) num_key_value_heads")
        if self.num_speculative_tokens < 0:
            raise ValueError("num_speculative_tokens must be >= 0")
        if mc.is_dsv4:
            # the compressor and the window / pooled-row attention are stated in PyTorch ops that read host-side batch facts
            if self.attention_tp != 1 or self.pp != 1 or self.num_speculative_tokens or self.enable_hisparse:
                raise ValueError("DeepSeek-V4 runs with attention_tp = pp = 1, without speculative decoding or the hot / cold tier")
            for r in mc.compress_ratios or []:
                if r and self.kvcache_block_size % r and r % self.kvcache_block_size:
                    raise ValueError("every compression ratio must divide kvcache_block_size or be a multiple of it")
            self.enforce_eager = True
        if self.num_speculative_tokens > 0:
            if mc.num_nextn_predict_layers < 1:
                raise ValueError("speculative decoding needs a model with MTP layers (num_nextn_predict_layers >= 1)")
            if self.pp > 1:
                raise ValueError("speculative decoding is not available with pipeline parallelism")
        if self.pp > 1:
            if self.mode != "prefill":
                raise ValueError("pipeline parallelism is a prefill-only pipeline: set mode='prefill'")
            self.enforce_eager = True
        if self.enable_hisparse and not mc.has_indexer:
            raise ValueError("enable_hisparse needs a DSA model (lightning indexer)")
        if self.enable_hisparse:
            # the hot / cold tier serves decode engines: prompts arrive by PD migration (or are fabricated with dummy_prefill)
            if self.mode != "decode":
                raise ValueError("enable_hisparse needs mode='decode' (prefill engines keep their cache on the device)")
            if self.disable_nsa or self.resolved_kv_dtype() != "fp8" and self.device != "cpu":
                raise ValueError("enable_hisparse needs the DSA indexer (disable_nsa=False) and kv_cache_dtype='fp8'")
            if self.num_speculative_tokens or self.attention_sp != 1 or self.num_host_kvcache_blocks or self.l3_dir:
                raise ValueError("enable_hisparse excludes speculative decoding, attention_sp > 1 and the host-swap / L3 tiers")
            hb = self.hisparse_device_buffer_size
            if hb % 64 or hb < mc.index_topk + 64:
                raise ValueError("hisparse_device_buffer_size must be a multiple of 64 and at least index_topk + 64")
        if self.dummy_prefill and self.mode != "decode":
            raise ValueError("dummy_prefill only applies to a decode engine (mode='decode'): prompts arrive as if migrated, with made-up cache rows")
        if self.eplb_redundant_experts:
            if not mc.n_routed_experts or mc.is_hybrid_gdn:
                raise ValueError("eplb_redundant_experts needs a DeepSeek or Qwen3 MoE model")
            if self.eplb_redundant_experts < 0 or (mc.n_routed_experts + self.eplb_redundant_experts) % self.ffn_ep:
                raise ValueError("experts + eplb_redundant_experts must divide evenly over ffn_ep")
        if mc.num_kv_shared_layers or mc.global_head_dim:
            # cache layers of different head dims are packed at the front of equal slabs: the page movers (host swap, the L3 file
            # tier, PD migration) assume one page size per family and are not offered for this family
            if self.num_host_kvcache_blocks or self.l3_dir or self.mode != "hybrid" or self.attention_tp != 1 or self.pp != 1:
                raise ValueError("models with per-layer head dims run as a hybrid engine with attention_tp = pp = 1 and no host / L3 tier")
        if self.ffn_dp != 1:
            raise ValueError("ffn_dp > 1 is not supported: the FFN view is (ffn_ep, ffn_tp)")
        if self.ffn_tp != 1:
            # FFN tensor parallelism shares the attention-TP group: dense MLPs and every expert are split by intermediate columns
            if mc.is_mla or mc.is_hybrid_gdn:
                raise ValueError("ffn_tp > 1 is offered for the GQA families (Qwen3 dense / MoE) only")
            if self.ffn_tp != self.attention_tp or self.ffn_ep != 1:
                raise ValueError("ffn_tp must equal attention_tp with ffn_ep = 1 (the FFN shards reuse the attention-TP group)")
            for what, size in (("intermediate_size", mc.intermediate_size if not mc.n_routed_experts or mc.first_k_dense_replace else 0),
                               ("moe_intermediate_size", mc.moe_intermediate_size if mc.n_routed_experts else 0)):
                if size and (size % self.ffn_tp or (mc.quant == "fp8" and (size // self.ffn_tp) % 128)):
                    raise ValueError(f"{what} must split evenly over ffn_tp (in 128-wide blocks for fp8 weights)")
        if mc.quant == "nvfp4":
            # packed e2m1 experts: the tensor-core kernel takes K in multiples of 256; experts are sharded over ffn_ep only
            if not mc.n_routed_experts:
                raise ValueError("NVFP4 quantisation applies to routed experts; this model has none")
            if self.ffn_tp != 1:
                raise ValueError("NVFP4 experts are sharded over ffn_ep only (ffn_tp must be 1)")
            width = getattr(mc, "routed_expert_hidden_size", None) or mc.hidden_size
            if width % 256 or mc.moe_intermediate_size % 256:
                raise ValueError("NVFP4 experts need hidden and moe_intermediate sizes in multiples of 256")
        if self.max_model_len is None:
            self.max_model_len = mc.max_position_embeddings
        if self.max_num_seqs < 1 or self.max_num_batched_tokens < 1:
            raise ValueError("max_num_seqs and max_num_batched_tokens must be positive")
        if not (0.0 < self.gpu_memory_utilization <= 1.0):
            raise ValueError("gpu_memory_utilization must be in (0, 1]")

    # ---- projections -----------------------------------------------------------------------
    def parallel_spec(self) -> ParallelSpec:
        return ParallelSpec(self.attention_dp, self.attention_sp, self.attention_tp, self.ffn_dp, self.ffn_ep, self.ffn_tp, self.pp)

    @property
    def world_size(self) -> int:
        return self.parallel_spec().world_size

    def resolved_scale_format(self) -> str:
        if self.fp8_scale_format != "auto":
            return self.fp8_scale_format
        return "ue8m0" if self.model_config.scale_fmt == "ue8m0" else "fp32"

    def resolved_kv_dtype(self) -> str:
        if self.kv_cache_dtype != "auto":
            return self.kv_cache_dtype
        return self.dtype

    def use_nsa(self) -> bool:
        return self.model_config.has_indexer and not self.disable_nsa

    def to_dict(self) -> Dict[str, Any]:
        d = {f.name: getattr(self, f.name) for f in fields(self) if f.name != "model_config"}
        d["model_config"] = self.model_config.to_dict()
        return d

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "Config":
        d = dict(d)
        mc = d.pop("model_config", None)
        known = {f.name for f in fields(cls)}
        bad = set(d) - known
        if bad:
            raise ValueError(f"unknown config fields: {sorted(bad)}")
        if mc is not None:
            d["model_config"] = ModelConfig.from_dict(mc) if isinstance(mc, dict) else mc
        return cls(**d)

    @classmethod
    def from_file(cls, path: str, **overrides) -> "Config":
        with open(path) as f:
            if path.endswith((".yaml", ".yml")):
                import yaml
                d = yaml.safe_load(f) or {}
            else:
                d = json.load(f)
        d.update(overrides)
        return cls.from_dict(d)
