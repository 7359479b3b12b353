"""Model architecture description shared by every model family, plus shape presets.

The fields follow the HF ``config.json`` names of the DeepSeek-V3 / Qwen3-MoE families so a
checkpoint directory can be read directly (the reference resolves the same fields through
``transformers.AutoConfig`` in dlengine/config.py:273-884).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, fields
from typing import Any, Dict, List, Optional


@dataclass
class ModelConfig:
    architecture: str = "DeepseekV3ForCausalLM"
    vocab_size: int = 129280
    hidden_size: int = 7168
    num_hidden_layers: int = 61
    num_attention_heads: int = 128
    num_key_value_heads: int = 128
    head_dim: int = 128                      # GQA families
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    rope_scaling: Optional[Dict[str, Any]] = None
    max_position_embeddings: int = 163840
    tie_word_embeddings: bool = False
    # dense MLP
    intermediate_size: int = 18432
    # MLA
    q_lora_rank: Optional[int] = 1536
    kv_lora_rank: int = 512
    qk_nope_head_dim: int = 128
    qk_rope_head_dim: int = 64
    v_head_dim: int = 128
    # MoE
    n_routed_experts: int = 256
    n_shared_experts: int = 1
    num_experts_per_tok: int = 8
    moe_intermediate_size: int = 2048
    first_k_dense_replace: int = 3
    moe_layer_freq: int = 1
    n_group: int = 8
    topk_group: int = 4
    norm_topk_prob: bool = True
    routed_scaling_factor: float = 2.5
    scoring_func: str = "sigmoid"            # "sigmoid" (DeepSeek-V3) or "softmax" (Qwen3-MoE, V2)
    topk_method: str = "noaux_tc"
    # GQA extras (Qwen3)
    qk_norm: bool = False
    attention_bias: bool = False
    # DSA lightning indexer (DeepSeek-V3.2)
    index_n_heads: int = 0
    index_head_dim: int = 128
    index_topk: int = 2048
    # hybrid linear attention (Qwen3.5): gated delta-net layers between full-attention layers
    layer_types: Optional[List[str]] = None  # per layer "linear_attention" | "full_attention"; None = all full attention
    full_attention_interval: int = 0         # used when layer_types is absent: every n-th layer is full attention
    linear_num_key_heads: int = 0
    linear_num_value_heads: int = 0
    linear_key_head_dim: int = 128
    linear_value_head_dim: int = 128
    linear_conv_kernel_dim: int = 4
    partial_rotary_factor: float = 1.0       # fraction of each head that is rotated
    attn_output_gate: bool = False           # q projection carries a per-head sigmoid gate for the attention output
    norm_unit_offset: bool = False           # RMSNorm weights are stored as the deviation from one
    shared_expert_intermediate_size: int = 0 # Qwen3.5-MoE: one always-on expert behind a sigmoid gate
    # Kimi delta attention (GLM5-next, Kimi-K3): the linear layers decay per key channel and sit between MLA layers
    linear_kind: str = "gdn"                 # "gdn" (scalar decay per head) | "kda" (decay per key channel)
    kda_gate_lower_bound: Optional[float] = None   # L < 0: log-decay = L * sigmoid(exp(A) (g + bias)); None: -exp(A) softplus(g + bias)
    mla_output_gate: bool = False            # MLA layers carry g_proj: the attention output is multiplied by sigmoid(g_proj(x))
    mla_skip_rope: bool = False              # MLA layers without rotary embedding (the rope dims are plain dims)
    # hyper-connections (GLM5-next): the hidden state is hc_mult parallel streams
    hc_mult: int = 0
    hc_sinkhorn_iters: int = 1
    hc_eps: float = 1e-6
    swiglu_limit: float = 0.0                # > 0: clamp up to [-L, L] and gate to <= L before silu(gate) * up
    mlp_layer_types: Optional[List[str]] = None    # per layer "dense" | "sparse"; None = first_k_dense_replace / moe_layer_freq rule
    # Gemma4: sliding-window / global attention layers with their own head dims and rotary tables, layers that reuse the
    # keys and values of an earlier layer, GeGLU, sandwich norms, per-layer input embeddings, soft-capped logits
    sliding_window: int = 0
    global_head_dim: int = 0                 # head dim of the full-attention layers when it differs from head_dim
    num_kv_shared_layers: int = 0            # the last this-many layers read the K / V of the last earlier layer of their type
    use_double_wide_mlp: bool = False        # KV-sharing layers carry an MLP of twice the intermediate size
    hidden_size_per_layer_input: int = 0
    vocab_size_per_layer_input: int = 0
    final_logit_softcapping: float = 0.0
    hidden_activation: str = "silu"
    rope_parameters_by_type: Optional[Dict[str, Any]] = None      # layer type -> {rope_theta, partial_rotary_factor, rope_type}
    # Kimi-K3: block attention residuals, latent experts, SiTU-GLU
    attn_res_block_size: int = 0             # > 0: every this-many layers the running residual sum is frozen into the bank
    routed_expert_hidden_size: int = 0       # > 0: routed experts work in a latent space of this width (down-proj, experts, norm, up-proj)
    activation_situ_beta: float = 0.0        # > 0: the gated activation is SiTU-GLU with this beta
    activation_situ_linear_beta: float = 0.0
    # DeepSeek-V4: one shared key / value row per token (head_dim wide, the last qk_rope_head_dim dims rotated), a sliding window of
    # raw rows plus rows pooled over `compress_ratios[layer]` tokens (0 = window only), a sink logit per head, a grouped low-rank
    # output projection, hash-routed first layers
    window_size: int = 0
    compress_ratios: Optional[List[int]] = None
    compress_rope_theta: float = 0.0         # rotary base of the layers that compress (0: rope_theta)
    o_lora_rank: int = 0
    o_groups: int = 0
    num_hash_layers: int = 0                 # the first this-many MoE layers pick experts from a token-id table
    # MTP
    num_nextn_predict_layers: int = 0
    # quantisation of linear / expert weights: None (use dtype) or "fp8" (e4m3, 128x128 block scales)
    quant: Optional[str] = None
    weight_block_size: List[int] = field(default_factory=lambda: [128, 128])
    # "ue8m0": the checkpoint's block scales are powers of two and activations are quantised the same way (reference
    # models/quant_config.py:39-44); None: plain fp32 scales
    scale_fmt: Optional[str] = None
    eos_token_id: Any = None
    bos_token_id: Any = None

    # ---- derived ---------------------------------------------------------------------------
    @property
    def is_mla(self) -> bool:
        return self.architecture in ("DeepseekV2ForCausalLM", "DeepseekV3ForCausalLM", "DeepseekV32ForCausalLM",
                                     "GlmMoeDsaForCausalLM", "KimiK2ForCausalLM", "Glm5NextForConditionalGeneration",
                                     "KimiK3ForConditionalGeneration")

    @property
    def is_dsv4(self) -> bool:
        return self.architecture.startswith("DeepseekV4")

    def compress_ratio(self, layer_idx: int) -> int:
        r = self.compress_ratios or []
        return int(r[layer_idx]) if layer_idx < len(r) else 0

    @property
    def is_hybrid_gdn(self) -> bool:
        return self.linear_num_value_heads > 0

    def attn_layer_type(self, layer_idx: int) -> str:
        """"sliding_attention" or "full_attention" for the families that mix window and global layers."""
        if self.layer_types and layer_idx < len(self.layer_types) and self.layer_types[layer_idx] == "sliding_attention":
            return "sliding_attention"
        return "full_attention"

    def attn_head_dim(self, layer_idx: int) -> int:
        return self.global_head_dim if (self.global_head_dim and self.attn_layer_type(layer_idx) == "full_attention") else self.head_dim

    @property
    def first_kv_shared_layer(self) -> int:
        return self.num_hidden_layers - self.num_kv_shared_layers if self.num_kv_shared_layers > 0 else self.num_hidden_layers

    def kv_source_layer(self, layer_idx: int) -> int:
        """The layer whose K / V cache layer `layer_idx` reads: itself, or for a KV-sharing layer the last earlier layer of the
        same attention type that keeps its own."""
        first = self.first_kv_shared_layer
        if layer_idx < first:
            return layer_idx
        kind = self.attn_layer_type(layer_idx)
        for j in range(first - 1, -1, -1):
            if self.attn_layer_type(j) == kind:
                return j
        raise ValueError(f"no earlier {kind} layer to share keys and values with")

    def layer_type(self, layer_idx: int) -> str:
        if not self.is_hybrid_gdn:
            return "full_attention"
        if self.layer_types and layer_idx < len(self.layer_types):
            return self.layer_types[layer_idx]
        n = self.full_attention_interval
        return "full_attention" if n > 0 and (layer_idx + 1) % n == 0 else "linear_attention"

    def num_layers_of(self, kind: str, upto: Optional[int] = None) -> int:
        return sum(1 for i in range(self.num_hidden_layers if upto is None else upto) if self.layer_type(i) == kind)

    @property
    def gdn_conv_dim(self) -> int:
        return 2 * self.linear_num_key_heads * self.linear_key_head_dim + self.linear_num_value_heads * self.linear_value_head_dim

    @property
    def has_indexer(self) -> bool:
        return self.index_n_heads > 0

    @property
    def qk_head_dim(self) -> int:
        return self.qk_nope_head_dim + self.qk_rope_head_dim

    @property
    def mla_cache_dim(self) -> int:
        return self.kv_lora_rank + self.qk_rope_head_dim

    @property
    def glu_act(self):
        """Gated activation of the MLPs and experts as the ops take it: None (SwiGLU), ("clamp", L) or ("situ", beta, linear_beta)."""
        if self.activation_situ_beta > 0:
            return ("situ", self.activation_situ_beta, self.activation_situ_linear_beta or None)
        if self.swiglu_limit > 0:
            return ("clamp", self.swiglu_limit)
        if self.hidden_activation.startswith("gelu"):
            return ("gelu_tanh",)
        return None

    def is_moe_layer(self, layer_idx: int) -> bool:
        if self.n_routed_experts <= 0:
            return False
        if self.mlp_layer_types and layer_idx < len(self.mlp_layer_types):
            return self.mlp_layer_types[layer_idx] != "dense"
        return layer_idx >= self.first_k_dense_replace and layer_idx % self.moe_layer_freq == 0

    def eos_ids(self) -> List[int]:
        e = self.eos_token_id
        if e is None:
            return []
        return list(e) if isinstance(e, (list, tuple)) else [int(e)]

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "ModelConfig":
        d = dict(d)
        if isinstance(d.get("text_config"), dict):        # multimodal wrappers keep the language model's fields one level down
            inner = dict(d.pop("text_config"))
            inner.setdefault("architectures", d.get("architectures"))
            for k in ("quantization_config", "eos_token_id", "bos_token_id", "tie_word_embeddings"):
                if k in d and k not in inner:
                    inner[k] = d[k]
            d = inner
        rp = d.pop("rope_parameters", None)
        if isinstance(rp, dict) and rp and all(isinstance(v, dict) for v in rp.values()):
            d["rope_parameters_by_type"] = rp                 # one table per layer type (Gemma4)
            rp = None
        if isinstance(rp, dict):
            d.setdefault("rope_theta", rp.get("rope_theta", 10000000.0))
            d.setdefault("partial_rotary_factor", rp.get("partial_rotary_factor", 1.0))
        archs = d.pop("architectures", None)
        if archs and "architecture" not in d:
            d["architecture"] = archs[0]
        q = d.pop("quantization_config", None)
        if q and (str(q.get("quant_algo", "")).upper() == "NVFP4" or q.get("quant_method") in ("nvfp4", "modelopt_fp4")):
            # ModelOpt NVFP4: routed experts (and any other linear the checkpoint quantised) as packed e2m1 with e4m3 block scales
            d["quant"] = "nvfp4"
        elif q and q.get("quant_method") == "fp8":
            d["quant"] = "fp8"
            d["weight_block_size"] = list(q.get("weight_block_size", [128, 128]))
            if q.get("scale_fmt"):
                d["scale_fmt"] = q["scale_fmt"]
        arch = d.get("architecture", "")
        la = d.pop("linear_attn_config", None)
        if isinstance(la, dict):                          # Kimi delta attention block of GLM5-next / Kimi-K3
            d["linear_kind"] = "kda"
            d["linear_num_key_heads"] = d["linear_num_value_heads"] = int(la["num_heads"])
            d["linear_key_head_dim"] = int(la["head_dim"])
            d["linear_value_head_dim"] = int(la.get("value_head_dim", la["head_dim"]))
            d["linear_conv_kernel_dim"] = int(la["short_conv_kernel_size"])
            d["kda_gate_lower_bound"] = float(la.get("gate_lower_bound", -5.0))
        if isinstance(d.get("layer_types"), list):         # anything that is not a linear layer is a full-attention layer
            d["layer_types"] = [t if t in ("linear_attention", "sliding_attention") else "full_attention" for t in d["layer_types"]]
        if arch.startswith("KimiK3"):
            if "num_experts" in d:
                d["n_routed_experts"] = d.pop("num_experts")
            if "num_experts_per_token" in d:
                d["num_experts_per_tok"] = d.pop("num_experts_per_token")
            if "num_shared_experts" in d:
                d["n_shared_experts"] = d.pop("num_shared_experts")
            d.setdefault("scoring_func", "sigmoid")
            d.setdefault("topk_method", "noaux_tc")
            d.setdefault("n_group", 1)
            d.setdefault("topk_group", 1)
            d.setdefault("routed_scaling_factor", 1.0)
            d["norm_topk_prob"] = float(d["routed_scaling_factor"]) == 1.0
            d.setdefault("mla_output_gate", True)
            d.setdefault("mla_skip_rope", True)
            d.setdefault("activation_situ_beta", 4.0)
            d.setdefault("activation_situ_linear_beta", 25.0)
            if d.get("attn_res_block_size") is None:
                d["attn_res_block_size"] = 0
        if arch.startswith("Gemma4"):
            d.setdefault("n_routed_experts", 0)
            d.setdefault("hidden_activation", "gelu_pytorch_tanh")
            d.setdefault("q_lora_rank", None)
            d.setdefault("tie_word_embeddings", True)
            for k in ("global_head_dim", "sliding_window", "num_kv_shared_layers", "hidden_size_per_layer_input", "vocab_size_per_layer_input",
                      "final_logit_softcapping"):
                if d.get(k) is None:
                    d[k] = 0
        if arch.startswith("DeepseekV4"):
            # the release's own spellings (reference models/deepseek_v4/deepseek_v4.py:2894-2921)
            for ours, theirs in (("hidden_size", "dim"), ("num_hidden_layers", "n_layers"), ("num_attention_heads", "n_heads"),
                                 ("qk_rope_head_dim", "rope_head_dim"), ("moe_intermediate_size", "moe_inter_dim"),
                                 ("num_experts_per_tok", "n_activated_experts"), ("rms_norm_eps", "norm_eps"),
                                 ("num_hash_layers", "n_hash_layers"), ("scoring_func", "score_func"),
                                 ("routed_scaling_factor", "route_scale"), ("max_position_embeddings", "max_seq_len")):
                if ours not in d and theirs in d:
                    d[ours] = d.pop(theirs)
            for k, v in (("num_key_value_heads", 1), ("n_shared_experts", 1), ("hc_mult", 4), ("hc_sinkhorn_iters", 20), ("hc_eps", 1e-6),
                         ("o_groups", 8), ("o_lora_rank", 1024), ("window_size", 128), ("index_topk", 512), ("scoring_func", "sqrtsoftplus"),
                         ("first_k_dense_replace", 0), ("n_group", 1), ("topk_group", 1), ("norm_topk_prob", True), ("head_dim", 512),
                         ("max_position_embeddings", 16384), ("routed_scaling_factor", 1.0)):
                d.setdefault(k, v)
            if d.get("swiglu_limit") is None:
                d["swiglu_limit"] = 0.0
        if arch.startswith("Glm5Next"):
            d.setdefault("swiglu_limit", 10.0)
            d.setdefault("hc_mult", 4)
        # Qwen3-MoE spellings
        if "num_experts" in d:
            d["n_routed_experts"] = d.pop("num_experts")
            d.setdefault("n_shared_experts", 0)
            d.setdefault("first_k_dense_replace", 0)
            d.setdefault("scoring_func", "softmax")
            d.setdefault("n_group", 1)
            d.setdefault("topk_group", 1)
            d.setdefault("routed_scaling_factor", 1.0)
            d.setdefault("qk_norm", True)
        if d.get("architecture", "").startswith("Qwen3_5"):
            d.setdefault("qk_norm", True)
            d.setdefault("attn_output_gate", True)
            d.setdefault("norm_unit_offset", True)
            d.setdefault("n_shared_experts", 0)
            d.setdefault("first_k_dense_replace", 0)
        if d.get("architecture", "").startswith("Qwen3") and "n_routed_experts" not in d:
            d.setdefault("n_routed_experts", 0)
            d.setdefault("qk_norm", True)
        known = {f.name for f in fields(cls)}
        return cls(**{k: v for k, v in d.items() if k in known})

    @classmethod
    def from_pretrained(cls, path: str) -> "ModelConfig":
        with open(os.path.join(path, "config.json")) as f:
            d = json.load(f)
        side = os.path.join(path, "hf_quant_config.json")          # where ModelOpt exports put the quantisation recipe
        if "quantization_config" not in d and os.path.exists(side):
            with open(side) as f:
                q = json.load(f).get("quantization", {})
            if q.get("quant_algo"):
                d["quantization_config"] = {"quant_method": "modelopt", **q}
        return cls.from_dict(d)

    def to_dict(self) -> Dict[str, Any]:
        d = {f.name: getattr(self, f.name) for f in fields(self)}
        d["architectures"] = [d.pop("architecture")]
        quant = d.pop("quant")
        if quant == "nvfp4":
            d["quantization_config"] = {"quant_method": "modelopt", "quant_algo": "NVFP4", "group_size": 16}
        if quant == "fp8":
            d["quantization_config"] = {"quant_method": "fp8", "fmt": "e4m3", "weight_block_size": d["weight_block_size"]}
            if d.get("scale_fmt"):
                d["quantization_config"]["scale_fmt"] = d["scale_fmt"]
        d.pop("weight_block_size")
        d.pop("scale_fmt", None)
        return d


def tiny_deepseek_v3(**over) -> ModelConfig:
    """The CPU plumbing shape: 2 layers (dense then MoE), hidden 256, 8 MLA heads, 8 experts top-2."""
    c = ModelConfig(architecture="DeepseekV3ForCausalLM", vocab_size=1024, hidden_size=256, num_hidden_layers=2,
                    num_attention_heads=8, num_key_value_heads=8, rms_norm_eps=1e-6, rope_theta=10000.0,
                    max_position_embeddings=4096, intermediate_size=512, q_lora_rank=128, kv_lora_rank=64,
                    qk_nope_head_dim=32, qk_rope_head_dim=16, v_head_dim=32, n_routed_experts=8, n_shared_experts=1,
                    num_experts_per_tok=2, moe_intermediate_size=128, first_k_dense_replace=1, n_group=1, topk_group=1,
                    norm_topk_prob=True, routed_scaling_factor=1.0, scoring_func="sigmoid", eos_token_id=None)
    for k, v in over.items():
        setattr(c, k, v)
    return c


def deepseek_v3(**over) -> ModelConfig:
    """DeepSeek-V3 / R1 shape: 61 layers, 256 experts top-8 (8 groups / top-4), fp8 block-scaled weights."""
    c = ModelConfig(quant="fp8", eos_token_id=1, num_nextn_predict_layers=1,
                    rope_scaling={"type": "yarn", "factor": 40, "original_max_position_embeddings": 4096,
                                  "beta_fast": 32, "beta_slow": 1, "mscale": 1.0, "mscale_all_dim": 1.0})
    for k, v in over.items():
        setattr(c, k, v)
    return c


def deepseek_v32(**over) -> ModelConfig:
    """DeepSeek-V3.2 shape: the V3 body plus a lightning indexer (64 heads x 128, top-2048) per layer."""
    return deepseek_v3(architecture="DeepseekV32ForCausalLM", index_n_heads=64, index_head_dim=128, index_topk=2048, **over)


def qwen3_235b(**over) -> ModelConfig:
    """Qwen3-235B-A22B shape: 94 layers, GQA 64/4 heads with q/k norm, 128 experts top-8 softmax routing."""
    c = ModelConfig(architecture="Qwen3MoeForCausalLM", vocab_size=151936, hidden_size=4096, num_hidden_layers=94,
                    num_attention_heads=64, num_key_value_heads=4, head_dim=128, rope_theta=1e6,
                    max_position_embeddings=40960, intermediate_size=12288, n_routed_experts=128, n_shared_experts=0,
                    num_experts_per_tok=8, moe_intermediate_size=1536, first_k_dense_replace=0, n_group=1, topk_group=1,
                    norm_topk_prob=True, routed_scaling_factor=1.0, scoring_func="softmax", qk_norm=True,
                    q_lora_rank=None, eos_token_id=151645)
    for k, v in over.items():
        setattr(c, k, v)
    return c


def tiny_qwen3_5(moe: bool = False, **over) -> ModelConfig:
    """CPU plumbing shape of the hybrid family: 4 layers (three gated delta-net, one gated full attention), hidden 128."""
    c = ModelConfig(architecture="Qwen3_5MoeForConditionalGeneration" if moe else "Qwen3_5ForConditionalGeneration", vocab_size=512,
                    hidden_size=128, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, head_dim=32, rope_theta=1e6,
                    max_position_embeddings=4096, intermediate_size=256, q_lora_rank=None, n_routed_experts=8 if moe else 0,
                    n_shared_experts=0, num_experts_per_tok=2, moe_intermediate_size=64, first_k_dense_replace=0, n_group=1,
                    topk_group=1, norm_topk_prob=True, routed_scaling_factor=1.0, scoring_func="softmax", qk_norm=True,
                    full_attention_interval=4, linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=32,
                    linear_value_head_dim=32, linear_conv_kernel_dim=4, partial_rotary_factor=0.25, attn_output_gate=True,
                    norm_unit_offset=True, shared_expert_intermediate_size=64 if moe else 0, eos_token_id=None)
    for k, v in over.items():
        setattr(c, k, v)
    return c


def qwen3_5_80b(**over) -> ModelConfig:
    """Qwen3.5-MoE shape of the 80B-A3B class: 48 layers (3 gated delta-net : 1 full attention), 512 experts top-10 + gated shared expert."""
    c = ModelConfig(architecture="Qwen3_5MoeForConditionalGeneration", vocab_size=151936, hidden_size=2048, num_hidden_layers=48,
                    num_attention_heads=16, num_key_value_heads=2, head_dim=256, rope_theta=1e7, max_position_embeddings=262144,
                    intermediate_size=5120, q_lora_rank=None, n_routed_experts=512, n_shared_experts=0, num_experts_per_tok=10,
                    moe_intermediate_size=512, first_k_dense_replace=0, n_group=1, topk_group=1, norm_topk_prob=True,
                    routed_scaling_factor=1.0, scoring_func="softmax", qk_norm=True, full_attention_interval=4,
                    linear_num_key_heads=16, linear_num_value_heads=32, linear_key_head_dim=128, linear_value_head_dim=128,
                    linear_conv_kernel_dim=4, partial_rotary_factor=0.25, attn_output_gate=True, norm_unit_offset=True,
                    shared_expert_intermediate_size=512, eos_token_id=151645)
    for k, v in over.items():
        setattr(c, k, v)
    return c


PRESETS = {"tiny-deepseek-v3": tiny_deepseek_v3, "deepseek-v3": deepseek_v3, "deepseek-v3.2": deepseek_v32,
           "qwen3-235b-a22b": qwen3_235b, "tiny-qwen3.5": tiny_qwen3_5, "qwen3.5-80b-a3b": qwen3_5_80b}


def tiny_glm5_next(**over) -> ModelConfig:
    """CPU-sized GLM5-next shape: delta-attention / sparse-attention layers alternating, 2 hyper-connection streams."""
    base = dict(architecture="Glm5NextForConditionalGeneration", vocab_size=512, hidden_size=128, num_hidden_layers=4,
                num_attention_heads=4, num_key_value_heads=4, q_lora_rank=48, kv_lora_rank=32, qk_nope_head_dim=16, qk_rope_head_dim=16,
                v_head_dim=16, intermediate_size=256, n_routed_experts=8, n_shared_experts=1, num_experts_per_tok=2, moe_intermediate_size=64,
                first_k_dense_replace=1, n_group=2, topk_group=1, max_position_embeddings=4096,
                layer_types=["linear_attention", "full_attention", "linear_attention", "full_attention"],
                mlp_layer_types=["dense", "sparse", "sparse", "sparse"], linear_kind="kda", linear_num_key_heads=2, linear_num_value_heads=2,
                linear_key_head_dim=32, linear_value_head_dim=32, linear_conv_kernel_dim=4, kda_gate_lower_bound=-5.0,
                hc_mult=2, hc_sinkhorn_iters=3, swiglu_limit=10.0, index_n_heads=2, index_head_dim=32, index_topk=64)
    base.update(over)
    return ModelConfig(**base)


def tiny_kimi_k3(**over) -> ModelConfig:
    """CPU-sized Kimi-K3 shape: delta-attention layers with every third layer NoPE MLA, residual blocks of 2 layers, latent experts."""
    base = dict(architecture="KimiK3ForConditionalGeneration", vocab_size=512, hidden_size=128, num_hidden_layers=5,
                num_attention_heads=4, num_key_value_heads=4, q_lora_rank=48, kv_lora_rank=32, qk_nope_head_dim=16, qk_rope_head_dim=16,
                v_head_dim=16, intermediate_size=256, n_routed_experts=8, n_shared_experts=1, num_experts_per_tok=2, moe_intermediate_size=64,
                first_k_dense_replace=1, n_group=1, topk_group=1, routed_scaling_factor=1.0, norm_topk_prob=True, max_position_embeddings=4096,
                layer_types=["linear_attention", "linear_attention", "full_attention", "linear_attention", "full_attention"],
                linear_kind="kda", linear_num_key_heads=2, linear_num_value_heads=2, linear_key_head_dim=32, linear_value_head_dim=32,
                linear_conv_kernel_dim=4, kda_gate_lower_bound=-5.0, mla_output_gate=True, mla_skip_rope=True, attn_res_block_size=2,
                routed_expert_hidden_size=64, activation_situ_beta=4.0, activation_situ_linear_beta=25.0)
    base.update(over)
    return ModelConfig(**base)


def tiny_deepseek_v4(**over) -> ModelConfig:
    """CPU-sized DeepSeek-V4 shape: a window-only layer, a ratio-4 (overlapping) and a ratio-8 compressing layer, 2 hyper-connection
    streams, the first MoE layer hash-routed."""
    base = dict(architecture="DeepseekV4ForCausalLM", vocab_size=512, hidden_size=128, num_hidden_layers=3, num_attention_heads=4,
                num_key_value_heads=1, head_dim=80, qk_rope_head_dim=16, q_lora_rank=48, o_lora_rank=32, o_groups=2, window_size=8,
                compress_ratios=[0, 4, 8], compress_rope_theta=40000.0, n_routed_experts=8, n_shared_experts=1, num_experts_per_tok=2,
                moe_intermediate_size=64, first_k_dense_replace=0, n_group=1, topk_group=1, routed_scaling_factor=1.5, norm_topk_prob=True,
                scoring_func="sqrtsoftplus", num_hash_layers=1, hc_mult=2, hc_sinkhorn_iters=3, swiglu_limit=10.0,
                max_position_embeddings=4096)
    base.update(over)
    return ModelConfig(**base)


PRESETS["tiny-deepseek-v4"] = tiny_deepseek_v4


def tiny_gemma4(**over) -> ModelConfig:
    """CPU-sized Gemma4 shape: two sliding-window layers per global layer, the last two layers reading shared keys / values,
    per-layer input embeddings, tied and soft-capped output."""
    base = dict(architecture="Gemma4ForCausalLM", vocab_size=512, hidden_size=128, num_hidden_layers=6, num_attention_heads=4,
                num_key_value_heads=2, head_dim=32, global_head_dim=64, intermediate_size=256, n_routed_experts=0, q_lora_rank=None,
                max_position_embeddings=4096, sliding_window=16, num_kv_shared_layers=2, use_double_wide_mlp=True,
                layer_types=["sliding_attention", "sliding_attention", "full_attention", "sliding_attention", "sliding_attention", "full_attention"],
                hidden_size_per_layer_input=16, vocab_size_per_layer_input=512, final_logit_softcapping=30.0,
                hidden_activation="gelu_pytorch_tanh", tie_word_embeddings=True,
                rope_parameters_by_type={"sliding_attention": {"rope_theta": 10000.0, "rope_type": "default"},
                                         "full_attention": {"rope_theta": 1000000.0, "rope_type": "proportional", "partial_rotary_factor": 0.25}})
    base.update(over)
    return ModelConfig(**base)
