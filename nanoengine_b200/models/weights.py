"""HF-layout weight handling: name mapping into the fused/stacked parameters of the models, a random
generator that emits tensors under the same names (so synthetic benchmarks exercise the real loading
path), safetensors shard iteration with expert-parallel pre-filtering, and a tiny checkpoint writer.

Parity: reference runtime/runner/loader.py:212-250 (iterate_weights), :34-53 (EP filter before the tensor
is read), :362-494 (per-expert -> stacked tensors), :90-119 (fp8 block dequant);
models/deepseek_v2/deepseek_v2_loader.py:36-121 (kv_b_proj -> kc/vc), :124-270.
"""
from __future__ import annotations

import glob
import json
import os
import re
import zlib
from typing import Callable, Dict, Iterable, Iterator, Optional, Tuple

import torch


from .config import ModelConfig

_EXPERT_RE = re.compile(r"\.(?:mlp|ffn)\.experts\.(\d+)\.")
_LAYER_RE = re.compile(r"^(?:model\.)?layers\.(\d+)\.")


def expert_owner_filter(cfg: ModelConfig, ep_size: int, ep_rank: int, layer_range=None) -> Callable[[str], bool]:
    """True for tensors this rank must read: its own experts and (with PP) its own layers."""
    per = max(1, cfg.n_routed_experts // max(1, ep_size)) if cfg.n_routed_experts else 1
    from ..parallel.eplb import active_plan
    plan = active_plan()
    per_phys = plan.num_physical // max(1, ep_size) if plan is not None else 0

    def keep(name: str) -> bool:
        m = _LAYER_RE.match(name)
        if m and layer_range is not None:
            li = int(m.group(1))
            if li < cfg.num_hidden_layers and not (layer_range[0] <= li < layer_range[1]):
                return False
        e = _EXPERT_RE.search(name)
        if e is not None:
            if plan is not None and m and int(m.group(1)) < plan.num_layers:
                # under a load-balancing plan an expert is read by every rank that holds one of its physical replicas
                return any(p // per_phys == ep_rank for p in plan.slots_of(int(m.group(1)), int(e.group(1))))
            return int(e.group(1)) // per == ep_rank
        return True

    return keep


def iterate_safetensors(path: str, keep: Optional[Callable[[str], bool]] = None, device="cpu") -> Iterator[Tuple[str, torch.Tensor]]:
    """Yield (name, tensor) from every *.safetensors shard; `keep` is consulted before a tensor is read."""
    from safetensors import safe_open
    shards = sorted(glob.glob(os.path.join(path, "*.safetensors")))
    if not shards:
        raise FileNotFoundError(f"no *.safetensors shards under {path!r}")
    for f in shards:
        with safe_open(f, framework="pt", device=str(device)) as sf:
            for name in sf.keys():
                if keep is None or keep(name):
                    yield name, sf.get_tensor(name)


def hf_param_shapes(cfg: ModelConfig, include_mtp: bool = False) -> Dict[str, Tuple[int, ...]]:
    """Every tensor name of an HF-layout checkpoint of this architecture with its (high-precision) shape."""
    H, V = cfg.hidden_size, cfg.vocab_size
    out: Dict[str, Tuple[int, ...]] = {"model.embed_tokens.weight": (V, H), "model.norm.weight": (H,), "lm_head.weight": (V, H)}
    if cfg.architecture.startswith("Gemma4"):
        return _gemma4_param_shapes(cfg, out)
    if cfg.is_dsv4:
        from .deepseek_v4 import dsv4_param_shapes
        return dsv4_param_shapes(cfg, out)

    def attn(p):
        if cfg.is_mla:
            nh, R, rope, nope, v = cfg.num_attention_heads, cfg.kv_lora_rank, cfg.qk_rope_head_dim, cfg.qk_nope_head_dim, cfg.v_head_dim
            if cfg.q_lora_rank:
                out[p + "q_a_proj.weight"] = (cfg.q_lora_rank, H)
                out[p + "q_a_layernorm.weight"] = (cfg.q_lora_rank,)
                out[p + "q_b_proj.weight"] = (nh * (nope + rope), cfg.q_lora_rank)
            else:
                out[p + "q_proj.weight"] = (nh * (nope + rope), H)
            out[p + "kv_a_proj_with_mqa.weight"] = (R + rope, H)
            out[p + "kv_a_layernorm.weight"] = (R,)
            out[p + "kv_b_proj.weight"] = (nh * (nope + v), R)
            out[p + "o_proj.weight"] = (H, nh * v)
            if cfg.mla_output_gate:
                out[p + "g_proj.weight"] = (nh * v, H)
            if cfg.has_indexer:
                out[p + "indexer.wq_b.weight"] = (cfg.index_n_heads * cfg.index_head_dim, cfg.q_lora_rank or H)
                out[p + "indexer.wk.weight"] = (cfg.index_head_dim, H)
                out[p + "indexer.k_norm.weight"] = (cfg.index_head_dim,)
                out[p + "indexer.k_norm.bias"] = (cfg.index_head_dim,)
                out[p + "indexer.weights_proj.weight"] = (cfg.index_n_heads, H)
        else:
            hd = cfg.head_dim
            out[p + "q_proj.weight"] = (cfg.num_attention_heads * hd * (2 if cfg.attn_output_gate else 1), H)
            out[p + "k_proj.weight"] = (cfg.num_key_value_heads * hd, H)
            out[p + "v_proj.weight"] = (cfg.num_key_value_heads * hd, H)
            out[p + "o_proj.weight"] = (H, cfg.num_attention_heads * hd)
            if cfg.qk_norm:
                out[p + "q_norm.weight"] = (hd,)
                out[p + "k_norm.weight"] = (hd,)

    def linear_attn(p):
        Hk, Hv, Dk, Dv = cfg.linear_num_key_heads, cfg.linear_num_value_heads, cfg.linear_key_head_dim, cfg.linear_value_head_dim
        out[p + "in_proj_qkv.weight"] = (cfg.gdn_conv_dim, H)
        out[p + "in_proj_z.weight"] = (Hv * Dv, H)
        out[p + "in_proj_a.weight"] = (Hv, H)
        out[p + "in_proj_b.weight"] = (Hv, H)
        out[p + "conv1d.weight"] = (cfg.gdn_conv_dim, 1, cfg.linear_conv_kernel_dim)
        out[p + "dt_bias"] = (Hv,)
        out[p + "A_log"] = (Hv,)
        out[p + "norm.weight"] = (Dv,)
        out[p + "out_proj.weight"] = (H, Hv * Dv)

    def layer(i, moe):
        p = f"model.layers.{i}."
        out[p + "input_layernorm.weight"] = (H,)
        out[p + "post_attention_layernorm.weight"] = (H,)
        if cfg.layer_type(i) == "linear_attention" and cfg.linear_kind == "kda":
            from .kda import kda_param_shapes
            kda_param_shapes(cfg, p + "self_attn.", out, low_rank_gate=cfg.linear_key_head_dim if cfg.hc_mult else None)
        elif cfg.layer_type(i) == "linear_attention":
            linear_attn(p + "linear_attn.")
        else:
            attn(p + "self_attn.")
        if cfg.hc_mult:
            for site in ("hc_attn", "hc_ffn"):
                out[p + site + "_fn"] = ((2 + cfg.hc_mult) * cfg.hc_mult, cfg.hc_mult * H)
                out[p + site + "_base"] = ((2 + cfg.hc_mult) * cfg.hc_mult,)
                out[p + site + "_scale"] = (3,)
        if cfg.attn_res_block_size and i < cfg.num_hidden_layers:
            for site in ("self_attention_res", "mlp_res"):
                out[p + site + "_norm.weight"] = (H,)
                out[p + site + "_proj.weight"] = (1, H)
        if moe and cfg.routed_expert_hidden_size:
            I, Z = cfg.moe_intermediate_size, cfg.routed_expert_hidden_size
            out[p + "mlp.gate.weight"] = (cfg.n_routed_experts, H)
            out[p + "mlp.gate.e_score_correction_bias"] = (cfg.n_routed_experts,)
            out[p + "mlp.routed_expert_down_proj.weight"] = (Z, H)
            out[p + "mlp.routed_expert_norm.weight"] = (Z,)
            out[p + "mlp.routed_expert_up_proj.weight"] = (H, Z)
            for e in range(cfg.n_routed_experts):
                out[p + f"mlp.experts.{e}.w1.weight"] = (I, Z)
                out[p + f"mlp.experts.{e}.w3.weight"] = (I, Z)
                out[p + f"mlp.experts.{e}.w2.weight"] = (Z, I)
            if cfg.n_shared_experts:
                Is = I * cfg.n_shared_experts
                out[p + "mlp.shared_experts.gate_proj.weight"] = (Is, H)
                out[p + "mlp.shared_experts.up_proj.weight"] = (Is, H)
                out[p + "mlp.shared_experts.down_proj.weight"] = (H, Is)
        elif moe:
            I = cfg.moe_intermediate_size
            out[p + "mlp.gate.weight"] = (cfg.n_routed_experts, H)
            if cfg.topk_method == "noaux_tc" and cfg.scoring_func == "sigmoid":
                out[p + "mlp.gate.e_score_correction_bias"] = (cfg.n_routed_experts,)
            for e in range(cfg.n_routed_experts):
                out[p + f"mlp.experts.{e}.gate_proj.weight"] = (I, H)
                out[p + f"mlp.experts.{e}.up_proj.weight"] = (I, H)
                out[p + f"mlp.experts.{e}.down_proj.weight"] = (H, I)
            if cfg.shared_expert_intermediate_size:
                Is = cfg.shared_expert_intermediate_size
                out[p + "mlp.shared_expert.gate_proj.weight"] = (Is, H)
                out[p + "mlp.shared_expert.up_proj.weight"] = (Is, H)
                out[p + "mlp.shared_expert.down_proj.weight"] = (H, Is)
                out[p + "mlp.shared_expert_gate.weight"] = (1, H)
            if cfg.n_shared_experts:
                Is = I * cfg.n_shared_experts
                out[p + "mlp.shared_experts.gate_proj.weight"] = (Is, H)
                out[p + "mlp.shared_experts.up_proj.weight"] = (Is, H)
                out[p + "mlp.shared_experts.down_proj.weight"] = (H, Is)
        else:
            I = cfg.intermediate_size
            out[p + "mlp.gate_proj.weight"] = (I, H)
            out[p + "mlp.up_proj.weight"] = (I, H)
            out[p + "mlp.down_proj.weight"] = (H, I)

    for i in range(cfg.num_hidden_layers):
        layer(i, cfg.is_moe_layer(i))
    if cfg.attn_res_block_size:
        out["model.output_attn_res_norm.weight"] = (H,)
        out["model.output_attn_res_proj.weight"] = (1, H)
    if include_mtp:
        for k in range(cfg.num_nextn_predict_layers):
            i = cfg.num_hidden_layers + k
            layer(i, cfg.n_routed_experts > 0)
            p = f"model.layers.{i}."
            out[p + "enorm.weight"] = (H,)
            out[p + "hnorm.weight"] = (H,)
            out[p + "eh_proj.weight"] = (H, 2 * H)
            out[p + "shared_head.norm.weight"] = (H,)
    return out


def _gemma4_param_shapes(cfg: ModelConfig, out):
    H, L, P = cfg.hidden_size, cfg.num_hidden_layers, cfg.hidden_size_per_layer_input
    if cfg.tie_word_embeddings:
        out.pop("lm_head.weight")
    if P:
        out["model.embed_tokens_per_layer.weight"] = (cfg.vocab_size_per_layer_input or cfg.vocab_size, L * P)
        out["model.per_layer_model_projection.weight"] = (L * P, H)
        out["model.per_layer_projection_norm.weight"] = (P,)
    for i in range(L):
        p = f"model.layers.{i}."
        hd, shared = cfg.attn_head_dim(i), cfg.kv_source_layer(i) != i
        out[p + "self_attn.q_proj.weight"] = (cfg.num_attention_heads * hd, H)
        out[p + "self_attn.k_proj.weight"] = (cfg.num_key_value_heads * hd, H)      # kept by the checkpoints for every layer
        out[p + "self_attn.v_proj.weight"] = (cfg.num_key_value_heads * hd, H)
        out[p + "self_attn.o_proj.weight"] = (H, cfg.num_attention_heads * hd)
        for nm in ("q_norm", "k_norm", "v_norm"):
            out[p + f"self_attn.{nm}.weight"] = (hd,)
        I = cfg.intermediate_size * (2 if (cfg.use_double_wide_mlp and shared) else 1)
        out[p + "mlp.gate_proj.weight"] = (I, H)
        out[p + "mlp.up_proj.weight"] = (I, H)
        out[p + "mlp.down_proj.weight"] = (H, I)
        for nm in ("input_layernorm", "post_attention_layernorm", "pre_feedforward_layernorm", "post_feedforward_layernorm"):
            out[p + nm + ".weight"] = (H,)
        out[p + "layer_scalar"] = (1,)
        if P:
            out[p + "per_layer_input_gate.weight"] = (P, H)
            out[p + "per_layer_projection.weight"] = (H, P)
            out[p + "post_per_layer_input_norm.weight"] = (H,)
    return out


def random_hf_weights(cfg: ModelConfig, seed: int = 0, device="cpu", keep: Optional[Callable[[str], bool]] = None,
                      include_mtp: bool = False, std: float = 0.02) -> Iterator[Tuple[str, torch.Tensor]]:
    """Random-init tensors under HF names.  Each tensor draws from its own generator seeded by (seed, name),
    so the values do not depend on which rank generates them or on the parallel layout."""
    dev = torch.device(device)
    for name, shape in hf_param_shapes(cfg, include_mtp).items():
        if keep is not None and not keep(name):
            continue
        g = torch.Generator(device=dev)
        g.manual_seed((seed * 1000003 + zlib.crc32(name.encode())) & 0x7FFFFFFFFFFF)
        if name.endswith("tid2eid"):            # token id -> its experts: distinct ids per row
            t = torch.rand(shape[0], cfg.n_routed_experts, generator=g, device=dev).argsort(-1)[:, : shape[1]].to(torch.int32)
        elif name.endswith("attn_sink"):
            t = 0.5 * torch.randn(shape, generator=g, device=dev, dtype=torch.float32)
        elif name.endswith("layer_scalar"):
            t = 1.0 + 0.05 * torch.randn(shape, generator=g, device=dev, dtype=torch.float32)
        elif name.endswith("A_log"):
            t = torch.log(1.0 + 3.0 * torch.rand(shape, generator=g, device=dev, dtype=torch.float32))
        elif name.endswith(("_fn", "_base")):
            t = 0.05 * torch.randn(shape, generator=g, device=dev, dtype=torch.float32)
        elif name.endswith("_scale") and len(shape) == 1 and shape[0] in (1, 3):
            t = 1.0 + 0.1 * torch.randn(shape, generator=g, device=dev, dtype=torch.float32)
        elif name.endswith("dt_bias"):
            t = 0.5 * torch.randn(shape, generator=g, device=dev, dtype=torch.float32)
        elif name.endswith("conv1d.weight"):
            t = 0.3 * torch.randn(shape, generator=g, device=dev, dtype=torch.float32)
        elif cfg.norm_unit_offset and name.endswith("norm.weight") and "linear_attn" not in name:
            t = 0.1 * torch.randn(shape, generator=g, device=dev, dtype=torch.float32)      # stored as the deviation from one
        elif name.endswith("norm.weight") and "k_norm" not in name or name.endswith("layernorm.weight"):
            t = 1.0 + 0.1 * torch.randn(shape, generator=g, device=dev, dtype=torch.float32)
        elif name.endswith("e_score_correction_bias") or name.endswith(".bias"):
            t = 0.01 * torch.randn(shape, generator=g, device=dev, dtype=torch.float32)
        elif name.endswith("k_norm.weight"):
            t = 1.0 + 0.1 * torch.randn(shape, generator=g, device=dev, dtype=torch.float32)
        else:
            t = std * torch.randn(shape, generator=g, device=dev, dtype=torch.float32)
        yield name, t


def _mlp_target(mod, leaf: str):
    return {"gate_proj": ("gate_up", 0), "up_proj": ("gate_up", 1), "down_proj": ("down", 0)}[leaf]


class _Pending:
    """Collects (weight, weight_scale_inv) pairs and halves of merged matrices until they are complete."""

    def __init__(self):
        self.w: Dict[str, torch.Tensor] = {}
        self.s: Dict[str, torch.Tensor] = {}

    def take(self, key):
        return self.w.pop(key), self.s.pop(key, None)


_NVFP4_PART = re.compile(r"(.*)\.(weight|weight_scale|weight_scale_2|input_scale)$")
_NVFP4_EXPERT = re.compile(r"model\.layers\.(\d+)\.mlp\.experts\.(\d+)\.(gate_proj|up_proj|down_proj)$")


def _deq(w, s):
    from ..ops import reference as ref
    return ref.dequant_fp8_block(w, s) if w.dtype == torch.float8_e4m3fn else w.float()


def load_deepseek_weights(model, weights: Iterable[Tuple[str, torch.Tensor]], mtp=None) -> int:
    """Feed HF-named tensors into a DeepseekV3ForCausalLM (and optionally its MTP head).  Returns tensors consumed.

    fp8 checkpoints deliver ``<name>.weight`` (e4m3) and ``<name>.weight_scale_inv``; both orders are accepted.
    Merged parameters (gate_up, qkv_a) are assembled from their parts; parts that arrive in fp8 for a merged
    fp8 target are copied block-wise with their scales, anything else goes through fp32.
    """
    cfg: ModelConfig = model.cfg
    n = 0
    fp8 = torch.float8_e4m3fn
    wbuf: Dict[str, torch.Tensor] = {}
    sbuf: Dict[str, torch.Tensor] = {}
    groups: Dict[str, Dict[str, Tuple[torch.Tensor, Optional[torch.Tensor]]]] = {}
    fbuf: Dict[str, Dict[str, torch.Tensor]] = {}
    quant_names = set()

    def layer_of(i):
        if i < cfg.num_hidden_layers:
            return model.model.layers[str(i)] if str(i) in model.model.layers else None
        return mtp.blocks[i - cfg.num_hidden_layers] if mtp is not None else None

    def merged_set(lin, parts):
        """parts: list of (w, s) in row order -> one QLinear."""
        if lin.quant == "fp8" and all(w.dtype == fp8 for w, _ in parts) and all(w.shape[0] % 128 == 0 for w, _ in parts[:-1]):
            lin.set_weight(torch.cat([w for w, _ in parts], 0), torch.cat([s for _, s in parts], 0))
        else:
            lin.set_weight(torch.cat([_deq(w, s) for w, s in parts], 0))

    def place(base: str, w: torch.Tensor, s: Optional[torch.Tensor]):
        nonlocal n
        n += 1
        if base == "model.embed_tokens":
            if model.model.embed_tokens is not None:
                model.model.embed_tokens.weight.copy_(w.to(model.model.embed_tokens.weight.dtype))
            return
        if base == "lm_head":
            model.lm_head.weight.copy_(w.to(model.lm_head.weight.dtype)); return
        if base == "model.norm":
            if model.model.norm is not None:
                model.model.norm.weight.copy_(w.to(model.model.norm.weight.dtype))
            return
        m = _LAYER_RE.match(base + ".")
        if not m:
            return
        li = int(m.group(1))
        L = layer_of(li)
        if L is None:
            n -= 1
            return
        rest = base[m.end():]
        if li >= cfg.num_hidden_layers and mtp is not None:
            k = li - cfg.num_hidden_layers
            if rest in ("enorm", "hnorm"):
                getattr(mtp, rest)[k].weight.copy_(w.to(mtp.enorm[k].weight.dtype)); return
            if rest == "eh_proj":
                mtp.eh_proj[k].set_weight(_deq(w, s)); return
            if rest == "shared_head.norm":
                mtp.final_norm[k].weight.copy_(w.to(mtp.final_norm[k].weight.dtype)); return
            if rest.startswith("shared_head.") or rest == "embed_tokens":
                return  # shared with the target model
        if rest in ("input_layernorm", "post_attention_layernorm"):
            getattr(L, rest).weight.copy_(w.to(getattr(L, rest).weight.dtype)); return
        if rest.startswith("self_attn."):
            A = L.self_attn
            leaf = rest[len("self_attn."):]
            if leaf in ("q_a_layernorm", "kv_a_layernorm"):
                getattr(A, leaf).weight.copy_(w.to(getattr(A, leaf).weight.dtype)); return
            if leaf == "kv_b_proj":
                A.set_kv_b(w, s); return
            if leaf == "g_proj":
                if A.g_proj is not None:
                    A.g_proj.set_weight(_deq(w, s))
                return
            if leaf in ("q_b_proj", "o_proj", "q_proj") or (leaf == "kv_a_proj_with_mqa" and not A.q_lora):
                getattr(A, leaf).set_weight(w, s); return
            if leaf in ("q_a_proj", "kv_a_proj_with_mqa"):
                g = groups.setdefault(f"{li}.qkv_a", {})
                g[leaf] = (w, s)
                if len(g) == 2:
                    merged_set(A.qkv_a_proj, [g["q_a_proj"], g["kv_a_proj_with_mqa"]]); groups.pop(f"{li}.qkv_a")
                return
            if leaf.startswith("indexer.") and A.indexer is not None:
                A.indexer.load(leaf[len("indexer."):], w, s); return
            return
        if rest.startswith("mlp."):
            leaf = rest[len("mlp."):]
            M = L.mlp
            if leaf == "gate":
                M.gate.weight.copy_(w.float()); return
            e = re.match(r"experts\.(\d+)\.(gate_proj|up_proj|down_proj)$", leaf)
            if e:
                eid, which = int(e.group(1)), e.group(2)[:-5]
                ex = M.experts
                if not ex.load_expert(eid, which, w, s):
                    n -= 1
                return
            tgt = M.shared_experts if leaf.startswith("shared_experts.") else M
            leaf2 = leaf.split(".")[-1]
            if leaf2 == "down_proj":
                tgt.down_proj.set_weight(w, s); return
            g = groups.setdefault(f"{li}.{'s' if tgt is not M else 'd'}.gate_up", {})
            g[leaf2] = (w, s)
            if len(g) == 2:
                merged_set(tgt.gate_up_proj, [g["gate_proj"], g["up_proj"]]); groups.pop(f"{li}.{'s' if tgt is not M else 'd'}.gate_up")
            return

    with torch.no_grad():
        for name, t in weights:
            if name.endswith(".e_score_correction_bias"):
                li = int(_LAYER_RE.match(name).group(1))
                L = layer_of(li)
                if L is not None and getattr(L.mlp, "gate", None) is not None and L.mlp.gate.e_score_correction_bias is not None:
                    L.mlp.gate.e_score_correction_bias.copy_(t.float()); n += 1
                continue
            if name.endswith("k_norm.bias"):
                li = int(_LAYER_RE.match(name).group(1))
                L = layer_of(li)
                if L is not None and L.self_attn.indexer is not None:
                    L.self_attn.indexer.load("k_norm.bias", t, None); n += 1
                continue
            part = _NVFP4_PART.match(name)
            if part and (cfg.quant == "nvfp4") and (part.group(2) != "weight" or t.dtype == torch.uint8):
                # ModelOpt NVFP4: routed experts keep the packed form; any other quantised linear is expanded once all three weight
                # tensors are in (its input_scale is not needed: it runs in bf16)
                base, kind = part.group(1), part.group(2)
                em = _NVFP4_EXPERT.match(base)
                L = layer_of(int(em.group(1))) if em else None
                if em and L is not None and getattr(L.mlp, "experts", None) is not None and L.mlp.experts.quant == "nvfp4":
                    if L.mlp.experts.load_expert_part(int(em.group(2)), em.group(3)[:-5], kind, t):
                        n += 1
                    continue
                if em and L is None:
                    continue
                fb = fbuf.setdefault(base, {})
                fb[kind] = t
                if all(k in fb for k in ("weight", "weight_scale", "weight_scale_2")):
                    from ..ops import reference as ref
                    w = ref.nvfp4_unpack(fb["weight"].to(torch.uint8), fb["weight_scale"].view(torch.float8_e4m3fn)) * fb["weight_scale_2"].float()
                    fbuf.pop(base)
                    place(base, w.to(torch.bfloat16), None)
                continue
            if name.endswith(".weight_scale_inv"):
                base = name[: -len(".weight_scale_inv")]
                if base in wbuf:
                    place(base, wbuf.pop(base), t)
                else:
                    sbuf[base] = t
                continue
            if not name.endswith(".weight"):
                continue
            base = name[: -len(".weight")]
            if t.dtype == fp8:
                if base in sbuf:
                    place(base, t, sbuf.pop(base))
                else:
                    wbuf[base] = t
            else:
                place(base, t, None)
    fbuf = {k: v for k, v in fbuf.items() if "weight" in v}          # a stray input_scale of a linear kept in bf16 is not an error
    if wbuf or groups or fbuf:
        raise ValueError(f"incomplete checkpoint: {list(wbuf)[:3]} {list(groups)[:3]} {list(fbuf)[:3]}")
    return n


def save_hf_checkpoint(path: str, cfg: ModelConfig, weights: Iterable[Tuple[str, torch.Tensor]], quantize_fp8: bool = False,
                       shard_bytes: int = 1 << 30, quantize_nvfp4: bool = False, nvfp4_input_scale: float = 32.0 / (6.0 * 448.0)) -> None:
    """Write a small HF-layout checkpoint (config.json + safetensors shards); used by tests and examples.  `quantize_nvfp4`: the
    MLP / expert projections in the ModelOpt NVFP4 layout (`weight` packed e2m1, `weight_scale` e4m3 per 16, `weight_scale_2`,
    `input_scale`), everything else in bf16."""
    from safetensors.torch import save_file
    from ..ops import reference as ref
    os.makedirs(path, exist_ok=True)
    cd = cfg.to_dict()
    if quantize_fp8:
        cd["quantization_config"] = {"quant_method": "fp8", "fmt": "e4m3", "weight_block_size": [128, 128]}
    if quantize_nvfp4:
        cd["quantization_config"] = {"quant_method": "modelopt", "quant_algo": "NVFP4", "group_size": 16}
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cd, f, indent=1)
    shard, size, idx = {}, 0, 0

    def flush():
        nonlocal shard, size, idx
        if shard:
            save_file(shard, os.path.join(path, f"model-{idx:05d}.safetensors"))
            shard, size, idx = {}, 0, idx + 1

    for name, t in weights:
        t = t.detach().cpu()
        big = t.dim() == 2 and name.endswith("proj.weight") and "indexer" not in name and "eh_proj" not in name
        if quantize_nvfp4 and big and ".mlp." in name and t.shape[1] % 16 == 0:
            q, sf, s2 = ref.nvfp4_quant_weight(t.float())
            base = name[: -len(".weight")]
            shard[name] = q.contiguous(); shard[base + ".weight_scale"] = sf.contiguous()
            shard[base + ".weight_scale_2"] = s2.reshape(()).clone(); shard[base + ".input_scale"] = torch.tensor(nvfp4_input_scale)
            size += q.numel() + sf.numel()
        elif quantize_fp8 and big:
            q, s = ref.quant_fp8_block(t)
            shard[name] = q.contiguous(); shard[name + "_scale_inv"] = s.contiguous()
            size += q.numel() + s.numel() * 4
        else:
            shard[name] = t.to(torch.bfloat16).contiguous() if t.dim() >= 1 else t
            size += t.numel() * 2
        if size >= shard_bytes:
            flush()
    flush()
