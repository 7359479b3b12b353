"""A dense, non-paged, non-batched, non-absorbed restatement of the DeepSeek-V3 forward pass working directly
on HF-named weights.  It shares no code with the engine's model and serves as its oracle."""
import math

import torch
import torch.nn.functional as F


def _rms(x, w, eps):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def _rope_interleaved(x, pos, theta):
    d = x.shape[-1]
    inv = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float64) / d))
    f = torch.outer(pos.double(), inv)
    cos, sin = f.cos().float(), f.sin().float()
    while cos.dim() < x.dim():
        cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    a, b = x[..., 0::2], x[..., 1::2]
    return torch.stack([a * cos - b * sin, b * cos + a * sin], -1).flatten(-2)


def dense_forward(cfg, W, tokens):
    """tokens: list[int] -> logits [len, vocab] (fp32)."""
    T = len(tokens)
    pos = torch.arange(T)
    h = W["model.embed_tokens.weight"][torch.tensor(tokens)].float()
    H, R, rope, nope, v = cfg.num_attention_heads, cfg.kv_lora_rank, cfg.qk_rope_head_dim, cfg.qk_nope_head_dim, cfg.v_head_dim
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        x = _rms(h, W[p + "input_layernorm.weight"], cfg.rms_norm_eps)
        a = p + "self_attn."
        if cfg.q_lora_rank:
            qc = _rms(x @ W[a + "q_a_proj.weight"].t(), W[a + "q_a_layernorm.weight"], cfg.rms_norm_eps)
            q = qc @ W[a + "q_b_proj.weight"].t()
        else:
            q = x @ W[a + "q_proj.weight"].t()
        q = q.view(T, H, nope + rope)
        kva = x @ W[a + "kv_a_proj_with_mqa.weight"].t()
        ckv = _rms(kva[:, :R], W[a + "kv_a_layernorm.weight"], cfg.rms_norm_eps)
        kpe = _rope_interleaved(kva[:, R:], pos, cfg.rope_theta)
        kv = (ckv @ W[a + "kv_b_proj.weight"].t()).view(T, H, nope + v)
        k = torch.cat([kv[..., :nope], kpe.unsqueeze(1).expand(T, H, rope)], -1)
        qq = torch.cat([q[..., :nope], _rope_interleaved(q[..., nope:], pos, cfg.rope_theta)], -1)
        s = torch.einsum("thd,shd->hts", qq, k) * (nope + rope) ** -0.5
        s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
        o = torch.einsum("hts,shv->thv", torch.softmax(s, -1), kv[..., nope:]).reshape(T, H * v)
        h = h + o @ W[a + "o_proj.weight"].t()
        x = _rms(h, W[p + "post_attention_layernorm.weight"], cfg.rms_norm_eps)
        m = p + "mlp."
        if cfg.is_moe_layer(i):
            scores = torch.sigmoid(x @ W[m + "gate.weight"].t()) if cfg.scoring_func == "sigmoid" else torch.softmax(x @ W[m + "gate.weight"].t(), -1)
            choice = scores + W.get(m + "gate.e_score_correction_bias", 0)
            if cfg.n_group > 1:
                g = choice.view(T, cfg.n_group, -1)
                keep = g.topk(2, -1).values.sum(-1).topk(cfg.topk_group, -1).indices
                mask = torch.zeros(T, cfg.n_group, dtype=torch.bool).scatter_(1, keep, True)
                choice = choice.masked_fill(~mask.repeat_interleave(g.shape[-1], 1), float("-inf"))
            idx = choice.topk(cfg.num_experts_per_tok, -1).indices
            w = scores.gather(1, idx)
            if cfg.norm_topk_prob:
                w = w / w.sum(-1, keepdim=True)
            w = w * cfg.routed_scaling_factor
            y = torch.zeros_like(x)
            for t in range(T):
                for j in range(idx.shape[1]):
                    e = int(idx[t, j])
                    ep = m + f"experts.{e}."
                    u = F.silu(x[t] @ W[ep + "gate_proj.weight"].t()) * (x[t] @ W[ep + "up_proj.weight"].t())
                    y[t] += w[t, j] * (u @ W[ep + "down_proj.weight"].t())
            if cfg.n_shared_experts:
                sp = m + "shared_experts."
                u = F.silu(x @ W[sp + "gate_proj.weight"].t()) * (x @ W[sp + "up_proj.weight"].t())
                y = y + u @ W[sp + "down_proj.weight"].t()
        else:
            u = F.silu(x @ W[m + "gate_proj.weight"].t()) * (x @ W[m + "up_proj.weight"].t())
            y = u @ W[m + "down_proj.weight"].t()
        h = h + y
    h = _rms(h, W["model.norm.weight"], cfg.rms_norm_eps)
    return h @ W["lm_head.weight"].t()
