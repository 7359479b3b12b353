"""Plain-PyTorch statements of every operator.

These are the numerical oracles for the CUDA kernels (tests compare each kernel against the
fp32 form here) and the execution path on CPU, where the engine runs its plumbing tests.
They play the role of the reference's generic back-ends (layers/backends/linear/generic.py,
experts/generic.py:237-273, attention/base.py:451-525 SDPA reference, layers/sampler.py:18-52).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

FP8_MAX = 448.0
FP8 = torch.float8_e4m3fn


# ---- norms -------------------------------------------------------------------------------------
class QAct:
    """A normalised activation in the two forms its consumers take: `x`, the bf16 (or fp32) rows that routers, gathers and
    non-quantised linears read, and - when the producing kernel emitted it - the 1x128 block-quantised copy (`q` e4m3 [T, H],
    `scales` fp32 [H/128, T]) that an fp8 linear multiplies directly.  Norms asked for `quant` return this object (the
    PyTorch statement leaves `q` empty), `linear` accepts it, everything else takes `dense(a)`.  An explicit value instead of
    an attribute riding on the tensor: a view or a cast cannot silently drop the quantised copy.
    Parity: reference layers/base_backend.py:14-26 (PrequantizedActivation) and the shared input quant of
    models/deepseek_v2/deepseek_v2.py:1139-1164."""
    __slots__ = ("x", "q", "scales")

    def __init__(self, x: torch.Tensor, q: Optional[torch.Tensor] = None, scales: Optional[torch.Tensor] = None):
        self.x, self.q, self.scales = x, q, scales

    @property
    def shape(self):
        return self.x.shape

    @property
    def device(self):
        return self.x.device

    @property
    def dtype(self):
        return self.x.dtype

    @property
    def is_cuda(self):
        return self.x.is_cuda


def dense(a):
    """The plain tensor behind an activation, whatever form it travels in."""
    return a.x if isinstance(a, QAct) else a


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, quant: bool = False, unit_offset: bool = False):
    """`quant`: the consumer is an fp8 linear - return a `QAct` (the CUDA body fills in the block-quantised copy).
    `unit_offset`: the stored weight is the deviation from one (Qwen3.5 / Gemma convention), applied as (1 + w) in fp32."""
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    wf = w.float() + 1.0 if unit_offset else w.float()
    y = (y * wf).to(x.dtype)
    return QAct(y) if quant else y


def add_rmsnorm(x: torch.Tensor, residual: Optional[torch.Tensor], w: torch.Tensor, eps: float, unit_offset: bool = False, quant: bool = False):
    """residual_out = x + residual (in the activation dtype); y = rmsnorm(residual_out) (a `QAct` when `quant`)."""
    if residual is not None:
        x = (x.float() + residual.float()).to(x.dtype)
    return rmsnorm(x, w, eps, quant, unit_offset), x


def layernorm(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    return F.layer_norm(x.float(), (x.shape[-1],), w.float(), None if b is None else b.float(), eps).to(x.dtype)


# ---- fp8 block quantisation ----------------------------------------------------------------------
# Process-wide scale format of the fp8 block quantisers (reference models/quant_config.py:39-44, `scale_fmt`): "ue8m0" rounds
# every group scale up to a power of two, the form the Blackwell tensor cores apply themselves.
SCALE_POW2 = [False]


def set_scale_format(fmt: Optional[str]) -> None:
    assert fmt in (None, "fp32", "ue8m0"), fmt
    SCALE_POW2[0] = fmt == "ue8m0"


def scale_format() -> str:
    return "ue8m0" if SCALE_POW2[0] else "fp32"


def _ceil_pow2(s: torch.Tensor) -> torch.Tensor:
    """Smallest power of two >= s, computed on the bits (exact, and the same on every device)."""
    b = s.float().contiguous().view(torch.int32)
    return ((b + 0x7FFFFF) & 0x7F800000).view(torch.float32)


def quant_fp8_1x128(x: torch.Tensor, ue8m0: Optional[bool] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-row, per-128-column groups: q = x / s (e4m3), s = amax/448 (rounded up to 2^k under the "ue8m0" scale format)."""
    if ue8m0 is None:
        ue8m0 = SCALE_POW2[0]
    T, K = x.shape
    assert K % 128 == 0
    g = x.float().view(T, K // 128, 128)
    amax = g.abs().amax(-1).clamp_min(1e-10)
    s = amax / FP8_MAX
    if ue8m0:
        s = _ceil_pow2(s)
    q = (g / s.unsqueeze(-1)).clamp(-FP8_MAX, FP8_MAX).to(FP8).view(T, K)
    return q, s


def dequant_fp8_1x128(q: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    T, K = q.shape
    return (q.float().view(T, K // 128, 128) * s.unsqueeze(-1)).view(T, K)


def quant_fp8_block(w: torch.Tensor, block: int = 128, ue8m0: Optional[bool] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """128x128 weight blocks: returns (w_fp8, weight_scale_inv) with w ~= w_fp8 * scale_inv."""
    if ue8m0 is None:
        ue8m0 = SCALE_POW2[0]
    *lead, N, K = w.shape
    pn, pk = (-N) % block, (-K) % block
    wf = F.pad(w.float(), (0, pk, 0, pn))
    Np, Kp = N + pn, K + pk
    g = wf.view(*lead, Np // block, block, Kp // block, block)
    amax = g.abs().amax(dim=(-3, -1)).clamp_min(1e-10)
    s = amax / FP8_MAX
    if ue8m0:
        s = _ceil_pow2(s)
    q = (g / s.unsqueeze(-1).unsqueeze(-3)).clamp(-FP8_MAX, FP8_MAX).to(FP8)
    q = q.view(*lead, Np, Kp)[..., :N, :K].contiguous()
    return q, s


def fp8_block_for_format(q: torch.Tensor, s: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """A checkpoint's fp8 weight and block scales in the process's scale format: unchanged unless the format is "ue8m0" and
    some scale is not a power of two, in which case the weight is dequantised and quantised again with rounded-up scales."""
    if not SCALE_POW2[0]:
        return q, s
    sf = s.float()
    if bool(((sf.contiguous().view(torch.int32) & 0x7FFFFF) == 0).all()):
        return q, sf
    return quant_fp8_block(dequant_fp8_block(q, sf), ue8m0=True)


def dequant_fp8_block(q: torch.Tensor, s: torch.Tensor, block: int = 128) -> torch.Tensor:
    *lead, N, K = q.shape
    se = s.repeat_interleave(block, -2).repeat_interleave(block, -1)[..., :N, :K]
    return q.float() * se


def linear(x: torch.Tensor, w: torch.Tensor, w_scale: Optional[torch.Tensor] = None, bias=None) -> torch.Tensor:
    """y = x @ w^T.  fp8 weights follow the DeepSeek recipe: activations quantised 1x128, fp32 accumulate."""
    x = dense(x)
    if w.dtype == FP8:
        xq, xs = quant_fp8_1x128(x.reshape(-1, x.shape[-1]))
        y = dequant_fp8_1x128(xq, xs) @ dequant_fp8_block(w, w_scale).t()
        y = y.view(*x.shape[:-1], w.shape[0]).to(x.dtype)
    else:
        y = F.linear(x, w)
    if bias is not None:
        y = y + bias
    return y


# ---- rotary ------------------------------------------------------------------------------------
def yarn_mscale(scale: float, mscale: float) -> float:
    return 1.0 if scale <= 1 else 0.1 * mscale * math.log(scale) + 1.0


def rope_inv_freq(dim: int, theta: float, scaling: Optional[dict]) -> Tuple[torch.Tensor, float]:
    """Inverse frequencies (+ attention-magnitude factor) for plain RoPE and YaRN."""
    inv = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
    if not scaling or scaling.get("type", scaling.get("rope_type")) != "yarn":
        return inv, 1.0
    factor = float(scaling["factor"])
    orig = int(scaling["original_max_position_embeddings"])
    beta_fast, beta_slow = float(scaling.get("beta_fast", 32)), float(scaling.get("beta_slow", 1))

    def corr_dim(n_rot):
        return dim * math.log(orig / (n_rot * 2 * math.pi)) / (2 * math.log(theta))

    low = max(math.floor(corr_dim(beta_fast)), 0)
    high = min(math.ceil(corr_dim(beta_slow)), dim - 1)
    ramp = ((torch.arange(dim // 2, dtype=torch.float32) - low) / max(high - low, 1e-3)).clamp(0, 1)
    inv_mask = 1.0 - ramp
    inv = inv / factor * (1 - inv_mask) + inv * inv_mask
    m = yarn_mscale(factor, float(scaling.get("mscale", 1.0))) / yarn_mscale(factor, float(scaling.get("mscale_all_dim", 0.0)))
    return inv, m


def rope_cos_sin_cache(dim: int, max_pos: int, theta: float, scaling: Optional[dict] = None) -> torch.Tensor:
    """[max_pos, dim] fp32: first half cos, second half sin (already multiplied by the YaRN magnitude)."""
    inv, m = rope_inv_freq(dim, theta, scaling)
    f = torch.outer(torch.arange(max_pos, dtype=torch.float32), inv)
    return torch.cat([f.cos() * m, f.sin() * m], -1)


def apply_rope(x: torch.Tensor, positions: torch.Tensor, cache: torch.Tensor, interleaved: bool) -> torch.Tensor:
    """x [T, ..., D].  interleaved=True rotates pairs (2i, 2i+1) (DeepSeek MLA); False rotates (i, i+D/2) (Qwen)."""
    D = x.shape[-1]
    cs = cache[positions.long()]
    cos, sin = cs[:, : D // 2], cs[:, D // 2:]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [D // 2]
    cos, sin = cos.view(shape), sin.view(shape)
    xf = x.float()
    if interleaved:
        a, b = xf[..., 0::2], xf[..., 1::2]
        out = torch.stack([a * cos - b * sin, b * cos + a * sin], -1).flatten(-2)
    else:
        a, b = xf[..., : D // 2], xf[..., D // 2:]
        out = torch.cat([a * cos - b * sin, b * cos + a * sin], -1)
    return out.to(x.dtype)


# ---- KV cache ------------------------------------------------------------------------------------
def mla_kv_store(cache: torch.Tensor, slot_mapping: torch.Tensor, ckv: torch.Tensor, k_pe: torch.Tensor) -> None:
    """cache [blocks, block_size, R+rope]; row = [normed latent | rotated rope key].
    An fp8 cache stores the clamped e4m3 cast of all R+rope values with no scale
    (reference triton/hopper/fp8_utils.py:275-281)."""
    row = torch.cat([ckv, k_pe], -1)
    flat = cache.view(-1, cache.shape[-1])
    keep = slot_mapping >= 0                     # padded tokens carry slot -1 and write nothing
    slots, row = slot_mapping[keep].long(), row[keep]
    if cache.dtype == FP8:
        row = row.float().clamp(-FP8_MAX, FP8_MAX).to(FP8)
        flat.view(torch.uint8)[slots] = row.view(torch.uint8)
    else:
        flat[slots] = row.to(cache.dtype)


def gqa_kv_store(k_cache, v_cache, slot_mapping, k, v) -> None:
    """k_cache/v_cache [blocks, block_size, kv_heads, head_dim]."""
    k_cache.view(-1, *k_cache.shape[2:])[slot_mapping.long()] = k.to(k_cache.dtype)
    v_cache.view(-1, *v_cache.shape[2:])[slot_mapping.long()] = v.to(v_cache.dtype)


def gqa_qkv_prepare(qkv: torch.Tensor, hq: int, hkv: int, hd: int, q_norm_w, k_norm_w, eps: float, unit_offset: bool, positions,
                    rope_cache: torch.Tensor, k_cache, v_cache, slot_mapping) -> torch.Tensor:
    """The GQA front end after the qkv projection: split [T, (hq + 2 hkv) * hd] into heads, per-head RMSNorm of q and k (when
    the weights are given), rotary embedding of both over the whole head (pairs (i, i + hd/2)), K and V rows stored into their
    paged cache slots.  Returns q [T, hq, hd] (reference models/qwen3_moe/qwen3_moe.py:58-146, triton/generic/kv_store.py:7)."""
    T = qkv.shape[0]
    q, k, v = qkv.split([hq * hd, hkv * hd, hkv * hd], -1)
    q, k, v = q.reshape(T, hq, hd), k.reshape(T, hkv, hd), v.reshape(T, hkv, hd)
    if q_norm_w is not None:
        q = rmsnorm(q.reshape(-1, hd), q_norm_w, eps, False, unit_offset).view(T, hq, hd)
    if k_norm_w is not None:
        k = rmsnorm(k.reshape(-1, hd), k_norm_w, eps, False, unit_offset).view(T, hkv, hd)
    q = apply_rope(q.contiguous(), positions, rope_cache, False)
    k = apply_rope(k.contiguous(), positions, rope_cache, False)
    keep = slot_mapping >= 0
    gqa_kv_store(k_cache, v_cache, slot_mapping[keep], k[keep], v[keep])
    return q


def _gather_rows(cache: torch.Tensor, block_table: torch.Tensor, n: int) -> torch.Tensor:
    bs = cache.shape[1]
    nb = (n + bs - 1) // bs
    rows = cache[block_table[:nb].long()].reshape(nb * bs, *cache.shape[2:])[:n]
    return rows.float() if rows.dtype != FP8 else rows.float()


# ---- attention -----------------------------------------------------------------------------------
def mla_attention_paged(q: torch.Tensor, cache: torch.Tensor, block_tables: torch.Tensor, cu_seqlens_q: torch.Tensor,
                        context_lens: torch.Tensor, scale: float, kv_lora_rank: int,
                        sparse_indices: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Absorbed MLA over the paged latent cache, causal within each sequence.

    q [T, H, R+rope] (already absorbed with W_UK and rotated); returns the latent output [T, H, R].
    Query token t of sequence i sits at absolute position context_len_i - q_len_i + (t - cu_q[i]).
    ``sparse_indices`` [T, topk] (physical token slots, -1 = none) restricts the keys (DSA).
    With an fp8 cache the query is clamped and cast to e4m3 too (reference mla/trtllm.py:93-204).
    """
    T, H, D = q.shape
    out = torch.zeros(T, H, kv_lora_rank, dtype=torch.float32, device=q.device)
    qf = q.float()
    if cache.dtype == FP8:
        qf = qf.clamp(-FP8_MAX, FP8_MAX).to(FP8).float()
    flat = cache.view(-1, cache.shape[-1])
    B = cu_seqlens_q.numel() - 1
    for i in range(B):
        lo, hi = int(cu_seqlens_q[i]), int(cu_seqlens_q[i + 1])
        if hi == lo:
            continue
        n = int(context_lens[i])
        ql = hi - lo
        if sparse_indices is None:
            kv = _gather_rows(cache, block_tables[i], n)                      # [n, D]
            s = torch.einsum("thd,nd->thn", qf[lo:hi], kv) * scale
            pos = torch.arange(n - ql, n, device=q.device).view(ql, 1, 1)
            mask = torch.arange(n, device=q.device).view(1, 1, n) > pos
            s = s.masked_fill(mask, float("-inf"))
            p = torch.softmax(s, -1)
            out[lo:hi] = torch.einsum("thn,nr->thr", p, kv[:, :kv_lora_rank])
        else:
            for t in range(lo, hi):
                idx = sparse_indices[t]
                idx = idx[idx >= 0].long()
                kv = flat[idx].float()
                s = torch.einsum("hd,nd->hn", qf[t], kv) * scale
                p = torch.softmax(s, -1)
                out[t] = torch.einsum("hn,nr->hr", p, kv[:, :kv_lora_rank])
    return out.to(q.dtype)


def gqa_attention_paged(q, k_cache, v_cache, block_tables, cu_seqlens_q, context_lens, scale, window: int = 0) -> torch.Tensor:
    """q [T, Hq, D]; caches [blocks, block_size, Hkv, D]; causal; returns [T, Hq, D].  `window` > 0: a query at position p sees
    key positions (p - window, p] only (sliding-window layers, reference layers/backends/attention/base.py:527-707)."""
    T, Hq, D = q.shape
    Hkv = k_cache.shape[2]
    out = torch.zeros(T, Hq, D, dtype=torch.float32, device=q.device)
    B = cu_seqlens_q.numel() - 1
    for i in range(B):
        lo, hi = int(cu_seqlens_q[i]), int(cu_seqlens_q[i + 1])
        if hi == lo:
            continue
        n, ql = int(context_lens[i]), hi - lo
        k = _gather_rows(k_cache, block_tables[i], n).repeat_interleave(Hq // Hkv, 1)   # [n, Hq, D]
        v = _gather_rows(v_cache, block_tables[i], n).repeat_interleave(Hq // Hkv, 1)
        s = torch.einsum("thd,nhd->thn", q[lo:hi].float(), k) * scale
        pos = torch.arange(n - ql, n, device=q.device).view(ql, 1, 1)
        keys = torch.arange(n, device=q.device).view(1, 1, n)
        s = s.masked_fill(keys > pos, float("-inf"))
        if window > 0:
            s = s.masked_fill(keys <= pos - window, float("-inf"))
        out[lo:hi] = torch.einsum("thn,nhd->thd", torch.softmax(s, -1), v)
    return out.to(q.dtype)


def attention_varlen(q, k, v, cu_seqlens, scale, causal: bool = False) -> torch.Tensor:
    """Attention over ragged sequences: q, k, v [T, H, D]; sequence i owns rows [cu[i], cu[i+1]).  Non-causal by default (the
    vision encoder, reference vl/vision/encoder.py:154-198)."""
    out = torch.empty_like(q)
    cu = cu_seqlens.tolist()
    for i in range(len(cu) - 1):
        lo, hi = cu[i], cu[i + 1]
        if hi == lo:
            continue
        s = torch.einsum("thd,nhd->htn", q[lo:hi].float(), k[lo:hi].float()) * scale
        if causal:
            n = hi - lo
            s = s.masked_fill(torch.ones(n, n, dtype=torch.bool, device=q.device).triu(1), float("-inf"))
        out[lo:hi] = torch.einsum("htn,nhd->thd", torch.softmax(s, -1), v[lo:hi].float()).to(q.dtype)
    return out


def mla_prefill_ragged(q: torch.Tensor, k_nope: torch.Tensor, k_rope: torch.Tensor, v: torch.Tensor, cu_seqlens, scale: float) -> torch.Tensor:
    """Non-absorbed MLA attention of prompts without a cached prefix: q [T, H, nope + rope] (rotary part rotated), k_nope
    [T, H, nope], k_rope [T, rope] shared by the heads, v [T, H, dv]; causal inside each sequence [cu[i], cu[i+1]).  Returns
    [T, H, dv] (reference models/deepseek_v2/deepseek_v2.py:1792-1816)."""
    T, H, _ = q.shape
    k = torch.cat([k_nope.float(), k_rope.float()[:, None, :].expand(T, H, k_rope.shape[-1])], -1)
    out = torch.empty(T, H, v.shape[-1], dtype=torch.float32, device=q.device)
    cu = cu_seqlens.tolist() if isinstance(cu_seqlens, torch.Tensor) else list(cu_seqlens)
    for i in range(len(cu) - 1):
        lo, hi = cu[i], cu[i + 1]
        if hi == lo:
            continue
        n = hi - lo
        s = torch.einsum("thd,nhd->htn", q[lo:hi].float(), k[lo:hi]) * scale
        s = s.masked_fill(torch.ones(n, n, dtype=torch.bool, device=q.device).triu(1), float("-inf"))
        out[lo:hi] = torch.einsum("htn,nhd->thd", torch.softmax(s, -1), v[lo:hi].float())
    return out.to(q.dtype)


def gelu(x: torch.Tensor, tanh: bool = True) -> torch.Tensor:
    return F.gelu(x.float(), approximate="tanh" if tanh else "none").to(x.dtype)


def merge_attention_states(o1, lse1, o2, lse2):
    """Combine two partial attention results over disjoint key sets (LSE-weighted)."""
    m = torch.maximum(lse1, lse2)
    w1, w2 = torch.exp(lse1 - m), torch.exp(lse2 - m)
    o = (o1.float() * w1.unsqueeze(-1) + o2.float() * w2.unsqueeze(-1)) / (w1 + w2).unsqueeze(-1)
    return o.to(o1.dtype), m + torch.log(w1 + w2)


# ---- MoE -----------------------------------------------------------------------------------------
def moe_route(logits: torch.Tensor, bias: Optional[torch.Tensor], top_k: int, n_group: int = 1, topk_group: int = 1,
              norm_topk_prob: bool = True, routed_scaling_factor: float = 1.0, scoring: str = "sigmoid",
              balance_ranks: int = 0, log2phy: Optional[torch.Tensor] = None, logcnt: Optional[torch.Tensor] = None):
    """DeepSeek ``noaux_tc`` routing and Qwen3 softmax routing.

    scores = sigmoid|softmax|sqrt(softplus) (logits fp32; the last is DeepSeek-V4's, reference models/deepseek_v4/deepseek_v4.py:40-47); choice = scores + bias; with n_group > 1 only the
    topk_group groups with the largest sum of their top-2 choices stay eligible; idx = top_k of
    choice; weights are the un-biased scores, renormalised and scaled
    (reference models/deepseek_v2/deepseek_v2.py:478-543, models/qwen3_moe/qwen3_moe.py:283-297).

    Two optional post-steps on the ids (the weights stay those of the chosen experts): `balance_ranks` > 0 replaces them by
    ids dealt evenly over that many expert-parallel ranks (a load-balance stand-in for random-init routers, reference
    layers/backends/experts/deep_gemm.py:47-67); `log2phy [E, R]` / `logcnt [E]` map every logical id to one of its
    physical replicas, picked by (row, k) hash so replicas share the load (reference experts/eplb.py, triton/generic/moe.py:561).
    """
    lf = logits.float()
    if lf.dim() == 3:          # partial sums of a split-K router product
        lf = lf.sum(0)
    scores = (torch.sigmoid(lf) if scoring == "sigmoid" else F.softplus(lf).sqrt() if scoring == "sqrtsoftplus" else torch.softmax(lf, -1))
    choice = scores + bias.float() if bias is not None else scores
    T, E = choice.shape
    if n_group > 1:
        g = choice.view(T, n_group, E // n_group)
        gs = g.topk(2, -1).values.sum(-1)
        keep = gs.topk(topk_group, -1).indices
        gmask = torch.zeros(T, n_group, dtype=torch.bool, device=logits.device).scatter_(1, keep, True)
        choice = choice.masked_fill(~gmask.unsqueeze(-1).expand(T, n_group, E // n_group).reshape(T, E), float("-inf"))
    idx = choice.topk(top_k, -1).indices
    w = scores.gather(1, idx)
    if norm_topk_prob:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    if balance_ranks > 0:
        i = torch.arange(T * top_k, device=idx.device).view(T, top_k)
        step = E // balance_ranks
        idx = ((i // balance_ranks) % step + (i % balance_ranks) * step) % E
    elif log2phy is not None:
        cnt = logcnt.to(idx.device).long()[idx]
        t = torch.arange(T, device=idx.device).view(T, 1)
        k = torch.arange(top_k, device=idx.device).view(1, top_k)
        h = (((t * 2654435761 + k * 40503) & 0xFFFFFFFF) >> 8) % cnt
        idx = log2phy.to(idx.device).long()[idx, h]
    return idx.to(torch.int32), (w * routed_scaling_factor).float()


_E2M1 = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def mxfp4_dequant(packed: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """OCP MXFP4 -> fp32.  packed [rows, cols / 2] uint8 holds two e2m1 values per byte (the even column in the low nibble);
    scale [rows, cols / 32] uint8 holds one e8m0 exponent (2^(s - 127)) per 32 consecutive columns."""
    p = packed.view(torch.uint8)
    lut = torch.tensor(_E2M1 + tuple(-v for v in _E2M1), dtype=torch.float32, device=p.device)
    lo, hi = lut[(p & 0xF).long()], lut[(p >> 4).long()]
    w = torch.stack([lo, hi], -1).reshape(p.shape[0], p.shape[1] * 2)
    sc = torch.exp2(scale.view(torch.uint8).float() - 127.0)
    return (w.view(p.shape[0], -1, 32) * sc.unsqueeze(-1)).reshape(p.shape[0], -1)


def mxfp4_quant(w: torch.Tensor):
    """fp32 [rows, cols] (cols a multiple of 32) -> (packed uint8 [rows, cols / 2], e8m0 scales uint8 [rows, cols / 32]); the
    inverse of `mxfp4_dequant` up to rounding (nearest e2m1 value, power-of-two scale that maps the block maximum to <= 6)."""
    r, c = w.shape
    blk = w.float().view(r, c // 32, 32)
    amax = blk.abs().amax(-1).clamp_min(2.0 ** -126)
    e = torch.ceil(torch.log2(amax / 6.0)).clamp(-127, 127)
    q = blk / torch.exp2(e).unsqueeze(-1)
    lut = torch.tensor(_E2M1, dtype=torch.float32, device=w.device)
    mag = (q.abs().unsqueeze(-1) - lut).abs().argmin(-1)
    code = (mag + (q < 0).long() * 8).view(r, c).to(torch.uint8)
    packed = code[:, 0::2] | (code[:, 1::2] << 4)
    return packed.contiguous(), (e + 127).to(torch.uint8).contiguous()


def glu_act(a: torch.Tensor, b: torch.Tensor, act=None) -> torch.Tensor:
    """Gated activation of (gate a, up b) in fp32.  act None: silu(a) b.  ("gelu_tanh",): tanh-approximated GELU(a) b.  ("clamp", L): up in [-L, L], gate <= L, then
    silu(a) b (reference layers/activation.py:86-92).  ("situ", beta, linear_beta): beta tanh(a / beta) sigmoid(a) times
    linear_beta tanh(b / linear_beta) (no clamp of b when linear_beta is None; reference kernel/triton/generic/situ.py:24-27)."""
    if act is None:
        return F.silu(a) * b
    if act[0] == "clamp":
        L = float(act[1])
        return F.silu(a.clamp(max=L)) * b.clamp(-L, L)
    if act[0] == "gelu_tanh":
        return F.gelu(a, approximate="tanh") * b
    if act[0] == "situ":
        beta, lb = float(act[1]), act[2]
        if lb:
            b = float(lb) * torch.tanh(b / float(lb))
        return beta * torch.tanh(a / beta) * torch.sigmoid(a) * b
    raise ValueError(f"unknown gated activation {act!r}")


def silu_and_mul(x: torch.Tensor, quant: bool = False, act=None) -> torch.Tensor:
    """`quant` is a hint for the CUDA body (emit only the block-quantised form for an fp8 consumer); ignored here."""
    a, b = x.float().chunk(2, -1)
    return glu_act(a, b, act).to(x.dtype)


def moe_experts(x, topk_idx, topk_w, w13, w2, w13_scale=None, w2_scale=None, expert_offset: int = 0, add_in=None, act=None) -> torch.Tensor:
    """Routed experts held locally: ids [expert_offset, expert_offset + E_local).  w13 [E, 2I, H], w2 [E, H, I].
    Returns the weighted sum over the local experts of each token (zeros where none is local).  `act`: see `glu_act`."""
    if callable(add_in):
        add_in = add_in()
    T, H = x.shape
    E = w13.shape[0]
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    for e in range(E):
        sel = (topk_idx == e + expert_offset)
        tok, slot = sel.nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        xe = x[tok]
        h = linear(xe, w13[e], None if w13_scale is None else w13_scale[e])
        h = silu_and_mul(h, act=act)
        y = linear(h, w2[e], None if w2_scale is None else w2_scale[e])
        out.index_add_(0, tok, y.float() * topk_w[tok, slot].unsqueeze(-1))
    out = out.to(x.dtype)
    return out if add_in is None else out + add_in


# ---- NVFP4 (packed e2m1 + one e4m3 scale per 16 elements + one fp32 scale per tensor) ---------------------------------
_E2M1 = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def _e2m1_codes(v: torch.Tensor) -> torch.Tensor:
    """Round to the nearest e2m1 value (ties to the even code, saturating at 6); returns 4-bit codes with the sign in bit 3."""
    grid = torch.tensor(_E2M1, dtype=torch.float32, device=v.device)
    d = (v.abs().unsqueeze(-1) - grid).abs() + torch.tensor([0.0, 1e-6] * 4, device=v.device)     # a tie goes to the even code
    code = d.argmin(-1)
    return (code | ((v < 0) & (code > 0)).long() << 3).to(torch.uint8)


def nvfp4_quant(x: torch.Tensor, gscale: torch.Tensor, row_group: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """x [R, K] -> (packed e2m1 uint8 [R, K/2], e4m3 scales [R, K/16]) with x ~= q * sf / gscale.  `gscale` (= 1 / input_scale of
    a ModelOpt checkpoint) is one number, or one per group with `row_group` [R] naming each row's group.
    Parity: the flashinfer `fp4_quantize` recipe the reference calls (layers/backends/experts/nvfp4.py:318-326)."""
    R, K = x.shape
    assert K % 16 == 0
    g = gscale.float().reshape(-1)
    g = g[0].expand(R) if row_group is None else g[row_group.long()]
    v = x.float().view(R, K // 16, 16)
    sf = (g.view(R, 1) * v.abs().amax(-1) / 6.0).clamp(max=FP8_MAX).to(FP8)
    sfv = sf.float()
    os = torch.where(sfv != 0, g.view(R, 1) / sfv.clamp_min(1e-30), torch.zeros_like(sfv))
    codes = _e2m1_codes(v * os.unsqueeze(-1)).view(R, K)
    return (codes[:, 0::2] | (codes[:, 1::2] << 4)).contiguous(), sf


def nvfp4_unpack(q: torch.Tensor, sf: torch.Tensor) -> torch.Tensor:
    """Packed e2m1 [..., K/2] and e4m3 scales [..., K/16] -> fp32 [..., K] (without the per-tensor scale)."""
    grid = torch.tensor(_E2M1 + tuple(-a for a in _E2M1), dtype=torch.float32, device=q.device)
    lo, hi = (q & 0xF).long(), (q >> 4).long()
    v = torch.stack([grid[lo], grid[hi]], -1).flatten(-2)
    return (v.view(*v.shape[:-1], -1, 16) * sf.float().unsqueeze(-1)).flatten(-2)


def nvfp4_quant_weight(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """The ModelOpt NVFP4 weight format: (packed [..., N, K/2], weight_scale e4m3 [..., N, K/16], weight_scale_2 fp32 per matrix)
    with w ~= e2m1 * weight_scale * weight_scale_2."""
    *lead, N, K = w.shape
    wf = w.float().reshape(-1, N, K)
    s2 = (wf.abs().amax(dim=(1, 2)) / (6.0 * FP8_MAX)).clamp_min(1e-12)
    qs, sfs = [], []
    for m, s in zip(wf, s2):
        q, sf = nvfp4_quant(m, (1.0 / s).reshape(1))
        qs.append(q); sfs.append(sf)
    return torch.stack(qs).view(*lead, N, K // 2), torch.stack(sfs).view(*lead, N, K // 16), s2.view(*lead) if lead else s2[0]


def nvfp4_gemm(a_q, a_sf, b_q, b_sf, alpha, masked_m=None, row_start=None, out_fp32: bool = False) -> torch.Tensor:
    """D = alpha[g] * (A_g B_g^T) over NVFP4 operands.  A [R, K/2] with B [G, N, K/2] in the contiguous grouped layout (row_start /
    masked_m as in the fp8 grouped GEMM) or G = 1; rows outside every group's range come back as zeros."""
    G, N = b_q.shape[0], b_q.shape[1]
    A = nvfp4_unpack(a_q, a_sf)
    out = torch.zeros(A.shape[0], N, dtype=torch.float32, device=A.device)
    al = torch.ones(G, device=A.device) if alpha is None else alpha.float().reshape(-1)
    for g in range(G):
        lo = 0 if row_start is None else int(row_start[g])
        n = A.shape[0] if masked_m is None else int(masked_m[g])
        if n > 0:
            out[lo:lo + n] = A[lo:lo + n] @ nvfp4_unpack(b_q[g], b_sf[g]).t() * al[g]
    return out if out_fp32 else out.to(torch.bfloat16)


def moe_experts_nvfp4(x, topk_idx, topk_w, w13_q, w13_sf, alpha1, a1_gscale, w2_q, w2_sf, alpha2, a2_gscale, expert_offset: int = 0,
                      add_in=None, act=None) -> torch.Tensor:
    """Routed experts with NVFP4 weights and activations (W4A4).  w13_q [E, 2I, H/2], w2_q [E, H, I/2] packed e2m1 with e4m3
    block scales; `a1_gscale` (one number) and `a2_gscale` [E] are the reciprocals of the checkpoint's input scales, `alpha1` /
    `alpha2` [E] = input_scale * weight_scale_2.  Parity: reference layers/backends/experts/nvfp4.py:143-160,205-220."""
    if callable(add_in):
        add_in = add_in()
    T, H = x.shape
    E = w13_q.shape[0]
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    for e in range(E):
        tok, slot = (topk_idx == e + expert_offset).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        xe = x[tok].to(torch.bfloat16)
        aq, asf = nvfp4_quant(xe, a1_gscale.reshape(-1)[:1])
        h = nvfp4_gemm(aq, asf, w13_q[e:e + 1], w13_sf[e:e + 1], alpha1[e:e + 1])
        h = silu_and_mul(h, act=act)
        hq, hsf = nvfp4_quant(h, a2_gscale.reshape(-1)[e:e + 1])
        y = nvfp4_gemm(hq, hsf, w2_q[e:e + 1], w2_sf[e:e + 1], alpha2[e:e + 1])
        out.index_add_(0, tok, y.float() * topk_w[tok, slot].unsqueeze(-1))
    out = out.to(x.dtype)
    return out if add_in is None else out + add_in


# ---- sampling ------------------------------------------------------------------------------------
def sample(logits: torch.Tensor, temperatures: torch.Tensor, generator: Optional[torch.Generator] = None,
           return_logprobs: bool = False):
    """Gumbel-max in log space with per-row temperature; rows with temperature < 1e-5 are greedy."""
    lf = logits.float()
    greedy = temperatures < 1e-5
    if bool(greedy.all()):
        tok = lf.argmax(-1)
    else:
        t = torch.where(greedy, torch.ones_like(temperatures), temperatures).unsqueeze(-1)
        u = torch.rand(lf.shape, generator=generator, device=lf.device, dtype=torch.float32).clamp_min(1e-20)
        g = -torch.log(-torch.log(u))
        tok = torch.where(greedy, lf.argmax(-1), (lf / t + g).argmax(-1))
    if not return_logprobs:
        return tok, None
    lp = torch.log_softmax(lf, -1).gather(1, tok.unsqueeze(-1)).squeeze(-1)
    return tok, lp


# ---- DSA lightning indexer -------------------------------------------------------------------------
def hadamard(x: torch.Tensor) -> torch.Tensor:
    """Normalised fast Walsh-Hadamard transform over the last dim (a power of two)."""
    n = x.shape[-1]
    y = x.float().reshape(-1, n)
    h = 1
    while h < n:
        y = y.view(-1, n // (2 * h), 2, h)
        y = torch.stack([y[:, :, 0] + y[:, :, 1], y[:, :, 0] - y[:, :, 1]], 2).reshape(-1, n)
        h *= 2
    return (y * n ** -0.5).view(x.shape).to(x.dtype)


def quant_fp8_per_token_pow2(x: torch.Tensor):
    """One power-of-two scale per row (indexer keys / queries)."""
    amax = x.float().abs().amax(-1, keepdim=True).clamp_min(1e-4)
    s = torch.exp2(torch.ceil(torch.log2(amax / FP8_MAX)))
    return (x.float() / s).clamp(-FP8_MAX, FP8_MAX).to(FP8), s.squeeze(-1)


def indexer_logits(q_fp8, q_scale, head_w, k_fp8, k_scale) -> torch.Tensor:
    """score(i, j) = sum_h w[i,h] * relu(q[i,h] . k[j]) (reference dsa/indexer/lightning.py:116-162).
    q_fp8 [T, Hi, D], q_scale [T, Hi], head_w [T, Hi], k_fp8 [N, D], k_scale [N] -> [T, N] fp32."""
    s = torch.einsum("thd,nd->thn", q_fp8.float(), k_fp8.float())
    s = torch.relu(s) * (q_scale.float() * head_w.float()).unsqueeze(-1)
    return s.sum(1) * k_scale.float().unsqueeze(0)


def indexer_topk(logits: torch.Tensor, valid_len: torch.Tensor, topk: int) -> torch.Tensor:
    """Row-wise top-k of the first valid_len[i] entries; -1 pads.  Returns int32 [T, topk] (logical positions)."""
    T, N = logits.shape
    masked = logits.masked_fill(torch.arange(N, device=logits.device).unsqueeze(0) >= valid_len.unsqueeze(1), float("-inf"))
    k = min(topk, N)
    v, idx = masked.topk(k, -1)
    idx = idx.masked_fill(torch.isinf(v), -1).to(torch.int32)
    if k < topk:
        idx = F.pad(idx, (0, topk - k), value=-1)
    return idx


def logical_to_physical(idx: torch.Tensor, block_table_rows: torch.Tensor, block_size: int) -> torch.Tensor:
    """block_table[idx // bs] * bs + idx % bs, -1 stays -1 (reference topk.cuh:250-430)."""
    safe = idx.clamp_min(0).long()
    phys = block_table_rows.gather(1, safe // block_size).long() * block_size + safe % block_size
    return torch.where(idx >= 0, phys, torch.full_like(phys, -1)).to(torch.int32)


def indexer_k_store(k: torch.Tensor, ln_w: torch.Tensor, ln_b: Optional[torch.Tensor], eps: float, positions: torch.Tensor,
                    rope_cache: torch.Tensor, rope_dim: int, cache: torch.Tensor, slots: torch.Tensor) -> None:
    """Indexer key path: LayerNorm -> RoPE on the first rope_dim dims (half-split pairs) -> Hadamard -> one power-of-two
    scale per token -> e4m3, written into the indexer cache.  cache [blocks, bs*(D+4)] uint8: key row `off` of a page
    sits at off*D, its fp32 scale at bs*D + off*4 (reference dsa/indexer/lightning.py:408-535, IndexerCache)."""
    D = k.shape[-1]
    k = layernorm(k, ln_w, ln_b, eps)
    k = torch.cat([apply_rope(k[..., :rope_dim], positions, rope_cache, False), k[..., rope_dim:]], -1)
    k8, ks = quant_fp8_per_token_pow2(hadamard(k))
    keep = slots >= 0
    slots, k8, ks = slots[keep], k8[keep], ks[keep]
    bs = cache.shape[1] // (D + 4)
    blk, off = (slots // bs).long(), (slots % bs).long()
    flat, page = cache.view(-1), cache.shape[1]
    kidx = (blk * page + off * D).unsqueeze(1) + torch.arange(D, device=cache.device)
    flat[kidx.reshape(-1)] = k8.view(torch.uint8).reshape(-1)
    sidx = (blk * page + bs * D + off * 4).unsqueeze(1) + torch.arange(4, device=cache.device)
    flat[sidx.reshape(-1)] = ks.float().contiguous().view(torch.uint8).reshape(-1)


def indexer_q_prep(q: torch.Tensor, positions: torch.Tensor, rope_cache: torch.Tensor, rope_dim: int):
    """Indexer query path: q [T, Hi, D] -> RoPE (first rope_dim dims) -> Hadamard -> per-(token, head) power-of-two scale
    -> (e4m3 [T, Hi, D], scales [T, Hi])."""
    T, Hi, D = q.shape
    q = torch.cat([apply_rope(q[..., :rope_dim], positions, rope_cache, False), q[..., rope_dim:]], -1)
    q8, qs = quant_fp8_per_token_pow2(hadamard(q).reshape(T * Hi, D))
    return q8.view(T, Hi, D), qs.view(T, Hi)


def indexer_gather(cache: torch.Tensor, block_table: torch.Tensor, n: int, D: int):
    bs = cache.shape[1] // (D + 4)
    nb = (n + bs - 1) // bs
    pages = cache[block_table[:nb].long()]
    keys = pages[:, : bs * D].reshape(nb * bs, D).view(FP8)[:n]
    scales = pages[:, bs * D:].contiguous().view(torch.float32).reshape(nb * bs)[:n]
    return keys, scales


def indexer_select(q8: torch.Tensor, q_scale: torch.Tensor, head_w: torch.Tensor, cache: torch.Tensor, block_tables: torch.Tensor,
                   cu_seqlens_q, context_lens, topk: int, logical: bool = False) -> torch.Tensor:
    """Per token: physical slots of the `topk` visible keys with the largest indexer score, -1 padded ([T, topk] int32).
    cu_seqlens_q / context_lens: host lists or tensors.  `logical`: return key positions instead of physical slots (the
    hot / cold tier maps them itself)."""
    T, Hi, D = q8.shape
    cu = cu_seqlens_q.tolist() if isinstance(cu_seqlens_q, torch.Tensor) else list(cu_seqlens_q)
    cl = context_lens.tolist() if isinstance(context_lens, torch.Tensor) else list(context_lens)
    bs = cache.shape[1] // (D + 4)
    out = torch.full((T, topk), -1, dtype=torch.int32, device=q8.device)
    for i in range(len(cl)):
        lo, hi = cu[i], cu[i + 1]
        if hi == lo:
            continue
        n = cl[i]
        keys, kscale = indexer_gather(cache, block_tables[i], n, D)
        logits = indexer_logits(q8[lo:hi], q_scale[lo:hi], head_w[lo:hi], keys, kscale)
        valid = torch.arange(n - (hi - lo) + 1, n + 1, device=q8.device)
        idx = indexer_topk(logits, valid, topk)
        out[lo:hi] = idx if logical else logical_to_physical(idx, block_tables[i:i + 1].expand(hi - lo, -1), bs)
    return out


# ---- hot / cold tier of the sparse-attention cache --------------------------------------------------------------------------
def hisparse_stage(L: dict, sel: torch.Tensor, slots: torch.Tensor, context_lens: torch.Tensor, block_tables: torch.Tensor):
    """Make the listed key positions of every sequence resident in its hot buffer and return their hot row ids.

    L: one layer's tier tensors (runtime/hisparse.py::HiSparseTier.layer).  sel [B, topk] key positions, -1 padded; the token
    being decoded sits at position context_len - 1 and always gets a row (the key kernel writes it afterwards, nothing is
    copied for it).  Positions already resident are stamped as used in this step; the others take, in ring order from the
    slot's cursor, rows that were not used in this step, evict their occupants and are copied in from the cold pages.
    Returns (hot_ids [B, topk] int32: slot * hot_rows + row, or -1; new_slot [B] int64: hot row id of the new token)."""
    p2h, h2p, stamp, cursor, stepc, cold, hot = L["pos_to_hot"], L["hot_to_pos"], L["stamp"], L["cursor"], L["step"], L["cold"], L["hot"]
    page_rows = L["page_rows"]
    B, topk = sel.shape
    hot_rows, max_ctx = h2p.shape[1], p2h.shape[1]
    out = torch.full((B, topk), -1, dtype=torch.int32, device=sel.device)
    new_slot = torch.zeros(B, dtype=torch.int64, device=sel.device)
    step = int(stepc[0]) + 1
    cold_rows = cold.reshape(-1, cold.shape[-1])
    for b in range(B):
        s = int(slots[b])
        new_pos = int(context_lens[b]) - 1
        row0 = s * hot_rows
        misses, i_new = [], -1
        for i, p in enumerate(sel[b].tolist()):
            if p < 0 or p >= max_ctx:
                continue
            if p == new_pos:
                i_new = i
                continue
            h = int(p2h[s, p])
            if h >= 0:
                stamp[s, h] = step
                out[b, i] = row0 + h
            else:
                misses.append(i)
        hn, need_new = -1, False
        if 0 <= new_pos < max_ctx:
            hn = int(p2h[s, new_pos])
            if hn >= 0:
                stamp[s, hn] = step
            else:
                need_new = True
        need = len(misses) + int(need_new)
        cur, victims, scanned = int(cursor[s]), [], 0
        for j in range(hot_rows):
            if len(victims) >= need:
                break
            h = (cur + j) % hot_rows
            if int(stamp[s, h]) != step:
                victims.append(h)
                scanned = j + 1

        def take(h, p):
            old = int(h2p[s, h])
            if old >= 0:
                p2h[s, old] = -1
            h2p[s, h] = p; p2h[s, p] = h; stamp[s, h] = step

        if need_new and victims:
            hn = victims[0]
            take(hn, new_pos)
        new_slot[b] = row0 + (hn if hn >= 0 else 0)
        if i_new >= 0 and hn >= 0:
            out[b, i_new] = row0 + hn
        for m, i in enumerate(misses):
            v = m + int(need_new)
            if v >= len(victims):
                continue                                  # hot buffer smaller than one step's demand: the key is dropped
            p, h = int(sel[b, i]), victims[v]
            take(h, p)
            out[b, i] = row0 + h
            page = int(block_tables[b, p // page_rows])
            hot[row0 + h] = cold_rows[page * page_rows + p % page_rows].to(hot.device)
        cursor[s] = (cur + scanned) % hot_rows
    stepc[0] = step
    return out, new_slot


def hisparse_writeback(hot: torch.Tensor, cold: torch.Tensor, new_slot: torch.Tensor, slot_mapping: torch.Tensor) -> None:
    """Copy the row just written for every sequence from its hot row to its logical row of the cold pages."""
    cold_rows = cold.reshape(-1, cold.shape[-1])
    cold_rows[slot_mapping.long().to(cold.device)] = hot[new_slot.long()].to(cold.device)


# ---- small GEMM-shaped helpers -------------------------------------------------------------------
def kmajor(w: torch.Tensor) -> torch.Tensor:
    """w [H, A, B] -> [H, B, A] contiguous, the operand layout the CUDA body of `bmm_absorb` multiplies with."""
    return w.transpose(1, 2).contiguous()


def bmm_absorb(x: torch.Tensor, w: torch.Tensor, out=None, wt=None) -> torch.Tensor:
    """Per-head matmul of MLA weight absorption: x [T, H, A], w [H, A, B] -> [T, H, B].  `wt` (the K-major copy of `w` that
    the weight's owner keeps for the CUDA body) is not needed here."""
    r = torch.einsum("tha,hab->thb", x.float(), w.float()).to(x.dtype)
    if out is not None:
        out.copy_(r)
        return out
    return r


def mla_absorb_rope(q: torch.Tensor, kc: torch.Tensor, positions: torch.Tensor, cache: torch.Tensor, nope: int, kc_t=None) -> torch.Tensor:
    """Absorbed MLA query [q_nope @ W_UK | rope(q_pe)]: q [T, H, nope + rope], kc [H, nope, R] -> [T, H, R + rope]."""
    return torch.cat([bmm_absorb(q[..., :nope], kc), apply_rope(q[..., nope:], positions, cache, True)], -1)


def mla_query(q: torch.Tensor, kc: torch.Tensor, positions: torch.Tensor, rope_cache: torch.Tensor, nope: int, kv_cache: torch.Tensor,
              dense: bool = True, kc_t=None) -> torch.Tensor:
    """Absorbed MLA query as the attention operator wants it.  The CUDA body may hand back e4m3 (clamped cast, no scale)
    when `kv_cache` is fp8 and the dense fp8 attention kernel will consume it; this statement always returns q's dtype."""
    return mla_absorb_rope(q, kc, positions, rope_cache, nope)


def mla_kv_prepare(kv_a: torch.Tensor, norm_w: torch.Tensor, eps: float, positions: torch.Tensor, rope_cache: torch.Tensor,
                   kv_cache: torch.Tensor, slot_mapping: torch.Tensor, R: int) -> None:
    """MLA key path: kv_a [T, R + rope] -> cache rows [RMSNorm(kv_a[:, :R]) | rope(kv_a[:, R:])] at `slot_mapping`
    (reference models/deepseek_v2/deepseek_v2.py:1139-1164 key half, then the KV write of T5)."""
    ckv = rmsnorm(kv_a[:, :R], norm_w, eps)
    k_pe = apply_rope(kv_a[:, R:], positions, rope_cache, True)
    mla_kv_store(kv_cache, slot_mapping, ckv, k_pe)


def router_logits(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """MoE router GEMM in fp32: x [T, H] (any dtype), w [E, H] fp32 -> [T, E] fp32."""
    return F.linear(x.float(), w.float())


def lm_head(hidden: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """Vocabulary projection; logits are returned in fp32."""
    return F.linear(hidden, w).float()


# ---- gated delta-net linear attention (Qwen3.5 family) -----------------------------------------------------
#
# Parity: reference runtime/layers/backends/delta_net/generic.py:170-329 (layer orchestration),
# components/conv.py (causal depthwise convolution with a carried window), components/recurrence.py:100-200
# (the delta rule, state [.., V, K]), components/output.py:17-62 (gated RMSNorm).

def gdn_conv(x: torch.Tensor, weight: torch.Tensor, conv_state: torch.Tensor, slots: torch.Tensor, cu_seqlens: torch.Tensor,
             fresh: torch.Tensor, uniform_one: bool = False) -> torch.Tensor:
    """Causal depthwise convolution + SiLU over ragged sequences, carrying a window of the last K-1 inputs per sequence.

    x [T, C]; weight [C, K]; conv_state [S, K-1, C] (this layer's pool, oldest input first); slots [B]; cu_seqlens [B+1];
    fresh [B] non-zero where the sequence starts here (its window is taken as zeros).  Returns y [T, C] in x's dtype and
    writes each sequence's new window back to its slot."""
    K = weight.shape[1]
    y = torch.empty_like(x)
    cu = cu_seqlens.tolist()
    w = weight.float()
    for i in range(len(cu) - 1):
        s, e = cu[i], cu[i + 1]
        if e <= s:
            continue
        slot = int(slots[i])
        win = conv_state[slot].float()
        if int(fresh[i]):
            win = torch.zeros_like(win)
        full = torch.cat([win, x[s:e].float()], 0)                     # [K-1 + n, C]
        acc = torch.zeros(e - s, x.shape[1], dtype=torch.float32, device=x.device)
        for j in range(K):
            acc += full[j: j + (e - s)] * w[:, j]
        y[s:e] = torch.nn.functional.silu(acc).to(x.dtype)
        conv_state[slot] = full[-(K - 1):].to(conv_state.dtype)
    return y


def gdn_gates(a: torch.Tensor, b: torch.Tensor, A_log: torch.Tensor, dt_bias: torch.Tensor):
    """log-decay g = -exp(A_log) * softplus(a + dt_bias) and write strength beta = sigmoid(b), both fp32 [T, Hv]."""
    g = -A_log.float().exp() * torch.nn.functional.softplus(a.float() + dt_bias.float())
    return g, b.float().sigmoid()


def _l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    return x * torch.rsqrt((x * x).sum(-1, keepdim=True) + eps)


def gdn_scan(q, k, v, g, beta, S):
    """Token-by-token delta rule for one sequence.  q, k [n, H, Dk] (normalised, q scaled); v [n, H, Dv]; g, beta [n, H];
    S [H, Dv, Dk] fp32.  Returns (o [n, H, Dv] fp32, S)."""
    out = []
    for t in range(q.shape[0]):
        S = S * g[t].exp()[:, None, None]
        Sk = torch.einsum("hvk,hk->hv", S, k[t])
        S = S + (beta[t][:, None] * (v[t] - Sk))[:, :, None] * k[t][:, None, :]
        out.append(torch.einsum("hvk,hk->hv", S, q[t]))
    return torch.stack(out, 0), S


def gdn_chunked(q, k, v, g, beta, S, chunk: int = 64):
    """The same recurrence evaluated chunk by chunk with matrix products (what a tensor-core prefill does).

    Inside a chunk with cumulative log-decay G_t, the per-token writes u_t solve the unit-lower-triangular system
    (I + A) U = beta * (V - exp(G) * K S0^T) with A[t, i] = beta_t exp(G_t - G_i) k_t.k_i for i < t; then
    o_t = exp(G_t) S0 q_t + sum_{i<=t} exp(G_t - G_i) (k_i.q_t) u_i and S_C = exp(G_C) S0 + sum_i exp(G_C - G_i) u_i k_i^T."""
    n, H, Dk = q.shape
    Dv = v.shape[-1]
    pad = (-n) % chunk
    if pad:
        z = lambda t: torch.cat([t, t.new_zeros(pad, *t.shape[1:])], 0)
        q, k, v, g, beta = z(q), z(k), z(v), z(g), z(beta)      # padded tokens: g = 0 (no decay), beta = 0 (no write)
    nc = (n + pad) // chunk
    # [H, nc, C, *]
    rs = lambda t: t.reshape(nc, chunk, H, -1).permute(2, 0, 1, 3)
    qc, kc, vc = rs(q), rs(k), rs(v)
    gc, bc = rs(g).squeeze(-1), rs(beta).squeeze(-1)             # [H, nc, C]
    G = gc.cumsum(-1)
    diff = G[..., :, None] - G[..., None, :]                     # G_t - G_i
    tril = torch.ones(chunk, chunk, dtype=torch.bool, device=q.device).tril()
    decay = torch.where(tril, diff, torch.full_like(diff, float("-inf"))).exp()          # i <= t
    kk = kc @ kc.transpose(-1, -2)
    A = (bc[..., :, None] * decay * kk).masked_fill(~tril.tril(-1), 0.0)
    eye = torch.eye(chunk, dtype=q.dtype, device=q.device)
    Tm = torch.linalg.solve_triangular(eye + A, eye.expand_as(A).contiguous(), upper=False)
    W = Tm @ (bc[..., None] * G.exp()[..., None] * kc)          # [H, nc, C, Dk]
    U0 = Tm @ (bc[..., None] * vc)                              # [H, nc, C, Dv]
    qk = (qc @ kc.transpose(-1, -2)) * decay                     # [H, nc, C(t), C(i)]
    eG = G.exp()[..., None]
    gl = G[..., -1]                                              # [H, nc]
    kdec = (gl[..., None] - G).exp()[..., None] * kc             # exp(G_C - G_i) k_i
    out = torch.empty(H, nc, chunk, Dv, dtype=q.dtype, device=q.device)
    for c in range(nc):
        St = S.transpose(-1, -2)                                 # [H, Dk, Dv]
        U = U0[:, c] - W[:, c] @ St
        out[:, c] = eG[:, c] * (qc[:, c] @ St) + qk[:, c] @ U
        S = gl[:, c].exp()[:, None, None] * S + U.transpose(-1, -2) @ kdec[:, c]
    o = out.permute(1, 2, 0, 3).reshape(nc * chunk, H, Dv)[:n]
    return o, S


def rmsnorm_gated(x: torch.Tensor, z: torch.Tensor, w: torch.Tensor, eps: float, out: Optional[torch.Tensor] = None,
                  sigmoid: bool = False) -> torch.Tensor:
    """w * rmsnorm(x) * silu(z) over the last dimension; result in z's dtype.  `sigmoid`: x * rstd * w * sigmoid(z) in fp32."""
    xf = x.float()
    if sigmoid:
        y = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float() * torch.sigmoid(z.float())).to(z.dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y
    xn = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(z.dtype)
    y = (w.to(z.dtype) * xn) * torch.nn.functional.silu(z.float()).to(z.dtype)
    if out is not None:
        out.copy_(y)
        return out
    return y


def kda_gates(raw_g: torch.Tensor, b: torch.Tensor, A_log: torch.Tensor, dt_bias: torch.Tensor, lower_bound: Optional[float]):
    """Kimi delta attention gates.  raw_g [T, H, Dk], b [T, H], A_log [H], dt_bias [H * Dk].  The log-decay per key channel is
    L * sigmoid(exp(A) (raw_g + bias)) when a lower bound L < 0 is given, else -exp(A) softplus(raw_g + bias); the write
    strength is sigmoid(b) (reference kernel/triton/fla/fused_recurrent.py:505-530)."""
    T, H, Dk = raw_g.shape
    x = raw_g.float() + dt_bias.float().view(1, H, Dk)
    A = A_log.float().exp().view(1, H, 1)
    g = lower_bound * torch.sigmoid(A * x) if lower_bound is not None and lower_bound < 0 else -A * torch.nn.functional.softplus(x)
    return g, b.float().sigmoid()


def kda_scan(q, k, v, g, beta, S):
    """Token-by-token delta rule with a decay per key channel.  q, k [n, H, Dk]; v [n, H, Dv]; g [n, H, Dk]; beta [n, H];
    S [H, Dv, Dk] fp32."""
    out = []
    for t in range(q.shape[0]):
        S = S * g[t].exp()[:, None, :]
        Sk = torch.einsum("hvk,hk->hv", S, k[t])
        S = S + (beta[t][:, None] * (v[t] - Sk))[:, :, None] * k[t][:, None, :]
        out.append(torch.einsum("hvk,hk->hv", S, q[t]))
    return torch.stack(out, 0), S


def kda_recurrent(q, k, v, raw_g, b, A_log, dt_bias, lower_bound, state, slots, cu_seqlens, fresh, gate, norm_w, eps: float) -> torch.Tensor:
    """Kimi delta attention over ragged sequences with a per-sequence state, followed by the sigmoid-gated RMSNorm
    x * rstd * w * sigmoid(gate) (reference layers/backends/delta_net/kda.py:300-377).  q, k [T, H, Dk], v and gate
    [T, H, Dv]; state [S, H, Dv, Dk] fp32.  Returns [T, H * Dv] in v's dtype."""
    T, H, Dk = q.shape
    Dv = v.shape[2]
    g, beta = kda_gates(raw_g.reshape(T, H, Dk), b, A_log, dt_bias, lower_bound)
    qn = _l2norm(q.float()) * (Dk ** -0.5)
    kn = _l2norm(k.float())
    vf = v.float()
    o = torch.empty(T, H, Dv, dtype=torch.float32, device=v.device)
    cu = cu_seqlens.tolist()
    for i in range(len(cu) - 1):
        s, e = cu[i], cu[i + 1]
        if e <= s:
            continue
        slot = int(slots[i])
        S = torch.zeros_like(state[slot]) if int(fresh[i]) else state[slot].clone()
        o[s:e], S = kda_scan(qn[s:e], kn[s:e], vf[s:e], g[s:e], beta[s:e], S)
        state[slot] = S
    y = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + eps) * norm_w.float() * torch.sigmoid(gate.float())
    return y.to(v.dtype).reshape(T, H * Dv)


def sigmoid_mul(o: torch.Tensor, g: torch.Tensor) -> torch.Tensor:
    """o * sigmoid(g) over rows [T, W] (g may be a strided view)."""
    return (o.float() * torch.sigmoid(g.float())).to(o.dtype)


def attn_res_mix(prefix: torch.Tensor, bank: torch.Tensor, valid: int, w_score: torch.Tensor, w_out: torch.Tensor, eps: float,
                 write_row: int = -1) -> torch.Tensor:
    """Block attention residual.  prefix [T, D] is the running sum since the last block boundary, bank [T, rows, D] holds the
    frozen block sums of which the first `valid` count.  Every candidate (bank rows, then the prefix) gets the score
    (cand . w_score) * rsqrt(mean(cand^2) + eps); the softmax mixture of the candidates is rounded to the activation dtype
    and RMS-normalised with `w_out`.  `write_row` >= 0 also stores the prefix into that bank row.
    Parity: reference models/kimi_k3/kimi_k3.py:103-161, kernel/triton/kimi_k3/attn_residual.py:17-140."""
    cand = torch.cat([bank[:, :valid], prefix[:, None]], 1).float()
    sc = (cand * w_score.float()).sum(-1) * torch.rsqrt(cand.square().mean(-1) + eps)
    mix = (sc.softmax(-1)[..., None] * cand).sum(1).to(prefix.dtype)
    if write_row >= 0:
        bank[:, write_row].copy_(prefix)
    return rmsnorm(mix, w_out, eps)


def mhc_split_weights(fn: torch.Tensor) -> torch.Tensor:
    """fp32 coefficient matrix [M, W] -> bf16 [2M padded to a multiple of 8, W]: rows [0, M) its bf16 rounding, rows [M, 2M)
    the bf16 rounding of what the first rows miss.  A bf16 product against both halves, added, equals the fp32 product to
    ~2^-17 relative."""
    hi = fn.float().to(torch.bfloat16)
    lo = (fn.float() - hi.float()).to(torch.bfloat16)
    rows = (2 * fn.shape[0] + 7) // 8 * 8
    out = torch.zeros(rows, fn.shape[1], dtype=torch.bfloat16, device=fn.device)
    out[: fn.shape[0]] = hi
    out[fn.shape[0]: 2 * fn.shape[0]] = lo
    return out


def mhc_pre(x: torch.Tensor, fn: torch.Tensor, base: torch.Tensor, scale: torch.Tensor, iters: int, eps: float, fn_split=None):
    """Hyper-connection pre-mix (`fn_split` is the CUDA body's prepared operand; unused here).  x [T, h, D] streams; fn [(2+h)h, h*D], base [(2+h)h], scale [3] fp32.  Returns the
    contracted sub-layer input y [T, D] and the post weights [T, h] and stream-mixing matrix [T, h, h] for `mhc_post`.
    Parity: reference models/glm5_next/glm5_next.py:27-70."""
    T, h, D = x.shape
    flat = x.flatten(1).float()
    r = torch.rsqrt(flat.square().mean(-1, keepdim=True) + eps)
    mixes = F.linear(flat, fn.float()) * r
    pre = torch.sigmoid(mixes[:, :h] * scale[0] + base[:h]) + eps
    post = 2 * torch.sigmoid(mixes[:, h: 2 * h] * scale[1] + base[h: 2 * h])
    comb = mixes[:, 2 * h:].view(T, h, h) * scale[2] + base[2 * h:].view(h, h)
    comb = comb.softmax(-1) + eps
    comb = comb / (comb.sum(-2, keepdim=True) + eps)
    for _ in range(max(0, iters - 1)):
        comb = comb / (comb.sum(-1, keepdim=True) + eps)
        comb = comb / (comb.sum(-2, keepdim=True) + eps)
    pre = pre.to(x.dtype)
    y = (pre.float().unsqueeze(-1) * x.float()).sum(1)
    return y.to(x.dtype), post.to(x.dtype), comb.to(x.dtype)


def mhc_post(x: torch.Tensor, res: torch.Tensor, post: torch.Tensor, comb: torch.Tensor) -> torch.Tensor:
    """Hyper-connection post-mix: out[t, i] = post[t, i] x[t] + sum_j comb[t, j, i] res[t, j]; x [T, D], res [T, h, D].
    Parity: reference models/glm5_next/glm5_next.py:96-97."""
    out = post.float().unsqueeze(-1) * x.float().unsqueeze(1) + torch.einsum("tji,tjd->tid", comb.float(), res.float())
    return out.to(res.dtype)


def sigmoid_gate(o: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """o * sigmoid(gate), the output gate of the hybrid family's full-attention layers (gate may be a strided view)."""
    return (o.float() * torch.sigmoid(gate.float())).to(o.dtype)


GDN_CHUNK_MIN_TOKENS = 64      # sequences at least this long go through the chunked form


def gdn_recurrent(q, k, v, a, b, A_log, dt_bias, state, slots, cu_seqlens, fresh, z, norm_w, eps: float, max_q_len: int = 1,
                  cu_host=None) -> torch.Tensor:
    """Gated delta rule over ragged sequences with a per-sequence state, followed by the gated RMSNorm.

    q, k [T, Hk, Dk] and v [T, Hv, Dv] are the convolved projections (Hv a multiple of Hk: value head h reads key head
    h // (Hv/Hk)); a, b [T, Hv]; state [S, Hv, Dv, Dk] fp32 (this layer's pool); slots [B]; cu_seqlens [B+1]; fresh [B];
    z [T, Hv, Dv] the output gate.  Returns [T, Hv*Dv] in v's dtype.  `max_q_len` and `cu_host` are planning hints for the
    CUDA body (which form to run, sequence boundaries without a device read-back); unused here."""
    T, Hk, Dk = q.shape
    Hv, Dv = v.shape[1], v.shape[2]
    rep = Hv // Hk
    g, beta = gdn_gates(a, b, A_log, dt_bias)
    qn = _l2norm(q.float()).repeat_interleave(rep, 1) * (Dk ** -0.5)
    kn = _l2norm(k.float()).repeat_interleave(rep, 1)
    vf = v.float()
    o = torch.empty(T, Hv, Dv, dtype=torch.float32, device=v.device)
    cu = cu_seqlens.tolist()
    for i in range(len(cu) - 1):
        s, e = cu[i], cu[i + 1]
        if e <= s:
            continue
        slot = int(slots[i])
        S = torch.zeros_like(state[slot]) if int(fresh[i]) else state[slot].clone()
        if e - s >= GDN_CHUNK_MIN_TOKENS:
            o[s:e], S = gdn_chunked(qn[s:e], kn[s:e], vf[s:e], g[s:e], beta[s:e], S)
        else:
            o[s:e], S = gdn_scan(qn[s:e], kn[s:e], vf[s:e], g[s:e], beta[s:e], S)
        state[slot] = S
    return rmsnorm_gated(o, z, norm_w, eps).reshape(T, Hv * Dv)


# ---- MTP draft verification -------------------------------------------------------------------------------
def mtp_greedy_verify(logits: torch.Tensor, drafts: torch.Tensor):
    """logits [B, N+1, V], drafts [B, N].  Returns (num_accepted [B] in 0..N, next_token [B]): the longest prefix with
    argmax(row_i) == d_{i+1}; the next token is the argmax of the first mismatching row, or of the bonus row
    (reference runtime/runner/mtp_runner.py:190-208)."""
    am = logits.argmax(-1)                                   # [B, N+1]
    match = (am[:, :-1] == drafts).to(torch.int64)
    acc = match.cumprod(1).sum(1)                            # [B]
    nxt = am.gather(1, acc.unsqueeze(1)).squeeze(1)
    return acc, nxt


def mtp_rejection_sample(logits: torch.Tensor, drafts: torch.Tensor, temperatures: torch.Tensor,
                         generator: Optional[torch.Generator] = None, uniforms: Optional[torch.Tensor] = None,
                         have: Optional[torch.Tensor] = None):
    """Speculative sampling for greedy (one-hot) drafts (reference runtime/runner/mtp_runner.py:111-187).

    Draft d_{i+1} is accepted with probability p_target(d_{i+1} | row i), one uniform coin per position; the accepted count
    is the length of the all-accepted prefix.  The next token is sampled from the target row at the first rejection with the
    rejected draft masked out (from the bonus row, unmasked, when everything was accepted) - which preserves the target
    distribution.  Rows with temperature < 1e-5 fall back to greedy verification.
    Returns (num_accepted [B], next_token [B], logprob_of_next [B] under the unmasked target row).
    """
    B, N1, V = logits.shape
    N = N1 - 1
    greedy = temperatures < 1e-5
    t = torch.where(greedy, torch.ones_like(temperatures), temperatures).view(B, 1, 1)
    logp = torch.log_softmax(logits.float() / t, -1)          # [B, N+1, V]
    p_draft = logp[:, :N].gather(2, drafts.long().unsqueeze(-1)).squeeze(-1).exp()    # [B, N]
    if uniforms is None:
        uniforms = torch.rand(B, N, generator=generator, device=logits.device, dtype=torch.float32)
    accept = (uniforms < p_draft).to(torch.int64)
    has = torch.ones(B, dtype=torch.bool, device=logits.device) if have is None else have.to(logits.device) != 0
    accept = accept * has.view(B, 1).to(torch.int64)
    acc = accept.cumprod(1).sum(1)
    row = logp.gather(1, acc.view(B, 1, 1).expand(B, 1, V)).squeeze(1)               # target row at the stop position
    masked = row.clone()
    rejected = (acc < N) & has
    if N > 0:
        rej_tok = drafts.long().gather(1, acc.clamp_max(N - 1).unsqueeze(1)).squeeze(1)
        masked[rejected, rej_tok[rejected]] = float("-inf")
    u = torch.rand(B, V, generator=generator, device=logits.device, dtype=torch.float32).clamp_min(1e-20)
    nxt = (masked - torch.log(-torch.log(u))).argmax(-1)
    g_acc, g_nxt = mtp_greedy_verify(logits, drafts)
    g_acc = torch.where(has, g_acc, torch.zeros_like(g_acc))
    g_nxt = torch.where(has, g_nxt, logits[:, 0].argmax(-1))
    acc = torch.where(greedy, g_acc, acc)
    nxt = torch.where(greedy, g_nxt, nxt)
    row = logp.gather(1, acc.view(B, 1, 1).expand(B, 1, V)).squeeze(1)
    return acc, nxt, row.gather(1, nxt.unsqueeze(1)).squeeze(1)


def mtp_verify(logits: torch.Tensor, drafts: torch.Tensor, temperatures: torch.Tensor, have: Optional[torch.Tensor] = None,
               coins: Optional[torch.Tensor] = None, generator: Optional[torch.Generator] = None, force_accept: Optional[int] = None,
               want_logprob: bool = False, seed: Optional[int] = None, seed_buf: Optional[torch.Tensor] = None):
    """One verify step for every sequence: logits [B, N+1, V] of rows [last token, d1..dN], drafts [B, N], temperatures [B],
    `have` [B] (0 = the sequence carries no drafts: nothing is accepted), `coins` [B, N] uniforms of the acceptance test.
    Returns (num_accepted int32 [B], next_token int64 [B], bundle int64 [B, N+1] = accepted drafts + next token, -1 beyond,
    extend_tokens int64 [B, N+1] = the predictor's token inputs for the draft-extend pass, logprob fp32 [B] or None).
    `force_accept` pins the accepted count and takes the arg-max of that row (benchmarks)."""
    B, N1, V = logits.shape
    N = N1 - 1
    drafts = drafts.long()
    lp = None
    if force_accept is not None:
        acc = torch.full((B,), min(force_accept, N), dtype=torch.int64, device=logits.device)
        nxt = logits.argmax(-1).gather(1, acc.unsqueeze(1)).squeeze(1)
    elif bool((temperatures < 1e-5).all()):
        acc, nxt = mtp_greedy_verify(logits, drafts)
        if have is not None:
            keep = have.to(logits.device) != 0
            acc = torch.where(keep, acc, torch.zeros_like(acc))
            nxt = torch.where(keep, nxt, logits[:, 0].argmax(-1))
    else:
        acc, nxt, lp = mtp_rejection_sample(logits, drafts, temperatures, generator, coins, have)
    if want_logprob or lp is not None:
        t = torch.where(temperatures < 1e-5, torch.ones_like(temperatures), temperatures).view(B, 1)
        row = logits.float().gather(1, acc.view(B, 1, 1).expand(B, 1, V)).squeeze(1) / t
        lp = torch.log_softmax(row, -1).gather(1, nxt.unsqueeze(1)).squeeze(1)
    idx = torch.arange(N1, device=logits.device).view(1, N1)
    dpad = torch.cat([drafts, drafts.new_zeros(B, 1)], 1)
    a = acc.view(B, 1)
    bundle = torch.where(idx < a, dpad, torch.where(idx == a, nxt.view(B, 1), torch.full_like(dpad, -1)))
    ext = torch.where(idx < a, dpad, nxt.view(B, 1).expand(B, N1))
    return acc.to(torch.int32), nxt, bundle, ext, lp


def mtp_chain_meta(base_len, num_accepted, block_tables, block_size: int, k: int, positions, slot_mapping, context_lens) -> None:
    """Positions, cache slots and context lengths of chain step `k` of the draft predictor: the token drafted at step k sits at
    position base_len + num_accepted + k - 1."""
    pos = (base_len.long() + num_accepted.long() + (k - 1))
    positions.copy_(pos)
    context_lens.copy_((pos + 1).to(context_lens.dtype))
    page = block_tables.long().gather(1, (pos // block_size).unsqueeze(1)).squeeze(1)
    slot_mapping.copy_(page * block_size + pos % block_size)


# ---- DeepSeek-V4: compressed KV + window attention with a sink -----------------------------------------------------------------
def fp8_qdq_pow2(x: torch.Tensor, block: int = 64) -> torch.Tensor:
    """Round-trip through e4m3 with one power-of-two scale per `block` values of the last dim (what a cache that stores the
    rows as fp8 would return).  Parity: reference models/deepseek_v4/deepseek_v4.py:549-590."""
    if x.numel() == 0:
        return x
    shape = x.shape
    v = x.float().reshape(-1, shape[-1] // block, block)
    amax = v.abs().amax(-1, keepdim=True).clamp(min=1e-4)
    s = torch.exp2(torch.ceil(torch.log2(amax / 448.0)))
    return ((v / s).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).float() * s).reshape(shape).to(x.dtype)


def dsv4_compress_extend(kv: torch.Tensor, score: torch.Tensor, kv_state: torch.Tensor, score_state: torch.Tensor, pos0: int, ratio: int,
                         d: int) -> torch.Tensor:
    """Feed `n` new tokens (positions pos0 .. pos0+n-1) of one sequence to a DeepSeek-V4 KV compressor and return the pooled
    rows [nb, d] fp32 of every block of `ratio` tokens that the new tokens complete (block j of the result starts at position
    (pos0 - pos0 % ratio) + j * ratio).

    kv / score [n, c*d] fp32 are the token projections (score already carries the position-in-block bias); c = 2 for ratio 4
    ("overlap": a block pools the second halves of its own rows together with the first halves of the previous block's rows),
    else 1.  kv_state / score_state [c*ratio, c*d] fp32 carry the rows of the unfinished block (and, with overlap, of the
    previous block) between calls and are updated in place; a fresh sequence starts from zeros / -inf.
    Parity: reference models/deepseek_v4/deepseek_v4.py:979-1077 (whole-prompt form), :1079-1176 (one token)."""
    overlap = kv.shape[1] == 2 * d
    off = ratio if overlap else 0
    m = pos0 % ratio
    full_kv = torch.cat([kv_state[off: off + m], kv], 0)
    full_sc = torch.cat([score_state[off: off + m], score], 0)
    nb = full_kv.shape[0] // ratio
    rem = full_kv.shape[0] - nb * ratio
    pooled = kv.new_zeros(0, d)
    if nb:
        bk = full_kv[: nb * ratio].view(nb, ratio, -1)
        bs = full_sc[: nb * ratio].view(nb, ratio, -1)
        if overlap:
            pk = torch.cat([kv_state[None, :ratio], bk[:-1]], 0)           # the block before each block
            ps = torch.cat([score_state[None, :ratio], bs[:-1]], 0)
            k2 = torch.cat([pk[..., :d], bk[..., d:]], 1)                  # [nb, 2r, d]
            s2 = torch.cat([ps[..., :d], bs[..., d:]], 1)
            pooled = (k2 * s2.softmax(1)).sum(1)
            kv_state[:ratio] = bk[-1]
            score_state[:ratio] = bs[-1]
        else:
            pooled = (bk * bs.softmax(1)).sum(1)
    kv_state[off:] = 0
    score_state[off:] = float("-inf")
    if rem:
        kv_state[off: off + rem] = full_kv[nb * ratio:]
        score_state[off: off + rem] = full_sc[nb * ratio:]
    return pooled


def sink_attention(q: torch.Tensor, kv: torch.Tensor, mask: torch.Tensor, sink: torch.Tensor, scale: float) -> torch.Tensor:
    """Multi-query attention whose keys are also its values, with one learned "sink" logit per head in the softmax denominator.
    q [T, H, D]; kv [T, L, D] (per-token candidate rows) or [L, D] (shared); mask [T, L] bool (True = attend); sink [H] fp32.
    A token with nothing to attend returns zeros.  Parity: reference models/deepseek_v4/deepseek_v4.py:1676-1704."""
    qf, kf = q.float(), kv.float()
    s = (torch.einsum("thd,tld->thl", qf, kf) if kv.dim() == 3 else torch.einsum("thd,ld->thl", qf, kf)) * scale
    s = s.masked_fill(~mask.unsqueeze(1), float("-inf"))
    mx = torch.maximum(s.amax(-1), sink.float().view(1, -1))
    p = torch.exp(s - mx.unsqueeze(-1))
    p = p / (p.sum(-1, keepdim=True) + torch.exp(sink.float().view(1, -1, 1) - mx.unsqueeze(-1)))
    p = p.to(q.dtype).float()
    return (torch.einsum("thl,tld->thd", p, kf) if kv.dim() == 3 else torch.einsum("thl,ld->thd", p, kf)).to(q.dtype)


def dsv4_compress_decode(kv: torch.Tensor, score: torch.Tensor, kv_states: torch.Tensor, score_states: torch.Tensor, slots: torch.Tensor,
                         positions: torch.Tensor, ratio: int, d: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """`dsv4_compress_extend` for one new token of each of B sequences at once, without a host read: kv / score [B, c*d],
    the carry pools [slots, c*ratio, c*d] (updated in place at rows `slots`), positions [B].  Returns the pooled rows [B, d]
    (zeros where the token does not finish a block) and the mask of sequences that finished one."""
    overlap = kv.shape[1] == 2 * d
    off = ratio if overlap else 0
    slots, m = slots.long(), positions.long() % ratio
    kv_states[slots, off + m] = kv
    score_states[slots, off + m] = score
    done = m == ratio - 1
    dm = done.view(-1, 1, 1)
    ks, ss = kv_states[slots], score_states[slots]
    if overlap:
        k2 = torch.cat([ks[:, :ratio, :d], ks[:, ratio:, d:]], 1)
        s2 = torch.cat([ss[:, :ratio, :d], ss[:, ratio:, d:]], 1)
    else:
        k2, s2 = ks, ss
    s2 = torch.where(dm, s2, torch.zeros_like(s2))                  # rows that pool nothing stay finite
    pooled = torch.where(done.unsqueeze(1), (k2 * s2.softmax(1)).sum(1), torch.zeros_like(k2[:, 0]))
    if overlap:                                                       # the finished block becomes the previous one
        kv_states[slots, :ratio] = torch.where(dm, ks[:, ratio:], ks[:, :ratio])
        score_states[slots, :ratio] = torch.where(dm, ss[:, ratio:], ss[:, :ratio])
    kv_states[slots, off:] = torch.where(dm, torch.zeros_like(ks[:, off:]), ks[:, off:])
    score_states[slots, off:] = torch.where(dm, torch.full_like(ss[:, off:], float("-inf")), ss[:, off:])
    return pooled, done


def dsv4_row_bytes(d: int, rd: int) -> int:
    """Bytes of one packed DeepSeek-V4 cache row: (d - rd) e4m3 values, rd bf16 values, one e8m0 scale byte per 64 e4m3 values
    padded (by at least one byte) to a multiple of 8.  584 for d = 512, rd = 64.
    Parity: reference models/deepseek_v4/deepseek_v4.py:592-612 (448 + 128 + 8)."""
    tiles = (d - rd) // 64
    return (d - rd) + 2 * rd + ((tiles + 8) // 8) * 8


def dsv4_pack_rows(kv: torch.Tensor, rd: int) -> torch.Tensor:
    """kv [N, d] -> uint8 [N, dsv4_row_bytes(d, rd)]: [e4m3 values | bf16 rotated dims | e8m0 scale bytes, zero padded].  The
    scale of a 64-value tile is the power of two fp8_qdq_pow2 uses, so rows that went through it are stored without loss."""
    N, d = kv.shape
    nope = d - rd
    tiles = nope // 64
    v = kv[:, :nope].float().reshape(N, tiles, 64)
    e = torch.ceil(torch.log2(v.abs().amax(-1).clamp(min=1e-4) / 448.0))                       # [N, tiles]
    q = (v / torch.exp2(e).unsqueeze(-1)).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).view(torch.uint8).reshape(N, nope)
    rope = kv[:, nope:].to(torch.bfloat16).contiguous().view(torch.uint8).reshape(N, 2 * rd)
    sc = torch.zeros(N, dsv4_row_bytes(d, rd) - nope - 2 * rd, dtype=torch.uint8, device=kv.device)
    sc[:, :tiles] = (e + 127).clamp(0, 254).to(torch.uint8)
    return torch.cat([q, rope, sc], 1)


def dsv4_unpack_rows(rows: torch.Tensor, d: int, rd: int, dtype=torch.float32) -> torch.Tensor:
    """uint8 [..., row_bytes] -> [..., d] in `dtype`."""
    nope = d - rd
    tiles = nope // 64
    lead = rows.shape[:-1]
    r = rows.reshape(-1, rows.shape[-1])
    q = r[:, :nope].contiguous().view(torch.float8_e4m3fn).float().reshape(-1, tiles, 64)
    s = torch.exp2(r[:, nope + 2 * rd: nope + 2 * rd + tiles].float() - 127.0).unsqueeze(-1)
    rope = r[:, nope: nope + 2 * rd].contiguous().view(torch.bfloat16).float()
    return torch.cat([(q * s).reshape(-1, nope), rope], 1).to(dtype).reshape(*lead, d)
