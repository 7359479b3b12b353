"""Qwen3-VL style vision transformer: patches -> embeddings the language model consumes in place of its image tokens.

A patch is `in_channels x temporal_patch x patch x patch` pixels flattened by the image processor; the encoder embeds it with
one matrix product, adds a learned position embedding interpolated bilinearly to the image's patch grid, runs `depth` blocks of
(LayerNorm, non-causal attention over the patches of one frame with a 2-D rotary embedding, LayerNorm, GELU MLP) and merges
every `merge x merge` neighbourhood into one output token through a two-layer MLP.

Parity: reference vl/vision/encoder.py - rotary table :41-72, MLP :75-91, patch embedding :94-122, merger :125-151, attention
:154-198, block :201-230, model :233-465 (rot_pos_emb :308-352, position interpolation :354-423, forward :425-465).

B200-first differences: every product goes through the tcgen05 GEMM of this package, LayerNorm / GELU / rotary are its CUDA
kernels, and attention addresses q / k / v in place through the generic paged-attention kernel (one row per "page", no padding
to the longest image, no per-image Python loop).
"""
from __future__ import annotations

import json
import os
import re
from dataclasses import dataclass, field, fields
from typing import Iterable, List, Tuple

import torch
import torch.nn as nn

from .. import ops
from ..models.layers import QLinear


@dataclass
class VisionConfig:
    hidden_size: int = 1152
    num_heads: int = 16
    depth: int = 27
    intermediate_size: int = 4304
    out_hidden_size: int = 4096
    in_channels: int = 3
    patch_size: int = 16
    temporal_patch_size: int = 2
    spatial_merge_size: int = 2
    num_position_embeddings: int = 2304
    hidden_act: str = "gelu_pytorch_tanh"
    deepstack_visual_indexes: List[int] = field(default_factory=list)

    @classmethod
    def from_dict(cls, d) -> "VisionConfig":
        known = {f.name for f in fields(cls)}
        return cls(**{k: v for k, v in dict(d).items() if k in known})

    @classmethod
    def from_pretrained(cls, path: str) -> "VisionConfig":
        with open(os.path.join(path, "config.json")) as f:
            d = json.load(f)
        return cls.from_dict(d.get("vision_config", d))

    @property
    def patch_dim(self) -> int:
        return self.in_channels * self.temporal_patch_size * self.patch_size * self.patch_size


class _LayerNorm(nn.Module):
    def __init__(self, dim, dtype, device, eps=1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype, device=device), requires_grad=False)
        self.bias = nn.Parameter(torch.zeros(dim, dtype=dtype, device=device), requires_grad=False)
        self.eps = eps

    def forward(self, x):
        return ops.layernorm(x, self.weight, self.bias, self.eps)


class VisionBlock(nn.Module):
    def __init__(self, c: VisionConfig, dtype, device):
        super().__init__()
        H = c.hidden_size
        self.heads, self.hd = c.num_heads, H // c.num_heads
        self.norm1, self.norm2 = _LayerNorm(H, dtype, device), _LayerNorm(H, dtype, device)
        self.qkv = QLinear(H, 3 * H, dtype, device, None, bias=True)
        self.proj = QLinear(H, H, dtype, device, None, bias=True)
        self.fc1 = QLinear(H, c.intermediate_size, dtype, device, None, bias=True)
        self.fc2 = QLinear(c.intermediate_size, H, dtype, device, None, bias=True)
        self.tanh = c.hidden_act == "gelu_pytorch_tanh"

    def forward(self, x, cu_seqlens, rope_rows, arange):
        T = x.shape[0]
        qkv = self.qkv(self.norm1(x)).view(T, 3, self.heads, self.hd)
        q = ops.apply_rope(qkv[:, 0].contiguous(), arange, rope_rows, False)
        k = ops.apply_rope(qkv[:, 1].contiguous(), arange, rope_rows, False)
        o = ops.attention_varlen(q, k, qkv[:, 2].contiguous(), cu_seqlens, self.hd ** -0.5, False)
        x = x + self.proj(o.reshape(T, -1))
        return x + self.fc2(ops.gelu(self.fc1(self.norm2(x)), self.tanh))


class PatchMerger(nn.Module):
    def __init__(self, c: VisionConfig, dtype, device, postshuffle_norm: bool = False):
        super().__init__()
        self.merged = c.hidden_size * c.spatial_merge_size ** 2
        self.post = postshuffle_norm
        self.norm = _LayerNorm(self.merged if postshuffle_norm else c.hidden_size, dtype, device)
        self.fc1 = QLinear(self.merged, self.merged, dtype, device, None, bias=True)
        self.fc2 = QLinear(self.merged, c.out_hidden_size, dtype, device, None, bias=True)

    def forward(self, x):
        x = self.norm(x.reshape(-1, self.merged)) if self.post else self.norm(x).reshape(-1, self.merged)
        return self.fc2(ops.gelu(self.fc1(x), False))


class VisionModel(nn.Module):
    def __init__(self, c: VisionConfig, dtype=torch.bfloat16, device="cpu"):
        super().__init__()
        self.cfg, self.dtype = c, dtype
        self.patch_embed = QLinear(c.patch_dim, c.hidden_size, dtype, device, None, bias=True)
        self.pos_embed = nn.Embedding(c.num_position_embeddings, c.hidden_size, dtype=dtype, device=device)
        self.side = int(c.num_position_embeddings ** 0.5)
        self.blocks = nn.ModuleList([VisionBlock(c, dtype, device) for _ in range(c.depth)])
        self.merger = PatchMerger(c, dtype, device)
        hd = c.hidden_size // c.num_heads
        self.register_buffer("inv_freq", 1.0 / (10000.0 ** (torch.arange(0, hd // 2, 2, dtype=torch.float32) / (hd // 2))).to(device), persistent=False)
        for p in self.parameters():
            p.requires_grad_(False)

    # ---- positions ---------------------------------------------------------------------------
    def _token_coords(self, grids: List[Tuple[int, int, int]]) -> torch.Tensor:
        """(row, column) of every token in the order the image processor emits patches: merge x merge neighbourhoods are
        contiguous, neighbourhoods row-major, frames one after another."""
        m = self.cfg.spatial_merge_size
        out = []
        for t, h, w in grids:
            r = (torch.arange(h // m)[:, None, None, None] * m + torch.arange(m)[None, None, :, None]).expand(h // m, w // m, m, m)
            c = (torch.arange(w // m)[None, :, None, None] * m + torch.arange(m)[None, None, None, :]).expand(h // m, w // m, m, m)
            out.append(torch.stack([r.reshape(-1), c.reshape(-1)], -1).repeat(t, 1))
        return torch.cat(out)

    def rope_rows(self, grids) -> torch.Tensor:
        """[T, head_dim] fp32 (cos | sin): the first quarter of the rotary angles follows the row, the second the column."""
        coords = self._token_coords(grids).to(self.inv_freq.device).float()
        ang = torch.cat([coords[:, :1] * self.inv_freq, coords[:, 1:] * self.inv_freq], -1)          # [T, head_dim / 2]
        return torch.cat([ang.cos(), ang.sin()], -1).contiguous()

    def pos_embed_rows(self, grids) -> torch.Tensor:
        """Learned position embedding interpolated bilinearly from the side x side table to each image's h x w grid, in token order."""
        m, S, W = self.cfg.spatial_merge_size, self.side, self.pos_embed.weight
        out = []
        for t, h, w in grids:
            hs, ws = torch.linspace(0, S - 1, h), torch.linspace(0, S - 1, w)
            hf, wf = hs.int(), ws.int()
            hc, wc = (hf + 1).clamp(max=S - 1), (wf + 1).clamp(max=S - 1)
            dh, dw = (hs - hf.float())[:, None], (ws - wf.float())[None, :]
            idx = [hf[:, None] * S + wf[None, :], hf[:, None] * S + wc[None, :], hc[:, None] * S + wf[None, :], hc[:, None] * S + wc[None, :]]
            wt = [(1 - dh) * (1 - dw), (1 - dh) * dw, dh * (1 - dw), dh * dw]
            e = sum(W[i.reshape(-1).long().to(W.device)].float() * x.reshape(-1, 1).to(W.device) for i, x in zip(idx, wt))      # [h*w, H]
            e = e.view(h // m, m, w // m, m, -1).permute(0, 2, 1, 3, 4).reshape(h * w, -1)
            out.append(e.repeat(t, 1))
        return torch.cat(out).to(W.dtype)

    # ---- forward -----------------------------------------------------------------------------
    @torch.inference_mode()
    def forward(self, patches: torch.Tensor, grid_thw) -> torch.Tensor:
        """patches [T, patch_dim]; grid_thw: (frames, height, width) in patches per image.  Returns [T / merge^2, out_hidden]."""
        grids = [tuple(int(v) for v in g) for g in (grid_thw.tolist() if isinstance(grid_thw, torch.Tensor) else grid_thw)]
        dev = self.pos_embed.weight.device
        x = self.patch_embed(patches.to(dev, self.dtype)) + self.pos_embed_rows(grids)
        rope = self.rope_rows(grids)
        lens = [h * w for t, h, w in grids for _ in range(t)]                 # attention stays inside one frame
        cu = torch.tensor([0] + torch.tensor(lens).cumsum(0).tolist(), dtype=torch.int32, device=dev)
        arange = torch.arange(x.shape[0], device=dev)
        for blk in self.blocks:
            x = blk(x, cu, rope, arange)
        return self.merger(x)

    # ---- weights ---------------------------------------------------------------------------
    @torch.no_grad()
    def load_weights(self, weights: Iterable[Tuple[str, torch.Tensor]]) -> int:
        """HF names under `visual.` / `model.visual.`: patch_embed.proj (a Conv3d kernel, flattened here), pos_embed, blocks.N.
        {norm1, norm2, attn.qkv, attn.proj, mlp.linear_fc1, mlp.linear_fc2}, merger.{norm, linear_fc1, linear_fc2}."""
        n = 0
        names = {"attn.qkv": "qkv", "attn.proj": "proj", "mlp.linear_fc1": "fc1", "mlp.linear_fc2": "fc2", "norm1": "norm1", "norm2": "norm2"}
        for name, t in weights:
            m = re.match(r"(?:model\.)?visual\.(.+)\.(weight|bias)$", name)
            if not m:
                continue
            key, kind = m.group(1), m.group(2)
            mod = None
            if key == "patch_embed.proj":
                mod, t = self.patch_embed, (t.flatten(1) if kind == "weight" else t)
            elif key == "pos_embed":
                self.pos_embed.weight.copy_(t.to(self.dtype)); n += 1; continue
            elif key.startswith("merger."):
                mod = {"norm": self.merger.norm, "linear_fc1": self.merger.fc1, "linear_fc2": self.merger.fc2}.get(key[7:])
            else:
                b = re.match(r"blocks\.(\d+)\.(.+)$", key)
                if b and int(b.group(1)) < len(self.blocks) and b.group(2) in names:
                    mod = getattr(self.blocks[int(b.group(1))], names[b.group(2)])
            if mod is None:
                continue
            if kind == "bias":
                mod.bias.copy_(t.to(mod.bias.dtype))
            elif isinstance(mod, QLinear):
                mod.set_weight(t.float())
            else:
                mod.weight.copy_(t.to(mod.weight.dtype))
            n += 1
        return n


def random_vision_weights(c: VisionConfig, seed: int = 0, std: float = 0.05):
    """Random tensors under the HF names (tests, benchmarks)."""
    g = torch.Generator().manual_seed(seed)
    H, I, M = c.hidden_size, c.intermediate_size, c.hidden_size * c.spatial_merge_size ** 2
    def r(*shape, s=std):
        return torch.randn(*shape, generator=g) * s
    yield "visual.patch_embed.proj.weight", r(H, c.in_channels, c.temporal_patch_size, c.patch_size, c.patch_size)
    yield "visual.patch_embed.proj.bias", r(H)
    yield "visual.pos_embed.weight", r(c.num_position_embeddings, H)
    for i in range(c.depth):
        p = f"visual.blocks.{i}."
        for nm, shape in (("norm1", (H,)), ("norm2", (H,))):
            yield p + nm + ".weight", 1.0 + r(*shape)
            yield p + nm + ".bias", r(*shape)
        for nm, (o, k) in (("attn.qkv", (3 * H, H)), ("attn.proj", (H, H)), ("mlp.linear_fc1", (I, H)), ("mlp.linear_fc2", (H, I))):
            yield p + nm + ".weight", r(o, k)
            yield p + nm + ".bias", r(o)
    yield "visual.merger.norm.weight", 1.0 + r(H)
    yield "visual.merger.norm.bias", r(H)
    yield "visual.merger.linear_fc1.weight", r(M, M)
    yield "visual.merger.linear_fc1.bias", r(M)
    yield "visual.merger.linear_fc2.weight", r(c.out_hidden_size, M)
    yield "visual.merger.linear_fc2.bias", r(c.out_hidden_size)
