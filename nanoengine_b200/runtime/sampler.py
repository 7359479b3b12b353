"""Token sampling.  Parity: reference layers/sampler.py:7-88 (Gumbel-max in log space, greedy when
temperature < 1e-5, argmax fast path for an all-greedy batch, optional log-probabilities)."""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops


class Sampler:
    def __init__(self, seed: int = 0, device="cpu"):
        self.gen = torch.Generator(device=device)
        self.gen.manual_seed(seed)

    def __call__(self, logits: torch.Tensor, temperatures: torch.Tensor, return_logprobs: bool = False):
        return ops.sample(logits, temperatures, self.gen, return_logprobs)
