"""Token shift: what a mixer reads, h_t, is first replaced by ``h_t + (h_{t-1} - h_t) * mu``
with a learned vector ``mu``; h_{t-1} is the previous token's h before ITS replacement, zeros
for a sequence's first token.  The previous h is carried per request and cache entry in a state
slot of the cache manager (32-bit, the width of the stream), so that a request may be fed in
portions of any size beside other requests.

The mixing itself runs inside the norm that produces h where that norm can
(``fuses_token_mix``); this part owns the vector and states the state.
"""

from __future__ import annotations

from typing import Mapping

import torch

from ..weights.loader import ParamSpec
from .base import BuildContext, StateSpec, TokenMix
from .registry import register_token_mix


@register_token_mix("token_shift")
class TokenShift(TokenMix):
    pad_safe = True   # padding tokens belong to no row: nothing is mixed into them or carried

    def __init__(self, size: int, name: str = "") -> None:
        """``name``: the vector's tensor name below the part's prefix ("" = the prefix itself)."""
        self.size, self.name = size, name
        self.mu: torch.Tensor | None = None

    def state_spec(self) -> StateSpec:
        return StateSpec((self.size,), torch.float32)

    def param_specs(self) -> dict[str, ParamSpec]:
        return {self.name: ParamSpec((self.size,), "gain")}

    def load(self, tensors: Mapping[str, torch.Tensor], ctx: BuildContext) -> None:
        self.mu = tensors[self.name].to(device=ctx.device, dtype=torch.float32).contiguous()
