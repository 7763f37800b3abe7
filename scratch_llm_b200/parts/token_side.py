"""A per-layer input from the tokens themselves: every token has a small vector per layer in
a table shared by all layers (``[vocab, layers * dim]``, layer i owns the columns
``[i * dim, (i + 1) * dim)``), which a gate computed from the stream lets through:

    e = table[token, layer's columns]
    y = W_proj ( act(W_gate x) * e )

The block adds ``norm(y)`` into the stream.  The table is one tensor for the whole model: its
name starts with "/" (an absolute tensor name), so every layer's part receives the same device
tensor.
"""

from __future__ import annotations

from typing import Mapping

import torch

from ..kernels import ops
from ..weights.loader import ParamSpec
from .base import BuildContext, SideInput
from .linear import Linear
from .registry import register_side_input


@register_side_input("token_table")
class TokenTableSide(SideInput):
    pad_safe = True   # every token by itself; a padding token has id 0

    def __init__(self, hidden_size: int, dim: int, layer: int, n_layers: int, vocab_size: int,
                 table: str, activation: str = "gelu_tanh",
                 names: Mapping[str, str] | None = None) -> None:
        if activation not in ops.ACTIVATIONS:
            raise ValueError(f"unknown activation {activation!r}")
        if not 0 <= layer < n_layers:
            raise ValueError(f"layer {layer} of {n_layers}")
        self.hidden_size, self.dim, self.layer, self.n_layers = hidden_size, dim, layer, n_layers
        self.vocab_size, self.table_name, self.activation = vocab_size, table, activation
        self.names = {"gate": "gate", "proj": "proj", **(names or {})}
        self.gate: Linear | None = None
        self.proj: Linear | None = None
        self.table: torch.Tensor | None = None

    def kernel_jobs(self, dtype: torch.dtype):
        return [ops.core_job("sllm_stream_ops")]

    def param_specs(self) -> dict[str, ParamSpec]:
        return {self.names["gate"]: ParamSpec((self.dim, self.hidden_size)),
                self.names["proj"]: ParamSpec((self.hidden_size, self.dim)),
                "/" + self.table_name: ParamSpec((self.vocab_size, self.n_layers * self.dim))}

    def load(self, tensors: Mapping[str, torch.Tensor], ctx: BuildContext) -> None:
        put = lambda t: t.to(device=ctx.device, dtype=ctx.dtype).contiguous()  # noqa: E731
        self.gate = Linear(put(tensors[self.names["gate"]]))
        self.proj = Linear(put(tensors[self.names["proj"]]))
        self.table = put(tensors["/" + self.table_name])   # (shared: already on the device)

    def forward(self, x: torch.Tensor, batch) -> torch.Tensor:
        a = self.gate(x)
        gated = torch.empty_like(a)
        ops.side_gate(a, batch.token_ids, self.table, self.layer * self.dim, gated,
                      self.activation, batch.pending_tokens)
        return self.proj(gated)
