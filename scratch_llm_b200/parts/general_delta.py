"""The generalized delta rule as a mixer: a recurrent layer whose state per request is one
matrix ``S`` [key channel, value channel] per head in 32-bit, with a decay and a removal rate
per key channel:

    r, k, v = W_r x, W_k x, W_v x                      (heads x key_dim, heads x value_dim)
    w = exp(-decay_scale * sigmoid(W_w2 tanh(W_w1 x) + w0))      (decay, through a low rank)
    a = sigmoid(W_a x + a_bias)                                   (removal rate)
    u = k / sqrt(|k|^2 + unit_eps)  per head                      (the unit key)
    S <- diag(w) S - (a * u) (u^T S) + k v^T   (both terms read the old S),   o = S^T r
    out = W_o ( rmsnorm_per_head(o) * gain * sigmoid(W_g x) )     (gain: one entry per channel
                                                                   of all heads)

What enters the recurrence besides the projections is 32-bit: the low-rank path after its first
product (tanh, the second product, sigmoid, exp), the removal rate, the unit key, the state and
the read-out.  The state lives in the cache manager's state slots, so a request may be fed in
portions of any size, beside other requests, and its slot is used again after it ends.
"""

from __future__ import annotations

import math
from typing import Mapping

import torch

from ..kernels import ops
from ..weights.loader import ParamSpec
from .base import BuildContext, CacheView, Mixer, PositionEncoding, StateSpec
from .linear import Linear
from .registry import register_mixer


@register_mixer("general_delta")
class GeneralDelta(Mixer):
    pad_safe = True   # padding tokens belong to no row: the recurrence never sees them

    def __init__(self, hidden_size: int, n_heads: int, key_dim: int, eps: float,
                 value_dim: int | None = None, decay_scale: float = math.exp(-0.5),
                 unit_eps: float = 1e-6, decay_rank: int | None = None,
                 names: Mapping[str, str] | None = None) -> None:
        """``decay_rank``: the low rank of the decay's pair of matrices, if the configuration
        says it; else the tensors' shape gives it at load."""
        if not 1 <= key_dim <= ops.GENERAL_DELTA_MAX_KEY_DIM:
            raise ValueError(f"key size {key_dim}: the kernel takes 1 to "
                             f"{ops.GENERAL_DELTA_MAX_KEY_DIM}")
        self.hidden_size, self.n_heads, self.key_dim = hidden_size, n_heads, key_dim
        self.value_dim = key_dim if value_dim is None else value_dim
        self.eps, self.decay_scale, self.unit_eps = float(eps), float(decay_scale), float(unit_eps)
        self.names = {"r": "r", "k": "k", "v": "v", "g": "g", "o": "o", "a": "a", "a_bias": "a.b",
                      "w1": "w1", "w2": "w2", "w0": "w0", "norm": "norm", **(names or {})}
        self.rank: int | None = decay_rank   # None: read from the matrices' shape at load
        self.proj: Linear | None = None  # [r; k; v; g]
        self.pre: Linear | None = None   # [a; w1], 32-bit output
        self.o: Linear | None = None
        self.w2t = self.w0 = self.a_bias = self.gain = None

    def state_spec(self) -> StateSpec:
        # the key size as the kernel stores it: whole lanes of 16 elements (no device is needed
        # to know it, so that a cache can be planned on the host)
        lanes = 1
        while lanes * 16 < self.key_dim:
            lanes *= 2
        return StateSpec((self.n_heads, self.value_dim, lanes * 16), torch.float32)

    def kernel_jobs(self, dtype: torch.dtype):
        return [ops.core_job("sllm_recurrent_ops"), ops.general_delta_library(self.key_dim)]

    def param_specs(self) -> dict[str, ParamSpec]:
        n, d = self.names, self.hidden_size
        hd, hv = self.n_heads * self.key_dim, self.n_heads * self.value_dim
        rank = -1 if self.rank is None else self.rank
        return {n["r"]: ParamSpec((hd, d)), n["k"]: ParamSpec((hd, d)), n["v"]: ParamSpec((hv, d)),
                n["g"]: ParamSpec((hv, d)), n["o"]: ParamSpec((d, hv)), n["a"]: ParamSpec((hd, d)),
                n["a_bias"]: ParamSpec((hd,), "gain"), n["w1"]: ParamSpec((rank, d)),
                n["w2"]: ParamSpec((hd, rank)), n["w0"]: ParamSpec((hd,), "gain"),
                n["norm"]: ParamSpec((hv,), "gain")}

    def load(self, tensors: Mapping[str, torch.Tensor], ctx: BuildContext) -> None:
        put = lambda t: t.to(device=ctx.device, dtype=ctx.dtype)  # noqa: E731
        f32 = lambda t: t.to(device=ctx.device, dtype=torch.float32).contiguous()  # noqa: E731
        n = self.names
        w1, w2 = tensors[n["w1"]], tensors[n["w2"]]
        if w1.shape[0] != w2.shape[1]:
            raise ValueError(f"the decay's low-rank matrices do not fit: {list(w1.shape)} and "
                             f"{list(w2.shape)}")
        self.rank = w1.shape[0]
        self.proj = Linear(torch.cat([put(tensors[n[k]]) for k in "rkvg"], 0).contiguous())
        self.pre = Linear(torch.cat([put(tensors[n["a"]]), put(w1)], 0).contiguous())
        self.o = Linear(put(tensors[n["o"]]).contiguous())
        self.w2t = f32(w2).t().contiguous()
        self.w0, self.a_bias = f32(tensors[n["w0"]]), f32(tensors[n["a_bias"]])
        self.gain = f32(tensors[n["norm"]])

    def forward(self, x, batch, cache: CacheView, write: bool, position: PositionEncoding):
        if not write:
            raise NotImplementedError("a run that only reads another run's recurrent state")
        H, D, V = self.n_heads, self.key_dim, self.value_dim
        hd, hv = H * D, H * V
        n = x.shape[0]
        proj = self.proj(x)                                  # [N, 2 H D + 2 H V]
        pre = self.pre(x, out_dtype=torch.float32)           # [N, H D + rank]: 32-bit from here
        wa = torch.empty((n, 2 * hd), dtype=torch.float32, device=proj.device)
        ops.lowrank_decay(pre, self.w2t, self.w0, self.a_bias, self.decay_scale, wa)
        # (padding tokens belong to no row: their read-out stays zero)
        o = (torch.zeros if batch.padded else torch.empty)((n, hv), dtype=torch.float32,
                                                           device=proj.device)
        ops.general_delta(proj, (0, hd, 2 * hd), wa, cache.state, batch.row_start,
                          batch.row_slot, o, batch.n_rows, H, D, V, self.unit_eps)
        out = torch.empty((n, hv), dtype=proj.dtype, device=proj.device)
        ops.head_norm_gate(o, proj[:, 2 * hd + hv:2 * hd + 2 * hv], self.gain, self.eps, out, H,
                           gate_activation="sigmoid")
        return self.o(out)
