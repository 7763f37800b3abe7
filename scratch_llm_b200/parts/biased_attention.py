"""Grouped-query attention without a rotation, whose positions enter through the scores:

* queries and keys get an RMS norm per head (gains of size head_dim shared by all heads);
* the queries may carry a position-dependent temperature
  ``1 + coef * ln(floor((p + 1) / every) + 1)``;
* ``slope_h * (i - j)`` is taken off the scaled score of query i and key j in head h, with
  ``slope_h = 2 ** (-slope_power * (h + 1) / H)``;
* a sliding window: query i sees keys j with ``0 <= i - j < window``;
* a learned sink per head joins the softmax's denominator (no key, no value, counted once);
* the values may be the keys themselves as projected, before their norm (no value matrix);
* an output gate ``sigmoid(W_g x)`` on the concatenated heads before the output projection.

Every one of these is a constructor argument, so another design can use a subset.  The cache
holds the normed keys in its K pages and the values in its V pages; the kernels are the
engine's attention kernels with the slopes and sinks as optional per-head vectors.
"""

from __future__ import annotations

from typing import Mapping

import torch

from ..kernels import ops
from ..weights.loader import ParamSpec
from .attention import TC_MIN_PACKED_QUERIES, decode_splits
from .base import BuildContext, CacheView, KVSpec, Mixer, PositionEncoding
from .linear import Linear
from .registry import register_mixer


@register_mixer("biased_attention")
class BiasedAttention(Mixer):
    pad_safe = True   # padding tokens are neither normed nor stored; empty rows leave the kernels

    def __init__(self, hidden_size: int, n_heads: int, n_kv_heads: int, head_dim: int,
                 scale: float, eps: float, window: int | None = None, qk_norm: bool = True,
                 value_is_key: bool = False, q_temp_coef: float = 0.0, q_temp_every: float = 1.0,
                 slope_power: float | None = None, sink: bool = False, gate: bool = False,
                 names: Mapping[str, str] | None = None) -> None:
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} query heads do not group evenly over {n_kv_heads} "
                             "kv heads")
        if not 1 <= head_dim <= 512:
            raise ValueError(f"head size {head_dim}: the attention kernels take 1 to 512")
        if window is not None and window < 1:
            raise ValueError(f"window must be at least 1, got {window}")
        if q_temp_coef and not q_temp_every > 0:
            raise ValueError(f"the query temperature's period must be positive, got {q_temp_every}")
        self.hidden_size, self.n_heads, self.n_kv_heads = hidden_size, n_heads, n_kv_heads
        self.head_dim, self.scale, self.eps, self.window = head_dim, float(scale), float(eps), window
        self.qk_norm, self.value_is_key = bool(qk_norm), bool(value_is_key)
        self.q_temp_coef, self.q_temp_every = float(q_temp_coef), float(q_temp_every)
        self.slope_power, self.has_sink, self.has_gate = slope_power, bool(sink), bool(gate)
        self.names = {"q": "q", "k": "k", "v": "v", "o": "o", "g": "g", "q_norm": "q.norm",
                      "k_norm": "k.norm", "sink": "sink", **(names or {})}
        self.proj: Linear | None = None
        self.o: Linear | None = None
        self.q_gain = self.k_gain = self.slopes = self.sinks = None

    def kv_spec(self) -> KVSpec:
        return KVSpec(self.n_kv_heads, self.head_dim, self.window)

    def kernel_jobs(self, dtype: torch.dtype):
        jobs = [ops.core_job("sllm_qk_norm_cache"), ops.core_job("sllm_stream_ops")]
        if dtype == torch.bfloat16 and self._tensor_cores():
            jobs.append(ops.attention_mma_library(self.head_dim))
            if self.head_dim % 64 == 0:
                jobs.append(ops.attention_tc_library(self.head_dim))
        else:
            jobs.append(ops.attention_library(self.head_dim))
        return jobs

    def _tensor_cores(self) -> bool:
        """Whether the tensor-core kernels take this head size (multiples of 16 up to 256); the
        CUDA-core kernel takes the rest."""
        return self.head_dim % 16 == 0 and self.head_dim <= ops.MMA_MAX_HEAD_DIM

    def _order(self) -> list[str]:
        """The fused projection's blocks of columns: queries, keys, [values], [gate]."""
        return ["q", "k"] + ([] if self.value_is_key else ["v"]) + (["g"] if self.has_gate else [])

    def param_specs(self) -> dict[str, ParamSpec]:
        hq, hk, d = self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim, self.hidden_size
        n = self.names
        specs = {n["q"]: ParamSpec((hq, d)), n["k"]: ParamSpec((hk, d)), n["o"]: ParamSpec((d, hq))}
        if not self.value_is_key:
            specs[n["v"]] = ParamSpec((hk, d))
        if self.has_gate:
            specs[n["g"]] = ParamSpec((hq, d))
        if self.qk_norm:
            specs[n["q_norm"]] = ParamSpec((self.head_dim,), "gain")
            specs[n["k_norm"]] = ParamSpec((self.head_dim,), "gain")
        if self.has_sink:
            specs[n["sink"]] = ParamSpec((self.n_heads,), "gain")
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor], ctx: BuildContext) -> None:
        put = lambda t: t.to(device=ctx.device, dtype=ctx.dtype)  # noqa: E731
        f32 = lambda t: t.to(device=ctx.device, dtype=torch.float32).contiguous()  # noqa: E731
        n = self.names
        self.proj = Linear(torch.cat([put(tensors[n[k]]) for k in self._order()], 0).contiguous())
        self.o = Linear(put(tensors[n["o"]]).contiguous())
        if self.qk_norm:
            self.q_gain, self.k_gain = f32(tensors[n["q_norm"]]), f32(tensors[n["k_norm"]])
        if self.has_sink:
            self.sinks = f32(tensors[n["sink"]])
        if self.slope_power is not None:
            H = self.n_heads
            self.slopes = torch.tensor([2.0 ** (-self.slope_power * (h + 1) / H) for h in range(H)],
                                       dtype=torch.float32, device=ctx.device)

    def forward(self, x, batch, cache: CacheView, write: bool, position: PositionEncoding):
        H, G, hd = self.n_heads, self.n_kv_heads, self.head_dim
        proj = self.proj(x)
        v_col0 = None if self.value_is_key else (H + G) * hd
        ops.qk_norm_kv_write(proj, batch.positions, batch.token_row, self.q_gain, self.k_gain,
                             self.eps, self.q_temp_coef, self.q_temp_every, v_col0, cache.pages,
                             cache.block_table, cache.page_size, H, G, hd, write)
        q = proj[:, :H * hd]
        # (padding tokens get no attention output: zeros, so that what follows stays finite)
        out = (torch.zeros if batch.padded else torch.empty)(
            (proj.shape[0], H * hd), dtype=proj.dtype, device=proj.device)
        g0 = (H + G + (0 if self.value_is_key else G)) * hd
        gate = proj[:, g0:g0 + H * hd] if self.has_gate else None
        if proj.dtype == torch.bfloat16 and self._tensor_cores():
            self._attend_tensor_cores(q, out, batch, cache, gate)   # (the gate in its epilogue)
        else:
            ops.attention_simt(q, cache.pages, cache.block_table, cache.page_size,
                               batch.row_start, batch.row_pos0, out, batch.n_rows, batch.max_new,
                               H, G, hd, self.scale, self.window, self.slopes, self.sinks)
            if gate is not None:
                ops.sigmoid_gate(out, gate)
        return self.o(out)

    def _attend_tensor_cores(self, q, out, batch, cache: CacheView, gate) -> None:
        """Rows with several new tokens go to the tcgen05 kernel where the longest of them fills
        one of its query tiles, else to the wide ``mma.sync`` kernel; rows with one token to the
        split kernel (as :class:`~.attention.GQAttention` does).  All take the slopes and sinks."""
        H, G, hd = self.n_heads, self.n_kv_heads, self.head_dim
        common = (q, cache.pages, cache.block_table, cache.page_size, batch.row_start,
                  batch.row_pos0, out)
        gate_after = None     # the gate as a kernel of its own over the whole step
        if batch.n_multi and batch.max_new_multi * (H // G) >= TC_MIN_PACKED_QUERIES and \
                ops.attention_tc_supports(H, G, hd, cache.page_size, self.window, biased=True):
            # scores, probabilities and output in tensor memory; this kernel has no gate
            ops.attention_tc(*common, batch.multi_rows, batch.n_multi, batch.max_new_multi, H, G,
                             hd, self.scale, self.window, self.slopes, self.sinks, biased=True)
            gate_after, gate = gate, None
        elif batch.n_multi:
            # a step of prompt portions alone is bound by its bytes: the gate then runs as a
            # kernel of its own with 16-byte accesses (the epilogue's scattered 4-byte loads cost
            # the wide kernel more); beside single tokens it stays in the epilogues
            if batch.n_single == 0:
                gate_after, gate = gate, None
            ops.attention_mma(*common, batch.multi_rows, batch.n_multi, batch.max_new_multi, H, G,
                              hd, self.scale, self.window, split=False, slopes=self.slopes,
                              sinks=self.sinks, gate=gate)
        if batch.n_single:
            context = batch.context_bucket if self.window is None \
                else min(batch.context_bucket, self.window + 64)
            n_splits = decode_splits(batch.n_single * G * (-(-(H // G) // 16)), context,
                                     ops.attention_decode_slots(hd))
            scratch = None
            if n_splits > 1:
                scratch = torch.empty(ops.attention_mma_scratch_floats(q.shape[0], H, hd, n_splits),
                                      dtype=torch.float32, device=q.device)
            # (where the launch fits the device at once the last CTA of a row merges the splits)
            ctas = batch.n_single * G * (-(-(H // G) // 16)) * n_splits
            ops.attention_mma(*common, batch.single_rows, batch.n_single, 1, H, G, hd, self.scale,
                              self.window, split=True, n_splits=n_splits, scratch=scratch,
                              slopes=self.slopes, sinks=self.sinks, gate=gate,
                              merge_inside=ctas <= ops.attention_decode_slots(hd))
        if gate_after is not None:
            ops.sigmoid_gate(out, gate_after)
