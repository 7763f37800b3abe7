"""Grouped-query attention over the paged cache.

q, k, v projections without bias (fused into one matrix at load), position encoding on q and
k, the new keys and values stored into the request's pages, causal attention in which query
head h reads kv head ``h // (n_heads / n_kv_heads)``, and the output projection:
src/scratch_llm/model.py:265-366 of the reference.  ``scale`` multiplies the scores
(``1/sqrt(head_dim)`` for this architecture, src/scratch_llm/model.py:177); ``window`` None
attends to every earlier key, a number to the last ``window`` of them.

Options for other designs: ``bias`` (q, k and v projections with biases, tensors
``<name>.b`` or as ``names`` says, added in 32-bit by the rotate-and-store kernel before the
rotation) and ``value_dim`` (values of another size than queries and keys).  The kernels and the
cache's pages have one head size: with a ``value_dim``, or a head size that is no multiple of
16, every head is padded with zero rows of its projection up to a common multiple of 16, which
changes no score (zeros meet zeros) and no output (the output projection gets zero columns).
In steps of single tokens the decode kernel adds the biases and turns the rotated part itself,
as it does for the plain form.
"""

from __future__ import annotations

from typing import Mapping

import torch

from ..kernels import ops
from ..weights.loader import ParamSpec
from .base import BuildContext, CacheView, KVSpec, Mixer, PositionEncoding
from .linear import Linear
from .registry import register_mixer


#: rows with several new tokens go to the tcgen05 attention kernel when the longest of them
#: fills at least one of its 128-query tiles (packed queries = new tokens x group size)
TC_MIN_PACKED_QUERIES = 128


def decode_splits(base_ctas: int, context: int, slots: int) -> int:
    """How many CTAs share the keys of one (row, kv head) in the split decode kernel: the count
    that minimises waves x (key tiles per CTA + fixed cost), a function of the batch's shape
    and of the context bucket alone, so that it is the same for every step that replays one
    captured graph.  ``slots``: CTAs of the split kernel resident on the GPU at once
    (:func:`scratch_llm_b200.kernels.ops.attention_decode_slots` reads it from the device)."""
    tiles = max(1, -(-context // 64))
    best, best_cost = 1, None
    for n in range(1, min(64, tiles) + 1):
        # waves x (key tiles per CTA + a CTA's fixed cost) + what the merge reads per split
        cost = -(-base_ctas * n // slots) * (-(-tiles // n) + 2) + (0.1 * n if n > 1 else 0)
        if best_cost is None or cost < best_cost:
            best, best_cost = n, cost
    return best


@register_mixer("gqa_attention")
class GQAttention(Mixer):
    pad_safe = True   # padding tokens are not stored, rows without tokens leave the kernels at once
    accepts_sink = True   # forward() takes sink=: the output projection may feed the stream itself

    def accepts_normed(self, n_tokens: int) -> bool:
        return self.qkv is not None and self.qkv.takes_normed(n_tokens)

    def __init__(self, hidden_size: int, n_heads: int, n_kv_heads: int, head_dim: int,
                 scale: float, window: int | None = None,
                 names: Mapping[str, str] | None = None, value_dim: int | None = None,
                 bias: bool = False) -> None:
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} query heads do not group evenly over {n_kv_heads} "
                             "kv heads")
        self.qk_dim, self.v_dim = head_dim, head_dim if value_dim is None else value_dim
        if value_dim is None and not bias:
            if head_dim % 16 or not 16 <= head_dim <= 512:
                raise ValueError(f"head size {head_dim}: the attention kernels take multiples of "
                                 "16 from 16 to 512")
        else:   # the common head size of the kernels and of the cache's pages
            if min(self.qk_dim, self.v_dim) < 1:
                raise ValueError("head sizes must be positive")
            head_dim = -(-max(self.qk_dim, self.v_dim) // 16) * 16
            if head_dim > 512:
                raise ValueError(f"head sizes {self.qk_dim} / {self.v_dim}: the attention "
                                 "kernels take up to 512")
        self.hidden_size, self.n_heads, self.n_kv_heads = hidden_size, n_heads, n_kv_heads
        self.head_dim, self.scale, self.window = head_dim, float(scale), window
        self.has_bias = bool(bias)
        self.names = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight",
                      "o": "o_proj.weight", **(names or {})}
        for n in "qkv":
            self.names.setdefault(n + "_bias", self.names[n] + ".b")
        self.qkv: Linear | None = None
        self.o: Linear | None = None
        self.bias: torch.Tensor | None = None

    def kernel_jobs(self, dtype: torch.dtype):
        if self.qk_dim == self.v_dim == self.head_dim and not self.has_bias:
            return None   # (the plain form says nothing: its libraries are prepared by head size)
        jobs = [ops.core_job("sllm_rope_cache")]
        if dtype == torch.bfloat16 and self.head_dim <= ops.MMA_MAX_HEAD_DIM:
            jobs.append(ops.attention_mma_library(self.head_dim))
            if ops.attention_tc_supports(self.n_heads, self.n_kv_heads, self.head_dim, 16,
                                         self.window):
                jobs.append(ops.attention_tc_library(self.head_dim))
        else:
            jobs.append(ops.attention_library(self.head_dim))
        return jobs

    def kv_spec(self) -> KVSpec:
        return KVSpec(self.n_kv_heads, self.head_dim, self.window)

    def param_specs(self) -> dict[str, ParamSpec]:
        H, G = self.n_heads, self.n_kv_heads
        specs = {self.names["q"]: ParamSpec((H * self.qk_dim, self.hidden_size)),
                 self.names["k"]: ParamSpec((G * self.qk_dim, self.hidden_size)),
                 self.names["v"]: ParamSpec((G * self.v_dim, self.hidden_size)),
                 self.names["o"]: ParamSpec((self.hidden_size, H * self.v_dim))}
        if self.has_bias:
            specs[self.names["q_bias"]] = ParamSpec((H * self.qk_dim,), "gain")
            specs[self.names["k_bias"]] = ParamSpec((G * self.qk_dim,), "gain")
            specs[self.names["v_bias"]] = ParamSpec((G * self.v_dim,), "gain")
        return specs

    def _padded_rows(self, t: torch.Tensor, heads: int, size: int) -> torch.Tensor:
        """[heads * size, ...] -> [heads * head_dim, ...] with zeros after each head's rows."""
        if size == self.head_dim:
            return t
        out = t.new_zeros((heads, self.head_dim) + tuple(t.shape[1:]))
        out[:, :size] = t.reshape((heads, size) + tuple(t.shape[1:]))
        return out.view((heads * self.head_dim,) + tuple(t.shape[1:]))

    def load(self, tensors: Mapping[str, torch.Tensor], ctx: BuildContext) -> None:
        put = lambda t: t.to(device=ctx.device, dtype=ctx.dtype)  # noqa: E731
        H, G = self.n_heads, self.n_kv_heads
        sizes = {"q": (H, self.qk_dim), "k": (G, self.qk_dim), "v": (G, self.v_dim)}
        self.qkv = Linear(torch.cat([self._padded_rows(put(tensors[self.names[n]]), *sizes[n])
                                     for n in "qkv"], 0).contiguous())
        o = put(tensors[self.names["o"]])
        self.o = Linear(self._padded_rows(o.t(), H, self.v_dim).t().contiguous())
        if self.has_bias:
            self.bias = torch.cat([self._padded_rows(
                tensors[self.names[n + "_bias"]].to(device=ctx.device, dtype=torch.float32),
                *sizes[n]) for n in "qkv"], 0).contiguous()

    def forward(self, x, batch, cache: CacheView, write: bool, position: PositionEncoding,
                sink=None):
        """``x``: the normed activations (or a :class:`~.stream.Normed`, see accepts_normed);
        ``sink``: where the output projection may put its result (a
        :class:`~.stream.StreamSink`), else the result is returned."""
        out = self._attend(x, batch, cache, write, position)
        return self.o(out) if sink is None else sink.finish(self.o, out)

    def _attend(self, x, batch, cache: CacheView, write: bool,
                position: PositionEncoding) -> torch.Tensor:
        H, G, hd = self.n_heads, self.n_kv_heads, self.head_dim
        qkv = self.qkv(x)
        if position.rotary_tables:
            cos, sin, interleaved = position.cos, position.sin, position.interleaved
        else:
            n = qkv.shape[0]
            position.apply(qkv[:, :H * hd].view(n, H, hd), qkv[:, H * hd:(H + G) * hd].view(n, G, hd),
                           batch.positions)
            cos = sin = None
            interleaved = True
        # (padding tokens get no attention output: zeros, so that what follows stays finite)
        out = (torch.zeros if batch.padded else torch.empty)(
            (qkv.shape[0], H * hd), dtype=qkv.dtype, device=qkv.device)
        if (cos is not None and qkv.dtype == torch.bfloat16 and batch.n_multi == 0
                and batch.n_single > 0 and H // G <= 16
                and ops.attention_decode_fused_supported(hd)):
            # a step of single tokens: the decode kernel rotates q and the new keys itself and
            # stores the new keys and values (one launch fewer, q and k make no round trip)
            self._decode_fused(qkv, out, batch, cache, (cos, sin, interleaved, write))
            return out
        ops.rope_kv_write(qkv, batch.positions, batch.token_row, cos, sin, cache.pages,
                          cache.block_table, cache.page_size, H, G, hd, interleaved, write,
                          self.bias)
        q = qkv[:, :H * hd]
        if qkv.dtype == torch.bfloat16 and hd <= ops.MMA_MAX_HEAD_DIM:
            self._attend_tensor_cores(q, out, batch, cache)
        else:
            ops.attention_simt(q, cache.pages, cache.block_table, cache.page_size,
                               batch.row_start, batch.row_pos0, out, batch.n_rows,
                               batch.max_new, H, G, hd, self.scale, self.window)
        return out

    def _n_splits(self, batch) -> int:
        H, G = self.n_heads, self.n_kv_heads
        return decode_splits(batch.n_single * G * (-(-(H // G) // 16)),
                             batch.context_bucket if self.window is None
                             else min(batch.context_bucket, self.window + 64),
                             ops.attention_decode_slots(self.head_dim))

    def _decode_fused(self, qkv, out, batch, cache: CacheView, rope) -> None:
        H, G, hd = self.n_heads, self.n_kv_heads, self.head_dim
        n_splits = self._n_splits(batch)
        scratch = None
        if n_splits > 1:
            scratch = torch.empty(ops.attention_mma_scratch_floats(qkv.shape[0], H, hd, n_splits),
                                  dtype=torch.float32, device=qkv.device)
        cos, sin, interleaved, write = rope
        # every row is single and the list names them in order: the kernel needs no list
        # (one load less on the way to a CTA's first keys)
        rows = None if batch.n_single == batch.n_rows else batch.single_rows
        # Where the launch fits the device at once, what counts is the chain of kernels: the CTA
        # that finishes last for a row and kv head merges the splits itself and no merge kernel
        # follows.  A launch of several rounds of CTAs is bound by its work, to which the count
        # and its fence in every CTA would add (5.57 against 5.38 ms a step at batch 64).
        ctas = batch.n_single * G * (-(-(H // G) // 16)) * n_splits
        inside = ctas <= ops.attention_decode_slots(hd)
        ops.attention_mma_decode(qkv, cache.pages, cache.block_table, cache.page_size,
                                 batch.row_start, batch.row_pos0, out, rows,
                                 batch.n_single, H, G, hd, self.scale, self.window, cos, sin,
                                 interleaved, write, n_splits, scratch, merge_inside=inside,
                                 bias=self.bias)

    def _attend_tensor_cores(self, q, out, batch, cache: CacheView) -> None:
        """Rows with several new tokens go to the wide kernel, rows with one to the split
        kernel, whose number of splits along the keys comes from :func:`decode_splits`."""
        H, G, hd = self.n_heads, self.n_kv_heads, self.head_dim
        common = (q, cache.pages, cache.block_table, cache.page_size, batch.row_start,
                  batch.row_pos0, out)
        if batch.n_multi:
            if ops.attention_tc_supports(H, G, hd, cache.page_size, self.window) \
                    and batch.max_new_multi * (H // G) >= TC_MIN_PACKED_QUERIES:
                # tcgen05 kernel: scores, probabilities and output in tensor memory
                ops.attention_tc(*common, batch.multi_rows, batch.n_multi, batch.max_new_multi,
                                 H, G, hd, self.scale)
            else:
                ops.attention_mma(*common, batch.multi_rows, batch.n_multi,
                                  batch.max_new_multi, H, G, hd, self.scale, self.window,
                                  split=False)
        if batch.n_single:
            n_splits = self._n_splits(batch)
            scratch = None
            if n_splits > 1:
                scratch = torch.empty(ops.attention_mma_scratch_floats(q.shape[0], H, hd, n_splits),
                                      dtype=torch.float32, device=q.device)
            # (where the launch fits the device at once the last CTA of a row merges the splits)
            ctas = batch.n_single * G * (-(-(H // G) // 16)) * n_splits
            ops.attention_mma(*common, batch.single_rows, batch.n_single, 1, H, G, hd,
                              self.scale, self.window, split=True, n_splits=n_splits,
                              scratch=scratch,
                              merge_inside=ctas <= ops.attention_decode_slots(hd))
