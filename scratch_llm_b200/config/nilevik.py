"""Typed configuration of the Nilevik decoder, read from ``config.json``.

Nilevik is a small decoder whose layers norm each branch's OUTPUT (``x + norm(branch(x))``) and
mix two kinds of sequence mixers, listed layer by layer in ``layers``:

* ``attention``: grouped-query attention without a rotation and without a value matrix (the
  values are the keys as projected), with per-head query/key norms, a query temperature that
  grows with the position, a distance penalty per head, a sliding window, a learned softmax
  sink per head and a sigmoid output gate (:mod:`scratch_llm_b200.parts.biased_attention`);
* ``delta``: the gated delta rule behind short convolutions
  (:mod:`scratch_llm_b200.parts.delta_rule`).

A layer may have a dense feed-forward with the tanh form of gelu on its gate, and every layer
ends with a gated per-token input from a table (:mod:`scratch_llm_b200.parts.token_side`).  The
embedding gets a sinusoidal position vector added and doubles as the output matrix.

config.json::

    {"architecture": "Nilevik", "vocab": V, "width": d, "norm": {"eps": e},
     "token_side": {"dim": s},
     "layers": [{"type": "attention",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "mask": {"size"},
                           "q_temp": {"coef", "every"}},
                 "mlp": {"kind": "dense", "ff": f} | null},
                {"type": "delta",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "conv"}, "mlp": ...}, ...]}

Tensors: ``embed``, ``side.embed``, ``final.norm``, and per layer i ``l<i>.norm1``, ``l<i>.norm2``,
``l<i>.mix.*``, ``l<i>.mlp.{gate,up,down}``, ``l<i>.side.{gate,proj,norm}``.
"""

from __future__ import annotations

import copy
import math
from dataclasses import dataclass, field
from typing import Any, Mapping

from .spec import LayerSpec, ModelSpec, PartSpec, sequential_order

#: constants the design fixes
SINUSOID_BASE = 10000.0
SLOPE_POWER = 8.0          # slope of head h of H: 2^(-8 (h + 1) / H)
#: the design has no longest position; this bounds the engine's block tables (config.json may
#: carry another bound as "max_position")
DEFAULT_MAX_POSITION = 1 << 17


def _positive_int(value: Any, what: str) -> int:
    if not isinstance(value, int) or isinstance(value, bool) or value < 1:
        raise ValueError(f"{what} must be a positive integer, got {value!r}")
    return value


def _number(value: Any, what: str) -> float:
    if isinstance(value, bool) or not isinstance(value, (int, float)) or not math.isfinite(value):
        raise ValueError(f"{what} must be a number, got {value!r}")
    return float(value)


@dataclass(frozen=True)
class NilevikConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: tuple[Mapping[str, Any], ...]
    side_dim: int | None = None
    max_position: int = DEFAULT_MAX_POSITION
    raw: Mapping[str, Any] = field(default_factory=dict, compare=False, repr=False)

    architecture = "Nilevik"

    def __post_init__(self) -> None:
        _positive_int(self.vocab, "vocab")
        _positive_int(self.width, "width")
        _positive_int(self.max_position, "max_position")
        if not (self.norm_eps > 0 and math.isfinite(self.norm_eps)):
            raise ValueError(f"norm.eps must be positive, got {self.norm_eps!r}")
        if self.side_dim is not None:
            _positive_int(self.side_dim, "token_side.dim")
        if not self.layers:
            raise ValueError("layers must list at least one layer")
        for i, layer in enumerate(self.layers):
            self._check_layer(i, layer)

    @staticmethod
    def _check_layer(i: int, layer: Mapping[str, Any]) -> None:
        kind, m = layer.get("type"), layer.get("mixer")
        if kind not in ("attention", "delta"):
            raise ValueError(f"layer {i}: type must be 'attention' or 'delta', got {kind!r}")
        if not isinstance(m, Mapping):
            raise ValueError(f"layer {i}: 'mixer' must give the mixer's sizes")
        for key in ("heads", "kv_heads", "dim", "vdim"):
            _positive_int(m.get(key), f"layer {i}: mixer.{key}")
        if m["heads"] % m["kv_heads"]:
            raise ValueError(f"layer {i}: {m['heads']} heads do not group evenly over "
                             f"{m['kv_heads']} kv_heads")
        if kind == "attention":
            if m["vdim"] != m["dim"]:
                raise ValueError(f"layer {i}: the values are the keys, so vdim must equal dim "
                                 f"(got {m['vdim']} and {m['dim']})")
            _number(m.get("scale"), f"layer {i}: mixer.scale")
            _positive_int((m.get("mask") or {}).get("size"), f"layer {i}: mixer.mask.size")
            temp = m.get("q_temp")
            if temp is not None:
                _number(temp.get("coef"), f"layer {i}: mixer.q_temp.coef")
                if not _number(temp.get("every"), f"layer {i}: mixer.q_temp.every") > 0:
                    raise ValueError(f"layer {i}: mixer.q_temp.every must be positive")
        else:
            _positive_int(m.get("conv"), f"layer {i}: mixer.conv")
        mlp = layer.get("mlp")
        if mlp is not None:
            if mlp.get("kind") != "dense":
                raise ValueError(f"layer {i}: mlp.kind must be 'dense', got {mlp.get('kind')!r}")
            _positive_int(mlp.get("ff"), f"layer {i}: mlp.ff")

    # -- config.json ---------------------------------------------------------------------

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "NilevikConfig":
        missing = [k for k in ("vocab", "width", "norm", "layers") if k not in raw]
        if missing:
            raise ValueError(f"config.json lacks required keys: {', '.join(missing)}")
        side = raw.get("token_side")
        return cls(vocab=raw["vocab"], width=raw["width"],
                   norm_eps=_number((raw["norm"] or {}).get("eps"), "norm.eps"),
                   layers=tuple(copy.deepcopy(dict(layer)) for layer in raw["layers"]),
                   side_dim=None if side is None else side.get("dim"),
                   max_position=raw.get("max_position", DEFAULT_MAX_POSITION),
                   raw=copy.deepcopy(dict(raw)))

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab,
                               "width": self.width, "norm": {"eps": self.norm_eps},
                               "layers": [copy.deepcopy(dict(layer)) for layer in self.layers]}
        if self.side_dim is not None:
            out["token_side"] = {"dim": self.side_dim}
        if self.max_position != DEFAULT_MAX_POSITION:
            out["max_position"] = self.max_position
        return out

    @property
    def vocab_size(self) -> int:
        return self.vocab

    # -- layers as data ------------------------------------------------------------------

    def _mixer(self, layer: Mapping[str, Any]) -> PartSpec:
        m = layer["mixer"]
        if layer["type"] == "attention":
            temp = m.get("q_temp") or {}
            return PartSpec("biased_attention", {
                "hidden_size": self.width, "n_heads": m["heads"], "n_kv_heads": m["kv_heads"],
                "head_dim": m["dim"], "scale": float(m["scale"]), "eps": self.norm_eps,
                "window": m["mask"]["size"], "qk_norm": True, "value_is_key": True,
                "q_temp_coef": float(temp.get("coef", 0.0)),
                "q_temp_every": float(temp.get("every", 1.0)),
                "slope_power": SLOPE_POWER, "sink": True, "gate": True})
        return PartSpec("gated_delta_rule", {
            "hidden_size": self.width, "n_heads": m["heads"], "n_kv_heads": m["kv_heads"],
            "key_dim": m["dim"], "value_dim": m["vdim"], "conv_taps": m["conv"],
            "eps": self.norm_eps})

    def model_spec(self) -> ModelSpec:
        norm = PartSpec("rmsnorm", {"size": self.width, "eps": self.norm_eps, "name": ""})
        none = PartSpec("none", {})
        layers = []
        for i, layer in enumerate(self.layers):
            parts = {"mixer": self._mixer(layer), "mixer_norm": norm, "position": none}
            names = {"mixer": "mix", "mixer_norm": "norm1", "feed_forward": "mlp",
                     "feed_forward_norm": "norm2", "side": "side", "side_norm": "side.norm"}
            if layer.get("mlp") is not None:
                parts["feed_forward"] = PartSpec("geglu", {
                    "hidden_size": self.width, "intermediate_size": layer["mlp"]["ff"],
                    "names": {"gate": "gate", "up": "up", "down": "down"}})
                parts["feed_forward_norm"] = norm
            if self.side_dim is not None:
                parts["side"] = PartSpec("token_table", {
                    "hidden_size": self.width, "dim": self.side_dim, "layer": i,
                    "n_layers": len(self.layers), "vocab_size": self.vocab,
                    "table": "side.embed", "activation": "gelu_tanh"})
                parts["side_norm"] = norm
            layers.append(LayerSpec(f"l{i}", "branch_norm", parts, names))
        return ModelSpec(
            hidden_size=self.width, vocab_size=self.vocab, max_position=self.max_position,
            layers=tuple(layers), order=sequential_order(len(layers)), final_norm=norm,
            embed_name="embed", final_norm_name="final.norm", lm_head_name="embed",
            tie_embeddings=True, position_sinusoid_base=SINUSOID_BASE)
