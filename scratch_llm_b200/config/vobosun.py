"""Typed configuration of the Vobosun decoder, read from ``config.json``.

Vobosun is a small decoder whose layers put a Dynamic-Tanh norm before AND after each branch
(``x + norm_b(branch(norm_a(x)))``, :class:`~scratch_llm_b200.parts.norm.DynamicTanh`), shift
what the mixer reads towards the previous token (:mod:`scratch_llm_b200.parts.token_shift`), and
mix two kinds of sequence mixers, listed layer by layer in ``layers``:

* ``attention``: grouped-query attention with biases on q, k and v, values of a size of their
  own, and rotary positions on the first ``rot.dims`` entries of each head in the split-half
  pairing, with every frequency divided by ``rot.scaling.factor``
  (:mod:`scratch_llm_b200.parts.attention`, :mod:`scratch_llm_b200.parts.position`);
* ``general_delta``: the generalized delta rule with a decay and a removal rate per key channel
  (:mod:`scratch_llm_b200.parts.general_delta`).

A layer's feed-forward is dense (``W_down xielu(W_up h)``), routed
(:mod:`scratch_llm_b200.parts.routed`) or absent.  A layer with ``weights_of: j`` runs layer j's
tensors once more, with a cache entry and state of its own.  The output matrix is not tied.

config.json::

    {"architecture": "Vobosun", "vocab": V, "width": d, "norm": {"eps": e},
     "layers": [{"type": "attention",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "scale",
                           "rot": {"base", "dims", "scaling": {"factor"}}},
                 "mlp": {"kind": "dense", "ff": f}},
                {"type": "general_delta", "mixer": {"heads", "dim"},
                 "mlp": {"kind": "moe", "expert": {"ff"}, "shared": {"ff"},
                         "router": {"experts", "identity", "top", "groups": {"count", "keep"}}}},
                {..., "weights_of": 1}, ...]}

Tensors: ``embed``, ``head``, ``final.norm{,.alpha,.b}``, and per layer i with tensors of its own
``l<i>.norm1``, ``l<i>.norm1b``, ``l<i>.norm2``, ``l<i>.norm2b`` (each with ``.alpha`` and ``.b``),
``l<i>.shift``, ``l<i>.mix.*`` and ``l<i>.mlp.*``.
"""

from __future__ import annotations

import copy
import math
from dataclasses import dataclass, field
from typing import Any, Mapping

from .spec import LayerSpec, ModelSpec, PartSpec, Run

#: constants the design fixes
DECAY_SCALE = math.exp(-0.5)    # the decay is exp(-DECAY_SCALE * sigmoid(.))
UNIT_KEY_EPS = 1e-6
#: the design has no longest position; this bounds the rotary tables and the block tables
#: (config.json may carry another bound as "max_position")
DEFAULT_MAX_POSITION = 1 << 17


def _positive_int(value: Any, what: str) -> int:
    if not isinstance(value, int) or isinstance(value, bool) or value < 1:
        raise ValueError(f"{what} must be a positive integer, got {value!r}")
    return value


def _count(value: Any, what: str) -> int:
    if not isinstance(value, int) or isinstance(value, bool) or value < 0:
        raise ValueError(f"{what} must be a non-negative integer, got {value!r}")
    return value


def _number(value: Any, what: str) -> float:
    if isinstance(value, bool) or not isinstance(value, (int, float)) or not math.isfinite(value):
        raise ValueError(f"{what} must be a number, got {value!r}")
    return float(value)


@dataclass(frozen=True)
class VobosunConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: tuple[Mapping[str, Any], ...]
    max_position: int = DEFAULT_MAX_POSITION
    raw: Mapping[str, Any] = field(default_factory=dict, compare=False, repr=False)

    architecture = "Vobosun"

    def __post_init__(self) -> None:
        _positive_int(self.vocab, "vocab")
        _positive_int(self.width, "width")
        _positive_int(self.max_position, "max_position")
        if not (self.norm_eps >= 0 and math.isfinite(self.norm_eps)):
            raise ValueError(f"norm.eps must not be negative, got {self.norm_eps!r}")
        if not self.layers:
            raise ValueError("layers must list at least one layer")
        for i, layer in enumerate(self.layers):
            self._check_layer(i, layer)

    def _check_layer(self, i: int, layer: Mapping[str, Any]) -> None:
        kind, m = layer.get("type"), layer.get("mixer")
        if kind not in ("attention", "general_delta"):
            raise ValueError(f"layer {i}: type must be 'attention' or 'general_delta', "
                             f"got {kind!r}")
        if not isinstance(m, Mapping):
            raise ValueError(f"layer {i}: 'mixer' must give the mixer's sizes")
        _positive_int(m.get("heads"), f"layer {i}: mixer.heads")
        _positive_int(m.get("dim"), f"layer {i}: mixer.dim")
        if kind == "attention":
            _positive_int(m.get("kv_heads"), f"layer {i}: mixer.kv_heads")
            _positive_int(m.get("vdim"), f"layer {i}: mixer.vdim")
            if m["heads"] % m["kv_heads"]:
                raise ValueError(f"layer {i}: {m['heads']} heads do not group evenly over "
                                 f"{m['kv_heads']} kv_heads")
            _number(m.get("scale"), f"layer {i}: mixer.scale")
            rot = m.get("rot")
            if rot is not None:
                dims = _positive_int(rot.get("dims"), f"layer {i}: mixer.rot.dims")
                if dims % 2 or dims > m["dim"]:
                    raise ValueError(f"layer {i}: rot.dims must be even and at most dim")
                if not _number(rot.get("base"), f"layer {i}: mixer.rot.base") > 0:
                    raise ValueError(f"layer {i}: rot.base must be positive")
                factor = (rot.get("scaling") or {}).get("factor", 1.0)
                if not _number(factor, f"layer {i}: mixer.rot.scaling.factor") > 0:
                    raise ValueError(f"layer {i}: rot.scaling.factor must be positive")
        mlp = layer.get("mlp")
        if mlp is not None:
            if mlp.get("kind") == "dense":
                _positive_int(mlp.get("ff"), f"layer {i}: mlp.ff")
            elif mlp.get("kind") == "moe":
                r = mlp.get("router") or {}
                _count(r.get("experts"), f"layer {i}: mlp.router.experts")
                _count(r.get("identity", 0), f"layer {i}: mlp.router.identity")
                _positive_int(r.get("top"), f"layer {i}: mlp.router.top")
                if r["experts"]:
                    _positive_int((mlp.get("expert") or {}).get("ff"), f"layer {i}: mlp.expert.ff")
                groups = r.get("groups")
                if groups is not None:
                    _positive_int(groups.get("count"), f"layer {i}: mlp.router.groups.count")
                    _positive_int(groups.get("keep"), f"layer {i}: mlp.router.groups.keep")
                if mlp.get("shared") is not None:
                    _positive_int(mlp["shared"].get("ff"), f"layer {i}: mlp.shared.ff")
            else:
                raise ValueError(f"layer {i}: mlp.kind must be 'dense' or 'moe', "
                                 f"got {mlp.get('kind')!r}")
        src = layer.get("weights_of")
        if src is not None:
            if not isinstance(src, int) or isinstance(src, bool) or not 0 <= src < len(self.layers) \
                    or src == i or self.layers[src].get("weights_of") is not None:
                raise ValueError(f"layer {i}: weights_of must name another layer that has "
                                 f"tensors of its own, got {src!r}")
            mine = {k: v for k, v in layer.items() if k != "weights_of"}
            if mine != dict(self.layers[src]):
                raise ValueError(f"layer {i}: a layer that uses layer {src}'s tensors must "
                                 "equal it in everything else")

    # -- config.json ---------------------------------------------------------------------

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "VobosunConfig":
        missing = [k for k in ("vocab", "width", "layers") if k not in raw]
        if missing:
            raise ValueError(f"config.json lacks required keys: {', '.join(missing)}")
        return cls(vocab=raw["vocab"], width=raw["width"],
                   norm_eps=_number((raw.get("norm") or {}).get("eps", 0.0), "norm.eps"),
                   layers=tuple(copy.deepcopy(dict(layer)) for layer in raw["layers"]),
                   max_position=raw.get("max_position", DEFAULT_MAX_POSITION),
                   raw=copy.deepcopy(dict(raw)))

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab,
                               "width": self.width, "norm": {"eps": self.norm_eps},
                               "layers": [copy.deepcopy(dict(layer)) for layer in self.layers]}
        if self.max_position != DEFAULT_MAX_POSITION:
            out["max_position"] = self.max_position
        return out

    @property
    def vocab_size(self) -> int:
        return self.vocab

    # -- layers as data ------------------------------------------------------------------

    def _mixer(self, layer: Mapping[str, Any]) -> tuple[PartSpec, PartSpec]:
        """(the mixer, its position encoding)."""
        m = layer["mixer"]
        if layer["type"] == "general_delta":
            return PartSpec("general_delta", {
                "hidden_size": self.width, "n_heads": m["heads"], "key_dim": m["dim"],
                "eps": self.norm_eps, "decay_scale": DECAY_SCALE, "unit_eps": UNIT_KEY_EPS,
                "decay_rank": m.get("decay_rank")}), PartSpec("none", {})
        mixer = PartSpec("gqa_attention", {
            "hidden_size": self.width, "n_heads": m["heads"], "n_kv_heads": m["kv_heads"],
            "head_dim": m["dim"], "value_dim": m["vdim"], "scale": float(m["scale"]),
            "window": None, "bias": True, "names": {"q": "q", "k": "k", "v": "v", "o": "o"}})
        rot = m.get("rot")
        if rot is None:
            return mixer, PartSpec("none", {})
        return mixer, PartSpec("rotary", {
            "head_dim": m["dim"] + m["dim"] % 2, "theta": float(rot["base"]),
            "max_position": self.max_position, "interleaved": False, "rot_dims": rot["dims"],
            "scaling_factor": float((rot.get("scaling") or {}).get("factor", 1.0))})

    def _feed_forward(self, mlp: Mapping[str, Any]) -> PartSpec:
        if mlp["kind"] == "dense":
            return PartSpec("act_mlp", {"hidden_size": self.width, "intermediate_size": mlp["ff"],
                                        "activation": "xielu"})
        r = mlp["router"]
        groups = r.get("groups") or {"count": 1, "keep": 1}
        shared = mlp.get("shared")
        return PartSpec("routed_experts", {
            "hidden_size": self.width, "expert_size": (mlp.get("expert") or {}).get("ff", 1),
            "experts": r["experts"], "identity": r.get("identity", 0), "top": r["top"],
            "groups": groups["count"], "keep_groups": groups["keep"],
            "shared_size": None if shared is None else shared["ff"]})

    def model_spec(self) -> ModelSpec:
        norm = PartSpec("dyt", {"size": self.width, "eps": self.norm_eps, "name": ""})
        names = {"mixer": "mix", "mixer_norm": "norm1", "mixer_out_norm": "norm1b",
                 "feed_forward": "mlp", "feed_forward_norm": "norm2",
                 "feed_forward_out_norm": "norm2b", "token_mix": "shift"}
        layers, index_of = [], {}
        for i, layer in enumerate(self.layers):
            if layer.get("weights_of") is not None:
                continue
            mixer, position = self._mixer(layer)
            parts = {"mixer": mixer, "mixer_norm": norm, "mixer_out_norm": norm,
                     "position": position,
                     "token_mix": PartSpec("token_shift", {"size": self.width, "name": ""})}
            if layer.get("mlp") is not None:
                parts["feed_forward"] = self._feed_forward(layer["mlp"])
                parts["feed_forward_norm"] = parts["feed_forward_out_norm"] = norm
            index_of[i] = len(layers)
            layers.append(LayerSpec(f"l{i}", "sandwich", parts, names))
        order = tuple(Run(layer=index_of[layer.get("weights_of", i)
                                         if layer.get("weights_of") is not None else i], cache=i)
                      for i, layer in enumerate(self.layers))
        return ModelSpec(
            hidden_size=self.width, vocab_size=self.vocab, max_position=self.max_position,
            layers=tuple(layers), order=order, final_norm=norm, embed_name="embed",
            final_norm_name="final.norm", lm_head_name="head", tie_embeddings=False)
