"""Small Nilevik configurations with random tensors of every kind (matrices, gains, taps,
decays, sinks), written as model folders, for the tests of that architecture."""

import json
import math
from pathlib import Path

import torch


def attention_layer(heads, kv_heads, dim, window, scale=None, coef=0.4, every=5, ff=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim,
             "scale": scale if scale is not None else 1.0 / math.sqrt(dim),
             "mask": {"size": window}}
    if coef is not None:
        mixer["q_temp"] = {"coef": coef, "every": every}
    return {"type": "attention", "mixer": mixer,
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def delta_layer(heads, kv_heads, dim, vdim, conv, ff=None):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim,
                                       "vdim": vdim, "conv": conv},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def config(vocab, width, layers, side_dim=8, eps=1e-5):
    out = {"architecture": "Nilevik", "vocab": vocab, "width": width, "norm": {"eps": eps},
           "layers": layers}
    if side_dim is not None:
        out["token_side"] = {"dim": side_dim}
    return out


# Sizes differ from one configuration to the next in everything: grouped and ungrouped heads,
# windows that are no multiple of a page, temperatures whose period is shorter than the
# requests, convolutions of 1 to 4 taps, value sizes other than key sizes, layers without a
# feed-forward, a model without the per-token side input, a delta layer first.
CONFIGS = {
    "P": config(97, 48, [attention_layer(4, 2, 16, window=21, every=5, ff=72),
                         delta_layer(4, 2, 16, 24, conv=4),
                         attention_layer(2, 1, 32, window=9, scale=0.3, coef=1.5, every=3),
                         delta_layer(2, 2, 8, 40, conv=2, ff=56)], side_dim=6, eps=1e-5),
    "Q": config(131, 64, [delta_layer(3, 1, 32, 16, conv=3, ff=80),
                          attention_layer(4, 4, 16, window=40, coef=None, ff=96),
                          delta_layer(1, 1, 16, 16, conv=1)], side_dim=None, eps=3e-6),
    # shapes of the tensor-core attention (head size 64), a window over several pages
    "R": config(300, 128, [attention_layer(4, 2, 64, window=70, every=16, ff=192),
                           delta_layer(2, 1, 64, 64, conv=3),
                           attention_layer(2, 2, 64, window=33, every=7)], side_dim=16),
}


def random_tensors(cfg, seed):
    """{name: tensor} for every tensor of the architecture, matrices as bfloat16-exact values
    in 32-bit (so that both precisions and the plain model hold the same numbers)."""
    g = torch.Generator().manual_seed(seed)

    def normal(shape, std=1.0, mean=0.0):
        t = torch.randn(shape, generator=g) * std + mean
        return t.to(torch.bfloat16).float()

    d, V = cfg["width"], cfg["vocab"]
    t = {"embed": normal((V, d)), "final.norm": normal((d,), 0.2, 1.0)}
    side = cfg.get("token_side")
    if side:
        t["side.embed"] = normal((V, len(cfg["layers"]) * side["dim"]))
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}."
        H, G, D, Vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        t[p + "norm1"] = normal((d,), 0.2, 1.0)
        if layer["type"] == "attention":
            t[p + "mix.q"] = normal((H * D, d), d ** -0.5)
            t[p + "mix.k"] = normal((G * D, d), d ** -0.5)
            t[p + "mix.g"] = normal((H * D, d), d ** -0.5)
            t[p + "mix.o"] = normal((d, H * D), (H * D) ** -0.5)
            t[p + "mix.q.norm"] = normal((D,), 0.3, 1.5)
            t[p + "mix.k.norm"] = normal((D,), 0.3, 1.5)
            t[p + "mix.sink"] = normal((H,), 1.0)
        else:
            K = m["conv"]
            t[p + "mix.q"] = normal((G * D, d), d ** -0.5)
            t[p + "mix.k"] = normal((G * D, d), d ** -0.5)
            t[p + "mix.v"] = normal((H * Vd, d), d ** -0.5)
            t[p + "mix.g"] = normal((H * Vd, d), d ** -0.5)
            t[p + "mix.o"] = normal((d, H * Vd), (H * Vd) ** -0.5)
            t[p + "mix.a"] = normal((H, d), d ** -0.5)
            t[p + "mix.b"] = normal((H, d), d ** -0.5)
            t[p + "mix.q.conv"] = normal((G * D, K), 0.6)
            t[p + "mix.k.conv"] = normal((G * D, K), 0.6)
            t[p + "mix.v.conv"] = normal((H * Vd, K), 0.6)
            t[p + "mix.A_log"] = normal((H,), 0.7, -1.0)
            t[p + "mix.dt_bias"] = normal((H,), 0.7)
            t[p + "mix.norm"] = normal((Vd,), 0.2, 1.0)
        if layer["mlp"] is not None:
            f = layer["mlp"]["ff"]
            t[p + "norm2"] = normal((d,), 0.2, 1.0)
            t[p + "mlp.gate"] = normal((f, d), d ** -0.5)
            t[p + "mlp.up"] = normal((f, d), d ** -0.5)
            t[p + "mlp.down"] = normal((d, f), f ** -0.5)
        if side:
            s = side["dim"]
            t[p + "side.gate"] = normal((s, d), d ** -0.5)
            t[p + "side.proj"] = normal((d, s), s ** -0.5)
            t[p + "side.norm"] = normal((d,), 0.2, 1.0)
    return t


def write_model(cfg, tensors, folder):
    from scratch_llm_b200.weights.safetensors_io import write_safetensors

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    write_safetensors(folder / "model.safetensors",
                      {k: v.to(torch.bfloat16) for k, v in tensors.items()})
    return folder


def relative_error(got, want):
    """Root mean square of the difference (its mean taken off) over that of the wanted row."""
    d = (got.double() - want.double())
    d = d - d.mean(-1, keepdim=True)
    w = want.double() - want.double().mean(-1, keepdim=True)
    return float(d.pow(2).mean(-1).sqrt().max() / w.pow(2).mean(-1).sqrt().mean())
