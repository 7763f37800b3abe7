"""Small Vobosun configurations with random tensors of every kind (matrices, biases, tanh-norm
scalars and offsets, shift vectors, low-rank decays, routers with corrections), written as model
folders, for the tests of that architecture."""

import copy
import math

import torch

from nilevik_util import relative_error, write_model  # noqa: F401  (shared test helpers)


def attention_layer(heads, kv_heads, dim, vdim=None, rot_dims=None, base=10000.0, factor=None,
                    scale=None, mlp=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim or dim,
             "scale": scale if scale is not None else 1.0 / math.sqrt(dim)}
    if rot_dims is not None:
        mixer["rot"] = {"base": base, "dims": rot_dims}
        if factor is not None:
            mixer["rot"]["scaling"] = {"factor": factor}
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def delta_layer(heads, dim, mlp=None):
    return {"type": "general_delta", "mixer": {"heads": heads, "dim": dim}, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, top, identity=0, groups=None, shared=None):
    router = {"experts": experts, "identity": identity, "top": top}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    out = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    if shared is not None:
        out["shared"] = {"ff": shared}
    return out


def again(layers, j):
    """Layer j's entry once more, using layer j's tensors."""
    return {**copy.deepcopy(layers[j]), "weights_of": j}


def config(vocab, width, layers, eps=1e-5):
    return {"architecture": "Vobosun", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "layers": layers}


def _x_layers():
    layers = [delta_layer(3, 24, mlp=moe(40, 5, 2, identity=1, groups=(3, 2), shared=24)),
              attention_layer(4, 2, 16, vdim=24, rot_dims=8, base=500.0, factor=2.0, mlp=dense(72)),
              attention_layer(2, 1, 32, rot_dims=32, base=10000.0, scale=0.3)]
    return layers + [again(layers, 1), again(layers, 0)]


def _z_layers():
    layers = [attention_layer(4, 1, 64, rot_dims=48, base=100000.0, factor=8.0, mlp=dense(192)),
              delta_layer(2, 64, mlp=moe(64, 6, 3, identity=2, groups=(4, 2), shared=64)),
              attention_layer(2, 2, 64, vdim=32, rot_dims=64, base=300.0,
                              mlp=moe(48, 3, 1, identity=0))]
    return layers + [again(layers, 1)]


# Sizes differ from one configuration to the next in everything: grouped and ungrouped heads,
# value sizes other than key sizes, rotations of a part of a head and of all of it, with and
# without a scaling factor, key sizes that are no multiple of 16, layers without a feed-forward,
# routers with and without groups, identity experts, a shared expert, one choice and several,
# layers that run another layer's tensors, a recurrent layer first.
CONFIGS = {
    "X": config(97, 48, _x_layers(), eps=1e-5),
    "Y": config(131, 64, [attention_layer(4, 4, 16, rot_dims=16, factor=4.0, mlp=moe(32, 4, 2)),
                          delta_layer(1, 32, mlp=dense(80)),
                          delta_layer(4, 16),
                          attention_layer(3, 1, 20, vdim=12, rot_dims=6, base=50.0,
                                          mlp=moe(16, 0, 1, identity=3, shared=40))], eps=3e-6),
    # shapes of the tensor-core attention (head size 64) and of the wider kernels
    "Z": config(300, 128, _z_layers(), eps=1e-6),
}


def random_tensors(cfg, seed, rank=6):
    """{name: tensor} for every tensor of the architecture, as bfloat16-exact values in 32-bit
    (so that both precisions and the plain model hold the same numbers)."""
    g = torch.Generator().manual_seed(seed)

    def normal(shape, std=1.0, mean=0.0):
        t = torch.randn(shape, generator=g) * std + mean
        return t.to(torch.bfloat16).float()

    d, V = cfg["width"], cfg["vocab"]
    t = {"embed": normal((V, d)), "head": normal((V, d), d ** -0.5)}

    def tanh_norm(name, alpha):
        t[name] = normal((d,), 0.2, 1.0)
        t[name + ".b"] = normal((d,), 0.1)
        t[name + ".alpha"] = normal((), 0.05, alpha)

    tanh_norm("final.norm", 0.5)
    for i, layer in enumerate(cfg["layers"]):
        if layer.get("weights_of") is not None:
            continue
        m, p = layer["mixer"], f"l{i}."
        tanh_norm(p + "norm1", 0.7)
        tanh_norm(p + "norm1b", 1.2)
        t[p + "shift"] = normal((d,), 0.3, 0.4)
        H, D = m["heads"], m["dim"]
        if layer["type"] == "attention":
            G, Dv = m["kv_heads"], m["vdim"]
            t[p + "mix.q"] = normal((H * D, d), d ** -0.5)
            t[p + "mix.k"] = normal((G * D, d), d ** -0.5)
            t[p + "mix.v"] = normal((G * Dv, d), d ** -0.5)
            t[p + "mix.q.b"] = normal((H * D,), 0.3)
            t[p + "mix.k.b"] = normal((G * D,), 0.3)
            t[p + "mix.v.b"] = normal((G * Dv,), 0.3)
            t[p + "mix.o"] = normal((d, H * Dv), (H * Dv) ** -0.5)
        else:
            for name in "rkvga":
                t[p + "mix." + name] = normal((H * D, d), d ** -0.5)
            t[p + "mix.a.b"] = normal((H * D,), 0.5)
            t[p + "mix.w1"] = normal((rank + i, d), d ** -0.5)
            t[p + "mix.w2"] = normal((H * D, rank + i), 0.6)
            t[p + "mix.w0"] = normal((H * D,), 1.0, -0.5)
            t[p + "mix.norm"] = normal((H * D,), 0.2, 1.0)
            t[p + "mix.o"] = normal((d, H * D), (H * D) ** -0.5)
        mlp = layer["mlp"]
        if mlp is None:
            continue
        tanh_norm(p + "norm2", 0.6)
        tanh_norm(p + "norm2b", 0.9)
        if mlp["kind"] == "dense":
            f = mlp["ff"]
            t[p + "mlp.up"] = normal((f, d), d ** -0.5)
            t[p + "mlp.down"] = normal((d, f), f ** -0.5)
            t[p + "mlp.act"] = normal((2,), 0.5, 0.3)
            continue
        r = mlp["router"]
        total = r["experts"] + r.get("identity", 0)
        t[p + "mlp.router"] = normal((total, d), 2.0 * d ** -0.5)
        # corrections large enough to change the choice, some negative: choice scores below 0
        t[p + "mlp.correction"] = normal((total,), 0.2, -0.05)
        f = mlp["expert"]["ff"]
        for e in range(r["experts"]):
            t[p + f"mlp.e{e}.gate"] = normal((f, d), d ** -0.5)
            t[p + f"mlp.e{e}.up"] = normal((f, d), d ** -0.5)
            t[p + f"mlp.e{e}.down"] = normal((d, f), f ** -0.5)
        if mlp.get("shared") is not None:
            s = mlp["shared"]["ff"]
            t[p + "mlp.shared.gate"] = normal((s, d), d ** -0.5)
            t[p + "mlp.shared.up"] = normal((s, d), d ** -0.5)
            t[p + "mlp.shared.down"] = normal((d, s), s ** -0.5)
    return t
