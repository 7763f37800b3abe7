"""A plain, slow implementation of the Vobosun decoder: whole sequences, no cache, one function
per mechanism, PyTorch on the CPU only (float64 by default).

Written from the design's equations in this file's own notation; it shares no code with
``scratch_llm_b200``.  It takes ``config.json`` as a plain dict and the tensors as a dict by
name.

Notation: ``T`` tokens of one sequence at positions ``0 .. T-1``; ``x`` is the residual
stream ``[T, width]``; ``h`` what a sublayer reads.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F


# ------------------------------------------------------------------------------ small pieces

def dyt(x, w, alpha, b):
    """Dynamic Tanh: no mean, no variance."""
    return torch.tanh(alpha * x) * w + b


def norm_of(t, name):
    return lambda x: dyt(x, t[name], t[name + ".alpha"], t[name + ".b"])


def token_shift(h, mu):
    """h_t + (h_{t-1} - h_t) * mu, with zeros before the first token; the h_{t-1} is the one
    before this replacement."""
    prev = torch.cat([torch.zeros_like(h[:1]), h[:-1]], 0)
    return h + (prev - h) * mu


def rms_unit(x, eps):
    return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)


def xielu(z, p, q):
    pos = F.softplus(p) * z * z + 0.5 * z
    neg = (0.5 + F.softplus(q)) * (torch.expm1(torch.clamp(z, max=0.0)) - z) + 0.5 * z
    return torch.where(z > 0, pos, neg)


def silu(z):
    return z * torch.sigmoid(z)


# ------------------------------------------------------------------------ mixer: attention

def rotate_half_layout(x, positions, dims, base, factor):
    """x [T, heads, D]: the first ``dims`` entries of each head are rotated, entry i with entry
    i + dims/2, by the angle p * base^(-2i/dims) / factor."""
    out = x.clone()
    half = dims // 2
    for i in range(half):
        f = base ** (-2.0 * i / dims) / factor
        a = positions.to(x.dtype) * f
        c, s = torch.cos(a)[:, None], torch.sin(a)[:, None]
        u, v = x[:, :, i], x[:, :, i + half]
        out[:, :, i] = u * c - v * s
        out[:, :, i + half] = v * c + u * s
    return out


def attention_mixer(h, w, m):
    """``h`` [T, width]; ``w`` the mixer's tensors by short name; ``m`` its config dict."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].T + w["q.b"]).view(T, H, D)
    k = (h @ w["k"].T + w["k.b"]).view(T, G, D)
    v = (h @ w["v"].T + w["v.b"]).view(T, G, Dv)
    rot = m.get("rot")
    if rot is not None:
        factor = (rot.get("scaling") or {}).get("factor", 1.0)
        pos = torch.arange(T)
        q = rotate_half_layout(q, pos, rot["dims"], rot["base"], factor)
        k = rotate_half_layout(k, pos, rot["dims"], rot["base"], factor)
    out = torch.zeros((T, H, Dv), dtype=h.dtype)
    for head in range(H):
        g = head // (H // G)
        for i in range(T):
            s = (k[: i + 1, g] @ q[i, head]) * m["scale"]
            p = torch.softmax(s, 0)
            out[i, head] = p @ v[: i + 1, g]
    return out.reshape(T, H * Dv) @ w["o"].T


# -------------------------------------------------------------- mixer: generalized delta rule

DECAY_SCALE = math.exp(-0.5)


def general_delta_mixer(h, w, m, eps):
    T = h.shape[0]
    H, D = m["heads"], m["dim"]
    r = (h @ w["r"].T).view(T, H, D)
    k = (h @ w["k"].T).view(T, H, D)
    v = (h @ w["v"].T).view(T, H, D)
    decay = torch.exp(-DECAY_SCALE * torch.sigmoid(torch.tanh(h @ w["w1"].T) @ w["w2"].T + w["w0"]))
    decay = decay.view(T, H, D)
    a = torch.sigmoid(h @ w["a"].T + w["a.b"]).view(T, H, D)
    u = k / torch.sqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
    S = torch.zeros((H, D, D), dtype=h.dtype)        # [head, key channel, value channel]
    o = torch.zeros((T, H, D), dtype=h.dtype)
    for t in range(T):
        for hd in range(H):
            old = S[hd]
            S[hd] = (decay[t, hd][:, None] * old
                     - torch.outer(a[t, hd] * u[t, hd], u[t, hd] @ old)
                     + torch.outer(k[t, hd], v[t, hd]))
            o[t, hd] = S[hd].T @ r[t, hd]
    o = rms_unit(o, eps).reshape(T, H * D) * w["norm"]
    return (o * torch.sigmoid(h @ w["g"].T)) @ w["o"].T


# ----------------------------------------------------------------------------- feed-forward

def dense_ff(h, w):
    p, q = w["act"][0], w["act"][1]
    return xielu(h @ w["up"].T, p, q) @ w["down"].T


def gated_expert(h, w, prefix):
    return (silu(h @ w[prefix + "gate"].T) * (h @ w[prefix + "up"].T)) @ w[prefix + "down"].T


def route(h, w, r):
    """Per token: the chosen router outputs and their weights."""
    n = r["experts"] + r.get("identity", 0)
    s = torch.softmax(h @ w["router"].T, -1)                      # [T, n]
    choice = s + w["correction"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    per = n // groups["count"]
    chosen, weights = [], []
    for t in range(h.shape[0]):
        c = choice[t].clone()
        gscore = [c[g * per:(g + 1) * per].max().item() for g in range(groups["count"])]
        best = sorted(range(groups["count"]), key=lambda g: (-gscore[g], g))[:groups["keep"]]
        for g in range(groups["count"]):
            if g not in best:
                c[g * per:(g + 1) * per] = -math.inf
        ids = sorted(range(n), key=lambda e: (-c[e].item(), e))[:r["top"]]
        wt = s[t, ids]
        chosen.append(ids)
        weights.append(wt / (wt.sum() + 1e-20))
    return chosen, weights


def moe_ff(h, w, mlp):
    r = mlp["router"]
    chosen, weights = route(h, w, r)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, wt in zip(chosen[t], weights[t]):
            if e >= r["experts"]:                                  # an identity expert
                out[t] += wt * h[t]
            else:
                out[t] += wt * gated_expert(h[t:t + 1], w, f"e{e}.")[0]
    if mlp.get("shared") is not None:
        out = out + gated_expert(h, w, "shared.")
    return out


# ------------------------------------------------------------------------------- the model

def sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def layer_forward(x, cfg, i, tensors):
    """One run of layer ``i`` (with the tensors of the layer it names, if it names one)."""
    layer = cfg["layers"][i]
    src = layer.get("weights_of", i)
    p = f"l{src}."
    eps = cfg["norm"]["eps"]
    h = token_shift(norm_of(tensors, p + "norm1")(x), tensors[p + "shift"])
    mw = sub(tensors, p + "mix.")
    if layer["type"] == "attention":
        y = attention_mixer(h, mw, layer["mixer"])
    elif layer["type"] == "general_delta":
        y = general_delta_mixer(h, mw, layer["mixer"], eps)
    else:
        raise ValueError(layer["type"])
    x = x + norm_of(tensors, p + "norm1b")(y)
    mlp = layer.get("mlp")
    if mlp is not None:
        h = norm_of(tensors, p + "norm2")(x)
        fw = sub(tensors, p + "mlp.")
        y = dense_ff(h, fw) if mlp["kind"] == "dense" else moe_ff(h, fw, mlp)
        x = x + norm_of(tensors, p + "norm2b")(y)
    return x


def forward(cfg, tensors, tokens, dtype=torch.float64, layers_out=None):
    """Logits [T, vocab] of one whole sequence.  ``layers_out``: a list that receives the
    stream after every layer run."""
    t = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    x = t["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    for i in range(len(cfg["layers"])):
        x = layer_forward(x, cfg, i, t)
        if layers_out is not None:
            layers_out.append(x.clone())
    return norm_of(t, "final.norm")(x) @ t["head"].T
