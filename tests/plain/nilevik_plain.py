"""A plain, slow implementation of the Nilevik decoder: whole sequences, no cache, one function
per mechanism, PyTorch on the CPU only (float64 by default).

Written from the design's equations in this file's own notation; it shares no code with
``scratch_llm_b200``.  It takes ``config.json`` as a plain dict and the tensors as a dict by
name.

Notation: ``T`` tokens of one sequence at positions ``0 .. T-1``; ``x`` is the residual
stream ``[T, width]``.
"""

from __future__ import annotations

import math

import torch


# ------------------------------------------------------------------------------ small pieces

def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rms_unit(x, eps):
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x, weight, eps):
    return rms_unit(x, eps) * weight


def sinusoid(positions, width, dtype):
    """[T, width]: entry 2i is sin(p * 10000^(-2i/width)), entry 2i+1 the cosine of the same."""
    out = torch.zeros((len(positions), width), dtype=dtype)
    for e in range(width):
        i = e // 2
        angle = positions.to(dtype) * (10000.0 ** (-2.0 * i / width))
        out[:, e] = torch.sin(angle) if e % 2 == 0 else torch.cos(angle)
    return out


def embed(tokens, table, width):
    positions = torch.arange(len(tokens))
    return table[tokens] + sinusoid(positions, width, table.dtype)


# ------------------------------------------------------------------------ mixer: attention

def query_temperature(p, coef, every):
    return 1.0 + coef * math.log(math.floor((p + 1) / every) + 1)


def head_slopes(n_heads):
    return [2.0 ** (-8.0 * (h + 1) / n_heads) for h in range(n_heads)]


def attention_mixer(h, w, m, eps):
    """``h`` [T, width]; ``w`` the mixer's tensors by short name; ``m`` its config dict."""
    T = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ w["q"].T).view(T, H, D)
    k = (h @ w["k"].T).view(T, G, D)
    v = k.clone()                                  # the values are the keys as projected
    q = rms_norm(q, w["q.norm"], eps)
    k = rms_norm(k, w["k.norm"], eps)
    temp = m.get("q_temp")
    if temp:
        for p in range(T):
            q[p] = q[p] * query_temperature(p, temp["coef"], temp["every"])
    slopes = head_slopes(H)
    window = m["mask"]["size"]
    out = torch.zeros((T, H, D), dtype=h.dtype)
    for head in range(H):
        g = head // (H // G)
        sink = w["sink"][head]
        for i in range(T):
            lo = max(0, i - window + 1)
            js = torch.arange(lo, i + 1)
            s = (k[lo:i + 1, g] @ q[i, head]) * m["scale"] - slopes[head] * (i - js).to(h.dtype)
            top = torch.maximum(s.max(), sink)
            e = torch.exp(s - top)
            denom = e.sum() + torch.exp(sink - top)   # the sink counts once, with no value
            out[i, head] = (e / denom) @ v[lo:i + 1, g]
    gate = torch.sigmoid(h @ w["g"].T)
    return (out.reshape(T, H * D) * gate) @ w["o"].T


# ---------------------------------------------------------------------------- mixer: delta

def causal_conv(x, taps):
    """``x`` [T, C]; ``taps`` [C, K], the last column multiplies the current token; zeros
    before the start."""
    T, C = x.shape
    K = taps.shape[1]
    out = torch.zeros_like(x)
    for t in range(T):
        for j in range(K):
            src = t - (K - 1 - j)
            if src >= 0:
                out[t] += taps[:, j] * x[src]
    return out


def silu(z):
    return z * torch.sigmoid(z)


def unit_vector(x):
    return x / torch.sqrt(x.pow(2).sum(dim=-1, keepdim=True) + 1e-6)


def delta_mixer(h, w, m, eps):
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ w["q"].T, w["q.conv"])).view(T, G, D)
    k = silu(causal_conv(h @ w["k"].T, w["k.conv"])).view(T, G, D)
    v = silu(causal_conv(h @ w["v"].T, w["v.conv"])).view(T, H, V)
    q = unit_vector(q) * D ** -0.5
    k = unit_vector(k)
    beta = torch.sigmoid(h @ w["b"].T)                                     # [T, H]
    decay = torch.exp(-torch.exp(w["A_log"]) *
                      torch.nn.functional.softplus(h @ w["a"].T + w["dt_bias"]))   # [T, H]
    out = torch.zeros((T, H, V), dtype=h.dtype)
    for head in range(H):
        g = head // (H // G)
        S = torch.zeros((D, V), dtype=h.dtype)
        for t in range(T):
            S = decay[t, head] * S
            u = beta[t, head] * (v[t, head] - S.T @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            out[t, head] = S.T @ q[t, g]
    out = rms_norm(out, w["norm"], eps)
    gate = silu(h @ w["g"].T).view(T, H, V)
    return (out * gate).reshape(T, H * V) @ w["o"].T


# ---------------------------------------------------------------------------- feed-forward

def dense_ff(h, w):
    return (gelu_tanh(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


# --------------------------------------------------------------------- per-layer token input

def token_side(x, tokens, layer, dim, side_table, w, eps):
    e = side_table[tokens][:, layer * dim:(layer + 1) * dim]
    y = (gelu_tanh(x @ w["gate"].T) * e) @ w["proj"].T
    return x + rms_norm(y, w["norm"], eps)


# ------------------------------------------------------------------------------- the model

def _sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(config, tensors, tokens, dtype=torch.float64, return_layers=False):
    """Logits [T, vocab] of one whole sequence (and, if asked, the stream after every layer)."""
    t = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    eps = config["norm"]["eps"]
    width = config["width"]
    x = embed(tokens, t["embed"], width)
    layers = []
    for i, layer in enumerate(config["layers"]):
        w = _sub(t, f"l{i}.mix.")
        mix = attention_mixer if layer["type"] == "attention" else delta_mixer
        x = x + rms_norm(mix(x, w, layer["mixer"], eps), t[f"l{i}.norm1"], eps)
        if layer.get("mlp") is not None:
            x = x + rms_norm(dense_ff(x, _sub(t, f"l{i}.mlp.")), t[f"l{i}.norm2"], eps)
        side = config.get("token_side")
        if side:
            x = token_side(x, tokens, i, side["dim"], t["side.embed"], _sub(t, f"l{i}.side."),
                           eps)
        layers.append(x.clone())
    logits = rms_norm(x, t["final.norm"], eps) @ t["embed"].T
    return (logits, torch.stack(layers)) if return_layers else logits
