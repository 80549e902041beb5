"""Plain float64 restatement of the Dibesun decoder (test oracle only; the product path never imports it).

Dibesun norms what a sublayer RETURNS, not what it reads:  x <- x + norm1(mixer(x)),  x <- x + norm2(ff(x)),  with an RMS
norm taken over equal consecutive parts of the vector. Its token mixer runs two branches on the same input and adds them
with fixed weights: chunk-local attention whose key weights are sigmoids (nothing is normalised over the keys, positions
enter only through the mask) and a linear attention with one fixed decay per head. The feed-forward block is a gated SiLU
unit, alone or as a routed mixture with a shared expert. The embedding table, unscaled, is also the output map.

One function per mechanism, whole sequences at a time, no cache and no batching. `weights` maps tensor names to float
arrays, `cfg` is the parsed config.json dictionary. h [T, W] is a sublayer's input; linear maps are stored [out, in].
"""
from __future__ import annotations

import numpy as np

F = np.float64


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def unit_rms(x, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def part_norm(x, w, groups, eps):
    """x [T, n] cut into `groups` equal consecutive parts, each brought to unit RMS; then the weight over the whole."""
    T, n = x.shape
    return unit_rms(x.reshape(T, groups, n // groups), eps).reshape(T, n) * w


def chunk_sigmoid_attention(h, w, pre, m, eps):
    """Keys of the query's own chunk (chunks counted from position 0) up to the query; weight sigmoid(capped score + b_h)."""
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    C = int(m["mask"]["size"]) if m.get("mask") else T            # no mask entry: all earlier keys
    scale, cap = float(m["scale"]), float(m.get("softcap", 0.0))   # no cap entry (or 0): scores as they are
    q = (unit_rms(h @ w[pre + "q"].T, eps) * w[pre + "q.norm"]).reshape(T, H, d)
    k = (unit_rms(h @ w[pre + "k"].T, eps) * w[pre + "k.norm"]).reshape(T, G, d)
    v = (h @ w[pre + "v"].T).reshape(T, G, dv)
    out = np.zeros((T, H, dv), dtype=F)
    for i in range(T):
        j0 = (i // C) * C
        for hh in range(H):
            g = hh // (H // G)
            s = (k[j0:i + 1, g] @ q[i, hh]) * scale
            if cap > 0.0:
                s = cap * np.tanh(s / cap)
            out[i, hh] = sigmoid(s + w[pre + "pb"][hh]) @ v[j0:i + 1, g]
    return out.reshape(T, H * dv) @ w[pre + "o"].T


def decayed_linear_attention(h, w, pre, m, eps):
    """Per head S <- decay_h S + k v^T, read-out S^T q after the write; the heads together are normed, gated and projected."""
    T = h.shape[0]
    H, d, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    decay = np.asarray(m["decay"], dtype=F)
    q = silu(h @ w[pre + "q"].T).reshape(T, H, d)
    k = silu(h @ w[pre + "k"].T).reshape(T, H, d)
    v = silu(h @ w[pre + "v"].T).reshape(T, H, dv)
    S = np.zeros((H, d, dv), dtype=F)
    o = np.zeros((T, H, dv), dtype=F)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = np.einsum("hde,hd->he", S, q[t])
    y = unit_rms(o.reshape(T, H * dv), eps) * w[pre + "norm"] * sigmoid(h @ w[pre + "g"].T)
    return y @ w[pre + "o"].T


def parallel_mixer(h, w, pre, m, eps):
    return (float(m["left_scale"]) * chunk_sigmoid_attention(h, w, pre + "left.", m["left"], eps)
            + float(m["right_scale"]) * decayed_linear_attention(h, w, pre + "right.", m["right"], eps))


def gated_unit(h, w, pre):
    return (silu(h @ w[pre + "gate"].T) * (h @ w[pre + "up"].T)) @ w[pre + "down"].T


def route(h, w, pre, r):
    """Chosen experts [T, top] (largest biased logits, ties to the lower index) and the softmax over the chosen logits."""
    z = h @ w[pre + "router"].T + w[pre + "router.b"]
    chosen = np.argsort(-z, axis=-1, kind="stable")[:, :int(r["top"])]
    zc = np.take_along_axis(z, chosen, axis=-1)
    e = np.exp(zc - zc.max(-1, keepdims=True))
    return chosen, e / e.sum(-1, keepdims=True)


def mixture(h, w, pre, mlp):
    chosen, weight = route(h, w, pre, mlp["router"])
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(chosen[t], weight[t]):
            out[t] += a * gated_unit(h[t:t + 1], w, f"{pre}e{e}.")[0]
    if mlp.get("shared"):
        out += gated_unit(h, w, pre + "shared.")
    return out


def feed_forward(h, w, pre, mlp):
    return mixture(h, w, pre, mlp) if mlp.get("kind", "dense") == "moe" else gated_unit(h, w, pre)


MIXERS = {"parallel": parallel_mixer}


def forward(cfg, weights, tokens, return_layers=False):
    """logits [T, vocab] (and the residual stream after every layer [L, T, W])."""
    w = {k: np.asarray(v, dtype=F) for k, v in weights.items()}
    eps, groups = float(cfg["norm"]["eps"]), int(cfg["norm"].get("groups", 1))
    x = w["embed"][np.asarray(tokens, dtype=np.int64)] * float(cfg["embedding"]["scale"])
    trace = []
    for li, L in enumerate(cfg["layers"]):
        p = f"l{li}."
        x = x + part_norm(MIXERS[L["type"]](x, w, p + "mix.", L["mixer"], eps), w[p + "norm1"], groups, eps)
        if L.get("mlp"):
            x = x + part_norm(feed_forward(x, w, p + "mlp.", L["mlp"]), w[p + "norm2"], groups, eps)
        trace.append(x.copy())
    logits = part_norm(x, w["final.norm"], groups, eps) @ w["embed"].T
    return (logits, np.stack(trace)) if return_layers else logits
