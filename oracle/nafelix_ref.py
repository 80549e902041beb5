"""Plain float64 restatement of the Nafelix decoder (test oracle only; the product path never imports it).

Nafelix keeps `streams` copies of the residual stream. A sublayer reads a weighted sum of the copies, u = sum_s a_s x_s,
normed (RMS, plain weight) and passed through a short causal convolution with a skip (h + conv(h)); what it returns, y,
goes back as x_t <- sum_s M[s, t] x_s + b_t y for all copies at once. Token mixers: softmax attention with a sliding
window, a per-head sink in the denominator, partial rotate-half rotation and an output gate -- alone (with biases and
unit-RMS queries and keys) or, with its heads' weights mixed across heads, beside a gated delta rule whose heads decay
at one input-dependent rate each; the two branches are RMS-normed over the width and averaged. Feed-forward blocks: a
dense block with a piecewise quadratic / exponential activation, or a routed mixture of clamped gated experts. A run
of layers may repeat with the same weights; every pass has a state of its own.

One function per mechanism, whole sequences at a time, no cache and no batching. `weights` maps tensor names to float
arrays, `cfg` is the parsed config.json dictionary. Linear maps are stored [out, in]; positions count from 0.
"""
from __future__ import annotations

import numpy as np

F = np.float64


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def unit_rms(x, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def causal_conv(x, taps_w):
    """x [T, C], taps_w [C, taps] with the last column on the current token; zeros before the start."""
    T, C = x.shape
    taps = taps_w.shape[1]
    xp = np.concatenate([np.zeros((taps - 1, C), dtype=F), x], 0)
    y = np.zeros_like(x)
    for j in range(taps):
        y += xp[j:j + T, :] * taps_w[:, j][None, :]
    return y


def rotate_half(x, positions, base, dims):
    """x [T, heads, d]: entry i of the first `dims` is paired with entry i + dims/2; the rest pass through."""
    half = dims // 2
    if half == 0:
        return x.copy()
    f = float(base) ** (-2.0 * np.arange(half, dtype=F) / dims)
    ang = np.asarray(positions, dtype=F)[:, None] * f[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    out = x.copy()
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def sink_softmax(scores, visible, sink):
    """Softmax over the visible keys of every query with one extra term exp(sink) in the denominator. scores [T, T]."""
    s = np.where(visible, scores, -np.inf)
    mx = np.maximum(s.max(-1, keepdims=True), sink)
    p = np.exp(s - mx)
    return p / (p.sum(-1, keepdims=True) + np.exp(sink - mx))


def window_attention(h, w, pre, m, eps, biases, unit_qk, talk):
    """Grouped-query attention over a sliding window. biases: q, k, v carry them; unit_qk: after the rotation q and k are
    brought to unit RMS per head; talk: the heads' weights are mixed by the matrix `talk` before they meet the values."""
    T = h.shape[0]
    H, G, d = int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
    dv = int(m.get("vdim", d))
    q, k, v = h @ w[pre + "q"].T, h @ w[pre + "k"].T, h @ w[pre + "v"].T
    if biases:
        q, k, v = q + w[pre + "q.b"], k + w[pre + "k.b"], v + w[pre + "v.b"]
    q, k, v = q.reshape(T, H, d), k.reshape(T, G, d), v.reshape(T, G, dv)
    pos = np.arange(T)
    rot = m.get("rot")
    if rot:
        q = rotate_half(q, pos, rot["base"], int(rot["dims"]))
        k = rotate_half(k, pos, rot["base"], int(rot["dims"]))
    if unit_qk:
        q, k = unit_rms(q, eps), unit_rms(k, eps)
    window = int(m["mask"]["size"]) if m.get("mask") else T
    ii, jj = pos[:, None], pos[None, :]
    visible = (jj <= ii) & (ii - jj < window)
    P = np.zeros((H, T, T), dtype=F)
    for hh in range(H):
        g = hh // (H // G)
        P[hh] = sink_softmax(q[:, hh, :] @ k[:, g, :].T * float(m["scale"]), visible, float(w[pre + "sink"][hh]))
    if talk:
        P = np.einsum("hg,gij->hij", w[pre + "talk"], P)
    out = np.zeros((T, H, dv), dtype=F)
    for hh in range(H):
        out[:, hh, :] = P[hh] @ v[:, hh // (H // G), :]
    gate = sigmoid(h @ w[pre + "g"].T)          # [T, H] (one per head) or [T, H * dv]
    out = out * gate[:, :, None] if gate.shape[1] == H and dv != 1 else out * gate.reshape(T, H, dv)
    return out.reshape(T, H * dv) @ w[pre + "o"].T


def head_delta(h, w, pre, m, eps):
    """Gated delta rule with one decay per head and token: S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = silu(causal_conv(h @ w[pre + "q"].T, w[pre + "q.conv"])).reshape(T, G, d)
    k = silu(causal_conv(h @ w[pre + "k"].T, w[pre + "k.conv"])).reshape(T, G, d)
    v = silu(causal_conv(h @ w[pre + "v"].T, w[pre + "v.conv"])).reshape(T, H, dv)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * d ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    beta = sigmoid(h @ w[pre + "b"].T)
    decay = np.exp(-np.exp(w[pre + "A_log"])[None, :] * softplus(h @ w[pre + "a"].T + w[pre + "dt_bias"]))
    S = np.zeros((H, d, dv), dtype=F)
    o = np.zeros((T, H, dv), dtype=F)
    for t in range(T):
        for hh in range(H):
            g = hh // (H // G)
            S[hh] = decay[t, hh] * S[hh]
            u = beta[t, hh] * (v[t, hh] - S[hh].T @ k[t, g])
            S[hh] = S[hh] + np.outer(k[t, g], u)
            o[t, hh] = S[hh].T @ q[t, g]
    o = unit_rms(o, eps) * w[pre + "norm"]
    return (o.reshape(T, H * dv) * silu(h @ w[pre + "g"].T)) @ w[pre + "o"].T


def parallel_mixer(h, w, pre, m, eps):
    left = window_attention(h, w, pre + "left.", m["left"], eps, biases=False, unit_qk=False, talk=True)
    right = head_delta(h, w, pre + "right.", m["right"], eps)
    return 0.5 * (unit_rms(left, eps) * w[pre + "left.out"] + unit_rms(right, eps) * w[pre + "right.out"])


def attention_mixer(h, w, pre, m, eps):
    return window_attention(h, w, pre, m, eps, biases=True, unit_qk=True, talk=False)


def piecewise_act(z, p, q):
    """z > 0: softplus(p) z^2 + z / 2; else (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2."""
    ap, aq = softplus(p), 0.5 + softplus(q)
    neg = np.minimum(z, 0.0)
    return np.where(z > 0, ap * z * z + 0.5 * z, aq * (np.expm1(neg) - neg) + 0.5 * z)


def dense_block(h, w, pre):
    p, q = w[pre + "act"]
    return piecewise_act(h @ w[pre + "up"].T, p, q) @ w[pre + "down"].T


def route(h, w, pre, r):
    """Chosen experts [T, top] and their weights: softmax over all experts, the largest `top`, renormalised."""
    z = h @ w[pre + "router"].T
    z = z - z.max(-1, keepdims=True)
    s = np.exp(z)
    s = s / s.sum(-1, keepdims=True)
    chosen = np.argsort(-s, axis=-1, kind="stable")[:, :int(r["top"])]
    weight = np.take_along_axis(s, chosen, axis=-1)
    return chosen, weight / (weight.sum(-1, keepdims=True) + 1e-20)


def clamped_expert(x, w, p, limit):
    g = np.minimum(w[p + "gate"] @ x, limit)
    u = np.clip(w[p + "up"] @ x, -limit, limit)
    return w[p + "down"] @ (g * sigmoid(1.702 * g) * (u + 1.0))


def mixture(h, w, pre, mlp):
    chosen, weight = route(h, w, pre, mlp["router"])
    limit = float(mlp["expert"]["limit"])
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(chosen[t], weight[t]):
            out[t] += a * clamped_expert(h[t], w, f"{pre}e{e}.", limit)
    return out


def feed_forward(h, w, pre, mlp):
    return dense_block(h, w, pre) if mlp.get("kind", "dense") == "dense" else mixture(h, w, pre, mlp)


def layer_runs(cfg):
    """Indices of the layers in the order they run: layers start .. stop-1 repeat `times` times."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def sublayer_input(xs, w, hc, norm, canon, eps):
    u = np.tensordot(w[hc + "in"], xs, axes=(0, 0)) if hc + "in" in w else xs[0]
    h = unit_rms(u, eps) * w[norm]
    return h + causal_conv(h, w[canon]) if canon in w else h


def write_back(xs, y, w, hc):
    if hc + "mix" not in w:
        return xs + y[None]
    return np.einsum("st,sij->tij", w[hc + "mix"], xs) + w[hc + "out"][:, None, None] * y[None]


def forward(cfg, weights, tokens, return_layers=False):
    """logits [T, vocab] (and the sum of the streams after every layer run [runs, T, W])."""
    w = {k: np.asarray(v, dtype=F) for k, v in weights.items()}
    eps = float(cfg["norm"]["eps"])
    S = int(cfg.get("streams", 1))
    x0 = w["embed"][np.asarray(tokens, dtype=np.int64)]
    xs = np.stack([x0] * S)
    trace = []
    for li in layer_runs(cfg):
        L, p = cfg["layers"][li], f"l{li}."
        h = sublayer_input(xs, w, p + "hc1.", p + "norm1", p + "canon1", eps)
        y = parallel_mixer(h, w, p + "mix.", L["mixer"], eps) if L["type"] == "parallel" else attention_mixer(h, w, p + "mix.", L["mixer"], eps)
        xs = write_back(xs, y, w, p + "hc1.")
        if L.get("mlp"):
            h = sublayer_input(xs, w, p + "hc2.", p + "norm2", p + "canon2", eps)
            xs = write_back(xs, feed_forward(h, w, p + "mlp.", L["mlp"]), w, p + "hc2.")
        trace.append(xs.sum(0))
    logits = (unit_rms(xs.sum(0), eps) * w["final.norm"]) @ w["head"].T
    return (logits, np.stack(trace)) if return_layers else logits
