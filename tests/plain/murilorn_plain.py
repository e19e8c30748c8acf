"""The Murilorn design, plainly: numpy, 64-bit, whole sequences, no cache.

One function per mechanism, written from the design's equations in the
notation below; shares no code with ``garuda_b200``. ``w`` maps tensor names to
arrays, ``cfg`` is the config.json dictionary. Matrices are ``[out, in]`` and
act as ``x @ W.T``.

    embedding      x_t = E[token_t] * embedding.scale
    norm           n(x) = x / sqrt(mean(x^2) + eps) * (1 + g)         (g stored about zero)
    streams        S copies X_1..X_S of the embedding output; for a sublayer f with
                   tensors a (in), b (out), M (mix, [from, to]):
                       u = sum_s a_s X_s,  y = f(n(u)),  X_t' = sum_s M[s, t] X_s + b_t y
                   the model's output stream is sum_s X_s
    layer          mixer sublayer, then feed-forward sublayer (if the layer has one)
    loop           layers start..stop-1 run ``times`` times in a row, each run with state of
                   its own; nothing else happens between the runs
    head           z = W_head n_final(x) * logit_scale;  logits = c tanh(z / c), c = logit_softcap
"""
from __future__ import annotations

import numpy as np


# ------------------------------------------------------------------ small functions
def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def rms_norm(x, g, eps):
    """x / sqrt(mean(x^2) + eps) * (1 + g) over the last axis."""
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * (1.0 + g)


def rms_plain(x, g, eps):
    """x / sqrt(mean(x^2) + eps) * g over the last axis (the weight is used as it is)."""
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * g


# ------------------------------------------------------------------ attention
def visible(i, j, size, keep_first):
    """Whether the query at position i reads the key at position j: causal, and either within
    the last ``size`` positions (i itself included) or among the first ``keep_first`` ones."""
    return j <= i and (i - j < size or j < keep_first)


def attention_weights(scores, mask):
    """p_j = exp(s_j) / (1 + sum_k exp(s_k)) over the visible keys: a softmax with one more
    entry of score zero that carries no value."""
    s = np.where(mask, scores, -np.inf)
    m = np.maximum(s.max(-1, keepdims=True), 0.0)
    e = np.exp(s - m)
    return e / (np.exp(-m) + e.sum(-1, keepdims=True))


def attention(h, w, p, m):
    """Grouped-query attention without any position encoding. ``m``: the mixer's sizes and
    constants (heads, kv_heads, dim, vdim, scale, softcap, mask.size, mask.keep_first)."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).reshape(T, H, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).reshape(T, G, d)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).reshape(T, G, dv)
    mask_cfg = m.get("mask")
    size = mask_cfg["size"] if mask_cfg else T + 1
    keep = mask_cfg.get("keep_first", 0) if mask_cfg else 0
    idx = np.arange(T)
    mask = np.array([[visible(i, j, size, keep) for j in idx] for i in idx])
    cap = m.get("softcap")
    out = np.zeros((T, H, dv))
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * m["scale"]
        if cap:
            s = cap * np.tanh(s / cap)
        out[:, head] = attention_weights(s, mask) @ v[:, g]
    return out.reshape(T, H * dv) @ w[p + "o"].T


# ------------------------------------------------------------------ gated delta rule with channel decay
def short_conv(x, taps):
    """Causal convolution over time, one filter per channel: ``taps [C, K]``, the last column
    weighs the current token, zeros stand before the sequence."""
    T, C = x.shape
    K = taps.shape[1]
    padded = np.concatenate([np.zeros((K - 1, C)), x], 0)
    out = np.zeros((T, C))
    for j in range(K):
        out += padded[j:j + T] * taps[:, j]
    return out


def unit(x):
    return x / np.sqrt((x * x).sum(-1, keepdims=True) + 1e-6)


def channel_delta(h, w, p, m, eps):
    """Per head a state S [dim, vdim] that starts at zero; per token, in this order:
        S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ w[p + "q"].T, w[p + "q.conv"])).reshape(T, G, d)
    k = silu(short_conv(h @ w[p + "k"].T, w[p + "k.conv"])).reshape(T, G, d)
    v = silu(short_conv(h @ w[p + "v"].T, w[p + "v.conv"])).reshape(T, H, dv)
    q = unit(q) * d ** -0.5
    k = unit(k)
    beta = sigmoid(h @ w[p + "b"].T)                                             # [T, H]
    a = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"]                   # [T, H * d]
    decay = np.exp(-np.exp(w[p + "A_log"])[None, :, None] * softplus(a).reshape(T, H, d))
    gate = sigmoid((h @ w[p + "g1"].T) @ w[p + "g2"].T).reshape(T, H, dv)
    out = np.zeros((T, H, dv))
    for head in range(H):
        g = head // (H // G)
        S = np.zeros((d, dv))
        for t in range(T):
            S = decay[t, head][:, None] * S
            u = beta[t, head] * (v[t, head] - S.T @ k[t, g])
            S = S + np.outer(k[t, g], u)
            out[t, head] = S.T @ q[t, g]
    out = rms_plain(out, w[p + "norm"], eps) * gate
    return out.reshape(T, H * dv) @ w[p + "o"].T


# ------------------------------------------------------------------ routed experts
def route(h, w, p, top):
    """Scores sigmoid(W_r h); the ``top`` largest (ties to the lower index) and their scores."""
    s = sigmoid(h @ w[p + "router"].T)
    order = np.argsort(-s, axis=-1, kind="stable")[:, :top]
    return order, np.take_along_axis(s, order, -1)


def expert(x, w, p):
    return (silu(x @ w[p + "gate"].T) * (x @ w[p + "up"].T)) @ w[p + "down"].T


def routed_experts(h, w, p, f):
    """sum over a token's chosen experts of expert(score * h): the score scales what goes in."""
    top = f["router"]["top"]
    idx, score = route(h, w, p, top)
    out = np.zeros((h.shape[0], w[p + "e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for j in range(top):
            out[t] += expert(score[t, j] * h[t][None, :], w, f"{p}e{idx[t, j]}.")[0]
    return out


# ------------------------------------------------------------------ the model
def run_order(cfg):
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def sublayer(X, fn, norm_w, eps, w, hc):
    """One sublayer on the streams ``X [S, T, d]`` (or on a single residual when ``hc`` is None)."""
    if hc is None:
        return X + fn(rms_norm(X[0], norm_w, eps))[None]
    a, b, M = w[hc + "in"], w[hc + "out"], w[hc + "mix"]
    u = np.einsum("s,std->td", a, X)
    y = fn(rms_norm(u, norm_w, eps))
    return np.einsum("sr,std->rtd", M, X) + b[:, None, None] * y[None]


def forward(cfg, w, tokens, layers_out=None):
    """Logits ``[T, vocab]`` (64-bit). ``layers_out``: a list that receives the sum of the
    streams after every layer run."""
    w = {n: np.asarray(a, dtype=np.float64) for n, a in w.items()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][np.asarray(tokens)] * cfg["embedding"]["scale"]
    streams = cfg.get("streams")
    X = np.stack([x] * (streams or 1))
    for i in run_order(cfg):
        layer, p = cfg["layers"][i], f"l{i}."
        m = layer["mixer"]
        if layer["type"] == "attention":
            mix = lambda h: attention(h, w, p + "mix.", m)
        elif layer["type"] == "channel_delta":
            mix = lambda h: channel_delta(h, w, p + "mix.", m, eps)
        else:
            raise ValueError(layer["type"])
        X = sublayer(X, mix, w[p + "norm1"], eps, w, p + "hc1." if streams else None)
        if layer.get("mlp") is not None:
            f = layer["mlp"]
            X = sublayer(X, lambda h: routed_experts(h, w, p + "mlp.", f), w[p + "norm2"], eps, w,
                         p + "hc2." if streams else None)
        if layers_out is not None:
            layers_out.append(X.sum(0))
    z = rms_norm(X.sum(0), w["final.norm"], eps) @ w["head"].T * cfg["logit_scale"]
    cap = cfg.get("logit_softcap")
    return cap * np.tanh(z / cap) if cap else z
