"""A plain, slow Kavenex decoder in numpy: one function per mechanism, whole
sequences at once, no cache. The oracle that the tests compare the engine with;
it shares no code with ``garuda_b200``.

Notation. ``x`` is the residual stream ``[T, d]``; ``m`` the residual
multiplier; ``W`` matrices are ``[out, in]`` and act as ``h @ W.T``.

* embedding:   ``x_t = E[token_t] * s``
* layer:       ``x += m * mixer(LN1(x)); x += m * ff(LN2(x)); x += m * side(x, token)``
* layer norm:  ``(x - mean) / sqrt(var + eps) * w + b`` (population variance)
* rms:         ``x / sqrt(mean(x^2) + eps)``
* loop:        layers ``[start, stop)`` run ``times`` times; before pass ``p`` the embedding
               output is added again (``p > 0``) and then row ``p`` of the step table
"""
from __future__ import annotations

import math

import numpy as np

F = np.float64


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdims=True)
    var = ((x - mu) ** 2).mean(-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * w + b


def rms(x, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def rotate_pairs(v, positions, base, dims):
    """Pairs ``(2i, 2i+1)`` of the first ``dims`` channels of ``v [T, ..., n]`` turned by
    ``pos * base^(-2i/dims)``; the other channels pass."""
    out = v.copy()
    i = np.arange(dims // 2, dtype=F)
    freq = base ** (-2.0 * i / dims)
    ang = np.asarray(positions, dtype=F)[:, None] * freq[None, :]
    shape = (len(positions),) + (1,) * (v.ndim - 2) + (dims // 2,)
    c, s = np.cos(ang).reshape(shape), np.sin(ang).reshape(shape)
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def latent_attention(h, w, p, mx, eps, positions, weights_out=None):
    """``mx``: the mixer's sizes. Keys and values of every head come from one latent vector per
    position (``kv_rank`` wide, RMS-normed) and one rotated key part shared by the heads.
    ``weights_out``: a list that receives every head's ``[T, T]`` attention weights."""
    T = h.shape[0]
    H, dn, dr, dv, rank = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
    q = (h @ w[p + "q"].T).reshape(T, H, dn + dr)
    q_nope, q_rot = q[..., :dn], q[..., dn:]
    dkv = h @ w[p + "dkv"].T
    c = rms(dkv[:, :rank], eps) * w[p + "dkv.norm"]
    k_rot = dkv[:, rank:]
    rot = mx["rot"]
    q_rot = rotate_pairs(q_rot, positions, rot["base"], rot["dims"])
    k_rot = rotate_pairs(k_rot, positions, rot["base"], rot["dims"])
    k_nope = (c @ w[p + "uk"].T).reshape(T, H, dn)
    v = (c @ w[p + "uv"].T).reshape(T, H, dv)
    out = np.zeros((T, H, dv), dtype=F)
    for hd in range(H):
        s = (q_nope[:, hd] @ k_nope[:, hd].T + q_rot[:, hd] @ k_rot.T) * mx["scale"]
        s = np.where(np.tril(np.ones((T, T), dtype=bool)), s, -np.inf)
        s = s - s.max(-1, keepdims=True)
        e = np.exp(s)
        if weights_out is not None:
            weights_out.append(e / e.sum(-1, keepdims=True))
        out[:, hd] = (e / e.sum(-1, keepdims=True)) @ v[:, hd]
    return out.reshape(T, H * dv) @ w[p + "o"].T


def dense_ff(h, w, p):
    return (gelu_tanh(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def expert(h, w, p, limit):
    g = np.minimum(h @ w[p + "gate"].T, limit)
    u = np.clip(h @ w[p + "up"].T, -limit, limit)
    return (g / (1.0 + np.exp(-1.702 * g)) * (u + 1.0)) @ w[p + "down"].T


def route(h, w, p, top):
    """(chosen experts ``[T, top]``, their weights): the ``top`` largest router logits, softmax
    over those only."""
    z = h @ w[p + "router"].T + w[p + "router.b"]
    idx = np.argsort(-z, axis=-1, kind="stable")[:, :top]
    zc = np.take_along_axis(z, idx, -1)
    e = np.exp(zc - zc.max(-1, keepdims=True))
    return idx, e / e.sum(-1, keepdims=True)


def moe_ff(h, w, p, mlp):
    idx, wt = route(h, w, p, mlp["router"]["top"])
    out = np.zeros((h.shape[0], w[p + "e0.down"].shape[0]), dtype=F)
    for t in range(h.shape[0]):
        for k in range(idx.shape[1]):
            out[t] += wt[t, k] * expert(h[t:t + 1], w, p + f"e{idx[t, k]}.", mlp["expert"]["limit"])[0]
    if mlp.get("shared"):
        out += expert(h, w, p + "shared.", mlp["shared"]["limit"])
    return out


def token_side(x, tokens, w, layer, dim, eps):
    e = w["side.embed"][np.asarray(tokens), layer * dim:(layer + 1) * dim]
    g = gelu_tanh(x @ w[f"l{layer}.side.gate"].T) * e
    y = g @ w[f"l{layer}.side.proj"].T
    return rms(y, eps) * w[f"l{layer}.side.norm"]


def run_layer(x, i, cfg, w, tokens, positions):
    L = cfg["layers"][i]
    eps, m = cfg["norm"]["eps"], cfg["residual_mult"]
    p = f"l{i}."
    h = layer_norm(x, w[p + "norm1"], w[p + "norm1.b"], eps)
    if L["type"] != "latent_attention":
        raise ValueError(L["type"])
    x = x + m * latent_attention(h, w, p + "mix.", L["mixer"], eps, positions)
    mlp = L.get("mlp")
    if mlp:
        h = layer_norm(x, w[p + "norm2"], w[p + "norm2.b"], eps)
        y = dense_ff(h, w, p + "mlp.") if mlp["kind"] == "dense" else moe_ff(h, w, p + "mlp.", mlp)
        x = x + m * y
    side = cfg.get("token_side")
    if side:
        x = x + m * token_side(x, tokens, w, i, side["dim"], eps)
    return x


def run_order(cfg):
    """[(layer, pass or None)]: the loop's layers repeated, the rest once. ``pass`` is set on the
    first layer of each pass."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    out = [(i, None) for i in range(a)]
    for t in range(times):
        out += [(i, t if i == a else None) for i in range(a, b)]
    return out + [(i, None) for i in range(b, n)]


def forward(cfg, weights, tokens, trace=None):
    """Logits ``[T, vocab]`` (float64). ``trace``: a list that receives ``x`` after every layer run."""
    w = {k: np.asarray(v, dtype=F) for k, v in weights.items()}
    tokens = list(tokens)
    positions = np.arange(len(tokens))
    x0 = w["embed"][np.asarray(tokens)] * cfg["embedding"]["scale"]
    x = x0.copy()
    for i, p in run_order(cfg):
        if p is not None:
            if p > 0:
                x = x + x0
            x = x + w["loop.step"][p]
        x = run_layer(x, i, cfg, w, tokens, positions)
        if trace is not None:
            trace.append(x.copy())
    eps = cfg["norm"]["eps"]
    return layer_norm(x, w["final.norm"], w["final.norm.b"], eps) @ w["head"].T
