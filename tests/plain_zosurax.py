"""Plain implementation of the Zosurax design: NumPy, float64, whole sequences, no cache, no batches.

One function per mechanism, written from the design's equations; nothing here is shared with the
library.  Weights come as a dict name -> array (tensor names of the weight file), the
configuration as the dict that config.json holds.

Notation: T tokens, W width, H query heads, G key/value heads, d per-head query/key size, e per-head
value size.  rms(x) = x / sqrt(mean(x^2) + eps) over the last axis.
"""
from __future__ import annotations

import numpy as np


def rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def token_shift(h, mu):
    """h_t <- h_t + (h_{t-1} - h_t) * mu, with h_{-1} = 0; the h on the right are the unshifted ones."""
    prev = np.zeros_like(h)
    prev[1:] = h[:-1]
    return h + (prev - h) * mu


def rotate(x, positions, base, n_rot, interleaved):
    """x [T, heads, d]: the first n_rot values of every head are rotated in pairs, pair i by the angle
    position * base^(-2i / n_rot); pairs are (i, i + n_rot/2), or (2i, 2i+1) when interleaved."""
    out = x.copy()
    half = n_rot // 2
    for i in range(half):
        a, b = (2 * i, 2 * i + 1) if interleaved else (i, i + half)
        ang = positions.astype(np.float64) * (float(base) ** (-2.0 * i / n_rot))
        c, s = np.cos(ang)[:, None], np.sin(ang)[:, None]
        u, v = x[:, :, a], x[:, :, b]
        out[:, :, a] = u * c - v * s
        out[:, :, b] = v * c + u * s
    return out


def causal_softmax_weights(q, k, scale):
    """q [T, H, d], k [T, G, d] -> weights [H, T, T], row i over keys j <= i."""
    T, H, _ = q.shape
    G = k.shape[1]
    w = np.zeros((H, T, T))
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            s = (k[:i + 1, g] @ q[i, h]) * scale
            s = np.exp(s - s.max())
            w[h, i, :i + 1] = s / s.sum()
    return w


def apply_weights(w, v):
    """w [H, T, T], v [T, G, e] -> [T, H * e]: head h reads the values of key/value head h // (H/G)."""
    H, T, _ = w.shape
    G, e = v.shape[1], v.shape[2]
    out = np.zeros((T, H, e))
    for h in range(H):
        out[:, h, :] = w[h] @ v[:, h // (H // G), :]
    return out.reshape(T, H * e)


def attention_normed(h, p, m, eps, positions):
    """Mixer 'attention': per-head weighted RMS norm of q and k, then half-split rotation, softmax."""
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ p["q"].T).reshape(T, H, d)
    k = (h @ p["k"].T).reshape(T, G, d)
    v = (h @ p["v"].T).reshape(T, G, e)
    q = rms(q, eps) * p["q.norm"]
    k = rms(k, eps) * p["k.norm"]
    rot = m.get("rot")
    if rot:
        q = rotate(q, positions, rot["base"], rot["dims"], False)
        k = rotate(k, positions, rot["base"], rot["dims"], False)
    w = causal_softmax_weights(q, k, m["scale"])
    return apply_weights(w, v) @ p["o"].T


def attention_talking(h, p, m, eps, positions):
    """Mixer 'attention_2': interleaved rotation, then unweighted RMS norm of q and k; the heads' softmax
    weights are mixed by the matrix `talk` before they meet the values."""
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ p["q"].T).reshape(T, H, d)
    k = (h @ p["k"].T).reshape(T, G, d)
    v = (h @ p["v"].T).reshape(T, G, e)
    rot = m.get("rot")
    if rot:
        q = rotate(q, positions, rot["base"], rot["dims"], True)
        k = rotate(k, positions, rot["base"], rot["dims"], True)
    q, k = rms(q, eps), rms(k, eps)
    w = causal_softmax_weights(q, k, m["scale"])
    mixed = np.einsum("hg,gij->hij", p["talk"], w)
    return apply_weights(mixed, v) @ p["o"].T


def hgrn2(h, p, m, eps):
    """Mixer 'hgrn2': per head a state S [d, e]; S <- diag(f) S + (1 - f) v^T, o = S^T q."""
    T = h.shape[0]
    H, d, e = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ p["q"].T).reshape(T, H, d)
    v = (h @ p["v"].T).reshape(T, H, e)
    low = p["lower"].reshape(H, d)
    f = low + (1.0 - low) * sigmoid(h @ p["f"].T + p["f.b"]).reshape(T, H, d)
    S = np.zeros((H, d, e))
    o = np.zeros((T, H, e))
    for t in range(T):
        for hh in range(H):
            S[hh] = f[t, hh][:, None] * S[hh] + np.outer(1.0 - f[t, hh], v[t, hh])
            o[t, hh] = S[hh].T @ q[t, hh]
    o = rms(o, eps) * p["norm"]
    return o.reshape(T, H * e) @ p["o"].T


def relu_squared_mlp(h, p):
    u = np.maximum(h @ p["up"].T, 0.0)
    return (u * u) @ p["down"].T


def sub(weights, prefix):
    return {k[len(prefix):]: np.asarray(v, dtype=np.float64) for k, v in weights.items() if k.startswith(prefix)}


def layer_order(cfg):
    """[(layer index, pass number or None)], pass number given for the first layer of each pass."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, None) for i in range(a)]
    for t in range(times):
        order += [(i, t if i == a else None) for i in range(a, b)]
    return order + [(i, None) for i in range(b, n)]


def forward(cfg, weights, tokens, return_layers=False):
    """Logits [T, vocab] of one whole sequence (and the residual rows after every layer run)."""
    W64 = {k: np.asarray(v, dtype=np.float64) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    tokens = np.asarray(tokens)
    positions = np.arange(len(tokens))
    x0 = W64["embed"][tokens]
    x = x0.copy()
    after = []
    for i, t in layer_order(cfg):
        L = cfg["layers"][i]
        pre = f"l{i}."
        if t is not None:
            if t > 0:
                x = x + x0
            x = x + W64["loop.step"][t]
        h = token_shift(rms(x, eps) * W64[pre + "norm1"], W64[pre + "shift"])
        p = sub(weights, pre + "mix.")
        if L["type"] == "hgrn2":
            y = hgrn2(h, p, L["mixer"], eps)
        elif L["type"] == "attention":
            y = attention_normed(h, p, L["mixer"], eps, positions)
        elif L["type"] == "attention_2":
            y = attention_talking(h, p, L["mixer"], eps, positions)
        else:
            raise ValueError(L["type"])
        x = x + y * W64[pre + "ls1"]
        if L.get("mlp") is not None:
            y = relu_squared_mlp(rms(x, eps) * W64[pre + "norm2"], sub(weights, pre + "mlp."))
            x = x + y * W64[pre + "ls2"]
        after.append(x.copy())
    logits = (rms(x, eps) * W64["final.norm"]) @ W64["embed"].T
    return (logits, np.stack(after)) if return_layers else logits

