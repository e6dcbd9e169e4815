"""Plain, slow NumPy implementation of the Ponusun design, one function per mechanism, whole
sequences, no cache, float64.  It is the oracle of the GPU tests and shares no code with the
library: loops over tokens, heads and keys where the library has kernels.

Notation.  x[t] is the residual row of token t (position t counted from 0 in its sequence).
  embedding        x[t] = E[token_t] + P[t]
  input conv       h[t] = x[t] + sum_{j<K} c[:, j] * x[t - (K-1) + j]          (x before the start is 0)
  attention        q = Wq h, k = Wk h, v = Wv h;  q <- q / rms(q) * gq  over ALL heads at once, k likewise
                   s[i, j] = q_i . k_j * scale - r1 * ln(1 + r2 * (i - j)),  j in (i - window, i]
                   o_i = sum_j softmax_j(s[i, :]) v_j,  y = Wo concat_heads(o)
  layer            x <- x + rms(mixer(x)) * n1;  x <- x + rms(ff(x)) * n2
  dense ff         Wd gelu(Wu x),  gelu(z) = z/2 (1 + erf(z / sqrt 2))
  expert ff        (1/top) sum_{e in table[token]} Wd_e (silu(Wg_e x) * (Wu_e x))  [+ sigmoid(sg . x) * Shared(x)]
  depth average    X_0 = embedding, X_{i+1} = result of layer i, next input = sum_{j<=i+1} a_i[j] X_j
  output           cap * tanh((H rms(x) * nf) / cap)
"""
from __future__ import annotations

import math

import numpy as np


def rms_unit(x: np.ndarray, eps: float) -> np.ndarray:
    """Each row divided by sqrt(mean of its squares + eps)."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def embed_with_positions(tokens, E: np.ndarray, P: np.ndarray) -> np.ndarray:
    return np.stack([E[tok] + P[t] for t, tok in enumerate(tokens)]).astype(np.float64)


def input_conv(x: np.ndarray, c: np.ndarray) -> np.ndarray:
    """c [channels, K].  h[t] = x[t] + sum_j c[:, j] * x[t - (K-1) + j]."""
    T, K = x.shape[0], c.shape[1]
    h = np.array(x, dtype=np.float64)
    for t in range(T):
        for j in range(K):
            s = t - (K - 1) + j
            if s >= 0:
                h[t] += c[:, j] * x[s]
    return h


def log_distance_attention(h, Wq, Wk, Wv, Wo, gq, gk, H, G, d, vd, scale, r1, r2, window, eps, kv=None):
    """Returns (y, (k, v)).  `kv`: keys (already normalised) and values of another layer to use instead
    of this layer's own projections.  window 0 = every earlier token is seen."""
    T = h.shape[0]
    q = rms_unit(h @ Wq.T, eps) * gq
    if kv is None:
        k = rms_unit(h @ Wk.T, eps) * gk
        v = h @ Wv.T
    else:
        k, v = kv
    out = np.zeros((T, H * vd))
    per = H // G
    for head in range(H):
        g = head // per
        for i in range(T):
            lo = 0 if window <= 0 else max(0, i - window + 1)
            s = np.empty(i + 1 - lo)
            for n, j in enumerate(range(lo, i + 1)):
                s[n] = q[i, head * d:(head + 1) * d] @ k[j, g * d:(g + 1) * d] * scale - r1[head] * math.log1p(r2[head] * (i - j))
            w = np.exp(s - s.max())
            w /= w.sum()
            for n, j in enumerate(range(lo, i + 1)):
                out[i, head * vd:(head + 1) * vd] += w[n] * v[j, g * vd:(g + 1) * vd]
    return out @ Wo.T, (k, v)


def gelu_erf(z):
    return np.array([0.5 * a * (1.0 + math.erf(a / math.sqrt(2.0))) for a in np.ravel(z)]).reshape(np.shape(z))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z / (1.0 + np.exp(-z))


def dense_ff(x, Wu, Wd):
    return gelu_erf(x @ Wu.T) @ Wd.T


def gated_ff(x, Wg, Wu, Wd):
    return (silu(x @ Wg.T) * (x @ Wu.T)) @ Wd.T


def table_experts(x, tokens, table, experts, shared=None, sg=None):
    """experts: list of (Wg, Wu, Wd); table [vocab, top]; shared: (Wg, Wu, Wd) or None; sg [width] or None."""
    y = np.zeros_like(x, dtype=np.float64)
    top = table.shape[1]
    for t, tok in enumerate(tokens):
        for e in table[tok]:
            y[t] += gated_ff(x[t:t + 1], *experts[int(e)])[0] / top
        if shared is not None:
            gate = 1.0 if sg is None else 1.0 / (1.0 + math.exp(-float(sg @ x[t])))
            y[t] += gate * gated_ff(x[t:t + 1], *shared)[0]
    return y


def depth_average(results, a):
    """results: [X_0 .. X_n]; a: n + 1 weights."""
    assert len(a) == len(results)
    return sum(float(a[j]) * results[j] for j in range(len(results)))


def softcap(z, cap):
    return cap * np.tanh(z / cap)


def forward(cfg: dict, W: dict, tokens, return_layers: bool = False):
    """cfg: the config.json dictionary; W: name -> float64 array (integer tables as they are).
    Logits [T, vocab] of every position of ONE sequence."""
    eps = cfg["norm"]["eps"]
    taps = (cfg.get("canon") or {}).get("taps", 0)
    x = embed_with_positions(tokens, W["embed"], W["pos"])
    results, kv_of, after = [x], {}, []
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        h = input_conv(x, W[p + "canon1"]) if taps else x
        src = m.get("kv_from")
        y, kv = log_distance_attention(
            h, W[p + "mix.q"], W.get(p + "mix.k"), W.get(p + "mix.v"), W[p + "mix.o"], W[p + "mix.q.norm"],
            W.get(p + "mix.k.norm"), m["heads"], m["kv_heads"], m["dim"], m.get("vdim", m["dim"]), m["scale"],
            W[p + "mix.r1"], W[p + "mix.r2"], (m.get("mask") or {}).get("size", 0), eps,
            kv=None if src is None else kv_of[src])
        if src is None:
            kv_of[i] = kv
        x = x + rms_unit(y, eps) * W[p + "norm1"]
        ml = L.get("mlp")
        if ml is not None:
            if ml["kind"] == "dense":
                f = dense_ff(x, W[p + "mlp.up"], W[p + "mlp.down"])
            else:
                ex = [(W[f"{p}mlp.e{e}.gate"], W[f"{p}mlp.e{e}.up"], W[f"{p}mlp.e{e}.down"])
                      for e in range(ml["router"]["experts"])]
                sh = None
                if ml.get("shared"):
                    sh = (W[p + "mlp.shared.gate"], W[p + "mlp.shared.up"], W[p + "mlp.shared.down"])
                f = table_experts(x, tokens, W[p + "mlp.table"], ex, sh,
                                  W[p + "mlp.shared.sg"].reshape(-1) if sh is not None else None)
            x = x + rms_unit(f, eps) * W[p + "norm2"]
        results.append(x)
        x = depth_average(results, W[p + "dwa"])
        after.append(x)
    logits = (rms_unit(x, eps) * W["final.norm"]) @ W["head"].T
    if cfg.get("logit_softcap") is not None:
        logits = softcap(logits, cfg["logit_softcap"])
    return (logits, after) if return_layers else logits
