"""A plain, slow restatement of the Viresun design in numpy: one function per mechanism, whole sequences at a
time, token by token where the design has a recurrence, no cache and no batching.  It shares nothing with the
engine; the tests compare the engine's logits with it.

A model is (config, weights): `config` is the dictionary of the design's config.json, `weights` maps the
file's tensor names to arrays.  Everything is computed in the arrays' own type (float64 in the tests).

Notation: x is the residual stream [n, width]; h a block's normalised input; position p counts from 0.
"""
import math

import numpy as np


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.maximum(z, 0.0) + np.log1p(np.exp(-np.abs(z)))


def rms(v, eps):
    """v / sqrt(mean(v^2) + eps) over the last axis."""
    return v / np.sqrt(np.mean(v * v, axis=-1, keepdims=True) + eps)


def scalar_norm(x, g, eps):
    """The blocks' and the model's norm: one gain for all coordinates."""
    return rms(x, eps) * g


def sinusoid(positions, width, dtype=np.float64):
    """Entry 2i is sin(p w_i), entry 2i + 1 cos(p w_i), w_i = 10000^(-2i / width)."""
    i = np.arange((width + 1) // 2)
    w = (10000.0 ** (-2.0 * i / width)).astype(dtype)
    ang = np.asarray(positions, dtype=dtype)[:, None] * w[None, :]
    out = np.zeros((len(positions), 2 * len(i)), dtype=dtype)
    out[:, 0::2] = np.sin(ang)
    out[:, 1::2] = np.cos(ang)
    return out[:, :width]


def embed(config, W, tokens):
    x = W["embed"][np.asarray(tokens)]
    x = x + sinusoid(np.arange(len(tokens)), config["width"], x.dtype)
    return scalar_norm(x, W["embed.norm"], config["norm"]["eps"])


# ---- mixer: attention under a sliding window with a bias by distance ----------------------------------------

def query_temperature(positions, q_temp):
    """1 + coef ln(floor((p + 1) / every) + 1)."""
    return 1.0 + q_temp["coef"] * np.log(np.floor((np.asarray(positions) + 1) / q_temp["every"]) + 1.0)


def window_attention(h, W, p, m, eps, trace=None):
    n = h.shape[0]
    H, G, D, E = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms((h @ W[p + "q"].T).reshape(n, H, D), eps)
    k = rms((h @ W[p + "k"].T).reshape(n, G, D), eps)
    v = (h @ W[p + "v"].T).reshape(n, G, E)
    if m.get("q_temp"):
        q = q * query_temperature(np.arange(n), m["q_temp"]).astype(q.dtype)[:, None, None]
    size = m["mask"]["size"] if m.get("mask") else n
    out = np.zeros((n, H, E), dtype=h.dtype)
    for a in range(H):
        g = a // (H // G)
        r1, r2 = W[p + "r1"][a], W[p + "r2"][a]
        for i in range(n):
            lo = max(0, i - size + 1)
            dist = (i - np.arange(lo, i + 1)).astype(h.dtype)
            s = (k[lo:i + 1, g] @ q[i, a]) * m["scale"] - r1 * np.log(1.0 + r2 * dist)
            w = np.exp(s - s.max())
            out[i, a] = (w / w.sum()) @ v[lo:i + 1, g]
    if trace is not None:
        trace["attention.q"] = q.reshape(n, H * D)
        trace["attention"] = out.reshape(n, H * E)
    return out.reshape(n, H * E) @ W[p + "o"].T


# ---- mixer: a state space per head with an input-dependent step ------------------------------------------------

def causal_conv(u, taps, bias):
    """y[t, c] = bias[c] + sum_j taps[c, j] u[t - (K - 1) + j, c], zeros before the start."""
    n, K = u.shape[0], taps.shape[1]
    padded = np.concatenate([np.zeros((K - 1, u.shape[1]), dtype=u.dtype), u], axis=0)
    y = np.tile(bias[None, :], (n, 1)).astype(u.dtype)
    for j in range(K):
        y = y + padded[j:j + n] * taps[:, j][None, :]
    return y


def state_space(h, W, p, m, eps, trace=None):
    n = h.shape[0]
    H, E, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * E
    proj = h @ W[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, W[p + "conv"], W[p + "conv.b"]))
    xs = xbc[:, :inner].reshape(n, H, E)
    B = xbc[:, inner:inner + G * N].reshape(n, G, N)
    C = xbc[:, inner + G * N:].reshape(n, G, N)
    dt = softplus(dt + W[p + "dt_bias"][None, :])
    decay = np.exp(-np.exp(W[p + "A_log"])[None, :] * dt)
    read = np.zeros((n, H, E), dtype=h.dtype)
    for a in range(H):
        g = a // (H // G)
        S = np.zeros((N, E), dtype=h.dtype)
        for t in range(n):
            S = decay[t, a] * S + dt[t, a] * np.outer(B[t, g], xs[t, a])
            read[t, a] = S.T @ C[t, g]
    y = read + W[p + "D"][None, :, None] * xs
    y = y.reshape(n, inner) * silu(z)
    parts = m["norm_groups"]
    y = rms(y.reshape(n, parts, inner // parts), eps).reshape(n, inner) * W[p + "norm"][None, :]
    if trace is not None:
        trace["memory"] = read.reshape(n, inner)          # what the state gives, before the skip, the gate and the norm
        trace["state_space"] = y
    return y @ W[p + "o"].T


# ---- feed-forwards --------------------------------------------------------------------------------------------

def dense_ff(h, W, p):
    return (np.maximum(h @ W[p + "gate"].T, 0.0) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def expert(h, W, p, limit):
    g = np.minimum(h @ W[p + "gate"].T, limit)
    u = np.clip(h @ W[p + "up"].T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ W[p + "down"].T


def routed_ff(h, W, p, mlp, trace=None):
    n = h.shape[0]
    top, limit = mlp["router"]["top"], mlp["expert"]["limit"]
    z = h @ W[p + "router"].T + W[p + "router.b"][None, :]
    out = np.zeros((n, W[p + "e0.down"].shape[0]), dtype=h.dtype)
    chosen = np.zeros((n, top), dtype=np.int64)
    for t in range(n):
        ids = np.argsort(-z[t], kind="stable")[:top]
        w = np.exp(z[t, ids] - z[t, ids].max())
        w = w / w.sum()
        chosen[t] = ids
        for e, we in zip(ids, w):
            out[t] += we * expert(h[t:t + 1], W, f"{p}e{e}.", limit)[0]
    if trace is not None:
        trace["router"] = z
        trace["chosen"] = chosen
    return out


# ---- the model -------------------------------------------------------------------------------------------------

def weights_layer(config, i):
    """The layer whose tensors layer i uses."""
    seen = set()
    while "weights_of" in config["layers"][i] and config["layers"][i]["weights_of"] is not None:
        if i in seen:
            raise ValueError("weights_of runs in a circle")
        seen.add(i)
        i = config["layers"][i]["weights_of"]
    return i


def layer_forward(x, W, config, i, trace=None):
    eps = config["norm"]["eps"]
    j = weights_layer(config, i)
    L = config["layers"][j]
    p = f"l{j}."
    h = scalar_norm(x, W[p + "norm1"], eps)
    if L["type"] == "attention":
        x = x + window_attention(h, W, p + "mix.", L["mixer"], eps, trace)
    elif L["type"] == "mamba2":
        x = x + state_space(h, W, p + "mix.", L["mixer"], eps, trace)
    else:
        raise ValueError(L["type"])
    if trace is not None:
        trace["mixer"] = x
    mlp = L.get("mlp")
    if mlp is None:
        return x
    h = scalar_norm(x, W[p + "norm2"], eps)
    if mlp["kind"] == "dense":
        x = x + dense_ff(h, W, p + "mlp.")
    elif mlp["kind"] == "moe":
        x = x + routed_ff(h, W, p + "mlp.", mlp, trace)
        if trace is not None:
            trace["routed"] = x
    else:
        raise ValueError(mlp["kind"])
    return x


def forward(config, W, tokens, traces=None):
    """Logits [n, vocab] of one sequence; `traces` (a list) receives a dictionary per layer run with the mechanisms'
    intermediate rows and the stream after the run under "out"."""
    x = embed(config, W, tokens)
    if traces is not None:
        traces.append({"embed": x})
    for i in range(len(config["layers"])):
        tr = {} if traces is not None else None
        x = layer_forward(x, W, config, i, tr)
        if traces is not None:
            tr["out"] = x
            traces.append(tr)
    return scalar_norm(x, W["final.norm"], config["norm"]["eps"]) @ W["head"].T


def generate_greedy(config, W, prompt, n_new):
    tokens = list(prompt)
    for _ in range(n_new):
        tokens.append(int(np.argmax(forward(config, W, tokens)[-1])))
    return tokens[len(prompt):]
