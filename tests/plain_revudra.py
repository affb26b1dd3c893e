"""A plain, slow restatement of the Revudra design in numpy: one function per mechanism, whole sequences at a
time, token by token where the design has a recurrence, no cache and no batching.  It shares nothing with the
engine; the tests compare the engine's logits with it.

A model is (config, weights): `config` is the dictionary of the design's config.json, `weights` maps the
file's tensor names to arrays.  Everything is computed in the arrays' own type (float64 in the tests).

Notation: x is the residual stream [n, width]; a sublayer reads x as it is and its result passes a norm before
it joins the stream, x <- x + m norm(sublayer(x)); position p counts from 0.
"""
import numpy as np


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def rms_norm(v, w, eps):
    """v / sqrt(mean(v^2) + eps) * w over the last axis."""
    return v / np.sqrt(np.mean(v * v, axis=-1, keepdims=True) + eps) * w


def embed(config, W, tokens):
    return W["embed"][np.asarray(tokens)] * config["embedding"]["scale"]


# ---- rotations ---------------------------------------------------------------------------------------------

def rotate(v, positions, rot, interleaved):
    """Rotates the first rot.dims values of the last axis of v [n, heads, size]; the rest pass.  Pair i is (i, i + dims/2) in the
    half layout and (2i, 2i + 1) in the interleaved one; its angle is p * base^(-2i/dims)."""
    dims = rot["dims"]
    half = dims // 2
    if half == 0:
        return v
    f = np.asarray(rot["base"], dtype=v.dtype) ** (-2.0 * np.arange(half) / dims)
    ang = np.asarray(positions, dtype=v.dtype)[:, None] * f[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    out = v.copy()
    if interleaved:
        a, b = v[..., 0:dims:2], v[..., 1:dims:2]
        out[..., 0:dims:2] = a * c - b * s
        out[..., 1:dims:2] = b * c + a * s
    else:
        a, b = v[..., :half], v[..., half:dims]
        out[..., :half] = a * c - b * s
        out[..., half:dims] = b * c + a * s
    return out


def softmax_with_sink(s, sink):
    """Weights of the scores s when the divisor also holds exp(sink), which has no value of its own."""
    top = max(s.max(), sink)
    w = np.exp(s - top)
    return w / (w.sum() + np.exp(sink - top))


# ---- mixer: attention under a sliding window -----------------------------------------------------------------

def window_attention(h, W, p, m, eps, shared, trace=None):
    """`shared` carries the first value-mixing layer's values from layer to layer."""
    n = h.shape[0]
    H, G, D, E = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = np.arange(n)
    q = rms_norm(h @ W[p + "q"].T, W[p + "q.norm"], eps).reshape(n, H, D)
    k = rms_norm(h @ W[p + "k"].T, W[p + "k.norm"], eps).reshape(n, G, D)
    v = (h @ W[p + "v"].T).reshape(n, G, E)
    q = rotate(q, pos, m["rot"], False)
    k = rotate(k, pos, m["rot"], False)
    if m.get("v_mix"):
        if "v_first" in shared:
            lam = W[p + "vmix"]
            v = (1.0 - lam) * v + lam * shared["v_first"].reshape(v.shape)      # a token's values side by side, however the heads cut them
        else:
            shared["v_first"] = v
    size = m["mask"]["size"]
    out = np.zeros((n, H, E), dtype=h.dtype)
    for a in range(H):
        g = a // (H // G)
        for i in range(n):
            lo = max(0, i - size + 1)
            s = (k[lo:i + 1, g] @ q[i, a]) * m["scale"]
            out[i, a] = softmax_with_sink(s, W[p + "sink"][a]) @ v[lo:i + 1, g]
    gated = out.reshape(n, H * E) * sigmoid(h @ W[p + "g"].T)
    if trace is not None:
        trace.update(q=q, k=k, v=v, attention=out.reshape(n, H * E), gated=gated)
    return gated @ W[p + "o"].T


# ---- mixer: a matrix memory per head with a fixed decay ------------------------------------------------------

def lightning(h, W, p, m, eps, trace=None):
    n = h.shape[0]
    H, D, E = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ W[p + "q"].T).reshape(n, H, D)
    k = silu(h @ W[p + "k"].T).reshape(n, H, D)
    v = silu(h @ W[p + "v"].T).reshape(n, H, E)
    out = np.zeros((n, H, E), dtype=h.dtype)
    for a in range(H):
        S = np.zeros((D, E), dtype=h.dtype)
        for t in range(n):
            S = m["decay"][a] * S + np.outer(k[t, a], v[t, a])
            out[t, a] = S.T @ q[t, a]
    if trace is not None:
        trace.update(memory=out.reshape(n, H * E))
    y = rms_norm(out.reshape(n, H * E), W[p + "norm"], eps) * sigmoid(h @ W[p + "g"].T)
    return y @ W[p + "o"].T


# ---- mixer: attention whose keys and values come from a latent row -------------------------------------------

def latent_attention(h, W, p, m, eps, trace=None):
    n = h.shape[0]
    H, D, R, E, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = np.arange(n)
    cq = rms_norm(h @ W[p + "dq"].T, W[p + "dq.norm"], eps)
    q = (cq @ W[p + "uq"].T).reshape(n, H, D + R)
    down = h @ W[p + "dkv"].T
    c = rms_norm(down[:, :C], W[p + "dkv.norm"], eps)
    shared_key = rotate(down[:, None, C:], pos, m["rot"], True)[:, 0]
    q_plain, q_rot = q[..., :D], rotate(q[..., D:], pos, m["rot"], True)
    k_plain = (c @ W[p + "uk"].T).reshape(n, H, D)
    v = (c @ W[p + "uv"].T).reshape(n, H, E)
    out = np.zeros((n, H, E), dtype=h.dtype)
    for a in range(H):
        for i in range(n):
            s = (k_plain[:i + 1, a] @ q_plain[i, a] + shared_key[:i + 1] @ q_rot[i, a]) * m["scale"]
            out[i, a] = softmax_with_sink(s, W[p + "sink"][a]) @ v[:i + 1, a]
    gate = sigmoid(h @ W[p + "g"].T)                     # one number a head
    gated = (out * gate[:, :, None]).reshape(n, H * E)
    if trace is not None:
        trace.update(latent=c, shared_key=shared_key, attention=out.reshape(n, H * E), gated=gated)
    return gated @ W[p + "o"].T


# ---- feed-forwards -------------------------------------------------------------------------------------------

def dense_ff(h, W, p):
    return np.maximum(h @ W[p + "up"].T, 0.0) ** 2 @ W[p + "down"].T


def expert(h, W, p):
    return (silu(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def table_ff(h, W, p, mlp, tokens):
    """Every token id has its experts in a table; each counts 1/top."""
    top = mlp["router"]["top"]
    y = np.zeros((h.shape[0], W[p + "e0.down"].shape[0]), dtype=h.dtype)
    for t, tok in enumerate(tokens):
        for e in W[p + "table"][tok]:
            y[t] += expert(h[t], W, f"{p}e{int(e)}.") / top
    return y


# ---- a layer and the model -------------------------------------------------------------------------------------

def layer_forward(x, W, config, i, tokens, shared, trace=None):
    l = config["layers"][i]
    eps, mult = config["norm"]["eps"], config["residual_mult"]
    p = f"l{i}."
    if l["type"] == "attention":
        y = window_attention(x, W, p + "mix.", l["mixer"], eps, shared, trace)
    elif l["type"] == "lightning":
        y = lightning(x, W, p + "mix.", l["mixer"], eps, trace)
    elif l["type"] == "latent_attention":
        y = latent_attention(x, W, p + "mix.", l["mixer"], eps, trace)
    else:
        raise ValueError(l["type"])
    if trace is not None:
        trace["mixer"] = y
    x = x + mult * rms_norm(y, W[p + "norm1"], eps)
    mlp = l.get("mlp")
    if mlp:
        y = dense_ff(x, W, p + "mlp.") if mlp["kind"] == "dense" else table_ff(x, W, p + "mlp.", mlp, tokens)
        if trace is not None:
            trace["feed_forward"] = y
        x = x + mult * rms_norm(y, W[p + "norm2"], eps)
    return x


def forward(config, W, tokens, traces=None):
    """Logits [n, vocab] of one sequence; `traces` (a list) receives a dictionary per layer with the mechanisms'
    intermediate rows and the stream after the layer under "out"."""
    x = embed(config, W, tokens)
    shared = {}
    if traces is not None:
        traces.append({"embed": x})
    for i in range(len(config["layers"])):
        tr = {} if traces is not None else None
        x = layer_forward(x, W, config, i, tokens, shared, tr)
        if traces is not None:
            tr["out"] = x
            traces.append(tr)
    return rms_norm(x, W["final.norm"], config["norm"]["eps"]) @ W["head"].T * config["logit_scale"]


def generate_greedy(config, W, prompt, n_new):
    tokens = list(prompt)
    for _ in range(n_new):
        tokens.append(int(np.argmax(forward(config, W, tokens)[-1])))
    return tokens[len(prompt):]
