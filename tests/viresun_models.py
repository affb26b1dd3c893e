"""Small Viresun configurations with random weights for the tests, written as model folders.

A differs from layer to layer in every size the design has: windows, temperatures, grouped and ungrouped key/value heads, query and
value sizes that differ, state spaces with one and several groups and convolutions of two to five taps, a block without a feed-forward,
experts of several shapes, and two layers that run on other layers' weights (an attention and a state space).  B has the sizes the
bfloat16 engine's tensor-core kernels take.  C has sizes that fit no kernel's pieces: a width that is no multiple of 8, value heads
wider than one tile of the state, a window of one position beside one wider than any prompt and a layer without a window, every expert
chosen (top = experts), a convolution of one tap.  D keeps sizes equal to one (heads, key/value heads, groups, one expert, a state of
one number, a value head of one value).
"""
from __future__ import annotations

import json
import os

import numpy as np


def attention(heads, kv_heads, dim, vdim, scale, window, coef=0.0, every=0):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=float(scale))
    if window:
        m["mask"] = dict(size=window)
    if every:
        m["q_temp"] = dict(coef=float(coef), every=every)
    return m


def state_space(heads, vdim, state, groups, conv, norm_groups):
    return dict(heads=heads, vdim=vdim, state=state, groups=groups, conv=conv, norm_groups=norm_groups)


def dense(ff):
    return dict(kind="dense", ff=ff)


def moe(experts, top, ff, limit):
    return dict(kind="moe", expert=dict(ff=ff, limit=float(limit)), router=dict(experts=experts, top=top))


def layer(mixer, mlp, weights_of=None):
    l = dict(type="mamba2" if "state" in mixer else "attention", mixer=mixer, mlp=mlp)
    if weights_of is not None:
        l["weights_of"] = weights_of
    return l


_A0 = layer(attention(4, 2, 12, 20, 0.3, 20, 0.5, 16), moe(6, 2, 24, 1.5))
_A1 = layer(state_space(4, 12, 10, 2, 4, 2), dense(136))
CONFIG_A = dict(architecture="Viresun", vocab=160, width=96, norm=dict(eps=1e-5), layers=[
    _A0,
    _A1,
    layer(attention(3, 3, 16, 8, 0.25, 33, 0.25, 7), None),
    dict(_A1, weights_of=1),
    layer(state_space(3, 24, 16, 1, 2, 1), moe(4, 1, 16, 0.75)),
    dict(_A0, weights_of=0),
    layer(state_space(6, 8, 6, 3, 5, 3), dense(48)),
])
CONFIG_B = dict(architecture="Viresun", vocab=200, width=128, norm=dict(eps=1e-6), layers=[
    layer(attention(4, 2, 64, 64, 0.125, 40, 0.5, 32), moe(8, 2, 64, 2.0)),
    layer(state_space(4, 32, 32, 2, 4, 2), dense(256)),
    layer(attention(8, 2, 32, 32, 0.18, 48, 1.0, 24), dense(128)),
    layer(state_space(2, 64, 64, 1, 4, 1), moe(4, 2, 128, 1.0)),
])
CONFIG_C = dict(architecture="Viresun", vocab=97, width=100, norm=dict(eps=1e-4), layers=[
    layer(attention(6, 1, 24, 40, 0.2, 1, 2.0, 5), moe(3, 3, 20, 1.25)),
    layer(attention(2, 2, 10, 6, 0.4, 1000, 0.3, 1), dense(50)),
    layer(state_space(2, 70, 10, 2, 1, 5), None),
    layer(attention(5, 5, 8, 8, 0.35, 0), dense(30)),
    layer(state_space(5, 6, 33, 5, 3, 2), moe(5, 2, 8, 0.5)),
])
_D0 = layer(state_space(1, 1, 1, 1, 2, 1), moe(1, 1, 8, 1.0))
CONFIG_D = dict(architecture="Viresun", vocab=64, width=48, norm=dict(eps=1e-5), layers=[
    _D0,
    layer(attention(1, 1, 1, 1, 1.0, 16, 1.0, 1), dense(1)),
    layer(attention(2, 1, 16, 16, 0.25, 31, 0.5, 64), dense(48)),
    dict(_D0, weights_of=0),
])
CONFIGS = {"A": (CONFIG_A, 31), "B": (CONFIG_B, 32), "C": (CONFIG_C, 33), "D": (CONFIG_D, 34)}


def to_bf16_values(a):
    """Rounds to values that bfloat16 holds, so that the file, the engine in either type and the plain model agree."""
    from liyab_b200.weights import bf16_to_f32, f32_to_bf16
    return bf16_to_f32(f32_to_bf16(np.asarray(a, dtype=np.float32)))


def random_weights(config, seed, router_std=3.0, router_bias_std=1.0):
    rng = np.random.default_rng(seed)
    V, W = config["vocab"], config["width"]
    out = {}

    def mat(name, rows, cols, std=None):
        out[name] = rng.normal(0.0, std if std is not None else cols ** -0.5, size=(rows, cols))

    def vec(name, n, mean, std):
        out[name] = rng.normal(mean, std, size=n)

    def one(name, mean, std):
        out[name] = np.asarray(rng.normal(mean, std))

    mat("embed", V, W, 1.0)
    one("embed.norm", 1.0, 0.1)
    mat("head", V, W)
    one("final.norm", 1.0, 0.1)
    for i, l in enumerate(config["layers"]):
        if l.get("weights_of") is not None:
            continue
        p, m = f"l{i}.", l["mixer"]
        one(p + "norm1", 1.0, 0.1)
        if l["type"] == "attention":
            H, G, D, E = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            mat(p + "mix.q", H * D, W)
            mat(p + "mix.k", G * D, W)
            mat(p + "mix.v", G * E, W)
            mat(p + "mix.o", W, H * E)
            out[p + "mix.r1"] = rng.uniform(0.0, 2.5, size=H)
            out[p + "mix.r2"] = rng.uniform(0.05, 0.4, size=H)
        else:
            H, E, N, G, K = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
            inner, channels = H * E, H * E + 2 * G * N
            mat(p + "mix.in", inner + channels + H, W)
            mat(p + "mix.conv", channels, K, K ** -0.5)
            vec(p + "mix.conv.b", channels, 0.0, 0.2)
            vec(p + "mix.dt_bias", H, -1.5, 0.8)
            vec(p + "mix.A_log", H, -1.0, 1.0)
            vec(p + "mix.D", H, 0.8, 0.2)
            vec(p + "mix.norm", inner, 1.0, 0.2)
            mat(p + "mix.o", W, inner)
        mlp = l["mlp"]
        if mlp:
            one(p + "norm2", 1.0, 0.1)
            if mlp["kind"] == "dense":
                mat(p + "mlp.gate", mlp["ff"], W)
                mat(p + "mlp.up", mlp["ff"], W)
                mat(p + "mlp.down", W, mlp["ff"])
            else:
                F, X = mlp["expert"]["ff"], mlp["router"]["experts"]
                mat(p + "mlp.router", X, W, router_std * W ** -0.5)
                vec(p + "mlp.router.b", X, 0.0, router_bias_std)
                for e in range(X):
                    mat(f"{p}mlp.e{e}.gate", F, W, 2.0 * W ** -0.5)      # wide enough for the cap to act on some values
                    mat(f"{p}mlp.e{e}.up", F, W, 2.0 * W ** -0.5)
                    mat(f"{p}mlp.e{e}.down", W, F)
    return {k: to_bf16_values(v) for k, v in out.items()}


def write_model(folder, config, weights):
    from liyab_b200.weights import f32_to_bf16, write_safetensors
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(config, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), {k: f32_to_bf16(v) for k, v in weights.items()},
                      tags={k: "BF16" for k in weights})
    return folder


def model_folder(base, name):
    config, seed = CONFIGS[name]
    weights = random_weights(config, seed)
    return write_model(os.path.join(base, f"viresun_{name}"), config, weights), config, weights
