"""Small Revudra configurations with random weights for the tests, written as model folders.

A differs from layer to layer in every size the design has: windows, grouped and ungrouped key/value heads, query and value sizes that
differ, rotations over part of a head and over all of it, three layers that blend values, memories with fast and slow decays, latent
attention with latents of several sizes, dense and table-routed feed-forwards with one and several experts a token, a block without a
feed-forward.  B has the sizes the bfloat16 engine's tensor-core kernels take.  C has sizes that fit no kernel's pieces: a width that is
no multiple of 8, a window of one position beside one wider than any prompt, a single layer that says it blends values (so none does),
every expert chosen (top = experts), a latent layer first, rotated parts of two values, no rotation at all.  D keeps sizes equal to one
(heads, key/value heads, one expert, heads of one value, a latent of one value).
"""
from __future__ import annotations

import json
import os

import numpy as np


def attention(heads, kv_heads, dim, vdim, scale, window, rot_dims, base=10000.0, v_mix=False):
    return dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=float(scale), mask=dict(size=window), rot=dict(base=float(base), dims=rot_dims),
                v_mix=v_mix)


def lightning(heads, dim, vdim, decay):
    assert len(decay) == heads
    return dict(heads=heads, dim=dim, vdim=vdim, decay=[float(d) for d in decay])


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base=10000.0):
    return dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, q_rank=q_rank, scale=float(scale), rot=dict(base=float(base), dims=rot_dim))


def dense(ff):
    return dict(kind="dense", ff=ff)


def moe(experts, top, ff):
    return dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top))


def layer(mixer, mlp):
    kind = "lightning" if "decay" in mixer else "latent_attention" if "kv_rank" in mixer else "attention"
    return dict(type=kind, mixer=mixer, mlp=mlp)


def model(vocab, width, eps, mult, embed_scale, logit_scale, layers):
    return dict(architecture="Revudra", vocab=vocab, width=width, norm=dict(eps=eps), residual_mult=mult, embedding=dict(scale=embed_scale),
                logit_scale=logit_scale, layers=layers)


CONFIG_A = model(160, 96, 1e-5, 0.6, 0.7, 1.5, [
    layer(lightning(3, 12, 20, [0.5, 0.9, 0.995]), moe(6, 2, 24)),
    layer(attention(4, 2, 12, 10, 0.3, 20, 8, 5000.0, True), dense(136)),
    layer(latent(3, 10, 6, 14, 24, 18, 0.25, 300.0), moe(4, 1, 16)),
    layer(attention(5, 5, 8, 4, 0.35, 33, 8, 100.0, True), None),
    layer(attention(2, 1, 16, 20, 0.25, 47, 4, 1e6, True), moe(5, 3, 8)),
    layer(lightning(2, 8, 8, [0.8, 0.97]), dense(48)),
    layer(latent(5, 4, 8, 8, 40, 7, 0.3), dense(40)),
])
CONFIG_B = model(200, 128, 1e-6, 0.8, 0.5, 2.0, [
    layer(attention(4, 2, 64, 64, 0.125, 40, 32, 10000.0, True), moe(8, 2, 64)),
    layer(lightning(4, 32, 32, [0.7, 0.9, 0.97, 0.999]), dense(256)),
    layer(latent(4, 32, 16, 32, 64, 48, 0.14), moe(4, 1, 128)),
    layer(attention(8, 4, 128, 32, 0.09, 48, 32, 5e5, True), dense(128)),
    layer(latent(16, 16, 32, 16, 128, 80, 0.15, 30000.0), None),
])
CONFIG_C = model(97, 100, 1e-4, 1.0, 1.0, 1.0, [
    layer(latent(2, 6, 2, 70, 10, 5, 0.4), moe(3, 3, 20)),
    layer(attention(6, 1, 24, 40, 0.2, 1, 0, 10000.0, True), dense(50)),
    layer(attention(2, 2, 10, 6, 0.4, 1000, 10), None),
    layer(lightning(5, 6, 33, [0.3, 0.6, 0.9, 0.99, 1.0]), moe(5, 2, 8)),
    layer(latent(3, 8, 0, 8, 12, 9, 0.35), dense(30)),
])
CONFIG_D = model(64, 48, 1e-5, 0.5, 2.0, 0.25, [
    layer(attention(1, 1, 2, 1, 1.0, 16, 2, 10.0, True), moe(1, 1, 8)),
    layer(lightning(1, 1, 1, [0.9]), dense(1)),
    layer(latent(1, 1, 2, 1, 1, 1, 1.0), moe(2, 1, 4)),
    layer(attention(2, 1, 16, 1, 0.25, 31, 16, 10000.0, True), dense(48)),
])
CONFIGS = {"A": (CONFIG_A, 41), "B": (CONFIG_B, 42), "C": (CONFIG_C, 43), "D": (CONFIG_D, 44)}


def to_bf16_values(a):
    """Rounds to values that bfloat16 holds, so that the file, the engine in either type and the plain model agree."""
    from liyab_b200.weights import bf16_to_f32, f32_to_bf16
    return bf16_to_f32(f32_to_bf16(np.asarray(a, dtype=np.float32)))


def random_weights(config, seed):
    """The file's tensors: floats rounded to bfloat16's values, the experts' tables as int32."""
    rng = np.random.default_rng(seed)
    V, W = config["vocab"], config["width"]
    out, tables = {}, {}

    def mat(name, rows, cols, std=None):
        out[name] = rng.normal(0.0, std if std is not None else cols ** -0.5, size=(rows, cols))

    def vec(name, n, mean, std):
        out[name] = rng.normal(mean, std, size=n)

    mat("embed", V, W, 1.0)
    mat("head", V, W)
    vec("final.norm", W, 1.0, 0.1)
    for i, l in enumerate(config["layers"]):
        p, m = f"l{i}.", l["mixer"]
        vec(p + "norm1", W, 1.0, 0.2)
        H, D, E = m["heads"], m["dim"], m["vdim"]
        if l["type"] == "attention":
            G = m["kv_heads"]
            mat(p + "mix.q", H * D, W)
            mat(p + "mix.k", G * D, W)
            mat(p + "mix.v", G * E, W)
            mat(p + "mix.g", H * E, W)
            vec(p + "mix.q.norm", H * D, 1.0, 0.3)
            vec(p + "mix.k.norm", G * D, 1.0, 0.3)
            out[p + "mix.vmix"] = np.asarray(rng.uniform(0.2, 0.8))
            vec(p + "mix.sink", H, 0.5, 1.0)
        elif l["type"] == "lightning":
            mat(p + "mix.q", H * D, W)
            mat(p + "mix.k", H * D, W)
            mat(p + "mix.v", H * E, W)
            mat(p + "mix.g", H * E, W)
            vec(p + "mix.norm", H * E, 1.0, 0.2)
        else:
            R, C, Q = m["rot_dim"], m["kv_rank"], m["q_rank"]
            mat(p + "mix.dq", Q, W)
            vec(p + "mix.dq.norm", Q, 1.0, 0.2)
            mat(p + "mix.uq", H * (D + R), Q)
            mat(p + "mix.dkv", C + R, W)
            vec(p + "mix.dkv.norm", C, 1.0, 0.2)
            mat(p + "mix.uk", H * D, C)
            mat(p + "mix.uv", H * E, C)
            vec(p + "mix.sink", H, 0.5, 1.0)
            mat(p + "mix.g", H, W, 2.0 * W ** -0.5)
        mat(p + "mix.o", W, H * E)
        mlp = l["mlp"]
        if mlp:
            vec(p + "norm2", W, 1.0, 0.2)
            if mlp["kind"] == "dense":
                mat(p + "mlp.up", mlp["ff"], W)
                mat(p + "mlp.down", W, mlp["ff"])
            else:
                F, X, top = mlp["expert"]["ff"], mlp["router"]["experts"], mlp["router"]["top"]
                for e in range(X):
                    mat(f"{p}mlp.e{e}.gate", F, W)
                    mat(f"{p}mlp.e{e}.up", F, W)
                    mat(f"{p}mlp.e{e}.down", W, F)
                tables[p + "mlp.table"] = np.stack([rng.permutation(X)[:top] for _ in range(V)]).astype(np.int32)
    weights = {k: to_bf16_values(v) for k, v in out.items()}
    weights.update(tables)
    return weights


def f64(weights):
    return {k: (v if v.dtype == np.int32 else np.asarray(v, dtype=np.float64)) for k, v in weights.items()}


def write_model(folder, config, weights):
    from liyab_b200.weights import f32_to_bf16, write_safetensors
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(config, f)
    floats = {k for k, v in weights.items() if v.dtype != np.int32}
    write_safetensors(os.path.join(folder, "model.safetensors"), {k: (f32_to_bf16(v) if k in floats else np.ascontiguousarray(v)) for k, v in weights.items()},
                      tags={k: "BF16" for k in floats})
    return folder


def model_folder(base, name):
    config, seed = CONFIGS[name]
    weights = random_weights(config, seed)
    return write_model(os.path.join(base, f"revudra_{name}"), config, weights), config, weights
