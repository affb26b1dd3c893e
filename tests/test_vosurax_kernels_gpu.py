"""The kernels behind gated mixers, matrix memories and routed experts, each by itself against float64 statements of the same
operation written here: norm with gains around zero, a row added to the stream, branches summed over their root mean squares,
queries and keys normalised per head into padded heads and cache pages, the gate on heads, the gated product, the matrix
memories (row by row and in pieces, both kinds, value tiles of every width, rows cut anywhere, slots in scrambled order) and
the routed experts (32-bit units and tensor cores)."""
from __future__ import annotations

import math

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def dev(a, dtype=None):
    import torch
    t = torch.as_tensor(np.ascontiguousarray(a)).cuda()
    return t.to(dtype) if dtype is not None else t


def host(t):
    return t.float().cpu().numpy().astype(np.float64)


def rms(v, eps):
    return v / np.sqrt((v * v).mean(axis=-1, keepdims=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def test_norm_with_gains_around_zero_and_added_row():
    import torch
    from liyab_b200 import ops
    rng = np.random.default_rng(0)
    x, w, v = rng.normal(size=(37, 100)), rng.normal(0, 0.3, size=100), rng.normal(size=100)
    out = ops.rms_offset(dev(x, torch.float32), dev(w, torch.float32), 1.0, 1e-4, torch.empty(37, 100, dtype=torch.float32, device="cuda"))
    assert np.abs(host(out) - rms(x, 1e-4) * (1.0 + w)).max() < 1e-5
    xs = dev(x, torch.float32)
    ops.add_row(xs, dev(v, torch.float32))
    assert np.abs(host(xs) - (x + v)).max() < 1e-6


@pytest.mark.parametrize("n", [1, 2, 3])
def test_branches_summed_over_their_root_mean_squares(n):
    import torch
    from liyab_b200 import ops
    rng = np.random.default_rng(n)
    x = rng.normal(size=(19, 70))
    ys = [rng.normal(0, 3.0 ** i, size=(19, 70)) for i in range(n)]
    ws = [rng.normal(1, 0.2, size=70) if i != 1 else None for i in range(n)]
    want = x + 0.5 * sum(rms(y, 1e-5) * (w if w is not None else 1.0) for y, w in zip(ys, ws))
    xs = dev(x, torch.float32)
    ops.rms_sum_add(xs, [dev(y, torch.float32) for y in ys], [dev(w, torch.float32) if w is not None else None for w in ws], 0.5, 1e-5)
    assert np.abs(host(xs) - want).max() < 1e-5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,D,E,P", [(4, 2, 12, 20, 20), (3, 1, 48, 8, 64), (1, 1, 1, 1, 4)])
def test_queries_and_keys_normalised_into_padded_heads(dtype, H, G, D, E, P):
    import torch
    from liyab_b200 import ops
    dt = getattr(torch, dtype)
    rng = np.random.default_rng(H)
    T, page = 9, 4
    cols = 5 + H * D + G * D + G * E + 3
    proj = rng.normal(size=(T, cols))
    qw, kw = rng.normal(1, 0.2, size=D), rng.normal(1, 0.2, size=D)
    slots = np.array([3, -1, 0, 11, 5, 6, 2, 9, 10], dtype=np.int32)
    cache = torch.full((3, 2, G, page, P), float("nan"), dtype=dt, device="cuda")
    q_out = torch.full((T, H * P), float("nan"), dtype=dt, device="cuda")
    ops.qk_norm_store(dev(proj, torch.float32), 5, 5 + H * D, 5 + H * D + G * D, dev(qw, torch.float32), dev(kw, torch.float32), q_out, cache, dev(slots),
                      H, G, D, E, P, page, True, 1e-5)
    tol = 1e-5 if dtype == "float32" else 2e-2
    q = proj[:, 5:5 + H * D].reshape(T, H, D)
    want_q = np.zeros((T, H, P))
    want_q[:, :, :D] = rms(q, 1e-5) * qw
    assert np.abs(host(q_out).reshape(T, H, P) - want_q).max() < tol
    k = rms(proj[:, 5 + H * D:5 + H * D + G * D].reshape(T, G, D), 1e-5) * kw
    v = proj[:, 5 + H * D + G * D:5 + H * D + G * D + G * E].reshape(T, G, E)
    got = host(cache)
    for t, s in enumerate(slots):
        if s < 0:
            continue
        pg, off = divmod(int(s), page)
        assert np.abs(got[pg, 0, :, off, :D] - k[t]).max() < tol and np.abs(got[pg, 1, :, off, :E] - v[t]).max() < tol
        assert np.all(got[pg, 0, :, off, D:] == 0) and np.all(got[pg, 1, :, off, E:] == 0)
    assert np.isnan(got[0, 0, 0, 1]).all()          # slot 1 belongs to no token


@pytest.mark.parametrize("norm,gate,gain", [(True, "silu", False), (True, "sigmoid", True), (False, "sigmoid", False), (False, None, False)])
def test_the_gate_on_heads(norm, gate, gain):
    import torch
    from liyab_b200 import ops
    rng = np.random.default_rng(3)
    T, H, E, P = 11, 3, 10, 16
    o, g, w = rng.normal(size=(T, H, P)), rng.normal(size=(T, H * E)), rng.normal(1, 0.3, size=H * E)
    out = torch.empty(T, H * E, dtype=torch.float32, device="cuda")
    ops.head_gate(dev(o.reshape(T, H * P), torch.float32), P, dev(g, torch.float32) if gate else None, dev(w, torch.float32) if gain else None, out, H, E, norm,
                  gate or "sigmoid", 1e-5)
    want = o[:, :, :E]
    if norm:
        want = rms(want, 1e-5)
    want = want.reshape(T, H * E) * (w if gain else 1.0)
    if gate:
        want = want * (sigmoid(g) if gate == "sigmoid" else g * sigmoid(g))
    assert np.abs(host(out) - want).max() < 1e-5


def plain_memory(q, k, v, zi, zf, decay, cap, S, nvec, m):
    """One head, row by row, from the state (S, n, m); returns the outputs and the state after."""
    out = np.zeros((q.shape[0], v.shape[1]))
    for t in range(q.shape[0]):
        if decay is not None:
            keep, take = decay, 1.0
        else:
            gi = cap * math.tanh(zi[t] / cap)
            z = cap * math.tanh(zf[t] / cap)
            gf = -(math.log1p(math.exp(-abs(z))) + max(-z, 0.0))
            new = max(gf + m, gi)
            keep, take, m = math.exp(gf + m - new), math.exp(gi - new), new
        S = keep * S + take * np.outer(k[t], v[t])
        nvec = keep * nvec + take * k[t]
        o = S.T @ q[t]
        out[t] = o if decay is not None else o / (max(abs(float(nvec @ q[t])), math.exp(-m)) + 1e-6)
    return out, S, nvec, m


@pytest.mark.parametrize("gated", [False, True])
@pytest.mark.parametrize("H,D,E,tile", [(2, 16, 24, 24), (3, 10, 70, 24), (1, 64, 128, 32), (2, 6, 5, 5), (1, 20, 130, 64), (2, 1, 1, 1)])
def test_matrix_memories_row_by_row_and_in_pieces(gated, H, D, E, tile):
    """Three requests of unequal length in one launch, each in several steps cut anywhere, through slots in scrambled order; every step once row by
    row, once in pieces and once with every piece a block of its own, from the same state; rotation of part of a head; against the plain recurrence in float64."""
    import torch
    from liyab_b200 import ops
    rng = np.random.default_rng(7 * H + D)
    lens, cuts = [75, 33, 1], [[40, 41, 75], [2, 33], [1]]
    rot = 0 if gated or D < 4 else (D // 4) * 2
    freq = np.array([50.0 ** (-2.0 * i / rot) for i in range(rot // 2)]) if rot else None
    cols = 2 * H * D + H * E + 2 * H
    rows = {r: rng.normal(0, 1.0, size=(n, cols)) for r, n in enumerate(lens)}
    decay = None if gated else rng.uniform(0.8, 1.0, size=H)
    cap, qs, ks = 7.0, D ** -0.5 if gated else 1.0, 1.0 if gated else D ** -0.5
    slots = {0: 2, 1: 0, 2: 3}
    floats = ops.memory_slot_floats(H, D, E, tile)
    states = {mode: torch.zeros(4, floats, dtype=torch.float32, device="cuda") for mode in (False, True, "pieces")}
    plain_state = {(r, h): (np.zeros((D, E)), np.zeros(D), 0.0) for r in rows for h in range(H)}
    at = {r: 0 for r in rows}
    for step in range(3):
        live = [r for r in rows if step < len(cuts[r])]
        parts = [rows[r][at[r]:cuts[r][step]] for r in live]
        pos = np.concatenate([np.arange(at[r], cuts[r][step]) for r in live]).astype(np.int32)
        q_start = np.concatenate([[0], np.cumsum([len(p) for p in parts])]).astype(np.int32)
        proj = np.concatenate(parts, axis=0)
        want = np.zeros((proj.shape[0], H * E))
        for i, r in enumerate(live):
            x = parts[i]
            for h in range(H):
                q = x[:, h * D:(h + 1) * D].copy()
                k = x[:, H * D + h * D:H * D + (h + 1) * D].copy()
                if rot:
                    half = rot // 2
                    ang = np.arange(at[r], cuts[r][step])[:, None] * freq[None, :]
                    for arr in (q, k):
                        a, b = arr[:, :half].copy(), arr[:, half:rot].copy()
                        arr[:, :half] = a * np.cos(ang) - b * np.sin(ang)
                        arr[:, half:rot] = b * np.cos(ang) + a * np.sin(ang)
                v = x[:, 2 * H * D + h * E:2 * H * D + (h + 1) * E]
                S, nv, m = plain_state[(r, h)]
                o, S, nv, m = plain_memory(q * qs, k * ks, v, x[:, 2 * H * D + H * E + h], x[:, 2 * H * D + H * E + H + h], None if gated else float(decay[h]), cap, S, nv, m)
                plain_state[(r, h)] = (S, nv, m)
                want[q_start[i]:q_start[i + 1], h * E:(h + 1) * E] = o
        for chunked in (False, True, "pieces"):
            out = torch.full((proj.shape[0], H * E), float("nan"), dtype=torch.float32, device="cuda")
            args = (dev(proj, torch.float32), 0, H * D, 2 * H * D, 2 * H * D + H * E if gated else None, 2 * H * D + H * E + H if gated else None,
                    None if gated else dev(decay, torch.float32), dev(freq, torch.float32) if rot else None, rot, dev(pos), dev(q_start),
                    dev(np.array([slots[r] for r in live], dtype=np.int32)), states[chunked], out, H, D, E, tile, qs, ks, cap)
            if chunked == "pieces":
                ops.matrix_memory_pieces(*args)
            else:
                ops.matrix_memory(*args, chunked)
            err = np.abs(host(out) - want).max() / max(np.abs(want).max(), 1e-30)
            assert err < 5e-5, f"step {step}, {chunked}: {err:.2e}"
        for r in live:
            at[r] = cuts[r][step]
    for other in (True, "pieces"):
        assert float((states[False] - states[other]).abs().max()) < 1e-3 * float(states[False].abs().max())
    assert float(states[False][1].abs().max()) == 0.0           # the slot no request used


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,E,top,width,inner", [(70, 6, 2, 96, 24), (3, 4, 1, 64, 16), (300, 16, 3, 128, 72), (40, 3, 3, 100, 10), (1, 1, 1, 8, 8),
                                                 (20, 5, 3, 128, 40), (9, 16, 2, 256, 72), (32, 2, 2, 64, 264)])
def test_routed_experts(dtype, T, E, top, width, inner):
    """Router, plan, both products and the sum against the plain statement; in bfloat16 the tensor-core products (and, for up to 64 pairs, the
    products a pair at a time) against the ones on the 32-bit units as well.  The router's matrix is large, so that the experts are chosen by clear margins in either type."""
    import torch
    from liyab_b200 import ops
    dt = getattr(torch, dtype)
    rng = np.random.default_rng(T + E)
    r16 = lambda a: host(dev(a, dt))
    h, x = r16(rng.normal(size=(T, width))), rng.normal(size=(T, width))
    router = r16(rng.normal(0, 6.0 / math.sqrt(width), size=(E, width)))
    gate_up = r16(rng.normal(0, width ** -0.5, size=(E, 2 * inner, width)))
    down = r16(rng.normal(0, inner ** -0.5, size=(E, width, inner)))
    z = h @ router.T
    order = np.argsort(-z, axis=1, kind="stable")[:, :top]
    want = x.copy()
    for t in range(T):
        for e in order[t]:
            a = sigmoid(z[t, e]) * h[t]
            g, u = gate_up[e, :inner] @ a, gate_up[e, inner:] @ a
            want[t] += down[e] @ (g * sigmoid(g) * u)
    results = {}
    for plain in ((False,) if dtype == "float32" else (False, True)):
        xs = dev(x, torch.float32)
        ids, weights = ops.routed_experts(dev(h, dt), dev(router, dt), dev(gate_up, dt), dev(down, dt), xs, top, plain=plain)
        margins = np.sort(z, axis=1)
        if E > top and (margins[:, E - top] - margins[:, E - top - 1]).min() > 0.05:
            assert np.array_equal(host(ids).astype(int), order)
            assert np.abs(host(weights) - sigmoid(np.take_along_axis(z, order, 1))).max() < 1e-5
        results[plain] = host(xs)
        err = np.abs(results[plain] - want).max() / np.abs(want - x).max()
        assert err < (1e-5 if dtype == "float32" else 2e-2), f"plain={plain}: {err:.2e}"
    if dtype == "bfloat16":
        assert np.abs(results[False] - results[True]).max() / np.abs(want - x).max() < 1e-2
