"""The kernels that came with Revudra, each by itself against a float64 statement written here: the sink in every attention kernel
(32-bit, scalar and tensor-core decode with split keys, mma.sync and tcgen05 prefill), queries, keys and values normed over the whole
projection, rotated and blended on their way to the cache, the norm over all heads with a gate, the activation over a projection's
columns, the square of relu in the products' epilogues, and the experts looked up by token id."""
from __future__ import annotations

import math

import numpy as np
import pytest
import torch

from test_kernels_gpu import _paged_case

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    return torch.device("cuda:0")


def reference_attention(refs, n_head, n_kv_head, scale, window, sink):
    """Weights exp(s_j) / (sum_j exp(s_j) + exp(sink_h)) over the keys j with 0 <= i - j < window (all earlier keys without one)."""
    outs = []
    group = n_head // n_kv_head
    for q, k, v, first in refs:
        Q, L = q.shape[0], k.shape[0]
        o = torch.zeros(Q, n_head, q.shape[2], dtype=torch.float64)
        pos = torch.arange(first, first + Q)[:, None]
        j = torch.arange(L)[None, :]
        mask = j <= pos
        if window > 0:
            mask &= j > pos - window
        for h in range(n_head):
            s = ((q[:, h] @ k[:, h // group].t()) * scale).masked_fill(~mask, float("-inf"))
            s = torch.cat([s, torch.full((Q, 1), float(sink[h]), dtype=torch.float64)], dim=1)       # the sink as a key of its own ...
            o[:, h] = torch.softmax(s, dim=-1)[:, :L] @ v[:, h // group]                              # ... that brings no value
        outs.append(o.reshape(Q, -1))
    return torch.cat(outs)


def sinks(n_head, seed, dev):
    s = np.random.default_rng(seed).uniform(-1.0, 4.0, n_head)
    s[0] = -1e30                                     # a head whose sink weighs nothing beside heads where it weighs much
    t = torch.tensor(s, dtype=torch.float32, device=dev)
    return t, t.double().cpu()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_head,n_kv_head,head_dim,page_size,window", [(4, 4, 16, 16, 0), (6, 2, 48, 32, 0), (5, 1, 64, 64, 70), (4, 2, 24, 16, 33), (2, 1, 64, 32, 7),
                                                                        (12, 3, 128, 16, 88)])
def test_generic_attention_with_sinks(dev, dtype, n_head, n_kv_head, head_dim, page_size, window):
    from liyab_b200 import ops
    lens, q_lens = [1, 37, 130, 64, 300], [1, 37, 2, 1, 45]
    scale = 0.9 / math.sqrt(head_dim)
    q, cache, tok_seq, positions, table, refs = _paged_case(dev, dtype, n_head, n_kv_head, head_dim, page_size, lens, q_lens, seed=head_dim + n_head)
    s, s64 = sinks(n_head, head_dim, dev)
    ref = reference_attention(refs, n_head, n_kv_head, scale, window, s64)
    without = reference_attention(refs, n_head, n_kv_head, scale, window, s64 * 0 - 1e30)
    assert (ref - without).abs().max().item() > 0.05, "the sinks do not show"
    out = torch.empty_like(q)
    ops.paged_attention_generic(q, cache, tok_seq, positions, table, out, q.shape[0], n_head, n_kv_head, head_dim, page_size, scale, window, sink=s)
    assert (out.double().cpu() - ref).abs().max().item() < (2e-5 if dtype == torch.float32 else 1.5e-2)
    # Without sinks the kernel is the one it was.
    ops.paged_attention_generic(q, cache, tok_seq, positions, table, out, q.shape[0], n_head, n_kv_head, head_dim, page_size, scale, window)
    assert (out.double().cpu() - without).abs().max().item() < (2e-5 if dtype == torch.float32 else 1.5e-2)


@pytest.mark.parametrize("n_head,n_kv_head,head_dim,page_size,window,splits", [
    (12, 12, 64, 16, 0, 1), (12, 12, 64, 16, 0, 5), (4, 4, 16, 16, 0, 3), (12, 3, 128, 16, 88, 4), (16, 2, 64, 64, 0, 7), (6, 3, 64, 16, 33, 4),
    (4, 4, 32, 16, 5, 16), (5, 5, 128, 32, 70, 2), (2, 1, 256, 16, 200, 9), (32, 2, 64, 16, 0, 3), (16, 1, 128, 16, 0, 8), (12, 3, 64, 16, 300, 12)])
def test_decode_attention_with_sinks(dev, n_head, n_kv_head, head_dim, page_size, window, splits):
    """One new token per request, keys split several ways: the sink joins once, where the ranges meet, however many there are."""
    from liyab_b200 import ops
    lens = [1, 2, 17, 64, 65, 300, 1024, 33]
    scale = 0.9 / math.sqrt(head_dim)
    q, cache, tok_seq, positions, table, refs = _paged_case(dev, torch.bfloat16, n_head, n_kv_head, head_dim, page_size, lens, [1] * len(lens),
                                                            seed=7 * head_dim + splits)
    S = len(lens)
    s, s64 = sinks(n_head, splits, dev)
    ref = reference_attention(refs, n_head, n_kv_head, scale, window, s64)
    assert (ref - reference_attention(refs, n_head, n_kv_head, scale, window, s64 * 0 - 1e30)).abs().max().item() > 0.05
    partial = torch.full((S * n_head * splits * (head_dim + 2),), float("nan"), device=dev)
    counters = torch.zeros(S * n_kv_head, dtype=torch.int32, device=dev)
    scalar, tensor = ops.decode_attention_kernels(n_head, n_kv_head, head_dim, page_size)
    kinds = ([False] if scalar else []) + ([True] if tensor else [])
    assert kinds
    for tensor_cores in kinds + kinds:                # each kernel twice over the same scratch
        out = torch.full_like(q, float("nan"))
        ops.decode_attention(q, cache, positions, table, out, partial, counters, S, n_head, n_kv_head, head_dim, page_size, scale, window, splits,
                             tensor_cores=tensor_cores, sink=s)
        assert (out.double().cpu() - ref).abs().max().item() < 1.5e-2, f"tensor_cores={tensor_cores}"
        assert int(counters.abs().sum()) == 0


@pytest.mark.parametrize("n_head,n_kv_head,head_dim,page_size,window", [
    (12, 12, 64, 16, 0), (4, 4, 16, 16, 0), (6, 2, 48, 32, 0), (5, 1, 64, 64, 0), (12, 3, 128, 16, 88), (4, 4, 32, 16, 40), (2, 1, 64, 32, 7), (3, 3, 64, 16, 100),
    (6, 3, 64, 64, 75)])
def test_prefill_attention_with_sinks(dev, n_head, n_kv_head, head_dim, page_size, window):
    """Prompt portions of every kind in one launch on both tensor-core kernels: a whole prompt, a portion that continues a long context,
    single tokens, two-token portions, portions that end inside a page and a tile."""
    from liyab_b200 import ops
    lens = [1, 37, 130, 64, 300, 2, 129, 1024]
    q_lens = [1, 37, 2, 1, 45, 2, 65, 200]
    scale = 0.9 / math.sqrt(head_dim)
    q, cache, tok_seq, positions, table, refs = _paged_case(dev, torch.bfloat16, n_head, n_kv_head, head_dim, page_size, lens, q_lens,
                                                            seed=head_dim + n_head + window)
    q_start = torch.tensor(np.concatenate([[0], np.cumsum(q_lens)]), dtype=torch.int32, device=dev)
    n_past = torch.tensor([l - ql for l, ql in zip(lens, q_lens)], dtype=torch.int32, device=dev)
    s, s64 = sinks(n_head, window + 1, dev)
    ref = reference_attention(refs, n_head, n_kv_head, scale, window, s64)
    assert (ref - reference_attention(refs, n_head, n_kv_head, scale, window, s64 * 0 - 1e30)).abs().max().item() > 0.05
    kinds = [False] + ([True] if ops.prefill_attention_tc_supports(n_head, n_kv_head, head_dim, page_size) else [])
    for tcgen05 in kinds:
        out = torch.full_like(q, float("nan"))
        ops.prefill_attention(q, cache, q_start, n_past, table, out, len(lens), max(q_lens), n_head, n_kv_head, head_dim, page_size, scale, window,
                              tcgen05=tcgen05, sink=s)
        assert ops.device_status() == 0
        err = (out.double().cpu() - ref).abs().max().item()
        assert err < 1.5e-2, (tcgen05, err)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,D,E,rot,norm_mode,blend", [(4, 2, 12, 10, 8, 2, "blend"), (6, 2, 128, 40, 96, 2, "source"), (3, 3, 8, 8, 8, 1, None), (2, 1, 6, 9, 0, 2, "blend"),
                                                        (1, 1, 2, 1, 2, 0, None), (5, 5, 16, 4, 4, 2, None)])
def test_queries_keys_and_values_on_their_way_to_the_cache(dev, dtype, H, G, D, E, rot, norm_mode, blend):
    """Norm over the whole projection (or a head, or none), rotation of part of a head at far positions, values blended or left for later
    layers, heads padded with zeros, pages in scrambled order, a negative slot that writes nothing."""
    from liyab_b200 import ops
    rng = np.random.default_rng(H * 100 + D)
    T, page, eps = 23, 16, 1e-5
    P = max(16, 1 << (max(D, E) - 1).bit_length()) if dtype == torch.bfloat16 else (max(D, E) + 3) // 4 * 4
    cols = H * D + G * D + G * E + 5
    proj = rng.standard_normal((T, cols))
    qw, kw = rng.uniform(0.5, 1.5, H * D if norm_mode == 2 else D), rng.uniform(0.5, 1.5, G * D if norm_mode == 2 else D)
    positions = rng.integers(0, 5000, T)
    freq = 700.0 ** (-2.0 * np.arange(rot // 2) / max(rot, 1))
    slots = rng.permutation(4 * page)[:T]
    slots[3] = -1
    lam = 0.37
    first = rng.standard_normal((T, G * E))

    def normed(x, w, heads):
        x = x.reshape(T, heads, D)
        if norm_mode == 1:
            return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * w
        if norm_mode == 2:
            flat = x.reshape(T, -1)
            return (flat / np.sqrt((flat * flat).mean(-1, keepdims=True) + eps) * w).reshape(T, heads, D)
        return x

    def rotated(x):
        ang = positions[:, None].astype(np.float64) * freq.astype(np.float32).astype(np.float64)[None, :]
        c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
        out = x.copy()
        a, b = x[..., :rot // 2], x[..., rot // 2:rot]
        out[..., :rot // 2], out[..., rot // 2:rot] = a * c - b * s, b * c + a * s
        return out

    q_ref = rotated(normed(proj[:, :H * D].copy(), qw, H))
    k_ref = rotated(normed(proj[:, H * D:H * D + G * D].copy(), kw, G))
    v_own = proj[:, H * D + G * D:H * D + G * D + G * E]
    v_ref = ((1 - lam) * v_own + lam * first if blend == "blend" else v_own).reshape(T, G, E)

    t = lambda a, ty=torch.float32: torch.tensor(np.asarray(a), dtype=ty, device=dev)
    q_out = torch.full((T, H * P), float("nan"), dtype=dtype, device=dev)
    cache = torch.full((4, 2, G, page, P), float("nan"), dtype=dtype, device=dev)
    shared = t(first) if blend == "blend" else torch.full((T, G * E), float("nan"), device=dev)
    ops.qkv_rotary_store(t(proj), 0, H * D, H * D + G * D, t(qw) if norm_mode else None, t(kw) if norm_mode else None, q_out, cache, t(slots, torch.int32), H, G, D, E, P, page,
                         norm_mode, eps, t(positions, torch.int32), t(freq) if rot else None, rot, v_first_in=shared if blend == "blend" else None,
                         v_first_out=shared if blend == "source" else None, blend=t([lam]) if blend == "blend" else None)
    tol = 2e-4 if dtype == torch.float32 else 2e-2            # angles of thousands of radians in 32-bit
    got_q = q_out.double().cpu().numpy().reshape(T, H, P)
    assert np.abs(got_q[..., :D] - q_ref).max() < tol * max(1.0, np.abs(q_ref).max()) and (got_q[..., D:] == 0).all()
    c = cache.double().cpu().numpy()
    for i in range(T):
        pg, off = divmod(int(slots[i]), page)
        if slots[i] < 0:
            continue
        assert np.abs(c[pg, 0, :, off, :D] - k_ref[i]).max() < tol * max(1.0, np.abs(k_ref).max()) and (c[pg, 0, :, off, D:] == 0).all()
        assert np.abs(c[pg, 1, :, off, :E] - v_ref[i]).max() < tol * max(1.0, np.abs(v_ref).max()) and (c[pg, 1, :, off, E:] == 0).all()
    assert np.isnan(c).sum() == (4 * page - (T - 1)) * 2 * G * P         # the token without a slot, and nothing else, left its place untouched
    if blend == "source":
        assert np.abs(shared.double().cpu().numpy() - v_own).max() < 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,gate", [(320, "sigmoid"), (60, "sigmoid"), (1, "silu"), (2050, "sigmoid"), (165, "silu"), (2048, "silu"), (768, "sigmoid")])
def test_norm_over_all_heads_with_a_gate(dev, dtype, width, gate):
    """Rows that split into 16-byte pieces (a warp a row) and rows that do not (a block a row), with and without gains and gates."""
    from liyab_b200 import ops
    rng = np.random.default_rng(width)
    eps = 1e-5
    t = lambda a: torch.tensor(a, dtype=torch.float32, device=dev)
    for pad, T in ((3, 9), (4, 9), (4, 70)):
        o, g, w = rng.standard_normal((T, width + pad)) * 3.0, rng.standard_normal((T, width)), rng.uniform(0.5, 1.5, width)
        sig = 1.0 / (1.0 + np.exp(-g))
        x = o[:, :width]
        ref = x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * w * (sig if gate == "sigmoid" else g * sig)
        out = torch.empty(T, width, dtype=dtype, device=dev)
        ops.row_norm_gate(t(o)[:, :width], t(g), t(w), out, gate, eps)
        assert np.abs(out.double().cpu().numpy() - ref).max() < (1e-5 if dtype == torch.float32 else 1.5e-2) * max(1.0, np.abs(ref).max())
        ops.row_norm_gate(t(o)[:, :width], None, None, out, gate, eps)
        ref = x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)
        assert np.abs(out.double().cpu().numpy() - ref).max() < (1e-5 if dtype == torch.float32 else 1.5e-2) * max(1.0, np.abs(ref).max())


@pytest.mark.parametrize("width,rows", [(160, 8), (768, 300), (100, 5), (98, 3), (2048, 9), (4100, 2), (4, 1)])
def test_sublayer_output_normed_and_added_to_the_stream(dev, width, rows):
    """x += m y / rms(y) * w, with the new rows also rounded for the part that reads the stream next: widths that take the warp-a-row form
    and ones that do not (no multiple of four, more than 2048 values), rows that start off 16 bytes, one row and hundreds."""
    from liyab_b200 import ops
    rng = np.random.default_rng(width + rows)
    x, y, w = rng.standard_normal((rows, width + 4)), rng.standard_normal((rows, width)) * 2.0, rng.uniform(0.5, 1.5, width)
    eps, m = 1e-5, 0.7
    ref = x[:, :width] + m * y / np.sqrt((y * y).mean(-1, keepdims=True) + eps) * w
    t = lambda a: torch.tensor(a, dtype=torch.float32, device=dev)
    for offset in (0, 1):          # rows that start on 16 bytes, and ones that do not
        xs = t(x)[:, offset:offset + width] if offset else t(x)[:, :width]
        want = ref if not offset else x[:, offset:offset + width] + (ref - x[:, :width])
        rounded = torch.full((rows, width), float("nan"), dtype=torch.bfloat16, device=dev)
        ops.rms_sum_add(xs, [t(y)], [t(w)], m, eps, rounded=rounded)
        assert np.abs(xs.double().cpu().numpy() - want).max() < 1e-5 * max(1.0, np.abs(want).max())
        assert (rounded.float() == xs.to(torch.bfloat16).float()).all()
        xs = t(x)[:, :width]
        ops.rms_sum_add(xs, [t(y)], [None], m, eps)
        assert np.abs(xs.double().cpu().numpy() - (x[:, :width] + m * y / np.sqrt((y * y).mean(-1, keepdims=True) + eps))).max() < 1e-5 * max(1.0, np.abs(ref).max())


@pytest.mark.parametrize("H,D,E,tile,act", [(3, 12, 20, 20, "silu"), (2, 32, 64, 32, "silu"), (1, 1, 1, 1, "sigmoid"), (4, 8, 33, 17, "silu"), (2, 64, 16, 16, "relu"), (2, 8, 5, 4, "sigmoid")])
def test_memory_with_activated_queries_keys_and_values(dev, H, D, E, tile, act):
    """S = g S + act(k) act(v)^T, o = S^T act(q) in all three forms of the recurrence (row by row, in pieces, a block a piece) from the same state:
    three requests of unequal length in scrambled slots, value tiles that do not divide the head (padded columns must stay out of it)."""
    from liyab_b200 import ops
    rng = np.random.default_rng(H * 10 + D)
    lens = [150, 1, 37]
    T = sum(lens)
    cols = 2 * H * D + H * E + 3
    proj = rng.standard_normal((T, cols))
    decay = rng.uniform(0.8, 0.999, H)
    f = {"silu": lambda z: z / (1 + np.exp(-z)), "sigmoid": lambda z: 1 / (1 + np.exp(-z)), "relu": lambda z: np.maximum(z, 0)}[act]
    q, k, v = (f(proj[:, :H * D]).reshape(T, H, D), f(proj[:, H * D:2 * H * D]).reshape(T, H, D), f(proj[:, 2 * H * D:2 * H * D + H * E]).reshape(T, H, E))
    ref = np.zeros((T, H, E))
    at = 0
    for n in lens:
        S = np.zeros((H, D, E))
        for t in range(at, at + n):
            S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
            ref[t] = np.einsum("hde,hd->he", S, q[t])
        at += n
    t32 = lambda a, ty=torch.float32: torch.tensor(np.asarray(a), dtype=ty, device=dev)
    q_start = t32(np.concatenate([[0], np.cumsum(lens)]), torch.int32)
    slots = t32([2, 0, 3], torch.int32)
    positions = t32(np.concatenate([np.arange(n) for n in lens]), torch.int32)
    floats = ops.memory_slot_floats(H, D, E, tile)
    outs = []
    for form in ("rows", "pieces", "blocks"):
        state = torch.zeros(4, floats, device=dev)
        out = torch.full((T, H * E), float("nan"), device=dev)
        if form == "blocks":
            ops.matrix_memory_pieces(t32(proj), 0, H * D, 2 * H * D, None, None, t32(decay), None, 0, positions, q_start, slots, state, out, H, D, E, tile, 1.0, 1.0, 0.0,
                                     qkv_act=act)
        else:
            ops.matrix_memory(t32(proj), 0, H * D, 2 * H * D, None, None, t32(decay), None, 0, positions, q_start, slots, state, out, H, D, E, tile, 1.0, 1.0, 0.0,
                              form == "pieces", qkv_act=act)
        got = out.double().cpu().numpy().reshape(T, H, E)
        assert np.abs(got - ref).max() < 2e-4 * max(1.0, np.abs(ref).max()), form
        outs.append((got, state.double().cpu().numpy()))
    for got, state in outs[1:]:          # the forms leave the same state behind
        assert np.abs(state - outs[0][1]).max() < 2e-4 * max(1.0, np.abs(outs[0][1]).max())


def test_activation_over_some_columns(dev):
    from liyab_b200 import ops
    rng = np.random.default_rng(3)
    for width, cols in ((50, 31), (64, 32), (2400, 2304)):       # rows in single floats, and in 16-byte pieces
        x = rng.standard_normal((37, width)) * 3.0
        for gate, f in (("silu", lambda z: z / (1 + np.exp(-z))), ("sigmoid", lambda z: 1 / (1 + np.exp(-z))), ("relu", lambda z: np.maximum(z, 0))):
            y = ops.activate_columns(torch.tensor(x, dtype=torch.float32, device=dev), cols, gate).double().cpu().numpy()
            assert np.abs(y[:, :cols] - f(x[:, :cols])).max() < 2e-6 and np.abs(y[:, cols:] - x[:, cols:]).max() < 1e-6      # float32 holds x to 1e-7


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("m,n,k", [(3, 96, 64), (16, 320, 160), (70, 200, 128), (300, 3072, 768)])
def test_square_of_relu_in_every_product(dev, dtype, m, n, k):
    """The chosen product kernel for few rows, dozens and hundreds (32-bit units, mma.sync rows, tcgen05 one tile and persistent)."""
    from liyab_b200 import ops
    rng = np.random.default_rng(m + n)
    a = torch.tensor(rng.standard_normal((m, k)), dtype=dtype, device=dev)
    w = torch.tensor(rng.standard_normal((n, k)) * k ** -0.5, dtype=dtype, device=dev)
    ref = torch.clamp(a.double() @ w.double().t(), min=0) ** 2
    out = torch.empty(m, n, dtype=dtype, device=dev)
    ops.linear(a, w, None, out, m, "relu2")
    assert ops.device_status() == 0
    assert (out.double() - ref).abs().max().item() < (1e-4 if dtype == torch.float32 else 3e-2) * max(1.0, ref.abs().max().item())


def test_experts_by_token_id(dev):
    from liyab_b200 import ops
    rng = np.random.default_rng(4)
    vocab, X, top = 50, 7, 3
    table = np.stack([rng.permutation(X)[:top] for _ in range(vocab)]).astype(np.int32)
    tokens = rng.integers(0, vocab, 41).astype(np.int32)
    ids, weights = ops.router_table(torch.tensor(tokens, device=dev), torch.tensor(table, device=dev), X)
    assert (ids.cpu().numpy() == table[tokens]).all() and (weights.cpu().numpy() == np.float32(1.0 / top)).all()
