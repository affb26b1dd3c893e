"""The kernels that came with Viresun, each by itself against a float64 statement written here: the penalty by distance in every
attention kernel (32-bit, scalar decode with split keys, mma.sync prefill, tcgen05 prefill), the sinusoid of the position with the
norm behind it, the gated norm in groups with a skip, the gates with a cap, the router with a bias, the convolution and step of the
state space with its state across cuts, and the recurrence with a factor a token and keys shared by a group's heads in its three forms."""
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


def reference_attention(refs, n_head, n_kv_head, scale, window, r1, r2):
    """softmax_j(q_i . k_j scale - r1_h ln(1 + r2_h (i - j))) v_j over the keys j with 0 <= i - j < window (all earlier keys without one)."""
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
        dist = (pos - j).clamp(min=0).double()
        for h in range(n_head):
            s = (q[:, h] @ k[:, h // group].t()) * scale - r1[h] * torch.log1p(r2[h] * dist)
            o[:, h] = torch.softmax(s.masked_fill(~mask, float("-inf")), dim=-1) @ v[:, h // group]
        outs.append(o.reshape(Q, -1))
    return torch.cat(outs)


def pairs(n_head, seed, dev):
    rng = np.random.default_rng(seed)
    r1, r2 = rng.uniform(0.0, 3.0, n_head), rng.uniform(0.02, 0.6, n_head)
    r1[0] = 0.0                                     # a head without a penalty beside heads with one
    d = torch.tensor(np.concatenate([r1, r2]), dtype=torch.float32, device=dev)
    return d, d[:n_head].double().cpu(), d[n_head:].double().cpu()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_head,n_kv_head,head_dim,page_size,window", [(4, 4, 16, 16, 0), (6, 2, 48, 32, 0), (5, 1, 64, 64, 70), (4, 2, 24, 16, 33), (2, 1, 64, 32, 7)])
def test_generic_attention_with_a_penalty_by_distance(dev, dtype, n_head, n_kv_head, head_dim, page_size, window):
    from liyab_b200 import ops
    lens, q_lens = [1, 37, 130, 64, 300], [1, 37, 2, 1, 45]
    scale = 0.9 / math.sqrt(head_dim)
    q, cache, tok_seq, positions, table, refs = _paged_case(dev, dtype, n_head, n_kv_head, head_dim, page_size, lens, q_lens, seed=head_dim + n_head)
    d, r1, r2 = pairs(n_head, head_dim, dev)
    ref = reference_attention(refs, n_head, n_kv_head, scale, window, r1, r2)
    plain_ref = reference_attention(refs, n_head, n_kv_head, scale, window, r1 * 0, r2)
    assert (ref - plain_ref).abs().max().item() > 0.05, "the penalty does not show"
    out = torch.empty_like(q)
    ops.paged_attention_generic(q, cache, tok_seq, positions, table, out, q.shape[0], n_head, n_kv_head, head_dim, page_size, scale, window, distance=d)
    assert (out.double().cpu() - ref).abs().max().item() < (2e-5 if dtype == torch.float32 else 1.5e-2)
    # Without the pairs the kernel is the one it was.
    ops.paged_attention_generic(q, cache, tok_seq, positions, table, out, q.shape[0], n_head, n_kv_head, head_dim, page_size, scale, window)
    assert (out.double().cpu() - plain_ref).abs().max().item() < (2e-5 if dtype == torch.float32 else 1.5e-2)


@pytest.mark.parametrize("n_head,n_kv_head,head_dim,page_size,window,splits", [
    (12, 12, 64, 16, 0, 1), (12, 12, 64, 16, 0, 5), (4, 4, 16, 16, 0, 3), (8, 2, 128, 16, 0, 4), (16, 2, 64, 64, 0, 7), (6, 3, 64, 16, 33, 4),
    (4, 4, 32, 16, 5, 16), (5, 5, 128, 32, 70, 2), (2, 1, 256, 16, 200, 9), (32, 2, 64, 16, 0, 3), (16, 1, 128, 16, 0, 8), (12, 3, 64, 16, 300, 12)])
def test_decode_attention_with_a_penalty_by_distance(dev, n_head, n_kv_head, head_dim, page_size, window, splits):
    """One new token per request, keys split several ways: a range's distances count from the query, not from the range's start."""
    from liyab_b200 import ops
    lens = [1, 2, 17, 64, 65, 300, 1024, 33]
    scale = 0.9 / math.sqrt(head_dim)
    q, cache, tok_seq, positions, table, refs = _paged_case(dev, torch.bfloat16, n_head, n_kv_head, head_dim, page_size, lens, [1] * len(lens),
                                                            seed=7 * head_dim + splits)
    S = len(lens)
    d, r1, r2 = pairs(n_head, splits, dev)
    ref = reference_attention(refs, n_head, n_kv_head, scale, window, r1, r2)
    assert (ref - reference_attention(refs, n_head, n_kv_head, scale, window, r1 * 0, r2)).abs().max().item() > 0.05
    partial = torch.full((S * n_head * splits * (head_dim + 2),), float("nan"), device=dev)
    counters = torch.zeros(S * n_kv_head, dtype=torch.int32, device=dev)
    scalar, tensor = ops.decode_attention_kernels(n_head, n_kv_head, head_dim, page_size)
    kinds = ([False] if scalar else []) + ([True] if tensor else [])
    assert kinds
    for tensor_cores in kinds + kinds:                # each kernel twice over the same scratch
        out = torch.full_like(q, float("nan"))
        ops.decode_attention(q, cache, positions, table, out, partial, counters, S, n_head, n_kv_head, head_dim, page_size, scale, window, splits,
                             tensor_cores=tensor_cores, distance=d)
        assert (out.double().cpu() - ref).abs().max().item() < 1.5e-2, f"tensor_cores={tensor_cores}"
        assert int(counters.abs().sum()) == 0


@pytest.mark.parametrize("n_head,n_kv_head,head_dim,page_size,window", [
    (12, 12, 64, 16, 0), (4, 4, 16, 16, 0), (6, 2, 48, 32, 0), (5, 1, 64, 64, 0), (2, 2, 128, 16, 0), (4, 4, 32, 16, 40), (2, 1, 64, 32, 7), (3, 3, 64, 16, 100),
    (6, 3, 64, 64, 75)])
def test_prefill_attention_with_a_penalty_by_distance(dev, n_head, n_kv_head, head_dim, page_size, window):
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
    d, r1, r2 = pairs(n_head, window + 1, dev)
    ref = reference_attention(refs, n_head, n_kv_head, scale, window, r1, r2)
    assert (ref - reference_attention(refs, n_head, n_kv_head, scale, window, r1 * 0, r2)).abs().max().item() > 0.05
    kinds = [False] + ([True] if ops.prefill_attention_tc_supports(n_head, n_kv_head, head_dim, page_size) else [])
    for tcgen05 in kinds:
        out = torch.full_like(q, float("nan"))
        ops.prefill_attention(q, cache, q_start, n_past, table, out, len(lens), max(q_lens), n_head, n_kv_head, head_dim, page_size, scale, window,
                              tcgen05=tcgen05, distance=d)
        assert ops.device_status() == 0
        err = (out.double().cpu() - ref).abs().max().item()
        assert err < 1.5e-2, (tcgen05, err)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,base,gain", [(48, 10000.0, True), (100, 500.0, True), (33, 10000.0, True), (256, 1e6, False), (2050, 10000.0, True)])
def test_sinusoid_of_the_position(dev, dtype, width, base, gain):
    """Far positions as exactly as near ones (the angle in 32-bit from a frequency held as two floats), odd widths, the norm behind it."""
    from liyab_b200 import ops
    rng = np.random.default_rng(width)
    vocab, eps = 50, 1e-5
    table = torch.from_numpy(rng.standard_normal((vocab, width))).to(dtype).to(dev)
    positions = np.array([0, 1, 2, 63, 64, 1000, 4095, 50000, 100001, 7], dtype=np.int32)
    tokens = rng.integers(0, vocab, size=len(positions)).astype(np.int32)
    g = torch.from_numpy(rng.normal(1.0, 0.2, size=width)).float().to(dev) if gain else None
    x = torch.full((len(positions), width), float("nan"), dtype=torch.float32, device=dev)
    ops.embed_sinusoid(torch.from_numpy(tokens).to(dev), torch.from_numpy(positions).to(dev), table, base, g, x, 1.0, eps)
    i = np.arange((width + 1) // 2)
    ang = positions[:, None].astype(np.float64) * (base ** (-2.0 * i / width))[None, :]
    e = np.zeros((len(positions), 2 * len(i)))
    e[:, 0::2], e[:, 1::2] = np.sin(ang), np.cos(ang)
    want = table.double().cpu().numpy()[tokens] + e[:, :width]
    if gain:
        want = want / np.sqrt((want ** 2).mean(axis=1, keepdims=True) + eps) * g.double().cpu().numpy()[None, :]
    # The angle's rounding is carried along (p w = a + r with both parts kept), so position 100,001 is as exact as position 1.
    assert np.abs(x.double().cpu().numpy() - want).max() < 2e-5 * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_head,vdim,groups,skip,gate,weight", [(4, 12, 2, True, True, True), (3, 24, 1, True, True, True), (6, 8, 3, False, True, False),
                                                                  (2, 70, 5, True, False, True), (1, 1, 1, True, True, True), (8, 64, 8, True, True, True)])
def test_gated_norm_in_groups(dev, out_dtype, n_head, vdim, groups, skip, gate, weight):
    """(o + D_h x) silu(z), each of `groups` equal parts over its own root mean square, times a gain: the gate before the norm."""
    from liyab_b200 import ops
    rng = np.random.default_rng(n_head * vdim)
    T, width, eps = 37, n_head * vdim, 1e-5
    o, x, z = (torch.from_numpy(rng.standard_normal((T, width))).float().to(dev) for _ in range(3))
    D = torch.from_numpy(rng.normal(0.8, 0.3, n_head)).float().to(dev)
    w = torch.from_numpy(rng.normal(1.0, 0.2, width)).float().to(dev)
    out = torch.full((T, width), float("nan"), dtype=out_dtype, device=dev)
    ops.gated_group_norm(o, x if skip else None, D if skip else None, vdim, z if gate else None, w if weight else None, out, groups, eps)
    y = o.double()
    if skip:
        y = y + D.double().repeat_interleave(vdim)[None, :] * x.double()
    if gate:
        y = y * (z.double() * torch.sigmoid(z.double()))
    parts = y.reshape(T, groups, width // groups)
    y = (parts / torch.sqrt((parts ** 2).mean(dim=-1, keepdim=True) + eps)).reshape(T, width)
    if weight:
        y = y * w.double()[None, :]
    err = (out.double() - y).abs().max().item() / y.abs().max().item()
    assert err < (1e-5 if out_dtype == torch.float32 else 6e-3)
    # The norm before the gate is another function: the test's inputs tell them apart.
    if gate and groups < width:
        other = o.double() + (D.double().repeat_interleave(vdim)[None, :] * x.double() if skip else 0)
        parts = other.reshape(T, groups, width // groups)
        other = (parts / torch.sqrt((parts ** 2).mean(dim=-1, keepdim=True) + eps)).reshape(T, width) * (z.double() * torch.sigmoid(z.double()))
        assert ((other * (w.double()[None, :] if weight else 1)) - y).abs().max().item() > 0.1


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_gates_with_a_cap_and_relu(dev, out_dtype):
    from liyab_b200 import ops
    rng = np.random.default_rng(3)
    T, inner, alpha, limit = 29, 50, 1.702, 1.25
    gu = torch.from_numpy(rng.standard_normal((T, 2 * inner)) * 2.0).float().to(dev)
    g, u = gu[:, :inner].double(), gu[:, inner:].double()
    assert (g > limit).any() and (u > limit).any() and (u < -limit).any() and (g < -limit).any()
    out = torch.empty((T, inner), dtype=out_dtype, device=dev)
    tol = 1e-6 if out_dtype == torch.float32 else 8e-3
    ops.gated_act_kind(gu, out, "capped", alpha, limit)
    gc, uc = g.clamp(max=limit), u.clamp(-limit, limit)
    want = gc * torch.sigmoid(alpha * gc) * (uc + 1.0)
    assert ((out.double() - want).abs() <= tol * (1 + want.abs())).all()
    ops.gated_act_kind(gu, out, "relu")
    want = g.clamp(min=0) * u
    assert ((out.double() - want).abs() <= tol * (1 + want.abs())).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts,top,width", [(12, 2, 96), (5, 5, 100), (1, 1, 48), (64, 6, 256), (7, 1, 33)])
def test_router_with_a_bias(dev, dtype, experts, top, width):
    """The largest `top` of W h + b (the bias decides which), their weights the softmax over the chosen logits only."""
    from liyab_b200 import ops
    rng = np.random.default_rng(experts * top)
    T = 41
    h = torch.from_numpy(rng.standard_normal((T, width))).to(dtype).to(dev)
    router = torch.from_numpy(rng.standard_normal((experts, width)) * 3.0 / math.sqrt(width)).to(dtype).to(dev)
    bias = torch.from_numpy(rng.normal(0.0, 2.0, experts)).float().to(dev)
    ids, weights = ops.router_topk(h, router, bias, top, True, True)
    z = h.double() @ router.double().t() + bias.double()[None, :]
    order = torch.argsort(-z, dim=1, stable=True)[:, :top]
    assert torch.equal(ids.long().cpu(), order.cpu())
    chosen = torch.gather(z, 1, order)
    want = torch.softmax(chosen, dim=1)
    assert (weights.double() - want).abs().max().item() < 2e-5
    if experts > top:
        without = torch.argsort(-(z - bias.double()[None, :]), dim=1, stable=True)[:, :top]
        assert not torch.equal(without, order), "the bias does not show"


def _t(a, dev, dtype=torch.float32):
    return torch.tensor(np.ascontiguousarray(a), dtype=dtype, device=dev)


@pytest.mark.parametrize("H,E,G,N,K,biases", [(4, 8, 2, 6, 4, True), (3, 5, 1, 7, 3, True), (2, 16, 2, 8, 1, False), (6, 4, 3, 2, 5, True),
                                              (1, 1, 1, 1, 2, False), (8, 32, 2, 64, 4, True), (4, 12, 4, 10, 2, True)])
def test_convolution_step_and_the_rows_of_the_recurrence(dev, H, E, G, N, K, biases):
    """Three requests of unequal length in steps cut anywhere (portions, then single tokens in steps of their own), through scrambled state
    slots: the convolution over the last K inputs with zeros before a sequence's start, SiLU, softplus of the step, and the rows
    [x | B | C | dt x | -exp(A) dt], against the same made from each whole sequence in float64.  Sizes with channel counts that are and are not
    multiples of four, and K = 4 beside other K."""
    from liyab_b200 import ops
    rng = np.random.default_rng(100 * H + K)
    inner, GN2 = H * E, 2 * G * N
    channels = inner + GN2
    cols = inner + channels + H                     # [z | x B C | dt]
    lens = [23, 9, 1]
    cuts = [[5, 6, 19, 20, 21, 22, 23], [2, 9], [1]]
    seqs = [rng.normal(0, 1.0, size=(n, cols)) for n in lens]
    taps, tap_bias = rng.normal(0, K ** -0.5, size=(channels, K)), rng.normal(0, 0.3, size=channels) if biases else None
    dt_bias, a_log = (rng.normal(-1.0, 0.8, size=H) if biases else None), rng.normal(-1.0, 1.0, size=H)

    def whole(u):
        xbc = u[:, inner:inner + channels]
        padded = np.concatenate([np.zeros((K - 1, channels)), xbc])
        conv = sum(padded[j:j + len(u)] * taps[:, j] for j in range(K)) + (tap_bias if biases else 0.0)
        act = conv / (1.0 + np.exp(-conv))
        dt = np.logaddexp(0.0, u[:, inner + channels:] + (dt_bias if biases else 0.0))
        return np.concatenate([act, act[:, :inner] * np.repeat(dt, E, axis=1), -np.exp(a_log) * dt], axis=1)

    want = [whole(u) for u in seqs]
    slots = [2, 0, 3]
    state = torch.zeros(4, max(1, (K - 1) * channels), dtype=torch.float32, device=dev)
    at = [0, 0, 0]
    for step in range(max(len(c) for c in cuts)):
        live = [r for r in range(3) if step < len(cuts[r])]
        parts = [seqs[r][at[r]:cuts[r][step]] for r in live]
        q_start = np.concatenate([[0], np.cumsum([len(p) for p in parts])]).astype(np.int32)
        tok_seq = np.concatenate([np.full(len(p), i) for i, p in enumerate(parts)]).astype(np.int32)
        proj = _t(np.concatenate(parts), dev)
        out = torch.full((proj.shape[0], 2 * inner + GN2 + H), float("nan"), dtype=torch.float32, device=dev)
        ops.ssm_prepare(proj, inner, inner + channels, _t(taps, dev), _t(tap_bias, dev) if biases else None, _t(dt_bias, dev) if biases else None,
                        _t(a_log, dev), state, _t(tok_seq, dev, torch.int32), _t(q_start, dev, torch.int32),
                        _t(np.array([slots[r] for r in live]), dev, torch.int32), out, H, E, GN2, all(len(p) == 1 for p in parts))
        ref = np.concatenate([want[r][at[r]:cuts[r][step]] for r in live])
        err = np.abs(out.double().cpu().numpy() - ref).max() / np.abs(ref).max()
        assert err < 2e-6, f"step {step}: {err:.2e}"
        for r in live:
            at[r] = cuts[r][step]
    assert float(state[1].abs().max()) == 0.0                  # the slot no request used
    if K > 1:                                                   # a request's state is its last K - 1 inputs, oldest first
        last = np.concatenate([np.zeros((K - 1, channels)), seqs[0][:, inner:inner + channels]])[-(K - 1):]
        assert np.abs(state[2].double().cpu().numpy().reshape(K - 1, channels) - last).max() < 1e-6


@pytest.mark.parametrize("H,G,N,E,tile", [(4, 2, 16, 24, 24), (6, 1, 10, 70, 24), (2, 2, 64, 64, 32), (3, 3, 6, 5, 5), (8, 2, 128, 64, 32), (1, 1, 1, 1, 1)])
def test_recurrence_with_a_factor_a_token_and_shared_keys(dev, H, G, N, E, tile):
    """S_t = exp(f_t) S_{t-1} + k_t v_t^T, o_t = S_t^T q_t with f <= 0 a number a token and head, heads of a group reading one key and query
    row: three requests in steps cut anywhere, every step row by row, in pieces and with a block per piece from the same state, against
    the recurrence in float64.  One head forgets almost nothing, one almost everything."""
    from liyab_b200 import ops
    rng = np.random.default_rng(11 * H + N)
    lens, cuts = [150, 33, 1], [[40, 41, 150], [2, 33], [1]]
    share = H // G
    cols = 2 * G * N + H * E + H                    # [q | k | v | f]
    rows = []
    for n in lens:
        x = rng.normal(0, 1.0, size=(n, cols))
        x[:, -H:] = -np.abs(rng.normal(0, 0.5, size=(n, H)))
        x[:, -H] *= 1e-3
        if H > 1:
            x[:, -1] -= 6.0
        rows.append(x)
    floats = ops.memory_slot_floats(H, N, E, tile)
    modes = (False, True, "pieces")
    states = {m: torch.zeros(4, floats, dtype=torch.float32, device=dev) for m in modes}
    S = {(r, h): np.zeros((N, E)) for r in range(3) for h in range(H)}
    slots, at = [2, 0, 3], [0, 0, 0]
    for step in range(3):
        live = [r for r in range(3) if step < len(cuts[r])]
        parts = [rows[r][at[r]:cuts[r][step]] for r in live]
        q_start = np.concatenate([[0], np.cumsum([len(p) for p in parts])]).astype(np.int32)
        pos = np.concatenate([np.arange(at[r], cuts[r][step]) for r in live]).astype(np.int32)
        want = np.zeros((int(q_start[-1]), H * E))
        for i, r in enumerate(live):
            for h in range(H):
                g = h // share
                for t, x in enumerate(parts[i]):
                    q, k = x[g * N:(g + 1) * N], x[G * N + g * N:G * N + (g + 1) * N]
                    v = x[2 * G * N + h * E:2 * G * N + (h + 1) * E]
                    S[(r, h)] = math.exp(x[2 * G * N + H * E + h]) * S[(r, h)] + np.outer(k, v)
                    want[q_start[i] + t, h * E:(h + 1) * E] = S[(r, h)].T @ q
        proj = _t(np.concatenate(parts), dev)
        for mode in modes:
            out = torch.full((proj.shape[0], H * E), float("nan"), dtype=torch.float32, device=dev)
            args = (proj, 0, G * N, 2 * G * N, None, 2 * G * N + H * E, None, None, 0, _t(pos, dev, torch.int32), _t(q_start, dev, torch.int32),
                    _t(np.array([slots[r] for r in live]), dev, torch.int32), states[mode], out, H, N, E, tile, 1.0, 1.0, 0.0)
            if mode == "pieces":
                ops.matrix_memory_pieces(*args, qk_share=share)
            else:
                ops.matrix_memory(*args, mode, qk_share=share)
            err = np.abs(out.double().cpu().numpy() - want).max() / max(np.abs(want).max(), 1e-30)
            assert err < 5e-5, f"step {step}, {mode}: {err:.2e}"
        for r in live:
            at[r] = cuts[r][step]
    for other in (True, "pieces"):
        assert float((states[False] - states[other]).abs().max()) <= 1e-3 * float(states[False].abs().max())
    assert float(states[False][1].abs().max()) == 0.0
