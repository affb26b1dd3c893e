"""The kernels that came with Viresun, each by itself against a float64 statement written here: the penalty by distance in every
attention kernel (32-bit, scalar decode with split keys, mma.sync prefill, tcgen05 prefill), the sinusoid of the position with the
norm behind it, the gated norm in groups with a skip, the gates with a cap, and the router with a bias."""
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
