"""Viresun in the engine against the plain implementation (plain_viresun.py): every mechanism by itself through the parts' taps,
then whole prompts, token-by-token decoding, portions down to two tokens, mixed batches with pages and state slots used again, keys
at the windows' edges and at page borders, states that reach far back, the first tokens of a sequence, long decoding, and greedy
generation through the engine's own entry point and scheduler."""
from __future__ import annotations

import copy
import os
import subprocess

import numpy as np
import pytest

import plain_viresun as plain
import trace_tools as tt
from viresun_models import CONFIGS, attention, dense, layer, model_folder, moe, random_weights, state_space, write_model

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# float32: largest |engine - plain| on a logit as a fraction of the largest |logit| of the sequence.
REL_TOL = 1e-4
LENGTHS = {"A": [150, 70, 33, 21, 7, 2, 1, 45], "B": [140, 72, 64, 1, 2, 97, 40], "C": [120, 47, 2, 64, 1, 33], "D": [100, 33, 32, 31, 2, 65]}


def tokens_of(name, i, n):
    config, seed = CONFIGS[name]
    return np.random.default_rng(1000 * seed + i).integers(0, config["vocab"], size=n).astype(int).tolist()


def request_set(name):
    return {f"r{i}": tokens_of(name, i, n) for i, n in enumerate(LENGTHS[name])}


def f64(weights):
    return {k: np.asarray(v, dtype=np.float64) for k, v in weights.items()}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    base = str(tmp_path_factory.mktemp("viresun"))
    out = {}
    for name in CONFIGS:
        path, config, weights = model_folder(base, name)
        out[name] = (path, config, f64(weights))
    return out


@pytest.fixture(scope="module")
def oracle(models):
    return {name: {r: plain.forward(config, weights, toks) for r, toks in request_set(name).items()}
            for name, (_, config, weights) in models.items()}


def make_engine(path, dtype, max_tokens, **options):
    from liyab_b200.engine import Replayer
    options.setdefault("max_requests", 4)
    return Replayer(path, dtype, max_tokens, **options)


def check(got, want, dtype, rel_tol=REL_TOL, flips=True):
    """float32: every logit within rel_tol of the plain model's.  bfloat16: per row, the root mean square of the difference (its mean
    taken off) over that of the sequence's logits; 8 bits of mantissa put it near a percent, and the median is held to 1.5 %.  Where two
    experts' logits lie close, a rounding sends a row to another expert, and the states carry that difference to the positions after it
    (`flips`): then up to a tenth of the rows may lie beyond 6 %, none beyond the logits' own spread, and the mean is held to 4 %.  Models
    whose routers decide by clear margins are held to 6 % in every row."""
    if dtype != "bfloat16":
        return tt.check_rows(got, want, rel_tol)
    errs = []
    for (r, pos), row in got.items():
        d = row.astype(np.float64) - want[r][pos]
        spread = want[r] - want[r].mean(axis=-1, keepdims=True)
        errs.append(np.sqrt(((d - d.mean()) ** 2).mean()) / np.sqrt((spread ** 2).mean()))
    errs = np.asarray(errs)
    assert np.isfinite(errs).all() and np.median(errs) <= 1.5e-2, f"median relative error {np.median(errs):.3e}"
    if flips:
        assert errs.mean() <= 4e-2, f"mean relative error {errs.mean():.3e}"
        assert (errs > 6e-2).mean() <= 0.10 and errs.max() < 1.0, f"{(errs > 6e-2).sum()} of {len(errs)} rows are off by more than 6 %, the worst by {errs.max():.2f}"
    else:
        assert errs.mean() <= 2e-2 and errs.max() <= 6e-2, f"mean {errs.mean():.3e}, {(errs > 6e-2).sum()} of {len(errs)} rows are off by more than 6 %"
    return {"mean": float(errs.mean()), "worst": float(errs.max())}


# What the plain model calls a part's output -> the name of the engine's tap.
TAPS = {"attention": "attention", "memory": "memory", "state_space": "state_space", "mixer": "mixer", "routed": "routed", "out": "block"}


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_every_mechanism_by_itself(name, models):
    """The parts' outputs, run by run, against the plain functions in float32: the embedded rows (sinusoid and norm), the attention's
    heads, what the state gives before skip, gate and norm, the gated and normed heads, the stream after the mixer, after the routed
    experts and after the block.  A whole prompt, then the same prompt cut in two and in three (state and cache)."""
    from liyab_b200.engine import StepEntry
    path, config, weights = models[name]
    toks = tokens_of(name, 50, 45)
    want = []
    plain.forward(config, weights, toks, traces=want)
    embedded, want = want[0]["embed"], want[1:]
    for cuts in ([len(toks)], [19, len(toks)], [2, 33, len(toks)]):
        engine = make_engine(path, "float32", 128)
        runs = [dict() for _ in want]
        first, at = [], [-1]

        def tap(n, rows):
            if n == "embed":
                first.append(rows)
                return
            if n == "final_norm":
                return
            if n == "mixer_norm":       # a block's first tap
                at[0] += 1
            runs[at[0] % len(want)].setdefault(n, []).append(rows)
        engine.set_tap(tap)
        engine.cache.open("a")
        lo = 0
        for hi in cuts:
            engine.step([StepEntry("a", toks[lo:hi], [])])
            lo = hi
        assert at[0] + 1 == len(cuts) * len(want)
        rows = np.concatenate(first, axis=0)
        assert np.abs(rows - embedded).max() / np.abs(embedded).max() < 2e-5, f"embedded rows (cuts {cuts})"
        for i, ref_run in enumerate(want):
            runs[i]["block"] = runs[i]["feed_forward" if "feed_forward" in runs[i] else "mixer"]      # the stream as the block leaves it
            for plain_name, tap_name in TAPS.items():
                if plain_name not in ref_run:
                    continue
                ref = ref_run[plain_name]
                rows = np.concatenate(runs[i][tap_name], axis=0)
                assert rows.shape == ref.shape, (plain_name, rows.shape, ref.shape)
                err = np.abs(rows - ref).max() / max(np.abs(ref).max(), 1e-30)
                assert err < 5e-5, f"{plain_name} of run {i} (cuts {cuts}): {err:.2e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_every_cutting_matches_plain(name, dtype, models, oracle):
    path, config, _ = models[name]
    reqs = request_set(name)
    want = oracle[name]
    n_rows = sum(len(t) for t in reqs.values())
    traces = {"whole": tt.whole(reqs), "one_by_one": tt.tail_one_by_one(reqs, 10 ** 6), "tail": tt.tail_one_by_one(reqs, 40),
              "portions": tt.changing_portions(reqs), "odd_portions": tt.changing_portions(reqs, sizes=(2, 31, 2, 17, 1, 3, 33, 16, 2))}
    for kind, steps in traces.items():
        engine = make_engine(path, dtype, max_tokens=256)
        got = tt.collect(engine, steps)
        assert len(got) == n_rows
        check(got, want, dtype)
    # Mixed batches over a pool for the trace's own peak and four state slots for all requests: pages and slots are used again.
    for seed in (3, 4):
        steps = tt.mixed(reqs, max_live=4, seed=seed)
        assert max(len(e) for e, _ in steps) >= 3
        engine = make_engine(path, dtype, max_tokens=tt.peak_tokens(steps, 64))
        got = tt.collect(engine, steps)
        assert len(got) == n_rows
        check(got, want, dtype)
        assert len(reqs) > 4 and engine.cache.state_slots_free() == 4


def test_batches_of_unequal_requests_match_each_alone(models):
    """The engine against itself: every request alone and all in mixed batches give the same logits up to rounding."""
    path, _, _ = models["A"]
    reqs = request_set("A")
    alone = tt.collect(make_engine(path, "float32", max_tokens=256), tt.whole(reqs))
    steps = tt.mixed(reqs, max_live=4, seed=11, portion=23)
    together = tt.collect(make_engine(path, "float32", max_tokens=tt.peak_tokens(steps, 64)), steps)
    assert alone.keys() == together.keys()
    scale = max(np.abs(r).max() for r in alone.values())
    assert max(np.abs(alone[k] - together[k]).max() for k in alone) / scale < 2e-5


@pytest.mark.parametrize("page_size", [16, 64])
def test_pages_of_other_sizes(page_size, models, oracle):
    path, _, _ = models["A"]
    engine = make_engine(path, "float32", max_tokens=512, page_size=page_size)
    got = tt.collect(engine, tt.changing_portions(request_set("A"), sizes=(63, 2, 1, 64, 17)))
    check(got, oracle["A"], "float32")


def sharp_model(base, window, kv_heads=1, every=9, coef=0.5):
    """One attention block whose scores are sharpened so that one key takes nearly all the weight: a key that is wrongly seen or
    wrongly hidden moves the logits by far more than rounding."""
    config = dict(architecture="Viresun", vocab=40, width=32, norm=dict(eps=1e-5), layers=[
        layer(attention(2, kv_heads, 8, 12, 5.0, window, coef, every), dense(40))])
    weights = random_weights(config, 77)
    return write_model(os.path.join(base, f"sharp_{window}_{kv_heads}"), config, weights), config, f64(weights)


@pytest.mark.parametrize("window", [16, 17, 15, 33, 5, 64])
def test_window_edges_in_prompts_and_in_decoding(window, tmp_path):
    """Windows that end on, just before and just after page borders; every position of a prompt and of decoding far past the window
    against the plain model; the plain model with a window one larger or one smaller must differ clearly (or the test shows nothing)."""
    path, config, weights = sharp_model(str(tmp_path), window, kv_heads=2 if window == 33 else 1)
    toks = np.random.default_rng(5).integers(0, config["vocab"], size=150).astype(int).tolist()
    want = plain.forward(config, weights, toks)
    for delta in (-1, 1):
        other = copy.deepcopy(config)
        other["layers"][0]["mixer"]["mask"]["size"] += delta
        moved = np.abs(plain.forward(other, weights, toks) - want).max(axis=1) / np.abs(want).max()
        assert (moved > 1e-2).sum() >= 5, "the weights do not show a window that is one off"
    reqs = {"a": toks}
    for steps in (tt.whole(reqs), tt.tail_one_by_one(reqs, 110), tt.changing_portions(reqs, sizes=(15, 2, 16, 17, 1, 33, 7))):
        for dtype, tol in (("float32", 1e-4), ("bfloat16", None)):
            engine = make_engine(path, dtype, max_tokens=192)
            got = tt.collect(engine, steps)
            if tol is not None:
                tt.check_rows(got, {"a": want}, tol)
            else:
                errs = np.array([np.abs(row - want[pos]).max() for (_, pos), row in got.items()]) / np.abs(want).max()
                assert np.median(errs) < 2e-2 and (errs > 0.15).mean() < 0.05, (np.median(errs), errs.max())
    # The cache unit keeps what the window can see, no more: pages behind it came back.
    from liyab_b200.engine import StepEntry
    engine = make_engine(path, "float32", max_tokens=192)
    engine.cache.open("a")
    engine.step([StepEntry("a", toks, [])])
    assert sum(engine.cache.pages_in_use().values()) <= (window + 15) // 16 + 1


def test_temperature_steps_and_penalty_show(tmp_path):
    """The queries' temperature moves at every multiple of `every` (position p has floor((p + 1) / every)), in prompts and in decoding,
    and the penalty by distance counts from the query's own position: the plain model without either, or with the temperature's steps
    moved by one position, differs clearly; the engine agrees with the plain model in every cutting and both types."""
    config = dict(architecture="Viresun", vocab=40, width=32, norm=dict(eps=1e-5), layers=[
        layer(attention(3, 1, 8, 8, 1.5, 40, 2.0, 7), dense(40)), layer(attention(2, 2, 16, 4, 0.8, 0, 1.0, 16), None)])
    weights = random_weights(config, 78)
    weights["l0.mix.r1"] = weights["l0.mix.r1"] * 0.0 + np.array([3.0, 0.0, 1.5])
    path = write_model(str(tmp_path / "temp"), config, weights)
    weights = f64(weights)
    toks = np.random.default_rng(6).integers(0, 40, size=130).astype(int).tolist()
    want = plain.forward(config, weights, toks)

    def moved(other_config=None, other_weights=None, temperature=None):
        real = plain.query_temperature
        if temperature is not None:
            plain.query_temperature = temperature
        try:
            got = plain.forward(other_config or config, other_weights or weights, toks)
        finally:
            plain.query_temperature = real
        return (np.abs(got - want).max(axis=1) / np.abs(want).max() > 1e-2).sum()

    no_temp = copy.deepcopy(config)
    for l in no_temp["layers"]:
        l["mixer"].pop("q_temp")
    assert moved(other_config=no_temp) >= 50, "the temperature does not show"
    assert moved(temperature=lambda p, t: 1.0 + t["coef"] * np.log(np.floor(np.asarray(p) / t["every"]) + 1.0)) >= 10, "a step one position late does not show"
    flat = dict(weights)
    flat["l0.mix.r1"], flat["l1.mix.r1"] = weights["l0.mix.r1"] * 0.0, weights["l1.mix.r1"] * 0.0
    assert moved(other_weights=flat) >= 50, "the penalty does not show"
    reqs = {"a": toks}
    for steps in (tt.whole(reqs), tt.tail_one_by_one(reqs, 100), tt.changing_portions(reqs, sizes=(6, 1, 7, 2, 8, 13, 64))):
        for dtype in ("float32", "bfloat16"):
            check(tt.collect(make_engine(path, dtype, max_tokens=192), steps), {"a": want}, dtype, flips=False)


def long_state_model(base):
    """One state-space block that forgets slowly (decays just under one), so that tokens hundreds of positions back still carry weight."""
    config = dict(architecture="Viresun", vocab=50, width=32, norm=dict(eps=1e-5), layers=[layer(state_space(4, 12, 8, 2, 4, 2), dense(40))])
    weights = random_weights(config, 5)
    weights["l0.mix.A_log"] = weights["l0.mix.A_log"] * 0.0 + np.array([-6.0, -5.0, -7.0, -4.5])
    return write_model(os.path.join(base, "long_state"), config, weights), config, f64(weights)


def test_states_reach_far_back(tmp_path):
    """420 tokens through a state that forgets slowly: whole (a block per piece of the prompt), decoded (row by row), in portions that end
    on and off page borders (pieces walked by one block).  A state that lost its first 200 tokens gives clearly different logits (shown
    on the plain model)."""
    path, config, weights = long_state_model(str(tmp_path))
    toks = np.random.default_rng(9).integers(1, 50, size=420).astype(int).tolist()
    want = plain.forward(config, weights, toks)
    lost = plain.forward(config, weights, toks[200:])
    assert (np.abs(lost - want[200:]).max(axis=1) / np.abs(want).max() > 1e-2).sum() >= 100, "the weights do not show a lost state"
    reqs = {"a": toks}
    for steps in (tt.whole(reqs), tt.tail_one_by_one(reqs, 30), tt.changing_portions(reqs, sizes=(255, 2, 64, 1, 17))):
        got = tt.collect(make_engine(path, "float32", max_tokens=448), steps)
        tt.check_rows(got, {"a": want}, 2e-4)
    check(tt.collect(make_engine(path, "bfloat16", max_tokens=448), tt.changing_portions(reqs, sizes=(130, 1, 1, 40))), {"a": want}, "bfloat16", flips=False)


def test_first_tokens_of_a_sequence(tmp_path):
    """A convolution over five inputs sees zeros before a sequence's start, also when the first portions are shorter than its reach and
    when the state slot was another request's before: the plain model with the first input repeated before the start differs clearly."""
    config = dict(architecture="Viresun", vocab=50, width=32, norm=dict(eps=1e-5), layers=[
        layer(state_space(2, 8, 6, 1, 5, 1), None), layer(attention(2, 1, 8, 8, 0.5, 4, 0.5, 2), dense(24))])
    weights = random_weights(config, 8)
    path = write_model(str(tmp_path / "first"), config, weights)
    weights = f64(weights)
    real = plain.causal_conv

    def repeated_start(u, taps, bias):
        K = taps.shape[1]
        return real(np.concatenate([np.tile(u[:1], (K - 1, 1)), u]), taps, bias)[K - 1:]

    reqs = {f"r{i}": np.random.default_rng(30 + i).integers(0, 50, size=n).astype(int).tolist() for i, n in enumerate((40, 9, 3, 1, 12))}
    want = {r: plain.forward(config, weights, t) for r, t in reqs.items()}
    plain.causal_conv = repeated_start
    try:
        other = plain.forward(config, weights, reqs["r0"])
    finally:
        plain.causal_conv = real
    assert (np.abs(other - want["r0"]).max(axis=1) / np.abs(want["r0"]).max() > 1e-2).sum() >= 3, "the weights do not show what stands before the start"
    for steps in (tt.whole(reqs), tt.tail_one_by_one(reqs, 10 ** 6), tt.changing_portions(reqs, sizes=(1, 1, 2, 1, 3, 2, 17))):
        got = tt.collect(make_engine(path, "float32", max_tokens=64, max_requests=1), steps)       # one state slot, used by every request in turn
        tt.check_rows(got, want, 1e-4)


def test_sharp_router_bias_and_weights_over_the_chosen(tmp_path):
    """Experts chosen by clear margins, one and several a row: the engine picks the plain model's experts in both types; the bias takes part
    in the choice, and the weights are the softmax over the chosen logits only (the plain model without the bias, or with the softmax over
    all experts, differs clearly)."""
    config = dict(architecture="Viresun", vocab=60, width=48, norm=dict(eps=1e-5), layers=[
        layer(state_space(2, 8, 8, 1, 3, 1), moe(7, 3, 24, 1.0)), layer(attention(2, 2, 8, 8, 0.4, 12), moe(5, 1, 16, 2.5)),
        layer(attention(1, 1, 8, 8, 0.4, 0), moe(4, 2, 8, 0.6))])
    weights = random_weights(config, 101, router_std=12.0, router_bias_std=4.0)        # a seed whose margins are clear
    path = write_model(str(tmp_path / "router"), config, weights)
    weights = f64(weights)
    toks = np.random.default_rng(27).integers(0, 60, size=48).astype(int).tolist()
    traces = []
    want = plain.forward(config, weights, toks, traces=traces)
    for trace, l in zip(traces[1:], config["layers"]):       # the last chosen expert and the best unchosen one are clearly apart
        z, top = -np.sort(-trace["router"], axis=1), l["mlp"]["router"]["top"]
        assert (z[:, top - 1] - z[:, top]).min() > 0.2, "the router's margins are not clear"
    no_bias = {k: (v * 0.0 if k.endswith("router.b") else v) for k, v in weights.items()}
    assert np.abs(plain.forward(config, no_bias, toks) - want).max() / np.abs(want).max() > 1e-2
    real = plain.routed_ff

    def softmax_over_all(h, W, p, mlp, trace=None):
        z = h @ W[p + "router"].T + W[p + "router.b"][None, :]
        w = np.exp(z - z.max(axis=1, keepdims=True))
        w = w / w.sum(axis=1, keepdims=True)
        y = np.zeros((h.shape[0], W[p + "e0.down"].shape[0]))
        for t in range(h.shape[0]):
            for e in np.argsort(-z[t], kind="stable")[:mlp["router"]["top"]]:
                y[t] += w[t, e] * plain.expert(h[t:t + 1], W, f"{p}e{e}.", mlp["expert"]["limit"])[0]
        return y

    plain.routed_ff = softmax_over_all
    try:
        other = plain.forward(config, weights, toks)
    finally:
        plain.routed_ff = real
    assert np.abs(other - want).max() / np.abs(want).max() > 1e-2
    for dtype in ("float32", "bfloat16"):
        for steps in (tt.whole({"a": toks}), tt.changing_portions({"a": toks}, sizes=(20, 1, 2, 9))):
            check(tt.collect(make_engine(path, dtype, max_tokens=128), steps), {"a": want}, dtype, flips=False)


def test_long_decoding_reuses_pages(models):
    """Decoding one token at a time far past every window: pages are freed behind the windows and handed out again, and the states run
    through 400 single steps."""
    path, config, weights = models["A"]
    toks = tokens_of("A", 99, 400)
    want = plain.forward(config, weights, toks)
    engine = make_engine(path, "float32", max_tokens=128)       # far fewer pages than 400 positions
    got = tt.collect(engine, tt.tail_one_by_one({"a": toks}, 395))
    assert len(got) == 400
    tt.check_rows(got, {"a": want}, 2e-4)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(dtype, models, oracle, tmp_path):
    path, config, _ = models["A"]
    reqs = request_set("A")
    steps = tt.mixed(reqs, max_live=4, seed=8)
    out_dir = str(tmp_path / "out")
    proc = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", path, "--dtype", dtype, "--out", out_dir,
                           "--max-tokens", str(tt.peak_tokens(steps))], input=tt.to_jsonl(steps), capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done ")] == [f"done {i}" for i in range(len(steps))]
    held, got = {}, {}
    for i, (entries, end) in enumerate(steps):
        data = np.fromfile(os.path.join(out_dir, f"{i}.f32"), dtype="<f4").reshape(-1, config["vocab"])
        row = 0
        for r, toks, want in entries:
            base = held.get(r, 0)
            for w in want:
                got[(r, base + w)] = data[row]
                row += 1
            held[r] = base + len(toks)
        assert row == data.shape[0]
    check(got, oracle["A"], dtype)


@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_through_the_engine(graphs, models):
    """Prompts of unequal length served together by the scheduler, greedy, against the plain model's own greedy continuation (compared
    while the plain model's best two logits are clearly apart)."""
    from liyab_b200.engine import Engine
    from liyab_b200.sampling import SamplingParams
    path, config, weights = models["A"]
    prompts = [tokens_of("A", 70 + i, n) for i, n in enumerate((37, 5, 1, 64, 18, 90))]
    engine = Engine(model=path, dtype="float32", context_length=256, max_requests=4, max_batched_tokens=48, cuda_graphs=graphs)
    results = engine.generate_batch(prompts, SamplingParams(max_tokens=24, temperature=0.0))
    engine.close()
    for prompt, res in zip(prompts, results):
        assert res.error is None and len(res.tokens) == 24
        seq = list(prompt)
        for tok in res.tokens:
            row = plain.forward(config, weights, seq)[-1]
            best = np.sort(row)[-2:]
            if best[1] - best[0] < 1e-3 * np.abs(row).max():
                break
            assert tok == int(np.argmax(row))
            seq.append(tok)


def test_command_line_and_sampling(models):
    """The command line generates greedily what the plain model would, and the engine's sampler with a seed gives the same tokens twice
    and other tokens with another seed."""
    import json
    from liyab_b200.engine import Engine
    from liyab_b200.sampling import SamplingParams
    path, config, weights = models["B"]
    prompt = tokens_of("B", 90, 9)
    cmd = [os.path.join(ROOT, "bin", "liyab-cli"), "-m", path, "-p", ",".join(map(str, prompt)), "-n", "8", "--temp", "0", "--dtype", "float32",
           "--ctx", "128", "--json"]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [json.loads(l) for l in proc.stdout.splitlines() if l.startswith("{")]
    seq = list(prompt)
    for tok in lines[1]["tokens"]:
        row = plain.forward(config, weights, seq)[-1]
        best = np.sort(row)[-2:]
        if best[1] - best[0] < 1e-3 * np.abs(row).max():
            break
        assert tok == int(np.argmax(row))
        seq.append(tok)
    draws = []
    for seed in (5, 5, 6):
        engine = Engine(model=path, dtype="bfloat16", context_length=128, max_requests=4)
        draws.append(engine.generate_tokens(prompt, SamplingParams(max_tokens=12, temperature=0.9, top_k=20, top_p=0.95, seed=seed)).tokens)
        engine.close()
    assert draws[0] == draws[1] and draws[0] != draws[2] and all(0 <= t < config["vocab"] for t in draws[2])

