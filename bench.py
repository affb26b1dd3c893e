#!/usr/bin/env python3
"""Decode and prefill throughput of the liyab_b200 engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--size small] [--layers L] [--dtype bfloat16]
    python bench.py --impl reference        # the reference's own tools on this machine's CPU, or why they cannot run
    python bench.py --design puzutar [--size small]   # Puzutar at GPT-2's layer sizes beside GPT-2 itself (see puzutar_line)
    python bench.py --design vosurax [--size small]   # Vosurax likewise (see vosurax_line)
    python bench.py --design viresun [--size small]   # Viresun beside Vosurax and GPT-2 (see viresun_line)
    python bench.py --design revudra [--size small]   # Revudra beside Vosurax and GPT-2 (see revudra_line)

A step is one decode step of the whole batch.  The default run has the layer
sizes of GPT-2 small (12 layers, width 768, 12 heads) with random weights, a batch of
8 requests and the benchmark context of 1024 positions: 512-token prompts, then
decoding (contexts 512 -> 1024; when a request reaches the model's last position
its cache is cut back to the prompt and decoding goes on, so any K can be timed).
`value` is decoded tokens per second timed with CUDA events over exactly K
steps (the library's own measurement, host/bench.cpp: the engine's step function,
sampling on the device, ids fed back without leaving it); `e2e` is the same through
the Python entry point (Engine.generate_batch: host token ids in, host token ids
out, per-step copies both ways included).  One JSON line is printed.  Beside the
headline it holds: `points` (batch 1 and 64) with `points_detail`, `prefill`
(2 x 1024 tokens), `roofline`, `fp32` (the 32-bit engine), `medium` and `xl`
(the other two GPT-2 sizes at their full layer counts), `mixed_xl` (64 requests
with prompts of 1..1024 tokens generated to position 1024 through the scheduler)
and `same` (the timed end-to-end run's tokens equal an untimed run's).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

GPT2_SMALL = dict(model_type="gpt2", n_layer=12, n_embd=768, n_head=12, n_inner=3072, vocab_size=50257,
                  n_positions=1024, layer_norm_epsilon=1e-5, activation_function="gelu_new",
                  scale_attn_by_inverse_layer_idx=False, tie_word_embeddings=True)
SIZES = {"small": GPT2_SMALL,
         "medium": dict(GPT2_SMALL, n_layer=24, n_embd=1024, n_head=16, n_inner=4096),
         "xl": dict(GPT2_SMALL, n_layer=48, n_embd=1600, n_head=25, n_inner=6400)}
PROMPT_LEN = 512
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
FP32_TFLOPS_NOMINAL = 80.0          # 32-bit units, no tensor cores; no measured figure exists for it


def peaks():
    """Measured denominators if the driver wrote them, else the stated fallback."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            raw = json.load(f)
        return {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]),
                "bf16_tflops_sustained": float(raw.get("bf16_tflops_sustained", raw["bf16_tflops"])), "source": "measured"}
    except (OSError, KeyError, ValueError):
        return dict(FALLBACK_PEAKS, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.05)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        mhz = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 6 for n, v in zip(names, r[2:6]) if v.lower().startswith("active")})
        mx = next((int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()), None)
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx, "reasons": reasons, "samples": len(mhz)}


def model_bytes_and_flops(cfg, dtype_bytes):
    d, ff, V, L = cfg["n_embd"], cfg["n_inner"], cfg["vocab_size"], cfg["n_layer"]
    per_layer = 4 * d * d + 2 * d * ff
    weight_bytes = dtype_bytes * (L * per_layer + V * d)        # every matrix once; the tied table once
    kv_per_pos = 2 * L * d * dtype_bytes

    def prefill_flops(seq_lens, rows):
        T = sum(seq_lens)
        return 2 * T * L * per_layer + sum(2 * L * d * s * s for s in seq_lens) + 2 * rows * V * d

    return weight_bytes, kv_per_pos, prefill_flops


def decode_point(replayer, cfg, dtype_bytes, batch, steps, warmup, pk, seed=0):
    """One device-timed decode measurement with its roofline fraction."""
    r = replayer.bench_decode(batch, PROMPT_LEN, steps, warmup, seed)
    weight_bytes, kv_per_pos, _ = model_bytes_and_flops(cfg, dtype_bytes)
    step_bytes = weight_bytes + batch * r["mean_context"] * kv_per_pos
    achieved = step_bytes / (r["ms_per_step"] / 1e3) / 1e9
    r.update(tok_s=batch / (r["ms_per_step"] / 1e3), step_bytes=step_bytes, achieved_gbs=achieved, frac=achieved / pk["hbm_gbs"])
    return r


def prefill_point(replayer, cfg, dtype_bytes, pk, dtype):
    n_seq = PREFILL_TOKENS // 1024
    r = replayer.bench_prefill(n_seq, 1024, 5)
    _, _, flops = model_bytes_and_flops(cfg, dtype_bytes)
    peak = pk["bf16_tflops"] if dtype == "bfloat16" else FP32_TFLOPS_NOMINAL
    ms = r["ms_per_step"]
    return {"value": round(PREFILL_TOKENS / (ms / 1e3), 1), "tokens": PREFILL_TOKENS, "ms": round(ms, 4),
            "frac": round(flops([1024] * n_seq, n_seq) / (ms / 1e3) / 1e12 / peak, 4), "median_ms": round(r["wall_ms_per_step"], 4),
            "launches": r["kernel_launches"]}


def detail(r):
    return {"tokens_per_s": round(r["tok_s"], 1), "ms_per_step": round(r["ms_per_step"], 4), "mean_context": round(r["mean_context"], 1),
            "frac": round(r["frac"], 4), "path": "fused" if r["fused_steps"] else ("graph" if r["graph_steps"] else "parts")}


def e2e_run(model_dir, dtype, batch, steps):
    """The same metric through Engine.generate_batch: host ids in, host ids out.  The workload runs twice (the first,
    untimed, also warms the engine up); `same` says that both runs gave the same tokens."""
    import numpy as np
    from liyab_b200 import Engine, EngineConfig, SamplingParams
    engine = Engine(EngineConfig(model=model_dir, dtype=dtype, max_requests=batch, max_batched_tokens=2048,
                                 num_pages=batch * 64, cuda_graphs=True))
    rng = np.random.default_rng(2)
    n_new = min(steps, engine.max_positions - PROMPT_LEN)
    prompts = [rng.integers(0, engine.vocab_size, size=PROMPT_LEN).tolist() for _ in range(batch)]
    params = SamplingParams(temperature=0.0, max_tokens=n_new, ignore_eos=True)
    untimed = engine.generate_batch(prompts, params)
    before = engine.stats()
    results = engine.generate_batch(prompts, params)
    after = engine.stats()
    decode_ms = max(r.stats.decode_ms for r in results)
    tokens = sum(max(0, r.stats.generated_tokens - 1) for r in results)
    n_steps = max(1, after["steps"] - before["steps"])
    out = {"value": round(tokens / (decode_ms / 1e3), 1) if decode_ms > 0 else 0.0, "unit": "tokens/s",
           "h2d_bytes_per_step": (after["h2d_bytes"] - before["h2d_bytes"]) // n_steps,
           "d2h_bytes_per_step": (after["d2h_bytes"] - before["d2h_bytes"]) // n_steps, "steps": n_new}
    same = [r.tokens for r in results] == [r.tokens for r in untimed]
    engine.close()
    return out, same


def mixed_run(model_dir, dtype, n_requests, budget):
    """64 requests with prompts of 1..positions tokens, each generated to the model's last position, all submitted at
    once: chunked prefill beside decoding through the scheduler; host ids in and out."""
    import numpy as np
    from liyab_b200 import Engine, EngineConfig, SamplingParams
    engine = Engine(EngineConfig(model=model_dir, dtype=dtype, max_requests=n_requests, max_batched_tokens=budget, page_size=16))
    P = engine.max_positions
    rng = np.random.default_rng(3)
    lens = rng.integers(1, P + 1, size=n_requests)
    prompts = [rng.integers(0, engine.vocab_size, size=int(k)).tolist() for k in lens]
    params = [SamplingParams(temperature=0.0, max_tokens=max(1, int(P - k)), ignore_eos=True) for k in lens]
    engine.generate_batch([p[:8] for p in prompts[:4]], SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))
    before = engine.stats()
    t0 = time.perf_counter()
    results = engine.generate_batch(prompts, params)
    seconds = time.perf_counter() - t0
    after = engine.stats()
    generated = sum(r.stats.generated_tokens for r in results)
    out = {"requests": n_requests, "prompt_tokens": int(lens.sum()), "generated_tokens": generated, "seconds": round(seconds, 3),
           "generated_tokens_per_s": round(generated / seconds, 1), "total_tokens_per_s": round((generated + int(lens.sum())) / seconds, 1),
           "steps": after["steps"] - before["steps"], "preemptions": after["preemptions"] - before["preemptions"],
           "batched_token_histogram": {k: a - b for k, a, b in zip(["1", "2-8", "9-32", "33-128", "129-512", "513-2048", ">2048"],
                                                                   after["histogram"], before["histogram"])},
           "finished": sorted({r.finish_reason for r in results}), "page_size": 16, "token_budget": budget}
    engine.close()
    return out


def size_block(tmp, size, dtype, steps, pk):
    """Decode at batch 1 / 8 / 64 and the 2,048-token prefill of one GPT-2 size at its full layer count."""
    from liyab_b200.engine import Replayer
    from liyab_b200.weights import write_random_model
    cfg = SIZES[size]
    dtype_bytes = 2 if dtype == "bfloat16" else 4
    folder = write_random_model(os.path.join(tmp, f"gpt2_{size}_{dtype}"), cfg, seed=0, dtype=dtype)
    rep = Replayer(folder, dtype, max_tokens=64 * 1024, max_requests=64, cuda_graphs=True, max_step_tokens=PREFILL_TOKENS)
    block = {"n_layer": cfg["n_layer"], "n_embd": cfg["n_embd"], "n_head": cfg["n_head"], "n_inner": cfg["n_inner"]}
    for b in (1, 8, 64):
        block[f"decode_b{b}"] = detail(decode_point(rep, cfg, dtype_bytes, b, steps, 3, pk))
    block["prefill"] = prefill_point(rep, cfg, dtype_bytes, pk, dtype)
    rep.close()
    return block, folder


def puzutar_config(size, layers=0):
    """Puzutar with the width, depth, head count, inner width and vocabulary of a GPT-2 size: heads of 48 unrotated and
    16 rotated query values and 64 value values (GPT-2's head size), a latent of a third of the width rounded up to 128,
    a window of 512, two norm groups, a side input of 64 values; of every four blocks the last two read the second's latent."""
    g = SIZES[size]
    L, W, H = layers or g["n_layer"], g["n_embd"], g["n_head"]
    rank = max(128, (W // 3 + 127) // 128 * 128)
    blocks = []
    for i in range(L):
        m = dict(heads=H, dim=48, rot_dim=16, vdim=64, kv_rank=rank, scale=0.125, mask=dict(size=512), rot=dict(base=1e6, dims=16))
        if i % 4 >= 2:
            m["kv_from"] = i - i % 4 + 1
        blocks.append(dict(type="latent_attention", mixer=m, mlp=dict(kind="dense", ff=g["n_inner"])))
    return dict(architecture="Puzutar", vocab=g["vocab_size"], width=W, norm=dict(eps=1e-5, groups=2), token_side=dict(dim=64),
                max_positions=g["n_positions"], layers=blocks)


def puzutar_bytes_and_flops(cfg, dtype_bytes):
    W, V, side = cfg["width"], cfg["vocab"], cfg["token_side"]["dim"]
    weights, per_pos_read, per_token, attn = V * W, 0, 0, []
    for l in cfg["layers"]:
        m, ff = l["mixer"], l["mlp"]["ff"]
        H, dq, rank, rot = m["heads"], m["dim"] + m["rot_dim"], m["kv_rank"], m["rot_dim"]
        mats = H * dq * W + (0 if "kv_from" in m else (rank + rot) * W) + H * m["dim"] * rank + H * m["vdim"] * rank + W * H * m["vdim"] + 2 * W * ff + 2 * side * W
        weights += mats
        per_token += mats
        per_pos_read += rank + rot                   # every block reads its (own or borrowed) latent rows once per request and step
        attn.append((H, rank, rot, m["mask"]["size"]))

    def prefill_flops(seq_lens, rows):
        total = 2 * sum(seq_lens) * per_token + 2 * rows * V * W
        for H, rank, rot, w in attn:                 # scores over rank + rot values and sums over rank values, on the latent rows
            total += sum(2 * H * (2 * rank + rot) * sum(min(i + 1, w) for i in range(s)) for s in seq_lens)
        return total

    return dtype_bytes * (weights + side * 0), dtype_bytes * per_pos_read, prefill_flops, [w for _, _, _, w in attn]


def puzutar_line(args) -> int:
    """--design puzutar: decode (batch 1 / 8 / 64, 512-token prompts) and prefill (2 x 1024 tokens) of Puzutar at the layer
    sizes of GPT-2 `--size`, and the same four figures of GPT-2 at that size, device-timed by the library's own measurement."""
    from liyab_b200.engine import Replayer
    from liyab_b200.weights import write_random_model
    pk = peaks()
    dtype_bytes = 2 if args.dtype == "bfloat16" else 4
    cfg = puzutar_config(args.size, args.layers)
    gpt = dict(SIZES[args.size], n_layer=args.layers or SIZES[args.size]["n_layer"])
    steps = min(args.steps, 128)
    out = {"design": "puzutar", "size": args.size, "dtype": args.dtype, "peaks": pk["source"],
           "config": {k: cfg[k] for k in ("width", "vocab", "norm", "token_side")} | {"layers": len(cfg["layers"]), "mixer": cfg["layers"][0]["mixer"],
                                                                                     "ff": cfg["layers"][0]["mlp"]["ff"]}}
    with tempfile.TemporaryDirectory(prefix="liyab_b200_bench_") as tmp:
        folder = write_random_model(os.path.join(tmp, "puzutar"), cfg, seed=0, dtype=args.dtype)
        rep = Replayer(folder, args.dtype, max_tokens=64 * 1024, max_requests=64, cuda_graphs=True, max_step_tokens=PREFILL_TOKENS)
        weight_bytes, row_bytes, flops, windows = puzutar_bytes_and_flops(cfg, dtype_bytes)
        block = {}
        for b in (1, 8, 64):
            r = rep.bench_decode(b, PROMPT_LEN, steps, 3, 0)
            seen = sum(min(r["mean_context"], w) for w in windows) / len(windows)
            step_bytes = weight_bytes + b * seen * row_bytes
            achieved = step_bytes / (r["ms_per_step"] / 1e3) / 1e9
            r.update(tok_s=b / (r["ms_per_step"] / 1e3), frac=achieved / pk["hbm_gbs"])
            block[f"decode_b{b}"] = detail(r) | {"launches_per_step": r["kernel_launches"] // steps}
        n_seq = PREFILL_TOKENS // 1024
        r = rep.bench_prefill(n_seq, 1024, 5)
        peak = pk["bf16_tflops"] if args.dtype == "bfloat16" else FP32_TFLOPS_NOMINAL
        block["prefill"] = {"value": round(PREFILL_TOKENS / (r["ms_per_step"] / 1e3), 1), "ms": round(r["ms_per_step"], 4),
                            "frac": round(flops([1024] * n_seq, n_seq) / (r["ms_per_step"] / 1e3) / 1e12 / peak, 4), "launches": r["kernel_launches"]}
        rep.close()
        out["puzutar"] = block
        out["gpt2"], _ = size_block(tmp, args.size, args.dtype, steps, pk) if not args.layers else ({}, None)
        if args.layers:
            gfolder = write_random_model(os.path.join(tmp, "gpt2"), gpt, seed=0, dtype=args.dtype)
            grep_ = Replayer(gfolder, args.dtype, max_tokens=64 * 1024, max_requests=64, cuda_graphs=True, max_step_tokens=PREFILL_TOKENS)
            gb = {f"decode_b{b}": detail(decode_point(grep_, gpt, dtype_bytes, b, steps, 3, pk)) for b in (1, 8, 64)}
            gb["prefill"] = prefill_point(grep_, gpt, dtype_bytes, pk, args.dtype)
            grep_.close()
            out["gpt2"] = gb
    print(json.dumps(out))
    return 0


def vosurax_config(size, layers=0):
    """Vosurax with the width, depth, head count, inner width and vocabulary of a GPT-2 size.  Of every four blocks the first is a
    retention (heads of 64 query and 128 value values, half of them rotated, dense feed-forward), the others are attention in chunks
    of 512 (heads of 64, a quarter as many key/value heads) beside a gated memory (half as many heads, 64 / 128 values) with 16
    experts of a quarter of the inner width, two a token, and a shared one.  Blocks 1 and 2 run twice; two blocks fewer, so that the
    runs equal GPT-2's layers."""
    g = SIZES[size]
    L, W, H = max(4, (layers or g["n_layer"]) - 2), g["n_embd"], g["n_head"]
    blocks = []
    for i in range(L):
        if i % 4 == 0:
            decay = [1.0 - 2.0 ** (-4 - 5 * h / H) for h in range(H)]
            blocks.append(dict(type="retention", mixer=dict(heads=H, dim=64, vdim=128, decay=decay, rot=dict(base=1e5, dims=32)), mlp=dict(kind="dense", ff=g["n_inner"])))
        else:
            mixer = dict(left=dict(heads=H, kv_heads=max(1, H // 4), dim=64, vdim=64, scale=0.125, mask=dict(size=512)),
                         right=dict(heads=max(1, H // 2), dim=64, vdim=128, gate_cap=15.0))
            blocks.append(dict(type="parallel", mixer=mixer, mlp=dict(kind="moe", expert=dict(ff=g["n_inner"] // 4), router=dict(experts=16, top=2),
                                                                      shared=dict(ff=g["n_inner"] // 4))))
    return dict(architecture="Vosurax", vocab=g["vocab_size"], width=W, norm=dict(eps=1e-5), loop=dict(start=1, stop=3, times=2),
                max_positions=g["n_positions"], layers=blocks)


def vosurax_bytes_and_flops(cfg, dtype_bytes, batch):
    """Bytes a decode step of `batch` requests must read (weights its rows touch, memories read and written, visible cache rows) and the
    FLOPs of a prefill (products with the weights a token uses, attention inside its chunk, the memories' updates and reads)."""
    W, V = cfg["width"], cfg["vocab"]
    loop = cfg["loop"]
    runs = [i for i in range(loop["start"])] + [i for _ in range(loop["times"]) for i in range(loop["start"], loop["stop"])] + list(range(loop["stop"], len(cfg["layers"])))
    step_bytes, token_flops, attn, mem = 2 * V * W * dtype_bytes, 2 * V * W, [], []
    for i in runs:
        l = cfg["layers"][i]
        m, mlp = l["mixer"], l["mlp"]
        if l["type"] == "retention":
            mats = W * m["heads"] * (2 * m["dim"] + 2 * m["vdim"]) + W * m["heads"] * m["vdim"]
            mem.append((m["heads"], m["dim"], m["vdim"]))
        else:
            a, r = m["left"], m["right"]
            mats = W * (a["heads"] * (a["dim"] + a["vdim"]) + a["kv_heads"] * (a["dim"] + a["vdim"])) + W * a["heads"] * a["vdim"]
            mats += W * r["heads"] * (2 * r["dim"] + 2 * r["vdim"] + 2) + W * r["heads"] * r["vdim"]
            mem.append((r["heads"], r["dim"], r["vdim"]))
            attn.append((a["heads"], a["kv_heads"], a["dim"], a["vdim"], a["mask"]["size"]))
        used = mats
        touched = mats
        if mlp["kind"] == "dense":
            used += 2 * W * mlp["ff"]
            touched += 2 * W * mlp["ff"]
        else:
            E, top, F, S = mlp["router"]["experts"], mlp["router"]["top"], mlp["expert"]["ff"], mlp["shared"]["ff"]
            used += E * W + 3 * W * (top * F + S)
            touched += E * W + 3 * W * S + 3 * W * F * E * (1.0 - (1.0 - top / E) ** batch)      # the experts a batch is expected to touch
        token_flops += 2 * used
        step_bytes += touched * dtype_bytes
    state_bytes = sum(2 * 4 * H * (D * E + D + 1) for H, D, E in mem)
    cache_row_bytes = [dtype_bytes * 2 * G * max(D, E) for _, G, D, E, _ in attn]

    def decode_bytes(mean_context):
        return step_bytes + batch * (state_bytes + sum(b * min(mean_context, c / 2) for b, (_, _, _, _, c) in zip(cache_row_bytes, attn)))

    def prefill_flops(seq_lens, rows):
        total = sum(seq_lens) * (token_flops - 2 * V * W) + 2 * rows * V * W
        for H, G, D, E, c in attn:
            total += sum(2 * H * (D + E) * sum(i % c + 1 for i in range(s)) for s in seq_lens)
        for H, D, E in mem:
            total += sum(seq_lens) * 4 * H * D * E
        return total

    return decode_bytes, prefill_flops


def vosurax_line(args) -> int:
    """--design vosurax: decode (batch 1 / 8 / 64, 512-token prompts) and prefill (2 x 1024 tokens) of Vosurax at the layer sizes of
    GPT-2 `--size`, and the same four figures of GPT-2 at that size, device-timed by the library's own measurement."""
    from liyab_b200.engine import Replayer
    from liyab_b200.weights import write_random_model
    pk = peaks()
    dtype_bytes = 2 if args.dtype == "bfloat16" else 4
    cfg = vosurax_config(args.size, args.layers)
    steps = min(args.steps, 128)
    out = {"design": "vosurax", "size": args.size, "dtype": args.dtype, "peaks": pk["source"],
           "config": {k: cfg[k] for k in ("width", "vocab", "norm", "loop")} | {"layers": len(cfg["layers"]), "retention": cfg["layers"][0], "parallel": cfg["layers"][1]}}
    with tempfile.TemporaryDirectory(prefix="liyab_b200_bench_") as tmp:
        folder = write_random_model(os.path.join(tmp, "vosurax"), cfg, seed=0, dtype=args.dtype)
        rep = Replayer(folder, args.dtype, max_tokens=64 * 1024, max_requests=64, cuda_graphs=True, max_step_tokens=PREFILL_TOKENS)
        block = {}
        for b in (1, 8, 64):
            decode_bytes, flops = vosurax_bytes_and_flops(cfg, dtype_bytes, b)
            r = rep.bench_decode(b, PROMPT_LEN, steps, 3, 0)
            achieved = decode_bytes(r["mean_context"]) / (r["ms_per_step"] / 1e3) / 1e9
            r.update(tok_s=b / (r["ms_per_step"] / 1e3), frac=achieved / pk["hbm_gbs"])
            block[f"decode_b{b}"] = detail(r) | {"launches_per_step": r["kernel_launches"] // steps}
        n_seq = PREFILL_TOKENS // 1024
        r = rep.bench_prefill(n_seq, 1024, 5)
        peak = pk["bf16_tflops"] if args.dtype == "bfloat16" else FP32_TFLOPS_NOMINAL
        block["prefill"] = {"value": round(PREFILL_TOKENS / (r["ms_per_step"] / 1e3), 1), "ms": round(r["ms_per_step"], 4),
                            "frac": round(flops([1024] * n_seq, n_seq) / (r["ms_per_step"] / 1e3) / 1e12 / peak, 4), "launches": r["kernel_launches"]}
        rep.close()
        out["vosurax"] = block
        if not args.layers:
            out["gpt2"], _ = size_block(tmp, args.size, args.dtype, steps, pk)
        else:
            gpt = dict(SIZES[args.size], n_layer=args.layers)
            gfolder = write_random_model(os.path.join(tmp, "gpt2"), gpt, seed=0, dtype=args.dtype)
            grep_ = Replayer(gfolder, args.dtype, max_tokens=64 * 1024, max_requests=64, cuda_graphs=True, max_step_tokens=PREFILL_TOKENS)
            gb = {f"decode_b{b}": detail(decode_point(grep_, gpt, dtype_bytes, b, steps, 3, pk)) for b in (1, 8, 64)}
            gb["prefill"] = prefill_point(grep_, gpt, dtype_bytes, pk, args.dtype)
            grep_.close()
            out["gpt2"] = gb
    print(json.dumps(out))
    return 0


def viresun_config(size, layers=0):
    """Viresun with the width, depth, head count, inner width and vocabulary of a GPT-2 size.  Of every four blocks the second is a state
    space (inner width twice the model's, heads of 64 values, a state of 128 numbers, two groups, a convolution over 4 inputs, the norm
    in two groups) with 16 experts of a quarter of the inner width, two a token, capped at 7; the others are attention under a window of
    512 (heads of 64, a quarter as many key/value heads, a temperature that steps every 128 positions, a penalty by distance), the first
    and third with a dense feed-forward, the fourth with the experts.  The last block runs on the second block's weights."""
    g = SIZES[size]
    L, W, H = max(4, layers or g["n_layer"]), g["n_embd"], g["n_head"]
    attn = dict(heads=H, kv_heads=max(1, H // 4), dim=64, vdim=64, scale=0.125, mask=dict(size=512), q_temp=dict(coef=0.5, every=128))
    ssm = dict(heads=2 * W // 64, vdim=64, state=128, groups=2, conv=4, norm_groups=2)
    dense = dict(kind="dense", ff=g["n_inner"])
    moe = dict(kind="moe", expert=dict(ff=g["n_inner"] // 4, limit=7.0), router=dict(experts=16, top=2))
    blocks = []
    for i in range(L):
        if i % 4 == 1:
            blocks.append(dict(type="mamba2", mixer=ssm, mlp=moe))
        else:
            blocks.append(dict(type="attention", mixer=attn, mlp=moe if i % 4 == 3 else dense))
    blocks[-1] = dict(blocks[1], weights_of=1)
    return dict(architecture="Viresun", vocab=g["vocab_size"], width=W, norm=dict(eps=1e-5), max_positions=g["n_positions"], layers=blocks)


def viresun_bytes_and_flops(cfg, dtype_bytes, batch):
    """Bytes a decode step of `batch` requests must read (weights its rows touch, states read and written, visible cache rows) and the
    FLOPs of a prefill (products with the weights a token uses, attention inside its window, the states' updates and reads)."""
    W, V = cfg["width"], cfg["vocab"]
    step_bytes, token_flops, attn, mem = 2 * V * W * dtype_bytes, 2 * V * W, [], []
    for l in cfg["layers"]:
        m, mlp = l["mixer"], l["mlp"]
        if l["type"] == "mamba2":
            inner, GN = m["heads"] * m["vdim"], m["groups"] * m["state"]
            mats = W * (2 * inner + 2 * GN + m["heads"]) + W * inner
            mem.append((m["heads"], m["state"], m["vdim"], (m["conv"] - 1) * (inner + 2 * GN)))
        else:
            mats = W * (m["heads"] * m["dim"] + m["kv_heads"] * (m["dim"] + m["vdim"])) + W * m["heads"] * m["vdim"]
            attn.append((m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["mask"]["size"]))
        used = touched = mats
        if mlp and mlp["kind"] == "dense":
            used += 3 * W * mlp["ff"]
            touched += 3 * W * mlp["ff"]
        elif mlp:
            E, top, F = mlp["router"]["experts"], mlp["router"]["top"], mlp["expert"]["ff"]
            used += E * W + 3 * W * top * F
            touched += E * W + 3 * W * F * E * (1.0 - (1.0 - top / E) ** batch)      # the experts a batch is expected to touch
        token_flops += 2 * used
        step_bytes += touched * dtype_bytes
    state_bytes = sum(2 * 4 * (H * N * E + conv) for H, N, E, conv in mem)
    cache_row_bytes = [dtype_bytes * 2 * G * max(D, E) for _, G, D, E, _ in attn]

    def decode_bytes(mean_context):
        return step_bytes + batch * (state_bytes + sum(b * min(mean_context, c) for b, (_, _, _, _, c) in zip(cache_row_bytes, attn)))

    def prefill_flops(seq_lens, rows):
        total = sum(seq_lens) * (token_flops - 2 * V * W) + 2 * rows * V * W
        for H, G, D, E, c in attn:
            total += sum(2 * H * (D + E) * sum(min(i + 1, c) for i in range(s)) for s in seq_lens)
        for H, N, E, _ in mem:
            total += sum(seq_lens) * 4 * H * N * E
        return total

    return decode_bytes, prefill_flops


def design_block(folder, dtype, steps, pk, bytes_and_flops):
    """Decode at batch 1 / 8 / 64 (512-token prompts) and a prefill of 2 x 1,024 tokens of the model in `folder`, device-timed by the library's
    own measurement; `bytes_and_flops(batch)` gives the step's bytes and the prefill's FLOPs for the fractions of the measured peaks."""
    from liyab_b200.engine import Replayer
    rep = Replayer(folder, dtype, max_tokens=64 * 1024, max_requests=64, cuda_graphs=True, max_step_tokens=PREFILL_TOKENS)
    block = {}
    for b in (1, 8, 64):
        decode_bytes, flops = bytes_and_flops(b)
        r = rep.bench_decode(b, PROMPT_LEN, steps, 3, 0)
        achieved = decode_bytes(r["mean_context"]) / (r["ms_per_step"] / 1e3) / 1e9
        r.update(tok_s=b / (r["ms_per_step"] / 1e3), frac=achieved / pk["hbm_gbs"])
        block[f"decode_b{b}"] = detail(r) | {"launches_per_step": r["kernel_launches"] // steps}
    n_seq = PREFILL_TOKENS // 1024
    r = rep.bench_prefill(n_seq, 1024, 5)
    peak = pk["bf16_tflops"] if dtype == "bfloat16" else FP32_TFLOPS_NOMINAL
    block["prefill"] = {"value": round(PREFILL_TOKENS / (r["ms_per_step"] / 1e3), 1), "ms": round(r["ms_per_step"], 4),
                        "frac": round(flops([1024] * n_seq, n_seq) / (r["ms_per_step"] / 1e3) / 1e12 / peak, 4), "launches": r["kernel_launches"]}
    rep.close()
    return block


def viresun_line(args) -> int:
    """--design viresun: decode (batch 1 / 8 / 64, 512-token prompts) and prefill (2 x 1024 tokens) of Viresun at the layer sizes of
    GPT-2 `--size`, and the same four figures of Vosurax (the engine's closest design: attention under a mask, a matrix state per head,
    routed experts) and of GPT-2 at that size."""
    from liyab_b200.weights import write_random_model
    pk = peaks()
    dtype_bytes = 2 if args.dtype == "bfloat16" else 4
    cfg = viresun_config(args.size, args.layers)
    steps = min(args.steps, 128)
    out = {"design": "viresun", "size": args.size, "dtype": args.dtype, "peaks": pk["source"],
           "config": {k: cfg[k] for k in ("width", "vocab", "norm")} | {"layers": len(cfg["layers"]), "attention": cfg["layers"][0], "state_space": cfg["layers"][1]}}
    with tempfile.TemporaryDirectory(prefix="liyab_b200_bench_") as tmp:
        folder = write_random_model(os.path.join(tmp, "viresun"), cfg, seed=0, dtype=args.dtype)
        out["viresun"] = design_block(folder, args.dtype, steps, pk, lambda b: viresun_bytes_and_flops(cfg, dtype_bytes, b))
        other = vosurax_config(args.size, args.layers + 2 if args.layers else 0)
        folder = write_random_model(os.path.join(tmp, "vosurax"), other, seed=0, dtype=args.dtype)
        out["vosurax"] = design_block(folder, args.dtype, steps, pk, lambda b: vosurax_bytes_and_flops(other, dtype_bytes, b))
        if not args.layers:
            out["gpt2"], _ = size_block(tmp, args.size, args.dtype, steps, pk)
    print(json.dumps(out))
    return 0


def revudra_config(size, layers=0):
    """Revudra with the width, depth, head count, inner width and vocabulary of a GPT-2 size.  Of every four blocks the first is attention
    under a window of 512 (heads of 64, a quarter as many key/value heads, half of a head rotated, values blended from the second such
    block on) with the dense feed-forward; the second and third are matrix memories (heads of 64 x 64, decays from 0.94 to 0.998) and the
    fourth attention over latent rows (heads of 48 + 16 rotated values, a latent of 256, queries through a latent of half the width);
    these three have 16 experts of a quarter of the inner width, two a token by the table."""
    g = SIZES[size]
    L, W, H = max(4, layers or g["n_layer"]), g["n_embd"], g["n_head"]
    attn = dict(heads=H, kv_heads=max(1, H // 4), dim=64, vdim=64, scale=0.125, mask=dict(size=512), rot=dict(base=1e6, dims=32), v_mix=True)
    memory = dict(heads=H, dim=64, vdim=64, decay=[1.0 - 2.0 ** (-4 - 5 * h / H) for h in range(H)])
    latent = dict(heads=H, dim=48, rot_dim=16, vdim=64, kv_rank=256, q_rank=W // 2, scale=0.125, rot=dict(base=1e4, dims=16))
    dense = dict(kind="dense", ff=g["n_inner"])
    moe = dict(kind="moe", expert=dict(ff=g["n_inner"] // 4), router=dict(experts=16, top=2))
    kinds = [("attention", attn, dense), ("lightning", memory, moe), ("lightning", memory, moe), ("latent_attention", latent, moe)]
    blocks = [dict(type=kinds[i % 4][0], mixer=kinds[i % 4][1], mlp=kinds[i % 4][2]) for i in range(L)]
    return dict(architecture="Revudra", vocab=g["vocab_size"], width=W, norm=dict(eps=1e-5), residual_mult=0.7, embedding=dict(scale=1.0), logit_scale=1.0,
                max_positions=g["n_positions"], layers=blocks)


def revudra_bytes_and_flops(cfg, dtype_bytes, batch):
    """Bytes a decode step of `batch` requests must read (weights its rows touch, memories read and written, visible cache rows) and the
    FLOPs of a prefill (products with the weights a token uses, attention inside its window or over the latent rows as it is computed, the
    memories' updates and reads)."""
    W, V = cfg["width"], cfg["vocab"]
    step_bytes, token_flops, attn, lat, mem = 2 * V * W * dtype_bytes, 2 * V * W, [], [], []
    for l in cfg["layers"]:
        m, mlp = l["mixer"], l["mlp"]
        H = m["heads"]
        if l["type"] == "attention":
            mats = W * (H * m["dim"] + m["kv_heads"] * (m["dim"] + m["vdim"]) + H * m["vdim"]) + W * H * m["vdim"]
            attn.append((H, m["kv_heads"], m["dim"], m["vdim"], m["mask"]["size"]))
        elif l["type"] == "lightning":
            mats = W * H * (2 * m["dim"] + 2 * m["vdim"]) + W * H * m["vdim"]
            mem.append((H, m["dim"], m["vdim"]))
        else:
            row = m["kv_rank"] + m["rot_dim"]
            mats = W * (m["q_rank"] + row + H) + m["q_rank"] * H * (m["dim"] + m["rot_dim"]) + H * m["kv_rank"] * (m["dim"] + m["vdim"]) + W * H * m["vdim"]
            lat.append((H, m["kv_rank"], m["rot_dim"]))
        used = touched = mats
        if mlp and mlp["kind"] == "dense":
            used += 2 * W * mlp["ff"]
            touched += 2 * W * mlp["ff"]
        elif mlp:
            E, top, F = mlp["router"]["experts"], mlp["router"]["top"], mlp["expert"]["ff"]
            used += 3 * W * top * F
            touched += 3 * W * F * E * (1.0 - (1.0 - top / E) ** batch)      # the experts a batch is expected to touch
        token_flops += 2 * used
        step_bytes += touched * dtype_bytes
    state_bytes = sum(2 * 4 * H * (D * E + D + 1) for H, D, E in mem)
    cache_row_bytes = [dtype_bytes * 2 * G * max(D, E) for _, G, D, E, _ in attn]
    latent_row_bytes = [dtype_bytes * (C + R) for _, C, R in lat]

    def decode_bytes(mean_context):
        return step_bytes + batch * (state_bytes + sum(b * min(mean_context, c) for b, (_, _, _, _, c) in zip(cache_row_bytes, attn)) +
                                     sum(b * mean_context for b in latent_row_bytes))

    def prefill_flops(seq_lens, rows):
        total = sum(seq_lens) * (token_flops - 2 * V * W) + 2 * rows * V * W
        for H, G, D, E, c in attn:
            total += sum(2 * H * (D + E) * sum(min(i + 1, c) for i in range(s)) for s in seq_lens)
        for H, C, R in lat:
            total += sum(2 * H * (2 * C + R) * s * (s + 1) // 2 for s in seq_lens)
        for H, D, E in mem:
            total += sum(seq_lens) * 4 * H * D * E
        return total

    return decode_bytes, prefill_flops


def revudra_line(args) -> int:
    """--design revudra: decode (batch 1 / 8 / 64, 512-token prompts) and prefill (2 x 1024 tokens) of Revudra at the layer sizes of
    GPT-2 `--size`, and the same four figures of Vosurax (the engine's closest design: attention with normed queries and keys under a
    mask and a gate, a matrix memory per head with a fixed decay, small gated experts) and of GPT-2 at that size."""
    from liyab_b200.weights import write_random_model
    pk = peaks()
    dtype_bytes = 2 if args.dtype == "bfloat16" else 4
    cfg = revudra_config(args.size, args.layers)
    steps = min(args.steps, 128)
    out = {"design": "revudra", "size": args.size, "dtype": args.dtype, "peaks": pk["source"],
           "config": {k: cfg[k] for k in ("width", "vocab", "norm")} | {"layers": len(cfg["layers"]), "attention": cfg["layers"][0]["mixer"],
                                                                         "memory": {k: v for k, v in cfg["layers"][1]["mixer"].items() if k != "decay"},
                                                                         "latent_attention": cfg["layers"][3]["mixer"], "experts": cfg["layers"][1]["mlp"]}}
    with tempfile.TemporaryDirectory(prefix="liyab_b200_bench_") as tmp:
        folder = write_random_model(os.path.join(tmp, "revudra"), cfg, seed=0, dtype=args.dtype)
        out["revudra"] = design_block(folder, args.dtype, steps, pk, lambda b: revudra_bytes_and_flops(cfg, dtype_bytes, b))
        other = vosurax_config(args.size, args.layers + 2 if args.layers else 0)
        folder = write_random_model(os.path.join(tmp, "vosurax"), other, seed=0, dtype=args.dtype)
        out["vosurax"] = design_block(folder, args.dtype, steps, pk, lambda b: vosurax_bytes_and_flops(other, dtype_bytes, b))
        if not args.layers:
            out["gpt2"], _ = size_block(tmp, args.size, args.dtype, steps, pk)
    print(json.dumps(out))
    return 0



def reference_arm(args) -> int:
    from baseline.reference_arm import run
    return run(args)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--size", default="small", choices=sorted(SIZES), help="the model of the headline figures")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration (reported)")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-points", action="store_true", help="the headline figure only")
    ap.add_argument("--no-extra", action="store_true", help="skip the 32-bit engine, the other sizes and the mixed workload")
    ap.add_argument("--design", default="gpt2", choices=["gpt2", "puzutar", "vosurax", "viresun", "revudra"],
                    help="puzutar, vosurax, viresun, revudra: that design at the layer sizes of GPT-2 --size beside GPT-2 itself (its own JSON line; the default run is unchanged)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.design == "puzutar":
        return puzutar_line(args)
    if args.design == "vosurax":
        return vosurax_line(args)
    if args.design == "viresun":
        return viresun_line(args)
    if args.design == "revudra":
        return revudra_line(args)
    if args.gpus != 1:
        print(f"bench.py measures a single-GPU engine; --gpus {args.gpus} is not supported (run with --gpus 1)")
        return 2
    args.warmup = max(args.warmup, 3)
    from liyab_b200.engine import Replayer
    from liyab_b200.weights import write_random_model
    full = SIZES[args.size]
    cfg = dict(full, n_layer=args.layers or full["n_layer"])
    dtype_bytes = 2 if args.dtype == "bfloat16" else 4
    pk = peaks()
    with tempfile.TemporaryDirectory(prefix="liyab_b200_bench_") as tmp:
        model_dir = write_random_model(os.path.join(tmp, f"gpt2_{args.size}"), cfg, seed=0, dtype=args.dtype)
        big = max(64, args.batch)
        rep = Replayer(model_dir, args.dtype, max_tokens=big * 1024, max_requests=big, cuda_graphs=True, max_step_tokens=PREFILL_TOKENS)
        decode_point(rep, cfg, dtype_bytes, args.batch, 20, args.warmup, pk)          # loads and warms everything up
        clocks = ClockSampler()
        clocks.start()
        main_run = decode_point(rep, cfg, dtype_bytes, args.batch, args.steps, args.warmup, pk)
        clock_info = clocks.stop()
        line = {
            "metric": f"GPT-2 {args.size} decode tokens/s (batch {args.batch}, 512-token prompts, contexts 512-1024)",
            "value": round(main_run["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(main_run["ms_per_step"], 4), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16" if args.dtype == "bfloat16" else "fp32",
            "data": "synthetic: uniform random token ids, random-init weights (seed 0)",
            "config": {"model": f"gpt2-{args.size}", "n_layer": cfg["n_layer"], "n_layer_full": full["n_layer"], "n_embd": cfg["n_embd"],
                       "n_head": cfg["n_head"], "n_inner": cfg["n_inner"], "vocab_size": cfg["vocab_size"],
                       "n_positions": cfg["n_positions"], "global_batch": args.batch, "seq_len": 1024,
                       "prompt_len": PROMPT_LEN, "mean_context": round(main_run["mean_context"], 1), "page_size": 16,
                       "parallelism": "single-gpu", "l2": "each step reads %.0f MB of weights and cache > 126 MB L2" % (main_run["step_bytes"] / 1e6),
                       "peaks": pk["source"], "decode_path": detail(main_run)["path"], "host": "C++ library through its C interface"},
            "gpu_launches": main_run["kernel_launches"],
            "roofline": {"bound": "hbm", "achieved": round(main_run["achieved_gbs"], 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": round(main_run["frac"], 4)},
            "clocks": clock_info,
        }
        if not args.no_points:
            points, details = {}, {}
            for b in (1, 64):
                r = decode_point(rep, cfg, dtype_bytes, b, min(args.steps, 256), 3, pk)
                points[f"decode_b{b}"] = round(r["tok_s"], 1)
                details[f"decode_b{b}"] = detail(r)
            line["points"] = points
            line["points_detail"] = details
            line["prefill"] = prefill_point(rep, cfg, dtype_bytes, pk, args.dtype)
            rep.close()
            line["e2e"], line["same"] = e2e_run(model_dir, args.dtype, args.batch, args.steps)
        else:
            rep.close()
        if not args.no_points and not args.no_extra:
            steps = min(args.steps, 64)
            other = "float32" if args.dtype == "bfloat16" else "bfloat16"
            if other == "float32":
                folder = write_random_model(os.path.join(tmp, "gpt2_small_f32"), SIZES["small"], seed=0, dtype="float32")
                rep32 = Replayer(folder, "float32", max_tokens=8 * 1024, max_requests=8, cuda_graphs=True, max_step_tokens=PREFILL_TOKENS)
                line["fp32"] = {"model": "gpt2-small", "decode_b8": detail(decode_point(rep32, SIZES["small"], 4, 8, steps, 3, pk)),
                                "prefill": prefill_point(rep32, SIZES["small"], 4, pk, "float32"),
                                "note": "true 32-bit: FMA products, float32 cache; prefill frac against %g TFLOP/s nominal" % FP32_TFLOPS_NOMINAL}
                rep32.close()
            for size in ("medium", "xl"):
                if size == args.size:
                    continue
                block, folder = size_block(tmp, size, args.dtype, steps, pk)
                line[size] = block
                if size == "xl":
                    line["mixed_xl"] = mixed_run(folder, args.dtype, 64, 2048)
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
