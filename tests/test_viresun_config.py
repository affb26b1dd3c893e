"""Viresun's configuration, model description, run order, checkpoint map and cache needs, without a GPU."""
from __future__ import annotations

import copy

import pytest

from liyab_b200.config import describe_config, slot, supported_architectures
from liyab_b200.status import LiyabError
from viresun_models import CONFIG_A, CONFIG_C, CONFIG_D


def test_registered_and_found_by_its_own_key():
    assert "viresun" in supported_architectures()
    assert describe_config(CONFIG_A)["architecture"] == "viresun"


def own_layers(config):
    return [l for l in config["layers"] if l.get("weights_of") is None]


def test_every_size_and_constant_comes_from_the_file():
    d = describe_config(CONFIG_A)["spec"]
    assert d["embedding"]["vocab_size"] == 160 and d["embedding"]["size"] == 96 and not d["head"]["tied"]
    pos = d["position"]
    assert pos["kind"] == "sinusoid" and pos["size"] == 96 and pos["base"] == 10000.0 and pos["norm"] and pos["eps"] == 1e-5
    assert d["final_norm"] == {"kind": "rms_norm", "size": 96, "groups": 1, "eps": 1e-5}
    assert len(d["layers"]) == 5                 # two of the seven run on another layer's weights
    for layer, raw in zip(d["layers"], own_layers(CONFIG_A)):
        assert layer["arrangement"] == "pre_norm"
        names = [s["name"] for s in layer["slots"]]
        assert names == (["mixer_norm", "mixer", "ff_norm", "feed_forward"] if raw["mlp"] else ["mixer_norm", "mixer"])
        m, r = slot(layer, "mixer"), raw["mixer"]
        if raw["type"] == "attention":
            assert m["kind"] == "gated_attention" and m["qk_norm"] and not m["qk_gain"] and not m["bias"] and m["gate"] == "none" and m["distance_bias"]
            assert (m["n_head"], m["n_kv_head"], m["dim"], m["vdim"], m["scale"], m["window"]) == (
                r["heads"], r["kv_heads"], r["dim"], r["vdim"], r["scale"], r["mask"]["size"])
            assert (m["q_temp_coef"], m["q_temp_every"]) == (r["q_temp"]["coef"], r["q_temp"]["every"]) and m["eps"] == 1e-5
        else:
            assert m["kind"] == "state_space" and m["eps"] == 1e-5
            assert (m["n_head"], m["vdim"], m["n_state"], m["groups"], m["taps"], m["norm_groups"]) == (
                r["heads"], r["vdim"], r["state"], r["groups"], r["conv"], r["norm_groups"])
        if raw["mlp"] and raw["mlp"]["kind"] == "moe":
            ff = slot(layer, "feed_forward")
            assert ff["kind"] == "routed" and (ff["experts"], ff["top"], ff["inner"]) == (raw["mlp"]["router"]["experts"], raw["mlp"]["router"]["top"], raw["mlp"]["expert"]["ff"])
            assert ff["activation"] == "capped" and ff["gate_limit"] == raw["mlp"]["expert"]["limit"] and ff["gate_alpha"] == 1.702
            assert ff["score"] == "softmax" and ff["renormalise"] and ff["weight_on"] == "output" and ff["router_bias"] and ff["shared_inner"] == 0
        elif raw["mlp"]:
            ff = slot(layer, "feed_forward")
            assert ff["kind"] == "gated" and ff["inner"] == raw["mlp"]["ff"] and ff["activation"] == "relu"
    # A layer without a mask sees every earlier key; one without a temperature has none.
    c = describe_config(CONFIG_C)["spec"]
    free = slot(c["layers"][3], "mixer")
    assert free["window"] == 0 and free["q_temp_every"] == 0 and free["q_temp_coef"] == 0.0


def test_a_layer_on_another_layers_weights_is_a_run_with_a_cache_of_its_own():
    d = describe_config(CONFIG_A)
    order = [(e["layer"], e["cache"]) for e in d["spec"]["run_order"]]
    assert order == [(0, 0), (1, 1), (2, 2), (1, 3), (3, 4), (0, 5), (4, 6)]
    ck = d["checkpoint"]
    assert "layers.4.mixer.proj.weight" in ck and "layers.5.mixer.proj.weight" not in ck
    # The fifth model layer is the file's l6: names follow the file's layer numbers, paths the layers with tensors.
    assert ck["layers.4.mixer.proj.weight"]["sources"][0]["name"] == "l6.mix.in"
    # A chain of references ends at the layer that has tensors.
    c = copy.deepcopy(CONFIG_D)
    c["layers"].append(dict(c["layers"][3], weights_of=3))
    assert [(e["layer"], e["cache"]) for e in describe_config(c)["spec"]["run_order"]] == [(0, 0), (1, 1), (2, 2), (0, 3), (0, 4)]


def test_checkpoint_map_joins_the_file_tensors():
    ck = describe_config(CONFIG_A)["checkpoint"]
    proj = ck["layers.0.mixer.proj.weight"]
    assert [s["name"] for s in proj["sources"]] == ["l0.mix.q", "l0.mix.k", "l0.mix.v"]
    assert [s["shape"] for s in proj["sources"]] == [[48, 96], [24, 96], [40, 96]]
    assert [s["name"] for s in ck["layers.0.mixer.distance"]["sources"]] == ["l0.mix.r1", "l0.mix.r2"]
    assert ck["layers.0.mixer_norm.weight"]["sources"][0] == {"name": "l0.norm1", "shape": []} and ck["layers.0.mixer_norm.weight"]["repeat"] == 96
    assert ck["position.norm.weight"]["sources"][0]["name"] == "embed.norm" and ck["final_norm.weight"]["sources"][0]["name"] == "final.norm"
    ss = {k.split("mixer.", 1)[1]: v["sources"][0] for k, v in ck.items() if k.startswith("layers.1.mixer.")}
    assert ss["proj.weight"] == {"name": "l1.mix.in", "shape": [48 + 48 + 40 + 4, 96]}
    assert ss["conv.weight"] == {"name": "l1.mix.conv", "shape": [88, 4]} and ss["conv.bias"] == {"name": "l1.mix.conv.b", "shape": [88]}
    assert ss["dt_bias"]["name"] == "l1.mix.dt_bias" and ss["a_log"]["name"] == "l1.mix.A_log" and ss["skip"]["name"] == "l1.mix.D"
    assert ss["norm.weight"] == {"name": "l1.mix.norm", "shape": [48]} and ss["out.weight"] == {"name": "l1.mix.o", "shape": [96, 48]}
    experts = ck["layers.0.feed_forward.experts.gate_up.weight"]
    assert [s["name"] for s in experts["sources"]][:4] == ["l0.mlp.e0.gate", "l0.mlp.e0.up", "l0.mlp.e1.gate", "l0.mlp.e1.up"] and len(experts["sources"]) == 12
    assert len(ck["layers.0.feed_forward.experts.down.weight"]["sources"]) == 6
    assert ck["layers.0.feed_forward.router.bias"]["sources"][0] == {"name": "l0.mlp.router.b", "shape": [6]}
    assert [s["name"] for s in ck["layers.1.feed_forward.gate_up.weight"]["sources"]] == ["l1.mlp.gate", "l1.mlp.up"]
    assert "layers.2.ff_norm.weight" not in ck


@pytest.mark.parametrize("damage, text", [
    (lambda c: c["layers"][0].__setitem__("type", "conv"), "attention, mamba2"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("kv_heads", 3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["q_temp"].__setitem__("every", 0), "every"),
    (lambda c: c["layers"][0]["mixer"]["mask"].__setitem__("size", 0), "size"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("groups", 3), "groups"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("norm_groups", 5), "norm_groups"),
    (lambda c: c["layers"][1]["mixer"].pop("state"), "state"),
    (lambda c: c["layers"][0]["mlp"]["router"].__setitem__("top", 7), "top"),
    (lambda c: c["layers"][0]["mlp"]["expert"].__setitem__("limit", 0.0), "limit"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "routed"), "dense, moe"),
    (lambda c: c["layers"][3].__setitem__("weights_of", 3), "itself"),
    (lambda c: c["layers"][3].__setitem__("weights_of", 9), "weights_of"),
    (lambda c: (c["layers"][0].__setitem__("weights_of", 5)), "circle"),
    (lambda c: c.pop("width"), "width"),
])
def test_bad_configurations_are_refused(damage, text):
    c = copy.deepcopy(CONFIG_A)
    damage(c)
    with pytest.raises(LiyabError) as e:
        describe_config(c)
    assert text in str(e.value)


def test_a_single_number_may_be_stored_without_a_shape_or_as_one_entry(tmp_path):
    """A norm's gain is one number for all coordinates; the file may hold it with the shape [] or [1], and the loader repeats it."""
    import numpy as np
    from liyab_b200.weights import load_parameters
    from viresun_models import random_weights, write_model
    weights = random_weights(CONFIG_D, 7)
    assert any(np.asarray(v).ndim == 0 for v in weights.values())
    as_lists = {k: (np.asarray(v).reshape(1) if np.asarray(v).ndim == 0 else v) for k, v in weights.items()}
    first = load_parameters(write_model(str(tmp_path / "plain"), CONFIG_D, weights))
    second = load_parameters(write_model(str(tmp_path / "lists"), CONFIG_D, as_lists))
    assert first.keys() == second.keys() and all(np.array_equal(first[k], second[k]) for k in first)
    gain = first["final_norm.weight"]
    assert gain.shape == (CONFIG_D["width"],) and np.all(gain == gain[0]) and gain[0] == np.float32(weights["final.norm"])
