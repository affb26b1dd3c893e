"""Revudra's configuration, model description, checkpoint map and cache needs, without a GPU."""
from __future__ import annotations

import copy

import numpy as np
import pytest

from liyab_b200.config import describe_config, slot, supported_architectures
from liyab_b200.status import LiyabError
from revudra_models import CONFIG_A, CONFIG_C, CONFIG_D, random_weights, write_model


def test_registered_and_found_by_its_own_key():
    assert "revudra" in supported_architectures()
    assert describe_config(CONFIG_A)["architecture"] == "revudra"


def test_every_size_and_constant_comes_from_the_file():
    d = describe_config(CONFIG_A)["spec"]
    assert d["embedding"] == {"vocab_size": 160, "size": 96, "scale": 0.7}
    assert not d["head"]["tied"] and d["head"]["logit_scale"] == 1.5 and d["position"]["kind"] == "none"
    assert d["final_norm"] == {"kind": "rms_norm", "size": 96, "groups": 1, "eps": 1e-5}
    assert len(d["layers"]) == 7 and [(e["layer"], e["cache"]) for e in d["run_order"]] == [(i, i) for i in range(7)]
    blends = []
    for layer, raw in zip(d["layers"], CONFIG_A["layers"]):
        assert layer["arrangement"] == "sublayer_norm" and layer["options"]["residual_scale"] == 0.6
        names = [s["name"] for s in layer["slots"]]
        assert names == (["mixer", "mixer_norm", "feed_forward", "ff_norm"] if raw["mlp"] else ["mixer", "mixer_norm"])
        assert slot(layer, "mixer_norm") == {"kind": "rms_norm", "size": 96, "groups": 1, "eps": 1e-5}
        m, r = slot(layer, "mixer"), raw["mixer"]
        if raw["type"] == "attention":
            assert m["kind"] == "gated_attention" and m["qk_norm"] and m["qk_norm_over"] == "projection" and m["sink"] and m["gate"] == "sigmoid" and not m["bias"]
            assert (m["n_head"], m["n_kv_head"], m["dim"], m["vdim"], m["scale"], m["window"]) == (r["heads"], r["kv_heads"], r["dim"], r["vdim"], r["scale"], r["mask"]["size"])
            assert (m["rot_dims"], m["rot_base"]) == (r["rot"]["dims"], r["rot"]["base"]) and m["eps"] == 1e-5
            blends.append(m["value_blend"])
        elif raw["type"] == "lightning":
            assert m["kind"] == "matrix_memory" and m["recurrence"] == "fixed_decay" and m["decay"] == r["decay"] and m["qkv_activation"] == "silu"
            assert m["norm_over"] == "all" and m["norm_gain"] and m["gate"] == "sigmoid" and m["rot_dims"] == 0
            assert (m["n_head"], m["dim"], m["vdim"]) == (r["heads"], r["dim"], r["vdim"])
        else:
            assert m["kind"] == "latent_attention" and m["rot_layout"] == "interleaved" and m["sink"] and m["head_gate"] and m["window"] == 0 and m["own_latent"]
            assert (m["n_head"], m["dim"], m["rot_dim"], m["rot_dims"], m["vdim"], m["kv_rank"], m["q_rank"], m["scale"], m["rot_base"]) == (
                r["heads"], r["dim"], r["rot_dim"], r["rot"]["dims"], r["vdim"], r["kv_rank"], r["q_rank"], r["scale"], r["rot"]["base"])
        if raw["mlp"] and raw["mlp"]["kind"] == "moe":
            ff = slot(layer, "feed_forward")
            assert ff["kind"] == "routed" and ff["route"] == "table" and ff["vocab"] == 160 and ff["activation"] == "silu" and ff["weight_on"] == "output"
            assert (ff["experts"], ff["top"], ff["inner"]) == (raw["mlp"]["router"]["experts"], raw["mlp"]["router"]["top"], raw["mlp"]["expert"]["ff"])
        elif raw["mlp"]:
            ff = slot(layer, "feed_forward")
            assert ff["kind"] == "dense" and ff["inner"] == raw["mlp"]["ff"] and ff["activation"] == "relu2" and not ff["bias"]
    # The first layer that blends values is their source, the later ones blend with it.
    assert blends == ["source", "blend", "blend"]
    # A lone such layer has no one to give its values to: nothing is blended, and its weight is a tensor without a use.
    c = describe_config(CONFIG_C)
    assert slot(c["spec"]["layers"][1], "mixer")["value_blend"] == "none"
    assert any("l1" in t and "vmix" in t for t in c["ignored_tensors"])


def test_checkpoint_map_names_the_files_tensors():
    d = describe_config(CONFIG_A)
    ck = d["checkpoint"]
    names = lambda path: [s["name"] for s in ck[path]["sources"]]
    assert names("layers.1.mixer.proj.weight") == ["l1.mix.q", "l1.mix.k", "l1.mix.v", "l1.mix.g"]
    assert names("layers.0.mixer.proj.weight") == ["l0.mix.q", "l0.mix.k", "l0.mix.v", "l0.mix.g"]
    assert names("layers.2.mixer.proj.weight") == ["l2.mix.dq", "l2.mix.dkv", "l2.mix.g"]
    assert names("layers.2.mixer.q_up.weight") == ["l2.mix.uq"] and names("layers.2.mixer.q_norm.weight") == ["l2.mix.dq.norm"]
    assert names("layers.3.mixer.blend") == ["l3.mix.vmix"] and ck["layers.3.mixer.blend"]["repeat"] == 1
    assert "layers.1.mixer.blend" not in ck and any("l1" in t and "vmix" in t for t in d["ignored_tensors"])
    assert names("layers.0.feed_forward.table") == ["l0.mlp.table"] and ck["layers.0.feed_forward.table"]["kind"] == "index"
    assert names("layers.0.feed_forward.experts.gate_up.weight")[:4] == ["l0.mlp.e0.gate", "l0.mlp.e0.up", "l0.mlp.e1.gate", "l0.mlp.e1.up"]
    assert "layers.3.ff_norm.weight" not in ck and any("l3" in t and "norm2" in t for t in d["ignored_tensors"])


def test_weights_load_as_the_engine_holds_them(tmp_path):
    from liyab_b200.weights import load_parameters
    weights = random_weights(CONFIG_D, 3)
    path = write_model(str(tmp_path / "d"), CONFIG_D, weights)
    for dtype in ("float32", "bfloat16"):
        p = load_parameters(path, dtype)
        assert p["layers.0.feed_forward.table"].dtype == np.int32 and p["layers.0.feed_forward.table"].shape == (64, 1)
        assert p["layers.3.mixer.blend"].shape == (1,) and p["layers.3.mixer.blend"].dtype == np.float32
        assert np.float32(weights["l3.mix.vmix"]) == p["layers.3.mixer.blend"][0]
        assert p["layers.2.mixer.proj.weight"].shape == (1 + 3 + 1, 48)
    # A tensor the design does not have is named in the refusal.
    weights["l1.mix.sink"] = weights["l0.mix.sink"]
    path = write_model(str(tmp_path / "bad"), CONFIG_D, weights)
    with pytest.raises(LiyabError, match="l1.mix.sink"):
        load_parameters(path, "float32")


@pytest.mark.parametrize("edit, message", [
    (lambda c: c["layers"][0].update(type="retention"), "type"),
    (lambda c: c["layers"][0]["mixer"].pop("decay"), "decay"),
    (lambda c: c["layers"][0]["mixer"].update(decay=[0.5, 0.5]), "decay"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=14), "rot.dims"),
    (lambda c: c["layers"][2]["mixer"].pop("q_rank"), "q_rank"),
    (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=8), "rot.dims"),
    (lambda c: c["layers"][3]["mixer"].update(vdim=6), "v_mix"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=7), "top"),
    (lambda c: c["layers"][1]["mlp"].update(kind="gated"), "kind"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["norm"].pop("eps"), "eps"),
])
def test_refusals_name_the_key(edit, message):
    config = copy.deepcopy(CONFIG_A)
    edit(config)
    with pytest.raises(LiyabError, match=message):
        describe_config(config)


def test_cache_units_of_the_three_mixers():
    """The units the design's mixers ask for, side by side in one manager: pages under a window leave when the window has passed them,
    the latent rows (one plane, no window) stay, the memories' slots are zeroed state that the next request takes over."""
    from liyab_b200.cache import CacheManager, KvNeed, StateNeed
    needs = {1: KvNeed(n_kv_head=2, head_dim=12, window=20), 2: KvNeed(n_kv_head=1, head_dim=30, window=0, planes=1)}
    cache = CacheManager(needs, {0: StateNeed((3 * (12 * 20 + 12 + 1),), "float32")}, page_size=16, num_pages=12, max_requests=2)
    cache.open("a")
    cache.reserve("a", 100)
    cache.commit("a", 100)
    in_use = cache.pages_in_use()
    assert sorted(in_use.values()) == [2, 7]        # the window keeps positions 81..99, the latent rows all hundred
    cache.open("b")
    assert cache.state_slots_free() == 0
    cache.close("a")
    cache.open("c")
    cache.close("b")
    cache.close("c")
    assert cache.state_slots_free() == 2 and sum(cache.pages_in_use().values()) == 0
    cache.check()
