"""Vogunex without a GPU: config.json is read into typed fields, optional keys switch mechanisms off, refusals name the key,
a layer that uses another's weights becomes a second run of that layer's block, the model's tensor list is what a checkpoint
of this design holds, and the cache manager gives a mixer that keeps several things a place for each."""
import json

import pytest
import torch

from vogunex_models import CONFIGS, make_model_dir, random_weights


def test_config_is_chosen_by_the_architecture_key_and_round_trips(tmp_path):
    from marin_b200.config import VogunexConfig, load_config

    cfg = load_config(make_model_dir(str(tmp_path / "a"), "A"))
    assert isinstance(cfg, VogunexConfig)
    assert (cfg.vocab_size, cfg.hidden_size, cfg.norm_eps, cfg.embedding_scale) == (77, 40, 1e-5, 3.0)
    assert [layer.type for layer in cfg.layers] == ["attention", "mamba2", "attention", "latent_attention", "mamba2", "latent_attention"]
    assert [layer.weights_of for layer in cfg.layers] == [None, None, 0, None, 1, 3]
    assert cfg.layers[0].mixer["mask"] == {"size": 9, "pool": 3} and cfg.layers[0].mixer["softcap"] == 5.0
    assert cfg.layers[0].mlp == {"kind": "dense", "ff": 56} and cfg.layers[3].mlp["shared"] is None
    again = VogunexConfig.from_dict(json.loads(json.dumps(cfg.to_json_dict())))
    assert again.to_json_dict() == cfg.to_json_dict() == CONFIGS["A"]
    edge = VogunexConfig.from_dict(CONFIGS["C"])
    assert edge.embedding_scale == 1.0 and edge.layers[0].weights_of == 2 and edge.layers[3].mixer["rot"] is None
    assert edge.layers[2].mixer["softcap"] is None and edge.layers[1].mlp is None


@pytest.mark.parametrize("damage, word", [
    (lambda c: c["layers"][0].__setitem__("type", "conv"), "type"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_heads"), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("heads", 3), "kv heads"),
    (lambda c: c["layers"][0]["mixer"]["mask"].__setitem__("size", 0), "size"),
    (lambda c: c["layers"][0]["mixer"]["mask"].__setitem__("pool", 0), "pool"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 7), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("softcap", -1.0), "softcap"),
    (lambda c: c["layers"][3]["mixer"].pop("q_rank"), "q_rank"),
    (lambda c: c["layers"][3]["mixer"]["rot"].__setitem__("dims", 4), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("groups", 2), "groups"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("norm_groups", 4), "norm_groups"),
    (lambda c: c["layers"][1]["mixer"].pop("conv"), "conv"),
    (lambda c: c["layers"][2].__setitem__("weights_of", 2), "weights_of"),
    (lambda c: c["layers"][2].__setitem__("weights_of", 4), "weights_of"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("vdim", 12), "differs"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "glu"), "mlp.kind"),
    (lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 6), "top"),
    (lambda c: c["layers"][1]["mlp"]["expert"].pop("limit"), "limit"),
    (lambda c: c["layers"][1]["mlp"]["shared"].pop("ff"), "ff"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c.__setitem__("width", "wide"), "width"),
])
def test_config_refusals_name_the_key(damage, word):
    from marin_b200.config import ConfigError, VogunexConfig

    raw = json.loads(json.dumps(CONFIGS["A"]))
    damage(raw)
    with pytest.raises(ConfigError, match=word):
        VogunexConfig.from_dict(raw)


@pytest.mark.parametrize("name", list(CONFIGS))
def test_the_models_tensor_list_is_the_checkpoints(tmp_path, name):
    from marin_b200.config import load_config
    from marin_b200.engine import build_model
    from marin_b200.weights import WeightError, load_tensors

    d = make_model_dir(str(tmp_path / name), name)
    model = build_model(load_config(d))
    want = random_weights(CONFIGS[name], 3)
    specs = {s.name: tuple(s.shape) for s in model.tensor_specs()}
    assert specs == {k: tuple(v.shape) for k, v in want.items()}
    loaded = load_tensors(d, model.tensor_specs(), model.spec.ignorable)
    assert set(loaded) == set(want)
    # a checkpoint that lacks a tensor, or brings one too many, is refused with their names
    from safetensors.torch import save_file
    import os

    broken = dict(want)
    gone = next(k for k in broken if k.endswith(".shift"))
    del broken[gone]
    broken["l0.mix.sink"] = torch.zeros(4, dtype=torch.bfloat16)
    save_file(broken, os.path.join(d, "model.safetensors"))
    with pytest.raises(WeightError) as err:
        load_tensors(d, model.tensor_specs(), model.spec.ignorable)
    assert gone in str(err.value) and "l0.mix.sink" in str(err.value)


def test_a_layer_with_anothers_weights_is_a_second_run_of_its_block():
    from marin_b200.config import VogunexConfig
    from marin_b200.models.vogunex import build_spec

    spec = build_spec(VogunexConfig.from_dict(CONFIGS["A"]))
    assert [layer.prefix for layer in spec.layers] == ["l0", "l1", "l3"]
    assert [e.layer for e in spec.schedule] == [0, 1, 0, 2, 1, 2] and all(e.cache_of is None for e in spec.schedule)
    later = build_spec(VogunexConfig.from_dict(CONFIGS["C"]))
    assert [layer.prefix for layer in later.layers] == ["l1", "l2", "l3", "l4", "l5", "l6"]
    assert [e.layer for e in later.schedule] == [1, 0, 1, 2, 3, 4, 5]
    mixer = spec.layers[0].mixer
    assert mixer.kind == "token_shifted" and mixer.params["tensor"] == "l0.shift" and mixer.params["inner"].kind == "pooled_attention"
    inner = mixer.params["inner"].params
    assert (inner["window"], inner["pool"], inner["softcap"], inner["talk"], inner["bias"]) == (9, 3, 5.0, True, True)
    experts = spec.layers[1].feedforward.params
    assert (experts["activation"], experts["act_limit"], experts["shared_limit"], experts["score"], experts["renormalize"]) == ("glu_capped", 0.8, 1.5, "softmax", True)


def test_every_run_gets_places_for_all_its_mixer_keeps():
    from marin_b200.cache import CacheManager
    from marin_b200.config import VogunexConfig
    from marin_b200.engine import build_model
    from marin_b200.parts.mixer import PagedKV, StateNeed

    model = build_model(VogunexConfig.from_dict(CONFIGS["A"]))
    needs = model.cache_needs()
    assert all(isinstance(n, tuple) and isinstance(n[0], StateNeed) and n[0].shape == (40,) for n in needs)
    assert needs[0][1] == PagedKV(2, 12, None, 10, pooled=3, pooled_window=9) and needs[3][1] == PagedKV(1, 26, 7, 20, values_in_keys=True)
    assert needs[1][1] == (StateNeed((3, 6, 10)), StateNeed((2, 3 * 10 + 12)))
    m = CacheManager(needs, [None] * len(needs), 4, 10, 2)
    assert [g.entries for g in m.groups] == [[0, 2], [3, 5]]            # the two runs of a block keep pages of their own
    assert m.place[0] == (("state", (0, 0)), (0, 0)) and m.place[2] == (("state", (2, 0)), (0, 1))
    assert m.place[4] == (("state", (4, 0)), (("state", (4, 1, 0)), ("state", (4, 1, 1))))
    assert len(m.state_needs) == 6 + 2 * 2
    # a page of four positions holds up to two pooled rows of a pool of three
    assert needs[0][1].pooled_rows(4) == 2 and needs[0][1].bytes_per_token(torch.bfloat16, 4) > needs[0][1].bytes_per_token(torch.bfloat16)
    with pytest.raises(ValueError):
        PagedKV(2, 12, 9, 10, pooled=3)
    # one decoded token of a long sequence reads the window and a third of what lies before it
    assert needs[0][1].bytes_read(309, torch.bfloat16) == (9 + 100) * needs[0][1].bytes_per_token(torch.bfloat16)
    # requests come and go: reserve, commit, release leave nothing behind
    a = m.admit("a")
    m.reserve("a", 12)
    m.commit("a", 12)
    assert [len([p for p in t if p >= 0]) for t in a.pages] == [3, 2]  # the pooled group keeps every page, the window of 7 dropped one
    m.release("a")
    m.check()
    assert all(g.pool.num_held == 0 for g in m.groups)
