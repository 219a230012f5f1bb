"""Nirotar without a GPU: config.json is read into typed fields, optional keys switch mechanisms off, refusals name the
key, the model's tensor list is what a checkpoint of this design holds, the parts carry the configuration's constants, and
the band-scaled rotation frequencies equal the plain implementation's."""
import json

import pytest
import torch

import plain_nirotar as plain
from nirotar_models import CONFIGS, make_model_dir, random_weights


def test_config_is_chosen_by_the_architecture_key_and_round_trips(tmp_path):
    from marin_b200.config import NirotarConfig, load_config

    cfg = load_config(make_model_dir(str(tmp_path / "a"), "A"))
    assert isinstance(cfg, NirotarConfig)
    assert (cfg.vocab_size, cfg.hidden_size, cfg.norm_eps) == (83, 48, 1e-5)
    assert [layer.type for layer in cfg.layers] == ["latent_attention", "attention", "latent_attention", "attention"]
    assert [layer.mixer.get("kv_from") for layer in cfg.layers] == [None, None, 0, None]
    assert cfg.layers[1].mixer["mask"] == {"size": 9} and cfg.layers[3].mixer["mask"] is None and cfg.layers[3].mixer["rot"] is None
    assert cfg.layers[1].mlp is None and cfg.layers[2].mlp["shared"] is None and cfg.layers[0].mlp["shared"] == {"ff": 40}
    again = NirotarConfig.from_dict(json.loads(json.dumps(cfg.to_json_dict())))
    assert again.to_json_dict() == cfg.to_json_dict() == CONFIGS["A"]


@pytest.mark.parametrize("damage, word", [
    (lambda c: c["layers"][0].__setitem__("type", "mamba"), "type"),
    (lambda c: c["layers"][1]["mixer"].pop("kv_heads"), "kv_heads"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("heads", 3), "kv heads"),
    (lambda c: c["layers"][1]["mixer"]["mask"].__setitem__("size", 0), "size"),
    (lambda c: c["layers"][1]["mixer"]["rot"].__setitem__("dims", 7), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"]["rot"]["scaling"].pop("low"), "low"),
    (lambda c: c["layers"][1]["mixer"]["rot"]["scaling"].__setitem__("high", 1.0), "high"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 8), "rot.dims"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("kv_from", 2), "kv_from"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("kv_from", 1), "kv_from"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("kv_rank", 24), "kv_rank"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "dense"), "mlp.kind"),
    (lambda c: c["layers"][0]["mlp"]["router"].__setitem__("top", 6), "top"),
    (lambda c: c["layers"][0]["mlp"]["shared"].pop("ff"), "ff"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c.__setitem__("width", "wide"), "width"),
])
def test_config_refusals_name_the_key(damage, word):
    from marin_b200.config import ConfigError, NirotarConfig

    raw = json.loads(json.dumps(CONFIGS["A"]))
    damage(raw)
    with pytest.raises(ConfigError, match=word):
        NirotarConfig.from_dict(raw)


@pytest.mark.parametrize("name", list(CONFIGS))
def test_the_models_tensor_list_is_the_checkpoints(tmp_path, name):
    from marin_b200.config import load_config
    from marin_b200.engine import build_model
    from marin_b200.weights import WeightError, load_tensors

    d = make_model_dir(str(tmp_path / "m"), name)
    weights = random_weights(CONFIGS[name], 3)
    model = build_model(load_config(d))
    specs = {s.name: tuple(s.shape) for s in model.tensor_specs()}
    assert specs == {k: tuple(v.shape) for k, v in weights.items()}
    loaded = load_tensors(d, model.tensor_specs(), model.spec.ignorable)
    tables = [k for k in loaded if k.endswith(".table")]
    assert tables and all(loaded[k].dtype == torch.int32 and torch.equal(loaded[k], weights[k]) for k in tables)
    # a layer that reads another's latent brings no down-projection of its own: one in the file is an error that names it
    if any(layer["mixer"].get("kv_from") is not None for layer in CONFIGS[name]["layers"]):
        from nirotar_models import write_model

        i = next(i for i, layer in enumerate(CONFIGS[name]["layers"]) if layer["mixer"].get("kv_from") is not None)
        extra = dict(weights)
        extra[f"l{i}.mix.dkv"] = torch.zeros(4, 4, dtype=torch.bfloat16)
        with pytest.raises(WeightError, match=f"l{i}.mix.dkv"):
            load_tensors(write_model(str(tmp_path / "x"), CONFIGS[name], extra), model.tensor_specs(), model.spec.ignorable)


def test_the_schedule_and_the_cache_needs_follow_the_layers():
    from marin_b200.config import NirotarConfig
    from marin_b200.engine import build_model
    from marin_b200.parts.mixer import PagedKV

    model = build_model(NirotarConfig.from_dict(CONFIGS["B"]))
    assert [e.cache_of for e in model.spec.schedule] == [None, None, 1, None, None]
    needs = model.cache_needs()
    assert needs[0] == PagedKV(1, 64, 70, 64) and needs[3] == PagedKV(2, 32, 16, 48) and needs[2] is None
    # a latent layer keeps one row per position, its values inside it: no value pages
    assert needs[1] == PagedKV(1, 80, None, 64, values_in_keys=True) and needs[4] == PagedKV(1, 128, None, 112, values_in_keys=True)
    assert needs[1].bytes_per_token(torch.bfloat16) == 80 * 2
    mix = [b.mixer for b in model.blocks]
    assert mix[0].learned_sink and mix[0].window == 70 and mix[0].position.interleaved and mix[0].qk_norm is None and not mix[0].bias
    assert mix[2].own_latent is False and mix[1].own_latent and "l2.mix.dkv" not in {s.name for s in mix[2].tensor_specs()}
    ff = model.blocks[0].feedforward
    assert (ff.routing, ff.activation, ff.weight_on, ff.top, ff.experts) == ("table", "relu2", "output", 2, 8) and ff.shared.intermediate == 128
    assert model.blocks[3].feedforward.shared is None and model.blocks[2].feedforward is None
    assert model.capturable()


def test_random_weights_of_the_package_give_a_usable_expert_table(tmp_path):
    from marin_b200.config import NirotarConfig
    from marin_b200.weights import write_random_model

    d = write_random_model(str(tmp_path / "r"), NirotarConfig.from_dict(CONFIGS["B"]), seed=5)
    w = plain.read_weights(d)
    table = w["l3.mlp.table"]
    assert table.dtype == torch.int32 and tuple(table.shape) == (160, 3) and int(table.min()) >= 0 and int(table.max()) < 6
    assert all(len(set(row.tolist())) == 3 for row in table)


@pytest.mark.parametrize("rot", [
    {"base": 50.0, "dims": 8, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 32}},
    {"base": 10000.0, "dims": 64, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}},
    {"base": 500000.0, "dims": 128, "scaling": {"factor": 32.0, "low": 2.0, "high": 5.0, "original": 8192}},
    {"base": 7.0, "dims": 6},
])
def test_band_scaled_frequencies(rot):
    """Fast pairs keep their frequency, slow ones are divided by the factor, those between are blended; all three bands occur."""
    from marin_b200.models.nirotar import _position
    from marin_b200.parts import lookup

    spec = _position(dict(rot, scaling=rot.get("scaling")), rot["dims"])
    part = lookup("position", spec.kind)(**spec.params)
    assert part.interleaved and part.rotary_dim == rot["dims"]
    want = plain.pair_frequencies(rot)
    if rot.get("scaling"):
        got = torch.tensor(part.frequencies(), dtype=torch.float64)
        torch.testing.assert_close(got, want, rtol=1e-12, atol=0)
        plain_f = torch.tensor([rot["base"] ** (-2.0 * i / rot["dims"]) for i in range(rot["dims"] // 2)], dtype=torch.float64)
        ratio = want / plain_f
        assert float(ratio.max()) == 1.0 and abs(float(ratio.min()) - 1.0 / rot["scaling"]["factor"]) < 1e-12
        assert rot["dims"] < 16 or bool(((ratio < 1.0) & (ratio > 1.0 / rot["scaling"]["factor"] + 1e-9)).any())
    else:
        assert spec.kind == "rope"


def test_which_prompt_kernel_a_head_layout_gets():
    """The tcgen05 prompt kernel takes keys and values of 64 or 128 alike, or page rows of 64 to 192 numbers whose first 64 or
    128 are the values; a latent layer asks for the kernels of its own layout and a name tells the layouts apart."""
    from marin_b200.kernels import build, ops

    assert ops.tc_sink_attention_supported(64, 64) and ops.tc_sink_attention_supported(128, 128)
    assert not ops.tc_sink_attention_supported(128, 64) and not ops.tc_sink_attention_supported(96, 96)
    for d, dv, ok in ((160, 128, True), (80, 64, True), (192, 128, True), (64, 64, True), (128, 96, False), (208, 128, False),
                      (72, 64, False), (112, 48, False), (256, 128, False)):
        assert ops.tc_sink_attention_supported(d, dv, True) == ok, (d, dv)
    jobs = ops.sink_attention_jobs(torch.bfloat16, 12, 1, 160, 128, values_in_keys=True)
    assert build.attention_tc_name(160, 12, 128, True) in jobs and jobs[build.attention_tc_name(160, 12, 128, True)][1][-1] == "V_IN_K"
    assert build.attention_tc_name(128, 4) == "mb_attention_tc_d128_g4" and build.attention_tc_name(128, 4) not in jobs
    assert not any("attention_tc" in n for n in ops.sink_attention_jobs(torch.bfloat16, 4, 1, 128, 96, values_in_keys=True))
    assert not any("attention_tc" in n for n in ops.sink_attention_jobs(torch.float32, 12, 1, 160, 128, values_in_keys=True))


def test_single_token_attention_is_split_into_whole_waves():
    """The chunks cover every key a token sees, a chunk is a multiple of 64 keys, and the CTAs of all chunks never leave a
    few for a wave of their own when fewer chunks fill one wave."""
    from marin_b200.kernels import ops

    places = ops.SINK_DECODE_CTAS_PER_SM * ops.SM_COUNT
    for requests, H, K, d, dv, span, window, shared in [(64, 32, 1, 160, 128, 4160, 0, True), (8, 32, 1, 160, 128, 4160, 0, True),
                                                       (8, 32, 8, 128, 128, 4160, 0, False), (1, 32, 8, 128, 128, 70000, 0, False),
                                                       (3, 12, 1, 32, 32, 500, 40, False), (64, 32, 8, 128, 128, 4160, 1024, False),
                                                       (2, 4, 2, 64, 64, 20, 0, False), (5, 6, 2, 64, 64, 129, 0, False)]:
        plan = ops.sink_decode_plan(torch.bfloat16, requests, H, K, d, dv, span, window, 0, shared)
        seen = min(span, window) if window else span
        assert plan.split % 64 == 0 and plan.split * plan.chunks >= seen + 63 and plan.split * (plan.chunks - 1) < seen + 63
        assert plan.chunks <= 1024 and (plan.split >= 128 or seen + 63 <= 128)
        ctas = requests * (H // ops.sink_group(H, K, shared)) * plan.chunks
        per_chunk = ctas // plan.chunks
        # more than a wave only if one chunk's CTAs alone exceed it, or the waves are full ones
        assert ctas <= places or per_chunk > places or ctas % places == 0 or plan.chunks == 1 or ctas / places > 1.5, (requests, H, K, plan.chunks)
    assert ops.sink_decode_plan(torch.bfloat16, 64, 32, 1, 160, 128, 4160, 0, 0, True).chunks == 4      # 512 CTAs in one wave, not 640 in two
    assert ops.sink_decode_plan(torch.float32, 8, 32, 8, 128, 128, 4160, 0, 0) is None                  # the plain kernel needs no plan
