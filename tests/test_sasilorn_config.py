"""The Sasilorn architecture without a GPU: configuration, schedule, tensor names, the plain implementation."""

import copy
import json

import pytest
import torch

import plain_sasilorn
from sasilorn_cases import CASES, one_layer
from dryft_flash_infer_b200.config import ConfigError, SasilornConfig, architecture_named, config_from_dict, load_config
from dryft_flash_infer_b200.engine.model import DecoderModel


def spec_of(config: dict):
    cfg = config_from_dict(config)
    return architecture_named(cfg.architecture).build(cfg)


@pytest.mark.parametrize("name", sorted(CASES))
def test_the_model_expects_the_tensors_the_plain_implementation_names(name):
    config = CASES[name]
    tensors = plain_sasilorn.random_tensors(config, 0)
    cfg = config_from_dict(config).with_tensor_shapes({k: tuple(v.shape) for k, v in tensors.items()})
    model = DecoderModel(architecture_named(cfg.architecture).build(cfg))
    expected = {e.name: tuple(e.decl.shape) for e in model.expected_tensors()}
    assert expected == {k: tuple(v.shape) for k, v in tensors.items()}


def test_a_layer_that_runs_anothers_tensors_is_a_second_entry_of_the_schedule():
    spec = spec_of(CASES["A"])
    assert len(spec.layers) == 3 and len(spec.schedule) == 4
    assert [e.layer for e in spec.schedule] == [0, 1, 0, 2]
    assert len({e.cache for e in spec.schedule}) == 4 and all(e.writes_cache for e in spec.schedule)
    model = DecoderModel(spec)
    kv, state = model.cache_needs()
    assert sorted(kv) == [0, 2] and sorted(state) == [0, 1, 2, 3]
    assert kv[0].head_dim == 16 and kv[0].v_head_dim == 24
    assert spec.residual_float32 and spec.layers[1].feed_forward is None


def test_sizes_come_from_the_tensors_where_the_file_is_silent():
    config = copy.deepcopy(CASES["B"])
    tensors = plain_sasilorn.random_tensors(config, 0)
    cfg = config_from_dict(config).with_tensor_shapes({k: tuple(v.shape) for k, v in tensors.items()})
    assert cfg.layers[0]["mixer"]["rank"] == tensors["l0.mix.w1"].shape[0]
    assert cfg.layers[2]["mixer"]["rank"] == tensors["l0.mix.w1"].shape[0]      # the layer that borrows layer 0
    assert cfg.layers[1]["mixer"]["right"]["rank"] == tensors["l1.mix.right.a1"].shape[0]
    assert cfg.layers[0]["mixer"]["vdim"] == 24


def test_save_and_load(tmp_path):
    cfg = config_from_dict(CASES["A"])
    cfg.save(tmp_path)
    raw = json.loads((tmp_path / "config.json").read_text())
    assert raw["architecture"] == "Sasilorn" and raw["width"] == 64
    assert load_config(tmp_path) == cfg and isinstance(cfg, SasilornConfig)


@pytest.mark.parametrize("change, word", [
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(tau=0.0), "tau"),
    (lambda c: c["layers"][0]["mlp"].update(kind="routed"), "dense"),
    (lambda c: c["layers"][2].update(weights_of=1), "another kind"),
    (lambda c: c["layers"][2].update(weights_of=2), "weights_of"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c["layers"][1]["mixer"].pop("dim"), "dim"),
])
def test_a_configuration_that_cannot_be_used_is_refused_by_name(change, word):
    config = copy.deepcopy(CASES["A"])
    change(config)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(config)


def test_the_plain_linear_attention_equals_its_sum_over_earlier_tokens():
    """``o_t = sum_(s<=t) (q_t . (prod_(s<r<=t) a_r) k_s) v_s``: the recurrence written out."""
    torch.manual_seed(0)
    sizes = {"heads": 2, "dim": 6, "vdim": 5, "tau": 3.0}
    T, width, rank = 9, 12, 4
    h = torch.randn(T, width, dtype=torch.float64)
    p = {"q": torch.randn(12, width), "k": torch.randn(12, width), "v": torch.randn(10, width), "g": torch.randn(10, width),
         "a1": torch.randn(rank, width), "a2": torch.randn(12, rank), "a2.b": torch.randn(12), "norm": torch.rand(5) + 0.5,
         "o": torch.eye(10)}
    p = {k: v.double() for k, v in p.items()}
    got = plain_sasilorn.gated_linear_attention(h, p, sizes, 1e-5)
    q = (h @ p["q"].T).view(T, 2, 6) * 6 ** -0.5
    k, v = (h @ p["k"].T).view(T, 2, 6), (h @ p["v"].T).view(T, 2, 5)
    a = torch.sigmoid(((h @ p["a1"].T) @ p["a2"].T + p["a2.b"]).view(T, 2, 6)) ** (1 / 3.0)
    out = torch.zeros(T, 2, 5, dtype=torch.float64)
    for t in range(T):
        for s in range(t + 1):
            through = a[s + 1: t + 1].prod(0)
            out[t] += ((q[t] * through * k[s]).sum(-1, keepdim=True)) * v[s]
    out = plain_sasilorn.unit_rms(out, 1e-5) * p["norm"]
    want = out.reshape(T, 10) * torch.nn.functional.silu(h @ p["g"].T)
    assert torch.allclose(got, want, atol=1e-10)


def test_the_plain_time_mixing_reads_the_token_itself_only_through_the_bonus():
    torch.manual_seed(1)
    config = one_layer("wkv")
    tensors = {k: v.double() for k, v in plain_sasilorn.random_tensors(config, 3, torch.float32).items()}
    p = {k[len("l0.mix."):]: v for k, v in tensors.items() if k.startswith("l0.mix.")}
    h = torch.randn(1, 48, dtype=torch.float64)
    one = plain_sasilorn.wkv_mixer(h, p, config["layers"][0]["mixer"], 1e-5)
    p0 = dict(p, u=torch.zeros_like(p["u"]))
    assert one.abs().max() > 1e-3
    assert plain_sasilorn.wkv_mixer(h, p0, config["layers"][0]["mixer"], 1e-5).abs().max() < 1e-12
    # a second token reads the first through the state, bonus or not
    two = plain_sasilorn.wkv_mixer(torch.cat([h, h * 0.5]), p0, config["layers"][0]["mixer"], 1e-5)
    assert two[1].abs().max() > 1e-3


def test_random_model_through_the_command_line(tmp_path):
    from dryft_flash_infer_b200.__main__ import main
    from dryft_flash_infer_b200.weights.safetensors_io import ModelFiles

    config = copy.deepcopy(CASES["C"])
    config["layers"][0]["mixer"]["rank"] = 12
    (tmp_path / "c.json").write_text(json.dumps(config))
    assert main(["random-model", "--config", str(tmp_path / "c.json"), "--seed", "5", "--out", str(tmp_path / "m")]) == 0
    files = ModelFiles(tmp_path / "m")
    assert files.info("l0.mix.w1")[1] == [12, 44] or tuple(files.info("l0.mix.w1")[1]) == (12, 44)
    assert tuple(files.info("l1.norm1.alpha")[1]) == ()
    assert "l1.mlp.up" not in files.names() and "l0.mlp.up" in files.names()
