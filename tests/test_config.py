"""Configuration and registry (CPU)."""
import json

import pytest

import vlrf_b200.models  # noqa: F401
from conftest import TINY_A, TINY_B
from vlrf_b200.config import ConfigError, GPT2Config, load_preset, preset_names, read_config_json
from vlrf_b200.registry import architecture_names, architecture_of, get_architecture, parse_config


def test_reads_every_key():
    for src in (TINY_A, TINY_B):
        cfg = GPT2Config.from_dict(src)
        for k, v in src.items():
            if k != "model_type":
                assert getattr(cfg, k) == v
    b = GPT2Config.from_dict(TINY_B)
    assert b.head_dim == 32 and b.inner_dim == 320 and b.activation == "gelu_erf"
    a = GPT2Config.from_dict(TINY_A)
    assert a.head_dim == 16 and a.activation == "gelu_tanh"


def test_n_inner_null_means_four_times_width():
    src = dict(TINY_A, n_inner=None)
    assert GPT2Config.from_dict(src).inner_dim == 4 * TINY_A["n_embd"]
    src.pop("n_inner")
    assert GPT2Config.from_dict(src).inner_dim == 4 * TINY_A["n_embd"]


def test_param_count_matches_the_tensors():
    from vlrf_b200.models.gpt2 import weight_spec
    for src in (TINY_A, TINY_B, load_preset("gpt2")):
        cfg = GPT2Config.from_dict(src)
        n = 0
        for s in weight_spec(cfg):
            k = 1
            for d in s.shape:
                k *= d
            n += k
        assert n == cfg.param_count()
    assert GPT2Config.from_dict(load_preset("gpt2")).param_count() == 124_439_808


@pytest.mark.parametrize("key", ["vocab_size", "n_positions", "n_embd", "n_layer", "n_head", "layer_norm_epsilon",
                                 "activation_function"])
def test_sizes_are_required_not_defaulted(key):
    src = dict(TINY_A)
    src.pop(key)
    with pytest.raises(ConfigError, match=key):
        GPT2Config.from_dict(src)


@pytest.mark.parametrize("patch,match", [
    (dict(n_embd=65), "multiple of n_head"),
    (dict(n_embd=120, n_head=12), "multiples of 16"),        # head size 10: refused here, not inside the first step
    (dict(n_embd=544, n_head=2), "multiples of 16 up to 256"),
    (dict(n_layer=0), "positive"),
    (dict(vocab_size=-1), "positive"),
    (dict(activation_function="relu"), "activation_function"),
    (dict(layer_norm_epsilon=0.0), "layer_norm_epsilon"),
    (dict(n_head="4"), "integer"),
    (dict(n_embd=64.5), "integer"),
    (dict(tie_word_embeddings=1), "true or false"),
    (dict(eos_token_id=512), "outside the vocabulary"),
    (dict(n_layer=None), "null"),
])
def test_bad_values_are_refused(patch, match):
    with pytest.raises(ConfigError, match=match):
        GPT2Config.from_dict(dict(TINY_A, **patch))


def test_registry_selects_by_model_type():
    assert "gpt2" in architecture_names()
    arch, cfg = parse_config(TINY_B)
    assert arch is get_architecture("gpt2") and isinstance(cfg, GPT2Config)
    with pytest.raises(ConfigError, match="registered: .*gpt2"):
        architecture_of({"model_type": "llama"})
    with pytest.raises(ConfigError, match="model_type"):
        architecture_of({})


def test_config_json_file_errors(tmp_path):
    with pytest.raises(ConfigError, match="cannot read"):
        read_config_json(tmp_path)
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        read_config_json(tmp_path)
    (tmp_path / "config.json").write_text("[1, 2]")
    with pytest.raises(ConfigError, match="JSON object"):
        read_config_json(tmp_path)
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    assert read_config_json(tmp_path)["n_embd"] == 64


def test_presets_are_data_and_parse():
    names = preset_names()
    assert {"gpt2", "gpt2-medium", "gpt2-xl", "tiny-a", "tiny-b"} <= set(names)
    for n in names:
        parse_config(load_preset(n))
    xl = GPT2Config.from_dict(load_preset("gpt2-xl"))
    assert (xl.n_layer, xl.n_embd, xl.n_head, xl.head_dim) == (48, 1600, 25, 64)


def test_round_trip_to_dict():
    cfg = GPT2Config.from_dict(TINY_B)
    assert GPT2Config.from_dict(cfg.to_dict()) == cfg
