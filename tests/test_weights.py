"""safetensors reading, the one error that lists every mismatch, random-weights mode (CPU)."""
import json
import struct

import pytest
import torch

import vlrf_b200.models  # noqa: F401
from conftest import TINY_A, TINY_B
from vlrf_b200.weights import (WeightError, open_model_dir, read_safetensors, write_random_model,
                               write_safetensors)
from vlrf_b200.weights.spec import TensorSpec, check_tensors, place


def test_round_trip_keeps_dtypes(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32).reshape(2, 3),
         "d": torch.randn(2, 2).to(torch.float16)}
    write_safetensors(tmp_path / "x.safetensors", t)
    back = read_safetensors(tmp_path / "x.safetensors")
    assert set(back) == set(t)
    for k in t:
        assert back[k].dtype == t[k].dtype and torch.equal(back[k], t[k])


def test_reader_matches_an_independent_reader(tmp_path, model_dirs):
    import plain_gpt2
    mine = read_safetensors(model_dirs["tiny_b"] / "model.safetensors")
    theirs = plain_gpt2.read_safetensors(model_dirs["tiny_b"] / "model.safetensors")
    assert set(mine) == set(theirs)
    for k in mine:
        assert torch.equal(mine[k].float(), theirs[k].float())


def test_file_errors(tmp_path):
    p = tmp_path / "m.safetensors"
    with pytest.raises(WeightError, match="cannot open"):
        read_safetensors(p)
    p.write_bytes(b"\x01\x02")
    with pytest.raises(WeightError, match="too short"):
        read_safetensors(p)
    p.write_bytes(struct.pack("<Q", 1000) + b"{}")
    with pytest.raises(WeightError, match="header length"):
        read_safetensors(p)
    p.write_bytes(struct.pack("<Q", 5) + b"{nope")
    with pytest.raises(WeightError, match="not valid JSON"):
        read_safetensors(p)
    h = json.dumps({"a": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    p.write_bytes(struct.pack("<Q", len(h)) + h + b"\0" * 8)
    with pytest.raises(WeightError, match="offsets"):
        read_safetensors(p)
    h = json.dumps({"a": {"dtype": "U8", "shape": [4], "data_offsets": [0, 4]}}).encode()
    p.write_bytes(struct.pack("<Q", len(h)) + h + b"\0" * 4)
    with pytest.raises(WeightError, match="unsupported dtype"):
        read_safetensors(p)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = write_random_model(TINY_A, 5, tmp_path / "m")
    t = dict(read_safetensors(d / "model.safetensors"))
    t = {k: v.clone() for k, v in t.items()}
    del t["h.1.mlp.c_fc.bias"]
    del t["ln_f.weight"]
    t["h.0.attn.c_attn.weight"] = torch.zeros(64, 100, dtype=torch.bfloat16)
    t["h.7.extra.weight"] = torch.zeros(3, dtype=torch.bfloat16)
    write_safetensors(d / "model.safetensors", t)
    with pytest.raises(WeightError) as e:
        open_model_dir(d)
    msg = str(e.value)
    assert "missing (2)" in msg and "h.1.mlp.c_fc.bias" in msg and "ln_f.weight" in msg
    assert "unexpected (1)" in msg and "h.7.extra.weight" in msg
    assert "wrong shape or type (1)" in msg and "expected [64, 192], found [64, 100]" in msg


def test_prefix_mask_buffers_and_tied_head_are_accepted(tmp_path):
    d = write_random_model(TINY_B, 6, tmp_path / "m")
    t = {k: v.clone() for k, v in read_safetensors(d / "model.safetensors").items()}  # the map goes stale on rewrite
    t2 = {"transformer." + k: v.clone() for k, v in t.items()}
    t2["transformer.h.0.attn.bias"] = torch.ones(1, 1, 8, 8)          # causal-mask buffer of HF checkpoints
    t2["transformer.h.0.attn.masked_bias"] = torch.tensor(-1e4)
    t2["lm_head.weight"] = t["wte.weight"].clone()                     # present but tied
    write_safetensors(d / "model.safetensors", t2)
    arch, cfg, w = open_model_dir(d)
    assert torch.equal(w["h.2.ln_2.bias"], t["h.2.ln_2.bias"])


def test_untied_head_is_required(tmp_path):
    cfg = dict(TINY_A, tie_word_embeddings=False)
    d = write_random_model(cfg, 7, tmp_path / "m")
    t = {k: v.clone() for k, v in read_safetensors(d / "model.safetensors").items()}
    assert "lm_head.weight" in t
    del t["lm_head.weight"]
    write_safetensors(d / "model.safetensors", t)
    with pytest.raises(WeightError, match="lm_head.weight"):
        open_model_dir(d)


def test_missing_files(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    with pytest.raises(WeightError, match="no model.safetensors"):
        open_model_dir(tmp_path)


def test_random_mode_is_seeded_and_nontrivial(tmp_path):
    a = read_safetensors(write_random_model(TINY_A, 1, tmp_path / "a") / "model.safetensors")
    b = read_safetensors(write_random_model(TINY_A, 1, tmp_path / "b") / "model.safetensors")
    c = read_safetensors(write_random_model(TINY_A, 2, tmp_path / "c") / "model.safetensors")
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert any(not torch.equal(a[k], c[k]) for k in a)
    assert a["wte.weight"].dtype == torch.bfloat16
    assert abs(float(a["h.0.ln_1.weight"].float().mean()) - 1.0) < 0.05
    assert float(a["h.0.attn.c_attn.bias"].float().abs().max()) > 0
    assert 0.015 < float(a["wte.weight"].float().std()) < 0.025
    cfg = json.loads((tmp_path / "a" / "config.json").read_text())
    assert cfg["model_type"] == "gpt2" and cfg["n_embd"] == 64
    f = read_safetensors(write_random_model(TINY_A, 1, tmp_path / "f", dtype=torch.float32) / "model.safetensors")
    assert f["wte.weight"].dtype == torch.float32


def test_placement_keeps_what_is_stored():
    m16, m32 = torch.randn(4, 4).to(torch.bfloat16), torch.randn(4, 4)
    v16, v32 = torch.randn(4).to(torch.bfloat16), torch.randn(4)
    assert place(m16, "matrix", torch.bfloat16, "cpu").dtype == torch.bfloat16
    assert place(v32, "vector", torch.bfloat16, "cpu").dtype == torch.float32      # stored in 32-bit stays so
    assert torch.equal(place(v16, "vector", torch.bfloat16, "cpu"), v16.float())    # widening is exact
    assert place(m16, "matrix", torch.float32, "cpu").dtype == torch.float32
    assert torch.equal(place(m32, "matrix", torch.float32, "cpu"), m32)
    assert place(torch.arange(4), "table", torch.bfloat16, "cpu").dtype == torch.int32


def test_check_tensors_types():
    specs = [TensorSpec("t", (2,), "table"), TensorSpec("w", (2, 2))]
    with pytest.raises(WeightError, match="integer table"):
        check_tensors({"t": torch.zeros(2), "w": torch.zeros(2, 2)}, specs)
    with pytest.raises(WeightError, match="floating point"):
        check_tensors({"t": torch.zeros(2, dtype=torch.int32), "w": torch.zeros(2, 2, dtype=torch.int32)}, specs)


def test_prefixes_and_ignorable_tensors_are_the_architectures_to_say(tmp_path):
    """Another architecture with a prefix of its own and a real tensor called like GPT-2's mask buffer: the loader
    takes both from its registry entry; nothing of GPT-2's conventions applies to it."""
    import dataclasses
    from vlrf_b200.config import ModelConfig, key
    from vlrf_b200.registry import Architecture, register_architecture, unregister_architecture

    @dataclasses.dataclass
    class OtherConfig(ModelConfig):
        model_type = "other_arch"
        width: int = key()

    def spec(cfg):
        return [TensorSpec("emb", (4, cfg.width)), TensorSpec("l0.attn.bias", (cfg.width,), "vector")]

    register_architecture(Architecture("other_arch", OtherConfig, spec, lambda cfg, gen: {}, lambda *a: None,
                                       prefixes=("", "model."), ignored_tensors=lambda cfg: ("*.rotary.inv_freq",)), replace=True)
    try:
        (tmp_path / "config.json").write_text(json.dumps({"model_type": "other_arch", "width": 6}))
        good = {"model.emb": torch.zeros(4, 6), "model.l0.attn.bias": torch.ones(6), "model.l0.rotary.inv_freq": torch.zeros(3)}
        write_safetensors(tmp_path / "model.safetensors", good)
        _, _, checked = open_model_dir(tmp_path)
        assert torch.equal(checked["l0.attn.bias"], torch.ones(6))          # a real tensor here, not a mask to skip
        # GPT-2's prefix is not this architecture's, and its own "*.attn.bias" is required, not ignorable
        write_safetensors(tmp_path / "model.safetensors", {"transformer.emb": torch.zeros(4, 6), "model.l0.rotary.inv_freq": torch.zeros(3)})
        with pytest.raises(WeightError) as e:
            open_model_dir(tmp_path)
        assert "emb" in str(e.value) and "l0.attn.bias" in str(e.value) and "transformer.emb" in str(e.value)
    finally:
        unregister_architecture("other_arch")
