"""The command line: `init` and `info` on the CPU, `run` on the GPU against the plain implementation."""
import json

import pytest

import plain_gpt2 as plain
from conftest import TINY_B


def run_cli(argv, capsys):
    from vlrf_b200.cli import main
    assert main(argv) == 0
    return capsys.readouterr().out


def test_init_writes_a_model_folder_and_info_reads_it(tmp_path, capsys):
    cfg_file = tmp_path / "cfg.json"
    cfg_file.write_text(json.dumps(TINY_B))
    out = run_cli(["init", "--config", str(cfg_file), "--out", str(tmp_path / "m"), "--seed", "9"], capsys)
    assert "seed 9" in out
    assert (tmp_path / "m" / "config.json").exists() and (tmp_path / "m" / "model.safetensors").exists()
    # the same seed gives the same bytes, another seed others
    run_cli(["init", "--config", str(cfg_file), "--out", str(tmp_path / "m2"), "--seed", "9"], capsys)
    run_cli(["init", "--config", str(cfg_file), "--out", str(tmp_path / "m3"), "--seed", "10"], capsys)
    same = (tmp_path / "m" / "model.safetensors").read_bytes()
    assert same == (tmp_path / "m2" / "model.safetensors").read_bytes()
    assert same != (tmp_path / "m3" / "model.safetensors").read_bytes()
    info = run_cli(["info", "--model", str(tmp_path / "m")], capsys)
    assert "architecture: gpt2" in info
    shown = json.loads(info[info.index("{"):info.rindex("}") + 1])
    for key in ("n_layer", "n_embd", "n_head", "n_inner", "vocab_size", "n_positions", "layer_norm_epsilon"):
        assert shown[key] == TINY_B[key]
    cfg, w = plain.read_model_dir(tmp_path / "m")
    n_params = sum(int(t.numel()) for t in w.values())
    assert f"parameters: {n_params:,}" in info


def test_init_takes_a_preset_name(tmp_path, capsys):
    run_cli(["init", "--config", "tiny-a", "--out", str(tmp_path / "a")], capsys)
    assert json.loads((tmp_path / "a" / "config.json").read_text())["n_embd"] == 64


def test_what_the_library_refuses_is_a_message_and_status_1(tmp_path, capsys):
    from vlrf_b200.cli import main
    assert main(["info", "--model", str(tmp_path / "nowhere")]) == 1
    assert "cannot read" in capsys.readouterr().err
    assert main(["init", "--config", "no-such-preset", "--out", str(tmp_path / "x")]) == 1
    err = capsys.readouterr().err
    assert "neither a preset" in err and "tiny-a" in err
    bad = tmp_path / "cfg.json"
    bad.write_text(json.dumps(dict(TINY_B, n_head=7)))              # 96 is no multiple of 7
    assert main(["init", "--config", str(bad), "--out", str(tmp_path / "y")]) == 1
    assert "n_head" in capsys.readouterr().err


def test_without_a_gpu_run_says_so(tmp_path, capsys):
    import torch
    if torch.cuda.is_available():
        pytest.skip("this machine has a GPU")
    from vlrf_b200.cli import main
    run_cli(["init", "--config", "tiny-a", "--out", str(tmp_path / "a")], capsys)
    assert main(["run", "--model", str(tmp_path / "a"), "--prompt-ids", "1,2", "--tokens", "2", "--greedy"]) == 1
    assert "no other execution path" in capsys.readouterr().err


def test_prompts_from_text_ids_and_file(tmp_path):
    import argparse

    from vlrf_b200.cli import _prompts
    ns = argparse.Namespace(prompts_file=None, prompt_ids=None, prompt="Hi!")
    # byte + 4, as the reference without a tokenizer; the cap at the vocabulary follows once the model is loaded
    assert _prompts(ns) == ([[ord("H") + 4, ord("i") + 4, ord("!") + 4]], True)
    assert _prompts(argparse.Namespace(prompts_file=None, prompt_ids="5, 17,3", prompt=None)) == ([[5, 17, 3]], False)
    f = tmp_path / "p.txt"
    f.write_text("1 2 3\n\n4,5\n")
    assert _prompts(argparse.Namespace(prompts_file=str(f), prompt_ids=None, prompt=None)) == ([[1, 2, 3], [4, 5]], False)
    with pytest.raises(SystemExit):
        _prompts(argparse.Namespace(prompts_file=None, prompt_ids=None, prompt=None))


@pytest.mark.gpu
def test_run_generates_what_the_plain_implementation_would(model_dirs, plain_models, tmp_path, capsys):
    cfg, w = plain_models["tiny_b"]
    f = tmp_path / "prompts.txt"
    f.write_text("5 17 3 900 44\n7\n")
    out = run_cli(["run", "--model", str(model_dirs["tiny_b"]), "--prompts-file", str(f), "--tokens", "6", "--greedy",
                   "--stop-id", "999", "--dtype", "float32"], capsys)
    outputs = [line for prev, line in zip(out.splitlines(), out.splitlines()[1:]) if prev.startswith("--- Output")]
    assert len(outputs) == 2
    for prompt, line in zip(([5, 17, 3, 900, 44], [7]), outputs):
        ids = list(prompt)
        for tok in (int(t) for t in line.split()):
            lg = plain.logits_all_positions(cfg, w, ids)[-1]
            assert float(lg.max() - lg[tok]) <= 2e-4 * float(lg.abs().max())
            ids.append(tok)
        assert len(ids) == len(prompt) + 6
    assert "12 generated" in out
