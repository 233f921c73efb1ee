"""A windowed mixer through the whole engine: a toy architecture, defined here and never shipped, whose layers are the
library's attention with a window of 70 keys (and one layer with all keys, so that the cache holds two groups with
storage of their own).  The cache gives blocks that lie before a sequence's window back to the pool while the
sequence lives; the kernels must never look at them.  Prompts arrive in portions that end at 63, 64 and 65 tokens
and in a portion of two tokens; decoding crosses block boundaries one token at a time; slots are given back and taken
again.  After every step the device's error word is silent and the cache's books are whole."""
import dataclasses
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
HEADS, WINDOW = 2, 70


def define_toy():
    from vlrf_b200.config import ModelConfig, key
    from vlrf_b200.engine.model import DecoderModel, LayerCall
    from vlrf_b200.parts import LayerNorm, LMHead, PreNormBlock, TokenEmbedding, get_part
    from vlrf_b200.registry import Architecture, register_architecture
    from vlrf_b200.weights.spec import TensorSpec, place

    @dataclasses.dataclass
    class ToyWindowConfig(ModelConfig):
        model_type = "toy_window"
        vocab_size: int = key()
        width: int = key()
        max_len: int = key()
        windows: str = key()           # per layer: the window, 0 = all keys; e.g. "70,0,70"

    def windows(cfg):
        return [int(x) for x in cfg.windows.split(",")]

    def spec(cfg):
        d = cfg.width
        s = [TensorSpec("emb", (cfg.vocab_size, d))]
        for i in range(len(windows(cfg))):
            s += [TensorSpec(f"l{i}.n1", (d,), "vector"), TensorSpec(f"l{i}.n2", (d,), "vector"),
                  TensorSpec(f"l{i}.qkv", (3 * d, d)), TensorSpec(f"l{i}.out", (d, d)),
                  TensorSpec(f"l{i}.ffn_in", (2 * d, d)), TensorSpec(f"l{i}.ffn_out", (d, 2 * d))]
        return s

    def rand(cfg, gen):
        out = {}
        for t in spec(cfg):
            # scores of a standard deviation of about 2 (a key outside the window would show); the other matrices
            # smaller, so that three layers of bfloat16 rounding stay well inside the bound
            std = 0.15 if t.name.endswith("qkv") or t.name == "emb" else (0.02 if t.name.endswith("out") else 0.08)
            out[t.name] = (1.0 if ".n" in t.name else 0.0) + std * torch.randn(t.shape, generator=gen)
        return out

    def build(cfg, weights, options):
        dt, dev = options.dtype, options.device
        m = lambda n: place(weights[n], "matrix", dt, dev)   # noqa: E731
        v = lambda n: place(weights[n], "vector", dt, dev)   # noqa: E731
        zeros = lambda n: torch.zeros(n, device=dev)         # noqa: E731
        d = cfg.width
        emb = m("emb")
        layers = []
        for i, win in enumerate(windows(cfg)):
            mixer = get_part("mixer", "causal_self_attention")(m(f"l{i}.qkv"), zeros(3 * d), m(f"l{i}.out"), zeros(d),
                                                               n_heads=HEADS, n_kv_heads=HEADS, head_dim=d // HEADS,
                                                               scale=1.0 / math.sqrt(d // HEADS), window=win)
            feed = get_part("feed_forward", "dense_mlp")(m(f"l{i}.ffn_in"), zeros(2 * d), m(f"l{i}.ffn_out"), zeros(d),
                                                         activation="gelu_tanh")
            layers.append(PreNormBlock(LayerNorm(v(f"l{i}.n1"), zeros(d), 1e-5), mixer, LayerNorm(v(f"l{i}.n2"), zeros(d), 1e-5), feed))
        return DecoderModel(config=cfg, embedding=TokenEmbedding(emb), layers=layers,
                            schedule=[LayerCall(i) for i in range(len(layers))],
                            final_norm=LayerNorm(torch.ones(d, device=dev), zeros(d), 1e-5), head=LMHead(emb),
                            options=options, max_seq_len=cfg.max_len)

    register_architecture(Architecture("toy_window", ToyWindowConfig, spec, rand, build), replace=True)


def toy_truth(cfg, w, ids):
    import plain_gpt2 as plain
    W = {k: v.double() for k, v in w.items()}
    d = cfg["width"]
    zeros, ones = torch.zeros(d, dtype=torch.float64), torch.ones(d, dtype=torch.float64)
    x = W["emb"][torch.tensor(ids)]
    for i, win in enumerate(int(t) for t in cfg["windows"].split(",")):
        h = plain.layer_norm(x, W[f"l{i}.n1"], zeros, 1e-5)
        q, k, v = (plain.split_heads(t, HEADS) for t in plain.split_qkv(h @ W[f"l{i}.qkv"].T, d))
        x = x + plain.merge_heads(plain.causal_attention(q, k, v, 1.0 / math.sqrt(d // HEADS), window=win)) @ W[f"l{i}.out"].T
        h = plain.layer_norm(x, W[f"l{i}.n2"], zeros, 1e-5)
        x = x + plain.gelu_tanh(h @ W[f"l{i}.ffn_in"].T) @ W[f"l{i}.ffn_out"].T
    return plain.layer_norm(x, ones, zeros, 1e-5) @ W["emb"].T


@pytest.mark.parametrize("dtype,tol", [("float32", 1e-4), ("bfloat16", 3e-2)])
@pytest.mark.parametrize("head_dim", [32, 64])
def test_a_window_of_keys_through_engine_cache_and_kernels(tmp_path, dtype, tol, head_dim):
    import plain_gpt2 as plain
    from conftest import random_ids, record_error, rel_err
    from engine_drives import poison
    from vlrf_b200.cache import KVNeed
    from vlrf_b200.engine import Engine, StepEntry, load_model
    from vlrf_b200.weights import write_random_model
    define_toy()
    cfg = dict(model_type="toy_window", vocab_size=150, width=HEADS * head_dim, max_len=330, windows=f"{WINDOW},0,{WINDOW}")
    d = write_random_model(cfg, 21, tmp_path / "toy_window", dtype=torch.float32)
    _, w = plain.read_model_dir(d)
    model = load_model(d, dtype)
    needs = model.cache_needs()
    assert needs[0] == KVNeed(HEADS, head_dim, "window", WINDOW) and needs[1] == KVNeed(HEADS, head_dim, "full") and needs[2] == needs[0]
    # the windowed group needs at most three blocks a sequence (70 keys may touch three blocks of 64); a cache of 12
    # blocks holds two sequences of 330 tokens only because blocks before the window come back to the pool
    eng = Engine(model, max_tokens=64 * 12)
    poison(eng)
    worst = 0.0

    def after_step():
        eng.check_device_errors()
        eng.cache.check()

    def error_of(got, truth, rows):
        """Largest absolute error over the logit scale of the whole request, as the other engine tests measure."""
        return float((got.double() - truth[rows]).abs().max() / truth.abs().max())

    def feed(slot, ids, truth, start, stop, want_all=True):
        nonlocal worst
        want = list(range(stop - start)) if want_all else [stop - start - 1]
        got = eng.step([StepEntry(slot, ids[start:stop], want)]).float().cpu()
        rows = list(range(start, stop)) if want_all else [stop - 1]
        err = error_of(got, truth, rows)
        assert torch.isfinite(got).all() and err < tol, (start, stop, err)
        worst = max(worst, err)
        after_step()

    for round_ in range(2):                                   # the second round finds slots and blocks used before
        seqs = [random_ids(150, 330, 40 + round_), random_ids(150, 200, 50 + round_)]
        truths = [toy_truth(cfg, w, ids) for ids in seqs]
        s0, s1 = eng.start_sequence(), eng.start_sequence()
        # sequence 0: portions that end at 63, 64, 65, then a two-token portion, a long one across two blocks, then tokens
        at = 0
        for stop in (63, 64, 65, 67, 200):
            feed(s0, seqs[0], truths[0], at, stop)
            at = stop
        # sequence 1 whole up to 130 in one step beside nothing, then both decode one by one across block boundaries
        feed(s1, seqs[1], truths[1], 0, 130)
        pos = [200, 130]
        while pos[0] < 330 or pos[1] < 200:
            entries, rows = [], []
            for i, (slot, ids) in enumerate(((s0, seqs[0]), (s1, seqs[1]))):
                if pos[i] < len(ids):
                    entries.append(StepEntry(slot, [ids[pos[i]]], [0]))
                    rows.append(i)
            got = eng.step(entries).float().cpu()
            for r, i in enumerate(rows):
                err = error_of(got[r:r + 1], truths[i], [pos[i]])
                assert err < tol, (i, pos[i], err)
                worst = max(worst, err)
                pos[i] += 1
                if pos[i] == len(seqs[i]):
                    eng.end_sequence((s0, s1)[i])
            after_step()
        assert eng.cache.slots.n_held == 0
    record_error("a window of keys through the engine", f"toy_window head {head_dim}", dtype, worst)
