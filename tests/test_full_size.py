"""The real sizes, held against the plain implementation: GPT-2 small at its full depth of twelve layers (the
benchmark's model), the medium layer shape with an unequal batch of eight, and the XL layer shape at batch four in
32-bit.  Random weights; the plain implementation runs in float64 on the host, which is what these tests cost."""
import pytest
import torch

import plain_gpt2 as plain
from conftest import TOL_BF16, TOL_F32, random_ids, record_error

pytestmark = [pytest.mark.gpu, pytest.mark.slow]


def run_batch(model_dir, dtype, prompts, n_decode, wanted):
    """A prompt step for all prompts (logits at `wanted[i]` positions of each), then n_decode steps of one token each,
    fed from the given ids; returns per request (positions, logits [len(positions), vocab])."""
    from engine_drives import poison
    from vlrf_b200.engine import Engine, StepEntry, load_model
    need = sum((len(p) + 63) // 64 * 64 for p in prompts)
    eng = Engine(load_model(model_dir, dtype), max_tokens=need)
    poison(eng)
    slots = [eng.start_sequence() for _ in prompts]
    first = [len(p) - n_decode for p in prompts]
    got = eng.step([StepEntry(s, p[:n], w) for s, p, n, w in zip(slots, prompts, first, wanted)]).float().cpu()
    out, at = [], 0
    for w in wanted:
        out.append((list(w), [got[at:at + len(w)].clone()]))
        at += len(w)
    for j in range(n_decode):
        got = eng.step([StepEntry(s, [p[n + j]], [0]) for s, p, n in zip(slots, prompts, first)]).float().cpu()
        for i, n in enumerate(first):
            out[i][0].append(n + j)
            out[i][1].append(got[i:i + 1].clone())
    eng.check_device_errors()
    eng.cache.check()
    return [(pos, torch.cat(rows)) for pos, rows in out]


def hold_against_plain(cfg, w, prompts, results, tol, what, dtype):
    worst = 0.0
    for ids, (pos, got) in zip(prompts, results):
        truth = plain.logits_all_positions(cfg, w, ids)
        err = float((got.double() - truth[pos]).abs().max() / truth.abs().max())
        assert torch.isfinite(got).all() and err < tol, (what, len(ids), err)
        worst = max(worst, err)
    record_error(what, "", dtype, worst)
    return worst


@pytest.fixture(scope="module")
def gpt2_small(tmp_path_factory):
    import vlrf_b200.models  # noqa: F401
    from vlrf_b200.config import load_preset
    from vlrf_b200.weights import write_random_model
    d = write_random_model(load_preset("gpt2"), 2024, tmp_path_factory.mktemp("gpt2_small"))
    return d, plain.read_model_dir(d)


@pytest.mark.parametrize("dtype,tol", [("float32", TOL_F32), ("bfloat16", TOL_BF16)])
def test_gpt2_small_at_full_depth(gpt2_small, dtype, tol):
    """Twelve layers, the vocabulary of 50,257: an unequal batch of four, three dozen positions wanted, eight decoded."""
    d, (cfg, w) = gpt2_small
    assert cfg["n_layer"] == 12 and cfg["vocab_size"] == 50257
    prompts = [random_ids(50257, n, 900 + n) for n in (300, 64, 17, 130)]
    wanted = [[0, 1, 63, 64, 127, 128, 200, 291], [0, 31, 55], [0, 8], [5, 64, 65, 121]]
    results = run_batch(d, dtype, prompts, 8, wanted)
    hold_against_plain(cfg, w, prompts, results, tol, "GPT-2 small, 12 layers, batch of 4", dtype)


@pytest.mark.parametrize("dtype,tol", [("float32", TOL_F32), ("bfloat16", TOL_BF16)])
def test_medium_layer_shape_with_an_unequal_batch_of_eight(tmp_path, dtype, tol):
    """Width 1,024, 16 heads, inner 4,096 (GPT-2 medium's layers), three of them; eight prompts of 16 to 768 tokens."""
    from vlrf_b200.weights import write_random_model
    cfg = dict(model_type="gpt2", n_layer=3, n_embd=1024, n_head=16, n_inner=4096, vocab_size=5003, n_positions=1024,
               layer_norm_epsilon=1e-5, activation_function="gelu_new", scale_attn_by_inverse_layer_idx=False,
               tie_word_embeddings=True, bos_token_id=0, eos_token_id=0)
    d = write_random_model(cfg, 31, tmp_path / "medium_shape")
    pc, w = plain.read_model_dir(d)
    gen = torch.Generator().manual_seed(5)
    lens = [16, 768] + torch.randint(16, 769, (6,), generator=gen).tolist()
    prompts = [random_ids(5003, n, 800 + i) for i, n in enumerate(lens)]
    wanted = [[0, (n - 4) // 2, n - 5] for n in lens]
    results = run_batch(d, dtype, prompts, 4, wanted)
    hold_against_plain(pc, w, prompts, results, tol, "medium layer shape, batch of 8, lengths 16 to 768", dtype)


def test_xl_layer_shape_at_batch_four_in_32_bit(tmp_path):
    """Width 1,600, 25 heads, inner 6,400 (GPT-2 XL's layers), two of them, float32: the full logits of a batch of four."""
    from vlrf_b200.weights import write_random_model
    cfg = dict(model_type="gpt2", n_layer=2, n_embd=1600, n_head=25, n_inner=6400, vocab_size=5003, n_positions=1024,
               layer_norm_epsilon=1e-5, activation_function="gelu_new", scale_attn_by_inverse_layer_idx=False,
               tie_word_embeddings=True, bos_token_id=0, eos_token_id=0)
    d = write_random_model(cfg, 32, tmp_path / "xl_shape")
    pc, w = plain.read_model_dir(d)
    prompts = [random_ids(5003, n, 850 + n) for n in (200, 64, 500, 33)]
    wanted = [list(range(0, n - 6, max(1, n // 12))) for n in (200, 64, 500, 33)]
    results = run_batch(d, "float32", prompts, 6, wanted)
    hold_against_plain(pc, w, prompts, results, TOL_F32, "XL layer shape, batch of 4", "float32")


def test_generation_at_the_medium_shape_greedy_and_with_a_temperature(tmp_path):
    """The batch of eight through the entry point, greedy and at temperature 0.8: greedy tokens are maxima of the plain
    logits; sampled tokens come again with the same seed and differ from the greedy ones somewhere."""
    from vlrf_b200 import Model, SamplingParams
    from vlrf_b200.weights import write_random_model
    cfg = dict(model_type="gpt2", n_layer=2, n_embd=1024, n_head=16, n_inner=4096, vocab_size=5003, n_positions=1024,
               layer_norm_epsilon=1e-5, activation_function="gelu_new", scale_attn_by_inverse_layer_idx=False,
               tie_word_embeddings=True, bos_token_id=0, eos_token_id=0)
    d = write_random_model(cfg, 33, tmp_path / "medium_generate")
    pc, w = plain.read_model_dir(d)
    gen = torch.Generator().manual_seed(6)
    lens = [16, 768] + torch.randint(16, 769, (6,), generator=gen).tolist()
    prompts = [random_ids(5003, n, 870 + i) for i, n in enumerate(lens)]
    model = Model.load(d, dtype="bfloat16", max_tokens=sum((n + 8 + 63) // 64 * 64 for n in lens))
    greedy = model.generate_ids(prompts, SamplingParams(max_new_tokens=6, do_sample=False, stop_token_ids=()))
    for p, r in list(zip(prompts, greedy))[:3]:
        ids = list(p)
        for t in r.new_tokens:
            lg = plain.logits_all_positions(pc, w, ids)[-1]
            assert float(lg.max() - lg[t]) <= 2 * TOL_BF16 * float(lg.abs().max())
            ids.append(t)
    sampled = SamplingParams(max_new_tokens=6, temperature=0.8, top_k=50, top_p=0.9, seed=3, stop_token_ids=())
    a, b = model.generate_ids(prompts, sampled), model.generate_ids(prompts, sampled)
    assert [r.new_tokens for r in a] == [r.new_tokens for r in b]
    assert [r.new_tokens for r in a] != [r.new_tokens for r in greedy]
    assert model.engine.cache.slots.n_held == 0
