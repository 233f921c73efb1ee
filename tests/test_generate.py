"""Generation through the Python entry point against the plain implementation."""
import pytest
import torch

import plain_gpt2 as plain
from conftest import TOL_BF16, TOL_F32, random_ids

pytestmark = pytest.mark.gpu


def check_greedy(cfg, w, prompt, new_tokens, tol):
    """Every generated token is a maximal logit of the plain implementation on the sequence so far
    (within the tolerance, so that a near-tie may fall either way)."""
    ids = list(prompt)
    for t in new_tokens:
        lg = plain.logits_all_positions(cfg, w, ids)[-1]
        assert float(lg.max() - lg[t]) <= 2 * tol * float(lg.abs().max()), (len(ids), t, int(lg.argmax()))
        ids.append(t)


@pytest.mark.parametrize("dtype,tol", [("float32", TOL_F32), ("bfloat16", TOL_BF16)])
@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_greedy_generation_of_a_batch(model_dirs, plain_models, name, dtype, tol):
    from vlrf_b200 import Model, SamplingParams
    cfg, w = plain_models[name]
    lens = [5, 17, 31] if name == "tiny_a" else [1, 9, 40, 100]
    steps = 16 if name == "tiny_a" else 24
    prompts = [random_ids(cfg["vocab_size"], n, 70 + n) for n in lens]
    model = Model.load(model_dirs[name], dtype=dtype, max_tokens=64 * 8)
    res = model.generate_ids(prompts, SamplingParams(max_new_tokens=steps, do_sample=False, stop_token_ids=()))
    for p, r in zip(prompts, res):
        assert r.prompt == p and r.tokens_generated == steps and r.finish_reason == "length"
        check_greedy(cfg, w, p, r.new_tokens, tol)
    if dtype == "float32":
        want = [plain.greedy_generate(cfg, w, p, steps) for p in prompts]
        assert [r.new_tokens for r in res] == want
    # each alone gives what the batch gave
    alone = [model.generate_ids(p, SamplingParams(max_new_tokens=steps, do_sample=False, stop_token_ids=())) for p in prompts]
    assert [a.new_tokens for a in alone] == [r.new_tokens for r in res]
    assert model.engine.cache.slots.n_held == 0
    model.engine.cache.check()


def test_stop_token_context_end_and_more_requests_than_slots(model_dirs, plain_models):
    from vlrf_b200 import Model, SamplingParams
    cfg, w = plain_models["tiny_a"]
    model = Model.load(model_dirs["tiny_a"], dtype="float32", max_tokens=256, n_slots=2)
    prompts = [random_ids(512, n, 80 + n) for n in (3, 30, 120, 7, 64)]
    free_run = model.generate_ids(prompts, SamplingParams(max_new_tokens=20, do_sample=False, stop_token_ids=()))
    assert free_run[2].finish_reason == "context" and len(free_run[2].token_ids) == 128
    model.engine.check_device_errors()        # the ended row, now padding, must not look like a bad position
    stop = free_run[0].new_tokens[4]
    res = model.generate_ids(prompts, SamplingParams(max_new_tokens=20, do_sample=False, stop_token_ids=(stop,)))
    first = free_run[0].new_tokens.index(stop)
    assert res[0].new_tokens == free_run[0].new_tokens[:first + 1] and res[0].finish_reason == "stop"
    for r, f in zip(res[1:], free_run[1:]):
        if stop not in f.new_tokens:
            assert r.new_tokens == f.new_tokens
    want = plain.greedy_generate(cfg, w, prompts[3], 20)
    assert free_run[3].new_tokens == want
    assert model.engine.cache.slots.n_held == 0


def test_sampling_is_seeded_and_independent_of_the_batch(model_dirs):
    from vlrf_b200 import Model, SamplingParams
    model = Model.load(model_dirs["tiny_b"], dtype="float32", max_tokens=1024)
    prompts = [random_ids(1000, n, 90 + n) for n in (4, 11, 25)]
    p = SamplingParams(max_new_tokens=12, temperature=0.8, top_k=50, top_p=0.9, seed=7, stop_token_ids=())
    a = model.generate_ids(prompts, p)
    b = model.generate_ids(prompts, p)
    assert [r.new_tokens for r in a] == [r.new_tokens for r in b]
    c = model.generate_ids(prompts, SamplingParams(max_new_tokens=12, temperature=0.8, top_k=50, top_p=0.9, seed=8,
                                                   stop_token_ids=()))
    assert [r.new_tokens for r in a] != [r.new_tokens for r in c]
    # request 0 alone: same stream (index 0), same logits → same tokens
    alone = model.generate_ids([prompts[0]], p)
    assert alone[0].new_tokens == a[0].new_tokens
    greedy = model.generate_ids(prompts, SamplingParams(max_new_tokens=12, temperature=0.0, stop_token_ids=()))
    greedy2 = model.generate_ids(prompts, SamplingParams(max_new_tokens=12, do_sample=False, stop_token_ids=()))
    assert [r.new_tokens for r in greedy] == [r.new_tokens for r in greedy2]


def test_penalties_change_what_is_generated(model_dirs):
    from vlrf_b200 import Model, SamplingParams
    model = Model.load(model_dirs["tiny_a"], dtype="float32", max_tokens=256)
    prompt = random_ids(512, 6, 95)
    base = model.generate_ids(prompt, SamplingParams(max_new_tokens=40, do_sample=False, stop_token_ids=()))
    blocked = model.generate_ids(prompt, SamplingParams(max_new_tokens=40, do_sample=False, stop_token_ids=(),
                                                       no_repeat_ngram_size=2, repetition_penalty=1.5))
    toks = blocked.new_tokens
    bigrams = list(zip(toks, toks[1:]))
    assert len(set(bigrams)) == len(bigrams)          # no bigram among the generated tokens repeats
    assert len(base.new_tokens) == 40


def test_get_logits_and_summary(model_dirs, plain_models):
    from vlrf_b200 import Model
    cfg, w = plain_models["tiny_b"]
    model = Model.load(model_dirs["tiny_b"], dtype="float32", max_tokens=256)
    ids = random_ids(1000, 33, 96)
    truth = plain.logits_all_positions(cfg, w, ids)
    last = model.get_logits(ids)
    assert last.shape == (1000,) and float((last.double() - truth[-1]).abs().max()) < 1e-4 * float(truth.abs().max())
    every = model.get_logits(ids, all_positions=True)
    assert every.shape == (33, 1000)
    assert "n_embd=96" in model.model_summary() and model.kv_cache_bytes() > 0


def test_generation_inside_inference_mode(model_dirs):
    """torch's inference mode keeps no version counters of tensors; whatever the kernels' dispatch derives
    from them must fall back, and the tokens stay the same."""
    from conftest import random_ids
    from vlrf_b200 import Model, SamplingParams
    prompts = [random_ids(1000, n, 900 + n) for n in (5, 21)]
    params = SamplingParams(max_new_tokens=10, do_sample=False, stop_token_ids=())
    want = Model.load(model_dirs["tiny_b"], dtype="bfloat16", max_tokens=256).generate_ids(prompts, params)
    with torch.inference_mode():
        model = Model.load(model_dirs["tiny_b"], dtype="bfloat16", max_tokens=256)
        got = model.generate_ids(prompts, params)
    assert [r.new_tokens for r in got] == [r.new_tokens for r in want]
