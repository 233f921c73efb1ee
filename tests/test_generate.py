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


@pytest.mark.parametrize("dtype,tol", [("float32", TOL_F32), ("bfloat16", TOL_BF16)])
def test_waiting_requests_take_freed_rows_at_the_next_step_boundary(model_dirs, plain_models, dtype, tol):
    """Ten requests on four rows with unequal ends: a waiting request's prompt runs in the step in which the others go
    on by one token, then it decodes with them in the replayed session.  Every request gets what it gets alone."""
    from vlrf_b200 import Model, SamplingParams
    cfg, w = plain_models["tiny_b"]
    model = Model.load(model_dirs["tiny_b"], dtype=dtype, max_tokens=64 * 12, n_slots=4)
    lens = [7, 30, 2, 65, 1, 12, 64, 3, 40, 9]
    news = [12, 2, 9, 1, 14, 3, 2, 11, 1, 6]
    prompts = [random_ids(cfg["vocab_size"], n, 300 + i) for i, n in enumerate(lens)]
    params = [SamplingParams(max_new_tokens=m, do_sample=False, stop_token_ids=()) for m in news]
    res = model.generate_ids(prompts, params)
    for p, m, r in zip(prompts, news, res):
        assert r.prompt == p and r.tokens_generated == m and r.finish_reason == "length"
        check_greedy(cfg, w, p, r.new_tokens, tol)
        if dtype == "float32":
            assert r.new_tokens == plain.greedy_generate(cfg, w, p, m)
    b = model.backend
    static_steps = sum(max(news[i:i + 4]) for i in range(0, 10, 4))
    assert b.prompt_steps + b.decode_steps < static_steps          # fewer steps than whole batches would take
    assert b.prompt_steps >= 3 and b.decode_steps > 0              # prompts joined running steps; decoding was replayed
    assert model.engine.cache.slots.n_held == 0
    model.engine.cache.check()
    model.engine.check_device_errors()


def test_a_request_that_ends_at_its_first_token_does_not_keep_the_rest_from_the_replayed_session(model_dirs, plain_models):
    from vlrf_b200 import Model, SamplingParams
    cfg, w = plain_models["tiny_a"]
    model = Model.load(model_dirs["tiny_a"], dtype="float32", max_tokens=512)
    prompts = [random_ids(512, n, 400 + n) for n in (9, 4, 20)]
    params = [SamplingParams(max_new_tokens=m, do_sample=False, stop_token_ids=()) for m in (10, 1, 10)]
    res = model.generate_ids(prompts, params)
    assert [r.new_tokens for r in res] == [plain.greedy_generate(cfg, w, p, m) for p, m in zip(prompts, (10, 1, 10))]
    assert model.backend.prompt_steps == 1 and model.backend.decode_steps == 9
    # the same when it ends by a stop token that its prompt's logits choose
    stop = res[0].new_tokens[0]
    again = model.generate_ids(prompts, [SamplingParams(max_new_tokens=10, do_sample=False, stop_token_ids=(stop,)),
                                         SamplingParams(max_new_tokens=10, do_sample=False, stop_token_ids=()),
                                         SamplingParams(max_new_tokens=10, do_sample=False, stop_token_ids=())])
    assert again[0].new_tokens == [stop] and again[0].finish_reason == "stop"
    assert again[2].new_tokens == res[2].new_tokens
    assert model.engine.cache.slots.n_held == 0


def test_penalties_and_blocked_ngrams_follow_the_plain_rules_token_by_token(model_dirs, plain_models):
    """Greedy generation under repetition / frequency / presence penalties and a blocked n-gram size: every token is the
    first maximum of the plain implementation's logits edited by the plain rules from the tokens generated so far."""
    import numpy as np
    from vlrf_b200 import Model, SamplingParams
    cfg, w = plain_models["tiny_a"]
    model = Model.load(model_dirs["tiny_a"], dtype="float32", max_tokens=512)
    prompts = [random_ids(512, n, 500 + n) for n in (6, 15)]
    p = SamplingParams(max_new_tokens=30, do_sample=False, stop_token_ids=(), repetition_penalty=1.3, frequency_penalty=0.2,
                       presence_penalty=0.1, no_repeat_ngram_size=3)
    res = model.generate_ids(prompts, p)
    for prompt, r in zip(prompts, res):
        ids, new = list(prompt), []
        for t in r.new_tokens:
            lg = plain.logits_all_positions(cfg, w, ids)[-1].numpy()
            counts = {}
            for g in new:
                counts[g] = counts.get(g, 0) + 1
            edited = plain.block_repeated_ngrams(plain.apply_penalties(lg, counts, 1.3, 0.2, 0.1), new, 3)
            best = float(edited.max())
            assert np.isfinite(edited[t]) and best - float(edited[t]) <= 2 * TOL_F32 * float(np.abs(lg).max()), (len(ids), t)
            ids.append(t)
            new.append(t)
