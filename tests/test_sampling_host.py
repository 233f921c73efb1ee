"""The host side of sampling: the options under the reference's names and defaults, and the counter-based
random stream that the kernel repeats bit for bit (the kernel's side of it is checked on the GPU)."""
import pytest

from vlrf_b200.sampling import SamplingParams
from vlrf_b200.sampling.rng import as_signed64, request_key, uniform01


def test_defaults_are_the_references():
    p = SamplingParams()             # include/model/generation_config.hpp:16-20, :45-47, :56; tools/vlrf_cli.cpp:38
    assert (p.max_new_tokens, p.temperature, p.top_p, p.top_k, p.do_sample) == (128, 0.8, 0.9, 50, True)
    assert (p.repetition_penalty, p.frequency_penalty, p.presence_penalty, p.no_repeat_ngram_size, p.seed) == (1.0, 0.0, 0.0, 0, 42)
    assert p.stop_token_ids is None and not p.greedy and not p.has_penalties
    p.validate()


def test_greedy_and_penalties_are_told_from_the_options():
    assert SamplingParams(do_sample=False).greedy and SamplingParams(temperature=0.0).greedy    # transformer.hpp:130
    assert SamplingParams(temperature=-1.0).greedy and not SamplingParams(temperature=0.01).greedy
    assert SamplingParams.greedy_params(7).max_new_tokens == 7 and SamplingParams.greedy_params().greedy
    for kw in (dict(repetition_penalty=1.1), dict(frequency_penalty=0.5), dict(presence_penalty=-0.5), dict(no_repeat_ngram_size=2)):
        assert SamplingParams(**kw).has_penalties
    assert not SamplingParams(no_repeat_ngram_size=1).has_penalties    # an "n-gram" of one token blocks nothing (:92-94)


@pytest.mark.parametrize("kw,match", [(dict(max_new_tokens=-1), "max_new_tokens"), (dict(top_p=-0.1), "top_p"),
                                      (dict(repetition_penalty=0.0), "repetition_penalty")])
def test_bad_options_are_refused(kw, match):
    with pytest.raises(ValueError, match=match):
        SamplingParams(**kw).validate()


def test_a_requests_stream_depends_on_seed_and_index_only():
    keys = {request_key(seed, i) for seed in (0, 1, 42, 2**40) for i in range(50)}
    assert len(keys) == 200 and all(0 <= k < 2**64 for k in keys)
    assert request_key(42, 3) == request_key(42, 3) != request_key(43, 3)
    assert request_key(42 + 2**64, 3) == request_key(42, 3)            # seeds are taken modulo 2^64
    k = request_key(42, 0)
    draws = [uniform01(k, n) for n in range(4096)]
    assert draws == [uniform01(k, n) for n in range(4096)]              # the n-th draw depends on (key, n) only
    assert all(0.0 <= u < 1.0 for u in draws) and all(u * 16777216 == int(u * 16777216) for u in draws)   # 24 bits
    assert 0.47 < sum(draws) / len(draws) < 0.53
    tenths = [sum(1 for u in draws if i / 10 <= u < (i + 1) / 10) for i in range(10)]
    assert min(tenths) > 330 and max(tenths) < 490                      # 409.6 expected in each
    assert len(set(draws[:1000])) > 990                                 # no short cycle
    other = [uniform01(request_key(42, 1), n) for n in range(64)]
    assert sum(1 for a, b in zip(draws, other) if a == b) <= 1          # another request, another stream
    assert uniform01(k, 2**32 + 5) == uniform01(k, 5)                   # the kernel's counter has 32 bits


def test_keys_fit_the_signed_tensor_that_carries_them():
    for key in (0, 1, 2**63 - 1, 2**63, 2**64 - 1, request_key(7, 7)):
        s = as_signed64(key)
        assert -2**63 <= s < 2**63 and s % 2**64 == key
