"""The host side of a step: what `Engine.plan` checks and the integer tables it lays out (CPU; the cache's
bookkeeping is real, the model is two numbers)."""
import types

import numpy as np
import pytest
import torch

from vlrf_b200.cache.sequence_cache import KVNeed, SequenceCache
from vlrf_b200.engine.step import Engine, StepEntry, StepError


def fake_engine(vocab=100, max_seq_len=128, max_tokens=512, n_slots=4):
    cache = SequenceCache([KVNeed(2, 16)] * 2, max_tokens=max_tokens, max_seq_len=max_seq_len, dtype=torch.float32,
                          device="cpu", n_slots=n_slots)
    return types.SimpleNamespace(model=types.SimpleNamespace(vocab_size=vocab, max_seq_len=max_seq_len), cache=cache)


def test_tables_of_a_ragged_step_that_continues_sequences():
    eng = fake_engine()
    a, b, c = (eng.cache.acquire() for _ in range(3))
    eng.cache.reserve(b, 70); eng.cache.advance(b, 70)               # b already holds 70 tokens
    p = Engine.plan(eng, [StepEntry(a, [5, 6, 7], [0, 2]), StepEntry(b, np.array([9], dtype=np.int32), [0]),
                          StepEntry(c, (1, 2), [])])
    assert (p["T"], p["B"], p["n_want"]) == (6, 3, 3)
    assert p["tokens"].tolist() == [5, 6, 7, 9, 1, 2] and p["tokens"].dtype == np.int32
    assert p["tok_slot"].tolist() == [a, a, a, b, c, c]
    assert p["tok_pos"].tolist() == [0, 1, 2, 70, 0, 1]              # positions go on from what each slot holds
    assert p["seq_slot"].tolist() == [a, b, c] and p["seq_start"].tolist() == [0, 3, 4, 6]
    assert p["seq_pos0"].tolist() == [0, 70, 0] and p["rows"].tolist() == [0, 2, 3]
    assert p["lens"] == [3, 1, 2] and p["pos0"] == [0, 70, 0]
    assert eng.cache.lengths[a] == 0                                 # planning changes nothing


def test_lists_tuples_and_arrays_give_the_same_tables():
    eng = fake_engine()
    s = eng.cache.acquire()
    ids = [3, 1, 4, 1, 5, 9, 2, 6]
    plans = [Engine.plan(eng, [StepEntry(s, t, [7])]) for t in (ids, tuple(ids), np.array(ids), np.array(ids, dtype=np.int32),
                                                               torch.tensor(ids).numpy())]
    for p in plans[1:]:
        assert p["tokens"].tolist() == plans[0]["tokens"].tolist() and p["rows"].tolist() == [7]


@pytest.mark.parametrize("entries,match", [
    (lambda s, t: [], "at least one sequence"),
    (lambda s, t: [StepEntry(s, [1], [0]), StepEntry(s, [2], [0])], "appears twice"),
    (lambda s, t: [StepEntry(t, [1], [0])], "not held"),
    (lambda s, t: [StepEntry(s, [], [])], "at least one token"),
    (lambda s, t: [StepEntry(s, [1] * 129, [0])], "exceed the 128 positions"),
    (lambda s, t: [StepEntry(s, [1, 100], [0])], "token id 100 lies outside the vocabulary of 100"),
    (lambda s, t: [StepEntry(s, [-1, 5], [0])], "token id -1 lies outside"),
    (lambda s, t: [StepEntry(s, [1, 2], [2])], "wanted place 2 is not among its 2 tokens"),
    (lambda s, t: [StepEntry(s, [1, 2], [-1])], "wanted place -1"),
])
def test_what_a_step_cannot_run_is_refused_before_anything_changes(entries, match):
    eng = fake_engine()
    held = eng.cache.acquire()
    free = next(i for i in range(eng.cache.n_slots) if i != held)
    with pytest.raises(StepError, match=match):
        Engine.plan(eng, entries(held, free))
    assert eng.cache.lengths[held] == 0
    eng.cache.check()


def test_a_sequence_may_fill_the_model_exactly_and_not_go_beyond():
    eng = fake_engine()
    s = eng.cache.acquire()
    eng.cache.reserve(s, 120); eng.cache.advance(s, 120)
    assert Engine.plan(eng, [StepEntry(s, [1] * 8, [7])])["tok_pos"].tolist() == list(range(120, 128))
    with pytest.raises(StepError, match="120 \\+ 9 tokens exceed"):
        Engine.plan(eng, [StepEntry(s, [1] * 9, [8])])
