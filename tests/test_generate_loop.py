"""The generation loop's decisions, with a scripted backend (CPU)."""
import pytest

from vlrf_b200.engine.generate import GenerationError, Request, generate, plan_batches, tokens_needed
from vlrf_b200.sampling import SamplingParams


class ScriptedBackend:
    """Every sequence 'generates' prompt[0]+1, +2, …; records what the loop asks for."""

    def __init__(self, max_tokens=1024, n_slots=4, max_seq_len=64):
        self.lim = (max_tokens, n_slots, 64, max_seq_len)
        self.free = list(range(n_slots))
        self.log = []
        self.tables = 0
        self.steps = 0

    def limits(self):
        return self.lim

    def open_table(self, n_rows, requests):
        self.tables += 1
        assert 1 <= n_rows <= self.lim[1]
        return {"slots": [None] * n_rows, "next": [None] * n_rows, "fed": [0] * n_rows, "open": set(), "closed": False}

    def admit(self, h, row, request):
        assert row not in h["open"] and not h["closed"], "a row is given to two requests"
        h["open"].add(row)
        h["slots"][row] = self.free.pop(0)
        h["next"][row] = request.prompt[0]
        h["fed"][row] = 0
        self.log.append(("admit", h["slots"][row], request.index))

    def run(self, h, rows, tokens):
        self.steps += 1
        assert rows == sorted(set(rows)) and set(rows) == h["open"], "a step runs every live row once"
        self.log.append(("run", [h["slots"][r] for r in rows], [len(t) for t in tokens]))
        out = []
        for r, t in zip(rows, tokens):
            assert len(t) == 1 or h["fed"][r] == 0, "only a row just admitted brings more than one token"
            h["fed"][r] += len(t)
            h["next"][r] += 1
            out.append(h["next"][r])
        return out

    def close_row(self, h, row):
        assert row in h["open"], "a row is closed twice"
        h["open"].remove(row)
        self.free.append(h["slots"][row])
        self.log.append(("close", h["slots"][row]))
        h["slots"][row] = None

    def close_table(self, h):
        assert not h["open"] and not h["closed"]
        h["closed"] = True


def greedy(n, **kw):
    return SamplingParams(max_new_tokens=n, do_sample=False, **kw)


def test_first_token_comes_from_the_prompt_step_and_the_last_is_not_fed_back():
    b = ScriptedBackend()
    (r,) = generate(b, [[10, 11, 12]], greedy(4))
    assert r.new_tokens == [11, 12, 13, 14] and r.finish_reason == "length" and r.token_ids == [10, 11, 12, 11, 12, 13, 14]
    runs = [e for e in b.log if e[0] == "run"]
    assert [e[2] for e in runs] == [[3], [1], [1], [1]]          # prompt once, then 3 single tokens: 4 samples
    assert b.free == [1, 2, 3, 0]


def test_stop_tokens_end_sequences_early_and_the_batch_shrinks():
    b = ScriptedBackend()
    params = [greedy(10, stop_token_ids=(13,)), greedy(10), greedy(2)]
    res = generate(b, [[10], [20, 21], [30]], params, eos_token_id=99)
    assert res[0].new_tokens == [11, 12, 13] and res[0].finish_reason == "stop" and res[0].hit_eos
    assert res[1].tokens_generated == 10 and res[1].finish_reason == "length"
    assert res[2].new_tokens == [31, 32] and res[2].finish_reason == "length"
    widths = [len(e[1]) for e in b.log if e[0] == "run"]
    assert widths == [3, 3, 2, 1, 1, 1, 1, 1, 1, 1]
    assert sorted(b.free) == [0, 1, 2, 3]


def test_default_stop_is_the_models_eos():
    b = ScriptedBackend()
    (r,) = generate(b, [[5]], greedy(10), eos_token_id=8)
    assert r.new_tokens == [6, 7, 8] and r.finish_reason == "stop"


def test_context_full_ends_a_sequence():
    b = ScriptedBackend(max_seq_len=8)
    (r,) = generate(b, [[1, 2, 3, 4, 5]], greedy(100))
    assert len(r.token_ids) == 8 and r.finish_reason == "context"
    (r,) = generate(b, [[1] * 8], greedy(5))
    assert r.new_tokens == [] and r.finish_reason == "context"
    with pytest.raises(GenerationError, match="exceeds"):
        generate(b, [[1] * 9], greedy(5))


def test_empty_prompt_starts_from_bos():
    b = ScriptedBackend()
    (r,) = generate(b, [[]], greedy(2), bos_token_id=40)
    assert r.prompt == [40] and r.new_tokens == [41, 42]
    with pytest.raises(GenerationError, match="bos_token_id"):
        generate(b, [[]], greedy(2))


def test_zero_new_tokens_runs_nothing():
    b = ScriptedBackend()
    (r,) = generate(b, [[1, 2]], greedy(0))
    assert r.new_tokens == [] and r.finish_reason == "length" and b.log == []


def test_waiting_requests_take_the_rows_of_those_that_ended():
    b = ScriptedBackend(max_tokens=256, n_slots=2)
    res = generate(b, [[i] for i in range(5)], greedy(3))
    assert [r.new_tokens for r in res] == [[i + 1, i + 2, i + 3] for i in range(5)]
    assert b.tables == 1 and sorted(b.free) == [0, 1]
    # 5 requests of 3 tokens on 2 rows: 3 + 3 + 3 steps, as with whole batches here (they all end together) …
    assert b.steps == 9
    # … but with unequal ends a waiting request joins at the next step boundary instead of waiting for the batch:
    # 10 requests, 4 rows; static batches of 4, 4, 2 would take 12 + 12 + 12 = 36 steps
    b = ScriptedBackend(max_tokens=4096, n_slots=4)
    lens = [12, 2, 3, 2, 12, 1, 1, 2, 12, 3]
    res = generate(b, [[10 * i] for i in range(10)], [greedy(n) for n in lens])
    assert [r.new_tokens for r in res] == [[10 * i + k + 1 for k in range(n)] for i, n in enumerate(lens)]
    assert b.steps == 16 and sorted(b.free) == [0, 1, 2, 3]          # 16 steps, not 36
    # a step that admits a request runs its prompt beside the others' single tokens
    runs = [e for e in b.log if e[0] == "run"]
    assert any(len(set(widths)) > 1 or len(widths) > 1 for _, _, widths in runs)
    admitted = [e[2] for e in b.log if e[0] == "admit"]
    assert admitted == list(range(10))                      # in their order
    # tokens, not only slots, bound a batch: 100-token prompts + 100 new → 256 tokens each
    reqs = [Request([0] * 100, greedy(100), i) for i in range(3)]
    assert tokens_needed(reqs[0], 64, 1024) == 256
    assert [len(x) for x in plan_batches(reqs, 512, 8, 64, 1024)] == [2, 1]
    with pytest.raises(GenerationError, match="cache holds"):
        plan_batches(reqs, 128, 8, 64, 1024)


def test_callback_can_stop_a_sequence():
    b = ScriptedBackend()
    seen = []

    def on_token(index, tok):
        seen.append((index, tok))
        return tok != 12

    (r,) = generate(b, [[10]], greedy(10), on_token=on_token)
    assert r.new_tokens == [11, 12] and r.finish_reason == "stop" and seen == [(0, 11), (0, 12)]


def test_an_error_in_a_step_gives_the_slots_back():
    class Failing(ScriptedBackend):
        def run(self, h, rows, tokens):
            if self.steps >= 2:
                raise RuntimeError("boom")
            return super().run(h, rows, tokens)

    b = Failing()
    with pytest.raises(RuntimeError, match="boom"):
        generate(b, [[1], [2]], greedy(5))
    assert sorted(b.free) == [0, 1, 2, 3]


class HashBackend(ScriptedBackend):
    """The next token is a function of everything the sequence has been fed so far (as with a real model), so a
    token fed twice, skipped or given to the wrong row changes all that follows."""

    def open_table(self, n_rows, requests):
        h = super().open_table(n_rows, requests)
        h["seen"] = [[] for _ in range(n_rows)]
        return h

    def admit(self, h, row, request):
        super().admit(h, row, request)
        h["seen"][row] = []

    def run(self, h, rows, tokens):
        assert len(set(rows)) == len(rows)
        self.steps += 1
        out = []
        for r, t in zip(rows, tokens):
            assert r in h["open"] and len(t) >= 1
            h["seen"][r].extend(t)
            assert len(h["seen"][r]) <= self.lim[3], "a sequence was fed beyond the model's positions"
            out.append(next_token_of(h["seen"][r]))
        held = sum((len(h["seen"][r]) + 63) // 64 * 64 for r in h["open"])
        assert held <= self.lim[0], "the live sequences hold more tokens than the cache has"
        return out


def next_token_of(history):
    x = 17
    for t in history:
        x = (x * 31 + t + 7) % 1009
    return x % 50


def alone(prompt, params, bos, eos, max_seq_len):
    """What one request generates by the rules, computed without the loop."""
    ids = list(prompt) if prompt else [bos]
    stop = params.stop_token_ids if params.stop_token_ids is not None else (eos,)
    new = []
    if params.max_new_tokens == 0:
        return new, "length"
    if len(ids) >= max_seq_len:
        return new, "context"
    while True:
        new.append(next_token_of(ids + new))
        if new[-1] in stop:
            return new, "stop"
        if len(new) >= params.max_new_tokens:
            return new, "length"
        if len(ids) + len(new) >= max_seq_len:
            return new, "context"


@pytest.mark.parametrize("seed", range(12))
def test_any_batching_gives_each_request_what_it_gets_alone(seed):
    import random
    rnd = random.Random(seed)
    max_seq_len = rnd.choice([16, 40, 64])
    n_slots = rnd.choice([1, 2, 3, 5, 8])
    max_tokens = 64 * rnd.choice([n_slots, max(1, n_slots // 2), 2 * n_slots])
    b = HashBackend(max_tokens=max_tokens, n_slots=n_slots, max_seq_len=max_seq_len)
    prompts, params = [], []
    for _ in range(rnd.randint(1, 14)):
        prompts.append([rnd.randrange(50) for _ in range(rnd.choice([0, 1, 2, 5, 9, max_seq_len - 1, max_seq_len]))])
        stop = rnd.choice([None, (), (3,), (1, 2, 3, 4, 5, 6, 7, 8, 9)])
        params.append(SamplingParams(max_new_tokens=rnd.choice([0, 1, 2, 7, 30, 100]), do_sample=False, stop_token_ids=stop))
    res = generate(b, prompts, params, bos_token_id=11, eos_token_id=4)
    assert len(res) == len(prompts)
    for p, sp, r in zip(prompts, params, res):
        want_new, want_reason = alone(p, sp, 11, 4, max_seq_len)
        assert (r.new_tokens, r.finish_reason) == (want_new, want_reason)
        assert r.token_ids == (list(p) if p else [11]) + want_new
    assert sorted(b.free) == list(range(n_slots))                   # every slot came back, none twice
