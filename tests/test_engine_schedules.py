"""Schedules of steps that the other engine tests do not run, each against the plain implementation in 32-bit and in
bfloat16: a replayed prompt-step graph fed other lengths and start positions than it was captured with; prompts that
arrive in portions, in a step that also holds a new prompt and a one-token row; and the decode session that
generation really uses (rows padded to a power of two, a captured graph, a split count chosen for the model's last
position) held against the plain logits at every tiny configuration."""
import pytest
import torch

import plain_gpt2 as plain
from conftest import TOL_BF16, TOL_F32, random_ids, record_error, rel_err
from engine_drives import poison

pytestmark = pytest.mark.gpu
DTYPES = [("float32", TOL_F32), ("bfloat16", TOL_BF16)]
MODELS = ["tiny_a", "tiny_b", "tiny_c", "tiny_d", "tiny_sharp"]


def engine_of(model_dirs, name, dtype, max_tokens):
    from vlrf_b200.engine import Engine, load_model
    eng = Engine(load_model(model_dirs[name], dtype), max_tokens=max_tokens)
    poison(eng)
    return eng


def check(got, truth, rows, tol, what, name, dtype):
    """got [len(rows), vocab] against truth[rows]."""
    err = rel_err(got, truth[rows])
    assert torch.isfinite(got).all() and err < tol, (what, err)
    record_error(what, name, dtype, err)


@pytest.mark.parametrize("dtype,tol", DTYPES)
@pytest.mark.parametrize("name", MODELS)
def test_a_replayed_prompt_step_takes_other_lengths_and_start_positions(model_dirs, plain_models, name, dtype, tol):
    """The engine captures a prompt step the second time it sees a shape (tokens, sequences, longest run, wanted rows)
    and replays it from then on.  Lengths (a, b, c) three times, then (a, b', c') with the same sum, then (a, b, c)
    continued from position p: all of the same shape, so the later ones run the graph captured for the first."""
    from vlrf_b200.engine import StepEntry
    cfg, w = plain_models[name]
    P = cfg["n_positions"]
    a, b, c, p = (100, 30, 20, 40) if P >= 160 else (60, 20, 12, 30)
    vocab = cfg["vocab_size"]
    eng = engine_of(model_dirs, name, dtype, 64 * 12)
    replays_before = len(eng._graphs)

    def run(lens, starts, seeds, what):
        reqs = [random_ids(vocab, s + n, seed) for n, s, seed in zip(lens, starts, seeds)]
        truth = [plain.logits_all_positions(cfg, w, ids) for ids in reqs]
        slots = [eng.start_sequence() for _ in reqs]
        if any(starts):
            eng.step([StepEntry(sl, r[:s], []) for sl, r, s in zip(slots, reqs, starts) if s > 0])
        want = [[0, n // 2, n - 1] for n in lens]
        got = eng.step([StepEntry(sl, r[s:], wn) for sl, r, s, wn in zip(slots, reqs, starts, want)]).float().cpu()
        at = 0
        for i, (s, wn) in enumerate(zip(starts, want)):
            check(got[at:at + 3], truth[i], [s + k for k in wn], tol, what, name, dtype)
            at += 3
        for sl in slots:
            eng.end_sequence(sl)
        eng.check_device_errors()

    for rep in range(3):
        run((a, b, c), (0, 0, 0), (11, 12, 13), f"prompt step, repeat {rep}")
    assert len(eng._graphs) == replays_before + 1                   # captured by now
    run((a, b - 5, c + 5), (0, 0, 0), (14, 15, 16), "replayed prompt step, other lengths")
    run((a, b, c), (p, 0, p // 2), (17, 18, 19), "replayed prompt step, other start positions")
    run((a, b, c), (0, 0, 0), (11, 12, 13), "replayed prompt step, the first lengths again")
    eng.cache.check()
    assert eng.cache.slots.n_held == 0


@pytest.mark.parametrize("dtype,tol", DTYPES)
@pytest.mark.parametrize("name", MODELS)
def test_prompts_in_portions_beside_a_new_prompt_and_a_single_token(model_dirs, plain_models, name, dtype, tol):
    """Sequence A gets 40 tokens, then 30 more in a step that also brings a whole new prompt B and one token of C
    (which has been decoding); then all three go on by single tokens.  Every position's logits are wanted."""
    from vlrf_b200.engine import StepEntry
    cfg, w = plain_models[name]
    vocab = cfg["vocab_size"]
    A, B, C = (random_ids(vocab, n, 200 + n) for n in (78, 23, 31))
    truth = {k: plain.logits_all_positions(cfg, w, ids) for k, ids in (("A", A), ("B", B), ("C", C))}
    eng = engine_of(model_dirs, name, dtype, 64 * 6)
    sa, sc = eng.start_sequence(), eng.start_sequence()
    got = eng.step([StepEntry(sa, A[:40], list(range(40))), StepEntry(sc, C[:20], list(range(20)))]).float().cpu()
    check(got[:40], truth["A"], list(range(40)), tol, "portions: first portion", name, dtype)
    check(got[40:], truth["C"], list(range(20)), tol, "portions: first portion", name, dtype)
    got = eng.step([StepEntry(sc, [C[20]], [0])]).float().cpu()
    check(got, truth["C"], [20], tol, "portions: one token", name, dtype)
    sb = eng.start_sequence()
    got = eng.step([StepEntry(sa, A[40:70], list(range(30))), StepEntry(sb, B[:17], list(range(17))),
                    StepEntry(sc, [C[21]], [0])]).float().cpu()
    check(got[:30], truth["A"], list(range(40, 70)), tol, "portions: second portion beside a new prompt and one token", name, dtype)
    check(got[30:47], truth["B"], list(range(17)), tol, "portions: a new prompt beside a portion", name, dtype)
    check(got[47:], truth["C"], [21], tol, "portions: one token beside prompts", name, dtype)
    # a two-token portion, then single tokens for all
    got = eng.step([StepEntry(sa, A[70:72], [0, 1]), StepEntry(sb, [B[17]], [0]), StepEntry(sc, [C[22]], [0])]).float().cpu()
    check(got[:2], truth["A"], [70, 71], tol, "portions: a two-token portion", name, dtype)
    check(got[2:3], truth["B"], [17], tol, "portions: one token", name, dtype)
    fed = {"A": 72, "B": 18, "C": 23}
    seqs = {"A": (sa, A), "B": (sb, B), "C": (sc, C)}
    while any(fed[k] < len(seqs[k][1]) for k in seqs):
        live = [k for k in seqs if fed[k] < len(seqs[k][1])]
        got = eng.step([StepEntry(seqs[k][0], [seqs[k][1][fed[k]]], [0]) for k in live]).float().cpu()
        for r, k in enumerate(live):
            check(got[r:r + 1], truth[k], [fed[k]], tol, "portions: decoding after them", name, dtype)
            fed[k] += 1
    eng.check_device_errors()
    for k in seqs:
        eng.end_sequence(seqs[k][0])
    eng.cache.check()


@pytest.mark.parametrize("dtype,tol", DTYPES)
@pytest.mark.parametrize("name", MODELS)
@pytest.mark.parametrize("use_graph", [False, True])
def test_the_decode_session_of_generation_gives_the_plain_logits(model_dirs, plain_models, name, dtype, tol, use_graph):
    """Five sequences in a session padded to eight rows, up to the model's last position; rows end on the way and one
    row is taken by another sequence (as the generation loop does when a request was waiting)."""
    from vlrf_b200.engine import StepEntry
    from vlrf_b200.engine.decode import DecodeSession
    cfg, w = plain_models[name]
    vocab, P = cfg["vocab_size"], cfg["n_positions"]
    lens = [P, P - 41, 66, 9, 30]
    starts = [P - 50, 64, 63, 1, 17]
    reqs = [random_ids(vocab, n, 600 + i) for i, n in enumerate(lens)]
    late = random_ids(vocab, 40, 700)                       # takes the row of the request that ends first
    truth = [plain.logits_all_positions(cfg, w, ids) for ids in reqs]
    late_truth = plain.logits_all_positions(cfg, w, late)
    eng = engine_of(model_dirs, name, dtype, 64 * 40)
    slots = [eng.start_sequence() for _ in reqs]
    eng.step([StepEntry(s, r[:n], []) for s, r, n in zip(slots, reqs, starts)])
    sess = DecodeSession(eng, slots, use_graph=use_graph, pad_to=8, use_program=False)
    sess.reserve_ahead(P)
    at = list(starts)
    rows = list(reqs)
    row_truth = list(truth)
    taken = False
    while any(p < len(r) for p, r in zip(at, rows)):
        sess.set_tokens([r[min(p, len(r) - 1)] for r, p in zip(rows, at)])
        lg = sess.step().float().cpu()
        for i, r in enumerate(rows):
            if at[i] < len(r):
                check(lg[i:i + 1], row_truth[i], [at[i]], tol, f"decode session (graph {use_graph})", name, dtype)
                at[i] += 1
                if at[i] == len(r):
                    sess.end_row(i)
                    eng.end_sequence(sess.slots[i])
                    if not taken:                            # another sequence takes the freed row: its prompt, then the session
                        taken = True
                        slot = eng.start_sequence()
                        first = eng.step([StepEntry(slot, late[:12], [11])]).float().cpu()
                        check(first, late_truth, [11], tol, "decode session: a prompt between its steps", name, dtype)
                        sess.take_row(i, slot)
                        eng.cache.reserve(slot, len(late))
                        eng.cache.sync_tables()
                        sess.sync_tables()
                        rows[i], row_truth[i], at[i] = late, late_truth, 12
    eng.check_device_errors()
    for i, s in enumerate(sess.slots):
        if sess.live[i]:
            eng.end_sequence(s)
    eng.cache.check()
