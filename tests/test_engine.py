"""The engine against the plain implementation: whole requests, the last 32 tokens one by one, batches
of unequal lengths one after another, long decoding and the first tokens — in 32-bit and in bfloat16."""
import pytest
import torch

import plain_gpt2 as plain
from conftest import TOL_BF16, TOL_F32, random_ids, record_error, rel_err
from engine_drives import drive_batches, drive_tail_one_by_one, drive_whole, poison

pytestmark = pytest.mark.gpu

DTYPES = [("float32", TOL_F32), ("bfloat16", TOL_BF16)]
#: request lengths per model: prompts of 5/17/31 and 1/9/40/100 tokens with their decode steps added, and longer ones
LENGTHS = {"tiny_a": [5 + 16, 17 + 16, 31 + 16, 70, 128], "tiny_b": [1 + 24, 9 + 24, 40 + 24, 100 + 24, 200, 256],
           "tiny_c": [3 + 20, 64 + 20, 65 + 20, 127 + 20, 250, 320], "tiny_d": [2 + 12, 33 + 12, 64 + 12, 100, 160],
           "tiny_sharp": [4 + 20, 63 + 20, 130 + 20, 257, 384]}
MODELS = ["tiny_a", "tiny_b", "tiny_c", "tiny_d", "tiny_sharp"]


@pytest.fixture(scope="module")
def requests_and_truth(plain_models):
    out = {}
    for name, (cfg, w) in plain_models.items():
        reqs = [random_ids(cfg["vocab_size"], n, 7 + i) for i, n in enumerate(LENGTHS[name])]
        truth = [plain.logits_all_positions(cfg, w, ids) for ids in reqs]
        out[name] = (reqs, truth)
    return out


def make_engine(model_dirs, name, dtype, max_tokens):
    from vlrf_b200.engine import Engine, load_model
    eng = Engine(load_model(model_dirs[name], dtype), max_tokens=max_tokens)
    poison(eng)
    return eng


def compare(got, truth, tol, what, model="", dtype=""):
    """Every position of every request within `tol`; the worst error is recorded under (what, model, dtype)."""
    worst = 0.0
    for i, (g, t) in enumerate(zip(got, truth)):
        assert g.shape == t.shape, f"{what}: request {i} has shape {tuple(g.shape)}, expected {tuple(t.shape)}"
        assert torch.isfinite(g).all(), f"{what}: request {i} has non-finite logits (something unwritten was read)"
        scale = float(t.abs().max())
        err = (g.double() - t).abs().max(dim=1).values / scale
        bad = (err > tol).nonzero()
        assert bad.numel() == 0, (f"{what}: request {i} (length {len(t)}) first differs at position {int(bad[0])} "
                                  f"with error {float(err[bad[0]]):.3e} of the logit scale (tolerance {tol:.0e})")
        worst = max(worst, float(err.max()))
    record_error(what, model, dtype or ("float32" if tol <= TOL_F32 else "bfloat16"), worst)
    return worst


@pytest.mark.parametrize("dtype,tol", DTYPES)
@pytest.mark.parametrize("name", MODELS)
def test_each_request_alone_and_whole(model_dirs, requests_and_truth, name, dtype, tol):
    reqs, truth = requests_and_truth[name]
    eng = make_engine(model_dirs, name, dtype, 384)
    compare(drive_whole(eng, reqs), truth, tol, "whole", name)
    eng.cache.check()
    assert eng.cache.slots.n_held == 0


@pytest.mark.parametrize("dtype,tol", DTYPES)
@pytest.mark.parametrize("name", MODELS)
def test_last_32_tokens_one_by_one(model_dirs, requests_and_truth, name, dtype, tol):
    reqs, truth = requests_and_truth[name]
    eng = make_engine(model_dirs, name, dtype, 384)
    compare(drive_tail_one_by_one(eng, reqs, 32), truth, tol, "prefix + 32 single tokens", name)


@pytest.mark.parametrize("dtype,tol", DTYPES)
@pytest.mark.parametrize("name", MODELS)
def test_unequal_batches_one_after_another(model_dirs, requests_and_truth, name, dtype, tol):
    reqs, truth = requests_and_truth[name]
    decode = {"tiny_a": 16, "tiny_b": 24, "tiny_c": 20, "tiny_d": 12, "tiny_sharp": 20}[name]
    prompt_lens = [max(1, len(r) - decode) for r in reqs]
    # a cache just large enough for one batch: the second batch must reuse slots and blocks of the first
    batch = 3 if name == "tiny_a" else 4
    order = list(reversed(range(len(reqs))))

    def need_of(rs):
        return max(sum((len(r) + 63) // 64 * 64 for r in rs[b:b + batch]) for b in range(0, len(rs), batch))

    need = max(need_of(reqs), need_of([reqs[i] for i in order]))
    eng = make_engine(model_dirs, name, dtype, need)
    got = drive_batches(eng, reqs, batch, prompt_lens)
    compare(got, truth, tol, "unequal batches", name)
    assert eng.cache.slots.n_held == 0
    # the same again in another order: every slot and block has been used before
    got2 = drive_batches(eng, [reqs[i] for i in order], batch, [prompt_lens[i] for i in order])
    compare(got2, [truth[i] for i in order], tol, "unequal batches, reused cache", name)


@pytest.mark.parametrize("dtype,tol", DTYPES)
def test_long_decoding_from_one_token(model_dirs, plain_models, dtype, tol):
    cfg, w = plain_models["tiny_b"]
    ids = random_ids(cfg["vocab_size"], cfg["n_positions"], 99)
    truth = plain.logits_all_positions(cfg, w, ids)
    eng = make_engine(model_dirs, "tiny_b", dtype, 256)
    got = drive_tail_one_by_one(eng, [ids], tail=len(ids) - 1)
    compare(got, [truth], tol, "decoding all 256 positions")


@pytest.mark.parametrize("dtype,tol", DTYPES)
@pytest.mark.parametrize("name", MODELS)
def test_first_tokens(model_dirs, plain_models, name, dtype, tol):
    cfg, w = plain_models[name]
    reqs = [random_ids(cfg["vocab_size"], n, 50 + n) for n in (1, 2, 3, 1)]
    truth = [plain.logits_all_positions(cfg, w, ids) for ids in reqs]
    eng = make_engine(model_dirs, name, dtype, 256)
    compare(drive_whole(eng, reqs), truth, tol, "first tokens, whole", name)
    compare(drive_batches(eng, reqs, 4, [1, 1, 1, 1]), truth, tol, "first tokens, batch", name)


@pytest.mark.parametrize("dtype,tol", DTYPES)
@pytest.mark.parametrize("name", ["tiny_c", "tiny_d"])
def test_a_batch_of_a_hundred_sequences(model_dirs, plain_models, name, dtype, tol):
    """More sequences in a decode step than the few-row kernels take (64): prompts of 1 to 40 tokens in one
    step, then ten single-token steps of a hundred rows that shrink as the short requests end."""
    cfg, w = plain_models[name]
    reqs = [random_ids(cfg["vocab_size"], 3 + (i * 7) % 40, 100 + i) for i in range(100)]
    truth = [plain.logits_all_positions(cfg, w, ids) for ids in reqs]
    eng = make_engine(model_dirs, name, dtype, 64 * len(reqs))
    got = drive_batches(eng, reqs, len(reqs), [max(1, len(r) - 10) for r in reqs])
    compare(got, truth, tol, "a batch of 100", name)
    assert eng.cache.slots.n_held == 0


def test_step_refuses_what_it_cannot_run(model_dirs):
    from vlrf_b200.cache import CacheError
    from vlrf_b200.engine import StepEntry, StepError
    eng = make_engine(model_dirs, "tiny_a", "float32", 192)
    s = eng.start_sequence()
    with pytest.raises(StepError, match="outside the vocabulary"):
        eng.step([StepEntry(s, [512], [0])])
    with pytest.raises(StepError, match="at least one token"):
        eng.step([StepEntry(s, [], [])])
    with pytest.raises(StepError, match="wanted place"):
        eng.step([StepEntry(s, [1, 2], [2])])
    with pytest.raises(StepError, match="exceed"):
        eng.step([StepEntry(s, [1] * 129, [])])
    with pytest.raises(StepError, match="twice"):
        eng.step([StepEntry(s, [1], []), StepEntry(s, [2], [])])
    with pytest.raises(StepError, match="not held"):
        eng.step([StepEntry(5, [1], [])])
    assert eng.length(s) == 0
    eng.step([StepEntry(s, [1] * 100, [])])
    s2 = eng.start_sequence()
    with pytest.raises(CacheError, match="cache full"):
        eng.step([StepEntry(s2, [1] * 65, [0])])
    assert eng.step([StepEntry(s2, [1] * 3, [])]).shape == (0, 512)
    eng.check_device_errors()


# ------------------------------------------------------------------------------------------------
# The real widths of GPT-2 small (768 wide, 12 heads of 64, inner 3072, vocabulary 50257, 1024 positions)
# with two layers: the tensor-core kernels meet the sizes they serve, tails of the vocabulary included.
GPT2_WIDE = dict(model_type="gpt2", n_layer=2, n_embd=768, n_head=12, n_inner=None, vocab_size=50257, n_positions=1024,
                 layer_norm_epsilon=1e-5, activation_function="gelu_new", scale_attn_by_inverse_layer_idx=False,
                 tie_word_embeddings=True, bos_token_id=50256, eos_token_id=50256)


#: the widths of GPT-2 XL (1600 wide, 25 heads of 64, inner 6400) with one layer and a small vocabulary
GPT2_XL_WIDE = dict(GPT2_WIDE, n_layer=1, n_embd=1600, n_head=25, vocab_size=1003, n_positions=512,
                    bos_token_id=1, eos_token_id=2)
WIDE = {"small": (GPT2_WIDE, 50257), "xl": (GPT2_XL_WIDE, 1003)}


@pytest.fixture(scope="module", params=["small", "xl"])
def wide_model(request, tmp_path_factory):
    from vlrf_b200.weights import write_random_model
    cfg_dict, vocab = WIDE[request.param]
    d = tmp_path_factory.mktemp("gpt2_wide_" + request.param)
    write_random_model(cfg_dict, 321, d)
    cfg, w = plain.read_model_dir(d)
    reqs = [random_ids(vocab, n, 400 + n) for n in (70, 150, 9)]
    truth = [plain.logits_all_positions(cfg, w, ids) for ids in reqs]
    return d, reqs, truth


@pytest.mark.parametrize("dtype,tol", DTYPES)
def test_gpt2_real_widths_whole_tail_and_batch(wide_model, dtype, tol):
    from vlrf_b200.engine import Engine, load_model
    d, reqs, truth = wide_model
    eng = Engine(load_model(d, dtype), max_tokens=64 * 8)
    poison(eng)
    compare(drive_whole(eng, reqs), truth, tol, "GPT-2 widths, whole")
    compare(drive_tail_one_by_one(eng, reqs, 20), truth, tol, "GPT-2 widths, prefix + 20 single tokens")
    compare(drive_batches(eng, reqs, 3, [50, 130, 1]), truth, tol, "GPT-2 widths, unequal batch")
    assert eng.cache.slots.n_held == 0


def test_launch_chaining_changes_no_bit(wide_model):
    """Kernels that begin while those ahead still run (and fetch weights, earlier keys and values ahead of
    their wait) must give exactly what plain stream order gives: the same logits, bit for bit, over prompt
    steps, decode steps and a replayed decode session."""
    from vlrf_b200.csrc import ops
    from vlrf_b200.engine import Engine, StepEntry, load_model
    from vlrf_b200.engine.decode import DecodeSession
    d, reqs, _ = wide_model
    model = load_model(d, "bfloat16")

    def run():
        eng = Engine(model, max_tokens=64 * 8)
        poison(eng)
        got = drive_tail_one_by_one(eng, reqs, 12)
        long = [r for r in reqs if len(r) > 41]
        slots = [eng.start_sequence() for _ in long]
        eng.step([StepEntry(s, r[:40], []) for s, r in zip(slots, long)])
        sess = DecodeSession(eng, slots, use_graph=True)
        sess.reserve_ahead(8)
        sess.set_tokens([r[40] for r in long])
        out = torch.zeros(len(slots), dtype=torch.int32, device=eng.device)
        for _ in range(6):
            got.append(sess.step_greedy(out).float().cpu().clone())
        for s in slots:
            eng.end_sequence(s)
        return got

    try:
        chained = run()
        ops.set_chained_launch(False)
        plain_order = run()
    finally:
        ops.set_chained_launch(True)
    assert len(chained) == len(plain_order)
    for a, b in zip(chained, plain_order):
        assert torch.equal(a, b)


@pytest.mark.parametrize("dtype,tol", DTYPES)
def test_decoding_to_the_last_position_at_xl_width(tmp_path, dtype, tol):
    """A prompt step, then a replayed decode session up to the model's last position, with a shorter sequence
    that ends on the way and stays in the batch as padding."""
    from vlrf_b200.engine import Engine, StepEntry, load_model
    from vlrf_b200.engine.decode import DecodeSession
    from vlrf_b200.weights import write_random_model
    d = write_random_model(GPT2_XL_WIDE, 77, tmp_path / "xl_wide")
    cfg, w = plain.read_model_dir(d)
    last = GPT2_XL_WIDE["n_positions"]
    reqs = [random_ids(1003, last, 500), random_ids(1003, 300, 501)]
    truth = [plain.logits_all_positions(cfg, w, ids) for ids in reqs]
    eng = Engine(load_model(d, dtype), max_tokens=2 * last)
    poison(eng)
    slots = [eng.start_sequence() for _ in reqs]
    pos = [400, 250]
    got = eng.step([StepEntry(s, r[:n], [n - 1]) for s, r, n in zip(slots, reqs, pos)]).float().cpu()
    for i, n in enumerate(pos):
        assert rel_err(got[i], truth[i][n - 1]) < tol
    sess = DecodeSession(eng, slots, use_graph=True)
    sess.reserve_ahead(last)
    while any(p < len(r) for p, r in zip(pos, reqs)):
        sess.set_tokens([r[min(p, len(r) - 1)] for r, p in zip(reqs, pos)])
        lg = sess.step().float().cpu()
        for i, r in enumerate(reqs):
            if pos[i] < len(r):
                assert rel_err(lg[i], truth[i][pos[i]]) < tol, (i, pos[i])
                pos[i] += 1
                if pos[i] == len(r):
                    sess.end_row(i)
    eng.check_device_errors()
    for s in slots:
        eng.end_sequence(s)
    assert eng.cache.slots.n_held == 0


def test_prompt_attention_dealt_to_parts_inside_the_engine(tmp_path, monkeypatch):
    """Long query tiles whose keys are dealt to several CTAs (forced here; the choice is by size otherwise):
    the mixer hands the scratch, the step is run three times so that it is captured and replayed, and every
    run gives the plain implementation's logits and the same bits."""
    from vlrf_b200.csrc import ops
    from vlrf_b200.engine import Engine, StepEntry, load_model
    from vlrf_b200.weights import write_random_model
    d = write_random_model(GPT2_XL_WIDE, 78, tmp_path / "xl_wide")
    cfg, w = plain.read_model_dir(d)
    reqs = [random_ids(1003, 512, 510), random_ids(1003, 300, 511)]
    rows = [[0, 127, 128, 400, 511], [5, 255, 299]]
    truth = [plain.logits_all_positions(cfg, w, ids) for ids in reqs]
    monkeypatch.setattr(ops, "PREFILL_ATTENTION_PARTS", 2)
    eng = Engine(load_model(d, "bfloat16"), max_tokens=1024)
    poison(eng)
    runs = []
    for _ in range(3):
        slots = [eng.start_sequence() for _ in reqs]
        runs.append(eng.step([StepEntry(s, r, want) for s, r, want in zip(slots, reqs, rows)]).float().cpu().clone())
        for s in slots:
            eng.end_sequence(s)
    eng.check_device_errors()
    at = 0
    for i, want in enumerate(rows):
        for r in want:
            assert rel_err(runs[0][at], truth[i][r]) < TOL_BF16, (i, r)
            at += 1
    assert torch.equal(runs[0], runs[1]) and torch.equal(runs[0], runs[2])
