"""The plain implementation against the reference's own CPU code (stored logits) and against itself.

tests/golden/*.npz hold logits that VLRF-org/VLRF's model code produced (tests/golden/make_golden.py);
the weights are drawn again here from the same seeds."""
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_gpt2 as plain

GOLDEN = Path(__file__).parent / "golden"
sys.path.insert(0, str(GOLDEN))
import make_golden  # noqa: E402


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b_tanh"])
def test_plain_matches_the_reference_code(name):
    case = make_golden.CASES[name]
    gold = np.load(GOLDEN / f"{name}.npz")
    cfg = case["cfg"]
    w = {k: v.double() for k, v in make_golden.draw_weights(cfg, case["seed"]).items()}
    ids = make_golden.draw_ids(cfg, case["seed"], case["n_ids"])
    full = plain.logits_all_positions(cfg, w, ids).numpy()
    mine = np.stack([full[p - 1] for p in case["prefixes"]] + [full[-1]])
    ref = gold["reference_logits"]
    assert ref.shape == mine.shape
    assert np.abs(ref - mine).max() <= 2e-6 * np.abs(mine).max() + 1e-6   # float32 reference vs float64 plain


def test_causality_a_later_token_changes_nothing_earlier(plain_models):
    cfg, w = plain_models["tiny_b"]
    ids = list(range(3, 40))
    a = plain.logits_all_positions(cfg, w, ids)
    ids2 = list(ids)
    ids2[30] = 999
    b = plain.logits_all_positions(cfg, w, ids2)
    assert torch.equal(a[:30], b[:30]) and not torch.allclose(a[30:], b[30:])


def test_parts_against_torch_builtins():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(7, 24, generator=g, dtype=torch.float64)
    gamma, beta = torch.randn(24, generator=g, dtype=torch.float64), torch.randn(24, generator=g, dtype=torch.float64)
    assert torch.allclose(plain.layer_norm(x, gamma, beta, 1e-5), torch.nn.functional.layer_norm(x, (24,), gamma, beta, 1e-5))
    assert torch.allclose(plain.gelu_erf(x), torch.nn.functional.gelu(x))
    assert torch.allclose(plain.gelu_tanh(x), torch.nn.functional.gelu(x, approximate="tanh"))
    q, k, v = (torch.randn(2, 9, 8, generator=g, dtype=torch.float64) for _ in range(3))
    want = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True, scale=0.3)
    assert torch.allclose(plain.causal_attention(q, k, v, 0.3), want)
    h = plain.split_heads(x, 3)
    assert h.shape == (3, 7, 8) and torch.equal(plain.merge_heads(h), x) and torch.equal(h[1, 2], x[2, 8:16])


def test_window_hides_old_keys():
    g = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn(1, 12, 4, generator=g, dtype=torch.float64) for _ in range(3))
    full = plain.causal_attention(q, k, v, 0.5)
    win = plain.causal_attention(q, k, v, 0.5, window=3)
    assert torch.allclose(full[:, :3], win[:, :3]) and not torch.allclose(full[:, 5:], win[:, 5:])
    # the query at position 7 sees keys 5, 6, 7 only
    alone = plain.causal_attention(q[:, 7:8], k[:, 5:8], v[:, 5:8], 0.5)   # causal mask of a 1-row query sees key 0 only
    s = (q[0, 7] @ k[0, 5:8].T) * 0.5
    p = torch.softmax(s, -1)
    assert torch.allclose(win[0, 7], p @ v[0, 5:8])
    del alone


def test_sampler_rules():
    logits = np.log(np.array([0.5, 0.3, 0.15, 0.05]))
    assert plain.sample_token(logits, 0.0, 0, 1.0, 0.99) == 0                      # temperature ≤ 0: argmax
    assert plain.argmax_first([1.0, 3.0, 3.0]) == 1                                # first maximal index
    assert [plain.sample_token(logits, 1.0, 0, 1.0, u) for u in (0.0, 0.49, 0.51, 0.79, 0.81, 0.96)] == [0, 0, 1, 1, 2, 3]
    assert plain.sample_token(logits, 1.0, 2, 1.0, 0.99) == 1                      # top-k 2 → {0,1}
    assert plain.sample_token(logits, 1.0, 0, 0.9, 0.99) == 1                      # cum .5,.8,.95>.9 → cut from rank 2
    assert plain.sample_token(logits, 1.0, 0, 0.4, 0.99) == 0                      # the most probable always stays
    pen = plain.apply_penalties([2.0, -2.0, 1.0], {0: 2, 1: 1}, 2.0, 0.5, 0.25)
    assert np.allclose(pen, [2.0 / 2 - 1.0 - 0.25, -4.0 - 0.5 - 0.25, 1.0])
    blocked = plain.block_repeated_ngrams(np.zeros(10), [1, 2, 3, 1, 2], 3)
    assert blocked[3] == -np.inf and np.isfinite(np.delete(blocked, 3)).all()
    assert np.isfinite(plain.block_repeated_ngrams(np.zeros(10), [1, 2, 3, 1, 2], 0)).all()


def test_greedy_generate_stops(plain_models):
    cfg, w = plain_models["tiny_a"]
    out = plain.greedy_generate(cfg, w, [1, 2, 3], 5)
    assert len(out) == 5
    out2 = plain.greedy_generate(cfg, w, [1, 2, 3], 5, stop_ids=(out[1],))
    assert out2 == out[:out.index(out[1]) + 1]
