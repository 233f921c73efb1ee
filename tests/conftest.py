import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
for p in (str(ROOT), str(ROOT / "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

#: two tiny GPT-2 configurations that differ in every size and option
TINY_A = dict(model_type="gpt2", n_layer=2, n_embd=64, n_head=4, n_inner=256, vocab_size=512, n_positions=128,
              layer_norm_epsilon=1e-5, activation_function="gelu_new", scale_attn_by_inverse_layer_idx=False,
              tie_word_embeddings=True, bos_token_id=0, eos_token_id=0)
TINY_B = dict(model_type="gpt2", n_layer=3, n_embd=96, n_head=3, n_inner=320, vocab_size=1000, n_positions=256,
              layer_norm_epsilon=1e-6, activation_function="gelu", scale_attn_by_inverse_layer_idx=True,
              tie_word_embeddings=True, bos_token_id=1, eos_token_id=2)
#: a third one with the head size of the real GPT-2 family (64), so that the kernels that serving uses
#: (tensor-core prompt attention, bulk-copy decode attention) run inside the engine tests too
TINY_C = dict(model_type="gpt2", n_layer=2, n_embd=192, n_head=3, n_inner=None, vocab_size=777, n_positions=320,
              layer_norm_epsilon=1e-5, activation_function="gelu_new", scale_attn_by_inverse_layer_idx=False,
              tie_word_embeddings=True, bos_token_id=5, eos_token_id=6)
#: a fourth one whose width (80 = 5 heads of 16) and inner size (136) are no multiples of 32 and whose vocabulary
#: is odd: tails in every product, no fused norm, row statistics with a short last segment
TINY_D = dict(model_type="gpt2", n_layer=2, n_embd=80, n_head=5, n_inner=136, vocab_size=333, n_positions=160,
              layer_norm_epsilon=1e-5, activation_function="gelu_new", scale_attn_by_inverse_layer_idx=True,
              tie_word_embeddings=True, bos_token_id=3, eos_token_id=4)
TINY = {"tiny_a": TINY_A, "tiny_b": TINY_B, "tiny_c": TINY_C, "tiny_d": TINY_D}

#: tolerances, fixed before the first measurement: the largest absolute logit error over the logit scale
#: (largest absolute logit of the plain implementation)
TOL_F32 = 1e-4
TOL_BF16 = 3e-2


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """Model folders of the two tiny configurations, written by the random-weights mode."""
    import vlrf_b200.models  # noqa: F401
    from vlrf_b200.weights import write_random_model
    out = {}
    for i, (name, cfg) in enumerate(TINY.items()):
        d = tmp_path_factory.mktemp(name)
        write_random_model(cfg, 100 + i, d)
        out[name] = d
    return out


@pytest.fixture(scope="session")
def plain_models(model_dirs):
    """(config dict, float64 weights) of each tiny model, read by the plain implementation's own reader."""
    import plain_gpt2
    return {name: plain_gpt2.read_model_dir(d) for name, d in model_dirs.items()}


def random_ids(vocab, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def rel_err(got, want):
    """Largest absolute difference over the largest absolute wanted value."""
    got = torch.as_tensor(got, dtype=torch.float64)
    want = torch.as_tensor(want, dtype=torch.float64)
    return float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))
