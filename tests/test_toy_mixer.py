"""A mixer with state of its own, defined here, is registered, built and stepped without touching the
framework's files: a new part, a new architecture, a cache need of fixed size per sequence.

The toy mixer keeps, per sequence, the running sum of its normed inputs and their count, and outputs a
projection of the running mean: out_t = W · mean(h_0 … h_t).  Its state is read before it is written, so
it shows whether a slot's state is zeroed on reuse and whether prefill leaves the state of the last token.
"""
import dataclasses
import json

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def define_toy():
    from vlrf_b200.cache import StateNeed
    from vlrf_b200.config import ModelConfig, key
    from vlrf_b200.engine.model import DecoderModel, LayerCall
    from vlrf_b200.parts import LayerNorm, LMHead, PreNormBlock, TokenEmbedding, get_part, register_part
    from vlrf_b200.registry import Architecture, register_architecture
    from vlrf_b200.weights.spec import TensorSpec, place

    @register_part("mixer", "running_mean", replace=True)
    class RunningMeanMixer:
        def __init__(self, w):
            self.w = w                                  # [width, width] float32
            self.width = w.shape[0]

        def cache_need(self):
            return StateNeed((self.width + 1,), torch.float32)      # the sum, and the count

        def forward(self, h, x, ctx, view, writes_cache=True):
            hf = h.float()
            for i in range(ctx.n_seqs):                 # plain torch: this is a test's toy, not a kernel
                slot = ctx.host_seq_slots[i]
                a = sum(ctx.host_seq_lens[:i])
                n = ctx.host_seq_lens[i]
                st = view.state[slot]
                sums = st[:self.width] + torch.cumsum(hf[a:a + n], 0)
                counts = st[self.width] + torch.arange(1, n + 1, device=h.device, dtype=torch.float32)
                x[a:a + n] += (sums / counts[:, None]) @ self.w.T
                if writes_cache:
                    st[:self.width] = sums[-1]
                    st[self.width] = counts[-1]

    @dataclasses.dataclass
    class ToyConfig(ModelConfig):
        model_type = "toy_state"
        vocab_size: int = key()
        width: int = key()
        n_layer: int = key()
        max_len: int = key()
        eps: float = key()
        layer_mixers: str = key()          # e.g. "running_mean,causal_self_attention,running_mean"

    def spec(cfg):
        s = [TensorSpec("emb", (cfg.vocab_size, cfg.width))]
        for i, kind in enumerate(cfg.layer_mixers.split(",")):
            s += [TensorSpec(f"l{i}.n1", (cfg.width,), "vector"), TensorSpec(f"l{i}.n2", (cfg.width,), "vector"),
                  TensorSpec(f"l{i}.ffn_in", (2 * cfg.width, cfg.width)), TensorSpec(f"l{i}.ffn_out", (cfg.width, 2 * cfg.width))]
            if kind == "running_mean":
                s.append(TensorSpec(f"l{i}.mix", (cfg.width, cfg.width), "vector"))
            else:
                s += [TensorSpec(f"l{i}.qkv", (3 * cfg.width, cfg.width)), TensorSpec(f"l{i}.out", (cfg.width, cfg.width))]
        return s

    def rand(cfg, gen):
        return {t.name: (1.0 if ".n" in t.name else 0.0) + 0.2 * torch.randn(t.shape, generator=gen) for t in spec(cfg)}

    def build(cfg, weights, options):
        dt, dev = options.dtype, options.device
        m = lambda n: place(weights[n], "matrix", dt, dev)   # noqa: E731
        v = lambda n: place(weights[n], "vector", dt, dev)   # noqa: E731
        zeros = lambda n: torch.zeros(n, device=dev)         # noqa: E731
        emb = m("emb")
        layers = []
        for i, kind in enumerate(cfg.layer_mixers.split(",")):
            if kind == "running_mean":
                mixer = get_part("mixer", kind)(v(f"l{i}.mix"))
            else:
                mixer = get_part("mixer", kind)(m(f"l{i}.qkv"), zeros(3 * cfg.width), m(f"l{i}.out"), zeros(cfg.width),
                                                n_heads=2, n_kv_heads=2, head_dim=cfg.width // 2, scale=0.25)
            ffn = get_part("feed_forward", "dense_mlp")(m(f"l{i}.ffn_in"), zeros(2 * cfg.width), m(f"l{i}.ffn_out"),
                                                        zeros(cfg.width), activation="gelu_tanh")
            layers.append(PreNormBlock(LayerNorm(v(f"l{i}.n1"), zeros(cfg.width), cfg.eps), mixer,
                                       LayerNorm(v(f"l{i}.n2"), zeros(cfg.width), cfg.eps), ffn))
        return DecoderModel(config=cfg, embedding=TokenEmbedding(emb), layers=layers,
                            schedule=[LayerCall(i) for i in range(len(layers))],
                            final_norm=LayerNorm(torch.ones(cfg.width, device=dev), zeros(cfg.width), cfg.eps),
                            head=LMHead(emb), options=options, max_seq_len=cfg.max_len)

    register_architecture(Architecture("toy_state", ToyConfig, spec, rand, build), replace=True)


def toy_truth(cfg, w, ids):
    """The toy model on one whole sequence, in float64, written out directly."""
    import plain_gpt2 as plain
    W = {k: v.double() for k, v in w.items()}
    x = W["emb"][torch.tensor(ids)]
    d = cfg["width"]
    zeros, ones = torch.zeros(d, dtype=torch.float64), torch.ones(d, dtype=torch.float64)
    for i, kind in enumerate(cfg["layer_mixers"].split(",")):
        h = plain.layer_norm(x, W[f"l{i}.n1"], zeros, cfg["eps"])
        if kind == "running_mean":
            mean = torch.cumsum(h, 0) / torch.arange(1, len(ids) + 1, dtype=torch.float64)[:, None]
            x = x + mean @ W[f"l{i}.mix"].T
        else:
            qkv = h @ W[f"l{i}.qkv"].T
            q, k, v = (plain.split_heads(t, 2) for t in plain.split_qkv(qkv, d))
            x = x + plain.merge_heads(plain.causal_attention(q, k, v, 0.25)) @ W[f"l{i}.out"].T
        h = plain.layer_norm(x, W[f"l{i}.n2"], zeros, cfg["eps"])
        x = x + plain.gelu_tanh(h @ W[f"l{i}.ffn_in"].T) @ W[f"l{i}.ffn_out"].T
    return plain.layer_norm(x, ones, zeros, cfg["eps"]) @ W["emb"].T


def test_toy_mixer_with_state_is_registered_built_and_stepped(tmp_path):
    import plain_gpt2 as plain
    from conftest import random_ids, rel_err
    from engine_drives import drive_batches, drive_tail_one_by_one, drive_whole
    from vlrf_b200.engine import Engine, load_model
    from vlrf_b200.weights import write_random_model
    define_toy()
    cfg = dict(model_type="toy_state", vocab_size=90, width=32, n_layer=3, max_len=96, eps=1e-5,
               layer_mixers="running_mean,causal_self_attention,running_mean")
    d = write_random_model(cfg, 3, tmp_path / "toy", dtype=torch.float32)
    assert json.loads((d / "config.json").read_text())["model_type"] == "toy_state"
    _, w = plain.read_model_dir(d)
    model = load_model(d, "float32")
    needs = model.cache_needs()
    assert [type(n).__name__ for n in needs] == ["StateNeed", "KVNeed", "StateNeed"]
    eng = Engine(model, max_tokens=256)
    assert len(eng.cache._groups) == 2            # the two state layers share a group; attention has its own
    reqs = [random_ids(90, n, 40 + n) for n in (50, 7, 23, 96)]
    truth = [toy_truth(cfg, w, ids) for ids in reqs]
    for drive, got in (("whole", drive_whole(eng, reqs)),
                       ("one by one", drive_tail_one_by_one(eng, reqs, 32)),
                       ("batches", drive_batches(eng, reqs, 2, [20, 3, 10, 60])),
                       ("batches again", drive_batches(eng, reqs, 2, [20, 3, 10, 60]))):
        for g, t in zip(got, truth):
            assert rel_err(g, t) < 1e-4, drive
