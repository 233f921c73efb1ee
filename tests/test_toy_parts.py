"""Parts of other kinds than GPT-2's, defined here and never shipped: a position encoding that acts on
queries and keys (a rotation by the token's position), a mixer that applies it and otherwise uses the
library's paged cache and attention kernel, and a feed-forward that routes every token to one of several
experts.  They are registered, chosen layer by layer by a toy configuration, built and stepped without a
change to the framework's files.  They are toys for the interfaces, not models of anyone's.
"""
import dataclasses
import json
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
HEADS = 2


def rotate(t, pos, base):
    """t [..., n, dh] rotated pairwise (first half with second half) by angle pos·base^(−2i/dh)."""
    dh = t.shape[-1]
    inv = base ** (-torch.arange(0, dh // 2, dtype=torch.float64, device=t.device) * 2.0 / dh)
    ang = pos.double()[:, None] * inv[None, :]
    cos, sin = torch.cos(ang).to(t.dtype), torch.sin(ang).to(t.dtype)
    a, b = t[..., :dh // 2], t[..., dh // 2:]
    return torch.cat([a * cos - b * sin, a * sin + b * cos], -1)


def define_toys():
    from vlrf_b200.cache import KVNeed
    from vlrf_b200.config import ModelConfig, key
    from vlrf_b200.csrc import ops
    from vlrf_b200.engine.model import DecoderModel, LayerCall
    from vlrf_b200.parts import LayerNorm, LMHead, PreNormBlock, TokenEmbedding, get_part, register_part
    from vlrf_b200.registry import Architecture, register_architecture
    from vlrf_b200.weights.spec import TensorSpec, place

    @register_part("position", "toy_rotation", replace=True)
    class ToyRotation:
        where = "qk"                                    # a mixer applies it to its queries and keys

        def __init__(self, base: float):
            self.base = float(base)

        def apply(self, t, positions):                  # t [n, heads, dh], positions int32 [n]
            return rotate(t.transpose(0, 1), positions, self.base).transpose(0, 1)

    @register_part("mixer", "toy_rotary_attention", replace=True)
    class ToyRotaryAttention:
        """Projections in torch, the rotation from the position part, then the library's cache append and
        attention kernel."""

        def __init__(self, w_qkv, w_out, *, n_heads, head_dim, scale, position):
            self.w_qkv, self.w_out = w_qkv, w_out
            self.n_heads, self.head_dim, self.scale, self.position = n_heads, head_dim, scale, position

        def cache_need(self):
            return KVNeed(self.n_heads, self.head_dim, "full")

        def forward(self, h, x, ctx, view, writes_cache=True):
            T, H, dh = ctx.n_tokens, self.n_heads, self.head_dim
            qkv = (h @ self.w_qkv.T).view(T, 3, H, dh)
            pos = ctx.tok_pos[:T]
            qkv[:, 0] = self.position.apply(qkv[:, 0], pos)
            qkv[:, 1] = self.position.apply(qkv[:, 1], pos)
            qkv = qkv.reshape(T, 3 * H * dh).contiguous()
            if writes_cache:
                ops.kv_append(qkv, H * dh, 2 * H * dh, view.k, view.v, view.block_table, ctx.tok_slot, ctx.tok_pos, T, H, dh,
                              ctx.dev_err)
            merged = torch.empty(T, H * dh, dtype=qkv.dtype, device=qkv.device)
            ops.attention_generic(qkv, 0, view.k, view.v, view.block_table, ctx.tok_slot, ctx.tok_pos, merged, T, H, H, dh,
                                  self.scale, 0, ctx.dev_err)
            x += (merged @ self.w_out.T).float()

    @register_part("feed_forward", "toy_routed", replace=True)
    class ToyRoutedFeedForward:
        """Every token goes to the expert whose router score is largest (scores in float32)."""
        replayable = False              # the host looks at which tokens each expert got: no graph replay of such a step

        def __init__(self, router, w_in, w_out):
            self.router, self.w_in, self.w_out = router, w_in, w_out       # [E, d], [E, f, d], [E, d, f]

        def forward(self, h, x, ctx):
            T = ctx.n_tokens
            choice = (h[:T].float() @ self.router.float().T).argmax(-1)
            for e in range(self.router.shape[0]):
                rows = (choice == e).nonzero().squeeze(-1)
                if rows.numel():
                    u = torch.nn.functional.gelu(h[rows] @ self.w_in[e].T, approximate="tanh")
                    x[rows] += (u @ self.w_out[e].T).float()

    @dataclasses.dataclass
    class ToyPartsConfig(ModelConfig):
        model_type = "toy_parts"
        vocab_size: int = key()
        width: int = key()
        max_len: int = key()
        eps: float = key()
        rotation_base: float = key()
        n_experts: int = key()
        layer_kinds: str = key()           # per layer "mixer/feed-forward", e.g. "rotary/routed,plain/dense"

    def kinds(cfg):
        return [k.split("/") for k in cfg.layer_kinds.split(",")]

    def spec(cfg):
        d, E = cfg.width, cfg.n_experts
        s = [TensorSpec("emb", (cfg.vocab_size, d))]
        for i, (mix, ffn) in enumerate(kinds(cfg)):
            s += [TensorSpec(f"l{i}.n1", (d,), "vector"), TensorSpec(f"l{i}.n2", (d,), "vector"),
                  TensorSpec(f"l{i}.qkv", (3 * d, d)), TensorSpec(f"l{i}.out", (d, d))]
            if ffn == "routed":
                s += [TensorSpec(f"l{i}.router", (E, d)), TensorSpec(f"l{i}.exp_in", (E, 2 * d, d)),
                      TensorSpec(f"l{i}.exp_out", (E, d, 2 * d))]
            else:
                s += [TensorSpec(f"l{i}.ffn_in", (2 * d, d)), TensorSpec(f"l{i}.ffn_out", (d, 2 * d))]
        return s

    def rand(cfg, gen):
        return {t.name: (1.0 if ".n" in t.name else 0.0) + 0.2 * torch.randn(t.shape, generator=gen) for t in spec(cfg)}

    def build(cfg, weights, options):
        dt, dev = options.dtype, options.device
        m = lambda n: place(weights[n], "matrix", dt, dev)   # noqa: E731
        v = lambda n: place(weights[n], "vector", dt, dev)   # noqa: E731
        zeros = lambda n: torch.zeros(n, device=dev)         # noqa: E731
        d = cfg.width
        scale = 1.0 / math.sqrt(d // HEADS)
        emb = m("emb")
        layers = []
        for i, (mix, ffn) in enumerate(kinds(cfg)):
            if mix == "rotary":
                mixer = get_part("mixer", "toy_rotary_attention")(
                    m(f"l{i}.qkv"), m(f"l{i}.out"), n_heads=HEADS, head_dim=d // HEADS, scale=scale,
                    position=get_part("position", "toy_rotation")(cfg.rotation_base))
            else:
                mixer = get_part("mixer", "causal_self_attention")(m(f"l{i}.qkv"), zeros(3 * d), m(f"l{i}.out"), zeros(d),
                                                                   n_heads=HEADS, n_kv_heads=HEADS, head_dim=d // HEADS,
                                                                   scale=scale)
            if ffn == "routed":
                feed = get_part("feed_forward", "toy_routed")(m(f"l{i}.router"), m(f"l{i}.exp_in"), m(f"l{i}.exp_out"))
            else:
                feed = get_part("feed_forward", "dense_mlp")(m(f"l{i}.ffn_in"), zeros(2 * d), m(f"l{i}.ffn_out"), zeros(d),
                                                             activation="gelu_tanh")
            layers.append(PreNormBlock(LayerNorm(v(f"l{i}.n1"), zeros(d), cfg.eps), mixer,
                                       LayerNorm(v(f"l{i}.n2"), zeros(d), cfg.eps), feed))
        return DecoderModel(config=cfg, embedding=TokenEmbedding(emb), layers=layers,
                            schedule=[LayerCall(i) for i in range(len(layers))],
                            final_norm=LayerNorm(torch.ones(d, device=dev), zeros(d), cfg.eps),
                            head=LMHead(emb), options=options, max_seq_len=cfg.max_len)

    register_architecture(Architecture("toy_parts", ToyPartsConfig, spec, rand, build), replace=True)


def toy_truth(cfg, w, ids):
    """The toy model on one whole sequence, in float64, written out directly; also each token's expert."""
    import plain_gpt2 as plain
    W = {k: v.double() for k, v in w.items()}
    x = W["emb"][torch.tensor(ids)]
    d, n = cfg["width"], len(ids)
    zeros, ones = torch.zeros(d, dtype=torch.float64), torch.ones(d, dtype=torch.float64)
    pos = torch.arange(n)
    scale = 1.0 / math.sqrt(d // HEADS)
    routes = []
    for i, kind in enumerate(cfg["layer_kinds"].split(",")):
        mix, ffn = kind.split("/")
        h = plain.layer_norm(x, W[f"l{i}.n1"], zeros, cfg["eps"])
        q, k, v = (plain.split_heads(t, HEADS) for t in plain.split_qkv(h @ W[f"l{i}.qkv"].T, d))
        if mix == "rotary":
            q, k = rotate(q, pos, cfg["rotation_base"]), rotate(k, pos, cfg["rotation_base"])
        x = x + plain.merge_heads(plain.causal_attention(q, k, v, scale)) @ W[f"l{i}.out"].T
        h = plain.layer_norm(x, W[f"l{i}.n2"], zeros, cfg["eps"])
        if ffn == "routed":
            scores = h @ W[f"l{i}.router"].T
            choice = scores.argmax(-1)
            top2 = scores.topk(2, -1).values
            routes.append((choice, top2[:, 0] - top2[:, 1]))
            y = torch.zeros_like(x)
            for t in range(n):
                e = int(choice[t])
                y[t] = plain.gelu_tanh(h[t] @ W[f"l{i}.exp_in"][e].T) @ W[f"l{i}.exp_out"][e].T
            x = x + y
        else:
            x = x + plain.gelu_tanh(h @ W[f"l{i}.ffn_in"].T) @ W[f"l{i}.ffn_out"].T
    return plain.layer_norm(x, ones, zeros, cfg["eps"]) @ W["emb"].T, routes


def test_rotation_on_queries_and_keys_and_routed_experts_are_registered_built_and_stepped(tmp_path):
    import plain_gpt2 as plain
    from conftest import random_ids, rel_err
    from engine_drives import drive_batches, drive_tail_one_by_one, drive_whole
    from vlrf_b200.engine import Engine, load_model
    from vlrf_b200.parts import get_part
    from vlrf_b200.weights import write_random_model
    define_toys()
    assert get_part("position", "toy_rotation").where == "qk"
    cfg = dict(model_type="toy_parts", vocab_size=70, width=32, max_len=80, eps=1e-5, rotation_base=50.0, n_experts=3,
               layer_kinds="rotary/routed,plain/dense,rotary/dense,plain/routed")
    d = write_random_model(cfg, 5, tmp_path / "toy_parts", dtype=torch.float32)
    assert json.loads((d / "config.json").read_text())["layer_kinds"] == cfg["layer_kinds"]
    _, w = plain.read_model_dir(d)
    model = load_model(d, "float32")
    assert [type(layer.mixer).__name__ for layer in model.layers] == ["ToyRotaryAttention", "CausalSelfAttention"] * 2
    assert [type(layer.feed_forward).__name__ for layer in model.layers] == \
        ["ToyRoutedFeedForward", "DenseMLP", "DenseMLP", "ToyRoutedFeedForward"]
    assert not model.replayable
    eng = Engine(model, max_tokens=256)
    reqs = [random_ids(70, n, 60 + n) for n in (40, 5, 19, 80)]
    truth = [toy_truth(cfg, w, ids) for ids in reqs]
    used = set()
    for _, routes in truth:
        for choice, margin in routes:
            # the comparison below means something only where float32 cannot flip a token's expert
            assert float(margin.min()) > 1e-4
            used |= set(choice.tolist())
    assert used == {0, 1, 2}                          # every expert gets tokens
    for drive, got in (("whole", drive_whole(eng, reqs)),
                       ("one by one", drive_tail_one_by_one(eng, reqs, 32)),
                       ("batches", drive_batches(eng, reqs, 2, [16, 2, 9, 50])),
                       ("batches again", drive_batches(eng, reqs, 2, [16, 2, 9, 50]))):
        for g, (t, _) in zip(got, truth):
            assert rel_err(g, t) < 1e-4, drive
