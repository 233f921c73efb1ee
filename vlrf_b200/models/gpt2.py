"""GPT-2: which tensors it has, how random ones are drawn, and how its parts are put together.

Tensor names and layouts are those of a Hugging Face checkpoint (reference:
tools/converter/convert_gpt2.py:98-139): `wte`, `wpe`, per layer `ln_1`, `attn.c_attn` (fused q/k/v,
Conv1D layout [in, out]), `attn.c_proj`, `ln_2`, `mlp.c_fc`, `mlp.c_proj`, and `ln_f`.  The reference's
converter transposes the Conv1D matrices and splits c_attn offline (:114-135); here they are transposed
once at load to [out, in] and c_attn stays fused, so every product is x·Wᵀ with the contraction
contiguous (include/model/compute.hpp:64-68).

The block is the pre-norm one (include/model/transformer_block.hpp:149-159): learned absolute
positions at the embedding, LayerNorm with bias, causal multi-head attention, a GELU MLP, a final
LayerNorm and a head tied to the embedding unless config.json says otherwise.
"""
from __future__ import annotations

import math

import torch

from ..config.gpt2 import GPT2Config
from ..engine.model import BuildOptions, DecoderModel, LayerCall
from ..parts import LMHead, TokenEmbedding, get_part
from ..registry import Architecture, register_architecture
from ..weights.spec import CheckedWeights, TensorSpec, place


def layer_layouts(cfg: GPT2Config) -> list[dict]:
    """Which parts each layer is made of.  GPT-2's layers are all alike; an architecture whose layers
    differ returns different entries here and nothing else changes."""
    return [dict(block="pre_norm", norm="layernorm", mixer="causal_self_attention", feed_forward="dense_mlp")
            for _ in range(cfg.n_layer)]


def weight_spec(cfg: GPT2Config) -> list[TensorSpec]:
    d, f = cfg.n_embd, cfg.inner_dim
    specs = [TensorSpec("wte.weight", (cfg.vocab_size, d)), TensorSpec("wpe.weight", (cfg.n_positions, d))]
    for i in range(cfg.n_layer):
        p = f"h.{i}."
        specs += [
            TensorSpec(p + "ln_1.weight", (d,), "vector"), TensorSpec(p + "ln_1.bias", (d,), "vector"),
            TensorSpec(p + "attn.c_attn.weight", (d, 3 * d)), TensorSpec(p + "attn.c_attn.bias", (3 * d,), "vector"),
            TensorSpec(p + "attn.c_proj.weight", (d, d)), TensorSpec(p + "attn.c_proj.bias", (d,), "vector"),
            TensorSpec(p + "ln_2.weight", (d,), "vector"), TensorSpec(p + "ln_2.bias", (d,), "vector"),
            TensorSpec(p + "mlp.c_fc.weight", (d, f)), TensorSpec(p + "mlp.c_fc.bias", (f,), "vector"),
            TensorSpec(p + "mlp.c_proj.weight", (f, d)), TensorSpec(p + "mlp.c_proj.bias", (d,), "vector"),
        ]
    specs += [TensorSpec("ln_f.weight", (d,), "vector"), TensorSpec("ln_f.bias", (d,), "vector")]
    if not cfg.tie_word_embeddings:
        specs.append(TensorSpec("lm_head.weight", (cfg.vocab_size, d)))
    return specs


def random_weights(cfg: GPT2Config, gen: torch.Generator) -> dict:
    """Matrices N(0, 0.02), the two output projections scaled by 1/sqrt(2·n_layer), biases N(0, 0.01),
    norm weights 1 + N(0, 0.02) and norm biases N(0, 0.02), so that no term of a formula is hidden by a
    zero or a one.  (The reference's random_init draws N(0, 0.02) matrices with zero biases and unit
    norms: include/model/transformer.hpp:566-629.)"""
    out = {}
    for spec in weight_spec(cfg):
        t = torch.randn(spec.shape, generator=gen, dtype=torch.float32)
        name = spec.name
        if name.endswith("ln_1.weight") or name.endswith("ln_2.weight") or name == "ln_f.weight":
            t = 1.0 + 0.02 * t
        elif ".ln_" in name or name.startswith("ln_f"):
            t = 0.02 * t
        elif name.endswith(".bias"):
            t = 0.01 * t
        elif name.endswith("c_proj.weight"):
            t = 0.02 / math.sqrt(2.0 * cfg.n_layer) * t
        else:
            t = 0.02 * t
        out[name] = t
    return out


def build(cfg: GPT2Config, weights: CheckedWeights, options: BuildOptions) -> DecoderModel:
    dt, dev = options.dtype, options.device

    def matrix(name, transpose=False):
        t = weights[name]
        if transpose:                      # Conv1D [in, out] → [out, in]
            t = t.t()
        return place(t, "matrix", dt, dev)

    def vector(name):
        return place(weights[name], "vector", dt, dev)

    positions = get_part("position", "learned_absolute")(matrix("wpe.weight"))
    wte = matrix("wte.weight")
    embedding = TokenEmbedding(wte, positions)
    head_dim = cfg.head_dim
    layers = []
    for i, layout in enumerate(layer_layouts(cfg)):
        p = f"h.{i}."
        norm_cls = get_part("norm", layout["norm"])
        scale = 1.0 / math.sqrt(head_dim) if cfg.scale_attn_weights else 1.0
        if cfg.scale_attn_by_inverse_layer_idx:
            scale = scale / float(i + 1)
        mixer = get_part("mixer", layout["mixer"])(
            matrix(p + "attn.c_attn.weight", True), vector(p + "attn.c_attn.bias"),
            matrix(p + "attn.c_proj.weight", True), vector(p + "attn.c_proj.bias"),
            n_heads=cfg.n_head, n_kv_heads=cfg.n_head, head_dim=head_dim, scale=scale, position=positions)
        ffn = get_part("feed_forward", layout["feed_forward"])(
            matrix(p + "mlp.c_fc.weight", True), vector(p + "mlp.c_fc.bias"),
            matrix(p + "mlp.c_proj.weight", True), vector(p + "mlp.c_proj.bias"), activation=cfg.activation)
        layers.append(get_part("block", layout["block"])(
            norm_cls(vector(p + "ln_1.weight"), vector(p + "ln_1.bias"), cfg.layer_norm_epsilon), mixer,
            norm_cls(vector(p + "ln_2.weight"), vector(p + "ln_2.bias"), cfg.layer_norm_epsilon), ffn))
    final_norm = get_part("norm", "layernorm")(vector("ln_f.weight"), vector("ln_f.bias"), cfg.layer_norm_epsilon)
    head = LMHead(wte if cfg.tie_word_embeddings else matrix("lm_head.weight"))
    return DecoderModel(config=cfg, embedding=embedding, layers=layers,
                        schedule=[LayerCall(i) for i in range(cfg.n_layer)], final_norm=final_norm, head=head,
                        options=options, max_seq_len=cfg.n_positions)


def ignored_tensors(cfg: GPT2Config) -> tuple:
    """What Hugging Face GPT-2 checkpoints carry but no computation reads: the causal-mask buffers
    (tools/converter/test_converters.py:113-114 has them skipped) and, with a tied head, the head's copy of the
    embedding (tools/converter/convert_gpt2.py:141-142)."""
    return ("*.attn.bias", "*.attn.masked_bias") + (("lm_head.weight",) if cfg.tie_word_embeddings else ())


GPT2 = register_architecture(Architecture(
    name="gpt2", config_cls=GPT2Config, weight_spec=weight_spec, random_weights=random_weights, build=build,
    prefixes=("", "transformer."),          # tools/converter/convert_gpt2.py:83-95 accepts both
    ignored_tensors=ignored_tensors))
