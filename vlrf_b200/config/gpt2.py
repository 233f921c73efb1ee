"""GPT-2's configuration, under the keys of its Hugging Face config.json.

The reference's converter maps these keys to its own dialect
(tools/converter/convert_gpt2.py:148-173; n_inner null ⇒ 4·n_embd at :155,
fallbacks in tools/converter/convert_safetensors.py:172-178) and its
`ModelConfig::check()` gives the size relations (include/model/config.hpp:127-140).
"""
from __future__ import annotations

import dataclasses

from .base import ConfigError, ModelConfig, key

#: activation_function spellings → the activation a feed-forward part implements
GPT2_ACTIVATIONS = {
    "gelu_new": "gelu_tanh",
    "gelu_pytorch_tanh": "gelu_tanh",
    "gelu_fast": "gelu_tanh",
    "gelu": "gelu_erf",
}


@dataclasses.dataclass
class GPT2Config(ModelConfig):
    model_type = "gpt2"

    vocab_size: int = key()
    n_positions: int = key()
    n_embd: int = key()
    n_layer: int = key()
    n_head: int = key()
    layer_norm_epsilon: float = key()
    activation_function: str = key()
    n_inner: int | None = key(default=None, nullable=True)
    scale_attn_weights: bool = key(default=True)
    scale_attn_by_inverse_layer_idx: bool = key(default=False)
    tie_word_embeddings: bool = key(default=True)
    bos_token_id: int | None = key(default=None, nullable=True)
    eos_token_id: int | None = key(default=None, nullable=True)

    def validate(self) -> None:
        for name in ("vocab_size", "n_positions", "n_embd", "n_layer", "n_head"):
            self._positive(name, getattr(self, name))
        if self.n_inner is not None:
            self._positive("n_inner", self.n_inner)
        if self.n_embd % self.n_head != 0:
            raise ConfigError(
                f"n_embd ({self.n_embd}) must be a multiple of n_head ({self.n_head})")
        if self.head_dim % 16 != 0 or self.head_dim > 256:
            raise ConfigError(
                f"n_embd / n_head = {self.head_dim}: this library's attention kernels take head sizes that are "
                f"multiples of 16 up to 256")
        if not self.layer_norm_epsilon > 0.0:
            raise ConfigError(f"layer_norm_epsilon must be positive, got {self.layer_norm_epsilon}")
        if self.activation_function not in GPT2_ACTIVATIONS:
            raise ConfigError(
                f"activation_function '{self.activation_function}' is not one of "
                + ", ".join(sorted(GPT2_ACTIVATIONS)))
        for name in ("bos_token_id", "eos_token_id"):
            v = getattr(self, name)
            if v is not None and not (0 <= v < self.vocab_size):
                raise ConfigError(f"{name} ({v}) lies outside the vocabulary of {self.vocab_size}")

    # derived sizes -------------------------------------------------------
    @property
    def head_dim(self) -> int:
        return self.n_embd // self.n_head

    @property
    def inner_dim(self) -> int:
        return self.n_inner if self.n_inner is not None else 4 * self.n_embd

    @property
    def activation(self) -> str:
        return GPT2_ACTIVATIONS[self.activation_function]

    def param_count(self) -> int:
        d, f, v, p, n = self.n_embd, self.inner_dim, self.vocab_size, self.n_positions, self.n_layer
        per_layer = (3 * d * d + 3 * d) + (d * d + d) + (d * f + f) + (f * d + d) + 4 * d
        head = 0 if self.tie_word_embeddings else v * d
        return v * d + p * d + n * per_layer + 2 * d + head
