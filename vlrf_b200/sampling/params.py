"""Options of one generation call, under the reference's names and defaults where it has them
(include/model/generation_config.hpp:15-73)."""
from __future__ import annotations

import dataclasses


@dataclasses.dataclass
class SamplingParams:
    max_new_tokens: int = 128          # generation_config.hpp:16
    temperature: float = 0.8           # :17; ≤ 0 means greedy (include/model/transformer.hpp:130)
    top_p: float = 0.9                 # :18; ≥ 1 keeps everything
    top_k: int = 50                    # :19; ≤ 0 keeps everything
    do_sample: bool = True             # :20; False = greedy (`--greedy` of tools/vlrf_cli.cpp:115)
    repetition_penalty: float = 1.0    # :45
    frequency_penalty: float = 0.0     # :46
    presence_penalty: float = 0.0      # :47
    no_repeat_ngram_size: int = 0      # :56
    #: token ids that end a sequence; None = the model's eos_token_id (transformer.hpp:504-507)
    stop_token_ids: tuple | None = None
    seed: int = 42                     # tools/vlrf_cli.cpp:38

    def validate(self) -> None:
        if self.max_new_tokens < 0:
            raise ValueError("max_new_tokens must not be negative")
        if self.top_p < 0:
            raise ValueError("top_p must not be negative")
        if self.repetition_penalty == 0:
            raise ValueError("repetition_penalty must not be zero")

    @property
    def greedy(self) -> bool:
        return (not self.do_sample) or self.temperature <= 0

    @property
    def has_penalties(self) -> bool:
        return (self.repetition_penalty != 1.0 or self.frequency_penalty != 0.0
                or self.presence_penalty != 0.0 or self.no_repeat_ngram_size > 1)

    @staticmethod
    def greedy_params(max_new_tokens: int = 128, **kw) -> "SamplingParams":
        return SamplingParams(max_new_tokens=max_new_tokens, do_sample=False, **kw)
