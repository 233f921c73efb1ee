"""The Python entry point, in the manner of the reference's C API (include/api/vlrf.h:116-295):
create a model from a folder, generate ids, get logits, query the context and the cache.

    model = Model.load("model_dir", dtype="bfloat16", max_tokens=4096)
    results = model.generate_ids([[464, 3290], [1212]], SamplingParams(max_new_tokens=16, do_sample=False))
    logits = model.get_logits([464, 3290])            # float32 [vocab] at the last position

Where the reference names a call, the method has that name without the `vlrf_` prefix:
vlrf_load_weights → load, vlrf_init_random → init_random, vlrf_generate_ids → generate_ids,
vlrf_get_logits → get_logits, vlrf_kv_cache_bytes → kv_cache_bytes, vlrf_model_summary → model_summary.
"""
from __future__ import annotations

import tempfile

import torch

from .engine.backend import DeviceBackend
from .engine.generate import generate
from .engine.loading import load_model
from .engine.step import Engine, StepEntry
from .sampling.params import SamplingParams
from .weights.model_dir import write_random_model


class Model:
    def __init__(self, decoder, *, max_tokens: int | None = None, n_slots: int | None = None):
        self.decoder = decoder
        self.config = decoder.config
        if max_tokens is None:
            max_tokens = decoder.max_seq_len
        self.engine = Engine(decoder, max_tokens=max_tokens, n_slots=n_slots)
        self.backend = DeviceBackend(self.engine)

    # -- construction -------------------------------------------------------------------------
    @classmethod
    def load(cls, model_dir, dtype="bfloat16", device="cuda:0", max_tokens: int | None = None,
             n_slots: int | None = None) -> "Model":
        """A folder with config.json and model.safetensors (vlrf_load_weights, vlrf.h:124)."""
        return cls(load_model(model_dir, dtype, device), max_tokens=max_tokens, n_slots=n_slots)

    @classmethod
    def init_random(cls, config: dict, seed: int = 1234, dtype="bfloat16", device="cuda:0",
                    max_tokens: int | None = None, n_slots: int | None = None) -> "Model":
        """Random weights for a configuration (vlrf_init_random, vlrf.h:120): the folder is written to a
        temporary place and loaded like any other."""
        with tempfile.TemporaryDirectory(prefix="vlrf_b200_random_") as tmp:
            write_random_model(config, seed, tmp)
            return cls.load(tmp, dtype, device, max_tokens, n_slots)

    # -- generation ---------------------------------------------------------------------------
    def generate_ids(self, prompts, params: SamplingParams | list | None = None, on_token=None) -> list:
        """Generate for a list of prompts (lists of token ids); returns one GenerationResult each
        (vlrf_generate_ids, vlrf.h:189; batched here)."""
        if params is None:
            params = SamplingParams()
        single = len(prompts) > 0 and isinstance(prompts[0], int)
        if single:
            prompts = [prompts]
        out = generate(self.backend, prompts, params, bos_token_id=getattr(self.config, "bos_token_id", None),
                       eos_token_id=getattr(self.config, "eos_token_id", None), on_token=on_token)
        return out[0] if single else out

    def get_logits(self, token_ids, all_positions: bool = False) -> torch.Tensor:
        """Logits of one whole sequence from an empty context, at the last position (vlrf_get_logits,
        vlrf.h:200; src/api/vlrf_api.cpp:464-479) or at every position; float32 on the host."""
        slot = self.engine.start_sequence()
        try:
            want = list(range(len(token_ids))) if all_positions else [len(token_ids) - 1]
            logits = self.engine.step([StepEntry(slot, list(token_ids), want)]).cpu()
            self.engine.check_device_errors()
        finally:
            self.engine.end_sequence(slot)
        return logits if all_positions else logits[0]

    # -- information --------------------------------------------------------------------------
    def kv_cache_bytes(self) -> int:
        return self.engine.cache.bytes()

    def model_summary(self) -> str:
        c = self.config
        fields = ", ".join(f"{k}={v}" for k, v in c.to_dict().items())
        return (f"{fields}\nweights on device: {self.decoder.weight_bytes() / 2**20:.1f} MiB "
                f"({self.decoder.act_dtype}); cache: {self.kv_cache_bytes() / 2**20:.1f} MiB for "
                f"{self.engine.cache.max_tokens} tokens in {self.engine.cache.n_slots} slots")
