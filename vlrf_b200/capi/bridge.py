"""What the C interface (vlrf_b200.h) calls: plain functions over plain values.

The C library passes integers, strings and the addresses of the caller's buffers; every function here returns
`(status, value)` and never raises, so the C side needs no knowledge of the package's exception types.  The
functions do nothing of their own: they hand over to `vlrf_b200.api.Model`, the entry point that Python callers use.
"""
from __future__ import annotations

import ctypes
import json
import os

OK, INVALID_ARG, OUT_OF_MEMORY, IO, BAD_MODEL, NOT_INIT, CTX_FULL, DEVICE, UNKNOWN = 0, 1, 2, 3, 4, 5, 6, 7, 99
FINISH = {"stop": 0, "length": 1, "context": 2}

_models: dict = {}
_next = [1]


class Sampling(ctypes.Structure):      # VlrfB200Sampling of vlrf_b200.h
    _fields_ = [("max_new_tokens", ctypes.c_int32), ("temperature", ctypes.c_float), ("top_p", ctypes.c_float),
                ("top_k", ctypes.c_int32), ("use_sampling", ctypes.c_int32), ("repetition_penalty", ctypes.c_float),
                ("frequency_penalty", ctypes.c_float), ("presence_penalty", ctypes.c_float),
                ("no_repeat_ngram_size", ctypes.c_int32), ("seed", ctypes.c_uint32), ("n_stop_ids", ctypes.c_int32),
                ("stop_ids", ctypes.c_int32 * 8), ("_reserved", ctypes.c_int32 * 7)]


class ModelInfo(ctypes.Structure):     # VlrfB200ModelInfo of vlrf_b200.h
    _fields_ = [(k, ctypes.c_int32) for k in ("vocab_size", "max_seq_len", "width", "n_layers", "cache_tokens",
                                              "cache_slots", "bos_token_id", "eos_token_id")] + \
               [("_reserved", ctypes.c_int32 * 8)]


def _status_of(exc: BaseException) -> int:
    from ..cache import CacheError
    from ..config.base import ConfigError
    from ..csrc import KernelError
    from ..engine.generate import GenerationError
    from ..engine.step import StepError
    from ..weights.safetensors_io import WeightError
    import torch
    if isinstance(exc, (MemoryError, torch.cuda.OutOfMemoryError)):
        return OUT_OF_MEMORY
    if isinstance(exc, (FileNotFoundError, PermissionError, IsADirectoryError)):
        return IO
    if isinstance(exc, WeightError):
        return IO if any(w in str(exc) for w in ("no model.safetensors", "cannot", "truncated", "shorter")) else BAD_MODEL
    if isinstance(exc, ConfigError):
        return IO if "cannot read" in str(exc) or "no config.json" in str(exc) else BAD_MODEL
    if isinstance(exc, CacheError):
        return CTX_FULL
    if isinstance(exc, GenerationError):
        return CTX_FULL if "cache holds" in str(exc) or "positions" in str(exc) else INVALID_ARG
    if isinstance(exc, StepError):
        return CTX_FULL if "positions of the model" in str(exc) else INVALID_ARG
    if isinstance(exc, KernelError):
        return DEVICE
    if isinstance(exc, (ValueError, TypeError, KeyError, IndexError)):
        return INVALID_ARG
    return UNKNOWN


def _guard(fn):
    def wrapped(*args):
        try:
            return OK, fn(*args)
        except BaseException as exc:  # noqa: BLE001 - every failure becomes a status and a message
            return _status_of(exc), f"{type(exc).__name__}: {exc}"
    wrapped.__name__ = fn.__name__
    return wrapped


def _model(handle: int):
    m = _models.get(handle)
    if m is None:
        raise LookupError("the handle holds no model: call vlrf_b200_load_dir or vlrf_b200_init_random first")
    return m


def _ints(address: int, n: int) -> list:
    return list((ctypes.c_int32 * n).from_address(address)) if n > 0 else []


def _put_text(text: str, address: int, cap: int) -> None:
    data = text.encode("utf-8")
    if cap <= 0 or len(data) + 1 > cap:
        raise ValueError(f"the text needs {len(data) + 1} bytes; the buffer holds {cap}")
    ctypes.memmove(address, data + b"\0", len(data) + 1)


def _config_of(text: str) -> dict:
    """A preset's name, the path of a config.json, or JSON text."""
    from ..config import load_preset, preset_names
    if text in preset_names():
        return load_preset(text)
    if os.path.isfile(text):
        with open(text) as f:
            return json.load(f)
    try:
        cfg = json.loads(text)
    except ValueError:
        from ..config.base import ConfigError
        raise ConfigError(f"'{text[:60]}' is neither a preset ({', '.join(sorted(preset_names()))}), nor a readable "
                          f"config.json, nor JSON text") from None
    if not isinstance(cfg, dict):
        raise ValueError("a configuration is a JSON object")
    return cfg


@_guard
def create() -> int:
    handle = _next[0]
    _next[0] += 1
    _models[handle] = None
    return handle


@_guard
def free(handle: int) -> None:
    _models.pop(handle, None)


@_guard
def load_dir(handle: int, model_dir: str, dtype: str, max_tokens: int, n_slots: int) -> None:
    from ..api import Model
    if handle not in _models:
        raise LookupError("unknown handle")
    _models[handle] = Model.load(model_dir, dtype=dtype or "bfloat16", max_tokens=max_tokens or None, n_slots=n_slots or None)


@_guard
def init_random(handle: int, config: str, seed: int, dtype: str, max_tokens: int, n_slots: int) -> None:
    from ..api import Model
    import vlrf_b200.models  # noqa: F401
    if handle not in _models:
        raise LookupError("unknown handle")
    _models[handle] = Model.init_random(_config_of(config), seed=seed, dtype=dtype or "bfloat16",
                                        max_tokens=max_tokens or None, n_slots=n_slots or None)


@_guard
def get_info(handle: int, address: int) -> None:
    m = _model(handle)
    info = ModelInfo.from_address(address)
    d = m.decoder
    info.vocab_size, info.max_seq_len, info.width, info.n_layers = d.vocab_size, d.max_seq_len, d.width, len(d.layers)
    info.cache_tokens, info.cache_slots = m.engine.cache.max_tokens, m.engine.cache.n_slots
    bos, eos = getattr(m.config, "bos_token_id", None), getattr(m.config, "eos_token_id", None)
    info.bos_token_id = -1 if bos is None else bos
    info.eos_token_id = -1 if eos is None else eos


@_guard
def get_config(handle: int, address: int, cap: int) -> None:
    _put_text(json.dumps(_model(handle).config.to_dict()), address, cap)


@_guard
def model_summary(handle: int, address: int, cap: int) -> None:
    _put_text(_model(handle).model_summary(), address, cap)


@_guard
def kv_cache_bytes(handle: int) -> int:
    return int(_model(handle).kv_cache_bytes())


def _params(address: int, n: int, default_seed) -> list:
    from ..sampling.params import SamplingParams
    out = []
    for i in range(n):
        s = Sampling.from_address(address + i * ctypes.sizeof(Sampling))
        if s.n_stop_ids > 8:
            raise ValueError("at most 8 stop ids")
        stop = None if s.n_stop_ids < 0 else tuple(s.stop_ids[:s.n_stop_ids])
        out.append(SamplingParams(max_new_tokens=s.max_new_tokens, temperature=s.temperature, top_p=s.top_p, top_k=s.top_k,
                                  do_sample=bool(s.use_sampling), repetition_penalty=s.repetition_penalty,
                                  frequency_penalty=s.frequency_penalty, presence_penalty=s.presence_penalty,
                                  no_repeat_ngram_size=s.no_repeat_ngram_size, stop_token_ids=stop, seed=int(s.seed)))
    return out


@_guard
def generate_ids(handle: int, ids_at: int, lens_at: int, n_prompts: int, params_at: int, n_params: int, out_at: int,
                 out_cap: int, out_lens_at: int, out_reasons_at: int) -> None:
    m = _model(handle)
    if n_prompts <= 0 or n_params not in (1, n_prompts) or out_cap < 0:
        raise ValueError("generate_ids: prompts, or one set of options or one per prompt")
    lens = _ints(lens_at, n_prompts)
    if any(n < 0 for n in lens):
        raise ValueError("generate_ids: a negative prompt length")
    flat = _ints(ids_at, sum(lens))
    prompts, at = [], 0
    for n in lens:
        prompts.append(flat[at:at + n])
        at += n
    params = _params(params_at, n_params, None)
    if any(p.max_new_tokens > out_cap for p in params):
        raise ValueError(f"generate_ids: max_new_tokens exceeds the {out_cap} ids a row of out_ids holds")
    results = m.generate_ids(prompts, params[0] if n_params == 1 else params)
    out = (ctypes.c_int32 * (n_prompts * out_cap)).from_address(out_at) if out_cap > 0 else None
    out_lens = (ctypes.c_int32 * n_prompts).from_address(out_lens_at)
    reasons = (ctypes.c_int32 * n_prompts).from_address(out_reasons_at) if out_reasons_at else None
    for i, r in enumerate(results):
        out_lens[i] = len(r.new_tokens)
        for j, t in enumerate(r.new_tokens):
            out[i * out_cap + j] = t
        if reasons is not None:
            reasons[i] = FINISH[r.finish_reason]


@_guard
def get_logits(handle: int, ids_at: int, n: int, out_at: int) -> None:
    m = _model(handle)
    if n <= 0:
        raise ValueError("get_logits: at least one token")
    logits = m.get_logits(_ints(ids_at, n)).contiguous()
    ctypes.memmove(out_at, logits.data_ptr(), logits.numel() * 4)


@_guard
def start_sequence(handle: int) -> int:
    return int(_model(handle).engine.start_sequence())


@_guard
def reset_slot(handle: int, slot: int) -> None:
    _model(handle).engine.end_sequence(slot)


@_guard
def context_length(handle: int, slot: int) -> int:
    eng = _model(handle).engine
    if not eng.cache.slots.is_held(slot):
        raise ValueError(f"slot {slot} is not held by a sequence")
    return int(eng.length(slot))


@_guard
def step(handle: int, n_entries: int, slots_at: int, counts_at: int, tokens_at: int, want_counts_at: int, want_at: int,
         out_at: int, out_rows_cap: int) -> None:
    from ..engine.step import StepEntry
    m = _model(handle)
    if n_entries <= 0:
        raise ValueError("step: at least one entry")
    slots, counts, want_counts = _ints(slots_at, n_entries), _ints(counts_at, n_entries), _ints(want_counts_at, n_entries)
    if any(c < 0 for c in counts + want_counts):
        raise ValueError("step: a negative count")
    tokens, want = _ints(tokens_at, sum(counts)), _ints(want_at, sum(want_counts))
    if sum(want_counts) > out_rows_cap:
        raise ValueError(f"step: {sum(want_counts)} rows of logits are wanted; out_logits holds {out_rows_cap}")
    entries, t_at, w_at = [], 0, 0
    for s, c, wc in zip(slots, counts, want_counts):
        entries.append(StepEntry(s, tokens[t_at:t_at + c], want[w_at:w_at + wc]))
        t_at += c
        w_at += wc
    logits = m.engine.step(entries)
    m.engine.check_device_errors()
    if logits.numel():
        host = logits.cpu().contiguous()
        ctypes.memmove(out_at, host.data_ptr(), host.numel() * 4)


@_guard
def presets(address: int, cap: int) -> None:
    from ..config import preset_names
    _put_text("\n".join(sorted(preset_names())), address, cap)


@_guard
def describe_dir(model_dir: str, address: int, cap: int) -> None:
    import vlrf_b200.models  # noqa: F401
    from ..config.base import read_config_json
    from ..registry import parse_config
    arch, cfg = parse_config(read_config_json(model_dir))
    text = f"architecture: {arch.name}\n{json.dumps(cfg.to_dict(), indent=2)}\n"
    if hasattr(cfg, "param_count"):
        text += f"parameters: {cfg.param_count():,}\n"
    _put_text(text, address, cap)


@_guard
def write_random_model(config: str, seed: int, out_dir: str) -> None:
    import vlrf_b200.models  # noqa: F401
    from ..weights import write_random_model as write
    write(_config_of(config), seed, out_dir)
