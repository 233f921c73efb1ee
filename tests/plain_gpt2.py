"""Plain, slow GPT-2: whole sequences, no cache, one function per part.

This is the oracle of the test suite.  It is written from the formulas of the
reference engine (VLRF-org/VLRF, paths below are relative to that project) and
shares no code with the ``vlrf_b200`` package: it has its own reader for
``model.safetensors``, its own config parsing and its own sampler.  Everything
runs on the CPU in float64 by default (``dtype=torch.float32`` is available to
see what 32-bit rounding alone does).

Weights come in the Hugging Face layout (Conv1D ``[in, out]``, fused
``c_attn``), which the reference's converter documents:
tools/converter/convert_gpt2.py:98-139.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch


# --------------------------------------------------------------------------
# reading a model folder (own code, not the package's loader)
# --------------------------------------------------------------------------
def read_safetensors(path) -> dict[str, torch.Tensor]:
    """u64 header length, JSON header, raw little-endian data
    (layout as read by tools/converter/convert_safetensors.py:54-88)."""
    raw = Path(path).read_bytes()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen].decode("utf-8"))
    base = 8 + hlen
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        b, e = meta["data_offsets"]
        buf = raw[base + b:base + e]
        shape = tuple(meta["shape"])
        dt = meta["dtype"]
        if dt == "F32":
            t = torch.from_numpy(np.frombuffer(buf, dtype="<f4").copy())
        elif dt == "F16":
            t = torch.from_numpy(np.frombuffer(buf, dtype="<f2").copy())
        elif dt == "BF16":
            # bf16 is the high half of an f32 (convert_safetensors.py:78-85)
            u16 = np.frombuffer(buf, dtype="<u2").astype(np.uint32) << 16
            t = torch.from_numpy(u16.view(np.float32).copy())
        elif dt == "I32":
            t = torch.from_numpy(np.frombuffer(buf, dtype="<i4").copy())
        else:
            raise ValueError(f"plain reader: dtype {dt} of {name}")
        out[name] = t.reshape(shape)
    return out


def read_model_dir(model_dir, dtype=torch.float64):
    model_dir = Path(model_dir)
    cfg = json.loads((model_dir / "config.json").read_text())
    weights = {k: (v.to(dtype) if v.is_floating_point() else v)
               for k, v in read_safetensors(model_dir / "model.safetensors").items()}
    return cfg, weights


def _w(weights, name):
    """Tensor by HF name, with or without the ``transformer.`` prefix
    (convert_gpt2.py:83-95)."""
    if name in weights:
        return weights[name]
    return weights["transformer." + name]


# --------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------
def embed_tokens(wte, ids):
    """x[t,:] = wte[id[t],:] — include/model/ops.hpp:615-626,
    include/model/transformer.hpp:340.  No scaling for GPT-2."""
    return wte[torch.as_tensor(ids, dtype=torch.long)]


def add_learned_positions(x, wpe, pos0=0):
    """x[t,:] += wpe[pos0+t,:] — include/model/transformer.hpp:350-361."""
    T = x.shape[0]
    if pos0 + T > wpe.shape[0]:
        raise ValueError("positions exceed n_positions")  # transformer.hpp:355-357
    return x + wpe[pos0:pos0 + T]


def layer_norm(x, gamma, beta, eps):
    """Two-pass, biased variance, 1/sqrt(var+eps) — include/model/ops.hpp:443-476."""
    mean = x.mean(dim=-1, keepdim=True)
    diff = x - mean
    var = (diff * diff).mean(dim=-1, keepdim=True) + eps
    return diff * (1.0 / torch.sqrt(var)) * gamma + beta


def conv1d(x, w_in_out, b):
    """HF Conv1D: y = x @ W[in,out] + b.  The reference computes the same as
    linear(x, W^T) + bias — include/model/compute.hpp:64-68,
    include/model/attention.hpp:98-105 — after the converter transposed W
    (convert_gpt2.py:114-135)."""
    return x @ w_in_out + b


def split_qkv(qkv, n_embd):
    """Fused c_attn output → q, k, v as thirds of the columns
    (convert_gpt2.py:114-125)."""
    return qkv[:, :n_embd], qkv[:, n_embd:2 * n_embd], qkv[:, 2 * n_embd:]


def split_heads(x, n_head):
    """[T, H*dh] → [H, T, dh]; head h owns columns h*dh…(h+1)*dh —
    include/model/attention.hpp:313-325."""
    T, d = x.shape
    return x.reshape(T, n_head, d // n_head).permute(1, 0, 2)


def merge_heads(x):
    """[H, T, dh] → [T, H*dh] — include/model/attention.hpp:447-455."""
    H, T, dh = x.shape
    return x.permute(1, 0, 2).reshape(T, H * dh)


def causal_attention(q, k, v, scale, window=0):
    """softmax(scale·q·kᵀ + causal mask)·v for whole sequences, dense.
    Scale 1/sqrt(dh): include/model/attention.hpp:373-374; key k visible to the
    query at position p iff k ≤ p: attention.hpp:253-260; masked = −inf;
    softmax with max subtraction ≡ the online form of attention.hpp:265-307.
    ``window`` > 0 additionally hides keys with k ≤ p − window (not GPT-2;
    used by kernel tests only)."""
    H, T, dh = q.shape
    s = torch.einsum("hqd,hkd->hqk", q, k) * scale
    qpos = torch.arange(T).view(T, 1)
    kpos = torch.arange(k.shape[1]).view(1, -1)
    hidden = kpos > qpos
    if window > 0:
        hidden = hidden | (kpos <= qpos - window)
    s = s.masked_fill(hidden, float("-inf"))
    s = s - s.max(dim=-1, keepdim=True).values
    p = torch.exp(s)
    p = p / p.sum(dim=-1, keepdim=True)
    return torch.einsum("hqk,hkd->hqd", p, v)


def gelu_tanh(x):
    """0.5·x·(1+tanh(0.7978845608028654·(x+0.044715·x³))) —
    include/model/ops.hpp:390-403."""
    return 0.5 * x * (1.0 + torch.tanh(0.7978845608028654 * (x + 0.044715 * x * x * x)))


def gelu_erf(x):
    """Exact form 0.5·x·(1+erf(x/√2)) for activation_function="gelu".  The
    reference has only the tanh form (ops.hpp:390-403); this rests on the
    definition of GELU."""
    return 0.5 * x * (1.0 + torch.erf(x / math.sqrt(2.0)))


ACTIVATIONS = {"gelu_new": gelu_tanh, "gelu_pytorch_tanh": gelu_tanh,
               "gelu_fast": gelu_tanh, "gelu": gelu_erf}


def attention_part(h, weights, prefix, cfg, layer_idx):
    """q/k/v projection, per-head causal attention, output projection —
    include/model/attention.hpp:89-186."""
    d, H = cfg["n_embd"], cfg["n_head"]
    qkv = conv1d(h, _w(weights, prefix + "attn.c_attn.weight"), _w(weights, prefix + "attn.c_attn.bias"))
    q, k, v = (split_heads(t, H) for t in split_qkv(qkv, d))
    scale = 1.0 / math.sqrt(d // H)
    if cfg.get("scale_attn_by_inverse_layer_idx", False):
        # not in the reference (it can only replace the scale through
        # attention_multiplier, attention.hpp:53,373-374): scale /= layer_idx+1
        scale = scale / float(layer_idx + 1)
    o = merge_heads(causal_attention(q, k, v, scale))
    return conv1d(o, _w(weights, prefix + "attn.c_proj.weight"), _w(weights, prefix + "attn.c_proj.bias"))


def mlp_part(h, weights, prefix, cfg):
    """fc → activation → proj — include/model/feedforward.hpp:50-77."""
    act = ACTIVATIONS[cfg.get("activation_function", "gelu_new")]
    u = conv1d(h, _w(weights, prefix + "mlp.c_fc.weight"), _w(weights, prefix + "mlp.c_fc.bias"))
    return conv1d(act(u), _w(weights, prefix + "mlp.c_proj.weight"), _w(weights, prefix + "mlp.c_proj.bias"))


def block(x, weights, layer_idx, cfg):
    """Pre-norm block: a = x + attn(LN1(x)); y = a + mlp(LN2(a)) —
    include/model/transformer_block.hpp:149-159."""
    p = f"h.{layer_idx}."
    eps = cfg.get("layer_norm_epsilon", 1e-5)
    h1 = layer_norm(x, _w(weights, p + "ln_1.weight"), _w(weights, p + "ln_1.bias"), eps)
    a = x + attention_part(h1, weights, p, cfg, layer_idx)
    h2 = layer_norm(a, _w(weights, p + "ln_2.weight"), _w(weights, p + "ln_2.bias"), eps)
    return a + mlp_part(h2, weights, p, cfg)


def final_norm_and_logits(x, weights, cfg):
    """LN_f then the LM head without bias; tied head = wte —
    include/model/transformer.hpp:398-414, :298-300.  Unlike the reference,
    which keeps the last row only, all rows are returned."""
    eps = cfg.get("layer_norm_epsilon", 1e-5)
    n = layer_norm(x, _w(weights, "ln_f.weight"), _w(weights, "ln_f.bias"), eps)
    if cfg.get("tie_word_embeddings", True):
        head = _w(weights, "wte.weight")
    else:
        head = weights["lm_head.weight"]
    return n @ head.T


def logits_all_positions(cfg, weights, ids):
    """Logits [T, vocab] of one whole sequence — include/model/transformer.hpp:335-424."""
    x = embed_tokens(_w(weights, "wte.weight"), ids)
    x = add_learned_positions(x, _w(weights, "wpe.weight"), 0)
    for layer_idx in range(cfg["n_layer"]):
        x = block(x, weights, layer_idx, cfg)
    return final_norm_and_logits(x, weights, cfg)


# --------------------------------------------------------------------------
# sampling (include/model/transformer.hpp:43-182)
# --------------------------------------------------------------------------
def argmax_first(logits):
    """First maximal index (std::max_element) — transformer.hpp:43-47."""
    logits = np.asarray(logits, dtype=np.float64)
    return int(np.argmax(logits))


def apply_penalties(logits, counts, repetition_penalty=1.0, frequency_penalty=0.0, presence_penalty=0.0):
    """transformer.hpp:54-84: for every token generated so far (count > 0):
    divide a positive logit (multiply a non-positive one) by the repetition
    penalty, then subtract frequency·count and presence."""
    out = np.array(logits, dtype=np.float64)
    for tok, c in counts.items():
        if c <= 0 or tok >= out.shape[0]:
            continue
        if repetition_penalty != 1.0:
            out[tok] = out[tok] / repetition_penalty if out[tok] > 0 else out[tok] * repetition_penalty
        out[tok] -= frequency_penalty * c
        out[tok] -= presence_penalty
    return out


def block_repeated_ngrams(logits, generated, n):
    """transformer.hpp:92-120: forbid every token that would complete an n-gram
    already present among the generated tokens."""
    out = np.array(logits, dtype=np.float64)
    if n <= 1 or len(generated) < n - 1:
        return out
    suffix = list(generated[len(generated) - (n - 1):])
    for start in range(0, len(generated) - n + 1):
        if list(generated[start:start + n - 1]) == suffix:
            out[generated[start + n - 1]] = -np.inf
    return out


def sample_token(logits, temperature, top_k, top_p, u):
    """transformer.hpp:124-182 with the uniform draw ``u`` given by the caller:
    logits/temperature → softmax → keep the k most probable → walk the tokens by
    descending probability and drop the first one whose running mass exceeds
    top_p together with all after it, the most probable one always staying
    (:159-165) → renormalise → first i with u ≤ cumulative sum, else the last."""
    logits = np.asarray(logits, dtype=np.float64)
    n = logits.shape[0]
    if temperature <= 0:
        return argmax_first(logits)
    z = logits / temperature
    z = z - z.max()
    p = np.exp(z)
    p = p / p.sum()
    order = np.argsort(-p, kind="stable")
    if 0 < top_k < n:
        p[order[top_k:]] = 0.0
    if top_p < 1.0:
        cum = 0.0
        for rank, idx in enumerate(order):
            cum += p[idx]
            if cum > top_p and rank > 0:
                p[order[rank:]] = 0.0
                break
    s = p.sum()
    if s < 1e-9:
        return argmax_first(logits)
    p = p / s
    cum = 0.0
    for i in range(n):
        cum += p[i]
        if u <= cum:
            return i
    return n - 1


def greedy_generate(cfg, weights, prompt, max_new_tokens, stop_ids=()):
    """Greedy decoding by re-running the whole sequence for every new token.
    The first new token comes from the logits at the last prompt position (the
    reference feeds the last prompt token twice, transformer.hpp:447-452,482;
    that quirk is not reproduced)."""
    ids = list(prompt)
    new = []
    for _ in range(max_new_tokens):
        if len(ids) >= cfg["n_positions"]:
            break
        nxt = argmax_first(logits_all_positions(cfg, weights, ids)[-1].numpy())
        ids.append(nxt)
        new.append(nxt)
        if nxt in stop_ids:
            break
    return new
