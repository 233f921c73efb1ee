"""Tensor-level entry to the kernels: checks, then raw pointers and the current stream.

Every function writes into tensors that the caller provides; nothing here allocates.  All tensors must
be contiguous CUDA tensors.  Sizes a kernel cannot take are refused with a `KernelError` that says why;
no function has a CPU or library fallback.
"""
from __future__ import annotations

import torch

from . import KernelError, call

F32, BF16 = 0, 1
ACT = {"none": 0, None: 0, "gelu_tanh": 1, "gelu_erf": 2}


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16, not {dt}")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def _dev(t: torch.Tensor, name: str, dtype=None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must live on the CUDA device (there is no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, not {t.dtype}")


def embed(wte, wpe, tokens, positions, out, dev_err) -> None:
    """out[t] = wte[tokens[t]] (+ wpe[positions[t]]), float32."""
    _dev(wte, "wte"); _dev(tokens, "tokens", torch.int32); _dev(out, "out", torch.float32)
    _dev(dev_err, "dev_err", torch.int32)
    T = tokens.shape[0]
    V, d = wte.shape
    P = 0
    if wpe is not None:
        _dev(wpe, "wpe", wte.dtype); _dev(positions, "positions", torch.int32)
        P = wpe.shape[0]
        if wpe.shape[1] != d or positions.shape[0] != T:
            raise KernelError("embed: position table or positions do not match")
    if out.shape[0] < T or out.shape[1] != d:
        raise KernelError("embed: output does not match")
    call("vlrf_embed", _ptr(wte), _ptr(wpe), dtype_code(wte.dtype), _ptr(tokens), _ptr(positions), _ptr(out),
         T, d, V, P, _ptr(dev_err), _stream())


def layernorm(x, gamma, beta, eps: float, out, rows=None) -> None:
    """out[r] = LN(x[rows[r]] if rows is given else x[r]); x float32, out float32 or bfloat16."""
    _dev(x, "x", torch.float32); _dev(gamma, "gamma", torch.float32); _dev(beta, "beta", torch.float32)
    _dev(out, "out")
    d = x.shape[1]
    n = x.shape[0]
    if rows is not None:
        _dev(rows, "rows", torch.int32)
        n = rows.shape[0]
    if gamma.shape[0] != d or beta.shape[0] != d or out.shape[1] != d or out.shape[0] < n:
        raise KernelError("layernorm: sizes do not match")
    call("vlrf_layernorm", _ptr(x), _ptr(rows), _ptr(gamma), _ptr(beta), _ptr(out), dtype_code(out.dtype), n, d,
         float(eps), _stream())


def linear(x, w, bias, out, *, act=None, residual=None, rows: int | None = None) -> None:
    """out = act(x · wᵀ + bias) (+ residual).  x [M,K], w [N,K] (same dtype), bias/residual float32,
    out [M,N] float32 or bfloat16.  `rows` limits M to the first rows of x/out/residual."""
    _dev(x, "x"); _dev(w, "w", x.dtype); _dev(out, "out")
    M = x.shape[0] if rows is None else rows
    K = x.shape[1]
    N = w.shape[0]
    if w.shape[1] != K or out.shape[1] != N or out.shape[0] < M or x.shape[0] < M:
        raise KernelError(f"linear: x {list(x.shape)}, w {list(w.shape)}, out {list(out.shape)} do not match")
    if bias is not None:
        _dev(bias, "bias", torch.float32)
        if bias.shape[0] != N:
            raise KernelError("linear: bias does not match")
    if residual is not None:
        _dev(residual, "residual", torch.float32)
        if residual.shape[1] != N or residual.shape[0] < M:
            raise KernelError("linear: residual does not match")
    if x.dtype == torch.float32 and out.dtype != torch.float32:
        raise KernelError("linear: float32 input gives float32 output")
    _linear_dispatch(x, w, bias, out, ACT[act], residual, M, N, K)


def _linear_dispatch(x, w, bias, out, act, residual, M, N, K) -> None:
    call("vlrf_gemm_simt", _ptr(x), _ptr(w), _ptr(bias), _ptr(residual), _ptr(out), M, N, K, K, N,
         dtype_code(x.dtype), dtype_code(out.dtype), act, _stream())


def kv_append(qkv, k_off: int, v_off: int, k_cache, v_cache, block_table, tok_slot, tok_pos, n_tokens: int,
              n_kv_heads: int, head_dim: int, dev_err) -> None:
    """Scatter the K and V columns of qkv rows into one layer's paged cache
    [block, kv_head, block_tokens, head_dim]."""
    _dev(qkv, "qkv"); _dev(k_cache, "k_cache", qkv.dtype); _dev(v_cache, "v_cache", qkv.dtype)
    _dev(block_table, "block_table", torch.int32); _dev(tok_slot, "tok_slot", torch.int32)
    _dev(tok_pos, "tok_pos", torch.int32); _dev(dev_err, "dev_err", torch.int32)
    nb, hkv, bt, dh = k_cache.shape
    if hkv != n_kv_heads or dh != head_dim or v_cache.shape != k_cache.shape:
        raise KernelError("kv_append: cache shape does not match the heads")
    if qkv.shape[0] < n_tokens or tok_slot.shape[0] < n_tokens or tok_pos.shape[0] < n_tokens:
        raise KernelError("kv_append: fewer rows than tokens")
    ld = qkv.shape[1]
    if max(k_off, v_off) + n_kv_heads * head_dim > ld:
        raise KernelError("kv_append: K/V columns lie outside the row")
    call("vlrf_kv_append", _ptr(qkv), dtype_code(qkv.dtype), ld, k_off, v_off, _ptr(k_cache), _ptr(v_cache),
         _ptr(block_table), block_table.shape[1], _ptr(tok_slot), _ptr(tok_pos), n_tokens, n_kv_heads, head_dim,
         bt, _ptr(dev_err), _stream())


def attention_generic(qkv, q_off: int, k_cache, v_cache, block_table, tok_slot, tok_pos, out, n_tokens: int,
                      n_heads: int, n_kv_heads: int, head_dim: int, scale: float, window: int, dev_err) -> None:
    """Each token's query attends the keys 0…position of its slot in the paged cache."""
    _dev(qkv, "qkv"); _dev(k_cache, "k_cache", qkv.dtype); _dev(v_cache, "v_cache", qkv.dtype)
    _dev(out, "out", qkv.dtype); _dev(block_table, "block_table", torch.int32)
    _dev(tok_slot, "tok_slot", torch.int32); _dev(tok_pos, "tok_pos", torch.int32)
    _dev(dev_err, "dev_err", torch.int32)
    nb, hkv, bt, dh = k_cache.shape
    if hkv != n_kv_heads or dh != head_dim or v_cache.shape != k_cache.shape:
        raise KernelError("attention: cache shape does not match the heads")
    if out.shape[1] != n_heads * head_dim or out.shape[0] < n_tokens or qkv.shape[0] < n_tokens:
        raise KernelError("attention: output does not match")
    if q_off + n_heads * head_dim > qkv.shape[1]:
        raise KernelError("attention: Q columns lie outside the row")
    call("vlrf_attn_generic", _ptr(qkv), dtype_code(qkv.dtype), qkv.shape[1], q_off, _ptr(k_cache), _ptr(v_cache),
         _ptr(block_table), block_table.shape[1], _ptr(tok_slot), _ptr(tok_pos), _ptr(out), out.shape[1],
         n_tokens, n_heads, n_kv_heads, head_dim, bt, float(scale), int(window), _ptr(dev_err), _stream())


def sample(logits, n_rows: int, out_tokens, *, temperature=None, top_k=None, top_p=None, rng_key=None,
           rng_ctr=None) -> None:
    """One token per row of float32 logits.  Rows with temperature ≤ 0 (or no temperature tensor at all)
    take the first maximal index; the others draw after top-k / top-p filtering."""
    _dev(logits, "logits", torch.float32); _dev(out_tokens, "out_tokens", torch.int32)
    V = logits.shape[1]
    if logits.shape[0] < n_rows or out_tokens.shape[0] < n_rows:
        raise KernelError("sample: fewer rows than asked for")
    if temperature is not None:
        _dev(temperature, "temperature", torch.float32)
        _dev(rng_key, "rng_key", torch.int64); _dev(rng_ctr, "rng_ctr", torch.int32)
    if top_k is not None:
        _dev(top_k, "top_k", torch.int32)
    if top_p is not None:
        _dev(top_p, "top_p", torch.float32)
    call("vlrf_sample", _ptr(logits), V, n_rows, V, _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(rng_key),
         _ptr(rng_ctr), _ptr(out_tokens), _stream())


def apply_penalties(logits, n_rows: int, generated, generated_len, *, repetition=None, frequency=None,
                    presence=None, no_repeat_ngram=None) -> None:
    """Edit logits in place from each row's generated tokens [n_rows, max_generated] and their count."""
    _dev(logits, "logits", torch.float32); _dev(generated, "generated", torch.int32)
    _dev(generated_len, "generated_len", torch.int32)
    for name, t, dt in (("repetition", repetition, torch.float32), ("frequency", frequency, torch.float32),
                        ("presence", presence, torch.float32), ("no_repeat_ngram", no_repeat_ngram, torch.int32)):
        if t is not None:
            _dev(t, name, dt)
    V = logits.shape[1]
    call("vlrf_apply_penalties", _ptr(logits), V, n_rows, V, _ptr(generated), generated.shape[1],
         _ptr(generated_len), _ptr(repetition), _ptr(frequency), _ptr(presence), _ptr(no_repeat_ngram), _stream())
