"""Tensor-level entry to the kernels: checks, then raw pointers and the current stream.

Every function writes into tensors that the caller provides; nothing here allocates.  All tensors must
be contiguous CUDA tensors.  Sizes a kernel cannot take are refused with a `KernelError` that says why;
no function has a CPU or library fallback.
"""
from __future__ import annotations

import os

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


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current CUDA stream's handle.  Asked for at every launch, so by the short way where torch has one
    (`torch.cuda.current_stream()` builds a Stream object: about 5 us, a quarter of a launch's host time)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
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


def embed(wte, wpe, tokens, positions, out, dev_err, stats: "RowStats | None" = None) -> None:
    """out[t] = wte[tokens[t]] (+ wpe[positions[t]]), float32.  With `stats` and few rows (a decode step) the rows'
    statistics are left there for the next product's LayerNorm."""
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
    keep = stats is not None and stats.takes(T, d)     # few rows: a decode step; leave their statistics
    if stats is not None:
        stats.written(out)
    call("vlrf_embed", _ptr(wte), _ptr(wpe), dtype_code(wte.dtype), _ptr(tokens), _ptr(positions), _ptr(out),
         T, d, V, P, _ptr(stats.buffer()) if keep else 0, _ptr(dev_err), _stream())
    if keep:
        stats.keep(out, T, d)


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


def linear(x, w, bias, out, *, act=None, residual=None, rows: int | None = None, kv_scatter=None,
           stats: "RowStats | None" = None) -> bool:
    """out = act(x · wᵀ + bias) (+ residual).  x [M,K], w [N,K] (same dtype), bias/residual float32,
    out [M,N] float32 or bfloat16.  `rows` limits M to the first rows of x/out/residual.  `kv_scatter`
    (see linear_layernorm) asks the kernel to write K/V columns into a cache as well; the return value
    says whether it did (only the tensor-core kernels can).  `stats`: where the statistics of float32 result rows
    are left when the kernel that takes the shape computes them (and where stale ones of `out` are forgotten)."""
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
    if stats is not None:
        stats.written(out)
    return _linear_dispatch(x, w, bias, out, ACT[act], residual, M, N, K, kv_scatter, stats)


#: head sizes that the attention kernels take (each checks it again; parts refuse others when they are built)
HEAD_DIM_STEP, HEAD_DIM_MAX = 16, 256
_SM_COUNT = None
USE_TCGEN05 = True
PREFILL_ATTENTION_TCGEN05 = True     # head size 64; off: the mma.sync kernel takes those too
PREFILL_ATTENTION_PARTS = None       # a number here overrides attention_prefill_parts (for measurements)
SKINNY_MAX_ROWS = 64
FUSED_NORM_MAX_ROWS = 16
SWAPPED_MIN_COLUMNS = 16384
#: Few-row products whose weight matrix has at least this many bytes go to the split-k tcgen05 kernel (the
#: second figure: with the LayerNorm fused in).  Measured on B200 inside whole decode steps, the split-k kernel
#: wins at every size of GPT-2's: its CTAs leave room on an SM for the next kernel's to begin ahead, and it
#: passes on the row statistics that the next LayerNorm needs.  The `mma.sync` kernel remains for the shapes
#: the split-k kernel refuses and for a LayerNorm of rows whose statistics nobody left.
SPLITK_MIN_WEIGHT_BYTES = 0
SPLITK_NORM_MIN_WEIGHT_BYTES = 0
_DEV_ERR = None


ROW_STATS_MAX_ROWS, ROW_STATS_MAX_WIDTH = 64, 8192


class RowStats:
    """Statistics of the float32 residual rows that a product has just written (per row and 32-column segment: sum
    and squared deviation from the segment's mean), kept so that the next product can apply a LayerNorm to those
    rows without reading them whole.  One buffer of fixed address (graphs capture it) on the device of the
    workspace that owns it; `of` says whose rows it describes: (the tensor, its torch version counter then, rows,
    width) or None.  The tensor is held, so its memory cannot be given to another tensor meanwhile.

    Who may trust them: a product of this module that is handed the same object and the same rows.  Who keeps them
    honest: every function of this module that writes a tensor and is handed the object forgets stale statistics;
    torch's in-place operations are seen by the version counter; and the block forgets them after any part that does
    not declare `leaves_row_stats` (parts/block.py), so a part that writes the residual with kernels of its own
    cannot leave them stale by omission."""

    def __init__(self, device):
        self.device = torch.device(device)
        self._buffer = None
        self.of = None

    def buffer(self) -> torch.Tensor:
        if self._buffer is None:
            self._buffer = torch.zeros(ROW_STATS_MAX_ROWS * (ROW_STATS_MAX_WIDTH // 32) * 2, dtype=torch.float32,
                                       device=self.device)
        return self._buffer

    def takes(self, rows: int, width: int) -> bool:
        return 0 < rows <= ROW_STATS_MAX_ROWS and width <= ROW_STATS_MAX_WIDTH

    def keep(self, t, rows: int, width: int) -> None:
        v = _version_of(t)
        self.of = (t, v, rows, width) if v >= 0 else None

    def forget(self) -> None:
        self.of = None

    def written(self, t) -> None:
        """`t` is being rewritten: statistics kept of it are stale."""
        if self.of is not None and t is not None and self.of[0].data_ptr() == t.data_ptr():
            self.of = None

    def describing(self, x, rows: int, width: int):
        """The statistics buffer if it describes exactly these rows as they are now, else None."""
        if self.of is None:
            return None
        held, version, n_rows, n_cols = self.of
        if held.data_ptr() == x.data_ptr() and _version_of(x) == version and (n_rows, n_cols) == (rows, width):
            return self._buffer
        return None


def _version_of(t) -> int:
    """torch's count of in-place changes of a tensor, or −1 where it is not kept (inference mode): then no
    statistics are kept either, since a change behind their back could not be seen."""
    try:
        return t._version
    except RuntimeError:
        return -1


def _splitk_takes(M: int, N: int, K: int, ldx: int, fused_norm: bool) -> bool:
    least = SPLITK_NORM_MIN_WEIGHT_BYTES if fused_norm else SPLITK_MIN_WEIGHT_BYTES
    if not USE_TCGEN05 or 2 * N * K < least or N >= SWAPPED_MIN_COLUMNS:
        return False
    from . import library
    return bool(library().vlrf_gemm_splitk_takes(M, N, K, ldx, 1 if fused_norm else 0))


def _dev_err() -> torch.Tensor:
    """The process-wide device error word for kernels whose callers pass none: int32 [1]; `device_errors()`
    reads and clears it."""
    global _DEV_ERR
    if _DEV_ERR is None:
        _DEV_ERR = torch.zeros(1, dtype=torch.int32, device="cuda")
    return _DEV_ERR


def set_chained_launch(on: bool) -> None:
    """Whether kernels are launched so that each may begin (fetch weights) while the one before it still
    runs.  On by default; off gives plain stream order."""
    call("vlrf_set_chained_launch", 1 if on else 0)


def device_errors() -> int:
    """Bits that kernels set in the shared error word since the last call (synchronises)."""
    if _DEV_ERR is None:
        return 0
    word = int(_DEV_ERR.item())
    if word:
        _DEV_ERR.zero_()
    return word


def sm_count() -> int:
    global _SM_COUNT
    if _SM_COUNT is None:
        import ctypes
        from . import library
        vals = [ctypes.c_int(0) for _ in range(4)]
        if library().vlrf_device_info(*[ctypes.byref(v) for v in vals]) != 0:
            raise KernelError("cannot query the device")
        _SM_COUNT = vals[0].value
    return _SM_COUNT


def _kv_args(kv_scatter, N: int) -> list:
    if kv_scatter is None:
        return [0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0]
    kc, vc, table, tok_slot, tok_pos, k_off, v_off, hkv, dh = kv_scatter
    _dev(kc, "k_cache", torch.bfloat16); _dev(vc, "v_cache", torch.bfloat16)
    _dev(table, "block_table", torch.int32); _dev(tok_slot, "tok_slot", torch.int32)
    _dev(tok_pos, "tok_pos", torch.int32)
    if kc.shape[1] != hkv or kc.shape[3] != dh or max(k_off, v_off) + hkv * dh > N:
        raise KernelError("cache scatter does not match the projection")
    return [_ptr(kc), _ptr(vc), _ptr(table), table.shape[1], _ptr(tok_slot), _ptr(tok_pos), k_off, v_off, hkv, dh,
            kc.shape[2]]


def _linear_dispatch(x, w, bias, out, act, residual, M, N, K, kv_scatter=None, stats=None) -> bool:
    bf16_out = out.dtype == torch.bfloat16
    if (x.dtype == torch.bfloat16 and M <= SKINNY_MAX_ROWS and K % 8 == 0 and USE_TCGEN05 and kv_scatter is None
            and N >= SWAPPED_MIN_COLUMNS):
        # few rows, very many columns (the head over the vocabulary): enough 128-row tiles of w to fill the GPU,
        # so w becomes the 128-row operand of the tcgen05 kernel and the rows of x its N
        call("vlrf_gemm_tcgen05", _ptr(x), _ptr(w), _ptr(bias), _ptr(residual), _ptr(out), M, N, K, K, N,
             dtype_code(out.dtype), act, *_kv_args(None, N), _ptr(_dev_err()), _stream())
        return False
    if x.dtype == torch.bfloat16 and M <= SKINNY_MAX_ROWS and _splitk_takes(M, N, K, K, False):
        # few rows, a large matrix: tiles of w on the tensor cores, the sum over k cut into parts
        scatter = kv_scatter is not None and bf16_out
        keep = stats is not None and not bf16_out and stats.takes(M, N)
        call("vlrf_gemm_splitk", _ptr(x), 0, _ptr(w), _ptr(bias), _ptr(residual), _ptr(out), dtype_code(out.dtype),
             M, N, K, K, N, act, 0, 0, 0.0, *_kv_args(kv_scatter if scatter else None, N), 0,
             _ptr(stats.buffer()) if keep else 0, _ptr(_dev_err()), _stream())
        if keep:
            stats.keep(out, M, N)
        return scatter
    if x.dtype == torch.bfloat16 and M <= SKINNY_MAX_ROWS and K % 32 == 0:
        # few rows: the product is bound by streaming w once
        scatter = kv_scatter is not None and bf16_out
        call("vlrf_gemm_skinny", _ptr(x), 0, _ptr(w), _ptr(bias), _ptr(residual), _ptr(out), dtype_code(out.dtype),
             M, N, K, K, N, act, 0, 0, 0.0, *_kv_args(kv_scatter if scatter else None, N), sm_count(), _ptr(_dev_err()),
             _stream())
        return scatter
    if x.dtype == torch.bfloat16 and K % 8 == 0 and USE_TCGEN05:
        # many rows: the tensor-core kernel (tcgen05, accumulator in tensor memory)
        scatter = kv_scatter is not None and bf16_out and kv_scatter[8] % 8 == 0 and kv_scatter[5] % 8 == 0
        call("vlrf_gemm_tcgen05", _ptr(x), _ptr(w), _ptr(bias), _ptr(residual), _ptr(out), M, N, K, K, N,
             dtype_code(out.dtype), act, *_kv_args(kv_scatter if scatter else None, N), _ptr(_dev_err()), _stream())
        return scatter
    call("vlrf_gemm_simt", _ptr(x), _ptr(w), _ptr(bias), _ptr(residual), _ptr(out), M, N, K, K, N,
         dtype_code(x.dtype), dtype_code(out.dtype), act, _stream())
    return False


def can_fuse_layernorm(n_rows: int, width: int, w_dtype: torch.dtype) -> bool:
    """Whether `linear_layernorm` takes this many rows of this width."""
    # with more rows, every CTA repeating the norm costs more than a norm kernel of its own
    if w_dtype != torch.bfloat16 or n_rows > FUSED_NORM_MAX_ROWS or n_rows < 1 or width % 32 != 0:
        return False
    from . import library
    return bool(library().vlrf_gemm_skinny_ln_fits(n_rows, width))


def linear_layernorm(x, gamma, beta, eps: float, w, bias, out, *, act=None, rows: int | None = None,
                     kv_scatter=None, stats: "RowStats | None" = None) -> None:
    """out = act(LayerNorm(x) · wᵀ + bias) for few rows, the norm fused into the product's prologue.
    x float32 [M,K]; w bfloat16 [N,K]; out bfloat16 or float32.  `kv_scatter` = (k_cache, v_cache,
    block_table, tok_slot, tok_pos, k_off, v_off, n_kv_heads, head_dim) also writes those columns of the
    result into one layer's paged cache."""
    _dev(x, "x", torch.float32); _dev(w, "w", torch.bfloat16); _dev(out, "out")
    _dev(gamma, "gamma", torch.float32); _dev(beta, "beta", torch.float32)
    M = x.shape[0] if rows is None else rows
    K, N = x.shape[1], w.shape[0]
    if w.shape[1] != K or out.shape[1] != N or out.shape[0] < M or gamma.shape[0] != K or beta.shape[0] != K:
        raise KernelError("linear_layernorm: sizes do not match")
    if bias is not None:
        _dev(bias, "bias", torch.float32)
    kv = _kv_args(kv_scatter, N)
    known = stats.describing(x, M, K) if stats is not None else None
    if stats is not None:
        stats.written(out)
    if known is not None and _splitk_takes(M, N, K, K, True):
        # the rows' statistics are at hand: each CTA normalises only the columns it multiplies
        call("vlrf_gemm_splitk", _ptr(x), 1, _ptr(w), _ptr(bias), 0, _ptr(out), dtype_code(out.dtype), M, N, K, K, N,
             ACT[act], _ptr(gamma), _ptr(beta), float(eps), *kv, _ptr(known), 0, _ptr(_dev_err()), _stream())
        return
    call("vlrf_gemm_skinny", _ptr(x), 1, _ptr(w), _ptr(bias), 0, _ptr(out), dtype_code(out.dtype), M, N, K, K, N,
         ACT[act], _ptr(gamma), _ptr(beta), float(eps), *kv, sm_count(), _ptr(_dev_err()), _stream())


def decode_splits(n_rows: int, n_heads: int, max_context: int) -> int:
    """Into how many parts a decode step cuts each context.  Measured inside whole steps of GPT-2 small,
    medium and XL: up to about 1.75 CTAs an SM in all, parts of at least 256 keys; more CTAs than that cost
    more (shared memory that the next kernel's CTAs would use, clusters to place) than they hide."""
    forced = os.environ.get("VLRF_B200_DECODE_SPLITS")
    if forced:
        return max(1, min(16, int(forced)))
    pairs = max(1, n_rows * n_heads)
    want = (7 * sm_count()) // (4 * pairs)
    return max(1, min(16, want, -(-max_context // 256)))


def attention_decode_needs_scratch(head_dim: int, n_split: int) -> bool:
    """Whether `attention_decode` with this split needs `partials` and `counters` (else the parts of a
    context merge inside a thread-block cluster)."""
    from . import library
    return bool(library().vlrf_attn_decode_needs_scratch(head_dim, n_split))


def attention_decode(qkv, q_off: int, k_cache, v_cache, block_table, tok_slot, tok_pos, out, n_rows: int,
                     n_heads: int, n_kv_heads: int, head_dim: int, scale: float, window: int, n_split: int,
                     partials, counters, dev_err) -> None:
    """One query per row attends the keys 0…position of its slot; the context is cut into n_split parts.
    partials: float32 scratch of n_rows·n_heads·n_split·(head_dim+2); counters: int32 [n_rows·n_heads],
    zero between calls."""
    _dev(qkv, "qkv"); _dev(k_cache, "k_cache", qkv.dtype); _dev(v_cache, "v_cache", qkv.dtype)
    _dev(out, "out", qkv.dtype); _dev(block_table, "block_table", torch.int32)
    _dev(tok_slot, "tok_slot", torch.int32); _dev(tok_pos, "tok_pos", torch.int32)
    _dev(dev_err, "dev_err", torch.int32)
    nb, hkv, bt, dh = k_cache.shape
    if hkv != n_kv_heads or dh != head_dim or v_cache.shape != k_cache.shape:
        raise KernelError("attention_decode: cache shape does not match the heads")
    if out.shape[1] != n_heads * head_dim or out.shape[0] < n_rows or qkv.shape[0] < n_rows:
        raise KernelError("attention_decode: output does not match")
    if n_split > 1 and partials is not None:
        _dev(partials, "partials", torch.float32); _dev(counters, "counters", torch.int32)
        if partials.numel() < n_rows * n_heads * n_split * (head_dim + 2) or counters.numel() < n_rows * n_heads:
            raise KernelError("attention_decode: scratch is too small")
    call("vlrf_attn_decode", _ptr(qkv), dtype_code(qkv.dtype), qkv.shape[1], q_off, _ptr(k_cache), _ptr(v_cache), nb,
         _ptr(block_table), block_table.shape[1], _ptr(tok_slot), _ptr(tok_pos), _ptr(out), out.shape[1], n_rows,
         n_heads, n_kv_heads, head_dim, bt, float(scale), int(window), int(n_split), _ptr(partials), _ptr(counters),
         _ptr(dev_err), _stream())


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
           rng_ctr=None, next_tokens=None, next_pos=None, row_slot=None) -> None:
    """One token per row of float32 logits.  Rows with temperature ≤ 0 (or no temperature tensor at all)
    take the first maximal index; the others draw after top-k / top-p filtering.  `next_tokens`,
    `next_pos`, `row_slot` (int32 [n_rows], optional): the kernel also writes each token into next_tokens
    and adds one to next_pos where row_slot is not −1, which is all a decode session needs to go on."""
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
    for name, t in (("next_tokens", next_tokens), ("next_pos", next_pos), ("row_slot", row_slot)):
        if t is not None:
            _dev(t, name, torch.int32)
            if t.shape[0] < n_rows:
                raise KernelError(f"sample: {name} has fewer rows than asked for")
    call("vlrf_sample", _ptr(logits), V, n_rows, V, _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(rng_key),
         _ptr(rng_ctr), _ptr(out_tokens), _ptr(next_tokens), _ptr(next_pos), _ptr(row_slot), _stream())


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


def attention_prefill_takes(dtype: torch.dtype, head_dim: int, block_tokens: int, row_width: int, q_off: int) -> bool:
    """Whether the tensor-core prompt attention takes these sizes."""
    if dtype != torch.bfloat16:
        return False
    from . import library
    return bool(library().vlrf_attn_prefill_takes(head_dim, block_tokens, row_width, q_off))


def attention_prefill_kind(dtype: torch.dtype, head_dim: int, block_tokens: int, row_width: int, q_off: int, out_width: int) -> str:
    """Which kernel prompt attention of these sizes runs on: "tcgen05" (bfloat16, head size 64), "mma.sync"
    (bfloat16, head sizes 64 and 128) or "CUDA cores" (everything else, and the 32-bit path)."""
    from . import library
    lib = library()
    if dtype == torch.bfloat16 and PREFILL_ATTENTION_TCGEN05 and lib.vlrf_attn_prefill_tc_takes(head_dim, block_tokens, row_width, q_off, out_width):
        return "tcgen05"
    if dtype == torch.bfloat16 and lib.vlrf_attn_prefill_takes(head_dim, block_tokens, row_width, q_off):
        return "mma.sync"
    return "CUDA cores"


def attention_decode_kind(dtype: torch.dtype, head_dim: int) -> str:
    """Which kernel decode attention runs on: "mma.sync" (bfloat16, head size 64) or "CUDA cores"."""
    return "mma.sync" if dtype == torch.bfloat16 and head_dim == 64 else "CUDA cores"


def attention_prefill_parts(dtype: torch.dtype, n_seqs: int, max_new: int, n_heads: int, head_dim: int, block_tokens: int,
                            row_width: int, q_off: int) -> int:
    """Into how many parts `attention_prefill` best deals the keys of a long tile of queries (1: not at all;
    more want scratch, see there).  A tile's key blocks are a chain, so a step with few tiles is bound by its
    longest one (`tiles` blocks, for sequences that start at 0), not by the SMs: all blocks together, spread
    over the two CTAs that an SM holds, come to `even` blocks each, and parts pay when the chain is the longer
    of the two."""
    from . import library
    lib = library()
    if not PREFILL_ATTENTION_TCGEN05 or dtype != torch.bfloat16 \
            or not lib.vlrf_attn_prefill_tc_takes(head_dim, block_tokens, row_width, q_off, n_heads * head_dim):
        return 1
    tiles = -(-max_new // lib.vlrf_attn_prefill_tc_tile())
    even = tiles * (tiles + 1) / 2 * n_heads * n_seqs / (2 * sm_count())
    parts = int(tiles / (1.3 * max(even, lib.vlrf_attn_prefill_tc_min_part_blocks())) + 0.5)   # 1.3: a part's own cost
    if PREFILL_ATTENTION_PARTS is not None:
        parts = PREFILL_ATTENTION_PARTS
    return max(1, min(parts, lib.vlrf_attn_prefill_tc_max_parts()))


def attention_prefill_scratch(n_seqs: int, max_new: int, n_heads: int, n_parts: int) -> tuple[int, int]:
    """(float32 elements of `partials`, int32 elements of `counters`) that `attention_prefill` wants for
    n_parts > 1."""
    from . import library
    lib = library()
    tiles = -(-max_new // lib.vlrf_attn_prefill_tc_tile()) * n_seqs * n_heads
    return tiles * n_parts * lib.vlrf_attn_prefill_tc_part_floats(), tiles


def attention_prefill(qkv, q_off: int, k_cache, v_cache, block_table, seq_slot, seq_start, seq_pos0, out,
                      n_tokens: int, n_seqs: int, max_new: int, n_heads: int, n_kv_heads: int, head_dim: int,
                      scale: float, window: int, dev_err, n_parts: int = 1, partials=None, counters=None) -> None:
    """Causal attention of every sequence's new tokens (rows seq_start[i] … seq_start[i+1]−1 of qkv, the
    first of them at position seq_pos0[i]) over the sequence's cache, which already holds these tokens'
    keys and values.  bfloat16, head size 64 or 128.  n_parts > 1 (see attention_prefill_parts) deals the keys
    of long tiles to several CTAs and wants float32 `partials` and zeroed int32 `counters` of the sizes that
    attention_prefill_scratch gives; the counters are left zero."""
    _dev(qkv, "qkv", torch.bfloat16); _dev(k_cache, "k_cache", torch.bfloat16); _dev(v_cache, "v_cache", torch.bfloat16)
    _dev(out, "out", torch.bfloat16); _dev(block_table, "block_table", torch.int32)
    _dev(seq_slot, "seq_slot", torch.int32); _dev(seq_start, "seq_start", torch.int32)
    _dev(seq_pos0, "seq_pos0", torch.int32); _dev(dev_err, "dev_err", torch.int32)
    nb, hkv, bt, dh = k_cache.shape
    if hkv != n_kv_heads or dh != head_dim or v_cache.shape != k_cache.shape:
        raise KernelError("attention_prefill: cache shape does not match the heads")
    if out.shape[1] != n_heads * head_dim or out.shape[0] < n_tokens or qkv.shape[0] < n_tokens:
        raise KernelError("attention_prefill: output does not match")
    if seq_slot.shape[0] < n_seqs or seq_start.shape[0] < n_seqs + 1 or seq_pos0.shape[0] < n_seqs:
        raise KernelError("attention_prefill: sequence tables are too short")
    from . import library
    if PREFILL_ATTENTION_TCGEN05 and library().vlrf_attn_prefill_tc_takes(head_dim, bt, qkv.shape[1], q_off, out.shape[1]):
        # head size 64: S and O on the tcgen05 tensor cores, accumulators in tensor memory
        if n_parts > 1:
            _dev(partials, "partials", torch.float32); _dev(counters, "counters", torch.int32)
            want = attention_prefill_scratch(n_seqs, max_new, n_heads, n_parts)
            if partials.numel() < want[0] or counters.numel() < want[1]:
                raise KernelError("attention_prefill: scratch is too small for %d parts" % n_parts)
        call("vlrf_attn_prefill_tc", _ptr(qkv), qkv.shape[1], q_off, _ptr(k_cache), _ptr(v_cache), nb, _ptr(block_table),
             block_table.shape[1], _ptr(seq_slot), _ptr(seq_start), _ptr(seq_pos0), _ptr(out), out.shape[1], n_tokens,
             n_seqs, max_new, n_heads, n_kv_heads, head_dim, bt, float(scale), int(window), int(n_parts),
             _ptr(partials) if n_parts > 1 else 0, _ptr(counters) if n_parts > 1 else 0, _ptr(dev_err), _stream())
        return
    call("vlrf_attn_prefill", _ptr(qkv), qkv.shape[1], q_off, _ptr(k_cache), _ptr(v_cache), nb, _ptr(block_table),
         block_table.shape[1], _ptr(seq_slot), _ptr(seq_start), _ptr(seq_pos0), _ptr(out), out.shape[1], n_tokens, n_seqs,
         max_new, n_heads, n_kv_heads, head_dim, bt, float(scale), int(window), _ptr(dev_err), _stream())
