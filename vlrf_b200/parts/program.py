"""A decode step as a list of operations that one persistent kernel runs.

A decode step of a few rows is some sixty small dependent operations; launched one by one, each pays its own
start-up.  A `DecodeProgram` is the same step written down once as data: the model's parts append their
operations (`emit_decode`), the list goes to the device, and `run()` is one launch of a kernel whose CTAs stay
resident and walk the list with a grid barrier after every operation (csrc/decode_program.cu).

The program knows three operations and no architecture:

    embed(table, positions_table, x)                         x[r] = table[token[r]] + positions_table[position[r]]
    product(inp, w, bias, out, norm=…, act=…, residual=…, kv_scatter=…)
                                                              out[r] = act(norm(inp[r]) · wᵀ + bias) (+ residual[r])
    attention(qkv, q_off, k_off, v_off, k_cache, v_cache, block_table, out, …)
                                                              one query per row and head over the paged cache

What one operation hands to the next lives in rows from `scratch(name, rows, cols, dtype)`: opaque to the parts,
which only pass them on; the kernel's operations wait for exactly the rows they read, so there is no barrier
between them.  What leaves the program (the logits) lies in `plain(...)` tensors.

A part that can state its decode step in these terms has a method `emit_decode(program, …)` (see the parts for
the arguments of each kind); it raises `NotFusable` if its sizes or options are outside what the kernel takes.
A model whose parts all have one decodes through a program; any other model decodes launch by launch as before.
"""
from __future__ import annotations

import torch

from ..csrc import KernelError, call, call_host, library, ops


class NotFusable(Exception):
    """This part, at these sizes, cannot be stated as operations of a decode program."""


NORM_KINDS = {None: 0, "layernorm": 1, "rmsnorm": 2}
F32, BF16, FLAGGED_F32, FLAGGED_BF16 = 0, 1, 2, 3


def norm_terms(norm):
    """(kind, weight, bias, eps) of a norm that says what it may be fused as, or NotFusable."""
    kind = getattr(norm, "fusable_as", None)
    if kind not in ("layernorm", "rmsnorm"):
        raise NotFusable(f"a norm of type {type(norm).__name__} does not say what it can be fused as")
    bias = getattr(norm, "bias", None) if kind == "layernorm" else None
    return kind, norm.weight, bias, float(norm.eps)


class FlaggedRows:
    """Rows that one operation of a program hands to a later one.  Every 8 bytes hold one float32 and a 32-bit flag,
    or three bfloat16 and a 16-bit flag; the flag says which operation of which launch wrote them, so a reader can
    wait for its data group by group and operations need no barrier between them (csrc/decode_program.cu).  `seg` > 0
    cuts a row's columns into segments that each begin a new (even-numbered) group: a head, so that one CTA writes
    whole groups.  Parts get these from `DecodeProgram.scratch` and only pass them on."""

    def __init__(self, storage: torch.Tensor, rows: int, cols: int, dtype: torch.dtype, seg: int):
        self.storage, self.rows, self.cols, self.dtype, self.seg = storage, rows, cols, dtype, seg
        self.fmt = FLAGGED_F32 if dtype == torch.float32 else FLAGGED_BF16
        self.ld = storage.numel() // rows                   # groups (8 bytes) a row
        self.writer = None                                  # index of the operation that wrote it last

    @staticmethod
    def groups_per_row(cols: int, dtype: torch.dtype, seg: int) -> int:
        per = 1 if dtype == torch.float32 else 3
        seg = seg if seg > 0 else cols
        per_segment = (-(-seg // per) + 1) // 2 * 2         # even: two groups are read at once
        return -(-cols // seg) * per_segment

    def data_ptr(self) -> int:
        return self.storage.data_ptr()


class DecodeProgram:
    def __init__(self, *, n_rows: int, tokens, tok_slot, tok_pos, dev_err, ws, act_dtype, max_context: int):
        lib = library()
        if act_dtype != torch.bfloat16:
            raise NotFusable("decode programs run the bfloat16 kernels only")
        if not (1 <= n_rows <= lib.vlrf_decode_program_max_rows()):
            raise NotFusable(f"{n_rows} rows; a decode program takes at most {lib.vlrf_decode_program_max_rows()}")
        self.n_rows, self.ws, self.act_dtype, self.max_context = n_rows, ws, act_dtype, int(max_context)
        self.tokens, self.tok_slot, self.tok_pos, self.dev_err = tokens, tok_slot, tok_pos, dev_err
        self.device = tokens.device
        self._op_bytes = lib.vlrf_decode_program_op_bytes()
        self._calls: list = []          # (entry point, arguments after the host buffer and index)
        self._keep: list = []           # tensors the operations point at
        self._flagged: dict = {}
        self._ops_dev = None
        self._sync = None

    # -- what the parts call ------------------------------------------------------------------------
    def scratch(self, name: str, rows: int, cols: int, dtype, seg: int = 0) -> FlaggedRows:
        """Rows that an operation writes and later ones read (the same rows for the same name and shape)."""
        key = (name, rows, cols, dtype, seg)
        buf = self._flagged.get(key)
        if buf is None:
            n = rows * FlaggedRows.groups_per_row(cols, dtype, seg)
            storage = torch.zeros(n, dtype=torch.int64, device=self.device)     # flag 0: written by nobody yet
            buf = self._flagged[key] = FlaggedRows(storage, rows, cols, dtype, seg)
        return buf

    def plain(self, name: str, rows: int, cols: int, dtype) -> torch.Tensor:
        """Plain rows for what leaves the program (the logits)."""
        return self.ws.get(name, rows, cols, dtype)

    def _buf(self, t, cols: int, reading: bool):
        """(pointer, format, ld, seg, dep) of a buffer argument: a plain tensor or flagged rows."""
        if isinstance(t, FlaggedRows):
            if t.cols != cols or t.rows < self.n_rows:
                raise NotFusable("flagged rows of another shape")
            if reading and t.writer is None:
                raise KernelError("a decode program reads rows that no operation of it has written")
            self._keep.append(t.storage)
            return t.data_ptr(), t.fmt, t.ld, t.seg, (t.writer if reading else -1)
        if not t.is_cuda or not t.is_contiguous() or t.dtype not in (torch.float32, torch.bfloat16) or t.shape[1] != cols \
                or t.shape[0] < self.n_rows:
            raise NotFusable("operands must be contiguous float32 or bfloat16 device tensors of the step's rows")
        self._keep.append(t)
        return t.data_ptr(), (F32 if t.dtype == torch.float32 else BF16), t.shape[1], 0, -1

    def embed(self, table, positions_table, x) -> None:
        if table.dtype != torch.bfloat16 or (positions_table is not None and positions_table.dtype != torch.bfloat16):
            raise NotFusable("embedding tables must be bfloat16")
        if x.dtype != torch.float32:
            raise NotFusable("the embedding writes float32 rows")
        ptr, fmt, ld, _, _ = self._buf(x, table.shape[1], reading=False)
        self._keep += [table, positions_table]
        self._calls.append(("vlrf_decode_op_embed", (
            table.data_ptr(), 0 if positions_table is None else positions_table.data_ptr(), self.tokens.data_ptr(),
            ptr, fmt, ld, table.shape[1], table.shape[0], 0 if positions_table is None else positions_table.shape[0])))
        if isinstance(x, FlaggedRows):
            x.writer = len(self._calls) - 1

    def product(self, inp, w, bias, out, *, norm=None, act=None, residual=None, kv_scatter=None) -> None:
        """out[r] = act(norm(inp[r]) · wᵀ + bias) (+ residual[r]) for the program's rows.  inp, out, residual: plain
        tensors or flagged rows [rows, K] / [rows, N] (float32 or bfloat16; a residual float32 like out); w bfloat16
        [N, K]; norm: None or (kind, weight, bias, eps) as `norm_terms` gives; kv_scatter = (k_cache, v_cache,
        block_table, k_off, v_off, n_kv_heads, head_dim)."""
        lib = library()
        N, K = w.shape
        kind, gamma, beta, eps = norm if norm is not None else (None, None, None, 0.0)
        if w.dtype != torch.bfloat16 or not w.is_cuda or not w.is_contiguous():
            raise NotFusable("weights must be contiguous bfloat16 device tensors")
        for t in (gamma, beta, bias):
            if t is not None and (t.dtype != torch.float32 or not t.is_cuda or not t.is_contiguous()):
                raise NotFusable("norm weights and biases are float32 device tensors")
        i_ptr, i_fmt, i_ld, i_seg, i_dep = self._buf(inp, K, reading=True)
        r_ptr, r_fmt, r_ld, r_dep = 0, 0, 0, -1
        if residual is not None:
            r_ptr, r_fmt, r_ld, _, r_dep = self._buf(residual, N, reading=True)
        o_ptr, o_fmt, o_ld, _, _ = self._buf(out, N, reading=False)
        if not lib.vlrf_decode_program_gemv_takes(self.n_rows, N, K, i_fmt, o_fmt, NORM_KINDS[kind]):
            raise NotFusable(f"a product of N={N}, K={K} over {self.n_rows} rows is not taken by the decode program")
        kv = (0, 0, 0, 0, 0, 0, 0, 0, 0)
        if kv_scatter is not None:
            kc, vc, table, k_off, v_off, hkv, dh = kv_scatter
            if kc.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or dh & (dh - 1) or kc.shape[2] & (kc.shape[2] - 1):
                raise NotFusable("the cache scatter writes bfloat16 heads whose size is a power of two")
            kv = (kc.data_ptr(), vc.data_ptr(), table.data_ptr(), table.shape[1], k_off, v_off, hkv, dh, kc.shape[2])
            self._keep += [kc, vc, table]
        self._keep += [w, bias, gamma, beta]
        self._calls.append(("vlrf_decode_op_gemv", (
            self.n_rows, i_ptr, i_fmt, i_ld, i_seg, i_dep, NORM_KINDS[kind], ops._ptr(gamma), ops._ptr(beta), float(eps),
            w.data_ptr(), ops._ptr(bias), N, K, ops.ACT[act], o_ptr, o_fmt, o_ld, r_ptr, r_fmt, r_ld, r_dep, *kv)))
        if isinstance(out, FlaggedRows):
            out.writer = len(self._calls) - 1

    def attention(self, qkv, q_off: int, k_off: int, v_off: int, k_cache, v_cache, block_table, out, *, n_heads: int,
                  n_kv_heads: int, head_dim: int, scale: float, window: int = 0) -> None:
        """out[r, head] = attention of the query at columns q_off… of qkv[r] over the keys 0…position of row r's slot.
        With flagged qkv rows (written by a product of this program whose cache scatter also stores them) the newest
        key and value are read from there, columns k_off… and v_off…; `out`: [rows, n_heads·head_dim] bfloat16, flagged
        rows with one segment a head (`scratch(…, seg=head_dim)`) or a plain tensor."""
        lib = library()
        bt = k_cache.shape[2]
        if qkv.dtype != torch.bfloat16 or k_cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
            raise NotFusable("attention operands must be bfloat16")
        if not lib.vlrf_decode_program_attention_takes(head_dim, bt):
            raise NotFusable(f"attention with head size {head_dim} is not taken by the decode program")
        if k_cache.numel() >= 2 ** 31:
            raise NotFusable("a cache pool of 2^31 elements or more")
        if isinstance(out, FlaggedRows) and out.seg != head_dim:
            raise NotFusable("flagged attention output has one segment a head")
        cols = qkv.cols if isinstance(qkv, FlaggedRows) else qkv.shape[1]
        i_ptr, i_fmt, i_ld, _, i_dep = self._buf(qkv, cols, reading=True)
        o_ptr, o_fmt, o_ld, _, _ = self._buf(out, n_heads * head_dim, reading=False)
        pairs = self.n_rows * n_heads
        # One CTA a (row, head) while a context is short: parts pay a merge through global memory (three more round
        # trips to L2) that only long contexts earn back.
        n_split = max(1, min(16, ops.sm_count() // pairs, self.max_context // 1024))
        partials = counters = None
        if n_split > 1:
            partials = self.ws.get("program_partials", pairs * n_split, head_dim + 2, torch.float32)
            counters = self.ws.get_zeroed("program_counters", pairs, torch.int32)
        self._keep += [k_cache, v_cache, block_table, partials, counters]
        self._calls.append(("vlrf_decode_op_attention", (
            i_ptr, i_fmt, i_ld, i_dep, cols, q_off, k_off, v_off, k_cache.data_ptr(), v_cache.data_ptr(), block_table.data_ptr(),
            block_table.shape[1], o_ptr, o_fmt, o_ld, n_heads, n_kv_heads, head_dim, bt, float(scale), int(window),
            n_split, ops._ptr(partials), ops._ptr(counters))))
        if isinstance(out, FlaggedRows):
            out.writer = len(self._calls) - 1

    # -- what the step calls --------------------------------------------------------------------------
    @property
    def n_ops(self) -> int:
        return len(self._calls)

    def finalize(self) -> None:
        """Write the operations down and copy them to the device."""
        if not self._calls:
            raise KernelError("a decode program without operations")
        host = torch.zeros(len(self._calls) * self._op_bytes, dtype=torch.uint8)
        for i, (name, args) in enumerate(self._calls):
            call_host(name, host.data_ptr(), i, *args)
        self._ops_dev = host.to(self.device)
        self._sync = torch.zeros(4, dtype=torch.int32, device=self.device)

    def run(self, trace=None) -> None:
        call("vlrf_decode_program_run", self._ops_dev.data_ptr(), len(self._calls), self.n_rows, self.tok_slot.data_ptr(),
             self.tok_pos.data_ptr(), self._sync.data_ptr(), self.dev_err.data_ptr(), ops._ptr(trace), ops._stream())

    def trace(self) -> torch.Tensor:
        """Runs the program once more and returns int64 [CTAs, operations + 1, 8]: nanoseconds at which each CTA began
        each operation ([:, i, 0]; [:, n, 0]: finished the last) and reached stages inside it ([:, i, 1…4]: rows
        staged, first weights landed, products done, results stored; 0 where a CTA had no share of the operation)."""
        t = torch.zeros(ops.sm_count(), len(self._calls) + 1, 8, dtype=torch.int64, device=self.device)
        self.run(t)
        return t.cpu()

    def profile(self) -> list:
        """Runs the program once more and returns for every operation (its kind, microseconds from the moment the
        last CTA had stored the results of the operation before to the moment the last CTA had stored this one's):
        the operation's share of the step's critical path."""
        t = self.trace()
        begin = int(t[:, 0, 0].min())
        done_before, out = begin, []
        for i, (name, _) in enumerate(self._calls):
            stored = t[:, i, 4]
            done = int(stored.max()) if int(stored.max()) > 0 else done_before
            out.append((name.replace("vlrf_decode_op_", ""), (done - done_before) / 1e3))
            done_before = done
        return out
