"""A decode step as a list of operations that one persistent kernel runs.

A decode step of a few rows is some sixty small dependent operations; launched one by one, each pays its own
start-up.  A `DecodeProgram` is the same step written down once as data: the model's parts append their
operations (`emit_decode`), the list goes to the device, and `run()` is one launch of a kernel whose CTAs stay
resident and walk the list with a grid barrier after every operation (csrc/decode_program.cu).

The program knows three operations and no architecture:

    embed(table, positions_table, x)                         x[r] = table[token[r]] + positions_table[position[r]]
    product(inp, w, bias, out, norm=…, act=…, residual=…, kv_scatter=…)
                                                              out[r] = act(norm(inp[r]) · wᵀ + bias) (+ residual[r])
    attention(qkv, q_off, k_cache, v_cache, block_table, out, …)
                                                              one query per row and head over the paged cache

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


def norm_terms(norm):
    """(kind, weight, bias, eps) of a norm that says what it may be fused as, or NotFusable."""
    kind = getattr(norm, "fusable_as", None)
    if kind not in ("layernorm", "rmsnorm"):
        raise NotFusable(f"a norm of type {type(norm).__name__} does not say what it can be fused as")
    bias = getattr(norm, "bias", None) if kind == "layernorm" else None
    return kind, norm.weight, bias, float(norm.eps)


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
        self._ops_dev = None
        self._sync = None

    # -- what the parts call ------------------------------------------------------------------------
    def scratch(self, name: str, rows: int, cols: int, dtype) -> torch.Tensor:
        return self.ws.get(name, rows, cols, dtype)

    def embed(self, table, positions_table, x) -> None:
        if table.dtype != torch.bfloat16 or (positions_table is not None and positions_table.dtype != torch.bfloat16):
            raise NotFusable("embedding tables must be bfloat16")
        if table.shape[1] % 2 != 0 or x.dtype != torch.float32 or x.shape[1] != table.shape[1]:
            raise NotFusable("embedding width")
        self._keep += [table, positions_table, x]
        self._calls.append(("vlrf_decode_op_embed", (
            table.data_ptr(), 0 if positions_table is None else positions_table.data_ptr(), self.tokens.data_ptr(),
            x.data_ptr(), table.shape[1], table.shape[0], 0 if positions_table is None else positions_table.shape[0])))

    def product(self, inp, w, bias, out, *, norm=None, act=None, residual=None, kv_scatter=None) -> None:
        """out[r] = act(norm(inp[r]) · wᵀ + bias) (+ residual[r]) for the program's rows.  inp float32 or bfloat16
        [rows, K]; w bfloat16 [N, K]; out float32 or bfloat16 [rows, N]; norm: None or (kind, weight, bias, eps) as
        `norm_terms` gives; kv_scatter = (k_cache, v_cache, block_table, k_off, v_off, n_kv_heads, head_dim)."""
        lib = library()
        N, K = w.shape
        in_f32 = inp.dtype == torch.float32
        kind, gamma, beta, eps = norm if norm is not None else (None, None, None, 0.0)
        if w.dtype != torch.bfloat16 or inp.shape[1] != K or out.shape[1] != N:
            raise NotFusable("product operands")
        if not lib.vlrf_decode_program_gemv_takes(self.n_rows, N, K, 1 if in_f32 else 0, NORM_KINDS[kind]):
            raise NotFusable(f"a product of N={N}, K={K} over {self.n_rows} rows is not taken by the decode program")
        for t in (inp, w, out, gamma, beta, bias, residual):
            if t is not None and (not t.is_cuda or not t.is_contiguous()):
                raise NotFusable("operands must be contiguous device tensors")
        for t in (gamma, beta, bias, residual):
            if t is not None and t.dtype != torch.float32:
                raise NotFusable("norm weights, bias and residual are float32")
        kv = (0, 0, 0, 0, 0, 0, 0, 0, 0)
        if kv_scatter is not None:
            kc, vc, table, k_off, v_off, hkv, dh = kv_scatter
            if kc.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
                raise NotFusable("the cache scatter writes bfloat16")
            kv = (kc.data_ptr(), vc.data_ptr(), table.data_ptr(), table.shape[1], k_off, v_off, hkv, dh, kc.shape[2])
            self._keep += [kc, vc, table]
        self._keep += [inp, w, bias, out, gamma, beta, residual]
        self._calls.append(("vlrf_decode_op_gemv", (
            self.n_rows, inp.data_ptr(), 1 if in_f32 else 0, inp.shape[1], NORM_KINDS[kind], ops._ptr(gamma), ops._ptr(beta),
            float(eps), w.data_ptr(), ops._ptr(bias), N, K, ops.ACT[act], out.data_ptr(),
            1 if out.dtype == torch.float32 else 0, out.shape[1], ops._ptr(residual), *kv)))

    def attention(self, qkv, q_off: int, k_cache, v_cache, block_table, out, *, n_heads: int, n_kv_heads: int,
                  head_dim: int, scale: float, window: int = 0) -> None:
        lib = library()
        bt = k_cache.shape[2]
        if qkv.dtype != torch.bfloat16 or k_cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
            raise NotFusable("attention operands must be bfloat16")
        if not lib.vlrf_decode_program_attention_takes(head_dim, bt) or q_off % 8 != 0 or qkv.shape[1] % 8 != 0:
            raise NotFusable(f"attention with head size {head_dim} is not taken by the decode program")
        pairs = self.n_rows * n_heads
        # One CTA a (row, head) while a context is short: parts pay a merge through global memory (three more round
        # trips to L2) that only long contexts earn back.
        n_split = max(1, min(16, ops.sm_count() // pairs, self.max_context // 1024))
        partials = counters = None
        if n_split > 1:
            partials = self.ws.get("program_partials", pairs * n_split, head_dim + 2, torch.float32)
            counters = self.ws.get_zeroed("program_counters", pairs, torch.int32)
        self._keep += [qkv, k_cache, v_cache, block_table, out, partials, counters]
        self._calls.append(("vlrf_decode_op_attention", (
            qkv.data_ptr(), qkv.shape[1], q_off, k_cache.data_ptr(), v_cache.data_ptr(), block_table.data_ptr(),
            block_table.shape[1], out.data_ptr(), out.shape[1], n_heads, n_kv_heads, head_dim, bt, float(scale), int(window),
            n_split, ops._ptr(partials), ops._ptr(counters))))

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

    def profile(self, cta: int = 0, stages: bool = False) -> list:
        """Runs the program once more and returns, for every operation, (its kind, microseconds from its begin to
        the next operation's begin) as CTA `cta` saw it: the operation and the grid barrier after it.  With
        `stages`, a third item: microseconds from the begin to [rows staged, first weights landed, products done,
        results stored, arrived at the barrier] (None where the operation has no such stage)."""
        trace = torch.zeros(len(self._calls) + 1, 8, dtype=torch.int64, device=self.device)
        self._sync[3] = cta
        self.run(trace)
        self._sync[3] = 0
        t = trace.cpu().tolist()
        out = []
        for i, (name, _) in enumerate(self._calls):
            item = (name.replace("vlrf_decode_op_", ""), (t[i + 1][0] - t[i][0]) / 1e3)
            if stages:
                item += ([round((t[i][k] - t[i][0]) / 1e3, 2) if t[i][k] else None for k in range(1, 8)],)
            out.append(item)
        return out
