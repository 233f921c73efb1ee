"""The step function: run the tokens it is given, as one batch, from the cache.

`Engine.step(entries)` takes for each sequence its next tokens and the places among them whose logits
are wanted.  All tokens of all sequences run as one flat batch (prompts of unequal lengths in one step,
or one token each); each token carries its sequence's slot and its position, so no padding exists and
what else is in the batch changes no result.  Only the given tokens are computed: everything earlier
comes from the cache that previous steps left.  The reference has one sequence and a `forward(ids,
use_cache)` that returns the last row (include/model/transformer.hpp:335-424).
"""
from __future__ import annotations

import dataclasses

import numpy as np
import torch

from ..cache import SequenceCache
from ..csrc import KernelError, library
from .capture import capture_into
from ..parts.context import StepContext, Workspace
from .model import DecoderModel

DEVERR_TEXT = {1: "a token id outside the vocabulary", 2: "a position outside the position table",
               4: "a token whose cache block is not mapped", 8: "a bounded wait that gave up"}


@dataclasses.dataclass
class StepEntry:
    slot: int
    tokens: list                 # token ids: a list, or an integer numpy array (which spares the step the conversion)
    want: list = dataclasses.field(default_factory=list)   # indices into `tokens`


class StepError(ValueError):
    """A step that cannot run as asked (checked on the host, before any launch)."""


class Engine:
    def __init__(self, model: DecoderModel, *, max_tokens: int, n_slots: int | None = None):
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device: this framework runs on the GPU only")
        library()  # fail now, loudly, if the kernels cannot be built or loaded
        self.model = model
        self.device = model.device
        self.cache = SequenceCache(model.cache_needs(), max_tokens=max_tokens, max_seq_len=model.max_seq_len,
                                   dtype=model.act_dtype, device=self.device, n_slots=n_slots)
        self.ws = Workspace(self.device)
        self.dev_err = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._meta_cap = 0
        self._meta_views = {}
        self._meta_host = None
        self._meta_dev = None
        self._meta_copied = None   # event: the last copy out of the pinned staging buffer has finished
        self.steps_run = 0
        # Steps of a shape seen before are replayed from a captured CUDA graph: the step's integer tables
        # live at fixed device addresses, so only their contents change from step to step.
        self.capture_repeated_steps = True
        self._graphs: dict = {}        # (tokens, sequences, longest run, wanted rows) -> (graph, logits)
        self._seen: dict = {}
        self._graph_generation = -1
        from ..csrc import ops
        ops._dev_err()             # exists before any capture

    # -- sequences ----------------------------------------------------------------------------
    def start_sequence(self) -> int:
        return self.cache.acquire()

    def end_sequence(self, slot: int) -> None:
        self.cache.release(slot)

    def length(self, slot: int) -> int:
        return self.cache.lengths[slot]

    # -- the step -----------------------------------------------------------------------------
    def _meta(self, n_ints: int):
        if n_ints > self._meta_cap:
            cap = max(1024, 2 * n_ints)
            self._meta_host = torch.empty(cap, dtype=torch.int32, pin_memory=True)
            self._meta_dev = torch.empty(cap, dtype=torch.int32, device=self.device)
            self._meta_cap = cap
            self._meta_views = {}
            self._graphs.clear()       # captured steps point into the old tables
        return self._meta_host, self._meta_dev

    def plan(self, entries: list) -> dict:
        """Check a step on the host and lay out its integer tables.  Raises StepError / CacheError and
        changes nothing if the step cannot run."""
        if not entries:
            raise StepError("a step needs at least one sequence")
        vocab, seen, arrays = self.model.vocab_size, set(), []
        for e in entries:
            if e.slot in seen:
                raise StepError(f"slot {e.slot} appears twice in one step")
            seen.add(e.slot)
            if not self.cache.slots.is_held(e.slot):
                raise StepError(f"slot {e.slot} is not held by a sequence")
            if len(e.tokens) == 0:
                raise StepError(f"slot {e.slot}: a step brings at least one token for each sequence")
            if self.cache.lengths[e.slot] + len(e.tokens) > self.model.max_seq_len:
                raise StepError(f"slot {e.slot}: {self.cache.lengths[e.slot]} + {len(e.tokens)} tokens exceed the "
                                f"{self.model.max_seq_len} positions of the model")
            # (a list is converted once: this is most of a long prompt's host time; an integer array is taken as it is)
            arr = e.tokens if isinstance(e.tokens, np.ndarray) and e.tokens.dtype.kind in "iu" else np.asarray(e.tokens, dtype=np.int64)
            if arr.min() < 0 or arr.max() >= vocab:
                bad = int(arr[(arr < 0) | (arr >= vocab)][0])
                raise StepError(f"slot {e.slot}: token id {bad} lies outside the vocabulary of {vocab}")
            arrays.append(arr)
            for w in e.want:
                if not (0 <= int(w) < len(e.tokens)):
                    raise StepError(f"slot {e.slot}: wanted place {w} is not among its {len(e.tokens)} tokens")
        T = sum(len(e.tokens) for e in entries)
        B = len(entries)
        n_want = sum(len(e.want) for e in entries)
        tokens = np.empty(T, dtype=np.int32)
        tok_slot = np.empty(T, dtype=np.int32)
        tok_pos = np.empty(T, dtype=np.int32)
        seq_slot = np.empty(B, dtype=np.int32)
        seq_start = np.empty(B + 1, dtype=np.int32)
        seq_pos0 = np.empty(B, dtype=np.int32)
        rows = np.empty(n_want, dtype=np.int32)
        at, r = 0, 0
        for i, e in enumerate(entries):
            n, p0 = len(e.tokens), self.cache.lengths[e.slot]
            tokens[at:at + n] = arrays[i]
            tok_slot[at:at + n] = e.slot
            tok_pos[at:at + n] = np.arange(p0, p0 + n, dtype=np.int32)
            seq_slot[i], seq_start[i], seq_pos0[i] = e.slot, at, p0
            for w in e.want:
                rows[r] = at + int(w)
                r += 1
            at += n
        seq_start[B] = T
        return dict(T=T, B=B, n_want=n_want, tokens=tokens, tok_slot=tok_slot, tok_pos=tok_pos,
                    seq_slot=seq_slot, seq_start=seq_start, seq_pos0=seq_pos0, rows=rows,
                    lens=[len(e.tokens) for e in entries], pos0=[int(p) for p in seq_pos0])

    def step(self, entries: list) -> torch.Tensor:
        """Run one step; returns float32 logits [wanted, vocab] on the device, in the order of the
        entries and of each entry's `want`.  The tensor is scratch that the next step overwrites."""
        p = self.plan(entries)
        for e in entries:  # all-or-nothing per sequence; a failure leaves earlier reservations, which are harmless
            self.cache.reserve(e.slot, self.cache.lengths[e.slot] + len(e.tokens))
        self.cache.sync_tables()
        T, B, n_want = p["T"], p["B"], p["n_want"]
        parts = [p["tokens"], p["tok_slot"], p["tok_pos"], p["seq_slot"], p["seq_start"], p["seq_pos0"], p["rows"]]
        n_ints = sum(a.size for a in parts)
        host, dev = self._meta(n_ints)
        if self._meta_copied is not None:
            self._meta_copied.synchronize()   # the staging buffer is free to overwrite
        # views of the tables' places in the staging buffers: the same for every step of the same sizes (making a
        # view costs about 2 us, and a step has nine)
        layout = (id(dev),) + tuple(a.size for a in parts)
        cached = self._meta_views.get(layout)
        if cached is None:
            if len(self._meta_views) > 64:
                self._meta_views.clear()
            views, at = [], 0
            for a in parts:
                views.append(dev[at:at + a.size])
                at += a.size
            cached = (host.numpy(), views, dev[:n_ints], host[:n_ints])
            self._meta_views[layout] = cached
        hnp, views, dev_all, host_all = cached
        at = 0
        for a in parts:
            hnp[at:at + a.size] = a
            at += a.size
        dev_all.copy_(host_all, non_blocking=True)
        if self._meta_copied is None:
            self._meta_copied = torch.cuda.Event()
        self._meta_copied.record()
        ctx = StepContext(
            n_tokens=T, tokens=views[0], tok_slot=views[1], tok_pos=views[2], n_seqs=B, seq_slot=views[3],
            seq_start=views[4], seq_pos0=views[5], max_new=max(p["lens"]),
            max_context=max(a + b for a, b in zip(p["pos0"], p["lens"])), logit_rows=views[6],
            n_logit_rows=n_want, act_dtype=self.model.act_dtype, dev_err=self.dev_err, ws=self.ws,
            host_seq_slots=[e.slot for e in entries], host_seq_lens=p["lens"], host_seq_pos0=p["pos0"])
        logits = self._forward(ctx, (T, B, ctx.max_new, n_want))
        for e in entries:
            self.cache.advance(e.slot, len(e.tokens))
        self.steps_run += 1
        return logits

    def _forward(self, ctx: StepContext, signature) -> torch.Tensor:
        """Run the model on the step, replaying a captured graph when a step of the same shape ran before."""
        if not self.capture_repeated_steps or ctx.max_new == 1 or not self.model.replayable:
            return self.model.forward(ctx, self.cache)     # single-token steps have DecodeSession's graph
        if self._graph_generation != self.ws.generation:
            self._graphs.clear()                           # scratch moved: captured addresses are stale
            self._graph_generation = self.ws.generation
        hit = self._graphs.get(signature)
        if hit is not None:
            hit[0].replay()
            return hit[1]
        n = self._seen.get(signature, 0)
        self._seen[signature] = n + 1
        if n == 0 or len(self._graphs) >= 16:
            logits = self.model.forward(ctx, self.cache)   # first time: plain launches (they size the scratch)
            self._graph_generation = self.ws.generation
            return logits
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with capture_into(graph):
            logits = self.model.forward(ctx, self.cache)
        if self.ws.generation != self._graph_generation:   # the capture itself had to allocate: do not keep it
            self._graph_generation = self.ws.generation
            return self.model.forward(ctx, self.cache)
        self._graphs[signature] = (graph, logits)
        graph.replay()
        return logits

    def check_device_errors(self) -> None:
        """Read the device's error word (synchronises) and raise if a kernel set a bit."""
        from ..csrc import ops
        word = int(self.dev_err.item()) | ops.device_errors()
        if word:
            self.dev_err.zero_()
            what = [txt for bit, txt in DEVERR_TEXT.items() if word & bit]
            raise KernelError("a kernel met " + "; ".join(what) + " and skipped it; results of this step are invalid")
