"""The generation loop: requests of unequal prompts, stop tokens, sequences that end early, and waiting
requests that take the places of those that ended.

The loop decides on the host and computes through a *backend* with six calls (the real one drives
`Engine.step` and the sampling kernels; tests give a scripted one):

    limits() -> (max_tokens, n_slots, block_tokens, max_seq_len)
    open_table(n_rows, requests) -> handle   a table of rows that hold sequences in turn; `requests`: all that
                                             will ever be admitted (their options decide what the table must be able to do)
    admit(handle, row, request)              the free row takes a cache slot and the request's sampling state
    run(handle, rows, tokens) -> list        one step for the listed rows (each a list of tokens to feed: a whole
                                             prompt for a row just admitted, one token for the others) and one
                                             sampled token per row, as host integers
    close_row(handle, row)                   the row's sequence has ended: its slot is given back, the row is free
    close_table(handle)

A request waits until a row is free and the cache can hold what it may come to need; it is admitted at the next
step boundary, its prompt runs in the same step in which the others go on by one token, and from the step after
it decodes with them.  Requests are admitted in their order, so what a request generates never depends on the
others (per-request random streams, see sampling/rng.py).

Differences from the reference's loop (include/model/transformer.hpp:439-547), all deliberate: many
sequences at once; the first new token is sampled from the prompt's last logits instead of feeding the
last prompt token a second time (:447-452, :482); an empty prompt starts from bos_token_id as there
(:450-451); a sequence ends at a stop token (:504-507), after max_new_tokens (:472) or when the
model's positions are used up (:473).
"""
from __future__ import annotations

import dataclasses

from ..sampling.params import SamplingParams


@dataclasses.dataclass
class Request:
    prompt: list
    params: SamplingParams
    index: int = 0          # position in the caller's list; also names the request's random stream


@dataclasses.dataclass
class GenerationResult:
    prompt: list
    new_tokens: list
    finish_reason: str      # "stop" | "length" | "context"

    @property
    def token_ids(self) -> list:          # prompt + new, as the reference returns (:429-434, :453, :494)
        return list(self.prompt) + list(self.new_tokens)

    @property
    def tokens_generated(self) -> int:
        return len(self.new_tokens)

    @property
    def hit_eos(self) -> bool:
        return self.finish_reason == "stop"


class GenerationError(ValueError):
    pass


def _round_up(n: int, unit: int) -> int:
    return (n + unit - 1) // unit * unit


def tokens_needed(req: Request, block_tokens: int, max_seq_len: int) -> int:
    """Cache tokens a request may come to hold: prompt plus all it may generate but the last token,
    which is never fed back; in whole blocks."""
    most = min(len(req.prompt) + max(req.params.max_new_tokens - 1, 0), max_seq_len)
    return _round_up(max(most, 1), block_tokens)


def plan_batches(requests: list, max_tokens: int, n_slots: int, block_tokens: int, max_seq_len: int) -> list:
    """Cut requests, in their order, into batches that fit the cache: at most n_slots sequences, and their
    worst-case token counts (in whole blocks) within max_tokens.  (`generate` admits request by request instead;
    this is for callers that want whole batches, like a replay of a fixed schedule.)"""
    batches, cur, used = [], [], 0
    for req in requests:
        if len(req.prompt) > max_seq_len:
            raise GenerationError(f"request {req.index}: a prompt of {len(req.prompt)} tokens exceeds the "
                                  f"{max_seq_len} positions of the model")
        need = tokens_needed(req, block_tokens, max_seq_len)
        if need > max_tokens:
            raise GenerationError(f"request {req.index} may hold {need} tokens; the cache holds {max_tokens}")
        if cur and (len(cur) >= n_slots or used + need > max_tokens):
            batches.append(cur)
            cur, used = [], 0
        cur.append(req)
        used += need
    if cur:
        batches.append(cur)
    return batches


def finish_reason(req: Request, new_tokens: list, stop_ids, max_seq_len: int):
    """Why the sequence ends after its latest token, or None if it goes on."""
    if new_tokens and new_tokens[-1] in stop_ids:
        return "stop"
    if len(new_tokens) >= req.params.max_new_tokens:
        return "length"
    if len(req.prompt) + len(new_tokens) >= max_seq_len:
        return "context"
    return None


def generate(backend, prompts: list, params, *, bos_token_id=None, eos_token_id=None, on_token=None) -> list:
    """Generate for every prompt; `params` is one SamplingParams for all or a list, one per prompt."""
    max_tokens, n_slots, block_tokens, max_seq_len = backend.limits()
    plist = params if isinstance(params, (list, tuple)) else [params] * len(prompts)
    if len(plist) != len(prompts):
        raise GenerationError("one SamplingParams per prompt, or one for all")
    requests = []
    for i, (prompt, p) in enumerate(zip(prompts, plist)):
        p.validate()
        prompt = [int(t) for t in prompt]
        if not prompt:
            if bos_token_id is None:
                raise GenerationError(f"request {i}: an empty prompt needs the model's bos_token_id")
            prompt = [int(bos_token_id)]
        requests.append(Request(prompt, p, i))
    default_stop = () if eos_token_id is None else (int(eos_token_id),)
    results = [None] * len(requests)
    waiting = []
    for req in requests:
        if len(req.prompt) > max_seq_len:
            raise GenerationError(f"request {req.index}: a prompt of {len(req.prompt)} tokens exceeds the "
                                  f"{max_seq_len} positions of the model")
        need = tokens_needed(req, block_tokens, max_seq_len)
        if need > max_tokens:
            raise GenerationError(f"request {req.index} may hold {need} tokens; the cache holds {max_tokens}")
        if req.params.max_new_tokens == 0:
            results[req.index] = GenerationResult(list(req.prompt), [], "length")
        elif len(req.prompt) >= max_seq_len:
            results[req.index] = GenerationResult(list(req.prompt), [], "context")
        else:
            waiting.append(req)
    if not waiting:
        return results
    n_rows = min(n_slots, len(waiting))
    handle = backend.open_table(n_rows, list(waiting))
    free_rows = list(range(n_rows))
    live: dict = {}                 # row -> [request, new tokens, tokens to feed next, stop ids, tokens it may hold]
    held = 0
    try:
        while waiting or live:
            # waiting requests, in their order, take free rows while the cache can hold what they may come to need
            while waiting and free_rows:
                need = tokens_needed(waiting[0], block_tokens, max_seq_len)
                if held + need > max_tokens:
                    break
                req = waiting.pop(0)
                row = free_rows.pop(0)
                backend.admit(handle, row, req)
                stops = req.params.stop_token_ids if req.params.stop_token_ids is not None else default_stop
                live[row] = [req, [], list(req.prompt), stops, need]
                held += need
            rows = sorted(live)
            sampled = backend.run(handle, rows, [live[r][2] for r in rows])
            for row, tok in zip(rows, sampled):
                req, new, _, stops, need = live[row]
                tok = int(tok)
                new.append(tok)
                reason = finish_reason(req, new, stops, max_seq_len)
                if on_token is not None and reason is None and on_token(req.index, tok) is False:
                    reason = "stop"
                if reason is None:
                    live[row][2] = [tok]
                else:
                    results[req.index] = GenerationResult(list(req.prompt), new, reason)
                    del live[row]
                    held -= need
                    backend.close_row(handle, row)
                    free_rows.append(row)
                    free_rows.sort()
    except BaseException:
        for row in list(live):
            try:
                backend.close_row(handle, row)
            except Exception:  # noqa: BLE001 - the first error is the one to report
                pass
        raise
    finally:
        backend.close_table(handle)
    return results
