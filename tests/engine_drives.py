"""Ways of driving the step function over the same requests, shared by the GPU tests.

Each drive returns, for every request, float32 logits at ALL its positions [len, vocab], collected from
however many steps the drive cut the request into."""
import torch

from vlrf_b200.engine.step import StepEntry


def poison(engine):
    """Fill every key/value pool with NaN: whatever a kernel reads without having written it shows."""
    for g in engine.cache._groups:
        if hasattr(g, "k"):
            g.k.fill_(float("nan"))
            g.v.fill_(float("nan"))


def drive_whole(engine, requests):
    """Each request alone and whole, in one step."""
    out = []
    for ids in requests:
        slot = engine.start_sequence()
        out.append(engine.step([StepEntry(slot, ids, list(range(len(ids))))]).float().cpu().clone())
        engine.end_sequence(slot)
    engine.check_device_errors()
    return out


def drive_tail_one_by_one(engine, requests, tail=32):
    """The prefix whole, then the last `tail` tokens one by one."""
    out = []
    for ids in requests:
        slot = engine.start_sequence()
        cut = max(1, len(ids) - tail)
        rows = [engine.step([StepEntry(slot, ids[:cut], list(range(cut)))]).float().cpu().clone()]
        for t in ids[cut:]:
            rows.append(engine.step([StepEntry(slot, [t], [0])]).float().cpu().clone())
        out.append(torch.cat(rows))
        engine.end_sequence(slot)
    engine.check_device_errors()
    return out


def drive_batches(engine, requests, batch_size, prompt_lens):
    """Batches of unequal lengths, one batch after another: the first prompt_lens[i] tokens of every
    request of a batch in one step, then one token each per step; a request leaves the batch when its
    tokens are used up, and its slot is given back at once."""
    out = [None] * len(requests)
    for b0 in range(0, len(requests), batch_size):
        idx = list(range(b0, min(len(requests), b0 + batch_size)))
        slots = {i: engine.start_sequence() for i in idx}
        got = {i: [] for i in idx}
        fed = {i: min(prompt_lens[i], len(requests[i])) for i in idx}
        logits = engine.step([StepEntry(slots[i], requests[i][:fed[i]], list(range(fed[i]))) for i in idx]).float().cpu()
        at = 0
        for i in idx:
            got[i].append(logits[at:at + fed[i]].clone())
            at += fed[i]
        live = list(idx)
        while True:
            for i in [i for i in live if fed[i] >= len(requests[i])]:
                engine.end_sequence(slots[i])
                live.remove(i)
            if not live:
                break
            logits = engine.step([StepEntry(slots[i], [requests[i][fed[i]]], [0]) for i in live]).float().cpu()
            for r, i in enumerate(live):
                got[i].append(logits[r:r + 1].clone())
                fed[i] += 1
        for i in idx:
            out[i] = torch.cat(got[i])
    engine.check_device_errors()
    engine.cache.check()
    return out
