"""`DecoderModel` as data, with stand-in parts (CPU): the schedule's rules, what each entry keeps in the cache,
whether steps may be replayed, and the bytes of the weights."""
import types

import pytest
import torch

from vlrf_b200.cache.sequence_cache import KVNeed, StateNeed
from vlrf_b200.engine.model import BuildOptions, DecoderModel, LayerCall


class Layer:
    def __init__(self, need, **parts):
        self._need = need
        for k, v in parts.items():
            setattr(self, k, v)

    def cache_need(self):
        return self._need


def model(layers, schedule):
    emb = types.SimpleNamespace(width=8, table=torch.zeros(10, 8))
    head = types.SimpleNamespace(vocab_size=10, weight=emb.table)          # tied: the same storage
    return DecoderModel(config=None, embedding=emb, layers=layers, schedule=schedule, final_norm=types.SimpleNamespace(),
                        head=head, options=BuildOptions(torch.float32, torch.device("cpu")), max_seq_len=32)


FULL, WINDOW, STATE = KVNeed(2, 16), KVNeed(2, 16, "window", 8), StateNeed((4,))


def test_a_layer_may_run_twice_and_read_another_entrys_cache():
    m = model([Layer(FULL), Layer(WINDOW), Layer(STATE), Layer(None)],
              [0, 1, LayerCall(0), LayerCall(0, reads_cache_of=0), 2, 3, LayerCall(1, reads_cache_of=1)])
    assert [c.layer for c in m.schedule] == [0, 1, 0, 0, 2, 3, 1]
    # one cache entry per schedule entry that keeps something of its own; readers and stateless layers keep nothing
    assert m.cache_needs() == [FULL, WINDOW, FULL, None, STATE, None, None]
    assert m.width == 8 and m.vocab_size == 10 and m.max_seq_len == 32


@pytest.mark.parametrize("schedule,match", [
    ([0, 5], "names layer 5"),
    ([LayerCall(0, reads_cache_of=0)], "earlier entry"),                               # itself
    ([0, LayerCall(0, reads_cache_of=2), 0], "earlier entry"),                         # a later one
    ([0, LayerCall(0, reads_cache_of=0), LayerCall(0, reads_cache_of=1)], "owns one"),  # a reader owns none
    ([0, LayerCall(1, reads_cache_of=0)], "shape differs"),                            # a window cannot read a full cache
])
def test_schedules_that_cannot_run_are_refused(schedule, match):
    with pytest.raises(ValueError, match=match):
        model([Layer(FULL), Layer(WINDOW)], schedule)


def test_a_part_that_asks_the_device_something_makes_steps_launch_plainly():
    plain_ff = types.SimpleNamespace()
    routed_ff = types.SimpleNamespace(replayable=False)
    assert model([Layer(FULL, feed_forward=plain_ff)], [0]).replayable
    assert not model([Layer(FULL, feed_forward=plain_ff), Layer(FULL, feed_forward=routed_ff)], [0, 1]).replayable
    layer = Layer(FULL)
    layer.replayable = False
    assert not model([layer], [0]).replayable


def test_weight_bytes_count_shared_storage_once():
    w = torch.zeros(4, 8, dtype=torch.bfloat16)
    layers = [Layer(FULL, mixer=types.SimpleNamespace(w=w, b=torch.zeros(4)), norms=[types.SimpleNamespace(g=torch.zeros(8))]),
              Layer(FULL, mixer=types.SimpleNamespace(w=w, b=torch.zeros(4)))]          # the same matrix in two layers
    m = model(layers, [0, 1])
    assert m.weight_bytes() == 10 * 8 * 4 + 4 * 8 * 2 + 4 * 4 + 8 * 4 + 4 * 4            # table (tied head), w once, b, g, b
