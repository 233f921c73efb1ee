"""Host-side helpers of a step that need no GPU: the named scratch of a step and the capture guard."""
import gc

import pytest
import torch

from vlrf_b200.parts.context import Workspace


def test_workspace_hands_out_the_same_view_until_the_buffer_moves():
    ws = Workspace("cpu")
    a = ws.get("h", 4, 8, torch.float32)
    assert a.shape == (4, 8) and ws.generation == 1
    assert ws.get("h", 4, 8, torch.float32) is a                     # kept: making a view costs as much as a check
    b = ws.get("h", 2, 8, torch.float32)                             # smaller: the same storage, another view
    assert b.data_ptr() == a.data_ptr() and ws.generation == 1
    c = ws.get("h", 16, 8, torch.float32)                            # larger: the buffer grows, old views are dropped
    assert ws.generation == 2 and c.shape == (16, 8)
    again = ws.get("h", 4, 8, torch.float32)
    assert again is not a and again.data_ptr() == c.data_ptr()
    assert ws.get("h", 4, 8, torch.bfloat16).dtype == torch.bfloat16 and ws.generation == 3   # another dtype: a new buffer
    other = ws.get("u", 4, 8, torch.float32)
    assert other.data_ptr() != ws.get("h", 4, 8, torch.bfloat16).data_ptr()


def test_a_frozen_workspace_refuses_to_grow_but_serves_what_fits():
    ws = Workspace("cpu")
    ws.get("h", 4, 8, torch.float32)
    z = ws.get_zeroed("counters", 10, torch.int32)
    assert int(z.abs().sum()) == 0
    ws.frozen = True
    assert ws.get("h", 2, 16, torch.float32).shape == (2, 16)
    assert ws.get_zeroed("counters", 5, torch.int32).numel() == 5
    with pytest.raises(RuntimeError, match="would have to grow"):
        ws.get("h", 5, 8, torch.float32)
    with pytest.raises(RuntimeError, match="would have to grow"):
        ws.get("new", 1, 1, torch.float32)
    with pytest.raises(RuntimeError, match="would have to grow"):
        ws.get_zeroed("counters", 11, torch.int32)
    assert ws.bytes() == 4 * 8 * 4 + 10 * 4


def test_the_view_table_stays_bounded():
    ws = Workspace("cpu")
    ws.get("h", 1, 4096, torch.float32)
    for rows in range(1, 3000):
        ws.get("h", 1, rows, torch.float32)
    assert len(ws._views) <= 1025 and ws.generation == 1


def test_captures_run_with_the_garbage_collector_held_off(monkeypatch):
    """`capture_into` wraps torch's capture; a stand-in for it shows what the guard does around it."""
    import contextlib

    from vlrf_b200.engine import capture
    seen = {}

    @contextlib.contextmanager
    def fake_graph(g):
        seen["enabled_at_entry"] = gc.isenabled()
        yield
        seen["enabled_at_exit"] = gc.isenabled()

    monkeypatch.setattr(capture.torch.cuda, "graph", fake_graph)
    assert gc.isenabled()
    with capture.capture_into(object()):
        assert not gc.isenabled()
    assert gc.isenabled() and seen == {"enabled_at_entry": False, "enabled_at_exit": False}
    with pytest.raises(ValueError):                                   # an error inside a capture puts the collector back too
        with capture.capture_into(object()):
            raise ValueError("boom")
    assert gc.isenabled()
    gc.disable()                                                      # … and leaves it off for a caller who had it off
    try:
        with capture.capture_into(object()):
            pass
        assert not gc.isenabled()
    finally:
        gc.enable()
