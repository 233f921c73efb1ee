"""The time stamps inside the decode kernels: a build of its own (VLRF_B200_KERNEL_TRACE=1) leaves a record per launch of
a replayed step; the ordinary build has none and says so."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent

SCRIPT = r"""
import sys, tempfile
import torch
from vlrf_b200 import log
from vlrf_b200.engine import Engine, StepEntry, load_model
from vlrf_b200.engine.decode import DecodeSession
from vlrf_b200.weights import write_random_model
from vlrf_b200.config import load_preset
import vlrf_b200.models
cfg = dict(load_preset("gpt2"), n_layer=2, vocab_size=1000, bos_token_id=0, eos_token_id=0)   # head size 64: the tensor-core kernels
with tempfile.TemporaryDirectory() as tmp:
    model = load_model(write_random_model(cfg, 5, tmp + "/m"), "bfloat16")
    eng = Engine(model, max_tokens=1024, n_slots=4)
    slots = [eng.start_sequence() for _ in range(4)]
    eng.step([StepEntry(s, list(range(3, 3 + 40 + 7 * i)), [39 + 7 * i]) for i, s in enumerate(slots)])
    sess = DecodeSession(eng, slots, use_graph=True)
    sess.reserve_ahead(8)
    sess.set_tokens([5, 6, 7, 8])
    for _ in range(4):
        sess.step()
    torch.cuda.synchronize()
    records = log.kernel_timeline()
    kinds = [r["kind"] for r in records]
    assert kinds.count(1) >= 8 and kinds.count(2) >= 2, kinds           # products and attention of the last steps
    last = records[-1]
    assert last["ctas"] > 0 and last["first"][0] is not None
    # within a launch the stations follow one another
    for r in records:
        seen = [v for v in r["last"] if v is not None]
        assert seen == sorted(seen) or r["kind"] != 1, r
    print(log.timeline_table(records, last=5))
    assert log.kernel_timeline() == []                                  # reading cleared the buffer
print("TRACE_OK")
"""


@pytest.mark.gpu
def test_a_build_with_stamps_records_the_kernels_of_a_replayed_step(tmp_path):
    env = dict(os.environ, VLRF_B200_KERNEL_TRACE="1", VLRF_B200_BUILD_DIR=str(tmp_path / "build"), PYTHONPATH=str(ROOT))
    (tmp_path / "build").mkdir()
    proc = subprocess.run([sys.executable, "-c", SCRIPT], env=env, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0 and "TRACE_OK" in proc.stdout, proc.stdout[-2000:] + proc.stderr[-3000:]


@pytest.mark.gpu
def test_the_ordinary_build_has_no_stamps_and_says_so():
    from vlrf_b200 import log
    from vlrf_b200.csrc import KernelError
    if os.environ.get("VLRF_B200_KERNEL_TRACE", "0") not in ("", "0"):
        pytest.skip("this run uses the build with stamps")
    with pytest.raises(KernelError, match="VLRF_B200_KERNEL_TRACE"):
        log.kernel_timeline()
