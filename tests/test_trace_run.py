"""bin/trace_run as a user runs it: a subprocess, JSON lines in, <step>.f32 files out."""
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_gpt2 as plain
from conftest import ROOT, TOL_BF16, TOL_F32, random_ids

pytestmark = pytest.mark.gpu


class Replay:
    def __init__(self, model_dir, dtype, out_dir, max_tokens):
        env = dict(os.environ)
        self.out_dir = Path(out_dir)
        self.p = subprocess.Popen([str(ROOT / "bin" / "trace_run"), "--model", str(model_dir), "--dtype", dtype, "--out",
                                   str(out_dir), "--max-tokens", str(max_tokens)], stdin=subprocess.PIPE,
                                  stdout=subprocess.PIPE, text=True, env=env)
        self.step = 0

    def send(self, entries, end=()):
        msg = {"step": self.step, "entries": entries, "end": list(end)}
        self.p.stdin.write(json.dumps(msg) + "\n")
        self.p.stdin.flush()
        line = self.p.stdout.readline().strip()
        assert line == f"done {self.step}", f"trace_run said {line!r} (exit {self.p.poll()})"
        f = self.out_dir / f"{self.step}.f32"
        self.step += 1
        return f

    def close(self):
        self.p.stdin.close()
        assert self.p.wait(timeout=120) == 0


def read(f, vocab):
    return torch.from_numpy(np.fromfile(f, dtype="<f4").reshape(-1, vocab).copy())


@pytest.mark.parametrize("dtype,tol", [("float32", TOL_F32), ("bfloat16", TOL_BF16)])
def test_replay_whole_tail_and_batches(model_dirs, plain_models, tmp_path, dtype, tol):
    cfg, w = plain_models["tiny_b"]
    V = cfg["vocab_size"]
    lens = [25, 33, 64, 124]
    reqs = {f"r{i}": random_ids(V, n, 20 + i) for i, n in enumerate(lens)}
    truth = {k: plain.logits_all_positions(cfg, w, ids) for k, ids in reqs.items()}

    def close_enough(got, want, what):
        err = float((got.double() - want).abs().max() / want.abs().max())
        assert got.shape == want.shape and err < tol, (what, err)

    rp = Replay(model_dirs["tiny_b"], dtype, tmp_path / "out", 64 * 5)
    # 1. each request alone and whole; only some places wanted
    for k, ids in reqs.items():
        want = [0, len(ids) // 2, len(ids) - 1]
        f = rp.send([{"id": k, "tokens": ids, "want": want}], end=[k])
        close_enough(read(f, V), truth[k][want], f"whole {k}")
    # 2. the prefix whole (nothing wanted: no file), then the last 32 tokens one by one
    k, ids = "r3", reqs["r3"]
    f = rp.send([{"id": k, "tokens": ids[:-32], "want": []}])
    assert not f.exists()
    for j in range(len(ids) - 32, len(ids)):
        f = rp.send([{"id": k, "tokens": [ids[j]], "want": [0]}], end=[k] if j == len(ids) - 1 else [])
        close_enough(read(f, V), truth[k][j:j + 1], f"tail position {j}")
    # 3. a batch of unequal lengths; shorter requests end earlier; then the same ids again on reused slots
    for round_ in range(2):
        names = list(reqs)
        prompt = {k: max(1, len(reqs[k]) - 24) for k in names}
        f = rp.send([{"id": k, "tokens": reqs[k][:prompt[k]], "want": [prompt[k] - 1]} for k in names])
        got = read(f, V)
        for r, k in enumerate(names):
            close_enough(got[r:r + 1], truth[k][prompt[k] - 1:prompt[k]], f"batch prompt {k}")
        fed = dict(prompt)
        live = list(names)
        # make the lengths end at different steps: r0 stops 10 tokens early, r1 5 tokens early
        stop_at = {"r0": len(reqs["r0"]) - 10, "r1": len(reqs["r1"]) - 5, "r2": len(reqs["r2"]), "r3": len(reqs["r3"])}
        while live:
            ending = [k for k in live if fed[k] + 1 >= stop_at[k]]
            f = rp.send([{"id": k, "tokens": [reqs[k][fed[k]]], "want": [0]} for k in live], end=ending)
            got = read(f, V)
            for r, k in enumerate(live):
                close_enough(got[r:r + 1], truth[k][fed[k]:fed[k] + 1], f"batch decode {k} at {fed[k]} (round {round_})")
                fed[k] += 1
            live = [k for k in live if k not in ending]
    rp.close()


@pytest.mark.parametrize("dtype,tol", [("float32", TOL_F32), ("bfloat16", TOL_BF16)])
def test_replay_of_prompts_that_arrive_in_portions(model_dirs, plain_models, tmp_path, dtype, tol):
    """40 tokens of a request, then 30 more in a step that also starts another request, then single tokens: the
    replay program takes such a schedule, and the logits are those of the whole sequences."""
    cfg, w = plain_models["tiny_c"]
    V = cfg["vocab_size"]
    a, b = random_ids(V, 75, 31), random_ids(V, 20, 32)
    ta, tb = plain.logits_all_positions(cfg, w, a), plain.logits_all_positions(cfg, w, b)

    def close_enough(got, want, what):
        err = float((got.double() - want).abs().max() / want.abs().max())
        assert got.shape == want.shape and err < tol, (what, err)

    rp = Replay(model_dirs["tiny_c"], dtype, tmp_path / "out", 64 * 3)
    f = rp.send([{"id": "a", "tokens": a[:40], "want": [0, 39]}])
    close_enough(read(f, V), ta[[0, 39]], "first portion")
    f = rp.send([{"id": "a", "tokens": a[40:70], "want": [0, 29]}, {"id": "b", "tokens": b[:15], "want": [14]}])
    got = read(f, V)
    close_enough(got[:2], ta[[40, 69]], "second portion")
    close_enough(got[2:], tb[[14]], "a new request beside it")
    for j in range(5):
        f = rp.send([{"id": "a", "tokens": [a[70 + j]], "want": [0]}, {"id": "b", "tokens": [b[15 + j]], "want": [0]}],
                    end=["a", "b"] if j == 4 else [])
        got = read(f, V)
        close_enough(got[:1], ta[[70 + j]], f"a at {70 + j}")
        close_enough(got[1:], tb[[15 + j]], f"b at {15 + j}")
    rp.close()
