#!/usr/bin/env python3
"""Makes tests/golden/*.npz: logits of VLRF-org/VLRF's own CPU model code on tiny random GPT-2 models,
next to the logits of the plain implementation (tests/plain_gpt2.py) on the same weights.

Run once, by hand, where the reference sources are mounted:

    python tests/golden/make_golden.py /path/to/VLRF

It compiles tests/golden/ref_logits.cpp against the reference's include folders (g++, CPU only), draws
weights from a fixed seed in the Hugging Face layout, rewrites them the way the reference's converter
does (tools/converter/convert_gpt2.py:98-139: transpose Conv1D, split c_attn in thirds, rename), runs
the reference on a few prefixes and on a prefix-then-one-by-one pass, and stores the reference's logits.
tests/test_plain.py draws the same weights again and compares the plain implementation with the stored
logits, so the comparison is repeated on every test run without the reference being present.

Cases: tiny A as it is; tiny B with the tanh GELU, because the reference has no erf GELU
(include/model/ops.hpp:390-403), and with the per-layer 1/(layer+1) scale set through the reference's
public attention_multiplier (include/model/attention.hpp:53,373-374).  The exact-erf GELU therefore rests
on its formula alone.
"""
import struct
import subprocess
import sys
import tempfile
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).parent
sys.path.insert(0, str(HERE.parent))
import plain_gpt2 as plain  # noqa: E402

CASES = {
    "tiny_a": dict(cfg=dict(n_layer=2, n_embd=64, n_head=4, n_inner=256, vocab_size=512, n_positions=128,
                            layer_norm_epsilon=1e-5, activation_function="gelu_new",
                            scale_attn_by_inverse_layer_idx=False, tie_word_embeddings=True),
                   seed=11, n_ids=31, prefixes=[1, 5, 17, 31]),
    "tiny_b_tanh": dict(cfg=dict(n_layer=3, n_embd=96, n_head=3, n_inner=320, vocab_size=1000, n_positions=256,
                                 layer_norm_epsilon=1e-6, activation_function="gelu_new",
                                 scale_attn_by_inverse_layer_idx=True, tie_word_embeddings=True),
                        seed=12, n_ids=100, prefixes=[1, 9, 40, 100]),
}


def draw_weights(cfg, seed):
    """HF-layout float32 weights from numpy's RandomState(seed); every tensor non-trivial."""
    rs = np.random.RandomState(seed)
    d, f, L = cfg["n_embd"], cfg["n_inner"], cfg["n_layer"]
    w = {}

    def n(shape, std, mean=0.0):
        return torch.from_numpy((mean + std * rs.standard_normal(shape)).astype(np.float32))

    w["wte.weight"] = n((cfg["vocab_size"], d), 0.02)
    w["wpe.weight"] = n((cfg["n_positions"], d), 0.02)
    for i in range(L):
        p = f"h.{i}."
        w[p + "ln_1.weight"], w[p + "ln_1.bias"] = n((d,), 0.02, 1.0), n((d,), 0.02)
        w[p + "attn.c_attn.weight"], w[p + "attn.c_attn.bias"] = n((d, 3 * d), 0.02), n((3 * d,), 0.01)
        w[p + "attn.c_proj.weight"], w[p + "attn.c_proj.bias"] = n((d, d), 0.02), n((d,), 0.01)
        w[p + "ln_2.weight"], w[p + "ln_2.bias"] = n((d,), 0.02, 1.0), n((d,), 0.02)
        w[p + "mlp.c_fc.weight"], w[p + "mlp.c_fc.bias"] = n((d, f), 0.02), n((f,), 0.01)
        w[p + "mlp.c_proj.weight"], w[p + "mlp.c_proj.bias"] = n((f, d), 0.02), n((d,), 0.01)
    w["ln_f.weight"], w["ln_f.bias"] = n((d,), 0.02, 1.0), n((d,), 0.02)
    return w


def draw_ids(cfg, seed, n_ids):
    return np.random.RandomState(seed + 1000).randint(0, cfg["vocab_size"], size=n_ids).tolist()


def to_reference_names(cfg, w):
    """convert_gpt2.py:98-139."""
    d = cfg["n_embd"]
    out = {"embed.weight": w["wte.weight"], "pos_embed.weight": w["wpe.weight"],
           "ln_final.weight": w["ln_f.weight"], "ln_final.bias": w["ln_f.bias"]}
    for i in range(cfg["n_layer"]):
        s, t = f"h.{i}.", f"layers.{i}."
        ca, cb = w[s + "attn.c_attn.weight"], w[s + "attn.c_attn.bias"]
        for j, nm in enumerate("qkv"):
            out[t + f"attn.{nm}_proj.weight"] = ca[:, j * d:(j + 1) * d].t().contiguous()
            out[t + f"attn.{nm}_proj.bias"] = cb[j * d:(j + 1) * d].contiguous()
        out[t + "attn.o_proj.weight"] = w[s + "attn.c_proj.weight"].t().contiguous()
        out[t + "attn.o_proj.bias"] = w[s + "attn.c_proj.bias"]
        out[t + "ffn.fc1.weight"] = w[s + "mlp.c_fc.weight"].t().contiguous()
        out[t + "ffn.fc1.bias"] = w[s + "mlp.c_fc.bias"]
        out[t + "ffn.fc2.weight"] = w[s + "mlp.c_proj.weight"].t().contiguous()
        out[t + "ffn.fc2.bias"] = w[s + "mlp.c_proj.bias"]
        for k in ("1", "2"):
            out[t + f"ln{k}.weight"] = w[s + f"ln_{k}.weight"]
            out[t + f"ln{k}.bias"] = w[s + f"ln_{k}.bias"]
    return out


def write_bin(path, tensors):
    with open(path, "wb") as f:
        f.write(struct.pack("<i", len(tensors)))
        for name, t in tensors.items():
            nb = name.encode()
            f.write(struct.pack("<i", len(nb)) + nb)
            f.write(struct.pack("<i", t.dim()))
            f.write(struct.pack(f"<{t.dim()}i", *t.shape))
            f.write(t.contiguous().numpy().astype("<f4").tobytes())


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py /path/to/VLRF")
    ref = Path(sys.argv[1])
    inc = ref / "include"
    with tempfile.TemporaryDirectory() as tmp:
        tmp = Path(tmp)
        exe = tmp / "ref_logits"
        cmd = ["g++", "-std=c++17", "-O2", "-mavx2", "-mfma", f"-I{inc}", f"-I{inc / 'model'}", f"-I{inc / 'backend'}",
               f"-I{inc / 'api'}", f"-I{inc / 'agent'}", str(HERE / "ref_logits.cpp"), "-o", str(exe), "-lpthread"]
        subprocess.run(cmd, check=True)
        for name, case in CASES.items():
            cfg, seed = case["cfg"], case["seed"]
            w = draw_weights(cfg, seed)
            ids = draw_ids(cfg, seed, case["n_ids"])
            write_bin(tmp / "w.bin", to_reference_names(cfg, w))
            args = [str(exe), str(tmp / "w.bin"), cfg["vocab_size"], cfg["n_embd"], cfg["n_inner"], cfg["n_head"],
                    cfg["n_layer"], cfg["n_positions"], repr(cfg["layer_norm_epsilon"]),
                    int(cfg["scale_attn_by_inverse_layer_idx"]), str(tmp / "o.bin"), len(ids), *ids,
                    len(case["prefixes"]), *case["prefixes"]]
            subprocess.run([str(a) for a in args], check=True)
            got = np.fromfile(tmp / "o.bin", dtype="<f4").reshape(len(case["prefixes"]) + 1, cfg["vocab_size"])
            w64 = {k: v.double() for k, v in w.items()}
            full = plain.logits_all_positions(cfg, w64, ids).numpy()
            mine = np.stack([full[p - 1] for p in case["prefixes"]] + [full[-1]])
            err = np.abs(got - mine).max()
            scale = np.abs(mine).max()
            print(f"{name}: reference vs plain max abs diff {err:.3e} (logit scale {scale:.3f})")
            np.savez_compressed(HERE / f"{name}.npz", reference_logits=got.astype(np.float32),
                                prefixes=np.array(case["prefixes"]), seed=seed, n_ids=case["n_ids"])


if __name__ == "__main__":
    main()
