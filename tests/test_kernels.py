"""Each kernel alone against its plain reference, at sizes other than the engine tests use."""
import math

import numpy as np
import pytest
import torch

import plain_gpt2 as plain
from conftest import rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def g(seed):
    return torch.Generator().manual_seed(seed)


def randn(*shape, seed=0, dtype=torch.float32, scale=1.0):
    return (torch.randn(*shape, generator=g(seed)) * scale).to(dtype)


def err_word():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("d,V,P", [(80, 300, 77), (1600, 1000, 50)])
def test_embed(dtype, d, V, P):
    from vlrf_b200.csrc import ops
    wte, wpe = randn(V, d, seed=1, dtype=dtype), randn(P, d, seed=2, dtype=dtype)
    tok = torch.randint(0, V, (45,), generator=g(3), dtype=torch.int32)
    pos = torch.randint(0, P, (45,), generator=g(4), dtype=torch.int32)
    out = torch.full((45, d), float("nan"), device=DEV)
    e = err_word()
    ops.embed(wte.to(DEV), wpe.to(DEV), tok.to(DEV), pos.to(DEV), out, e)
    want = plain.embed_tokens(wte.double(), tok.tolist()) + wpe.double()[pos.long()]
    assert rel_err(out.cpu(), want) < 1e-6 and int(e.item()) == 0
    ops.embed(wte.to(DEV), None, tok.to(DEV), None, out, e)
    assert torch.equal(out.cpu(), wte.float()[tok.long()])
    # an id outside the table is clamped and reported, never read out of bounds
    bad = tok.clone(); bad[7] = V + 5
    ops.embed(wte.to(DEV), wpe.to(DEV), bad.to(DEV), pos.to(DEV), out, e)
    assert int(e.item()) == 1


@pytest.mark.parametrize("out_dtype,tol", [(torch.float32, 2e-6), (torch.bfloat16, 5e-3)])
@pytest.mark.parametrize("d,eps", [(80, 1e-3), (1000, 1e-5), (1600, 1e-6), (16, 1e-5)])
def test_layernorm(out_dtype, tol, d, eps):
    from vlrf_b200.csrc import ops
    x = randn(33, d, seed=5) * 3 + 1.5
    gamma, beta = randn(d, seed=6) * 0.5 + 1, randn(d, seed=7)
    want = plain.layer_norm(x.double(), gamma.double(), beta.double(), eps)
    out = torch.empty(33, d, dtype=out_dtype, device=DEV)
    ops.layernorm(x.to(DEV), gamma.to(DEV), beta.to(DEV), eps, out)
    assert rel_err(out.float().cpu(), want) < tol
    rows = torch.tensor([32, 0, 5, 5], dtype=torch.int32)
    out2 = torch.empty(4, d, dtype=out_dtype, device=DEV)
    ops.layernorm(x.to(DEV), gamma.to(DEV), beta.to(DEV), eps, out2, rows.to(DEV))
    assert rel_err(out2.float().cpu(), want[rows.long()]) < tol


def test_layernorm_small_variance_uses_eps():
    from vlrf_b200.csrc import ops
    x = torch.full((2, 64), 3.0) + randn(2, 64, seed=8) * 1e-4
    gamma, beta = torch.ones(64), torch.zeros(64)
    for eps in (1e-5, 1e-6):
        out = torch.empty(2, 64, device=DEV)
        ops.layernorm(x.to(DEV), gamma.to(DEV), beta.to(DEV), eps, out)
        assert rel_err(out.cpu(), plain.layer_norm(x.double(), gamma.double(), beta.double(), eps)) < 1e-3


# ------------------------------------------------------------------------------------------------
GEMM_SHAPES = [(1, 53, 19), (37, 53, 19), (64, 64, 16), (130, 200, 72), (3, 1000, 96), (257, 96, 320),
               # few rows and K a multiple of 32: the weight-streaming kernel of the decode step
               (8, 2304, 768), (64, 200, 96), (17, 50, 64), (33, 1000, 320), (1, 768, 3072), (9, 17, 32),
               # many rows and K a multiple of 8: the tcgen05 kernel (tails in M, N and K)
               # few rows, very many columns: the tcgen05 kernel with the operands' roles exchanged
               (1, 16500, 64), (8, 20000, 96), (17, 16385, 128), (40, 16400, 72), (64, 17000, 64),
               (65, 64, 64), (128, 128, 128), (300, 768, 768), (1000, 200, 1600), (129, 1000, 72), (2048, 320, 96)]


def f32_sum_tol(K):
    """What float32 accumulation of K products may lose against float64, relative to the largest result:
    rounding errors of 2^-24 each add up like a random walk, so the bound grows with sqrt(K); 2e-6 is the
    floor that the short sums of the small shapes were given from the start."""
    return max(2e-6, 4.0 * math.sqrt(K) * 2.0 ** -24)


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
@pytest.mark.parametrize("in_dtype,out_dtype,tol", [(torch.float32, torch.float32, None),
                                                    (torch.bfloat16, torch.float32, None),
                                                    (torch.bfloat16, torch.bfloat16, 5e-3)])
@pytest.mark.parametrize("act", [None, "gelu_tanh", "gelu_erf"])
def test_linear(M, N, K, in_dtype, out_dtype, tol, act):
    from vlrf_b200.csrc import ops
    tol = tol if tol is not None else f32_sum_tol(K)
    x, w = randn(M, K, seed=9, dtype=in_dtype), randn(N, K, seed=10, dtype=in_dtype, scale=0.3)
    bias, res = randn(N, seed=11), randn(M, N, seed=12)
    want = x.double() @ w.double().T + bias.double()
    if act == "gelu_tanh":
        want = plain.gelu_tanh(want)
    elif act == "gelu_erf":
        want = plain.gelu_erf(want)
    out = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
    ops.linear(x.to(DEV), w.to(DEV), bias.to(DEV), out, act=act)
    assert rel_err(out.float().cpu(), want) < tol
    if out_dtype == torch.float32:   # residual sum in place, as the blocks use it
        acc = res.clone().to(DEV)
        ops.linear(x.to(DEV), w.to(DEV), bias.to(DEV), acc, act=act, residual=acc)
        assert rel_err(acc.cpu(), want + res.double()) < tol
        nob = torch.empty(M, N, device=DEV)
        ops.linear(x.to(DEV), w.to(DEV), None, nob)
        assert rel_err(nob.cpu(), x.double() @ w.double().T) < tol


@pytest.mark.parametrize("M,N,K", [(1, 96, 64), (8, 2304, 768), (13, 200, 96), (16, 320, 96), (9, 130, 1600), (16, 130, 768)])
@pytest.mark.parametrize("out_dtype,act", [(torch.bfloat16, None), (torch.bfloat16, "gelu_tanh"), (torch.float32, "gelu_erf")])
def test_linear_with_fused_layernorm(M, N, K, out_dtype, act):
    from vlrf_b200.csrc import ops
    assert ops.can_fuse_layernorm(M, K, torch.bfloat16)
    x = randn(M, K, seed=16) * 2 + 0.5
    gamma, beta = randn(K, seed=17) * 0.3 + 1, randn(K, seed=18) * 0.2
    w, b = randn(N, K, seed=19, dtype=torch.bfloat16, scale=0.2), randn(N, seed=20)
    eps = 1e-5
    h = plain.layer_norm(x.double(), gamma.double(), beta.double(), eps)
    h = h.to(torch.bfloat16).double()       # the kernel rounds the normed rows to bfloat16 for the tensor cores
    want = h @ w.double().T + b.double()
    if act:
        want = (plain.gelu_tanh if act == "gelu_tanh" else plain.gelu_erf)(want)
    out = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
    ops.linear_layernorm(x.to(DEV), gamma.to(DEV), beta.to(DEV), eps, w.to(DEV), b.to(DEV), out, act=act)
    # a normed value that lies within rounding of a bfloat16 tie may round the other way than float64's
    assert rel_err(out.float().cpu(), want) < (6e-3 if out_dtype == torch.bfloat16 else 3e-3)


def test_fused_projection_writes_keys_and_values_into_the_cache():
    from vlrf_b200.csrc import ops
    H, Hkv, dh, K, M = 4, 2, 16, 96, 5
    N = (H + 2 * Hkv) * dh
    x = randn(M, K, seed=21)
    gamma, beta = torch.ones(K), torch.zeros(K)
    w, b = randn(N, K, seed=22, dtype=torch.bfloat16, scale=0.2), randn(N, seed=23)
    kc = torch.full((6, Hkv, 64, dh), float("nan"), dtype=torch.bfloat16, device=DEV)
    vc = torch.full_like(kc, float("nan"))
    table = torch.tensor([[3, 1], [5, -1], [2, 0]], dtype=torch.int32)
    slot = torch.tensor([0, 2, -1, 1, 2], dtype=torch.int32)      # row 2 is padding; rows 1 and 4 share slot 2
    pos = torch.tensor([70, 5, 0, 63, 64], dtype=torch.int32)
    out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    ops.linear_layernorm(x.to(DEV), gamma.to(DEV), beta.to(DEV), 1e-5, w.to(DEV), b.to(DEV), out,
                         kv_scatter=(kc, vc, table.to(DEV), slot.to(DEV), pos.to(DEV), H * dh, (H + Hkv) * dh, Hkv, dh))
    o = out.cpu()
    for m in range(M):
        if slot[m] < 0:
            continue
        blk = int(table[slot[m], pos[m] // 64])
        assert torch.equal(kc[blk, :, pos[m] % 64].cpu().reshape(-1), o[m, H * dh:(H + Hkv) * dh])
        assert torch.equal(vc[blk, :, pos[m] % 64].cpu().reshape(-1), o[m, (H + Hkv) * dh:])
    written = (~torch.isnan(kc.float())).sum().item()
    assert written == 4 * Hkv * dh                                   # nothing else was touched


@pytest.fixture
def split_k_always(monkeypatch):
    """Send every few-row bfloat16 product to the split-k tensor-core kernel, whatever its size."""
    from vlrf_b200.csrc import ops
    monkeypatch.setattr(ops, "SPLITK_MIN_WEIGHT_BYTES", 0)
    monkeypatch.setattr(ops, "SPLITK_NORM_MIN_WEIGHT_BYTES", 0)
    return ops


# few and many tiles, one and many parts, 64- and 128-row tiles, tails in M, N and K
SPLIT_K_SHAPES = [(1, 200, 72), (8, 512, 256), (16, 1600, 1600), (17, 1000, 320), (33, 136, 200), (64, 768, 3072),
                  (5, 96, 64), (8, 6400, 1600), (40, 130, 8), (4, 1600, 6400), (12, 768, 3072), (16, 200, 4096)]


@pytest.mark.parametrize("M,N,K", SPLIT_K_SHAPES)
@pytest.mark.parametrize("out_dtype,tol", [(torch.float32, None), (torch.bfloat16, 5e-3)])
@pytest.mark.parametrize("act", [None, "gelu_tanh"])
def test_linear_split_k(split_k_always, M, N, K, out_dtype, tol, act):
    ops = split_k_always
    assert ops._splitk_takes(M, N, K, K, False)
    tol = tol if tol is not None else f32_sum_tol(K)
    x, w = randn(M, K, seed=31, dtype=torch.bfloat16), randn(N, K, seed=32, dtype=torch.bfloat16, scale=0.3)
    bias, res = randn(N, seed=33), randn(M, N, seed=34)
    want = x.double() @ w.double().T + bias.double()
    if act == "gelu_tanh":
        want = plain.gelu_tanh(want)
    out = torch.full((M + 1, N), float("nan"), dtype=out_dtype, device=DEV)
    ops.linear(x.to(DEV), w.to(DEV), bias.to(DEV), out, act=act, rows=M)
    assert rel_err(out[:M].float().cpu(), want) < tol
    assert torch.isnan(out[M].float()).all()                     # no row beyond M is written
    if out_dtype == torch.float32:
        acc = res.clone().to(DEV)
        ops.linear(x.to(DEV), w.to(DEV), bias.to(DEV), acc, act=act, residual=acc)
        assert rel_err(acc.cpu(), want + res.double()) < tol
        again = res.clone().to(DEV)                              # the same again: the sum does not depend on timing
        ops.linear(x.to(DEV), w.to(DEV), bias.to(DEV), again, act=act, residual=again)
        assert torch.equal(acc, again)
    assert ops.device_errors() == 0


@pytest.mark.parametrize("M,N,K", [(1, 96, 64), (8, 2304, 768), (13, 200, 200), (16, 320, 96), (9, 4800, 1600), (7, 130, 1000)])
@pytest.mark.parametrize("out_dtype,act", [(torch.bfloat16, None), (torch.bfloat16, "gelu_tanh"), (torch.float32, None)])
def test_split_k_layernorm_from_row_statistics(split_k_always, M, N, K, out_dtype, act):
    """A product that writes float32 residual rows leaves their per-segment statistics; the next product
    normalises with them.  Rows with a large common offset show a variance that is not computed as a
    deviation from the mean."""
    ops = split_k_always
    eps = 1e-5
    stats = ops.RowStats(DEV)
    w0, x0 = randn(K, 64, seed=41, dtype=torch.bfloat16), randn(M, 64, seed=42, dtype=torch.bfloat16)
    x = (randn(M, K, seed=43) * 0.5 + 300.0).to(DEV)             # mean 300, deviation about 8
    ops.linear(x0.to(DEV), w0.to(DEV), None, x, residual=x, stats=stats)
    assert stats.describing(x, M, K) is not None
    gamma, beta = randn(K, seed=44) * 0.3 + 1, randn(K, seed=45) * 0.2
    w, b = randn(N, K, seed=46, dtype=torch.bfloat16, scale=0.2), randn(N, seed=47)

    def want_for(rows):
        h = plain.layer_norm(rows.double().cpu(), gamma.double(), beta.double(), eps).to(torch.bfloat16).double()
        y = h @ w.double().T + b.double()
        return plain.gelu_tanh(y) if act == "gelu_tanh" else y

    tol = 6e-3 if out_dtype == torch.bfloat16 else 3e-3
    out = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
    ops.linear_layernorm(x, gamma.to(DEV), beta.to(DEV), eps, w.to(DEV), b.to(DEV), out, act=act, stats=stats)
    assert rel_err(out.float().cpu(), want_for(x)) < tol
    # rows changed behind the statistics' back: by torch in place, by a kernel of this library, by a caller's own
    x.mul_(0.5)
    assert stats.describing(x, M, K) is None
    if ops.can_fuse_layernorm(M, K, torch.bfloat16):             # (the kernel that reads whole rows takes this width)
        ops.linear_layernorm(x, gamma.to(DEV), beta.to(DEV), eps, w.to(DEV), b.to(DEV), out, act=act, stats=stats)
        assert rel_err(out.float().cpu(), want_for(x)) < tol
    ops.linear(x0.to(DEV), w0.to(DEV), None, x, residual=x, stats=stats)
    assert stats.describing(x, M, K) is not None
    # the embedding leaves statistics of the rows it writes, too
    table = (randn(50, K, seed=48) * 3 + 20).to(DEV)
    ops.embed(table, None, torch.arange(M, dtype=torch.int32, device=DEV) * 3, None, x,
              torch.zeros(1, dtype=torch.int32, device=DEV), stats=stats)
    assert stats.describing(x, M, K) is not None
    ops.linear_layernorm(x, gamma.to(DEV), beta.to(DEV), eps, w.to(DEV), b.to(DEV), out, act=act, stats=stats)
    assert rel_err(out.float().cpu(), want_for(x)) < tol
    # a product that is handed no statistics keeps none, and one that rewrites the rows without them forgets them
    ops.linear(x0.to(DEV), w0.to(DEV), None, x, residual=x, stats=stats)
    stats.forget()
    assert stats.describing(x, M, K) is None
    other = ops.RowStats(DEV)
    ops.linear(x0.to(DEV), w0.to(DEV), None, x, residual=x)
    assert other.describing(x, M, K) is None
    assert ops.device_errors() == 0


def test_split_k_projection_writes_keys_and_values_into_the_cache(split_k_always):
    ops = split_k_always
    H, Hkv, dh, K, M = 4, 2, 16, 96, 5
    N = (H + 2 * Hkv) * dh
    table = torch.tensor([[3, 1], [5, -1], [2, 0]], dtype=torch.int32)
    slot = torch.tensor([0, 2, -1, 1, 2], dtype=torch.int32)      # row 2 is padding; rows 1 and 4 share slot 2
    pos = torch.tensor([70, 5, 0, 63, 64], dtype=torch.int32)
    w, b = randn(N, K, seed=52, dtype=torch.bfloat16, scale=0.2), randn(N, seed=53)
    for fused_norm in (False, True):
        kc = torch.full((6, Hkv, 64, dh), float("nan"), dtype=torch.bfloat16, device=DEV)
        vc = torch.full_like(kc, float("nan"))
        scatter = (kc, vc, table.to(DEV), slot.to(DEV), pos.to(DEV), H * dh, (H + Hkv) * dh, Hkv, dh)
        out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
        if fused_norm:
            x = torch.zeros(M, K, device=DEV)
            stats = ops.RowStats(DEV)
            ops.linear(randn(M, 64, seed=54, dtype=torch.bfloat16).to(DEV), randn(K, 64, seed=55, dtype=torch.bfloat16).to(DEV),
                       None, x, stats=stats)
            assert stats.describing(x, M, K) is not None
            ops.linear_layernorm(x, torch.ones(K, device=DEV), torch.zeros(K, device=DEV), 1e-5, w.to(DEV), b.to(DEV), out,
                                 kv_scatter=scatter, stats=stats)
        else:
            assert ops.linear(randn(M, K, seed=51, dtype=torch.bfloat16).to(DEV), w.to(DEV), b.to(DEV), out, kv_scatter=scatter)
        o = out.cpu()
        for m in range(M):
            if slot[m] < 0:
                continue
            blk = int(table[slot[m], pos[m] // 64])
            assert torch.equal(kc[blk, :, pos[m] % 64].cpu().reshape(-1), o[m, H * dh:(H + Hkv) * dh])
            assert torch.equal(vc[blk, :, pos[m] % 64].cpu().reshape(-1), o[m, (H + Hkv) * dh:])
        assert (~torch.isnan(kc.float())).sum().item() == 4 * Hkv * dh     # nothing else was touched
    assert ops.device_errors() == 0


@pytest.mark.parametrize("width", [64, 96, 128, 160, 192, 224, 256])
def test_tcgen05_tile_widths(width):
    """Every tile width of the tcgen05 product, forced (the choice by size would pick one): tails in M, N and K,
    float32 with the residual in place, bfloat16 with an activation, and the cache scatter with heads of 8 columns
    (16-byte pieces) and of 16 and 64 (32-byte pieces)."""
    from vlrf_b200.csrc import library, ops
    lib = library()
    assert lib.vlrf_gemm_tcgen05_force_width(width) == 0
    try:
        M, N, K = 300, 1000, 200
        x, w = randn(M, K, seed=90, dtype=torch.bfloat16), randn(N, K, seed=91, dtype=torch.bfloat16, scale=0.3)
        bias, res = randn(N, seed=92), randn(M, N, seed=93)
        want = x.double() @ w.double().T + bias.double()
        acc = res.clone().to(DEV)
        ops.linear(x.to(DEV), w.to(DEV), bias.to(DEV), acc, residual=acc)
        assert rel_err(acc.cpu(), want + res.double()) < f32_sum_tol(K)
        out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
        ops.linear(x.to(DEV), w.to(DEV), bias.to(DEV), out, act="gelu_tanh")
        assert rel_err(out.float().cpu(), plain.gelu_tanh(want)) < 5e-3
        for H, Hkv, dh in ((6, 3, 8), (4, 2, 16), (3, 3, 64)):
            Nq = (H + 2 * Hkv) * dh
            T = 150
            wq, bq = randn(Nq, K, seed=94, dtype=torch.bfloat16, scale=0.2), randn(Nq, seed=95)
            table = torch.tensor([[3, 1, 4], [5, 0, -1]], dtype=torch.int32)
            slot = torch.tensor([0] * 100 + [-1] * 10 + [1] * 40, dtype=torch.int32)
            pos = torch.tensor(list(range(60, 160)) + [0] * 10 + list(range(30, 70)), dtype=torch.int32)
            kc = torch.full((6, Hkv, 64, dh), float("nan"), dtype=torch.bfloat16, device=DEV)
            vc = torch.full_like(kc, float("nan"))
            o = torch.empty(T, Nq, dtype=torch.bfloat16, device=DEV)
            assert ops.linear(randn(T, K, seed=96, dtype=torch.bfloat16).to(DEV), wq.to(DEV), bq.to(DEV), o,
                              kv_scatter=(kc, vc, table.to(DEV), slot.to(DEV), pos.to(DEV), H * dh, (H + Hkv) * dh, Hkv, dh))
            oc = o.cpu()
            for m in range(T):
                if slot[m] < 0:
                    continue
                blk = int(table[slot[m], pos[m] // 64])
                assert torch.equal(kc[blk, :, pos[m] % 64].cpu().reshape(-1), oc[m, H * dh:(H + Hkv) * dh])
                assert torch.equal(vc[blk, :, pos[m] % 64].cpu().reshape(-1), oc[m, (H + Hkv) * dh:])
            assert (~torch.isnan(kc.float())).sum().item() == 140 * Hkv * dh     # nothing else was touched
        assert ops.device_errors() == 0
    finally:
        lib.vlrf_gemm_tcgen05_force_width(0)


def test_split_k_rows_do_not_depend_on_the_batch(split_k_always):
    import os
    if os.environ.get("VLRF_B200_SPLITK_MMA"):
        pytest.skip("the environment sends the products another way than the rule this test states")
    ops = split_k_always
    x, w, b = randn(64, 320, seed=56, dtype=torch.bfloat16), randn(1000, 320, seed=57, dtype=torch.bfloat16), randn(1000, seed=58)
    full = torch.empty(64, 1000, device=DEV)
    ops.linear(x.to(DEV), w.to(DEV), b.to(DEV), full)
    for rows in (1, 5, 9, 20):
        few = torch.empty(rows, 1000, device=DEV)
        ops.linear(x[41:41 + rows].contiguous().to(DEV), w.to(DEV), b.to(DEV), few)
        if rows > 16:
            assert torch.equal(full[41:41 + rows], few)
        else:
            # up to 16 rows the sums are formed by another instruction (four accumulators a k block): the same values
            # up to the rounding of float32 sums, and the same whatever else is in such a batch
            assert rel_err(few.cpu(), full[41:41 + rows].cpu()) < 2e-6
            alone = torch.empty(1, 1000, device=DEV)
            ops.linear(x[41:42].contiguous().to(DEV), w.to(DEV), b.to(DEV), alone)
            assert torch.equal(alone, few[:1])


def test_linear_rows_do_not_depend_on_the_batch():
    from vlrf_b200.csrc import ops
    x, w, b = randn(70, 96, seed=13), randn(200, 96, seed=14), randn(200, seed=15)
    full = torch.empty(70, 200, device=DEV)
    ops.linear(x.to(DEV), w.to(DEV), b.to(DEV), full)
    one = torch.empty(1, 200, device=DEV)
    ops.linear(x[41:42].contiguous().to(DEV), w.to(DEV), b.to(DEV), one)
    assert torch.equal(full[41:42], one)


# ------------------------------------------------------------------------------------------------
def paged(k, v, n_blocks, order_seed, dtype):
    """Put [H, C, dh] keys and values of one sequence into a pool with scattered blocks; unused pool
    entries are NaN."""
    H, C, dh = k.shape
    nb = (C + 63) // 64
    perm = torch.randperm(n_blocks, generator=g(order_seed))[:nb]
    kp = torch.full((n_blocks, H, 64, dh), float("nan"), dtype=dtype)
    vp = torch.full((n_blocks, H, 64, dh), float("nan"), dtype=dtype)
    for i, b in enumerate(perm.tolist()):
        n = min(64, C - 64 * i)
        kp[b, :, :n] = k[:, 64 * i:64 * i + n].to(dtype)
        vp[b, :, :n] = v[:, 64 * i:64 * i + n].to(dtype)
    return kp, vp, perm.to(torch.int32)


def run_attention(q, k, v, *, dtype, scale, window=0, past=None, impl="generic", n_split=1, scratch=True):
    """q [H, T, dh] are the LAST T positions of a context of C = k.shape[1] tokens."""
    from vlrf_b200.csrc import ops
    H, T, dh = q.shape
    Hkv, C, _ = k.shape
    kp, vp, blocks = paged(k, v, 12, 21, dtype)
    table = torch.full((3, 10), -1, dtype=torch.int32)
    table[1, :blocks.numel()] = blocks
    qkv = torch.zeros(T, H * dh + 5 * 16, dtype=dtype)          # q sits at an offset inside a wider row
    qkv[:, 16:16 + H * dh] = q.permute(1, 0, 2).reshape(T, H * dh).to(dtype)
    out = torch.full((T, H * dh), float("nan"), dtype=dtype, device=DEV)
    e = err_word()
    slot = torch.full((T,), 1, dtype=torch.int32)
    pos = torch.arange(C - T, C, dtype=torch.int32)
    if impl == "decode" and not scratch:
        # the parts of a context merge inside a thread-block cluster: no scratch
        assert not ops.attention_decode_needs_scratch(dh, n_split)
        for _ in range(2):
            out.fill_(float("nan"))
            ops.attention_decode(qkv.to(DEV), 16, kp.to(DEV), vp.to(DEV), table.to(DEV), slot.to(DEV), pos.to(DEV), out,
                                 T, H, Hkv, dh, scale, window, n_split, None, None, e)
    elif impl == "decode":
        partials = torch.full((T * H * n_split * (dh + 2),), float("nan"), device=DEV)
        counters = torch.zeros(T * H, dtype=torch.int32, device=DEV)
        for _ in range(2):       # twice: the counters must be back at zero after a call
            out.fill_(float("nan"))
            ops.attention_decode(qkv.to(DEV), 16, kp.to(DEV), vp.to(DEV), table.to(DEV), slot.to(DEV), pos.to(DEV), out,
                                 T, H, Hkv, dh, scale, window, n_split, partials, counters, e)
        assert int(counters.abs().sum()) == 0
    else:
        ops.attention_generic(qkv.to(DEV), 16, kp.to(DEV), vp.to(DEV), table.to(DEV), slot.to(DEV), pos.to(DEV), out,
                              T, H, Hkv, dh, scale, window, e)
    assert int(e.item()) == 0
    return out.float().cpu().reshape(T, H, dh).permute(1, 0, 2)


def plain_attention(q, k, v, scale, window=0):
    H, T, dh = q.shape
    Hkv, C, _ = k.shape
    rep = H // Hkv
    kk, vv = k.repeat_interleave(rep, 0).double(), v.repeat_interleave(rep, 0).double()
    qq = torch.zeros(H, C, dh, dtype=torch.float64)
    qq[:, C - T:] = q.double()
    return plain.causal_attention(qq, kk, vv, scale, window)[:, C - T:]


ATT_CASES = [  # H, Hkv, dh, T, C   (tails, decode, continuation — as tests/test_flash_attention.cpp:96-121)
    (3, 3, 16, 37, 37), (4, 4, 32, 130, 130), (2, 2, 64, 1, 200), (2, 1, 64, 200, 500), (6, 2, 48, 64, 64),
    (4, 1, 80, 65, 129), (1, 1, 128, 5, 70), (5, 5, 256, 3, 66), (12, 12, 64, 128, 128),
]


@pytest.mark.parametrize("H,Hkv,dh,T,C", ATT_CASES)
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 1.5e-2)])
def test_attention_generic(H, Hkv, dh, T, C, dtype, tol):
    q, k, v = randn(H, T, dh, seed=30), randn(Hkv, C, dh, seed=31), randn(Hkv, C, dh, seed=32)
    if dtype == torch.bfloat16:   # the kernel sees bfloat16 inputs; compare on what it sees
        q, k, v = (t.to(dtype).float() for t in (q, k, v))
    scale = 0.7 / math.sqrt(dh)
    got = run_attention(q, k, v, dtype=dtype, scale=scale)
    assert rel_err(got, plain_attention(q, k, v, scale)) < tol


@pytest.mark.parametrize("H,Hkv,dh,T,C", ATT_CASES + [(12, 12, 64, 8, 1024 - 400), (25, 25, 64, 2, 33)])
@pytest.mark.parametrize("n_split", [1, 2, 5, 16])
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 1.5e-2)])
def test_attention_decode_split_context(H, Hkv, dh, T, C, n_split, dtype, tol):
    """The decode kernel takes any rows (here the last T positions of one context), any split count."""
    if T > 40:
        T = 40
    q, k, v = randn(H, T, dh, seed=30), randn(Hkv, C, dh, seed=31), randn(Hkv, C, dh, seed=32)
    if dtype == torch.bfloat16:
        q, k, v = (t.to(dtype).float() for t in (q, k, v))
    scale = 0.7 / math.sqrt(dh)
    got = run_attention(q, k, v, dtype=dtype, scale=scale, impl="decode", n_split=n_split)
    assert rel_err(got, plain_attention(q, k, v, scale)) < tol
    from vlrf_b200.csrc import ops
    if n_split > 1 and not ops.attention_decode_needs_scratch(dh, n_split):
        again = run_attention(q, k, v, dtype=dtype, scale=scale, impl="decode", n_split=n_split, scratch=False)
        assert torch.equal(again, got)                       # the same merge, in shared memory instead of scratch


@pytest.mark.parametrize("far", [0, 63, 64, 257, 511])
@pytest.mark.parametrize("n_split", [1, 4])
def test_attention_decode_finds_one_far_key_and_respects_a_window(far, n_split):
    H, dh, C = 2, 64, 512
    q, k, v = randn(H, 1, dh, seed=36), randn(H, C, dh, seed=37) * 0.1, randn(H, C, dh, seed=38)
    k[:, far] = q[:, 0] * 4.0
    got = run_attention(q, k, v, dtype=torch.float32, scale=1.0, impl="decode", n_split=n_split)
    assert rel_err(got[:, 0], v[:, far]) < 1e-4
    for window in (1, 33, 200, 512 - far, 511 - far):
        got = run_attention(q, k, v, dtype=torch.float32, scale=1.0, window=window, impl="decode", n_split=n_split)
        assert rel_err(got, plain_attention(q, k, v, 1.0, window)) < 2e-5


@pytest.mark.parametrize("far", [0, 31, 32, 255, 256, 511, 639])
@pytest.mark.parametrize("n_split", [1, 3])
def test_attention_decode_bf16_finds_one_far_key_and_respects_a_window(far, n_split):
    """The same for the tensor-core decode kernel (bfloat16, head size 64) over 20 chunks of 32 keys, so that a
    warp reads up to three chunks through its buffer: a chunk dropped, read twice or read before it has landed
    shows as a wrong value, not as a small error."""
    H, dh, C = 3, 64, 640
    q, k, v = (t.to(torch.bfloat16).float() for t in (randn(H, 1, dh, seed=66), randn(H, C, dh, seed=67) * 0.1, randn(H, C, dh, seed=68)))
    k[:, far] = (q[:, 0] * 4.0).to(torch.bfloat16).float()
    got = run_attention(q, k, v, dtype=torch.bfloat16, scale=1.0, impl="decode", n_split=n_split)
    assert rel_err(got[:, 0], v[:, far]) < 1e-2
    for window in (1, 33, 200, C - far, C - 1 - far):
        if window < 1:
            continue
        got = run_attention(q, k, v, dtype=torch.bfloat16, scale=1.0, window=window, impl="decode", n_split=n_split,
                            scratch=(n_split == 1))
        assert rel_err(got, plain_attention(q, k, v, 1.0, window)) < 1.5e-2


@pytest.mark.parametrize("window", [1, 31, 32, 33, 64, 100])
def test_attention_window_edges(window):
    H, dh, T, C = 2, 32, 150, 150
    q, k, v = randn(H, T, dh, seed=33), randn(H, C, dh, seed=34), randn(H, C, dh, seed=35)
    # make the key just outside each query's window the one it would like best
    for t in range(window, C):
        k[:, t - window] = 0
    got = run_attention(q, k, v, dtype=torch.float32, scale=0.2, window=window)
    assert rel_err(got, plain_attention(q, k, v, 0.2, window)) < 2e-5
    k2 = k.clone()
    k2[:, 3] = q[:, 3 + window] * 50 if 3 + window < T else k2[:, 3]   # would dominate if it were seen
    got2 = run_attention(q, k2, v, dtype=torch.float32, scale=0.2, window=window)
    assert rel_err(got2[:, 3 + window], plain_attention(q, k2, v, 0.2, window)[:, 3 + window]) < 2e-5


@pytest.mark.parametrize("far", [0, 63, 64, 257, 511])
def test_attention_finds_one_far_key(far):
    """One key among hundreds carries the whole weight: the output must be that key's value."""
    H, dh, C = 2, 64, 512
    q, k, v = randn(H, 1, dh, seed=36), randn(H, C, dh, seed=37) * 0.1, randn(H, C, dh, seed=38)
    k[:, far] = q[:, 0] * 4.0
    got = run_attention(q, k, v, dtype=torch.float32, scale=1.0)
    assert rel_err(got[:, 0], v[:, far]) < 1e-4
    assert rel_err(got, plain_attention(q, k, v, 1.0)) < 2e-5


PREFILL_CASES = [  # H, Hkv, dh, [(tokens already cached, new tokens)], window
    (2, 2, 64, [(0, 64)], 0), (3, 3, 64, [(0, 1), (0, 65), (0, 200)], 0), (4, 2, 64, [(37, 100), (128, 3), (0, 64)], 0),
    (2, 1, 128, [(0, 130), (64, 70)], 0), (12, 12, 64, [(0, 300), (250, 50)], 0), (2, 2, 64, [(0, 260), (100, 90)], 70),
    (2, 2, 128, [(5, 140)], 64),
    # long rows: many key blocks per query tile, tiles of unequal length, a continuation across block pairs
    (3, 3, 64, [(0, 1024), (0, 700)], 0), (2, 2, 64, [(0, 600), (300, 500)], 200), (2, 1, 64, [(127, 130), (129, 1), (63, 66)], 0),
    (2, 2, 64, [(900, 300), (0, 513)], 0), (1, 1, 64, [(0, 800)], 520),
]


@pytest.mark.parametrize("kernel", ["tcgen05", "tcgen05_parts2", "tcgen05_parts3", "mma_sync"])
@pytest.mark.parametrize("H,Hkv,dh,seqs,window", PREFILL_CASES)
def test_attention_prefill_tensor_cores(monkeypatch, kernel, H, Hkv, dh, seqs, window):
    """Ragged batches with unequal lengths and continuations, grouped heads, a window; the cache is NaN
    outside what the sequences hold, and freed-looking rows inside their last blocks are NaN too.  With
    parts, long tiles' keys are dealt to several CTAs that meet in scratch: it starts as NaN, is used twice,
    and both runs give the same bits whichever CTA came last."""
    from vlrf_b200.csrc import ops
    if kernel.startswith("tcgen05") and dh != 64:
        pytest.skip("the tcgen05 kernel takes head size 64")
    monkeypatch.setattr(ops, "PREFILL_ATTENTION_TCGEN05", kernel.startswith("tcgen05"))
    n_parts = int(kernel[-1]) if "parts" in kernel else 1
    dtype = torch.bfloat16
    scale = 0.8 / math.sqrt(dh)
    n_blocks = sum((p + n + 63) // 64 for p, n in seqs) + 2
    kc = torch.full((n_blocks, Hkv, 64, dh), float("nan"), dtype=dtype)
    vc = torch.full((n_blocks, Hkv, 64, dh), float("nan"), dtype=dtype)
    order = torch.randperm(n_blocks, generator=g(50)).tolist()
    max_blocks = max((p + n + 63) // 64 for p, n in seqs) + 1
    table = torch.full((len(seqs) + 1, max_blocks), -1, dtype=torch.int32)
    T = sum(n for _, n in seqs)
    W = (H + 2 * Hkv) * dh
    qkv = torch.zeros(T, W, dtype=dtype)
    starts, want, at = [0], [], 0
    for i, (p0, n) in enumerate(seqs):
        C = p0 + n
        q = randn(H, n, dh, seed=60 + i).to(dtype).float()
        k = randn(Hkv, C, dh, seed=70 + i).to(dtype).float()
        v = randn(Hkv, C, dh, seed=80 + i).to(dtype).float()
        if C > 40:                          # one far key that a late query likes best
            k[:, 3] = q[:Hkv, -1] * 3.0 if Hkv <= H else k[:, 3]
        for b in range((C + 63) // 64):
            blk = order.pop()
            table[i + 1, b] = blk           # slot i+1 (slot 0 stays unused)
            m = min(64, C - 64 * b)
            kc[blk, :, :m] = k[:, 64 * b:64 * b + m].to(dtype)
            vc[blk, :, :m] = v[:, 64 * b:64 * b + m].to(dtype)
        qkv[at:at + n, :H * dh] = q.permute(1, 0, 2).reshape(n, H * dh).to(dtype)
        want.append(plain_attention(q, k, v, scale, window))
        at += n
        starts.append(at)
    out = torch.full((T, H * dh), float("nan"), dtype=dtype, device=DEV)
    e = err_word()
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device=DEV)  # noqa: E731
    assert ops.attention_prefill_takes(dtype, dh, 64, W, 0)
    max_new = max(n for _, n in seqs)
    partials = counters = None
    if n_parts > 1:
        n_floats, n_counters = ops.attention_prefill_scratch(len(seqs), max_new, H, n_parts)
        partials = torch.full((n_floats,), float("nan"), device=DEV)
        counters = torch.zeros(n_counters, dtype=torch.int32, device=DEV)
    args = (qkv.to(DEV), 0, kc.to(DEV), vc.to(DEV), table.to(DEV), i32(list(range(1, len(seqs) + 1))), i32(starts),
            i32([p for p, _ in seqs]))
    ops.attention_prefill(*args, out, T, len(seqs), max_new, H, Hkv, dh, scale, window, e, n_parts, partials, counters)
    assert int(e.item()) == 0
    if n_parts > 1:
        assert int(counters.abs().sum()) == 0
        again = torch.full_like(out, float("nan"))
        ops.attention_prefill(*args, again, T, len(seqs), max_new, H, Hkv, dh, scale, window, e, n_parts, partials, counters)
        assert int(e.item()) == 0 and int(counters.abs().sum()) == 0
        assert torch.equal(again.view(torch.int16), out.view(torch.int16))
    got = out.float().cpu()
    assert torch.isfinite(got).all()
    for i, (p0, n) in enumerate(seqs):
        mine = got[starts[i]:starts[i + 1]].reshape(n, H, dh).permute(1, 0, 2)
        assert rel_err(mine, want[i]) < 1.5e-2, (i, p0, n)


def test_kv_append_writes_each_token_where_its_slot_says():
    from vlrf_b200.csrc import ops
    Hkv, dh, T = 3, 16, 70
    for dtype in (torch.float32, torch.bfloat16):
        qkv = randn(T, 5 * Hkv * dh, seed=39, dtype=dtype)
        kc = torch.zeros(6, Hkv, 64, dh, dtype=dtype, device=DEV)
        vc = torch.zeros_like(kc)
        table = torch.tensor([[4, 1, -1], [2, 5, 0]], dtype=torch.int32)
        slot = torch.tensor([0] * 30 + [1] * 40, dtype=torch.int32)
        pos = torch.cat([torch.arange(50, 80), torch.arange(100, 140)]).to(torch.int32)
        e = err_word()
        ops.kv_append(qkv.to(DEV), 2 * Hkv * dh, 4 * Hkv * dh, kc, vc, table.to(DEV), slot.to(DEV), pos.to(DEV), T, Hkv,
                      dh, e)
        assert int(e.item()) == 0
        for t in range(T):
            b = int(table[slot[t], pos[t] // 64])
            assert torch.equal(kc[b, :, pos[t] % 64].cpu().reshape(-1), qkv[t, 2 * Hkv * dh:3 * Hkv * dh])
            assert torch.equal(vc[b, :, pos[t] % 64].cpu().reshape(-1), qkv[t, 4 * Hkv * dh:5 * Hkv * dh])
        assert float(kc[3].abs().sum()) == 0          # an unmapped block stays untouched
        # a token whose block is not mapped is skipped and reported
        pos2 = pos.clone(); pos2[0] = 130
        ops.kv_append(qkv.to(DEV), 2 * Hkv * dh, 4 * Hkv * dh, kc, vc, table.to(DEV), slot.to(DEV), pos2.to(DEV), T,
                      Hkv, dh, e)
        assert int(e.item()) == 4


# ------------------------------------------------------------------------------------------------
def test_argmax_takes_the_first_maximum():
    from vlrf_b200.csrc import ops
    V = 50257
    lg = randn(5, V, seed=40)
    lg[0, 777] = lg[0, 40000] = 9.0
    lg[1, V - 1] = 9.0
    lg[2, 0] = 9.0
    out = torch.zeros(5, dtype=torch.int32, device=DEV)
    ops.sample(lg.to(DEV), 5, out)
    assert out.tolist() == [777, V - 1, 0, int(lg[3].argmax()), int(lg[4].argmax())]


@pytest.mark.parametrize("V", [1000, 50257])
def test_sampling_matches_the_plain_sampler(V):
    from vlrf_b200.csrc import ops
    from vlrf_b200.sampling.rng import as_signed64, request_key, uniform01
    n = 48
    lg = randn(n, V, seed=41) * 2.0
    rs = np.random.RandomState(5)
    temp = rs.choice([0.0, 0.5, 0.8, 1.0, 1.7], n).astype(np.float32)
    top_k = rs.choice([0, 1, 5, 50, V, V + 10], n).astype(np.int32)
    top_p = rs.choice([1.0, 0.9, 0.5, 0.05, 0.999], n).astype(np.float32)
    keys = [request_key(42, i) for i in range(n)]
    d = lambda a, dt: torch.tensor(a, dtype=dt, device=DEV)  # noqa: E731
    ctr = torch.zeros(n, dtype=torch.int32, device=DEV)
    key_t = d([as_signed64(k) for k in keys], torch.int64)
    out = torch.zeros(n, dtype=torch.int32, device=DEV)
    lg_d = lg.to(DEV)
    for draw in range(3):
        ops.sample(lg_d, n, out, temperature=d(temp, torch.float32), top_k=d(top_k, torch.int32),
                   top_p=d(top_p, torch.float32), rng_key=key_t, rng_ctr=ctr)
        got = out.tolist()
        mismatches = []
        for i in range(n):
            u = uniform01(keys[i], draw)
            want = plain.sample_token(lg[i].numpy(), float(temp[i]), int(top_k[i]), float(top_p[i]), u)
            if got[i] != want:
                # float32 vs float64 may differ where u falls within rounding of a boundary: accept a neighbour
                # of the boundary only if both candidates are kept tokens with cumulative masses that close
                p = np.exp((lg[i].numpy().astype(np.float64) - lg[i].numpy().max()) / max(float(temp[i]), 1e-9))
                mismatches.append((i, got[i], want, p[got[i]] / p.sum(), p[want] / p.sum()))
        assert len(mismatches) <= 1, mismatches
    assert (ctr.cpu().numpy() == np.where(temp > 0, 3, 0)).all()   # greedy rows draw nothing


def test_sampling_distribution_and_filters():
    """Many draws of one row: frequencies follow the renormalised kept probabilities."""
    from vlrf_b200.csrc import ops
    V, n = 37, 4096
    base = torch.log(torch.tensor([0.3, 0.2, 0.2, 0.1, 0.1] + [0.1 / 32] * 32))
    lg = base.repeat(n, 1).contiguous().to(DEV)
    d = lambda a, dt: torch.tensor(a, dtype=dt, device=DEV)  # noqa: E731
    keys = torch.arange(1, n + 1, dtype=torch.int64, device=DEV) * 7919
    out = torch.zeros(n, dtype=torch.int32, device=DEV)

    def draw(k, p):
        ctr = torch.zeros(n, dtype=torch.int32, device=DEV)
        ops.sample(lg, n, out, temperature=d([1.0] * n, torch.float32), top_k=d([k] * n, torch.int32),
                   top_p=d([p] * n, torch.float32), rng_key=keys, rng_ctr=ctr)
        return np.bincount(out.cpu().numpy(), minlength=V) / n

    f = draw(0, 1.0)
    assert abs(f[0] - 0.3) < 0.03 and abs(f[1] - 0.2) < 0.03 and abs(f[5:].sum() - 0.1) < 0.02
    f = draw(3, 1.0)          # ties at the cut (0.2, 0.2) both inside; 0.1s outside
    assert f[3:].sum() == 0 and abs(f[0] - 0.3 / 0.7) < 0.03
    f = draw(2, 1.0)          # the cut falls between the two tokens of equal probability: the lower index stays
    assert f[2:].sum() == 0 and f[1] > 0.3
    f = draw(0, 0.75)         # cumulative .3 .5 .7 .8>.75 → keep three
    assert f[3:].sum() == 0 and abs(f[2] - 0.2 / 0.7) < 0.03
    f = draw(0, 0.1)          # the most probable always stays
    assert f[0] == 1.0


def test_penalties_and_ngram_block():
    from vlrf_b200.csrc import ops
    V, n = 300, 6
    lg = randn(n, V, seed=42)
    gen = torch.zeros(n, 12, dtype=torch.int32)
    lens = torch.tensor([0, 5, 5, 12, 7, 3], dtype=torch.int32)
    rs = np.random.RandomState(9)
    hist = [list(rs.randint(0, 6, size=int(m))) for m in lens]     # few distinct tokens: repeats are certain
    for i, h in enumerate(hist):
        gen[i, :len(h)] = torch.tensor(h, dtype=torch.int32)
    rep = [1.0, 1.3, 1.0, 2.0, 1.0, 0.8]
    freq = [0.0, 0.0, 0.7, 0.2, 0.0, 0.1]
    pres = [0.0, 0.5, 0.0, 0.1, 0.0, 0.0]
    ngram = [0, 0, 2, 3, 2, 1]
    d = lambda a, dt: torch.tensor(a, dtype=dt, device=DEV)  # noqa: E731
    got = lg.clone().to(DEV)
    ops.apply_penalties(got, n, gen.to(DEV), lens.to(DEV), repetition=d(rep, torch.float32),
                        frequency=d(freq, torch.float32), presence=d(pres, torch.float32),
                        no_repeat_ngram=d(ngram, torch.int32))
    got = got.cpu().numpy()
    for i in range(n):
        counts = {}
        for t in hist[i]:
            counts[int(t)] = counts.get(int(t), 0) + 1
        want = plain.apply_penalties(lg[i].numpy(), counts, rep[i], freq[i], pres[i])
        want = plain.block_repeated_ngrams(want, [int(t) for t in hist[i]], ngram[i])
        fin = np.isfinite(want)
        assert (np.isfinite(got[i]) == fin).all()
        assert np.allclose(got[i][fin], want[fin], rtol=1e-6, atol=1e-6)
    assert np.array_equal(got[0], lg[0].numpy())      # nothing generated yet: untouched
