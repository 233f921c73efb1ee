"""The decode program (a decode step as one persistent kernel): each of its operations alone against the plain
functions at sizes other than the engine's, chains of operations (the grid barrier and the weight ring across
operations), and whole decode sessions of the tiny models against the plain implementation."""
import math

import pytest
import torch

import plain_gpt2 as plain
from conftest import TOL_BF16, random_ids, rel_err
from test_kernels import err_word, g, paged, plain_attention, randn

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
BF = torch.bfloat16


def program_for(n_rows, *, tokens=None, slot=None, pos=None, max_context=1024):
    from vlrf_b200.parts.context import Workspace
    from vlrf_b200.parts.program import DecodeProgram
    tokens = torch.zeros(n_rows, dtype=torch.int32) if tokens is None else tokens
    slot = torch.zeros(n_rows, dtype=torch.int32) if slot is None else slot
    pos = torch.zeros(n_rows, dtype=torch.int32) if pos is None else pos
    e = err_word()
    prog = DecodeProgram(n_rows=n_rows, tokens=tokens.to(DEV), tok_slot=slot.to(DEV), tok_pos=pos.to(DEV), dev_err=e,
                         ws=Workspace(DEV), act_dtype=BF, max_context=max_context)
    return prog, e


def unpack_flagged(buf):
    """The values in flagged rows (groups of 8 bytes: a float32 and a flag, or three bfloat16 and a flag), as [rows, cols]."""
    groups = buf.storage.cpu().view(buf.rows, buf.ld)
    seg = buf.seg if buf.seg > 0 else buf.cols
    if buf.dtype == torch.float32:
        vals = groups.view(torch.float32).reshape(buf.rows, buf.ld, 2)[:, :, 0]
        per, gps = 1, (seg + 1) // 2 * 2
    else:
        vals = groups.view(torch.bfloat16).reshape(buf.rows, buf.ld, 4)[:, :, :3].reshape(buf.rows, buf.ld * 3)
        per, gps = 3, (-(-seg // 3) + 1) // 2 * 2
    cols = [(c // seg) * gps * per + c % seg for c in range(buf.cols)]
    return vals[:, cols]


def plain_norm(x, kind, gamma, beta, eps):
    if kind == "layernorm":
        return plain.layer_norm(x, gamma, beta, eps)
    if kind == "rmsnorm":
        return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * gamma
    return x


PRODUCTS = [(1, 96, 64), (8, 2304, 768), (5, 1000, 320), (16, 130, 1600), (13, 777, 192), (8, 768, 3072), (16, 100, 6400),
            (3, 20011, 96), (9, 50, 4096), (2, 8, 32), (16, 50257, 64)]


@pytest.mark.parametrize("rows,N,K", PRODUCTS)
@pytest.mark.parametrize("kind", [None, "layernorm", "rmsnorm"])
def test_product_alone(rows, N, K, kind):
    from vlrf_b200.csrc import library
    in_f32 = kind is not None or K <= 768
    if not library().vlrf_decode_program_gemv_takes(rows, N, K, 0 if in_f32 else 1, 0, {None: 0, "layernorm": 1, "rmsnorm": 2}[kind]):
        pytest.skip("a float32 input wider than the registers of a warp hold is refused (the model then decodes launch by launch)")
    x = randn(rows, K, seed=1) * 2 + 0.5
    if not in_f32:
        x = x.to(BF).float()
    w = randn(N, K, seed=2, dtype=BF, scale=0.3)
    bias, res = randn(N, seed=3), randn(rows, N, seed=4)
    gamma, beta = randn(K, seed=5) * 0.3 + 1, randn(K, seed=6)
    eps = 1e-5
    h = plain_norm(x.double(), kind, gamma.double(), beta.double(), eps).to(BF).double()   # the kernel stages bfloat16 rows
    want = h @ w.double().T + bias.double()
    for act, out_dtype, use_res in ((None, torch.float32, True), ("gelu_tanh", BF, False), ("gelu_erf", torch.float32, False)):
        prog, e = program_for(rows)
        out = torch.full((rows, N), float("nan"), dtype=out_dtype, device=DEV)
        acc = res.clone().to(DEV)
        target = acc if use_res else out
        norm = None if kind is None else (kind, gamma.to(DEV), beta.to(DEV) if kind == "layernorm" else None, eps)
        prog.product(x.to(DEV) if in_f32 else x.to(BF).to(DEV), w.to(DEV), bias.to(DEV), target, norm=norm, act=act,
                     residual=acc if use_res else None)
        prog.finalize()
        for _ in range(2):
            if use_res:
                acc.copy_(res)
            prog.run()
        ref = want
        if act == "gelu_tanh":
            ref = plain.gelu_tanh(want)
        elif act == "gelu_erf":
            ref = plain.gelu_erf(want)
        if use_res:
            ref = ref + res.double()
        tol = 5e-3 if out_dtype == BF else max(2e-6, 4.0 * math.sqrt(K) * 2.0 ** -24)
        assert rel_err(target.float().cpu(), ref) < tol, (act, out_dtype)
        assert int(e.item()) == 0 and prog._sync.tolist() == [2, 0, 0, 0]     # two launches counted, nothing else left behind


@pytest.mark.parametrize("rows", [1, 7, 16])
@pytest.mark.parametrize("d,F", [(192, 544), (768, 3072), (1600, 6400), (64, 100)])
def test_a_chain_of_operations_each_reading_what_the_one_before_wrote(rows, d, F):
    """embed → LayerNorm product (GELU, bfloat16) → product + residual → RMS product: every operation waits, group by
    group, for the rows that other CTAs write just before (no barrier lies between them), and the weight ring runs
    across the four operations.  Widths that are no multiples of 3 and 6, and an inner width staged in chunks."""
    V, P, N3 = 300, 40, 1000
    F -= F % 32
    wte, wpe = randn(V, d, seed=1, dtype=BF), randn(P, d, seed=2, dtype=BF)
    w1, b1 = randn(F, d, seed=3, dtype=BF, scale=0.2), randn(F, seed=4)
    w2, b2 = randn(d, F, seed=5, dtype=BF, scale=0.2), randn(d, seed=6)
    w3 = randn(N3, d, seed=7, dtype=BF, scale=0.2)
    g1, be1, g3 = randn(d, seed=8) * 0.2 + 1, randn(d, seed=9) * 0.2, randn(d, seed=10) * 0.2 + 1
    tok = torch.randint(0, V, (rows,), generator=g(11), dtype=torch.int32)
    pos = torch.randint(0, P, (rows,), generator=g(12), dtype=torch.int32)
    prog, e = program_for(rows, tokens=tok, pos=pos)
    x = prog.scratch("x", rows, d, torch.float32)          # what an operation hands to the next: flagged rows
    u = prog.scratch("u", rows, F, BF)
    out = torch.full((rows, N3), float("nan"), device=DEV)
    prog.embed(wte.to(DEV), wpe.to(DEV), x)
    prog.product(x, w1.to(DEV), b1.to(DEV), u, norm=("layernorm", g1.to(DEV), be1.to(DEV), 1e-5), act="gelu_tanh")
    prog.product(u, w2.to(DEV), b2.to(DEV), x, residual=x)
    prog.product(x, w3.to(DEV), None, out, norm=("rmsnorm", g3.to(DEV), None, 1e-6))
    prog.finalize()
    runs = []
    for _ in range(3):
        prog.run()
        runs.append(out.cpu().clone())
    x0 = wte.double()[tok.long()] + wpe.double()[pos.long()]
    h1 = plain.layer_norm(x0, g1.double(), be1.double(), 1e-5).to(BF).double()
    uu = plain.gelu_tanh(h1 @ w1.double().T + b1.double()).to(BF).double()
    x1 = x0 + uu @ w2.double().T + b2.double()
    h3 = plain_norm(x1, "rmsnorm", g3.double(), None, 1e-6).to(BF).double()
    want = h3 @ w3.double().T
    assert rel_err(runs[0], want) < 1e-2
    assert torch.equal(runs[0], runs[1]) and torch.equal(runs[0], runs[2])
    assert int(e.item()) == 0


def test_embedding_clamps_and_reports_a_bad_token_and_skips_padding_rows():
    d, V, P = 64, 100, 30
    wte, wpe = randn(V, d, seed=1, dtype=BF), randn(P, d, seed=2, dtype=BF)
    tok = torch.tensor([5, V + 9, 7, 3], dtype=torch.int32)
    pos = torch.tensor([0, 1, 29, 4], dtype=torch.int32)
    slot = torch.tensor([0, 1, 2, -1], dtype=torch.int32)
    prog, e = program_for(4, tokens=tok, slot=slot, pos=pos)
    x = torch.full((4, d), float("nan"), device=DEV)
    prog.embed(wte.to(DEV), wpe.to(DEV), x)
    prog.finalize()
    prog.run()
    assert int(e.item()) == 1
    assert torch.equal(x[0].cpu(), wte[5].float() + wpe[0].float())
    assert torch.equal(x[2].cpu(), wte[7].float() + wpe[29].float())
    assert torch.isfinite(x).all()


def attention_case(H, Hkv, dh, T, C, *, window=0, max_context=1024, k=None, v=None, q=None, scale=None):
    """The last T positions of one context of C tokens as T rows of a decode step (each row a sequence of its own
    that shares the blocks), through a program of one attention operation."""
    q = randn(H, T, dh, seed=30) if q is None else q
    k = randn(Hkv, C, dh, seed=31) if k is None else k
    v = randn(Hkv, C, dh, seed=32) if v is None else v
    q, k, v = (t.to(BF).float() for t in (q, k, v))
    scale = 0.7 / math.sqrt(dh) if scale is None else scale
    kp, vp, blocks = paged(k, v, 40, 21, BF)
    table = torch.full((T + 2, 34), -1, dtype=torch.int32)
    for r in range(T):
        table[r + 1, :blocks.numel()] = blocks
    qkv = torch.zeros(T, H * dh + 5 * 16, dtype=BF)
    qkv[:, 16:16 + H * dh] = q.permute(1, 0, 2).reshape(T, H * dh).to(BF)
    slot = torch.arange(1, T + 1, dtype=torch.int32)
    pos = torch.arange(C - T, C, dtype=torch.int32)
    prog, e = program_for(T, slot=slot, pos=pos, max_context=max_context)
    out = torch.full((T, H * dh), float("nan"), dtype=BF, device=DEV)
    prog.attention(qkv.to(DEV), 16, 0, 0, kp.to(DEV), vp.to(DEV), table.to(DEV), out, n_heads=H, n_kv_heads=Hkv, head_dim=dh,
                   scale=scale, window=window)
    prog.finalize()
    for _ in range(2):
        out.fill_(float("nan"))
        prog.run()
    assert int(e.item()) == 0
    counters = prog.ws._bufs.get("program_counters")
    assert counters is None or int(counters.abs().sum()) == 0
    return out.float().cpu().reshape(T, H, dh).permute(1, 0, 2), plain_attention(q, k, v, scale, window)


@pytest.mark.parametrize("H,Hkv,dh,T,C", [(3, 3, 16, 16, 37), (4, 4, 32, 9, 130), (2, 2, 64, 1, 200), (2, 1, 64, 16, 500),
                                          (1, 1, 128, 5, 70), (5, 5, 256, 3, 66), (12, 12, 64, 8, 1024 - 400), (25, 25, 64, 2, 33),
                                          (6, 2, 32, 4, 2000)])
@pytest.mark.parametrize("max_context", [100, 1024, 4096])
def test_attention_alone(H, Hkv, dh, T, C, max_context):
    got, want = attention_case(H, Hkv, dh, T, C, max_context=max_context)
    assert rel_err(got, want) < 1.5e-2


@pytest.mark.parametrize("far", [0, 31, 32, 255, 256, 511, 639])
@pytest.mark.parametrize("max_context", [64, 2048])
def test_attention_finds_one_far_key_and_respects_a_window(far, max_context):
    H, dh, C = 3, 64, 640
    q, k, v = (t.to(BF).float() for t in (randn(H, 1, dh, seed=66), randn(H, C, dh, seed=67) * 0.1, randn(H, C, dh, seed=68)))
    k[:, far] = (q[:, 0] * 4.0).to(BF).float()
    got, _ = attention_case(H, H, dh, 1, C, q=q, k=k, v=v, scale=1.0, max_context=max_context)
    assert rel_err(got[:, 0], v[:, far]) < 1e-2
    for window in (1, 33, 200, C - far, C - 1 - far):
        if window < 1:
            continue
        got, want = attention_case(H, H, dh, 1, C, q=q, k=k, v=v, scale=1.0, window=window, max_context=max_context)
        assert rel_err(got, want) < 1.5e-2, window


def test_product_writes_keys_and_values_into_the_paged_cache():
    rows, d, Hkv, dh = 6, 128, 2, 32
    N = d + 2 * Hkv * dh
    x = randn(rows, d, seed=1)
    w, b = randn(N, d, seed=2, dtype=BF, scale=0.3), randn(N, seed=3)
    slot = torch.tensor([2, 0, -1, 1, 3, 4], dtype=torch.int32)
    pos = torch.tensor([0, 63, 5, 64, 130, 7], dtype=torch.int32)
    table = torch.full((5, 4), -1, dtype=torch.int32)
    table[0, 0], table[1, 1], table[2, 0], table[3, 2], table[4, 0] = 7, 3, 1, 0, 5
    kc = torch.full((8, Hkv, 64, dh), float("nan"), dtype=BF, device=DEV)
    vc = torch.full((8, Hkv, 64, dh), float("nan"), dtype=BF, device=DEV)
    prog, e = program_for(rows, slot=slot, pos=pos)
    out = torch.empty(rows, N, dtype=BF, device=DEV)
    prog.product(x.to(DEV), w.to(DEV), b.to(DEV), out, kv_scatter=(kc, vc, table.to(DEV), d, d + Hkv * dh, Hkv, dh))
    prog.finalize()
    prog.run()
    assert int(e.item()) == 0
    want = (x.to(BF).double() @ w.double().T + b.double()).to(BF)
    assert rel_err(out.float().cpu(), want.double()) < 5e-3
    written = 0
    for r in range(rows):
        if int(slot[r]) < 0:
            continue
        blk = int(table[int(slot[r]), int(pos[r]) // 64])
        for h in range(Hkv):
            assert torch.equal(kc[blk, h, int(pos[r]) % 64].cpu(), out[r, d + h * dh:d + (h + 1) * dh].cpu())
            assert torch.equal(vc[blk, h, int(pos[r]) % 64].cpu(), out[r, d + (Hkv + h) * dh:d + (Hkv + h + 1) * dh].cpu())
            written += 2 * dh
    assert int(torch.isfinite(kc.float()).sum() + torch.isfinite(vc.float()).sum()) == written   # and nothing else


@pytest.mark.parametrize("H,Hkv,dh,rows,C,window", [(4, 4, 16, 5, 40, 0), (4, 2, 32, 16, 130, 0), (12, 12, 64, 8, 600, 0),
                                                     (2, 1, 128, 3, 200, 50), (5, 5, 64, 4, 65, 1), (2, 2, 256, 2, 64, 0)])
def test_projection_attention_projection_inside_one_program(H, Hkv, dh, rows, C, window):
    """What a mixer emits: q/k/v projection (into flagged rows and the cache) → attention (its newest key and value
    taken from those rows, the earlier ones from the cache; output one segment a head) → output projection.  Every row
    is a sequence of its own at its own position; the cache holds its earlier keys and NaN where the newest belongs."""
    d = 96
    width_q, width_kv = H * dh, Hkv * dh
    N = width_q + 2 * width_kv
    scale = 0.9 / math.sqrt(dh)
    x = randn(rows, d, seed=1)
    wqkv, bqkv = randn(N, d, seed=2, dtype=BF, scale=0.3), randn(N, seed=3)
    wo, bo = randn(d, width_q, seed=4, dtype=BF, scale=0.2), randn(d, seed=5)
    lens = [C - 3 * r for r in range(rows)]                     # tokens each sequence holds before this step
    nb = (C + 64) // 64
    kc = torch.full((rows * nb + 3, Hkv, 64, dh), float("nan"), dtype=BF)
    vc = torch.full((rows * nb + 3, Hkv, 64, dh), float("nan"), dtype=BF)
    table = torch.full((rows + 1, nb + 1), -1, dtype=torch.int32)
    order = torch.randperm(rows * nb + 3, generator=g(9)).tolist()
    past_k = [randn(Hkv, n, dh, seed=20 + r).to(BF) for r, n in enumerate(lens)]
    past_v = [randn(Hkv, n, dh, seed=40 + r).to(BF) for r, n in enumerate(lens)]
    for r, n in enumerate(lens):
        for i in range(n // 64 + 1):
            blk = order.pop()
            table[r + 1, i] = blk
            m = min(64, n - 64 * i)
            if m > 0:
                kc[blk, :, :m] = past_k[r][:, 64 * i:64 * i + m]
                vc[blk, :, :m] = past_v[r][:, 64 * i:64 * i + m]
    slot = torch.arange(1, rows + 1, dtype=torch.int32)
    pos = torch.tensor(lens, dtype=torch.int32)
    prog, e = program_for(rows, slot=slot, pos=pos)
    kc_d, vc_d = kc.to(DEV), vc.to(DEV)
    qkv = prog.scratch("qkv", rows, N, BF)
    merged = prog.scratch("merged", rows, width_q, BF, seg=dh)
    out = torch.full((rows, d), float("nan"), device=DEV)
    prog.product(x.to(DEV), wqkv.to(DEV), bqkv.to(DEV), qkv, kv_scatter=(kc_d, vc_d, table.to(DEV), width_q, width_q + width_kv, Hkv, dh))
    prog.attention(qkv, 0, width_q, width_q + width_kv, kc_d, vc_d, table.to(DEV), merged, n_heads=H, n_kv_heads=Hkv,
                   head_dim=dh, scale=scale, window=window)
    prog.product(merged, wo.to(DEV), bo.to(DEV), out)
    prog.finalize()
    runs = []
    for _ in range(2):
        prog.run()
        runs.append(out.cpu().clone())
    assert int(e.item()) == 0
    proj = (x.to(BF).double() @ wqkv.double().T + bqkv.double()).to(BF)
    held = unpack_flagged(qkv)
    want = torch.zeros(rows, d, dtype=torch.float64)
    for r, n in enumerate(lens):
        q = proj[r, :width_q].reshape(H, 1, dh).float()
        k_new = proj[r, width_q:width_q + width_kv].reshape(Hkv, 1, dh)
        v_new = proj[r, width_q + width_kv:].reshape(Hkv, 1, dh)
        k = torch.cat([past_k[r], k_new], dim=1).float()
        v = torch.cat([past_v[r], v_new], dim=1).float()
        att = plain_attention(q, k, v, scale, window)[:, 0].reshape(-1).to(BF).double()
        want[r] = att @ wo.double().T + bo.double()
        # the newest key and value were also stored for later steps: the very values that attention used
        blk = int(table[r + 1, n // 64])
        assert torch.equal(kc_d[blk, :, n % 64].cpu().reshape(-1), held[r, width_q:width_q + width_kv])
        assert torch.equal(vc_d[blk, :, n % 64].cpu().reshape(-1), held[r, width_q + width_kv:])
    assert rel_err(held.double(), proj.double()) < 5e-3
    assert rel_err(runs[0], want) < 2e-2
    assert torch.equal(runs[0], runs[1])


# ---- whole sessions ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", ["tiny_a", "tiny_b", "tiny_c"])
@pytest.mark.parametrize("use_graph", [False, True])
def test_a_decode_session_runs_as_a_program_and_gives_the_plain_logits(model_dirs, plain_models, name, use_graph):
    from engine_drives import poison
    from vlrf_b200.engine import Engine, StepEntry, load_model
    from vlrf_b200.engine.decode import DecodeSession
    cfg, w = plain_models[name]
    n_pos = cfg["n_positions"]
    lens = [n_pos, n_pos - 37, 70, 33]
    starts = [30, 64, 1, 20]
    reqs = [random_ids(cfg["vocab_size"], n, 900 + i) for i, n in enumerate(lens)]
    truth = [plain.logits_all_positions(cfg, w, ids) for ids in reqs]
    eng = Engine(load_model(model_dirs[name], "bfloat16"), max_tokens=64 * 24)
    poison(eng)
    slots = [eng.start_sequence() for _ in reqs]
    eng.step([StepEntry(s, r[:n], []) for s, r, n in zip(slots, reqs, starts)])
    sess = DecodeSession(eng, slots, use_graph=use_graph, pad_to=8, use_program=True)
    assert sess.program is not None, sess.program_refused
    sess.reserve_ahead(n_pos)
    at = list(starts)
    worst = 0.0
    while any(p < len(r) for p, r in zip(at, reqs)):
        sess.set_tokens([r[min(p, len(r) - 1)] for r, p in zip(reqs, at)])
        lg = sess.step().float().cpu()
        for i, r in enumerate(reqs):
            if at[i] < len(r):
                err = rel_err(lg[i], truth[i][at[i]])
                assert err < TOL_BF16, (i, at[i], err)
                worst = max(worst, err)
                at[i] += 1
                if at[i] == len(r):
                    sess.end_row(i)
    eng.check_device_errors()
    assert sess.kernels_per_step == 1
    for s in slots:
        eng.end_sequence(s)
    eng.cache.check()


def test_a_model_whose_sizes_the_program_refuses_decodes_launch_by_launch(model_dirs):
    from vlrf_b200.engine import Engine, StepEntry, load_model
    from vlrf_b200.engine.decode import DecodeSession
    eng = Engine(load_model(model_dirs["tiny_d"], "bfloat16"), max_tokens=256)     # width 80: no multiple of 32
    slot = eng.start_sequence()
    eng.step([StepEntry(slot, [1, 2, 3], [])])
    sess = DecodeSession(eng, [slot], use_graph=False, use_program=True)
    assert sess.program is None and "K=80" in sess.program_refused
    sess.set_tokens([4])
    assert torch.isfinite(sess.step()).all()
