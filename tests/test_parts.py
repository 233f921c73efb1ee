"""Each part alone against the plain implementation's function for it, at sizes of its own."""
import math

import pytest
import torch

import plain_gpt2 as plain
from conftest import rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def randn(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale


def make_ctx(cache, seqs, dtype, ws=None):
    """A StepContext for sequences [(slot, first position, n tokens)], blocks reserved."""
    from vlrf_b200.parts import StepContext, Workspace
    tok_slot, tok_pos, starts = [], [], [0]
    for slot, p0, n in seqs:
        cache.reserve(slot, p0 + n)
        tok_slot += [slot] * n
        tok_pos += list(range(p0, p0 + n))
        starts.append(starts[-1] + n)
    cache.sync_tables()
    T = len(tok_slot)
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device=DEV)  # noqa: E731
    return StepContext(n_tokens=T, tokens=i32([0] * T), tok_slot=i32(tok_slot), tok_pos=i32(tok_pos), n_seqs=len(seqs),
                       seq_slot=i32([s[0] for s in seqs]), seq_start=i32(starts), seq_pos0=i32([s[1] for s in seqs]),
                       max_new=max(s[2] for s in seqs), max_context=max(s[1] + s[2] for s in seqs),
                       logit_rows=i32([]), n_logit_rows=0, act_dtype=dtype,
                       dev_err=torch.zeros(1, dtype=torch.int32, device=DEV), ws=ws or Workspace(DEV),
                       host_seq_slots=[s[0] for s in seqs], host_seq_lens=[s[2] for s in seqs], host_seq_pos0=[s[1] for s in seqs])


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("H,Hkv,dh", [(5, 5, 16), (4, 2, 48)])
def test_attention_part_whole_then_continued(dtype, tol, H, Hkv, dh):
    """x += attention(h) for two sequences of unequal lengths in one step, then one more token each;
    compared with the plain attention on the whole sequences."""
    from vlrf_b200.cache import SequenceCache
    from vlrf_b200.parts import CausalSelfAttention
    d = 80
    wq = H * dh + 2 * Hkv * dh
    w_qkv, b_qkv = randn(wq, d, seed=1, scale=0.2), randn(wq, seed=2, scale=0.1)
    w_out, b_out = randn(d, H * dh, seed=3, scale=0.2), randn(d, seed=4, scale=0.1)
    scale = 0.9 / math.sqrt(dh)
    cast = lambda t: t.to(dtype).to(DEV)  # noqa: E731
    att = CausalSelfAttention(cast(w_qkv), b_qkv.to(DEV), cast(w_out), b_out.to(DEV), n_heads=H, n_kv_heads=Hkv,
                              head_dim=dh, scale=scale)
    cache = SequenceCache([att.cache_need()], max_tokens=512, max_seq_len=256, dtype=dtype, device=DEV)
    cache.view(0).k.fill_(float("nan")); cache.view(0).v.fill_(float("nan"))
    lens = [70, 9]
    hs = [randn(n + 1, d, seed=10 + i) for i, n in enumerate(lens)]
    xs = [randn(n + 1, d, seed=20 + i) for i, n in enumerate(lens)]
    wd = lambda t: t.to(dtype).double()  # noqa: E731  (what the part sees)

    def truth(h):
        qkv = wd(h) @ wd(w_qkv).T + b_qkv.double()
        q, k, v = qkv[:, :H * dh], qkv[:, H * dh:H * dh + Hkv * dh], qkv[:, H * dh + Hkv * dh:]
        qh, kh, vh = plain.split_heads(q, H), plain.split_heads(k, Hkv), plain.split_heads(v, Hkv)
        rep = H // Hkv
        o = plain.merge_heads(plain.causal_attention(qh, kh.repeat_interleave(rep, 0), vh.repeat_interleave(rep, 0), scale))
        return o @ wd(w_out).T + b_out.double()

    want = [x.double() + truth(h) for x, h in zip(xs, hs)]
    slots = [cache.acquire(), cache.acquire()]
    # step 1: all but the last token of each sequence, as one flat batch
    ctx = make_ctx(cache, [(slots[0], 0, lens[0]), (slots[1], 0, lens[1])], dtype)
    h = torch.cat([hs[0][:-1], hs[1][:-1]]).to(dtype).to(DEV)
    x = torch.cat([xs[0][:-1], xs[1][:-1]]).to(DEV)
    att.forward(h, x, ctx, cache.view(0))
    for s, n in zip(slots, lens):
        cache.advance(s, n)
    got = x.cpu()
    assert rel_err(got[:lens[0]], want[0][:-1]) < tol and rel_err(got[lens[0]:], want[1][:-1]) < tol
    # step 2: the last token of each, order of the batch swapped
    ctx = make_ctx(cache, [(slots[1], lens[1], 1), (slots[0], lens[0], 1)], dtype, ctx.ws)
    h = torch.stack([hs[1][-1], hs[0][-1]]).to(dtype).to(DEV)
    x = torch.stack([xs[1][-1], xs[0][-1]]).to(DEV)
    att.forward(h, x, ctx, cache.view(0))
    got = x.cpu()
    assert rel_err(got[0], want[1][-1]) < tol and rel_err(got[1], want[0][-1]) < tol
    assert int(ctx.dev_err.item()) == 0


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("act", ["gelu_tanh", "gelu_erf"])
def test_dense_mlp(dtype, tol, act):
    from vlrf_b200.parts import DenseMLP, Workspace
    d, F, T = 48, 200, 19
    w1, b1, w2, b2 = randn(F, d, seed=1, scale=0.3), randn(F, seed=2), randn(d, F, seed=3, scale=0.3), randn(d, seed=4)
    h, x = randn(T, d, seed=5), randn(T, d, seed=6)
    mlp = DenseMLP(w1.to(dtype).to(DEV), b1.to(DEV), w2.to(dtype).to(DEV), b2.to(DEV), activation=act)

    class Ctx:
        n_tokens, act_dtype, ws = T, dtype, Workspace(DEV)

    xd = x.clone().to(DEV)
    mlp.forward(h.to(dtype).to(DEV), xd, Ctx)
    wd = lambda t: t.to(dtype).double()  # noqa: E731
    f = plain.gelu_tanh if act == "gelu_tanh" else plain.gelu_erf
    want = x.double() + f(wd(h) @ wd(w1).T + b1.double()) @ wd(w2).T + b2.double()
    assert rel_err(xd.cpu(), want) < tol
    with pytest.raises(ValueError, match="activation"):
        DenseMLP(w1, b1, w2, b2, activation="relu")


def test_layernorm_part_and_embedding_and_head():
    from vlrf_b200.parts import LayerNorm, LearnedAbsolutePositions, LMHead, TokenEmbedding, Workspace
    d, V, P, T = 48, 130, 40, 11
    gamma, beta = randn(d, seed=1) + 1, randn(d, seed=2)
    x = randn(T, d, seed=3) * 2
    ln = LayerNorm(gamma.to(DEV), beta.to(DEV), 1e-4)
    out = torch.empty(T, d, device=DEV)
    ln(x.to(DEV), out)
    assert rel_err(out.cpu(), plain.layer_norm(x.double(), gamma.double(), beta.double(), 1e-4)) < 2e-6
    wte, wpe = randn(V, d, seed=4), randn(P, d, seed=5)
    emb = TokenEmbedding(wte.to(DEV), LearnedAbsolutePositions(wpe.to(DEV)))
    tok = torch.randint(0, V, (T,), generator=torch.Generator().manual_seed(6), dtype=torch.int32)
    pos = torch.tensor([0, 1, 2, 3, 4, 5, 6, 0, 1, 38, 39], dtype=torch.int32)

    class Ctx:
        tokens, tok_pos, dev_err, ws = tok.to(DEV), pos.to(DEV), torch.zeros(1, dtype=torch.int32, device=DEV), Workspace(DEV)

    xe = torch.empty(T, d, device=DEV)
    emb(Ctx, xe)
    want = torch.cat([plain.add_learned_positions(plain.embed_tokens(wte.double(), tok[:7].tolist()), wpe.double(), 0),
                      plain.add_learned_positions(plain.embed_tokens(wte.double(), tok[7:9].tolist()), wpe.double(), 0),
                      plain.add_learned_positions(plain.embed_tokens(wte.double(), tok[9:].tolist()), wpe.double(), 38)])
    assert rel_err(xe.cpu(), want) < 1e-6
    head = LMHead(wte.to(DEV))
    lg = torch.empty(T, V, device=DEV)
    head(out, lg, T)
    assert rel_err(lg.cpu(), out.cpu().double() @ wte.double().T) < 2e-6


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 3e-2)])
def test_pre_norm_block(dtype, tol):
    """One whole block on one sequence against the plain block()."""
    from vlrf_b200.cache import SequenceCache
    from vlrf_b200.parts import CausalSelfAttention, DenseMLP, LayerNorm, PreNormBlock
    d, H, F, T = 48, 3, 112, 23
    cfg = dict(n_embd=d, n_head=H, layer_norm_epsilon=1e-4, activation_function="gelu", scale_attn_by_inverse_layer_idx=True)
    names = {"ln_1.weight": (d,), "ln_1.bias": (d,), "attn.c_attn.weight": (d, 3 * d), "attn.c_attn.bias": (3 * d,),
             "attn.c_proj.weight": (d, d), "attn.c_proj.bias": (d,), "ln_2.weight": (d,), "ln_2.bias": (d,),
             "mlp.c_fc.weight": (d, F), "mlp.c_fc.bias": (F,), "mlp.c_proj.weight": (F, d), "mlp.c_proj.bias": (d,)}
    w = {}
    for i, (n, shape) in enumerate(names.items()):
        t = randn(*shape, seed=30 + i, scale=0.3)
        if n.endswith("weight") and len(shape) == 1:
            t = t + 1
        w["h.2." + n] = t.to(dtype).float() if len(shape) == 2 else t
    mat = lambda n: w["h.2." + n].t().contiguous().to(dtype).to(DEV)  # noqa: E731
    vec = lambda n: w["h.2." + n].to(DEV)  # noqa: E731
    scale = 1 / math.sqrt(d // H) / 3.0
    blk = PreNormBlock(
        LayerNorm(vec("ln_1.weight"), vec("ln_1.bias"), 1e-4),
        CausalSelfAttention(mat("attn.c_attn.weight"), vec("attn.c_attn.bias"), mat("attn.c_proj.weight"),
                            vec("attn.c_proj.bias"), n_heads=H, n_kv_heads=H, head_dim=d // H, scale=scale),
        LayerNorm(vec("ln_2.weight"), vec("ln_2.bias"), 1e-4),
        DenseMLP(mat("mlp.c_fc.weight"), vec("mlp.c_fc.bias"), mat("mlp.c_proj.weight"), vec("mlp.c_proj.bias"),
                 activation="gelu_erf"))
    cache = SequenceCache([blk.cache_need()], max_tokens=64, max_seq_len=64, dtype=dtype, device=DEV)
    slot = cache.acquire()
    x = randn(T, d, seed=50)
    xd = x.clone().to(DEV)
    blk.forward(xd, make_ctx(cache, [(slot, 0, T)], dtype), cache.view(0))
    want = plain.block(x.double(), {k: v.double() for k, v in w.items()}, 2, cfg)
    assert rel_err(xd.cpu(), want) < tol
