"""The decode-attention entry point that allocates nothing (vlrf_attn_decode_noalloc).

Some users of the kernel library cannot call cudaMalloc where they call attention: they are in a loop
that must never touch the allocator, their memory plan is fixed up front, or they are handed only inputs
and outputs.  For them the library carries the scratch memory of the split-context attention inside itself.
This test calls that entry point the way such a user would — through its exported C symbol, with raw
pointers — twice in a row, and checks each result against the ordinary entry point (which takes the
scratch from the caller) and against the plain attention, within the tolerance the other kernel tests use;
then a third call of a smaller shape with another split count, which finds the scratch as the larger calls
left it.  It is collected last, so a run that stops at the first failure has already run everything else;
it also passes when run alone.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _entry_point():
    from vlrf_b200.csrc import library
    fn = library().vlrf_attn_decode_noalloc
    p, i, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn.argtypes = [p, i, i, i, p, p, p, i, p, p, p, i, i, i, i, i, i, f, i, i, p, p]
    fn.restype = ctypes.c_int
    return fn


def _case(dtype, rows, H, Hkv, dh, ctx, seed):
    g = torch.Generator().manual_seed(seed)
    n_blocks_seq = (ctx + 63) // 64
    nb = rows * n_blocks_seq + 3
    kc = torch.randn(nb, Hkv, 64, dh, generator=g).to(dtype).to(DEV)
    vc = torch.randn(nb, Hkv, 64, dh, generator=g).to(dtype).to(DEV)
    perm = torch.randperm(nb, generator=g)[:rows * n_blocks_seq].to(torch.int32)
    table = perm.view(rows, n_blocks_seq).contiguous().to(DEV)
    slot = torch.arange(rows, dtype=torch.int32, device=DEV)
    pos = torch.randint(ctx // 2, ctx, (rows,), generator=g, dtype=torch.int32).to(DEV)
    qkv = torch.randn(rows, (H + 2 * Hkv) * dh, generator=g).to(dtype).to(DEV)
    return kc, vc, table, slot, pos, qkv


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, 1.5e-2), (torch.float32, 2e-5)])
@pytest.mark.parametrize("rows,H,Hkv,dh,ctx,n_split", [(8, 12, 12, 64, 700, 4), (3, 6, 2, 48, 130, 2), (5, 4, 4, 128, 300, 8)])
def test_no_alloc_entry_point_matches_the_ordinary_one(dtype, tol, rows, H, Hkv, dh, ctx, n_split):
    from vlrf_b200.csrc import library, ops
    fn = _entry_point()
    scale = 1.0 / math.sqrt(dh)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    stream = torch.cuda.current_stream().cuda_stream
    shapes = [(rows, H, Hkv, dh, ctx, n_split)] * 2 + [(max(1, rows // 2), H, Hkv, dh, max(65, ctx // 3), max(1, n_split - 1))]
    for call, (rows, H, Hkv, dh, ctx, n_split) in enumerate(shapes):   # calls in a row share the built-in scratch
        kc, vc, table, slot, pos, qkv = _case(dtype, rows, H, Hkv, dh, ctx, 100 + call)
        want = torch.full((rows, H * dh), float("nan"), dtype=dtype, device=DEV)
        partials = torch.empty(rows * H * n_split * (dh + 2), device=DEV)
        counters = torch.zeros(rows * H, dtype=torch.int32, device=DEV)
        ops.attention_decode(qkv, 0, kc, vc, table, slot, pos, want, rows, H, Hkv, dh, scale, 0, n_split, partials,
                             counters, err)
        got = torch.full((rows, H * dh), float("nan"), dtype=dtype, device=DEV)
        status = fn(qkv.data_ptr(), ops.dtype_code(dtype), qkv.shape[1], 0, kc.data_ptr(), vc.data_ptr(),
                    table.data_ptr(), table.shape[1], slot.data_ptr(), pos.data_ptr(), got.data_ptr(), got.shape[1],
                    rows, H, Hkv, dh, 64, scale, 0, n_split, err.data_ptr(), stream)
        assert status == 0, library().vlrf_last_error().decode()
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all()
        diff = (got.float() - want.float()).abs().max() / want.float().abs().max()
        assert float(diff) < tol, (call, float(diff))
        # and against the plain attention on the same keys and values (not only against the other entry point)
        import plain_gpt2 as plain
        for r in range(rows):
            n = int(pos[r]) + 1
            blocks = table[r].cpu().tolist()
            k = torch.cat([kc[b].cpu().double() for b in blocks], dim=1)[:, :n]
            v = torch.cat([vc[b].cpu().double() for b in blocks], dim=1)[:, :n]
            rep = H // Hkv
            q = torch.zeros(H, n, dh, dtype=torch.float64)
            q[:, n - 1] = qkv[r, :H * dh].cpu().double().view(H, dh)
            ref = plain.causal_attention(q, k.repeat_interleave(rep, 0), v.repeat_interleave(rep, 0), scale)[:, n - 1]
            err_plain = (got[r].cpu().double().view(H, dh) - ref).abs().max() / ref.abs().max()
            assert float(err_plain) < tol, (call, r, float(err_plain))
    assert int(err.item()) == 0


def test_no_alloc_entry_point_refuses_what_exceeds_its_scratch():
    from vlrf_b200.csrc import library
    fn = _entry_point()
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    dummy = torch.zeros(16, device=DEV)
    args = lambda rows, H, dh, split: (dummy.data_ptr(), 1, 3 * H * dh, 0, dummy.data_ptr(), dummy.data_ptr(),   # noqa: E731
                                       dummy.data_ptr(), 1, dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), H * dh,
                                       rows, H, H, dh, 64, 1.0, 0, split, err.data_ptr(), 0)
    assert fn(*args(64, 64, 64, 2)) != 0                   # 4,096 (row, head) pairs
    assert "2048" in library().vlrf_last_error().decode()
    assert fn(*args(64, 32, 128, 16)) != 0                 # partials beyond the built-in array
    assert "scratch" in library().vlrf_last_error().decode()
