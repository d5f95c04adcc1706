"""Oracle restatements of goldens the reference only has inline in its check functions, cross-checked against
independent formulations (float64, torch SDPA) and against each other."""
import math

import torch

from oracle import attention, codecs, moe


def _experts(gen, ne=6, h=64, fe=32):
    gw, gs = codecs.random_mxfp4((ne, 2 * fe, h), gen)
    dw, ds = codecs.random_mxfp4((ne, h, fe), gen)
    return gw, gs, dw, ds


def test_experts_decode_against_float64():
    g = torch.Generator().manual_seed(0)
    gw, gs, dw, ds = _experts(g)
    T, H, K, FE = 5, 64, 3, 32
    h2 = torch.randn((T, H), generator=g).to(torch.bfloat16)
    base = (torch.randn((T, H), generator=g) * 0.5).to(torch.bfloat16)
    ids = torch.stack([torch.randperm(6, generator=g)[:K] for _ in range(T)]).to(torch.int32)
    rw = torch.softmax(torch.randn((T, K), generator=g), -1)
    out = moe.experts_decode(h2, base, ids, rw, gw, gs, dw, ds)
    ref = base.double().clone()
    for t in range(T):
        for i in range(K):
            e = int(ids[t, i])
            wc, wd = codecs.dequant_mxfp4(gw[e], gs[e]).double(), codecs.dequant_mxfp4(dw[e], ds[e]).double()
            gu = wc @ h2[t].double()
            ref[t] += rw[t, i].double() * (wd @ (torch.nn.functional.silu(gu[:FE]) * gu[FE:]))
    assert (out.double() - ref).abs().max() / ref.square().mean().sqrt() < 6e-2  # the golden's own bf16 rounding points


def test_slots_and_combine_equal_decode_experts():
    """prefill form (permute -> slots -> combine) reproduces the decode form token by token"""
    g = torch.Generator().manual_seed(1)
    gw, gs, dw, ds = _experts(g)
    T, H, K, G = 9, 64, 2, 4
    h2 = torch.randn((T, H), generator=g).to(torch.bfloat16)
    base = torch.randn((T, H), generator=g).to(torch.bfloat16)
    ids = torch.stack([torch.randperm(6, generator=g)[:K] for _ in range(T)]).to(torch.int32)
    rw = torch.softmax(torch.randn((T, K), generator=g), -1)
    tok, srw, loc, n = moe.permute(ids, rw, G)
    assert n == tok.shape[0] and (tok[:-1, 0] <= tok[1:, 0]).all()
    sout = moe.slots(h2, tok, srw, gw, gs, dw, ds, out_dtype=torch.float32)
    out = moe.combine(base, loc, sout.reshape(-1, H))
    ref = moe.experts_decode(h2, base, ids, rw, gw, gs, dw, ds)
    assert (out.float() - ref.float()).abs().max() <= 2 ** -6 * ref.float().abs().max()
    # unused rows carry weight zero and therefore zero output
    assert (sout.reshape(-1, H)[srw.reshape(-1) == 0] == 0).all()


def test_permute_is_stable_counting_sort():
    ids = torch.tensor([[2, 0], [0, 1], [2, 1], [0, 2]], dtype=torch.int32)
    rw = torch.arange(8).float().reshape(4, 2)
    tok, srw, loc, n = moe.permute(ids, rw, G=2)
    assert tok[:, 0].tolist() == [0, 0, 1, 2, 2]
    assert tok[0, 1:].tolist() == [0, 1] and tok[1, 1].item() == 3  # expert 0: tokens 0, 1, 3 in index order
    assert srw[1, 1].item() == 0.0
    for t in range(4):
        for k in range(2):
            s, j = divmod(int(loc[k, t]), 2)
            assert tok[s, 0] == ids[t, k] and tok[s, 1 + j] == t and srw[s, j] == rw[t, k]


def test_moe_pre_shapes_and_gate():
    g = torch.Generator().manual_seed(3)
    T, H, FS, NE = 4, 64, 32, 16
    x1 = torch.randn((T, H), generator=g).to(torch.bfloat16)
    ln2 = 1 + 0.02 * torch.randn(H, generator=g)
    wg, wu, wd = (torch.randn(s, generator=g) * 0.05 for s in ((FS, H), (FS, H), (H, FS)))
    wr = torch.randn((NE, H), generator=g).to(torch.bfloat16)
    base, h2, logits = moe.moe_pre(x1, ln2, wg, wu, wd, wr, torch.zeros(H, dtype=torch.bfloat16))
    assert base.dtype == torch.bfloat16 and h2.shape == (T, H) and logits.dtype == torch.float32
    # zero shared-expert gate weight -> sigmoid(0) = 1/2 of the shared expert
    h = h2.float()
    sh = moe.bf(torch.nn.functional.silu(moe.bf(h @ wg.T)) * moe.bf(h @ wu.T)) @ wd.T
    assert torch.equal(base, (x1.float() + 0.5 * sh).to(torch.bfloat16))


def _paged_case(g, ctxs, P=8, HKV=2, D=16, HQ=4, fp8=False):
    n_pages = [max(1, math.ceil(c / P)) if c else 0 for c in ctxs]
    total = sum(n_pages) + 3
    cache = torch.randn((total, 2, P, HKV, D), generator=g).to(torch.bfloat16)
    perm = torch.randperm(total, generator=g).to(torch.int32)
    indptr = torch.tensor([0] + list(torch.tensor(n_pages).cumsum(0)), dtype=torch.int32)
    indices = perm[: sum(n_pages)].contiguous()
    last = torch.tensor([(c - (n - 1) * P) if n else 0 for c, n in zip(ctxs, n_pages)], dtype=torch.int32)
    q = torch.randn((len(ctxs), HQ, D), generator=g).to(torch.bfloat16)
    return q, cache, indptr, indices, last


def test_paged_decode_against_sdpa_noncontiguous_pages():
    g = torch.Generator().manual_seed(4)
    ctxs = [1, 8, 9, 37, 0]
    q, cache, indptr, indices, last = _paged_case(g, ctxs)
    out = attention.paged_decode(q, cache, indptr, indices, last)
    assert attention.valid_kv_len(indptr, last, 8).tolist() == ctxs
    for b, c in enumerate(ctxs):
        if c == 0:
            assert (out[b] == 0).all()
            continue
        k, v = attention.gather_kv(cache, indptr, indices, last, b)
        ref = attention.sdpa_decode_reference(q[b].float(), k, v)
        torch.testing.assert_close(out[b].float(), ref, rtol=2e-2, atol=2e-2)


def test_paged_decode_current_token_and_cache_write():
    g = torch.Generator().manual_seed(5)
    ctxs = [0, 5, 16]  # history lengths; 16 = exactly two full pages: the new row opens a third page
    P = 8
    q, cache, _, _, _ = _paged_case(g, [c + 1 for c in ctxs])
    n_pages = [c // P + 1 for c in ctxs]
    indptr = torch.tensor([0, *torch.tensor(n_pages).cumsum(0).tolist()], dtype=torch.int32)
    indices = torch.randperm(cache.shape[0], generator=g)[: sum(n_pages)].to(torch.int32)
    last = torch.tensor([c % P for c in ctxs], dtype=torch.int32)  # history rows in the last page
    k_new = torch.randn((3, 2, 16), generator=g).to(torch.bfloat16)
    v_new = torch.randn((3, 2, 16), generator=g).to(torch.bfloat16)
    out = attention.paged_decode(q, cache, indptr, indices, last, k_new=k_new, v_new=v_new)
    loc = torch.stack([indices[indptr[1:].long() - 1], last], 1)
    before = cache.clone()
    attention.store_paged_kv(cache, loc, k_new, v_new)
    out2 = attention.paged_decode(q, cache, indptr, indices, last + 1)
    assert torch.equal(out.view(torch.int16), out2.view(torch.int16))
    before[loc[:, 0].long(), :, loc[:, 1].long()] = cache[loc[:, 0].long(), :, loc[:, 1].long()]
    assert torch.equal(before.view(torch.int16), cache.view(torch.int16))  # only the addressed rows changed


def test_fp8_kv_forms():
    g = torch.Generator().manual_seed(6)
    x = torch.randn((5, 2, 16), generator=g).to(torch.bfloat16)
    c = codecs.kv_quant_fp8(x)
    assert c.dtype == torch.float8_e4m3fn
    assert (codecs.kv_dequant_fp8(c) - x.float()).abs().max() < 0.07 * x.float().abs().max()
    sc = x.float().abs().amax((0, 2)) / 448
    c2 = codecs.kv_quant_fp8(x, sc)
    assert (codecs.kv_dequant_fp8(c2, sc) - x.float()).abs().max() < 0.07 * x.float().abs().max()


def test_fp8_rowwise_gemm():
    g = torch.Generator().manual_seed(7)
    w = torch.randn((24, 64), generator=g) * 0.02
    q8, s = codecs.quant_fp8_rowwise(w)
    x = torch.randn((3, 64), generator=g).to(torch.bfloat16)
    out = codecs.fp8_gemm(x, q8, torch.ones(3), s)
    ref = x.double() @ codecs.dequant_fp8_rowwise(q8, s).double().T
    assert (out.double() - ref).abs().max() / ref.square().mean().sqrt() < 3e-2


def test_paged_prefill_equals_decode_token_by_token():
    """the prefill golden on T tokens = the decode golden applied to each token with the history it sees"""
    g = torch.Generator().manual_seed(8)
    P, hist, T = 8, 5, 7
    q1, cache, indptr, indices, last = _paged_case(g, [hist + T], P=P)
    q = torch.randn((T, 4, 16), generator=g).to(torch.bfloat16)
    out = attention.paged_prefill(q, cache, torch.tensor([0, T], dtype=torch.int32), indptr, indices, last)
    for i in range(T):
        n = hist + i + 1
        npg = (n + P - 1) // P
        dec = attention.paged_decode(q[i:i + 1], cache, torch.tensor([0, npg], dtype=torch.int32), indices[:npg],
                                     torch.tensor([n - (npg - 1) * P], dtype=torch.int32))
        assert torch.equal(out[i].view(torch.int16), dec[0].view(torch.int16))
