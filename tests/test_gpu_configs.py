"""GPU parity at the sizes the hot path is quoted on (configurations 2, 3 and 4, and the benchmark's own attention
launch), against the CPU oracle on identical seeded inputs.

The big tensors (KV caches of one to two GB) are generated on the device from a seeded generator; the oracle is run on
a fixed sample of sequences whose pages are copied back bit for bit, so both sides see the same bytes.  Every check
goes through assert_parity, which records the strict figure max|err| / RMS.
"""
import threading

import pytest
import torch

from conftest import assert_parity, rel_rms_err
from oracle import attention as oattn, gdn as ogdn, moe as omoe
from _cases import dequant_shared, gdn_step_case, moe_case

pytestmark = pytest.mark.gpu
P, HKV, HQ, D = 64, 2, 16, 256


@pytest.fixture(scope="module")
def q35():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    import ax_dsl_kernels_b200 as m
    yield m
    assert m.device_status() == 0


def _paged_on_device(ctxs, seed, fp8):
    """configuration-2 inputs on the GPU: cache [pages, 2, 64, 2, 256] ~ N(0, 1), physical pages a random permutation,
    q ~ N(0, 1); FP8 variant e4m3(x / scale_h) with scale_h = amax_h / 448 per (K | V, head)"""
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(seed)
    n_pages = [(c + P - 1) // P for c in ctxs]
    total = sum(n_pages)
    cache = torch.empty((total, 2, P, HKV, D), dtype=torch.bfloat16, device=dev)
    for i in range(0, total, 2048):
        cache[i:i + 2048] = torch.randn((min(2048, total - i), 2, P, HKV, D), generator=g, device=dev).to(torch.bfloat16)
    indices = torch.randperm(total, generator=g, device=dev).to(torch.int32)
    indptr = torch.tensor([0, *torch.tensor(n_pages).cumsum(0).tolist()], dtype=torch.int32, device=dev)
    last = torch.tensor([c - (n - 1) * P for c, n in zip(ctxs, n_pages)], dtype=torch.int32, device=dev)
    q = torch.randn((len(ctxs), HQ, D), generator=g, device=dev).to(torch.bfloat16)
    kv_scale = None
    if fp8:
        amax = torch.zeros((2, HKV), device=dev)
        for i in range(0, total, 2048):
            amax = torch.maximum(amax, cache[i:i + 2048].float().abs().amax((0, 2, 4)))
        kv_scale = (amax / 448.0).contiguous()
        c8 = torch.empty(cache.shape, dtype=torch.float8_e4m3fn, device=dev)
        for i in range(0, total, 2048):
            c8[i:i + 2048] = (cache[i:i + 2048].float() / kv_scale.reshape(1, 2, 1, HKV, 1)).to(torch.float8_e4m3fn)
        cache = c8
    return q, cache, indptr, indices, last, kv_scale


def _oracle_on_sample(q, cache, indptr, indices, last, kv_scale, sample, sm_scale):
    """the CPU golden on the sampled sequences: their pages copied back in table order (same bytes, compact ids)"""
    refs = []
    for b in sample:
        rows = indices[int(indptr[b]):int(indptr[b + 1])].long()
        sub = cache[rows].cpu()
        n = sub.shape[0]
        refs.append(oattn.paged_decode(q[b:b + 1].cpu(), sub, torch.tensor([0, n], dtype=torch.int32),
                                       torch.arange(n, dtype=torch.int32), last[b:b + 1].cpu(), sm_scale=sm_scale,
                                       kv_scale=None if kv_scale is None else kv_scale.cpu()))
    return torch.cat(refs, 0)


@pytest.mark.parametrize("fp8", [False, True], ids=["bf16", "fp8_per_head_scale"])
def test_config2_batch64_contexts_1024_to_16384(q35, fp8):
    """configuration 2 exactly: batch 64, seed 1, contexts uniform in [1024, 16384], page 64, permuted pages,
    softmax scale 1/16; the oracle runs on 8 sequences including the longest and the shortest"""
    ctxs = torch.randint(1024, 16385, (64,), generator=torch.Generator().manual_seed(1)).tolist()
    q, cache, indptr, indices, last, kvs = _paged_on_device(ctxs, seed=1, fp8=fp8)
    out = torch.full_like(q, float("nan"))
    q35.paged_attention_decode(q, cache, indptr, indices, last, out, sm_scale=1.0 / 16, kv_scale=kvs)
    assert torch.isfinite(out).all()
    order = sorted(range(64), key=lambda b: ctxs[b])
    sample = sorted({order[0], order[-1], 0, 9, 23, 37, 50, 63})
    ref = _oracle_on_sample(q, cache, indptr, indices, last, kvs, sample, 1.0 / 16)
    assert_parity(out[sample].cpu(), ref, per_seq=True)


def test_benchmark_attention_launch_batch64_context16384(q35):
    """the benchmark's own attention launch (64 sequences of exactly 16384 tokens, 2.1 GB of bf16 KV): 4 sequences
    against the oracle"""
    ctxs = [16384] * 64
    q, cache, indptr, indices, last, _ = _paged_on_device(ctxs, seed=1000, fp8=False)
    out = torch.full_like(q, float("nan"))
    q35.paged_attention_decode(q, cache, indptr, indices, last, out, sm_scale=1.0 / 16)
    assert torch.isfinite(out).all()
    sample = [0, 21, 42, 63]
    ref = _oracle_on_sample(q, cache, indptr, indices, last, None, sample, 1.0 / 16)
    assert_parity(out[sample].cpu(), ref, per_seq=True)


def test_config3_decode_batch64_32_value_heads(q35):
    """configuration 3, decode: 64 sequences x 32 value / 16 key heads, fp32 state ~ N(0, 0.03^2), all of it against
    the golden recurrence"""
    q, k, v, g, beta, s0 = gdn_step_case(B=64, NK=16, NV=32, seed=2)
    o_ref, s_ref = ogdn.recurrent(q, k, v, g, beta, s0)
    o, s1 = q35.gdn_recurrent_step(q[:, 0].cuda(), k[:, 0].cuda(), v[:, 0].cuda(), g[:, 0].cuda(), beta[:, 0].cuda(),
                                   s0.cuda(), state_out=torch.empty_like(s0).cuda())
    assert_parity(o.cpu(), o_ref[:, 0])
    torch.testing.assert_close(s1.cpu(), s_ref, rtol=0, atol=3e-3)  # the reference's temporal-state tolerance


def test_config3_prefill_16384_tokens_two_heads_against_recurrence(q35):
    """configuration 3, prefill: 16384 tokens, 32 value / 16 key heads, chunk 64, zero initial state.  The kernel runs
    all heads; value heads 5 and 30 (key heads 2 and 15) are compared with the token recurrence: the unrounded float64
    form (strict 2e-2) and the reference's bf16-rounding golden, whose own distance to float64 is recorded beside it."""
    T, NK, NV = 16384, 16, 32
    g = torch.Generator().manual_seed(2)
    q = (ogdn.l2norm(torch.randn((1, T, NK, 128), generator=g)).float() * 128 ** -0.5).to(torch.bfloat16)
    k = ogdn.l2norm(torch.randn((1, T, NK, 128), generator=g))
    v = torch.randn((1, T, NV, 128), generator=g).to(torch.bfloat16)
    beta = torch.sigmoid(torch.randn((1, T, NV), generator=g)).to(torch.bfloat16)
    gg = -torch.nn.functional.softplus(torch.randn((1, T, NV), generator=g))
    s0 = torch.zeros((1, NV, 128, 128))
    o, s1 = q35.gdn_chunk_prefill(q.cuda(), k.cuda(), v.cuda(), gg.cuda(), beta.cuda(), s0.cuda())
    vh = [5, 30]
    kh = [h // (NV // NK) for h in vh]
    sub = (q[:, :, kh].contiguous(), k[:, :, kh].contiguous(), v[:, :, vh].contiguous(), gg[:, :, vh].contiguous(),
           beta[:, :, vh].contiguous(), s0[:, vh].contiguous())
    o64, s64 = ogdn.recurrent_f64(*sub)
    og, sg = ogdn.recurrent(*sub)
    got = o[:, :, vh].cpu()
    d_golden = rel_rms_err(og.double(), o64)
    # recorded first, judged after: the kernel against float64, and against the golden with the golden's own distance
    # to float64 added to the limit
    lim = max(2e-2, 1.5 * d_golden)
    r64 = assert_parity(got.double(), o64, tol=lim, name="config3 prefill 16384: kernel vs float64 recurrence "
                        f"(the bf16-rounding golden itself is {d_golden:.3e} away)")
    rg = assert_parity(got, og, tol=lim + d_golden, name="config3 prefill 16384: kernel vs bf16 golden")
    assert r64["strict_max_err_over_rms"] <= lim and rg["strict_max_err_over_rms"] <= lim + d_golden
    assert (s1[:, vh].cpu().double() - s64).abs().max().item() <= max(4e-3, 1.5 * (sg.double() - s64).abs().max().item())


def test_config4_decode_moe_block_64_tokens_256_experts(q35):
    """configuration 4, decode: one moe_block call on 64 tokens, 256 experts top-8 + shared expert, seed 3; routing
    ids bit-exact, output within tolerance of the golden"""
    T = 64
    x1, w = moe_case(T, NE=256, seed=3)
    sg, su, sd = dequant_shared(w)
    ref, ids, rw, logits = omoe.moe_block(x1, w["ln2"], sg, su, sd, w["w_router"], w["w_shg"], w["e_gw"], w["e_gs"],
                                          w["e_dw"], w["e_ds"], 8)
    wd = {k: v.cuda() for k, v in w.items()}
    out, gids, grw, glog = q35.moe_block(x1.cuda(), wd, 8)
    assert torch.equal(gids.cpu(), ids)
    torch.testing.assert_close(grw.cpu(), rw, rtol=1e-4, atol=1e-6)
    assert_parity(out.cpu(), ref, bf16_step=True)
    out2, _, _, _ = q35.moe_block(x1.cuda(), wd, 8, overlap=False)
    assert_parity(out2.cpu(), ref, bf16_step=True, name="config4 decode, moe_pre -> route -> moe_experts sequence")
    q35.prepare_moe_weights(wd)  # one-call decode form
    out3, gids3, _, _ = q35.moe_block(x1.cuda(), wd, 8)
    assert torch.equal(gids3.cpu(), ids)
    assert_parity(out3.cpu(), ref, bf16_step=True, name="config4 decode, one-call moe.block")


# ------------------------------------------------------------------------------------------------ one-call decode block
def _tile_ref(s, paired):
    """the tiled scale layout stated in words: block (plane, tile, K / 128) of 512 bytes, byte [l * 16 + c * 4 + b] =
    scale of tile row l + 32 c for inputs 128 s + 32 b ..; a paired tile = 64 gate rows then 64 up rows"""
    planes, rows, KB = s.shape
    tiles, KS = rows // 128, KB // 4
    m = torch.arange(128)
    t = torch.arange(tiles).reshape(-1, 1)
    row = torch.where(m < 64, t * 64 + m, rows // 2 + t * 64 + (m - 64)) if paired else t * 128 + m
    src = s[:, row]                                                  # [planes, tiles, 128 (m = l + 32 c), KB]
    src = src.reshape(planes, tiles, 4, 32, KS, 4)                   # c, l, stage, b
    return src.permute(0, 1, 4, 3, 2, 5).reshape(planes, tiles, KS, 512).contiguous()


@pytest.mark.parametrize("paired", [True, False])
def test_tile_scales_layout_bit_exact(q35, paired):
    g = torch.Generator().manual_seed(3)
    s = torch.randint(0, 256, (3, 256, 16), generator=g, dtype=torch.int32).to(torch.uint8)
    got = q35.tile_scales(s.cuda(), paired).cpu()
    assert torch.equal(got.reshape(-1), _tile_ref(s, paired).reshape(-1))


@pytest.mark.parametrize("T,NE", [(1, 32), (7, 32), (33, 64), (64, 256)])
def test_moe_block_one_call_decode_form(q35, T, NE):
    """role moe.block (norm + router, route + plan, quantise, ONE persistent gate-up + down kernel with the shared
    expert as a group, combine) against the golden and against the role-by-role path on the same weights"""
    x1, w = moe_case(T, NE=NE, seed=100 + T)
    w["ln2"] = 1 + 0.05 * torch.randn(2048, generator=torch.Generator().manual_seed(T))
    sg, su, sd = dequant_shared(w)
    ref, ids, rw, logits = omoe.moe_block(x1, w["ln2"], sg, su, sd, w["w_router"], w["w_shg"], w["e_gw"], w["e_gs"],
                                          w["e_dw"], w["e_ds"], 8)
    wd = {k: v.cuda() for k, v in w.items()}
    old, oids, _, ologits = q35.moe_block(x1.cuda(), wd, 8)
    old, oids, ologits = old.clone(), oids.clone(), ologits.clone()
    q35.prepare_moe_weights(wd)
    out = torch.full_like(x1, float("nan")).cuda()
    out, gids, grw, glog = q35.moe_block(x1.cuda(), wd, 8, out)
    assert q35.device_status() == 0
    assert torch.equal(glog, ologits)          # same order of operations as the role-by-role router: same bits
    assert torch.equal(gids, oids) and torch.equal(gids.cpu(), ids)
    torch.testing.assert_close(grw.cpu(), rw, rtol=1e-4, atol=1e-6)
    assert torch.isfinite(out).all()
    assert_parity(out.cpu(), ref, bf16_step=True)
    assert_parity(out.cpu(), old.cpu(), bf16_step=True, name=f"moe.block vs role-by-role path, T={T}")
    out2 = torch.empty_like(out)
    q35.moe_block(x1.cuda(), wd, 8, out2)
    assert torch.equal(out.view(torch.int16), out2.view(torch.int16))  # run-to-run bitwise determinism


@pytest.mark.parametrize("T,NE,lo,hi", [(7, 16, 0, 16), (64, 32, 8, 24), (512, 256, 96, 128)])
def test_moe_experts_tiled_scales_decode_form(q35, T, NE, lo, hi):
    """moe.experts with tiled scales (the per-rank step of expert parallelism: gathered tokens, global ids, this rank's
    planes): the one-kernel form must agree with the role's general form on base / out and on partial sums, and a
    sample of tokens with the golden"""
    g = torch.Generator().manual_seed(T + NE)
    h2 = torch.randn((T, 2048), generator=g).to(torch.bfloat16)
    base = (torch.randn((T, 2048), generator=g) * 0.5).to(torch.bfloat16)
    ids, rw = omoe.route(torch.randn((T, NE), generator=g), 8)
    if T == 7:
        ids[3, 5] = ids[3, 1]  # an expert listed twice
    from oracle import codecs
    e_gw, e_gs = codecs.random_mxfp4((hi - lo, 1024, 2048), g, -8, 0)
    e_dw, e_ds = codecs.random_mxfp4((hi - lo, 2048, 512), g, -8, 0)
    dev = [t.cuda() for t in (h2, base, ids, rw, e_gw, e_gs, e_dw, e_ds)]
    gs_t, ds_t = q35.tile_scales(dev[5], True), q35.tile_scales(dev[7], False)
    eb = torch.tensor([lo], dtype=torch.int32).cuda()
    p_old = torch.full((T, 2048), float("nan")).cuda()
    p_new = torch.full((T, 2048), float("nan")).cuda()
    common = dict(h2=dev[0], ids=dev[2], rw=dev[3], e_gw=dev[4], e_gs=dev[5], e_dw=dev[6], e_ds=dev[7], expert_base=eb)
    q35.run("moe.experts", partial_out=p_old, **common)
    q35.run("moe.experts", partial_out=p_new, e_gs_tiled=gs_t, e_ds_tiled=ds_t, **common)
    assert q35.device_status() == 0
    assert torch.isfinite(p_new).all()
    assert_parity(p_new.cpu(), p_old.cpu(), bf16_step=True, name=f"moe.experts tiled vs general, partial sums, T={T}")
    if lo == 0 and hi == NE:
        ref = omoe.experts_decode(h2, base, ids, rw, e_gw, e_gs, e_dw, e_ds)
        out = torch.full_like(h2, float("nan")).cuda()
        q35.moe_experts(*dev, out, e_gs_tiled=gs_t, e_ds_tiled=ds_t)
        assert_parity(out.cpu(), ref, bf16_step=True)
    else:
        zero = torch.zeros((1, 2048), dtype=torch.bfloat16)
        for t in range(0, T, max(1, T // 6)):
            ref = torch.zeros(2048)
            for i in range(8):
                e = int(ids[t, i]) - lo
                if 0 <= e < hi - lo:
                    ref += rw[t, i] * omoe.experts_decode(h2[t:t + 1], zero, torch.tensor([[e]], dtype=torch.int32),
                                                          torch.ones((1, 1)), e_gw, e_gs, e_dw, e_ds).float()[0]
            if ref.abs().max() > 0:
                assert_parity(p_new[t].cpu(), ref, bf16_step=True)
            else:
                assert (p_new[t] == 0).all()


# ------------------------------------------------------------------------------------------------ router near-ties
def test_route_logits_one_and_two_ulps_apart_around_kth_place(q35):
    """The kernel orders experts by their LOGITS (descending, exact ties to the lower id); the reference's host router
    sorts the fp32 softmax PROBABILITIES.  Two logits one ulp apart can round to the same probability, and then the
    probability sort takes the lower id where the logit order takes the larger logit.  Checked here: the kernel follows
    the logit order exactly, and wherever its ids differ from the probability-sorted golden the experts involved have
    EQUAL golden probabilities (so either choice is a valid top-k of the golden's own numbers)."""
    T, NE, K = 32, 256, 8
    g = torch.Generator().manual_seed(77)
    logits = torch.randn((T, NE), generator=g)
    for t in range(T):
        srt = torch.sort(logits[t], descending=True)
        kth = srt.values[K - 1].clone()
        lo_id, hi_id = sorted((int(srt.indices[K - 1]), int(srt.indices[K])))
        ulps = 1 + (t % 2)
        bits = kth.view(torch.int32)
        nxt = (bits + (ulps if kth > 0 else -ulps)).view(torch.float32)  # `ulps` steps larger
        logits[t, lo_id] = kth        # the lower id holds the SMALLER logit ...
        logits[t, hi_id] = nxt        # ... the higher id the larger one, `ulps` apart
    ids, rw = q35.route(logits.cuda(), K)
    by_logit = torch.sort(logits, dim=-1, descending=True, stable=True).indices[:, :K].to(torch.int32)
    assert torch.equal(ids.cpu(), by_logit)
    gold_ids, gold_rw = omoe.route(logits, K)
    pr = torch.softmax(logits, -1)
    differing = 0
    for t in range(T):
        a, b = set(ids[t].tolist()), set(gold_ids[t].tolist())
        if a != b:
            differing += 1
            pa = sorted(float(pr[t, e]) for e in a - b)
            pb = sorted(float(pr[t, e]) for e in b - a)
            assert pa == pb, "ids differ from the golden on experts whose golden probabilities are not equal"
    torch.testing.assert_close(rw.cpu().sort(-1).values, gold_rw.sort(-1).values, rtol=1e-5, atol=1e-7)
    print(f"rows whose ids differ from the probability-sorted golden: {differing} of {T}")


# ------------------------------------------------------------------------------------------------ duplicate ids
@pytest.mark.parametrize("T,K,NE", [(6, 4, 16), (640, 8, 16)], ids=["one_cta_plan", "three_kernel_plan"])
def test_moe_experts_token_listing_an_expert_twice(q35, T, K, NE):
    """ids is a caller tensor: a token may list an expert twice.  The golden adds rw * d for every listed pair; the
    kernels give the expert one row weighted by the sum (both routing-plan forms)."""
    from _cases import moe_case as mk
    _, w = mk(1, NE=NE, seed=5)
    g = torch.Generator().manual_seed(T)
    h2 = torch.randn((T, 2048), generator=g).to(torch.bfloat16)
    base = (torch.randn((T, 2048), generator=g) * 0.5).to(torch.bfloat16)
    ids, rw = omoe.route(torch.randn((T, NE), generator=g), K)
    ids[2, K - 1] = ids[2, 0]
    ids[T - 1, 1] = ids[T - 1, 2]
    sample = sorted({0, 2, T // 2, T - 1})
    ref = omoe.experts_decode(h2[sample], base[sample], ids[sample], rw[sample], w["e_gw"], w["e_gs"], w["e_dw"], w["e_ds"])
    out = torch.full_like(h2, float("nan")).cuda()
    q35.moe_experts(h2.cuda(), base.cuda(), ids.cuda(), rw.cuda(), w["e_gw"].cuda(), w["e_gs"].cuda(), w["e_dw"].cuda(),
                    w["e_ds"].cuda(), out)
    assert torch.isfinite(out).all()
    assert_parity(out.cpu()[sample], ref, bf16_step=True)


def test_qk_prep_with_mrope_rows(q35, golden):
    """multimodal RoPE: rows built from position_ids [3, T] (sections 11, 11, 10, interleaved) through attn.qk_prep
    against the golden's q / k norm + NeoX rotation with the reference-mixed tables"""
    from oracle.moe import rmsnorm
    f = golden("mrope")
    T, HQn, HKVn, Dn = 9, 4, 1, 256
    g = torch.Generator().manual_seed(6)
    qg = torch.randn((T, HQn, 2 * Dn), generator=g).to(torch.bfloat16)
    k = torch.randn((T, HKVn, Dn), generator=g).to(torch.bfloat16)
    qn, kn = 1 + 0.1 * torch.randn(Dn, generator=g), 1 + 0.1 * torch.randn(Dn, generator=g)
    cos, sin = q35.mrope_cos_sin(f["position_ids"], 64, 1e7, (11, 11, 10), True, device="cuda")
    q_out = torch.empty((T, HQn, Dn), dtype=torch.bfloat16, device="cuda")
    k_out = torch.empty((T, HKVn, Dn), dtype=torch.bfloat16, device="cuda")
    gate = torch.empty_like(q_out)
    q35.run("attn.qk_prep", qg=qg.cuda(), k=k.cuda(), q_norm=qn.cuda(), k_norm=kn.cuda(), cos=cos, sin=sin, q_out=q_out,
            k_out=k_out, gate_out=gate)
    rc, rs = f["cos_interleaved"], f["sin_interleaved"]
    q_ref = oattn.rope_neox(rmsnorm(qg[..., :Dn], qn), rc[:, None, :], rs[:, None, :], 64)
    k_ref = oattn.rope_neox(rmsnorm(k, kn), rc[:, None, :], rs[:, None, :], 64)
    assert_parity(q_out.cpu(), q_ref)
    assert_parity(k_out.cpu(), k_ref)
    assert torch.equal(gate.cpu(), qg[..., Dn:])


def test_attention_split_over_eight_ranks_emulated_on_one_gpu(q35):
    """configuration-2 heads (16 q / 2 kv) over 8 ranks: four ranks share a KV head and split every sequence's pages;
    each rank's unnormalised partial (attn.paged_decode with part_* outputs) and attn.lse_merge, run here one rank
    after the other on this GPU, against the unsplit role and the oracle"""
    from ax_dsl_kernels_b200 import parallel
    from _cases import paged_case
    world = 8
    q, cache, indptr, indices, last, _ = paged_case([1000, 3, 64, 0, 2500, 129], seed=5)
    B, HQn, Dn = q.shape
    full = q35.paged_attention_decode(q.cuda(), cache.cuda(), indptr.cuda(), indices.cuda(), last.cuda())
    parts = {}
    gathered = torch.full((world, B, 8, Dn + 2), float("nan"), device="cuda")  # what the all-gather would deliver
    for rank in range(world):
        pl = parallel.attention_split(HQn, 2, world, rank)
        ip, ix, lp = parallel.split_page_table(indptr, indices, last, 64, pl["share"], pl["shares"])
        ql = q[:, pl["q0"]:pl["q1"]].contiguous().cuda()
        pm = torch.full((B, 8), float("nan"), device="cuda")
        pln = torch.full((B, 8), float("nan"), device="cuda")
        po = torch.full((B, 8, Dn), float("nan"), device="cuda")
        q35.run("attn.paged_decode", q=ql, paged_kv_cache=cache[:, :, :, pl["kv0"]:pl["kv1"]].contiguous().cuda(),
                indptr=ip.cuda(), indices=ix.cuda(), last_page_len=lp.cuda(), part_m=pm, part_l=pln, part_o=po)
        parts[(pl["kv0"], pl["share"])] = (pm, pln, po)
        # the one-message form of the same launch: o | m | l written straight into the rank's slot
        q35.run("attn.paged_decode", q=ql, paged_kv_cache=cache[:, :, :, pl["kv0"]:pl["kv1"]].contiguous().cuda(),
                indptr=ip.cuda(), indices=ix.cuda(), last_page_len=lp.cuda(), part_packed=gathered[rank])
        assert torch.equal(gathered[rank][..., :Dn], po) and torch.equal(gathered[rank][..., Dn], pm)
        assert torch.equal(gathered[rank][..., Dn + 1], pln)
    S = world // 2
    pm = torch.stack([torch.cat([parts[(kv, s)][0] for kv in range(2)], 1) for s in range(S)])
    pln = torch.stack([torch.cat([parts[(kv, s)][1] for kv in range(2)], 1) for s in range(S)])
    po = torch.stack([torch.cat([parts[(kv, s)][2] for kv in range(2)], 1) for s in range(S)])
    out = torch.full_like(full, float("nan"))
    q35.run("attn.lse_merge", part_m=pm.contiguous(), part_l=pln.contiguous(), part_o=po.contiguous(), out=out)
    out2 = torch.full_like(full, float("nan"))
    q35.run("attn.lse_merge", packed=gathered, out=out2)
    assert torch.equal(out, out2)
    ref = oattn.paged_decode(q, cache, indptr, indices, last)
    nz = [0, 1, 2, 4, 5]
    assert (out[3] == 0).all()
    assert_parity(out.cpu()[nz], ref[nz], per_seq=True)
    assert_parity(out.cpu()[nz], full.cpu()[nz], per_seq=True, name="attention split over 8 ranks vs the unsplit role")


def test_qwen3_moe_one_call_contract_by_the_reference_names(q35):
    """qwen3_moe(inputs, output): the sgl line's entry point bound by its own names (w_norm in the zero-centred form,
    separate gate / up planes, shared_expert_mlp_*); same kernels as moe_block, so the same bits, and parity with the
    oracle block.  Contract violations raise ValueError as the reference's wrapper does."""
    T = 64
    x1, w = moe_case(T, seed=3)
    dw = {k: v.cuda() for k, v in w.items()}
    ref_out = q35.moe_block(x1.cuda(), q35.prepare_moe_weights(dict(dw)), 8)[0].clone()
    FE = w["e_gw"].shape[1] // 2
    inputs = dict(x=x1.cuda().reshape(4, 16, -1), w_norm=(w["ln2"] - 1).cuda(), w_route=dw["w_router"],
                  w_gate=dw["e_gw"][:, :FE].contiguous(), w_scale_gate=dw["e_gs"][:, :FE].contiguous(),
                  w_up=dw["e_gw"][:, FE:].contiguous(), w_scale_up=dw["e_gs"][:, FE:].contiguous(),
                  w_down=dw["e_dw"], w_scale_down=dw["e_ds"], shared_expert_gate=dw["w_shg"].float(),
                  w_shared_expert_mlp_gate=dw["w_gate"], w_scale_shared_expert_mlp_gate=dw["s_gate"],
                  w_shared_expert_mlp_up=dw["w_up"], w_scale_shared_expert_mlp_up=dw["s_up"],
                  w_shared_expert_mlp_down=dw["w_down"], w_scale_shared_expert_mlp_down=dw["s_down"],
                  top_k=8, norm_topk_prob=True)
    out = q35.qwen3_moe(inputs, mode="expert_parallel", core_num=4)
    assert out.shape == (4, 16, x1.shape[1])
    assert torch.equal(out.reshape(T, -1), ref_out)
    fused = dict(inputs, w_gate=dw["e_gw"], w_scale_gate=dw["e_gs"], w_up=None, w_scale_up=None)
    out2 = torch.full_like(out, float("nan"))
    assert q35.qwen3_moe(fused, out2) is out2 and torch.equal(out2, out)
    sg, su, sd = dequant_shared(w)
    oref = omoe.moe_block(x1, w["ln2"], sg, su, sd, w["w_router"], w["w_shg"], w["e_gw"], w["e_gs"], w["e_dw"],
                          w["e_ds"], 8)[0]
    assert_parity(out.reshape(T, -1).cpu(), oref, bf16_step=True)
    with pytest.raises(ValueError):
        q35.qwen3_moe(inputs, mode="data_parallel")
    with pytest.raises(ValueError):
        q35.qwen3_moe(dict(inputs, norm_topk_prob=False))
    with pytest.raises(ValueError):
        q35.qwen3_moe(inputs, torch.empty((T, 7), dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(ValueError):  # NVFP4 scales (E4M3 per 16) are refused, not misread
        q35.qwen3_moe(dict(fused, w_scale_gate=torch.zeros((256, 2 * FE, 128), dtype=torch.float8_e4m3fn, device="cuda"),
                           w_norm=(w["ln2"] - 1).cuda().clone()))


@pytest.mark.parametrize("T", [1, 64, 200])
def test_moe_front_one_launch_head_of_the_block(q35, T):
    """moe.front (RMSNorm + router + gate dot + softmax + top-k in one launch) against the role sequence
    moe.norm_router -> moe.route and against the oracle's routing: ids bit-exact, rows and weights equal or within
    fp32 rounding of the sum order"""
    x1, w = moe_case(T, NE=256, seed=50 + T)
    w["ln2"] = 1 + 0.05 * torch.randn(2048, generator=torch.Generator().manual_seed(T))
    d = {k: v.cuda() for k, v in w.items()}
    x = x1.cuda()
    mk = lambda *s, dt=torch.float32: torch.full(s, float("nan") if dt != torch.int32 else -7, dtype=dt, device="cuda")  # noqa: E731
    h2a, lga, gta = mk(T, 2048, dt=torch.bfloat16), mk(T, 256), mk(T)
    q35.run("moe.norm_router", x1=x, ln2=d["ln2"], w_router=d["w_router"], w_shg=d["w_shg"].reshape(-1), h2_out=h2a,
            logits_out=lga, gate_out=gta)
    ida, rwa = q35.route(lga, 8)
    h2b, lgb, gtb, idb, rwb = mk(T, 2048, dt=torch.bfloat16), mk(T, 256), mk(T), mk(T, 8, dt=torch.int32), mk(T, 8)
    q35.run("moe.front", x1=x, ln2=d["ln2"], w_router=d["w_router"], w_shg=d["w_shg"].reshape(-1), h2_out=h2b,
            logits_out=lgb, gate_out=gtb, ids=idb, rw=rwb)
    assert torch.equal(h2a, h2b)
    assert (lga - lgb).abs().max().item() <= 1e-4 * lga.abs().max().item()
    assert (gta - gtb).abs().max().item() <= 1e-4 * max(1.0, gta.abs().max().item())
    oids, orw = omoe.route(lgb.cpu(), 8)
    assert torch.equal(idb.cpu(), oids)
    assert (rwb.cpu() - orw).abs().max().item() <= 1e-5
    same = (ida == idb).all(1)
    assert same.float().mean().item() >= 0.98  # (the two kernels' logits differ in the last bits: a near-tie may flip)
    assert (rwa[same] - rwb[same]).abs().max().item() <= 1e-4


def test_expert_parallel_exchange_kernels_two_ranks_emulated_on_one_gpu(q35):
    """ep.publish / ep.wait / ep.reduce with two ranks' exchange buffers in this one GPU's memory, the ranks run one
    after the other: rows, ids and weights land in slice `rank` of BOTH buffers, the flags carry the exchange count,
    and every rank's output is its dense part plus both ranks' partial sums of its tokens.  No kernel is made to wait
    here: a rank publishes with no_wait, ep.wait runs once both have published, and the test raises the done flags the
    other rank's reduce would raise (it plays that rank) before each reduce."""
    N, T, H, K = 2, 8, 512, 4
    g = torch.Generator().manual_seed(41)
    al = lambda n: (n + 255) // 256 * 256  # noqa: E731
    o_h2 = 1024
    o_ids = o_h2 + al(N * T * H * 2)
    o_rw = o_ids + al(N * T * K * 4)
    o_par = o_rw + al(N * T * K * 4)
    total = o_par + al(N * T * H * 4)
    bufs = [torch.zeros(total, dtype=torch.uint8, device="cuda") for _ in range(N)]
    peers = torch.tensor([b.data_ptr() for b in bufs], dtype=torch.int64, device="cuda").view(torch.uint8)
    view = lambda b, off, n, dt, shape: b[off:off + n].view(dt).view(shape)  # noqa: E731
    regs = [dict(h2_all=view(b, o_h2, N * T * H * 2, torch.bfloat16, (N * T, H)),
                 ids_all=view(b, o_ids, N * T * K * 4, torch.int32, (N * T, K)),
                 rw_all=view(b, o_rw, N * T * K * 4, torch.float32, (N * T, K)),
                 partial=view(b, o_par, N * T * H * 4, torch.float32, (N * T, H))) for b in bufs]
    ranks = [torch.tensor([r], dtype=torch.int32, device="cuda") for r in range(N)]
    flag = torch.ones(1, dtype=torch.int32, device="cuda")
    for step in (1, 2):  # two exchanges: the flags count them
        h2 = [torch.randn((T, H), generator=g).to(torch.bfloat16).cuda() for _ in range(N)]
        ids = [torch.randint(0, 64, (T, K), generator=g, dtype=torch.int32).cuda() for _ in range(N)]
        rw = [torch.rand((T, K), generator=g).cuda() for _ in range(N)]
        for r in range(N):
            q35.run("ep.publish", h2=h2[r], ids=ids[r], rw=rw[r], peers=peers, rank=ranks[r], exchange=bufs[r],
                    no_wait=flag, h2_all=regs[r]["h2_all"], ids_all=regs[r]["ids_all"], rw_all=regs[r]["rw_all"])
        for r in range(N):
            q35.run("ep.wait", peers=peers, rank=ranks[r], exchange=bufs[r])
        for r in range(N):
            hdr = bufs[r][:1024].view(torch.int32)
            assert int(hdr[0]) == step and hdr[64:64 + N].tolist() == [step] * N  # epoch, gather flags
            assert torch.equal(regs[r]["h2_all"], torch.cat(h2)) and torch.equal(regs[r]["ids_all"], torch.cat(ids))
            assert torch.equal(regs[r]["rw_all"], torch.cat(rw))
        part = [torch.randn((N * T, H), generator=g).cuda() for _ in range(N)]
        base = [torch.randn((T, H), generator=g).to(torch.bfloat16).cuda() for _ in range(N)]
        for r in range(N):
            regs[r]["partial"].copy_(part[r])
            bufs[r][:1024].view(torch.int32)[128:128 + N] = step  # the done flags the ranks' reduces would raise
        for r in range(N):
            out = torch.full((T, H), float("nan"), dtype=torch.bfloat16, device="cuda")
            q35.run("ep.reduce", base=base[r], partial=regs[r]["partial"], peers=peers, rank=ranks[r], exchange=bufs[r],
                    out=out)
            ref = base[r].float()
            for p in range(N):
                ref = ref + part[p][r * T:(r + 1) * T]
            assert torch.equal(out, ref.to(torch.bfloat16))
    assert q35.device_status() == 0
    before = bufs[0].clone()
    q35.run("ep.wait", peers=peers, rank=ranks[1], exchange=bufs[0])  # peers[rank] must be this rank's own buffer:
    assert q35.device_status() == 0x4000 and torch.equal(bufs[0], before)  # recorded, nothing touched
    assert q35.device_status() == 0


# ------------------------------------------------------------------------------------------------ robustness
def test_bounded_wait_reports_instead_of_hanging(q35):
    """a device-side wait that can never complete (a barrier nothing arrives at, 4096 polls) gives up, sets the
    wait-timeout bit of the status word and returns; the library works normally afterwards"""
    polls = torch.tensor([4096], dtype=torch.int32, device="cuda")
    result = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    q35.run("debug.wait_probe", polls=polls, result=result)
    torch.cuda.synchronize()
    assert int(result.item()) == 1
    st = q35.device_status()
    assert st & 4, st
    assert q35.device_status() == 0
    ids, _ = q35.route(torch.randn((4, 64), device="cuda"), 4)
    assert ids.shape == (4, 4) and q35.device_status() == 0


def test_two_host_threads_own_streams_bitwise_equal(q35):
    """two host threads call in at the same time, each on its own stream with its own scratch: both must produce the
    bytes a single-threaded call produces (the library keeps no state that one call could disturb for another)"""
    from _cases import paged_case
    q, cache, indptr, indices, last, _ = [t.cuda() if t is not None else None for t in paged_case([300, 17, 1500, 64])]
    ref = q35.paged_attention_decode(q, cache, indptr, indices, last, sm_scale=1.0 / 16)
    torch.cuda.synchronize()
    outs, errs = [None, None], []

    def work(i):
        try:
            s = torch.cuda.Stream()
            with torch.cuda.stream(s):
                for _ in range(20):
                    o = q35.paged_attention_decode(q, cache, indptr, indices, last, sm_scale=1.0 / 16)
                s.synchronize()
            outs[i] = o
        except Exception as e:  # noqa: BLE001
            errs.append(e)

    th = [threading.Thread(target=work, args=(i,)) for i in range(2)]
    [t.start() for t in th]
    [t.join() for t in th]
    assert not errs, errs
    for o in outs:
        assert torch.equal(o.view(torch.int16), ref.view(torch.int16))


def test_oneshot_all_reduce_two_ranks_emulated_on_one_gpu(q35):
    """ar.oneshot with two ranks' exchange buffers in this GPU's memory.  A rank's kernel waits for the other's flag, so
    the ranks cannot run one after the other for real; the test plays the other rank instead: before rank r's launch it
    writes the other rank's addend into r's slot and raises that flag by hand.  Checked: the sum (rank order), the
    store of r's addend into BOTH buffers, the flags, and the alternation of the two slot sets."""
    N, n = 2, 8 * 512
    slot = (n * 4 + 255) // 256 * 256
    bufs = [torch.zeros(1024 + 2 * N * slot, dtype=torch.uint8, device="cuda") for _ in range(N)]
    peers = torch.tensor([b.data_ptr() for b in bufs], dtype=torch.int64, device="cuda").view(torch.uint8)
    ranks = [torch.tensor([r], dtype=torch.int32, device="cuda") for r in range(N)]
    g = torch.Generator().manual_seed(3)
    for epoch in (1, 2, 3):
        par = (epoch & 1) * N * slot
        xs = [torch.randn(n, generator=g).cuda() for _ in range(N)]
        for r in range(N):
            o = 1 - r
            # the other rank's part of this exchange, as its kernel would have left it in r's buffer
            bufs[r][1024 + par + o * slot:1024 + par + o * slot + n * 4].view(torch.float32).copy_(xs[o])
            bufs[r][:1024].view(torch.int32)[64 + o] = epoch
            out = torch.full((n,), float("nan"), device="cuda")
            q35.run("ar.oneshot", x=xs[r], peers=peers, rank=ranks[r], exchange=bufs[r], out=out)
            assert torch.equal(out, xs[0] + xs[1])
            hdr = bufs[r][:1024].view(torch.int32)
            assert int(hdr[0]) == epoch and int(hdr[64 + r]) == epoch
            for b in bufs:  # r's addend reached both buffers
                assert torch.equal(b[1024 + par + r * slot:1024 + par + r * slot + n * 4].view(torch.float32), xs[r])
    assert q35.device_status() == 0


def test_exchange_wait_runs_out_and_reports_instead_of_hanging(q35):
    """A rank whose peer never publishes: ep.wait polls a flag that nothing raises, gives up after its poll budget
    (about a second), records the wait site in the status word and returns; the next wait gives up at once while the
    bit is still set, and after the host has read (and cleared) the status the exchange works again."""
    import time
    N, T, H, K = 2, 8, 512, 4
    al = lambda n: (n + 255) // 256 * 256  # noqa: E731
    o_h2, o_ids = 1024, 1024 + al(N * T * H * 2)
    o_rw = o_ids + al(N * T * K * 4)
    total = o_rw + al(N * T * K * 4)
    bufs = [torch.zeros(total, dtype=torch.uint8, device="cuda") for _ in range(N)]
    peers = torch.tensor([b.data_ptr() for b in bufs], dtype=torch.int64, device="cuda").view(torch.uint8)
    rank0 = torch.tensor([0], dtype=torch.int32, device="cuda")
    rank1 = torch.tensor([1], dtype=torch.int32, device="cuda")
    flag = torch.ones(1, dtype=torch.int32, device="cuda")
    view = lambda b, off, n, dt, shape: b[off:off + n].view(dt).view(shape)  # noqa: E731
    regs = lambda b: dict(h2_all=view(b, o_h2, N * T * H * 2, torch.bfloat16, (N * T, H)),  # noqa: E731
                          ids_all=view(b, o_ids, N * T * K * 4, torch.int32, (N * T, K)),
                          rw_all=view(b, o_rw, N * T * K * 4, torch.float32, (N * T, K)))
    h2 = torch.zeros((T, H), dtype=torch.bfloat16, device="cuda")
    ids = torch.zeros((T, K), dtype=torch.int32, device="cuda")
    rw = torch.zeros((T, K), device="cuda")
    assert q35.device_status() == 0
    q35.run("ep.publish", h2=h2, ids=ids, rw=rw, peers=peers, rank=rank0, exchange=bufs[0], no_wait=flag, **regs(bufs[0]))
    q35.run("ep.wait", peers=peers, rank=rank0, exchange=bufs[0])  # rank 1 never publishes
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    q35.run("ep.wait", peers=peers, rank=rank0, exchange=bufs[0])
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 0.5  # gives up at once while the timeout is on record
    st = q35.device_status()
    assert st & 0x4 and st & 0x800, hex(st)
    assert q35.device_status() == 0
    q35.run("ep.publish", h2=h2, ids=ids, rw=rw, peers=peers, rank=rank1, exchange=bufs[1], no_wait=flag, **regs(bufs[1]))
    q35.run("ep.wait", peers=peers, rank=rank0, exchange=bufs[0])  # now both have published exchange 1
    torch.cuda.synchronize()
    assert q35.device_status() == 0
