"""Sublayers and the hybrid stack (GDN / gated attention / dense SwiGLU with FP8 per-row weights) through the host
layer functions against the CPU oracle stack, configuration-1 style at a reduced width."""
import pytest
import torch

from conftest import assert_parity, rel_rms_err
from oracle import attention as oattn, gdn as ogdn, stack as ostack
from _cases import stack_case

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def q35():
    assert torch.cuda.is_available()
    import ax_dsl_kernels_b200 as m
    yield m
    assert m.device_status() == 0


def to_dev(ws):
    return [{k: v.cuda() for k, v in w.items()} for w in ws]


def cosine(a, b):
    return torch.nn.functional.cosine_similarity(a.flatten().double(), b.flatten().double(), dim=0).item()


@pytest.mark.parametrize("T", [1, 70])
def test_gdn_sublayer(q35, T):
    kw, ow = stack_case("g", seed=3)
    g = torch.Generator().manual_seed(T)
    x = (torch.randn((1, T, 512), generator=g) * 0.5).to(torch.bfloat16)
    res = (torch.randn((1, T, 512), generator=g) * 0.5).to(torch.bfloat16)
    s0 = torch.randn((1, 4, 128, 128), generator=g) * 0.03
    cq, ck, cv = ((torch.randn((1, 3, wd), generator=g) * 0.03).to(torch.bfloat16) for wd in (256, 256, 512))
    ref, s_ref, c_ref = ogdn.gdn_sublayer(x, res, ow[0], s0, torch.cat((cq, ck, cv), -1))
    fused, s1, conv = q35.layers.gdn(x.cuda(), res.cuda(), to_dev(kw)[0], s0.cuda(), (cq.cuda(), ck.cuda(), cv.cuda()))
    # the new conv-state rows are projection outputs: equal up to a bf16 rounding step
    assert_parity(torch.cat([c.cpu() for c in conv], -1), c_ref)
    assert rel_rms_err(fused.cpu(), ref) <= (2e-2 if T == 1 else 5e-2)
    torch.testing.assert_close(s1.cpu(), s_ref, rtol=0, atol=4e-3)


def test_dense_mlp(q35):
    kw, ow = stack_case("a", seed=5)
    g = torch.Generator().manual_seed(1)
    x1 = torch.randn((9, 512), generator=g).to(torch.bfloat16)
    ref = ostack.dense_mlp(x1, ow[0]["ln2"], ow[0]["w_gate"], ow[0]["w_up"], ow[0]["w_down"])
    out = q35.layers.mlp_residual(x1.cuda(), to_dev(kw)[0])
    assert_parity(out.cpu(), ref)


def test_attention_sublayer_decode_and_prefill(q35):
    kw, ow = stack_case("a", seed=7)
    cfg = dict(heads=4, kv_heads=1, head_dim=128)
    g = torch.Generator().manual_seed(2)
    P, T = 64, 90
    cache = torch.zeros((4, 2, P, 1, 128), dtype=torch.bfloat16)
    gcache = cache.cuda()
    indices = torch.tensor([2, 0, 3, 1], dtype=torch.int32)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32)  # noqa: E731
    x = (torch.randn((T, 512), generator=g) * 0.5).to(torch.bfloat16)
    cos, sin = oattn.rope_cos_sin(torch.arange(T), 32, 1e7)
    ref = ostack.attn_sublayer(x, ow[0], cache, i32([0, 2]), indices, i32([T - P]), cos, sin, rot=32, qo_indptr=i32([0, T]),
                               **cfg)
    dw = to_dev(kw)[0]
    out = q35.layers.attention(x.cuda(), dw, cos.cuda(), sin.cuda(), gcache, i32([0, 2]).cuda(), indices.cuda(),
                               i32([T - P]).cuda(), qo_indptr=i32([0, T]).cuda(), **cfg)
    assert_parity(out.cpu(), ref)
    assert rel_rms_err(gcache.cpu(), cache) <= 2e-2
    # one decode token on top of the prefilled cache
    xd = (torch.randn((1, 512), generator=g) * 0.5).to(torch.bfloat16)
    cosd, sind = oattn.rope_cos_sin(torch.tensor([T]), 32, 1e7)
    loc = i32([[int(indices[T // P]), T % P]])
    refd = ostack.attn_sublayer(xd, ow[0], cache, i32([0, T // P + 1]), indices, i32([T % P]), cosd, sind, rot=32,
                                cache_location=loc, **cfg)
    outd = q35.layers.attention(xd.cuda(), dw, cosd.cuda(), sind.cuda(), gcache, i32([0, T // P + 1]).cuda(),
                                indices.cuda(), i32([T % P]).cuda(), cache_location=loc.cuda(), **cfg)
    assert_parity(outd.cpu(), refd)


def test_hybrid_stack_prefill_then_decode(q35):
    """g g g a stack: prefill of 70 tokens, then 3 decode steps; per-step outputs against the CPU oracle stack
    (the reference's gate for stacks is a cosine on the hidden states, models/qwen35_2b/whole/src/q35_step.py:533)"""
    kinds = "ggga"
    kw, ow = stack_case(kinds, seed=11)
    cfg = dict(heads=4, kv_heads=1, head_dim=128, rot=32, theta=1e7, page_size=64, max_tokens=256)
    ref_stack = ostack.HybridStack(ow, kinds, **cfg)
    gpu_stack = q35.layers.HybridStack(to_dev(kw), kinds, **cfg)
    g = torch.Generator().manual_seed(4)
    x = (torch.randn((70, 512), generator=g) * 0.05).to(torch.bfloat16)
    ref = ref_stack.forward(x)
    out = gpu_stack.forward(x.cuda())
    assert cosine(out.cpu().float(), ref.float()) >= 0.999
    assert rel_rms_err(out.cpu(), ref) <= 0.1
    for step in range(3):
        xd = (torch.randn((1, 512), generator=g) * 0.05).to(torch.bfloat16)
        ref, out = ref_stack.forward(xd), gpu_stack.forward(xd.cuda())
        assert cosine(out.cpu().float(), ref.float()) >= 0.999, step
    assert gpu_stack.pos == ref_stack.pos == 73


def test_configuration1_stack_full_shape(q35):
    """Configuration 1: hidden 2048, 8 layers (3 GDN : 1 gated attention), 16 q / 2 kv heads of 256, RoPE theta 1e7 on
    64 channels, GDN 16 key / 16 value heads of 128, FFN 6144, FP8 E4M3 per-row weights N(0, 0.02), batch 1,
    512-token prefill then 64 decode steps, seed 0."""
    kinds = "gggaggga"
    kw, ow = stack_case(kinds, H=2048, F=6144, heads=16, kv_heads=2, head_dim=256, NK=16, NV=16, DV=128, seed=0)
    cfg = dict(heads=16, kv_heads=2, head_dim=256, rot=64, theta=1e7, page_size=64, max_tokens=640)
    ref_stack = ostack.HybridStack(ow, kinds, **cfg)
    gpu_stack = q35.layers.HybridStack(to_dev(kw), kinds, **cfg)
    g = torch.Generator().manual_seed(0)
    emb = (torch.randn((576, 2048), generator=g) * 0.05).to(torch.bfloat16)
    ref, out = ref_stack.forward(emb[:512]), gpu_stack.forward(emb[:512].cuda())
    assert cosine(out.cpu().float(), ref.float()) >= 0.999
    worst = 1.0
    for t in range(512, 576):
        ref, out = ref_stack.forward(emb[t:t + 1]), gpu_stack.forward(emb[t:t + 1].cuda())
        worst = min(worst, cosine(out.cpu().float(), ref.float()))
    assert worst >= 0.999, worst


def test_configuration5_group_shape(q35):
    """Configuration 5 shapes on one block of the 27B-class decode group (pattern g g g a): hidden 5120, 24 q / 4 kv
    heads of 256, GDN 48 value / 16 key heads of 128, FFN 17408, FP8 E4M3 per-row weights; a 96-token prefill (not a
    multiple of the GDN chunk or the page) and 4 decode steps against the CPU oracle stack."""
    kinds = "ggga"
    kw, ow = stack_case(kinds, H=5120, F=17408, heads=24, kv_heads=4, head_dim=256, NK=16, NV=48, DV=128, seed=4)
    cfg = dict(heads=24, kv_heads=4, head_dim=256, rot=64, theta=1e7, page_size=64, max_tokens=128)
    ref_stack = ostack.HybridStack(ow, kinds, **cfg)
    gpu_stack = q35.layers.HybridStack(to_dev(kw), kinds, **cfg)
    g = torch.Generator().manual_seed(4)
    emb = (torch.randn((100, 5120), generator=g) * 0.05).to(torch.bfloat16)
    ref, out = ref_stack.forward(emb[:96]), gpu_stack.forward(emb[:96].cuda())
    assert cosine(out.cpu().float(), ref.float()) >= 0.999
    for t in range(96, 100):
        ref, out = ref_stack.forward(emb[t:t + 1]), gpu_stack.forward(emb[t:t + 1].cuda())
        assert cosine(out.cpu().float(), ref.float()) >= 0.999, t


def test_tensor_parallel_sublayers_two_ranks_emulated_on_one_gpu(q35):
    """heads / FFN columns split over 2 ranks (ax_dsl_kernels_b200/parallel.py); both ranks run one after the other on
    this GPU and the `reduce` hook of the second adds the first one's partial, which is what the all-reduce does"""
    from ax_dsl_kernels_b200 import parallel
    kw, ow = stack_case("ga", heads=4, kv_heads=2, NK=2, NV=4, seed=11)
    dkw = to_dev(kw)
    g = torch.Generator().manual_seed(4)
    B = 3
    x = (torch.randn((B, 1, 512), generator=g) * 0.5).to(torch.bfloat16)

    def both(run):
        held = {}

        def first(p):
            held["p"] = p.clone()
            return p

        def second(p):
            return p.add_(held["p"])

        run(0, first)
        return run(1, second)

    # GDN sublayer, decode
    s0 = torch.randn((B, 4, 128, 128), generator=g) * 0.03
    conv = [(torch.randn((B, 3, wd), generator=g) * 0.03).to(torch.bfloat16) for wd in (256, 256, 512)]
    zero = torch.zeros_like(x)
    ref, s_ref, _ = ogdn.gdn_sublayer(x, zero, ow[0], s0, torch.cat(conv, -1))
    states = {}

    def run_gdn(rank, reduce):
        lw = parallel.shard_gdn_weights(dkw[0], rank, 2)
        cl = [c[..., rank * c.shape[-1] // 2:(rank + 1) * c.shape[-1] // 2].contiguous().cuda() for c in conv]
        fused, st, _ = q35.layers.gdn(x.cuda(), zero.cuda(), lw, s0[:, rank * 2:rank * 2 + 2].contiguous().cuda(),
                                      tuple(cl), reduce=reduce)
        states[rank] = st.cpu()
        return fused

    assert_parity(both(run_gdn).cpu(), ref)
    torch.testing.assert_close(torch.cat((states[0], states[1]), 1), s_ref, rtol=0, atol=4e-3)

    # attention sublayer, decode on 70 tokens of history; each rank keeps its own KV head's cache
    P, hist = 64, 70
    cache = torch.randn((2 * B, 2, P, 2, 128), generator=g).to(torch.bfloat16)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32)  # noqa: E731
    indptr, indices = i32([0, 2, 4, 6]), i32([3, 0, 5, 1, 2, 4])
    last, loc = i32([hist - P] * B), i32([[0, hist - P], [1, hist - P], [4, hist - P]])
    cos, sin = oattn.rope_cos_sin(torch.tensor([hist] * B), 32, 1e7)
    x2 = x.reshape(B, 512)
    ref = ostack.attn_sublayer(x2, ow[1], cache.clone(), indptr, indices, last, cos, sin, heads=4, kv_heads=2,
                               head_dim=128, rot=32, cache_location=loc)

    def run_attn(rank, reduce):
        aw, hl, kl = parallel.shard_attention_weights(dkw[1], rank, 2, 4, 2, 128)
        assert (hl, kl) == (2, 1)
        return q35.layers.attention(x2.cuda(), aw, cos.cuda(), sin.cuda(), cache[:, :, :, rank:rank + 1].contiguous().cuda(),
                                    indptr.cuda(), indices.cuda(), last.cuda(), heads=hl, kv_heads=kl, head_dim=128,
                                    cache_location=loc.cuda(), reduce=reduce)

    assert_parity(both(run_attn).cpu(), ref)

    # dense FFN
    ref = ostack.dense_mlp(x2, ow[0]["ln2"], ow[0]["w_gate"], ow[0]["w_up"], ow[0]["w_down"])
    out = both(lambda rank, reduce: q35.layers.mlp_residual(x2.cuda(), parallel.shard_mlp_weights(dkw[0], rank, 2),
                                                            reduce=reduce))
    assert_parity(out.cpu(), ref)


def test_decode_group_batched_sequences_match_per_sequence_oracle(q35):
    """DecodeGroup: B sequences with different histories through a g g a stack in one batched step per token.  Every
    sequence's history is built on the CPU by the oracle stack (prefill), its caches and states are copied into the
    group's batched buffers, and two batched decode steps are compared with each oracle's own decode steps."""
    kinds = "gga"
    kw, ow = stack_case(kinds, seed=21)
    cfg = dict(heads=4, kv_heads=1, head_dim=128, rot=64, theta=1e7)
    hist = [0, 5, 70]
    B, H, P, max_tokens = len(hist), 512, 64, 192
    g = torch.Generator().manual_seed(4)
    oracles = []
    for h in hist:
        o = ostack.HybridStack(ow, kinds, page_size=P, max_tokens=max_tokens, **cfg)
        if h:
            o.forward((torch.randn((h, H), generator=g) * 0.5).to(torch.bfloat16))
        oracles.append(o)
    grp = q35.layers.DecodeGroup(to_dev(kw), kinds, batch=B, max_tokens=max_tokens, page_size=P, **cfg)
    npp = grp.npp
    for b, o in enumerate(oracles):
        for i, kind in enumerate(kinds):
            if kind == "g":
                grp.state[i][b].copy_(o.state[i][0])
                widths = [c.shape[-1] for c in grp.conv[i]]
                for c, part in zip(grp.conv[i], torch.split(o.conv[i][0], widths, dim=-1)):
                    c[b].copy_(part)
            else:
                grp.cache[i][b * npp:(b + 1) * npp].copy_(o.cache[i])
    grp.set_context(hist)
    for step in range(2):
        x = (torch.randn((B, H), generator=g) * 0.5).to(torch.bfloat16)
        got = grp.step(x.cuda()).cpu()
        ref = torch.cat([o.forward(x[b:b + 1]) for b, o in enumerate(oracles)], 0)
        for b in range(B):
            assert cosine(got[b], ref[b]) >= 0.999, (step, b)
        assert rel_rms_err(got, ref) <= 5e-2
    assert grp.ctx == [h + 2 for h in hist]
    # the written KV rows are where the oracle wrote them
    a = kinds.index("a")
    for b, o in enumerate(oracles):
        got_c, ref_c = grp.cache[a][b * npp:(b + 1) * npp].cpu().float(), o.cache[a].float()
        assert (got_c - ref_c).abs().max() <= 0.05 * ref_c.abs().max()


def test_mtp_block_against_reference_golden(q35, golden):
    """speculative.mtp_step (norms, fc of the concatenated rows, gated attention on the block's own paged KV, dense
    SwiGLU, head norm -- MXFP4 projections) on the reference's mtp_step fixture: three chained rows"""
    from oracle import codecs
    f = golden("mtp")
    H, Fi, HQ, HKV, D, ROT = (int(v) for v in f["dims"])
    w = {}
    for k, t in f.items():
        if k.startswith("w."):
            w[k[2:]] = t.cuda()
    P = 256
    cache = torch.zeros((1, 2, P, HKV, D), dtype=torch.bfloat16, device="cuda")
    h = f["h0"].reshape(1, H).cuda()
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")  # noqa: E731
    for pos in range(f["e"].shape[0]):
        cos, sin = q35.rope_cos_sin(torch.tensor([pos]), ROT, 1e7, device="cuda")
        hn, y = q35.speculative.mtp_step(f["e"][pos].reshape(1, H).cuda(), h, w, cos, sin, cache, i32([0, 1 if pos else 0]),
                                         i32([0]), i32([pos]), i32([[0, pos]]), heads=HQ, kv_heads=HKV, head_dim=D)
        assert cosine(y.cpu().float(), f["y"][pos]) >= 0.999, pos
        assert rel_rms_err(hn.cpu().float().reshape(-1), f["h_next"][pos]) <= 5e-2, pos
        h = hn
    got = cache.cpu().reshape(1, 2, P, HKV * D).float()
    assert (got - f["kv"].float()).abs().max() <= 0.03 * f["kv"].float().abs().max()


def test_verify_rows_equal_decode_steps_and_accept_rolls_back(q35):
    """speculative.verify: 4 candidate rows per sequence in one pass = 4 oracle decode steps, row by row; accept()
    commits a prefix (different per sequence) and the next decode step continues from exactly there"""
    kinds = "ga"
    kw, ow = stack_case(kinds, seed=33)
    cfg = dict(heads=4, kv_heads=1, head_dim=128, rot=64, theta=1e7)
    hist, R, H, P, max_tokens = [3, 61], 4, 512, 64, 192
    B = len(hist)
    g = torch.Generator().manual_seed(8)

    def fresh_oracles():
        gg = torch.Generator().manual_seed(99)
        os_ = []
        for hlen in hist:
            o = ostack.HybridStack(ow, kinds, page_size=P, max_tokens=max_tokens, **cfg)
            o.forward((torch.randn((hlen, H), generator=gg) * 0.5).to(torch.bfloat16))
            os_.append(o)
        return os_

    oracles = fresh_oracles()
    grp = q35.layers.DecodeGroup(to_dev(kw), kinds, batch=B, max_tokens=max_tokens, page_size=P, **cfg)
    npp = grp.npp
    for b, o in enumerate(oracles):
        grp.state[0][b].copy_(o.state[0][0])
        widths = [c.shape[-1] for c in grp.conv[0]]
        for c, part in zip(grp.conv[0], torch.split(o.conv[0][0], widths, dim=-1)):
            c[b].copy_(part)
        grp.cache[1][b * npp:(b + 1) * npp].copy_(o.cache[1])
    grp.set_context(hist)
    x = (torch.randn((B, R, H), generator=g) * 0.5).to(torch.bfloat16)
    res = q35.speculative.verify(grp, x.cuda())
    ref_rows = torch.stack([torch.cat([o.forward(x[b, r:r + 1]) for r in range(R)], 0) for b, o in enumerate(oracles)], 0)
    for b in range(B):
        for r in range(R):
            assert cosine(res.out[b, r].cpu().float(), ref_rows[b, r].float()) >= 0.999, (b, r)
    assert grp.ctx == hist  # nothing committed yet
    # accept 1 row of sequence 0 and 3 of sequence 1, then one plain decode step
    n_acc = [1, 3]
    q35.speculative.accept(grp, res, n_acc)
    assert grp.ctx == [h + n for h, n in zip(hist, n_acc)]
    oracles = fresh_oracles()
    for b, o in enumerate(oracles):
        for r in range(n_acc[b]):
            o.forward(x[b, r:r + 1])
    nxt = (torch.randn((B, H), generator=g) * 0.5).to(torch.bfloat16)
    got = grp.step(nxt.cuda()).cpu()
    ref = torch.cat([o.forward(nxt[b:b + 1]) for b, o in enumerate(oracles)], 0)
    for b in range(B):
        assert cosine(got[b].float(), ref[b].float()) >= 0.999, b


def test_decode_group_bound_through_packs_and_banks(q35):
    """A `decode.group` role in the reference's binding form (small parameters in packs, projections in phase banks
    k_b<phase>_<bank>, value heads in the GGUF's tiled order, conv taps reversed) is turned into per-layer weights by
    packs.group_layers on the GPU and stepped: the output must equal the step of the group built from the plain weights
    bit for bit (same kernels, same bytes)."""
    from ax_dsl_kernels_b200 import packs
    from test_packs_cpu import reference_form_group
    kinds = "gggaggga"
    NK, NV = 2, 4
    kw, _ = stack_case(kinds, seed=9, NK=NK, NV=NV)
    manifest, tensors = reference_form_group(kw, kinds, NK, NV)
    bound = {n: t.cuda() for n, t in tensors.items()}
    layers, got_kinds = packs.group_layers(manifest, "decode.group", bound)
    cfg = dict(heads=4, kv_heads=1, head_dim=128, rot=64, theta=1e7)
    B, H = 3, 512
    outs = []
    for ws in (to_dev(kw), layers):
        grp = q35.layers.DecodeGroup(ws, "".join(got_kinds), batch=B, max_tokens=128, **cfg)
        grp.set_context([0, 3, 64])
        gx = torch.Generator().manual_seed(2)
        y = [grp.step((torch.randn((B, H), generator=gx) * 0.5).to(torch.bfloat16).cuda()).cpu() for _ in range(2)]
        outs.append(torch.stack(y))
    assert torch.isfinite(outs[0].float()).all()
    assert torch.equal(outs[0], outs[1])


def test_decode_group_fused_projections_match_separate_ones(q35):
    """DecodeGroup concatenates the projections that share an input (q k v z a b; q+gate k v; gate up) at load time;
    two steps of the fused group against the group that keeps them separate"""
    kinds = "gga"
    kw, _ = stack_case(kinds, seed=33)
    cfg = dict(heads=4, kv_heads=1, head_dim=128, rot=64, theta=1e7)
    B, H = 5, 512
    outs = []
    for fuse in (True, False):
        grp = q35.layers.DecodeGroup(to_dev(kw), kinds, batch=B, max_tokens=128, fuse=fuse, **cfg)
        assert ("w_qkvzab" in grp.layers[0]) == fuse and ("w_gateup" in grp.layers[2]) == fuse
        grp.set_context([0, 1, 63, 64, 100])
        gx = torch.Generator().manual_seed(8)
        outs.append(torch.stack([grp.step((torch.randn((B, H), generator=gx) * 0.5).to(torch.bfloat16).cuda()).cpu()
                                 for _ in range(2)]))
    assert rel_rms_err(outs[0], outs[1]) <= 2e-2
    assert cosine(outs[0], outs[1]) >= 0.9995
