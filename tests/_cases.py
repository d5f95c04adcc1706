"""Seeded synthetic inputs shared by the GPU parity tests, the smoke check and the benchmark (shapes and value
distributions of the five configurations the hot path is quoted on; seeds: C1 0, C2 1, C3 2, C4 3, C5 4)."""
import math

import torch

from oracle import codecs, gdn as ogdn


def moe_case(T, H=2048, NE=256, FE=512, FS=512, K=8, seed=3, shared_fmt="mxfp4"):
    g = torch.Generator().manual_seed(seed)
    x1 = torch.randn((T, H), generator=g).to(torch.bfloat16)
    ln2 = torch.ones(H)
    # router rows of norm ~1/sqrt(H) times the RMS-normalised h2 give logits ~ N(0, 1)
    w_router = (torch.randn((NE, H), generator=g) / math.sqrt(H)).to(torch.bfloat16)
    w_shg = (torch.randn((H,), generator=g) / math.sqrt(H)).to(torch.bfloat16)
    w = dict(ln2=ln2, w_router=w_router, w_shg=w_shg)
    w["e_gw"], w["e_gs"] = codecs.random_mxfp4((NE, 2 * FE, H), g)
    w["e_dw"], w["e_ds"] = codecs.random_mxfp4((NE, H, FE), g)
    if shared_fmt == "mxfp4":
        for n, shp in (("gate", (FS, H)), ("up", (FS, H)), ("down", (H, FS))):
            w["w_" + n], w["s_" + n] = codecs.random_mxfp4(shp, g)
    else:
        for n, shp in (("gate", (FS, H)), ("up", (FS, H)), ("down", (H, FS))):
            w["w_" + n], w["s_" + n] = codecs.quant_mxfp8(torch.randn(shp, generator=g) * 0.02)
    return x1, w


def dequant_shared(w):
    if w["w_gate"].dtype == torch.uint8:
        return tuple(codecs.dequant_mxfp4(w["w_" + n], w["s_" + n]) for n in ("gate", "up", "down"))
    return tuple(codecs.dequant_mxfp8(w["w_" + n], w["s_" + n]) for n in ("gate", "up", "down"))


def paged_case(ctxs, P=64, HKV=2, HQ=16, D=256, seed=1, fp8=False, extra_pages=3, per_head_scale=True):
    g = torch.Generator().manual_seed(seed)
    B = len(ctxs)
    n_pages = [(c + P - 1) // P for c in ctxs]
    total = sum(n_pages) + extra_pages
    kv = torch.randn((total, 2, P, HKV, D), generator=g).to(torch.bfloat16)
    perm = torch.randperm(total, generator=g).to(torch.int32)
    indptr = torch.tensor([0, *torch.tensor(n_pages).cumsum(0).tolist()], dtype=torch.int32)
    indices = perm[: sum(n_pages)].contiguous()
    last = torch.tensor([(c - (n - 1) * P) if n else 0 for c, n in zip(ctxs, n_pages)], dtype=torch.int32)
    q = torch.randn((B, HQ, D), generator=g).to(torch.bfloat16)
    kv_scale = None
    if fp8:
        if per_head_scale:
            kv_scale = (kv.float().abs().amax((0, 2, 4)) / 448.0).contiguous()  # [2, HKV]
            cache = torch.stack([codecs.kv_quant_fp8(kv[:, i], kv_scale[i]) for i in range(2)], 1).contiguous()
        else:
            cache = codecs.kv_quant_fp8(kv)
    else:
        cache = kv
    return q, cache, indptr, indices, last, kv_scale


def gdn_step_case(B=64, NK=16, NV=32, D=128, seed=2):
    g = torch.Generator().manual_seed(seed)
    q = ogdn.l2norm(torch.randn((B, 1, NK, D), generator=g))
    q = (q.float() * D ** -0.5).to(torch.bfloat16)
    k = ogdn.l2norm(torch.randn((B, 1, NK, D), generator=g))
    v = torch.randn((B, 1, NV, D), generator=g).to(torch.bfloat16)
    beta = torch.sigmoid(torch.randn((B, 1, NV), generator=g)).to(torch.bfloat16)
    gg = -torch.nn.functional.softplus(torch.randn((B, 1, NV), generator=g))
    state = torch.randn((B, NV, D, D), generator=g) * 0.03
    return q, k, v, gg, beta, state


def stack_case(kinds, H=512, F=1024, heads=4, kv_heads=1, head_dim=128, NK=2, NV=4, DV=128, seed=0, gated=True):
    """weights of a hybrid stack in the configuration-1 style: projections N(0, 0.02) quantised to FP8 E4M3 with
    per-row fp32 scales, norms 1 + N(0, 0.02), A_log = log U(1, 16), conv taps N(0, 0.1)
    (value distributions of models/qwen35_2b/whole/src/q35_step.py:313-321).
    Returns (kernel weights: quantised pairs, oracle weights: dequantised fp32) per layer."""
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(s, generator=g)  # noqa: E731
    kernel, golden = [], []

    def quant(kw, ow, name, shape):
        q8, sc = codecs.quant_fp8_rowwise(rn(*shape) * 0.02)
        kw["w_" + name], kw["s_" + name] = q8, sc
        ow["w_" + name] = codecs.dequant_fp8_rowwise(q8, sc)

    KD, VD = NK * DV, NV * DV
    for kind in kinds:
        kw, ow = {}, {}
        if kind == "g":
            for name, shape in (("q", (KD, H)), ("k", (KD, H)), ("v", (VD, H)), ("z", (VD, H)), ("a", (NV, H)),
                                ("b", (NV, H)), ("o", (H, VD))):
                quant(kw, ow, name, shape)
            for n, width in (("q", KD), ("k", KD), ("v", VD)):
                kw[f"w_{n}_conv"] = ow[f"w_{n}_conv"] = (rn(width, 4) * 0.1).to(torch.bfloat16)
            kw["input_norm_w"] = ow["input_norm_w"] = (1 + 0.02 * rn(H)).to(torch.bfloat16)
            kw["a_log"] = ow["a_log"] = (torch.rand(NV, generator=g) * 15 + 1).log()
            kw["dt_bias"] = ow["dt_bias"] = (rn(NV) * 0.02).to(torch.bfloat16)
            kw["o_norm_w"] = ow["o_norm_w"] = (1 + 0.02 * rn(DV)).to(torch.bfloat16)
        else:
            for name, shape in (("q", (heads * head_dim * (2 if gated else 1), H)), ("k", (kv_heads * head_dim, H)),
                                ("v", (kv_heads * head_dim, H)), ("o", (H, heads * head_dim))):
                quant(kw, ow, name, shape)
            kw["ln1"] = ow["ln1"] = 1 + 0.02 * rn(H)
            kw["q_norm"] = ow["q_norm"] = 1 + 0.02 * rn(head_dim)
            kw["k_norm"] = ow["k_norm"] = 1 + 0.02 * rn(head_dim)
        for name, shape in (("gate", (F, H)), ("up", (F, H)), ("down", (H, F))):
            quant(kw, ow, name, shape)
        kw["ln2"] = ow["ln2"] = 1 + 0.02 * rn(H)
        kernel.append(kw)
        golden.append(ow)
    return kernel, golden
