"""Paged GQA attention of the Qwen3.5 decoder (CPU oracle; test infrastructure only).

Page-table form of the reference's sgl line: paged_kv_cache [pages, 2, P, HKV, D] (K plane, V plane per page),
indptr [B + 1], indices [pages used], last_page_len [B]
(models/qwen35_35b_a3b/sgl/python/sgl_kernel_axera/attention/flash_attn.py:2549-2587).
"""
import math

import torch
import torch.nn.functional as F

from .codecs import kv_dequant_fp8, kv_dequant_int8_rows, kv_quant_fp8, kv_quant_int8_rows
from .moe import bf, rmsnorm


def valid_kv_len(indptr, last_page_len, page):
    """(n_pages - 1) * P + last_page_len, 0 for a sequence without pages (flash_attn.py:2354-2358)."""
    n = (indptr[1:] - indptr[:-1]).long()
    return torch.where(n > 0, (n - 1) * page + last_page_len.long(), torch.zeros_like(n))


def gather_kv(cache, indptr, indices, last_page_len, b, kv_scale=None, row_scale=None):
    """history K, V of sequence b as fp32 [ctx, HKV, D] (golden gather,
    models/qwen35_35b_a3b/sgl/tests/test_qwen35_runtime.py:76-79)."""
    P = cache.shape[2]
    rows = indices[int(indptr[b]):int(indptr[b + 1])].long()
    ctx = int(valid_kv_len(indptr, last_page_len, P)[b])
    k = cache[rows, 0].reshape(-1, *cache.shape[3:])[:ctx]
    v = cache[rows, 1].reshape(-1, *cache.shape[3:])[:ctx]
    if row_scale is not None:  # int8 rows with a bf16 scale per row and head: row_scale [pages, 2, P, HKV]
        sk = row_scale[rows, 0].reshape(-1, row_scale.shape[-1])[:ctx]
        sv = row_scale[rows, 1].reshape(-1, row_scale.shape[-1])[:ctx]
        return kv_dequant_int8_rows(k, sk), kv_dequant_int8_rows(v, sv)
    if cache.dtype == torch.float8_e4m3fn:
        ks = vs = None
        if kv_scale is not None:
            ks, vs = kv_scale[0], kv_scale[1]
        return kv_dequant_fp8(k, ks), kv_dequant_fp8(v, vs)
    return k.float(), v.float()


def paged_decode(q, cache, indptr, indices, last_page_len, sm_scale=None, kv_scale=None, k_new=None, v_new=None,
                 row_scale=None):
    """One query token per sequence over its paged history (+ optionally the current token's own k / v row, which the
    kernel takes from registers instead of the cache, flash_attn.py:2088-2124).

    q [B, HQ, D] bf16; k_new / v_new [B, HKV, D] bf16; kv_scale [2, HKV] fp32 for a per-head-scaled FP8 cache (None with
    an FP8 cache: the constant-8 form).  softmax(q k^T * sm_scale) v in fp32 -> bf16, query head h uses KV head
    h // (HQ / HKV) (golden: scaled_dot_product_attention(enable_gqa=True),
    models/qwen35_35b_a3b/sgl/tests/test_qwen35_runtime.py:80-85).  A sequence with no key at all gives zeros."""
    B, HQ, D = q.shape
    HKV = cache.shape[3]
    G = HQ // HKV
    scale = 1.0 / math.sqrt(D) if sm_scale is None else float(sm_scale)
    out = torch.zeros((B, HQ, D))
    for b in range(B):
        k, v = gather_kv(cache, indptr, indices, last_page_len, b, kv_scale, row_scale)
        if k_new is not None:
            k = torch.cat([k, k_new[b].float()[None]], 0)
            v = torch.cat([v, v_new[b].float()[None]], 0)
        if k.shape[0] == 0:
            continue
        qb = q[b].float().reshape(HKV, G, D)
        s = torch.einsum("hgd,lhd->hgl", qb, k) * scale
        p = torch.softmax(s, -1)
        out[b] = torch.einsum("hgl,lhd->hgd", p, v).reshape(HQ, D)
    return out.to(torch.bfloat16)


def paged_decode_partial(q, cache, indptr, indices, last_page_len, sm_scale=None, kv_scale=None, row_scale=None):
    """the unnormalised partial of paged_decode over the given pages: m (maximum score in the log2 domain), l (sum of
    2^(s - m)), o (sum of 2^(s - m) v) per (sequence, query head) -- what one of several devices that split a KV head's
    pages contributes (flash_attn.py:2393-2474).  A sequence without keys gives l = 0."""
    B, HQ, D = q.shape
    HKV = cache.shape[3]
    G = HQ // HKV
    scale = (1.0 / math.sqrt(D) if sm_scale is None else float(sm_scale)) * math.log2(math.e)
    m = torch.full((B, HQ), float("-inf"))
    ln = torch.zeros((B, HQ))
    o = torch.zeros((B, HQ, D))
    for b in range(B):
        k, v = gather_kv(cache, indptr, indices, last_page_len, b, kv_scale, row_scale)
        if k.shape[0] == 0:
            continue
        s = torch.einsum("hgd,lhd->hgl", q[b].float().reshape(HKV, G, D), k) * scale
        mb = s.amax(-1)
        p = torch.exp2(s - mb[..., None])
        m[b], ln[b] = mb.reshape(HQ), p.sum(-1).reshape(HQ)
        o[b] = torch.einsum("hgl,lhd->hgd", p, v).reshape(HQ, D)
    return m, ln, o


def lse_merge(pm, pl, po):
    """merge of partials [S, B, HQ(, D)] by log-sum-exp (q35_layer_mc.py:361-379) -> bf16 [B, HQ, D]"""
    live = pl > 0
    M = torch.where(live, pm, torch.full_like(pm, float("-inf"))).amax(0)
    f = torch.where(live, torch.exp2(pm - M), torch.zeros_like(pm))
    L = (pl * f).sum(0)
    o = (po * f[..., None]).sum(0)
    return torch.where(L[..., None] > 0, o / L[..., None].clamp_min(1e-38), torch.zeros_like(o)).to(torch.bfloat16)


def paged_prefill(q, cache, qo_indptr, indptr, indices, last_page_len, sm_scale=None, kv_scale=None, row_scale=None):
    """T new tokens per sequence against the paged cache that already holds their K / V rows, causal:
    token i of a sequence with `hist` earlier tokens sees keys 0 .. hist + i (prefill form of the decode golden;
    reference kernels: flash_attn.py:471-610, models/qwen35_2b/whole/src/q35_prefill.py:250-318).
    q [Ttot, HQ, D] bf16, sequences delimited by qo_indptr [B + 1].  An FP8 cache is read back through its dequantised
    rows, the new tokens' own rows included (models/qwen38_27b/prefill/sgl_kv8_kvf8.patch: every K / V tile comes from
    the cache); kv_scale [2, HKV] as in paged_decode."""
    Ttot, HQ, D = q.shape
    HKV = cache.shape[3]
    G = HQ // HKV
    scale = 1.0 / math.sqrt(D) if sm_scale is None else float(sm_scale)
    out = torch.zeros((Ttot, HQ, D))
    for b in range(qo_indptr.numel() - 1):
        q0, q1 = int(qo_indptr[b]), int(qo_indptr[b + 1])
        if q1 == q0:
            continue
        k, v = gather_kv(cache, indptr, indices, last_page_len, b, kv_scale, row_scale)
        hist = k.shape[0] - (q1 - q0)
        qb = q[q0:q1].float().reshape(q1 - q0, HKV, G, D)
        s = torch.einsum("thgd,lhd->thgl", qb, k) * scale
        pos = hist + torch.arange(q1 - q0)
        mask = torch.arange(k.shape[0])[None, :] > pos[:, None]
        s = s.masked_fill(mask[:, None, None, :], float("-inf"))
        out[q0:q1] = torch.einsum("thgl,lhd->thgd", torch.softmax(s, -1), v).reshape(q1 - q0, HQ, D)
    return out.to(torch.bfloat16)


def store_paged_kv(cache, cache_location, k_new, v_new, kv_scale=None, row_scale=None):
    """write the current token's K / V rows at (page, offset) per sequence (flash_attn.py:53-84); FP8 caches store
    e4m3(x * 8) (models/qwen38_27b/decode/q35_group.py:244-249) or e4m3(x / scale_h) with kv_scale [2, HKV]."""
    for b in range(k_new.shape[0]):
        page, off = int(cache_location[b, 0]), int(cache_location[b, 1])
        if row_scale is not None:  # int8 rows, their scales stored alongside (kv_write_paged, q35_group.py:253-260)
            for kv, row in ((0, k_new[b]), (1, v_new[b])):
                q8, sc = kv_quant_int8_rows(row)
                cache[page, kv, off] = q8.to(cache.dtype) if cache.dtype == torch.int8 else q8.view(torch.uint8)
                row_scale[page, kv, off] = sc
        elif cache.dtype == torch.float8_e4m3fn:
            ks = vs = None
            if kv_scale is not None:
                ks, vs = kv_scale[0], kv_scale[1]
            cache[page, 0, off] = kv_quant_fp8(k_new[b], ks)
            cache[page, 1, off] = kv_quant_fp8(v_new[b], vs)
        else:
            cache[page, 0, off] = k_new[b].to(cache.dtype)
            cache[page, 1, off] = v_new[b].to(cache.dtype)
    return cache


def rope_neox(x, cos, sin, rot):
    """NeoX-style rotation of the first `rot` channels (halves rot/2 apart), the rest passed through
    (attn_utils/common.py:248-301; golden test_qwen35_runtime.py:66-72).  x [..., D] bf16, cos / sin [..., rot/2]."""
    a, b = x[..., : rot // 2].float(), x[..., rot // 2: rot].float()
    c, s = cos.float(), sin.float()
    y = x.clone()
    y[..., : rot // 2] = (a * c - b * s).to(x.dtype)
    y[..., rot // 2: rot] = (b * c + a * s).to(x.dtype)
    return y


def rope_cos_sin(pos, rot, theta):
    """models/qwen35_2b/whole/src/q35_step.py:408-411 (fp32 here; the kernels take them as inputs)."""
    inv = 1.0 / (theta ** (torch.arange(0, rot, 2, dtype=torch.int64).float() / rot))
    f = torch.as_tensor(pos).float().reshape(-1, 1) * inv
    return f.cos(), f.sin()


def mrope_channel_axis(section, interleaved):
    """which of the three position rows (0 = temporal, 1 = height, 2 = width) rotary pair c follows
    (mrope_channel_masks, models/qwen35_35b_a3b/sgl/python/sgl_kernel_axera/attention/attn_utils/common.py:316-335):
    chunked: the first t pairs follow T, the next h follow H, the rest W; interleaved: pairs 1, 4, 7, ... below 3 h follow
    H, pairs 2, 5, 8, ... below 3 w follow W, every other pair T."""
    t, h, w = (int(v) for v in section)
    half = t + h + w
    axis = torch.zeros(half, dtype=torch.long)
    if interleaved:
        axis[1:h * 3:3] = 1
        axis[2:w * 3:3] = 2
    else:
        axis[t:t + h] = 1
        axis[t + h:] = 2
    return axis


def mrope_cos_sin(position_ids, rot, theta, section=(11, 11, 10), interleaved=True):
    """M-RoPE rows for T tokens from position_ids [3, T]: pair c rotates by position_ids[axis(c), t] * inv_freq[c]
    (gather_mrope_cos_sin / mix_mrope_tables, attn_utils/common.py:338-398).  Returns cos, sin [T, rot / 2] fp32."""
    inv = 1.0 / (theta ** (torch.arange(0, rot, 2, dtype=torch.int64).float() / rot))
    axis = mrope_channel_axis(section, interleaved)
    pos = position_ids.float()[axis].T  # [T, rot / 2]
    f = pos * inv
    return f.cos(), f.sin()


def attn_layer_decode(x, w, cache, indptr, indices, last_page_len, cache_location, cos, sin, *, heads, kv_heads,
                      head_dim, rot, gated=True, eps=1e-6, sm_scale=None, kv_scale=None):
    """Decode attention sublayer on B sequences (one token each), golden of
    models/qwen35_35b_a3b/sgl/tests/test_qwen35_runtime.py:57-93: RMSNorm -> q(+gate) / k / v projections (bf16) ->
    q / k RMSNorm -> RoPE -> cache write -> attention over history + current token -> sigmoid gate -> o-proj ->
    residual.  w: ln1 [H] f32, w_q [HQ * D * (2 if gated), H] (per head [q | gate], models/qwen35_2b/whole/src/
    q35_step.py:192-194), w_k, w_v [HKV * D, H], q_norm, k_norm [D] f32, w_o [H, HQ * D] -- DEQUANTIZED fp32.
    x [B, H] bf16.  Returns out [B, H] bf16 (cache updated in place)."""
    B, H = x.shape
    n = rmsnorm(x, w["ln1"], eps).float()
    qg = bf(n @ w["w_q"].float().T).reshape(B, heads, -1)
    q, gate = (qg[..., :head_dim], qg[..., head_dim:]) if gated else (qg, None)
    k = bf(n @ w["w_k"].float().T).reshape(B, kv_heads, head_dim)
    v = bf(n @ w["w_v"].float().T).reshape(B, kv_heads, head_dim).to(torch.bfloat16)
    q = rmsnorm(q, w["q_norm"], eps)
    k = rmsnorm(k, w["k_norm"], eps)
    q = rope_neox(q, cos[:, None, :], sin[:, None, :], rot)
    k = rope_neox(k, cos[:, None, :], sin[:, None, :], rot)
    attn = paged_decode(q, cache, indptr, indices, last_page_len, sm_scale, kv_scale, k_new=k, v_new=v).float()
    store_paged_kv(cache, cache_location, k, v, kv_scale)
    if gated:
        attn = bf(attn * torch.sigmoid(gate))
    o = bf(attn.reshape(B, -1) @ w["w_o"].float().T)
    return (x.float() + o).to(torch.bfloat16), q, k, v


def sdpa_decode_reference(q, k_hist, v_hist):
    """independent formulation used to cross-check paged_decode in the CPU tests: torch SDPA with GQA on one
    sequence, q [HQ, D], k / v [L, HKV, D] (all fp32)."""
    o = F.scaled_dot_product_attention(q[None, :, None, :].double(), k_hist.permute(1, 0, 2)[None].double(),
                                       v_hist.permute(1, 0, 2)[None].double(), enable_gqa=True)
    return o[0, :, 0].float()
