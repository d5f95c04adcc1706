"""Host side of paged attention decode, page-table form of the reference's sgl line
(flash_attention(x, weights, position_ids, output, cache, indptr, indices, last_page_len, *, cache_location),
models/qwen35_35b_a3b/sgl/python/sgl_kernel_axera/attention/flash_attn.py:2549-2665), extended from one request to a
batch of independent sequences."""
import torch

from . import _lib


def paged_attention_decode(q, paged_kv_cache, indptr, indices, last_page_len, out=None, *, sm_scale=None,
                           kv_scale=None, k_new=None, v_new=None, cache_location=None, paged_kv_scale=None):
    """q [B, HQ, D] bf16; paged_kv_cache [pages, 2, P, HKV, D] bf16 or float8_e4m3fn; indptr [B+1], indices,
    last_page_len [B] int32.  History length = (pages - 1) * P + last_page_len.  k_new / v_new [B, HKV, D]: the current
    token, attended to from its own row and (with cache_location [B, 2] = page, offset) written into the cache.
    kv_scale [2, HKV] fp32: per-head dequantisation scales of an FP8 cache (default: the constant 1/8 form).
    paged_kv_scale [pages, 2, P, HKV] bf16: the cache is int8 (torch.int8 or bytes) with one scale per cached row and
    head (the reference's KV8 form, models/qwen38_27b/decode/q35_group.py:198-264).
    sm_scale: float or fp32 [1] tensor (default 1/sqrt(D))."""
    if q.dtype != torch.bfloat16:
        raise TypeError("paged_attention_decode: q must be bfloat16")
    if paged_kv_cache.dim() != 5 or paged_kv_cache.shape[1] != 2:
        raise ValueError("paged_attention_decode: paged_kv_cache must be [pages, 2, P, HKV, D]")
    out = torch.empty_like(q) if out is None else out
    kw = dict(q=q, paged_kv_cache=paged_kv_cache, indptr=indptr, indices=indices, last_page_len=last_page_len, out=out)
    if sm_scale is not None:
        kw["sm_scale"] = sm_scale if isinstance(sm_scale, torch.Tensor) else torch.tensor(
            [float(sm_scale)], dtype=torch.float32, device=q.device)
    if kv_scale is not None:
        kw["kv_scale"] = kv_scale
    if paged_kv_scale is not None:
        kw["paged_kv_scale"] = paged_kv_scale
    if k_new is not None:
        kw["k_new"], kw["v_new"] = k_new, v_new
    _lib.run("attn.paged_decode", **kw)
    if cache_location is not None and k_new is not None:
        kv_write(paged_kv_cache, cache_location, k_new, v_new, kv_scale, paged_kv_scale)
    return out


def kv_write(paged_kv_cache, cache_location, k_new, v_new, kv_scale=None, paged_kv_scale=None):
    """store_paged_kv: rows k_new[b], v_new[b] at (page, offset) = cache_location[b].  FP8 caches quantise with
    kv_scale (or x 8); an int8 cache quantises every row and head with its own scale, stored into paged_kv_scale."""
    kw = dict(paged_kv_cache=paged_kv_cache, cache_location=cache_location, k_new=k_new, v_new=v_new)
    if kv_scale is not None:
        kw["kv_scale"] = kv_scale
    if paged_kv_scale is not None:
        kw["paged_kv_scale"] = paged_kv_scale
    _lib.run("attn.kv_write", **kw)
    return paged_kv_cache


def paged_attention_prefill(q, paged_kv_cache, qo_indptr, indptr, indices, last_page_len, out=None, *, sm_scale=None,
                            k_new=None, v_new=None, kv_scale=None, paged_kv_scale=None):
    """Causal attention of T new tokens per sequence over the paged cache.  q [Ttot, HQ, D] bf16 with the sequences
    delimited by qo_indptr [B + 1]; the page table (indptr / indices / last_page_len) describes each sequence INCLUDING
    its new tokens.  k_new / v_new [Ttot, HKV, D], when given, are first written into the cache at the new tokens'
    positions (otherwise the cache must already hold them).  Page size must be a multiple of 64.  An FP8 (E4M3) cache
    holds x * 8, or x / kv_scale[kv, head] with kv_scale [2, HKV]; new rows are quantised as they are written."""
    out = torch.empty_like(q) if out is None else out
    kw = dict(q=q, paged_kv_cache=paged_kv_cache, qo_indptr=qo_indptr, indptr=indptr, indices=indices,
              last_page_len=last_page_len, out=out)
    if kv_scale is not None:
        kw["kv_scale"] = kv_scale
    if paged_kv_scale is not None:  # int8 cache: [pages, 2, P, HKV] bf16 row scales (read, and written for new rows)
        kw["paged_kv_scale"] = paged_kv_scale
    if sm_scale is not None:
        kw["sm_scale"] = sm_scale if isinstance(sm_scale, torch.Tensor) else torch.tensor(
            [float(sm_scale)], dtype=torch.float32, device=q.device)
    if k_new is not None:
        kw["k_new"], kw["v_new"] = k_new, v_new
    _lib.run("attn.paged_prefill", **kw)
    return out


def rope_cos_sin(positions, rot, theta, device=None):
    """cos / sin rows [T, rot / 2] fp32 of plain RoPE for integer positions [T] (the tables attn.qk_prep takes;
    models/qwen35_2b/whole/src/q35_step.py:408-411)."""
    pos = torch.as_tensor(positions)
    device = device if device is not None else pos.device
    inv = 1.0 / (theta ** (torch.arange(0, rot, 2, dtype=torch.int64).float() / rot))
    f = pos.to(torch.float32).reshape(-1, 1).cpu() * inv.reshape(1, -1)
    return f.cos().to(device).contiguous(), f.sin().to(device).contiguous()


def mrope_cos_sin(position_ids, rot, theta, mrope_section=(11, 11, 10), interleaved=True, device=None):
    """cos / sin rows [T, rot / 2] fp32 of multimodal RoPE from position_ids [3, T] (temporal, height, width): rotary
    pair c turns by position_ids[axis(c), t] * inv_freq[c], where axis(c) follows mrope_section = (t, h, w) pairs --
    chunked (T pairs first, then H, then W) or interleaved (pairs 1, 4, 7, ... below 3 h follow H, pairs 2, 5, 8, ...
    below 3 w follow W, the rest T).  Reference: gather_mrope_cos_sin / mrope_channel_masks
    (models/qwen35_35b_a3b/sgl/python/sgl_kernel_axera/attention/attn_utils/common.py:316-398).  The rows feed
    attn.qk_prep exactly like plain RoPE rows; text-only input (three equal rows) gives plain RoPE."""
    pos = torch.as_tensor(position_ids)
    if pos.dim() != 2 or pos.shape[0] != 3:
        raise ValueError("mrope_cos_sin: position_ids must be [3, T]")
    t, h, w = (int(v) for v in mrope_section)
    if min(t, h, w) < 0 or 2 * (t + h + w) != rot:
        raise ValueError(f"mrope_cos_sin: mrope_section {tuple(mrope_section)} must sum to rot / 2 = {rot // 2}")
    device = device if device is not None else pos.device
    axis = torch.zeros(rot // 2, dtype=torch.long)
    if interleaved:
        axis[1:h * 3:3] = 1
        axis[2:w * 3:3] = 2
    else:
        axis[t:t + h] = 1
        axis[t + h:] = 2
    inv = 1.0 / (theta ** (torch.arange(0, rot, 2, dtype=torch.int64).float() / rot))
    f = pos.to(torch.float32).cpu()[axis].T * inv.reshape(1, -1)
    return f.cos().to(device).contiguous(), f.sin().to(device).contiguous()
