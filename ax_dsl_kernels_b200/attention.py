"""Host side of paged attention decode, page-table form of the reference's sgl line
(flash_attention(x, weights, position_ids, output, cache, indptr, indices, last_page_len, *, cache_location),
models/qwen35_35b_a3b/sgl/python/sgl_kernel_axera/attention/flash_attn.py:2549-2665), extended from one request to a
batch of independent sequences."""
import torch

from . import _lib


def paged_attention_decode(q, paged_kv_cache, indptr, indices, last_page_len, out=None, *, sm_scale=None,
                           kv_scale=None, k_new=None, v_new=None, cache_location=None):
    """q [B, HQ, D] bf16; paged_kv_cache [pages, 2, P, HKV, D] bf16 or float8_e4m3fn; indptr [B+1], indices,
    last_page_len [B] int32.  History length = (pages - 1) * P + last_page_len.  k_new / v_new [B, HKV, D]: the current
    token, attended to from its own row and (with cache_location [B, 2] = page, offset) written into the cache.
    kv_scale [2, HKV] fp32: per-head dequantisation scales of an FP8 cache (default: the constant 1/8 form).
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
    if k_new is not None:
        kw["k_new"], kw["v_new"] = k_new, v_new
    _lib.run("attn.paged_decode", **kw)
    if cache_location is not None and k_new is not None:
        kv_write(paged_kv_cache, cache_location, k_new, v_new, kv_scale)
    return out


def kv_write(paged_kv_cache, cache_location, k_new, v_new, kv_scale=None):
    """store_paged_kv: rows k_new[b], v_new[b] at (page, offset) = cache_location[b]."""
    kw = dict(paged_kv_cache=paged_kv_cache, cache_location=cache_location, k_new=k_new, v_new=v_new)
    if kv_scale is not None:
        kw["kv_scale"] = kv_scale
    _lib.run("attn.kv_write", **kw)
    return paged_kv_cache


def paged_attention_prefill(q, paged_kv_cache, qo_indptr, indptr, indices, last_page_len, out=None, *, sm_scale=None,
                            k_new=None, v_new=None):
    """Causal attention of T new tokens per sequence over the paged cache.  q [Ttot, HQ, D] bf16 with the sequences
    delimited by qo_indptr [B + 1]; the page table (indptr / indices / last_page_len) describes each sequence INCLUDING
    its new tokens.  k_new / v_new [Ttot, HKV, D], when given, are first written into the cache at the new tokens'
    positions (otherwise the cache must already hold them).  Page size must be a multiple of 64."""
    out = torch.empty_like(q) if out is None else out
    kw = dict(q=q, paged_kv_cache=paged_kv_cache, qo_indptr=qo_indptr, indptr=indptr, indices=indices,
              last_page_len=last_page_len, out=out)
    if sm_scale is not None:
        kw["sm_scale"] = sm_scale if isinstance(sm_scale, torch.Tensor) else torch.tensor(
            [float(sm_scale)], dtype=torch.float32, device=q.device)
    if k_new is not None:
        kw["k_new"], kw["v_new"] = k_new, v_new
    _lib.run("attn.paged_prefill", **kw)
    return out
