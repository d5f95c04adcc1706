"""The allocation-free attention entry point, called through the C ABI.

Who needs it: a host that cannot hand the library a workspace because it cannot allocate device memory at call time
(all of its buffers were planned and frozen before the first token, or its memory belongs to another component's pool).
q35_attn_paged_decode_static keeps the split-KV scratch in an array built into the library instead.

Checked here: its output equals the workspace-taking role's output on the same inputs, on two calls in a row (the
second call finds the first call's leftovers in the shared scratch), and oversized shapes are refused with a status.
"""
import ctypes

import pytest
import torch

from _cases import paged_case

pytestmark = pytest.mark.gpu


def _call_static(L, q, cache, indptr, indices, last, out, sm_scale=None, kv_scale=None):
    B, HQ, D = q.shape
    pages, _, P, HKV, _ = cache.shape
    ptr = lambda t: ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)  # noqa: E731
    dtype = 9 if cache.dtype == torch.bfloat16 else 11
    return L.q35_attn_paged_decode_static(
        ptr(q), ptr(cache), dtype, ptr(indptr), ptr(indices), ptr(last), ptr(sm_scale), ptr(kv_scale), ptr(out),
        B, HQ, HKV, D, P, pages, indices.numel(), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


@pytest.mark.parametrize("fp8", [False, True])
def test_static_scratch_entry_point_matches_workspace_role_twice(fp8):
    assert torch.cuda.is_available()
    import ax_dsl_kernels_b200 as q35
    L = q35._lib.lib()
    L.q35_attn_paged_decode_static.restype = ctypes.c_int
    for rep, ctxs in enumerate(([1, 63, 64, 65, 700, 0, 2500], [900, 3, 128, 4000])):  # two calls in a row
        q, cache, indptr, indices, last, kvs = [t.cuda() if t is not None else None
                                                for t in paged_case(ctxs, seed=10 + rep, fp8=fp8)]
        scale = torch.tensor([1.0 / 16], device="cuda")
        ref = q35.paged_attention_decode(q, cache, indptr, indices, last, sm_scale=scale, kv_scale=kvs)
        out = torch.full_like(q, float("nan"))
        rc = _call_static(L, q, cache, indptr, indices, last, out, scale, kvs)
        assert rc == 0, L.q35_last_error().decode()
        torch.cuda.synchronize()
        if not fp8:  # same kernel, same split of the work: bit-identical
            assert torch.equal(out.view(torch.int16), ref.view(torch.int16))
        else:
            # the role runs the one-byte formats with eight warps per CTA (two tiles in flight), the fixed scratch of
            # this entry point is sized for four: the same arithmetic per tile, merged in a different order
            # -- two roundings of almost equal fp32 values: equal, or one bf16 step apart
            o, r = out.float(), ref.float()
            rms = r.square().mean((1, 2), keepdim=True).sqrt()
            assert ((o - r).abs() <= r.abs() * 2.0 ** -7 + 4e-3 * rms).all()
    assert q35.device_status() == 0


def test_static_scratch_entry_point_rejects_oversized_shapes():
    import ax_dsl_kernels_b200 as q35
    L = q35._lib.lib()
    L.q35_attn_paged_decode_static.restype = ctypes.c_int
    B = 2048  # (B * HKV + SMs) * 4 slots of 8.25 KB is far beyond 16 MiB
    q = torch.zeros((B, 16, 256), dtype=torch.bfloat16, device="cuda")
    cache = torch.zeros((4, 2, 64, 2, 256), dtype=torch.bfloat16, device="cuda")
    indptr = torch.zeros(B + 1, dtype=torch.int32, device="cuda")
    indices = torch.zeros(4, dtype=torch.int32, device="cuda")
    last = torch.zeros(B, dtype=torch.int32, device="cuda")
    rc = _call_static(L, q, cache, indptr, indices, last, torch.empty_like(q))
    assert rc == 6  # Q35_ERR_WORKSPACE
    assert b"built-in array" in L.q35_last_error()
