"""MoE block of the Qwen3.5 decoder (CPU oracle; test infrastructure only).

Follows the "q35" kernel line of the reference: router logits and routing weights in fp32, the routing weight
applied to the fp32 down-projection output, shared-expert gate sigmoid in fp32.
"""
import torch
import torch.nn.functional as F

from .codecs import dequant_mxfp4

EPS = 1e-6


def bf(x):
    """round to bf16, keep computing in fp32"""
    return x.to(torch.bfloat16).float()


def rmsnorm(x, w, eps=EPS):
    """fp32 x / sqrt(mean x^2 + eps) * w -> bf16; w is the effective multiplier (the host passes 1 + weight,
    models/qwen35_2b/whole/src/q35_step.py:346-348;
    models/qwen35_35b_a3b/sgl/python/sgl_kernel_axera/attention/attn_utils/common.py:216-228)."""
    xf = x.float()
    return (xf * torch.rsqrt(xf.square().mean(-1, keepdim=True) + eps) * w.float()).to(torch.bfloat16)


def moe_pre(x1, ln2, w_gate, w_up, w_down, w_router, w_shg, eps=EPS):
    """Dense part of the MoE block (models/qwen35_2b/whole/src/q35_moe.py:123-137).

    x1 [T, H] bf16; ln2 [H] fp32; w_gate / w_up [FS, H], w_down [H, FS] DEQUANTIZED fp32; w_router [NE, H] bf16;
    w_shg [H] bf16.  Returns base [T, H] bf16, h2 [T, H] bf16, logits [T, NE] fp32."""
    h2 = rmsnorm(x1, ln2, eps)
    h = h2.float()
    g, u = bf(h @ w_gate.float().T), bf(h @ w_up.float().T)
    act = bf(F.silu(g) * u)
    sh = act @ w_down.float().T
    gate = (h * w_shg.float()).sum(-1, keepdim=True)
    base = (x1.float() + sh * torch.sigmoid(gate)).to(torch.bfloat16)
    logits = h @ w_router.float().T
    return base, h2, logits


def route(logits, top_k):
    """softmax fp32 over all experts -> top-k -> weights / their sum (models/qwen35_2b/whole/src/q35_moe.py:293-297),
    batched over tokens.  Order: descending probability, ties to the lower expert id (the rule the reference checks
    its on-device top-k against, models/qwen35_2b/whole/src/q35_layer_mc.py:1494-1499)."""
    pr = torch.softmax(logits.float(), -1)
    sv, si = torch.sort(pr, dim=-1, descending=True, stable=True)
    v, ids = sv[..., :top_k], si[..., :top_k]
    return ids.to(torch.int32), (v / v.sum(-1, keepdim=True)).float()


def experts_decode(h2, base, ids, rw, e_gw, e_gs, e_dw, e_ds):
    """out[t] = bf16(base[t] + sum_i rw[t, i] * down_e(bf16(silu(g) * u))), g | u = bf16(h2[t] @ Wc_e.T)
    (golden inside experts_check, models/qwen35_2b/whole/src/q35_moe.py:227-238; kernel
    moe_experts_gu, :101-112).  Planar expert tensors as the prefill kernels take them
    (models/qwen35_2b/whole/src/q35_moe_prefill.py:103-113): e_gw [NE, 2 FE, H/2] u8 (gate rows then up rows),
    e_gs [NE, 2 FE, H/32], e_dw [NE, H, FE/2], e_ds [NE, H, FE/32]."""
    T, H = h2.shape
    FE = e_gw.shape[1] // 2
    acc = base.float().clone()
    cache = {}
    for t in range(T):
        x = h2[t].float()
        for i in range(ids.shape[1]):
            e = int(ids[t, i])
            if e not in cache:
                cache[e] = (dequant_mxfp4(e_gw[e], e_gs[e]), dequant_mxfp4(e_dw[e], e_ds[e]))
            wc, wd = cache[e]
            gu = bf(wc @ x)
            a = bf(F.silu(gu[:FE]) * gu[FE:])
            acc[t] += rw[t, i] * (wd @ a)
    return acc.to(torch.bfloat16)


def slots(h2, tok, rw, e_gw, e_gs, e_dw, e_ds, out_dtype=torch.bfloat16):
    """Slot-grouped routed experts of a prefill group (golden inside slots_px_check,
    models/qwen35_2b/whole/src/q35_moe_prefill.py:239-246; kernel moe_slots_px :150-166).
    tok [S, 1 + G] int32: column 0 the slot's expert, then G token rows of h2 (unused rows: any token, rw 0);
    out[s, g] = rw[s, g] * down(bf16(silu(g) * u))."""
    S, G = rw.shape
    FE = e_gw.shape[1] // 2
    out = torch.zeros((S, G, h2.shape[1]))
    for s in range(S):
        e = int(tok[s, 0])
        wc, wd = dequant_mxfp4(e_gw[e], e_gs[e]), dequant_mxfp4(e_dw[e], e_ds[e])
        xi = h2[tok[s, 1:].long()].float()
        gu = bf(xi @ wc.T)
        a = bf(F.silu(gu[:, :FE]) * gu[:, FE:])
        out[s] = rw[s].reshape(G, 1) * (a @ wd.T)
    return out.to(out_dtype)


def combine(base, loc, sout):
    """out[t] = bf16(base[t] + sum_k sout[loc[k, t]]) in fp32 (models/qwen35_2b/whole/src/q35_moe_prefill.py:201-214,
    golden :266)."""
    return (base.float() + sout.float()[loc.long()].sum(0)).to(torch.bfloat16)


def permute(ids, rw, G, S=None):
    """Token -> slot permutation (host code of the reference's adapter, not in its repository; rule stated at
    models/qwen35_2b/whole/src/q35_moe_prefill.py:150-152,194-195: a slot is one expert and up to G token rows,
    unused rows point at any token with weight 0).  Counting sort by expert id, stable in token index: experts in
    id order, each expert's tokens in index order split into ceil(n / G) slots.
    Returns tok [S, 1 + G] i32, srw [S, G] f32, loc [K, T] i32 (row of the flattened [S * G] slot output)."""
    T, K = ids.shape
    order = torch.sort(ids.reshape(-1).long(), stable=True).indices  # pair index p = t * K + k
    e_sorted = ids.reshape(-1).long()[order]
    rows = []
    loc = torch.zeros((K, T), dtype=torch.int32)
    tok_rows, rw_rows = [], []
    start = 0
    n = e_sorted.numel()
    while start < n:
        e = int(e_sorted[start])
        stop = start
        while stop < n and int(e_sorted[stop]) == e:
            stop += 1
        for s0 in range(start, stop, G):
            pairs = order[s0:min(s0 + G, stop)]
            t_row = torch.zeros(1 + G, dtype=torch.int32)
            w_row = torch.zeros(G)
            t_row[0] = e
            slot = len(tok_rows)
            for j, p in enumerate(pairs.tolist()):
                t, k = divmod(p, K)
                t_row[1 + j] = t
                w_row[j] = rw[t, k]
                loc[k, t] = slot * G + j
            tok_rows.append(t_row)
            rw_rows.append(w_row)
        start = stop
    n_used = len(tok_rows)
    S = n_used if S is None else S
    assert n_used <= S
    tok = torch.zeros((S, 1 + G), dtype=torch.int32)
    srw = torch.zeros((S, G))
    if n_used:
        tok[:n_used] = torch.stack(tok_rows)
        srw[:n_used] = torch.stack(rw_rows)
    return tok, srw, loc, n_used


def moe_block(x1, ln2, sh_gate, sh_up, sh_down, w_router, w_shg, e_gw, e_gs, e_dw, e_ds, top_k, eps=EPS):
    """whole block: dense part -> route -> routed experts; sh_* are dequantized shared-expert weights"""
    base, h2, logits = moe_pre(x1, ln2, sh_gate, sh_up, sh_down, w_router, w_shg, eps)
    ids, rw = route(logits, top_k)
    return experts_decode(h2, base, ids, rw, e_gw, e_gs, e_dw, e_ds), ids, rw, logits
