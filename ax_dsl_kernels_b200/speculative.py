"""Speculative-decode pieces of the 27B-class decode group, composed from the library's roles (host side, no math of
its own): the MTP draft block and the multi-row verify pass.

Reference: the MTP block `mtp_kernel` (models/qwen38_27b/mtp/mtp_kernel.py, golden mtp_step in
models/qwen38_27b/mtp/mtp_ref.py:202-239) and the 4-row verify group (models/qwen38_27b/verify/verify_group_m4.py;
attention over one KV pass for the rows: attention_split_qa_rows, models/qwen38_27b/decode/q35_group.py:656-734).
"""
import torch

from . import layers
from .moe import linear


def mtp_step(e, h, w, cos, sin, cache, indptr, indices, last_page_len, cache_location, *, heads, kv_heads, head_dim,
             sm_scale=None):
    """One MTP row for B sequences: the embedding e [B, H] of token x_p and the target model's final-norm hidden h [B, H]
    of position p - 1 ->
        z = fc([RMSNorm(e) * ln_e | RMSNorm(h) * ln_h]);  y = decoder layer(z) on the block's OWN paged KV;
        h_next = RMSNorm(y) * head_norm
    w: the reference's names -- ln_e, ln_h, ln1, ln2, head_norm, q_norm, k_norm (effective multipliers, fp32) and the
    quantised projections (w_x, s_x) for x in fc q k v o gate up down (w_q per head [q | gate]).  The page table
    describes the block's HISTORY, cache_location [B, 2] the slot of this row (as layers.attention).  cos / sin [B, rot/2].
    Returns (h_next [B, H] bf16, y [B, H] bf16)."""
    en, _, _ = layers.rmsnorm(e, w["ln_e"])
    hn, _, _ = layers.rmsnorm(h, w["ln_h"])
    z = linear(torch.cat([en, hn], -1), w["w_fc"], w["s_fc"])
    x1 = layers.attention(z, w, cos, sin, cache, indptr, indices, last_page_len, heads=heads, kv_heads=kv_heads,
                          head_dim=head_dim, cache_location=cache_location, gated=True, sm_scale=sm_scale)
    y = layers.mlp_residual(x1, w)
    h_next, _, _ = layers.rmsnorm(y, w["head_norm"])
    return h_next, y


class VerifyResult:
    """what DecodeGroup.verify returns: out [B, R, H], and per GDN layer the states after each row (to roll back to the
    accepted prefix)"""

    def __init__(self, out, states, convs):
        self.out, self.states, self.convs = out, states, convs


def verify(group, x):
    """R candidate tokens per sequence through a layers.DecodeGroup in ONE pass, without committing them: x [B, R, H]
    -> VerifyResult.  Attention layers take all rows of a sequence at once (causal among themselves, one pass over
    the sequence's KV; their K / V rows are written at positions ctx .. ctx + R - 1, later rows simply get overwritten
    when a shorter prefix is accepted).  GDN layers run the rows in order on a copy of the state and keep the state
    after every row.  Row r of the result equals what r + 1 decode steps would give."""
    B, R, H = x.shape
    P, npp, dev = group.P, group.npp, group.dev
    ctx = group.ctx
    if max(ctx) + R > npp * P:
        raise ValueError("verify: the rows do not fit the caches")
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)  # noqa: E731
    n_tot = [(c + R + P - 1) // P for c in ctx]
    indptr = i32([0, *torch.tensor(n_tot).cumsum(0).tolist()])
    indices = i32([b * npp + i for b, n in enumerate(n_tot) for i in range(n)])
    last = i32([c + R - (n - 1) * P for c, n in zip(ctx, n_tot)])
    qo = i32([R * b for b in range(B + 1)])
    pos = torch.tensor([c + r for c in ctx for r in range(R)], dtype=torch.float32)
    inv = 1.0 / (group.theta ** (torch.arange(0, group.rot, 2, dtype=torch.int64).float() / group.rot))
    f = pos.reshape(-1, 1) * inv.reshape(1, -1)
    cos, sin = f.cos().to(dev).contiguous(), f.sin().to(dev).contiguous()
    states, convs = {}, {}
    cur = x
    for i, (w, kind) in enumerate(zip(group.layers, group.kinds)):
        if kind == "g":
            st = group.state[i].clone()
            cv = tuple(c.clone() for c in group.conv[i])
            snaps, csnaps, rows = [], [], []
            for r in range(R):
                xr = cur[:, r].contiguous()
                fused, st, cv = layers.gdn(xr.reshape(B, 1, H), torch.zeros_like(xr).reshape(B, 1, H), w, st, cv,
                                           reduce=group.reduce)
                rows.append(fused.reshape(B, H))
                snaps.append(st)
                csnaps.append(cv)
            states[i], convs[i] = snaps, csnaps
            x1 = torch.stack(rows, 1).reshape(B * R, H)
        else:
            x1 = layers.attention(cur.reshape(B * R, H), w, cos, sin, group.cache[i], indptr, indices, last, qo_indptr=qo,
                                  gated=group.gated, sm_scale=group.sm_scale, reduce=group.reduce, **group.cfg)
        cur = layers.mlp_residual(x1.reshape(B * R, H), w, reduce=group.reduce).reshape(B, R, H)
    return VerifyResult(cur, states, convs)


def accept(group, result, n_accepted):
    """commit the first n_accepted[b] rows of a verify pass for every sequence: GDN states and conv states roll to the
    snapshot after that row (n = 0 keeps the old state), contexts advance; KV rows beyond the accepted prefix stay in
    the caches as garbage past the context and are overwritten by later tokens."""
    n_accepted = [int(n) for n in n_accepted]
    for i, snaps in result.states.items():
        for b, n in enumerate(n_accepted):
            if n > 0:
                group.state[i][b].copy_(snaps[n - 1][b])
                for dst, src in zip(group.conv[i], result.convs[i][n - 1]):
                    dst[b].copy_(src[b])
    group.set_context([c + n for c, n in zip(group.ctx, n_accepted)])
