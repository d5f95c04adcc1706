"""Speculative-decode pieces of the 27B-class group (CPU oracle; test infrastructure only).

mtp_step restates the reference's MTP block golden (models/qwen38_27b/mtp/mtp_ref.py:172-239): the row at position p
pairs the embedding of token x_p with the target model's final-norm hidden h_(p-1):
    z = fc([enorm(e) | hnorm(h)]);  y = DecoderLayer(z, the block's own KV at position p);  h_next = head_norm(y)
The decoder layer is a gated attention sublayer (q / k RMSNorm, partial NeoX RoPE, causal attention over the block's
paged KV, sigmoid gate, o-proj + residual) and a dense SwiGLU block.  Everything in fp32, as the golden computes it.
The 4-row verify has no golden of its own in the reference beyond "the rows equal four decode steps"; the tests use the
oracle stack token by token for it."""
import torch
import torch.nn.functional as F

EPS = 1e-6


def rmsnorm(x, w):
    xf = x.float()
    return xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + EPS) * w.float()


def rope(x, pos, rot, theta):
    """mtp_ref.py:163-170: NeoX halves on the first rot channels"""
    half = rot // 2
    inv = 1.0 / (theta ** (torch.arange(0, rot, 2, dtype=torch.float64) / rot))
    ang = torch.tensor(float(pos), dtype=torch.float64) * inv
    cos, sin = ang.cos().float(), ang.sin().float()
    y = x.clone()
    x1, x2 = x[..., :half], x[..., half:rot]
    y[..., :half] = x1 * cos - x2 * sin
    y[..., half:rot] = x2 * cos + x1 * sin
    return y


def mtp_step(e, h, pos, kv, a, *, heads, kv_heads, head_dim, rot=64, theta=1e7, block=256):
    """one MTP row (mtp_ref.py:202-239).  e, h [H]; kv [pages, 2, block, HKV * D] bf16, appended to at `pos`;
    a: DEQUANTISED weights and effective norm multipliers by the reference's names.  Returns (h_next, y) fp32 [H]."""
    H = e.numel()
    HQ, HKV, D = heads, kv_heads, head_dim
    en, hn = rmsnorm(e.reshape(H), a["ln_e"]), rmsnorm(h.reshape(H), a["ln_h"])
    z = torch.cat([en, hn]).reshape(1, 2 * H) @ a["w_fc"].float().T
    x = rmsnorm(z, a["ln1"]).reshape(H)
    qg = (x.reshape(1, H) @ a["w_q"].float().T).reshape(HQ, 2 * D)
    q = rmsnorm(qg[:, :D], a["q_norm"])
    gate = qg[:, D:]
    k = rmsnorm((x.reshape(1, H) @ a["w_k"].float().T).reshape(HKV, D), a["k_norm"])
    v = (x.reshape(1, H) @ a["w_v"].float().T).reshape(HKV, D)
    q, k = rope(q, pos, rot, theta), rope(k, pos, rot, theta)
    page, cell = divmod(pos, block)
    kv[page, 0, cell] = k.reshape(HKV * D).bfloat16()
    kv[page, 1, cell] = v.reshape(HKV * D).bfloat16()
    rows = [divmod(p, block) for p in range(pos + 1)]
    kb = torch.stack([kv[pg, 0, c].float().reshape(HKV, D) for pg, c in rows], 0)
    vb = torch.stack([kv[pg, 1, c].float().reshape(HKV, D) for pg, c in rows], 0)
    g = HQ // HKV
    scores = torch.einsum("hgd,phd->ghp", q.reshape(HKV, g, D).float(), kb) * (D ** -0.5)
    attn = torch.einsum("ghp,phd->hgd", torch.softmax(scores, dim=-1), vb).reshape(HQ * D)
    attn = attn * torch.sigmoid(gate.float().reshape(HQ * D))
    x1 = z.reshape(H) + attn.reshape(1, HQ * D) @ a["w_o"].float().T
    h2 = rmsnorm(x1, a["ln2"])
    act = F.silu(h2.reshape(1, H) @ a["w_gate"].float().T) * (h2.reshape(1, H) @ a["w_up"].float().T)
    y = (x1 + act @ a["w_down"].float().T).reshape(H)
    return rmsnorm(y, a["head_norm"]), y
