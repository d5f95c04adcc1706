"""Hybrid decoder stack on the CPU (oracle; test infrastructure only): layers of GDN sublayer + dense SwiGLU block
("g") or gated attention sublayer + dense SwiGLU block ("a"), pattern g g g a as the reference's layer loop
(models/qwen35_2b/whole/src/q35_step.py:438-470).  Weights are DEQUANTISED fp32 (the reference checks its kernels
against torch on the quantise -> dequantise round trip, models/qwen35_2b/whole/src/q35_moe.py:281-282)."""
import torch
import torch.nn.functional as F

from . import attention as oattn
from . import gdn as ogdn
from .moe import bf, rmsnorm


def dense_mlp(x1, ln2, w_gate, w_up, w_down, eps=1e-6):
    """x1 + down(bf16(silu(gate h) * up h)), h = RMSNorm(x1) * ln2; projections round to bf16
    (mlp_block, models/qwen35_2b/whole/src/q35_step.py:118-146)."""
    h = rmsnorm(x1, ln2, eps).float()
    g, u = bf(h @ w_gate.float().T), bf(h @ w_up.float().T)
    act = bf(F.silu(g) * u)
    return (x1.float() + bf(act @ w_down.float().T)).to(torch.bfloat16)


def attn_sublayer(x, w, cache, indptr, indices, last_page_len, cos, sin, *, heads, kv_heads, head_dim, rot, gated=True,
                  qo_indptr=None, cache_location=None, eps=1e-6):
    """decode (qo_indptr None: one token per sequence, page table = history, row written at cache_location) or prefill
    (page table includes the new tokens, rows written at their positions); golden structure of
    models/qwen35_35b_a3b/sgl/tests/test_qwen35_runtime.py:57-93."""
    if qo_indptr is None:
        out, _, _, _ = oattn.attn_layer_decode(x, w, cache, indptr, indices, last_page_len, cache_location, cos, sin,
                                               heads=heads, kv_heads=kv_heads, head_dim=head_dim, rot=rot, gated=gated,
                                               eps=eps)
        return out
    R = x.shape[0]
    n = rmsnorm(x, w["ln1"], eps).float()
    qg = bf(n @ w["w_q"].float().T).reshape(R, heads, -1)
    q, gate = (qg[..., :head_dim], qg[..., head_dim:]) if gated else (qg, None)
    k = bf(n @ w["w_k"].float().T).reshape(R, kv_heads, head_dim)
    v = bf(n @ w["w_v"].float().T).reshape(R, kv_heads, head_dim).to(torch.bfloat16)
    q = oattn.rope_neox(rmsnorm(q, w["q_norm"], eps), cos[:, None, :], sin[:, None, :], rot)
    k = oattn.rope_neox(rmsnorm(k, w["k_norm"], eps), cos[:, None, :], sin[:, None, :], rot)
    P = cache.shape[2]
    for b in range(qo_indptr.numel() - 1):
        q0, q1 = int(qo_indptr[b]), int(qo_indptr[b + 1])
        total = int(oattn.valid_kv_len(indptr, last_page_len, P)[b])
        for i in range(q1 - q0):
            pos = total - (q1 - q0) + i
            page = int(indices[int(indptr[b]) + pos // P])
            cache[page, 0, pos % P] = k[q0 + i]
            cache[page, 1, pos % P] = v[q0 + i]
    attn = oattn.paged_prefill(q, cache, qo_indptr, indptr, indices, last_page_len).float()
    if gated:
        attn = bf(attn * torch.sigmoid(gate))
    o = bf(attn.reshape(R, -1) @ w["w_o"].float().T)
    return (x.float() + o).to(torch.bfloat16)


class HybridStack:
    def __init__(self, layers, kinds, *, heads, kv_heads, head_dim, rot, theta, page_size=64, max_tokens=1024, gated=True):
        self.layers, self.kinds = layers, kinds
        self.cfg = dict(heads=heads, kv_heads=kv_heads, head_dim=head_dim, rot=rot, gated=gated)
        self.theta, self.P, self.rot = theta, page_size, rot
        n_pages = (max_tokens + page_size - 1) // page_size
        self.pos = 0
        self.state, self.conv, self.cache = {}, {}, {}
        for i, (w, kind) in enumerate(zip(layers, kinds)):
            if kind == "g":
                NV, DV = w["a_log"].numel(), w["o_norm_w"].numel()
                self.state[i] = torch.zeros((1, NV, DV, DV))
                width = w["w_q"].shape[0] * 2 + w["w_v"].shape[0]
                self.conv[i] = torch.zeros((1, 3, width), dtype=torch.bfloat16)
            else:
                self.cache[i] = torch.zeros((n_pages, 2, page_size, kv_heads, head_dim), dtype=torch.bfloat16)
        self.indices = torch.arange(n_pages, dtype=torch.int32)

    def forward(self, x):
        T, P = x.shape[0], self.P
        cos, sin = oattn.rope_cos_sin(torch.arange(self.pos, self.pos + T), self.rot, self.theta)
        i32 = lambda v: torch.tensor(v, dtype=torch.int32)  # noqa: E731
        for i, (w, kind) in enumerate(zip(self.layers, self.kinds)):
            if kind == "g":
                fused, self.state[i], self.conv[i] = ogdn.gdn_sublayer(x.reshape(1, T, -1), torch.zeros_like(x).reshape(1, T, -1),
                                                                        w, self.state[i], self.conv[i])
                x1 = fused.reshape(T, -1)
            elif T == 1:
                hist = self.pos
                x1 = attn_sublayer(x, w, self.cache[i], i32([0, hist // P + 1]), self.indices, i32([hist % P]), cos, sin,
                                   cache_location=i32([[hist // P, hist % P]]), **self.cfg)
            else:
                total = self.pos + T
                npg = (total + P - 1) // P
                x1 = attn_sublayer(x, w, self.cache[i], i32([0, npg]), self.indices, i32([total - (npg - 1) * P]), cos,
                                   sin, qo_indptr=i32([0, T]), **self.cfg)
            x = dense_mlp(x1, w["ln2"], w["w_gate"], w["w_up"], w["w_down"])
        self.pos += T
        return x
