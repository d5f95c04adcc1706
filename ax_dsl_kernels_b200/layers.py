"""Decoder sublayers and the hybrid stack, composed from the library's roles (host side, no math of its own).

Mirrors the reference's layer entry points: the GDN sublayer `gdn(hidden_states, residual, weights, temporal_state,
conv_state, ...)` (models/qwen35_35b_a3b/sgl/python/sgl_kernel_axera/attention/gdn.py:2499-2597), the attention
sublayer `flash_attention(x, weights, position_ids, output, cache, indptr, indices, last_page_len, cache_location=...)`
(.../attention/flash_attn.py:2549-2665), the dense SwiGLU block `mlp_block` (models/qwen35_2b/whole/src/q35_step.py:
118-146) and the layer loop `NpuModel.step` (q35_step.py:438-470, pattern g g g a).

Quantised projections are (weight, scale) pairs: MXFP4 / MXFP8 with E8M0 block scales or FP8 E4M3 with per-row fp32
scales (`linear` role).  Everything runs on the GPU through the C ABI; nothing here falls back to torch math.
"""
import torch

from . import _lib
from .attention import paged_attention_decode, paged_attention_prefill
from .gdn import gdn_chunk_prefill, gdn_conv1d_silu, gdn_recurrent_step
from .moe import fuse_rows, linear, linear_multi


def _empty(shape, dtype, like):
    return torch.empty(shape, dtype=dtype, device=like.device)


_scalars = {}


def _scalar(value, device):
    """fp32 [1] tensor holding `value` on `device`, made once (a host-to-device copy per call would break CUDA-graph
    capture of a sublayer and costs more than the kernels it feeds)"""
    key = (float(value), device.type, device.index)
    t = _scalars.get(key)
    if t is None:
        t = _scalars[key] = torch.tensor([float(value)], dtype=torch.float32, device=device)
    return t


def rmsnorm(x, w, residual=None, eps=None, folded=False):
    """plain: y = x_norm * w.  folded (GDN sublayer): y = bf16(base * w) and sqrt(mean base^2 + eps) returned for the
    projections to divide by.  With a residual, base = bf16(x + residual) is returned as well."""
    y = torch.empty_like(x)
    kw = dict(x=x, w=w, y=y)
    base = xsqrt = None
    if residual is not None:
        base = torch.empty_like(x)
        kw.update(residual=residual, base_out=base)
    if folded:
        xsqrt = _empty((x.numel() // x.shape[-1],), torch.float32, x)
        kw["xsqrt_out"] = xsqrt
    if eps is not None:
        kw["eps"] = _scalar(eps, x.device)
    _lib.run("norm.rms", **kw)
    return y, base, xsqrt


def _proj(x, w, name, **kw):
    return linear(x, w["w_" + name], w["s_" + name], **kw)


def finish_residual(base, partial, out=None):
    """out = bf16(base + partial): closes a sublayer whose output projection was summed in fp32 (over tensor-parallel
    ranks) before the residual is added."""
    out = torch.empty_like(base) if out is None else out
    _lib.run("moe.finish", base=base, partial=partial, out=out)
    return out


def gdn(hidden_states, residual, weights, temporal_state, conv_state, *, input_norm_eps=1e-6, o_norm_eps=1e-6,
        reduce=None, in_place=False):
    """GDN sublayer on [B, T, H] (T = 1: recurrent step, T > 1: chunked prefill).  weights: input_norm_w, (w_x, s_x) for
    x in q k v z a b o, w_q_conv / w_k_conv / w_v_conv [C, 4], a_log, dt_bias, o_norm_w.  conv_state: tuple (q, k, v) of
    [B, 3, C] bf16.  Returns (fused [B, T, H], temporal_state_out, conv_state_out) -- the reference returns
    (zeros, residual_out, state_out, conv_out); fused is its residual_out.
    reduce (tensor parallel, weights = this rank's heads): called with the fp32 partial of the output projection
    [B * T, H], returns the sum over ranks; the residual is added after it.
    in_place: the new temporal and conv states overwrite the given tensors (state_out == state_in, as the reference's
    resident state buffers) instead of being returned in fresh ones."""
    w = weights
    B, T, H = hidden_states.shape
    R = B * T
    x2 = hidden_states.reshape(R, H)
    xs, base, xsqrt = rmsnorm(x2, w["input_norm_w"], residual=residual.reshape(R, H), eps=input_norm_eps, folded=True)
    if "w_qkvzab" in w:  # the six projections fused by rows at load time (fuse_layer): one pass over one weight
        proj = dict(zip("qkvzab", linear_multi(xs, w["w_qkvzab"], w["s_qkvzab"], w["n_qkvzab"], row_div=xsqrt)))
    else:
        proj = {n: _proj(xs, w, n, row_div=xsqrt) for n in ("q", "k", "v", "z", "a", "b")}
    KD, VD = proj["q"].shape[1], proj["v"].shape[1]
    NV = w["a_log"].numel()
    DV = VD // NV
    NK = KD // DV
    conv_out = []
    mixed = {}
    for n, st in zip(("q", "k", "v"), conv_state):
        y, so = gdn_conv1d_silu(proj[n].reshape(B, T, -1), w[f"w_{n}_conv"], st, conv_out=st if in_place else None)
        mixed[n] = y
        conv_out.append(so)
    qn = torch.empty_like(mixed["q"]).reshape(R, NK, DV)
    kn = torch.empty_like(qn)
    g = _empty((R, NV), torch.float32, x2)
    beta = _empty((R, NV), torch.bfloat16, x2)
    _lib.run("gdn.prep", q=mixed["q"].reshape(R, NK, DV), k=mixed["k"].reshape(R, NK, DV), a=proj["a"], b=proj["b"],
             a_log=w["a_log"], dt_bias=w["dt_bias"], q_out=qn, k_out=kn, g=g, beta=beta)
    v = mixed["v"].reshape(B, T, NV, DV)
    state_out = temporal_state if in_place else torch.empty_like(temporal_state)
    if T == 1:
        core, state_out = gdn_recurrent_step(qn.reshape(B, NK, DV), kn.reshape(B, NK, DV), v.reshape(B, NV, DV),
                                             g.reshape(B, NV), beta.reshape(B, NV), temporal_state,
                                             state_out=state_out)
    else:
        core, state_out = gdn_chunk_prefill(qn.reshape(B, T, NK, DV), kn.reshape(B, T, NK, DV), v,
                                            g.reshape(B, T, NV), beta.reshape(B, T, NV), temporal_state,
                                            state_out=state_out)
    normed = torch.empty_like(proj["z"]).reshape(R, NV, DV)
    kw = dict(core=core.reshape(R, NV, DV), z=proj["z"].reshape(R, NV, DV), w=w["o_norm_w"], y=normed)
    if o_norm_eps is not None:
        kw["eps"] = _scalar(o_norm_eps, x2.device)
    _lib.run("gdn.out_norm", **kw)
    if reduce is None:
        fused = _proj(normed.reshape(R, VD), w, "o", residual=base)
    else:
        fused = finish_residual(base, reduce(_proj(normed.reshape(R, VD), w, "o", out_dtype=torch.float32)))
    return fused.reshape(B, T, H), state_out, tuple(conv_out)


def attention(x, weights, cos, sin, cache, indptr, indices, last_page_len, *, heads, kv_heads, head_dim,
              cache_location=None, qo_indptr=None, gated=True, sm_scale=None, reduce=None):
    """Attention sublayer.  x [R, H] bf16: R = B sequences x 1 token (decode: the page table describes the HISTORY and
    cache_location [B, 2] says where the new row goes) or the concatenated new tokens of B sequences (prefill:
    qo_indptr [B + 1] given, the page table INCLUDES the new tokens).  weights: ln1 [H] f32 (effective multiplier),
    (w_q, s_q) [HQ * D * (2 if gated), H] per head [q | gate], (w_k, s_k), (w_v, s_v), q_norm, k_norm [D] f32,
    (w_o, s_o).  cos / sin [R, rot / 2] f32.  The cache is updated in place.  Returns x + o_proj(attention).
    reduce: as in gdn() (heads / kv_heads are then this rank's counts)."""
    w = weights
    R, H = x.shape
    n, _, _ = rmsnorm(x, w["ln1"])
    if "w_qkv" in w:
        qg, k, v = linear_multi(n, w["w_qkv"], w["s_qkv"], w["n_qkv"])
        v = v.reshape(R, kv_heads, head_dim)
    else:
        qg = _proj(n, w, "q")
        k = _proj(n, w, "k")
        v = _proj(n, w, "v").reshape(R, kv_heads, head_dim)
    q = _empty((R, heads, head_dim), torch.bfloat16, x)
    kr = _empty((R, kv_heads, head_dim), torch.bfloat16, x)
    kw = dict(qg=qg, k=k, q_norm=w["q_norm"], k_norm=w["k_norm"], cos=cos, sin=sin, q_out=q, k_out=kr)
    gate = None
    if gated:
        gate = torch.empty_like(q)
        kw["gate_out"] = gate
    _lib.run("attn.qk_prep", **kw)
    if qo_indptr is None:
        attn = paged_attention_decode(q, cache, indptr, indices, last_page_len, sm_scale=sm_scale, k_new=kr, v_new=v,
                                      cache_location=cache_location)
    else:
        attn = paged_attention_prefill(q, cache, qo_indptr, indptr, indices, last_page_len, sm_scale=sm_scale,
                                       k_new=kr, v_new=v)
    if gated:
        gated_attn = torch.empty_like(attn)
        _lib.run("act.sigmoid_gate", a=attn, b=gate, y=gated_attn)
        attn = gated_attn
    if reduce is None:
        return _proj(attn.reshape(R, heads * head_dim), w, "o", residual=x)
    return finish_residual(x, reduce(_proj(attn.reshape(R, heads * head_dim), w, "o", out_dtype=torch.float32)))


def mlp_residual(x1, weights, reduce=None):
    """dense SwiGLU block: x1 + down(bf16(silu(gate h) * up h)), h = RMSNorm(x1) * ln2 (q35_step.py:118-146).
    reduce: as in gdn() (gate / up rows and down columns are then this rank's slice of the intermediate size, the
    split of the reference's multi-core form, models/qwen35_2b/whole/src/q35_layer_mc.py:129-136)."""
    w = weights
    h2, _, _ = rmsnorm(x1, w["ln2"])
    if "w_gateup" in w:
        g, u = linear_multi(h2, w["w_gateup"], w["s_gateup"], w["n_gateup"])
    else:
        g = _proj(h2, w, "gate")
        u = _proj(h2, w, "up")
    act = torch.empty_like(g)
    _lib.run("act.silu_mul", a=g, b=u, y=act)
    if reduce is None:
        return _proj(act, w, "down", residual=x1)
    return finish_residual(x1, reduce(_proj(act, w, "down", out_dtype=torch.float32)))


def fuse_layer(weights, kind):
    """A copy of one layer's weight dict with the projections that share an input concatenated by rows (GDN: q k v z a
    b; attention: q+gate k v; MLP: gate up), so that a decode step reads each of them in one launch sequence.  Made once
    at load time; costs one copy of those weights (the separate tensors are dropped from the copy, not from the
    caller's dict).  Layers whose projections differ in format stay as they are."""
    w = dict(weights)
    if kind == "g":
        fuse_rows(w, ("q", "k", "v", "z", "a", "b"), "qkvzab")
    else:
        fuse_rows(w, ("q", "k", "v"), "qkv")
    return fuse_rows(w, ("gate", "up"), "gateup")


class HybridStack:
    """layers of kind "g" (GDN sublayer + MLP) or "a" (attention sublayer + MLP) for ONE sequence, with its recurrent
    states, conv states and paged KV caches (one cache per attention layer, shared page table)."""

    def __init__(self, layers, kinds, *, heads, kv_heads, head_dim, rot, theta, page_size=64, max_tokens=1024,
                 gated=True, reduce=None):
        self.layers, self.kinds = layers, kinds
        self.reduce = reduce  # tensor parallel: layers hold this rank's shards, heads / kv_heads its counts
        self.cfg = dict(heads=heads, kv_heads=kv_heads, head_dim=head_dim)
        self.rot, self.theta, self.P, self.gated = rot, theta, page_size, gated
        dev = layers[0]["ln2"].device
        n_pages = (max_tokens + page_size - 1) // page_size
        self.pos = 0
        self.state, self.conv, self.cache = {}, {}, {}
        for i, (w, kind) in enumerate(zip(layers, kinds)):
            if kind == "g":
                NV = w["a_log"].numel()
                DV = w["o_norm_w"].numel()
                self.state[i] = torch.zeros((1, NV, DV, DV), dtype=torch.float32, device=dev)
                self.conv[i] = tuple(torch.zeros((1, 3, w[f"w_{n}_conv"].shape[0]), dtype=torch.bfloat16, device=dev)
                                     for n in ("q", "k", "v"))
            else:
                self.cache[i] = torch.zeros((n_pages, 2, page_size, kv_heads, head_dim), dtype=torch.bfloat16,
                                            device=dev)
        self.indices = torch.arange(n_pages, dtype=torch.int32, device=dev)
        self.dev = dev

    def _rope(self, positions):
        inv = 1.0 / (self.theta ** (torch.arange(0, self.rot, 2, dtype=torch.int64).float() / self.rot))
        f = positions.float().reshape(-1, 1) * inv.reshape(1, -1)
        return f.cos().to(self.dev).contiguous(), f.sin().to(self.dev).contiguous()

    def forward(self, x):
        """x [T, H] bf16: T = 1 decode, T > 1 prefill of the next T positions.  Returns [T, H]."""
        T = x.shape[0]
        P = self.P
        cos, sin = self._rope(torch.arange(self.pos, self.pos + T))
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=self.dev)  # noqa: E731
        for i, (w, kind) in enumerate(zip(self.layers, self.kinds)):
            if kind == "g":
                zero = torch.zeros_like(x)
                fused, self.state[i], self.conv[i] = gdn(x.reshape(1, T, -1), zero.reshape(1, T, -1), w, self.state[i],
                                                         self.conv[i], reduce=self.reduce)
                x1 = fused.reshape(T, -1)
            elif T == 1:
                hist = self.pos
                x1 = attention(x, w, cos, sin, self.cache[i], i32([0, hist // P + 1]), self.indices, i32([hist % P]),
                               cache_location=i32([[hist // P, hist % P]]), gated=self.gated, reduce=self.reduce, **self.cfg)
            else:
                total = self.pos + T
                npg = (total + P - 1) // P
                x1 = attention(x, w, cos, sin, self.cache[i], i32([0, npg]), self.indices, i32([total - (npg - 1) * P]),
                               qo_indptr=i32([0, T]), gated=self.gated, reduce=self.reduce, **self.cfg)
            x = mlp_residual(x1, w, reduce=self.reduce)
        self.pos += T
        return x


class DecodeGroup:
    """One decode step of a stack of layers for B sequences at once: the batched form of the reference's decode group
    (group_body, models/qwen38_27b/decode/q35_group.py:413-437; decode_qwen35_blocks, models/qwen35_35b_a3b/sgl/python/
    sgl_kernel_axera/models/qwen36_35b_a3b/decode.py:23-110).  Every attention layer owns a paged KV cache
    [B * pages_per_seq, 2, P, HKV, D] over ONE page table shared by the layers (sequence b owns pages
    b * pages_per_seq ...); GDN layers own temporal states [B, NV, DV, DV] and conv states, updated in place.
    The page table, write locations and RoPE rows live on the device and change only in advance(), so step() issues no
    host-to-device copy and can be captured into a CUDA graph.
    reduce: tensor parallel (layers = this rank's shards, heads / kv_heads its counts), as in gdn()."""

    def __init__(self, layers, kinds, *, batch, heads, kv_heads, head_dim, rot, theta, max_tokens, page_size=64,
                 gated=True, reduce=None, kv_dtype=torch.bfloat16, fuse=True):
        self.kinds, self.B = kinds, batch
        # fuse: projections that share an input are concatenated by rows once, here (see fuse_layer)
        self.layers = [fuse_layer(w, k) for w, k in zip(layers, kinds)] if fuse else layers
        layers = self.layers
        self.reduce, self.gated = reduce, gated
        self.cfg = dict(heads=heads, kv_heads=kv_heads, head_dim=head_dim)
        self.rot, self.theta, self.P = rot, theta, page_size
        self.npp = (max_tokens + page_size - 1) // page_size
        dev = layers[0]["ln2"].device
        self.dev = dev
        self.state, self.conv, self.cache = {}, {}, {}
        for i, (w, kind) in enumerate(zip(layers, kinds)):
            if kind == "g":
                NV, DV = w["a_log"].numel(), w["o_norm_w"].numel()
                self.state[i] = torch.zeros((batch, NV, DV, DV), dtype=torch.float32, device=dev)
                self.conv[i] = tuple(torch.zeros((batch, 3, w[f"w_{n}_conv"].shape[0]), dtype=torch.bfloat16, device=dev)
                                     for n in ("q", "k", "v"))
            else:
                self.cache[i] = torch.zeros((batch * self.npp, 2, page_size, kv_heads, head_dim), dtype=kv_dtype,
                                            device=dev)
        self.sm_scale = _scalar(head_dim ** -0.5, dev)
        self.set_context([0] * batch)

    def set_context(self, ctx):
        """history length of every sequence (tokens already in the caches and states)"""
        ctx = [int(c) for c in ctx]
        if len(ctx) != self.B or max(ctx) >= self.npp * self.P:
            raise ValueError("DecodeGroup.set_context: one length per sequence, below the cache size")
        self.ctx = ctx
        P, npp = self.P, self.npp
        n_hist = [(c + P - 1) // P for c in ctx]
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=self.dev)  # noqa: E731
        self.indptr = i32([0, *torch.tensor(n_hist).cumsum(0).tolist()])
        self.indices = i32([b * npp + i for b, n in enumerate(n_hist) for i in range(n)] or [0])
        self.last_page_len = i32([c - (n - 1) * P if n else 0 for c, n in zip(ctx, n_hist)])
        self.cache_location = i32([[b * npp + c // P, c % P] for b, c in enumerate(ctx)])
        inv = 1.0 / (self.theta ** (torch.arange(0, self.rot, 2, dtype=torch.int64).float() / self.rot))
        f = torch.tensor(ctx, dtype=torch.float32).reshape(-1, 1) * inv.reshape(1, -1)
        self.cos, self.sin = f.cos().to(self.dev).contiguous(), f.sin().to(self.dev).contiguous()

    def advance(self):
        """every sequence has taken one more token"""
        self.set_context([c + 1 for c in self.ctx])

    def step(self, x, advance=True):
        """x [B, H] bf16, one token per sequence -> [B, H]"""
        B = self.B
        zero = torch.zeros_like(x)
        for i, (w, kind) in enumerate(zip(self.layers, self.kinds)):
            if kind == "g":
                fused, _, _ = gdn(x.reshape(B, 1, -1), zero.reshape(B, 1, -1), w, self.state[i], self.conv[i],
                                  reduce=self.reduce, in_place=True)
                x1 = fused.reshape(B, -1)
            else:
                x1 = attention(x, w, self.cos, self.sin, self.cache[i], self.indptr, self.indices, self.last_page_len,
                               cache_location=self.cache_location, gated=self.gated, sm_scale=self.sm_scale,
                               reduce=self.reduce, **self.cfg)
            x = mlp_residual(x1, w, reduce=self.reduce)
        if advance:
            self.advance()
        return x
