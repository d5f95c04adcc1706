"""Gated delta net layer of the Qwen3.5 decoder (CPU oracle; test infrastructure only).

Restates the reference's torch goldens in models/qwen35_35b_a3b/sgl/tests/test_gdn_attn.py: value heads in grouped
(Hugging Face) order, key head = value head // (NV / NK); conv taps in checkpoint order (oldest first).
"""
import torch
import torch.nn.functional as F


def causal_conv1d_silu(x, weight, state_in):
    """depthwise causal conv over [state; x] then SiLU; taps accumulate with a bf16 rounding per tap
    (test_gdn_attn.py:241-257).  x [B, T, C] bf16, weight [C, K] bf16 (column K-1 multiplies the current token),
    state_in [B, K-1, C] bf16 oldest row first.  Returns (y [B, T, C] bf16, state_out [B, K-1, C])."""
    state_len = state_in.shape[1]
    ksz = weight.shape[1]
    assert state_len == ksz - 1
    conv_in = torch.cat((state_in, x), dim=1)
    out = torch.zeros_like(x)
    for off in range(ksz):
        s0 = state_len - off
        term = conv_in[:, s0:s0 + x.shape[1], :].float() * weight[:, ksz - 1 - off].float().reshape(1, 1, -1)
        out = (out.float() + term).to(x.dtype)
    state_out = conv_in[:, -state_len:, :] if state_len else conv_in[:, :0, :]
    return F.silu(out.float()).to(x.dtype), state_out


def l2norm(x, eps=1e-6):
    """x / sqrt(sum x^2 + eps) -> bf16 (test_gdn_attn.py:264-265;
    models/qwen35_35b_a3b/sgl/python/sgl_kernel_axera/attention/gdn.py:919-931)."""
    xf = x.float()
    return (xf / torch.sqrt(xf.square().sum(-1, keepdim=True) + eps)).to(torch.bfloat16)


def gates(a, b, a_log, dt_bias):
    """g = -exp(A_log) * softplus(a + dt_bias) fp32, beta = sigmoid(b) bf16 (test_gdn_attn.py:267-270; gdn.py:934-949).
    a, b [B, T, NV] bf16; a_log, dt_bias [NV]."""
    nv = a.shape[-1]
    g = -torch.exp(a_log.float()).reshape(1, 1, nv) * F.softplus(a.float() + dt_bias.float().reshape(1, 1, nv))
    return g, torch.sigmoid(b.float()).to(torch.bfloat16)


def recurrent(q, k, v, g, beta, state_in):
    """token-by-token gated delta rule (the loop of gdn_reference, test_gdn_attn.py:272-296; kernel
    gdn_recurrent_step gdn.py:952-989).  q [B, T, NK, DK] bf16 already L2-normalised and scaled by DK^-0.5,
    k [B, T, NK, DK] bf16 L2-normalised, v [B, T, NV, DV] bf16, g [B, T, NV] fp32, beta [B, T, NV] bf16,
    state_in [B, NV, DK, DV] fp32.  Per token and value head:
      S *= exp(g); p = bf16(k . S); err = bf16(bf16(v - p) * beta); S += k (x) err; o = bf16(q . S)."""
    B, T, NV, DV = v.shape
    rep = NV // q.shape[2]
    state = state_in.clone().float()
    out = torch.empty(v.shape, dtype=torch.bfloat16)
    kh = torch.arange(NV) // rep
    for t in range(T):
        kt = k[:, t, kh].float()  # [B, NV, DK]
        qt = q[:, t, kh].float()
        state *= torch.exp(g[:, t]).reshape(B, NV, 1, 1)
        pred = torch.einsum("bhk,bhkv->bhv", kt, state).to(torch.bfloat16)
        err = ((v[:, t].float() - pred.float()).to(torch.bfloat16).float()
               * beta[:, t].float().reshape(B, NV, 1)).to(torch.bfloat16)
        state += torch.einsum("bhk,bhv->bhkv", kt, err.float())
        out[:, t] = torch.einsum("bhk,bhkv->bhv", qt, state).to(torch.bfloat16)
    return out, state


def gdn_core(q, k, v, a, b, a_log, dt_bias, state_in):
    """gdn_reference (test_gdn_attn.py:260-296): L2 norms, q scale, gates, recurrence."""
    dk = q.shape[-1]
    qn = (l2norm(q).float() * dk ** -0.5).to(torch.bfloat16)
    kn = l2norm(k)
    g, beta = gates(a, b, a_log, dt_bias)
    return recurrent(qn, kn, v, g, beta, state_in)


def linear_bf16(x, w):
    return torch.matmul(x.float(), w.float().transpose(-1, -2)).to(torch.bfloat16)


def gdn_sublayer(hidden, residual, w, temporal_state, conv_state, input_norm_eps=1e-6, o_norm_eps=1e-6):
    """whole GDN sublayer (reference(), test_gdn_attn.py:427-474): residual add -> folded RMSNorm
    (bf16(x * w) -> projection -> / sqrt(mean x^2 + eps)) -> q/k/v conv+SiLU -> recurrence -> gated RMSNorm * SiLU(z)
    -> out projection + residual.  w holds (dequantized) w_q, w_k, w_v, w_z, w_a, w_b, w_*_conv [C, K], a_log,
    dt_bias, o_norm_w, w_o, input_norm_w.  conv_state [B, K-1, 2 KD + VD] = q | k | v channels.
    Returns (fused [B, T, H] bf16, state_out fp32, conv_state_out)."""
    batch, seq, _ = hidden.shape
    kw, vw = w["w_q"].shape[0], w["w_v"].shape[0]
    nv, dk, dv = temporal_state.shape[1:]
    nk = kw // dk
    qs, ks, vs = torch.split(conv_state, (kw, kw, vw), dim=-1)
    base = (hidden.float() + residual.float()).to(torch.bfloat16)
    xs = (base.float() * w["input_norm_w"].float().reshape(1, 1, -1)).to(torch.bfloat16)
    xr = torch.sqrt(base.float().square().mean(-1, keepdim=True) + input_norm_eps)

    def project(name):
        return (linear_bf16(xs, w[name]).float() / xr).to(torch.bfloat16)

    q, qso = causal_conv1d_silu(project("w_q"), w["w_q_conv"], qs)
    k, kso = causal_conv1d_silu(project("w_k"), w["w_k_conv"], ks)
    v, vso = causal_conv1d_silu(project("w_v"), w["w_v_conv"], vs)
    q = q.reshape(batch, seq, nk, dk)
    k = k.reshape(batch, seq, nk, dk)
    v = v.reshape(batch, seq, nv, dv)
    z = project("w_z").reshape(batch, seq, nv, dv)
    core, st = gdn_core(q, k, v, project("w_a"), project("w_b"), w["a_log"], w["dt_bias"], temporal_state)
    var = core.float().square().mean(-1, keepdim=True)
    normed = (core.float() * torch.rsqrt(var + o_norm_eps) * w["o_norm_w"].float().reshape(1, 1, 1, dv)).to(torch.bfloat16)
    normed = (normed.float() * F.silu(z.float()).to(torch.bfloat16).float()).to(torch.bfloat16)
    attn = linear_bf16(normed.reshape(batch, seq, nv * dv), w["w_o"])
    fused = (base.float() + attn.float()).to(torch.bfloat16)
    return fused, st, torch.cat((qso, kso, vso), dim=-1)


def recurrent_f64(q, k, v, g, beta, state_in):
    """the same recurrence without any intermediate rounding, in float64: the cross-check used by the CPU tests and
    the yardstick for the chunked prefill kernel's own rounding."""
    B, T, NV, DV = v.shape
    rep = NV // q.shape[2]
    S = state_in.double().clone()
    out = torch.empty(v.shape, dtype=torch.float64)
    kh = torch.arange(NV) // rep
    for t in range(T):
        kt, qt = k[:, t, kh].double(), q[:, t, kh].double()
        S *= torch.exp(g[:, t].double()).reshape(B, NV, 1, 1)
        pred = torch.einsum("bhk,bhkv->bhv", kt, S)
        err = (v[:, t].double() - pred) * beta[:, t].double().reshape(B, NV, 1)
        S += torch.einsum("bhk,bhv->bhkv", kt, err)
        out[:, t] = torch.einsum("bhk,bhkv->bhv", qt, S)
    return out, S
