"""Host side of the gated delta net kernels (reference: gdn_recurrent_step and the conv helper of
models/qwen35_35b_a3b/sgl/python/sgl_kernel_axera/attention/gdn.py:952-989, 187-251)."""
import torch

from . import _lib


def gdn_recurrent_step(q, k, v, g, beta, state_in, o=None, state_out=None):
    """one token per sequence: S *= exp(g); p = k.S; err = (v - p) * beta; S += k (x) err; o = q.S.
    q, k [B, NK, 128] bf16 (L2-normalised, q already scaled), v [B, NV, 128] bf16, g [B, NV] fp32, beta [B, NV] bf16,
    state_in [B, NV, 128, 128] fp32.  state_out may be state_in (in place)."""
    o = torch.empty_like(v) if o is None else o
    state_out = state_in if state_out is None else state_out
    _lib.run("gdn.step", q=q, k=k, v=v, g=g, beta=beta, state_in=state_in, o=o, state_out=state_out)
    return o, state_out


def gdn_conv1d_silu(x, conv_w, conv_in, y=None, conv_out=None):
    """causal depthwise conv1d + SiLU with state: x [B, T, C] bf16, conv_w [C, KW] (checkpoint tap order),
    conv_in [B, KW-1, C] oldest row first.  Returns (y, conv_out)."""
    y = torch.empty_like(x) if y is None else y
    conv_out = torch.empty_like(conv_in) if conv_out is None else conv_out
    _lib.run("gdn.conv", x=x, conv_w=conv_w.reshape(conv_w.shape[0], -1), conv_in=conv_in, y=y, conv_out=conv_out)
    return y, conv_out


def gdn_chunk_prefill(q, k, v, g, beta, state_in, o=None, state_out=None):
    """T tokens of the gated delta rule in chunks of 64 (the prefill form of gdn_recurrent_step; reference
    gdn_stable_chunk, models/qwen35_35b_a3b/sgl/python/sgl_kernel_axera/attention/gdn.py:1122-1212).
    q, k [B, T, NK, 128] bf16 (L2-normalised, q scaled by 128^-0.5), v [B, T, NV, 128] bf16, g [B, T, NV] fp32,
    beta [B, T, NV] bf16, state_in [B, NV, 128, 128] fp32.  Returns (o [B, T, NV, 128] bf16, state_out)."""
    o = torch.empty_like(v) if o is None else o
    state_out = torch.empty_like(state_in) if state_out is None else state_out
    _lib.run("gdn.chunk_prefill", q=q, k=k, v=v, g=g, beta=beta, state_in=state_in, o=o, state_out=state_out)
    return o, state_out
