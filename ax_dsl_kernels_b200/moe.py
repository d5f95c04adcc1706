"""Host side of the MoE block, mirroring the reference's kernel entry points by name and argument meaning.

Reference entry points (models/qwen35_2b/whole/src/): q35_moe.py `route` (:293-297), `moe_pre` (:123-137),
`moe_experts` / `moe_experts_gu` (:73-112); q35_moe_prefill.py `moe_slots_px(h2, tok, rw, e_gw, e_gs, e_dw, e_ds, out)`
(:150-166) and `moe_combine(base, loc, sout, out)` (:201-214).  Outputs are caller-allocated tensors, as there.
"""
import torch

from . import _lib


def _u8(t):
    return t.view(torch.uint8) if t.dtype != torch.uint8 else t


def route(logits, top_k, ids=None, rw=None):
    """softmax over all experts -> top-k -> weights / their sum, per token.  logits [T, NE] fp32 on the GPU.
    Returns (ids [T, K] int32, rw [T, K] fp32); exact ties go to the lower expert id."""
    if logits.dtype != torch.float32:
        raise TypeError("route: logits must be float32")
    lg = logits.reshape(-1, logits.shape[-1])
    T = lg.shape[0]
    ids = torch.empty((T, top_k), dtype=torch.int32, device=lg.device) if ids is None else ids
    rw = torch.empty((T, top_k), dtype=torch.float32, device=lg.device) if rw is None else rw
    _lib.run("moe.route", logits=lg, ids=ids, rw=rw)
    return ids, rw


def moe_pre(x1, ln2, w_gate, s_gate, w_up, s_up, w_down, s_down, w_router, w_shg, out, h2_out, logits_out):
    """dense part of the block: out = x1 + sigmoid(h2 . w_shg) * shared_expert(h2), h2 = RMSNorm(x1) * ln2,
    logits = h2 @ w_router^T (fp32).  Shared-expert weights MXFP4 (uint8 pairs) or MXFP8 (e4m3), E8M0 scales."""
    _lib.run("moe.pre", x1=x1, ln2=ln2, w_gate=w_gate, s_gate=_u8(s_gate), w_up=w_up, s_up=_u8(s_up), w_down=w_down,
             s_down=_u8(s_down), w_router=w_router, w_shg=w_shg.reshape(-1), out=out, h2_out=h2_out,
             logits_out=logits_out)
    return out, h2_out, logits_out


def moe_experts(h2, base, ids, rw, e_gw, e_gs, e_dw, e_ds, out, e_gs_tiled=None, e_ds_tiled=None):
    """out[t] = base[t] + sum_i rw[t, i] * down_e(silu(gate_e h2[t]) * up_e h2[t]), e = ids[t, i].
    Planar MXFP4 expert tensors (gate rows then up rows in e_gw), picked on the device by id; at batch 1 this is the
    reference's moe_experts_gu with the K experts bound by address.  With the tiled scale tensors of
    prepare_moe_weights() a decode-sized batch runs as one persistent gate-up + down kernel."""
    kw = dict(h2=h2, base=base, ids=ids, rw=rw, e_gw=_u8(e_gw), e_gs=_u8(e_gs), e_dw=_u8(e_dw), e_ds=_u8(e_ds), out=out)
    if e_gs_tiled is not None:
        kw.update(e_gs_tiled=e_gs_tiled, e_ds_tiled=e_ds_tiled)
    _lib.run("moe.experts", **kw)
    return out


def moe_slots_px(h2, tok, rw, e_gw, e_gs, e_dw, e_ds, out, n_slots=None):
    """slot s = expert tok[s, 0] on the G token rows tok[s, 1:] of h2; out[s, g] = rw[s, g] * expert(h2[tok]).
    n_slots (int32 [1], optional): slots at or beyond it are skipped and their rows zeroed."""
    kw = dict(h2=h2, tok=tok, rw=rw, e_gw=_u8(e_gw), e_gs=_u8(e_gs), e_dw=_u8(e_dw), e_ds=_u8(e_ds), out=out)
    if n_slots is not None:
        kw["n_slots"] = n_slots
    _lib.run("moe.slots", **kw)
    return out


def moe_combine(base, loc, sout, out):
    """out[t] = base[t] + sum_k sout[loc[k, t]] (fp32 accumulate, bf16 out)."""
    _lib.run("moe.combine", base=base, loc=loc, sout=sout.reshape(-1, sout.shape[-1]), out=out)
    return out


def moe_permute(ids, rw, n_experts, G, S=None):
    """token -> slot tables for the slot kernels: experts in id order, each expert's tokens in index order,
    ceil(n / G) slots per expert (unused rows: token 0 with weight 0).
    Returns tok [S, 1+G] i32, srw [S, G] f32, loc [K, T] i32, n_slots i32 [1], counts [NE] i32."""
    T, K = ids.shape
    if S is None:
        S = min(T * K, (T * K + G - 1) // G + n_experts)
    dev = ids.device
    tok = torch.empty((S, 1 + G), dtype=torch.int32, device=dev)
    srw = torch.empty((S, G), dtype=torch.float32, device=dev)
    loc = torch.empty((K, T), dtype=torch.int32, device=dev)
    n_slots = torch.empty((1,), dtype=torch.int32, device=dev)
    counts = torch.empty((n_experts,), dtype=torch.int32, device=dev)
    _lib.run("moe.permute", ids=ids, rw=rw, tok=tok, srw=srw, loc=loc, n_slots=n_slots, counts=counts)
    return tok, srw, loc, n_slots, counts


_side_streams = {}
_block_bufs = {}


def _side_stream(dev):
    key = (dev.type, dev.index)
    if key not in _side_streams:
        _side_streams[key] = torch.cuda.Stream(device=dev)
    return _side_streams[key]


def tile_scales(s, paired):
    """E8M0 scales [planes, rows, K/32] (or [rows, K/32]) re-laid into the 512-byte blocks the decode kernel copies to
    tensor memory (roles mx.tile_scales.paired / .plain): a load-time conversion, same bytes in another order.
    paired: rows = gate rows followed by up rows, a tile takes 64 of each."""
    s = _u8(s).contiguous()
    out = torch.empty_like(s)
    _lib.run("mx.tile_scales.paired" if paired else "mx.tile_scales.plain", s=s, out=out)
    return out


def prepare_moe_weights(w):
    """adds the tiled scale tensors the one-call decode block (`moe.block`) reads -- e_gs_tiled, e_ds_tiled and, for an
    MXFP4 shared expert, s_gate_up_tiled, s_down_tiled -- to a weight dict, once, at load time.  Returns the dict."""
    if "e_gs_tiled" not in w:
        w["e_gs_tiled"] = tile_scales(w["e_gs"], True)
        w["e_ds_tiled"] = tile_scales(w["e_ds"], False)
        if "w_gate" in w and w["w_gate"].dtype == torch.uint8:
            w["s_gate_up_tiled"] = tile_scales(torch.cat([_u8(w["s_gate"]), _u8(w["s_up"])], 0), True)
            w["s_down_tiled"] = tile_scales(w["s_down"], False)
    return w


def _one_call_ok(x1, w, top_k):
    """shapes the one-call decode block takes: tiled scales present, decode-sized batch, MXFP4 shared expert of the
    routed experts' shape, sizes that are multiples of 512"""
    if "e_gs_tiled" not in w or "s_gate_up_tiled" not in w:
        return False
    T, H = x1.shape
    NE, FE2 = w["e_gw"].shape[0], w["e_gw"].shape[1]
    return (T * top_k <= 4096 and NE * ((T + 31) // 32) <= 4096 and NE < 1024 and H % 512 == 0 and H <= 8192
            and (FE2 // 2) % 512 == 0 and w["w_gate"].shape[0] == FE2 // 2 and w["w_router"].shape[0] == NE)


def moe_block(x1, w, top_k, out=None, overlap=True):
    """whole block on T tokens: dense part -> router -> routed experts.  w: dict with ln2, w_gate, s_gate, w_up,
    s_up, w_down, s_down, w_router, w_shg, e_gw, e_gs, e_dw, e_ds.  Returns (out, ids, rw, logits); ids, rw and logits
    are scratch tensors of this module, valid until the next call with the same shapes (clone them to keep them).

    A weight dict that went through prepare_moe_weights() takes the one-call decode form (role `moe.block`: five
    launches on one stream) for decode-sized batches.  Otherwise: overlap=True runs the shared expert on a second
    stream while the main stream routes and runs the routed experts (the two only meet in the final sum);
    overlap=False is the plain moe_pre -> route -> moe_experts sequence."""
    T, H = x1.shape
    dev = x1.device
    NE = w["w_router"].shape[0]
    key = (dev.index, T, H, NE, top_k)
    bufs = _block_bufs.get(key)
    if bufs is None:
        bufs = _block_bufs[key] = dict(
            base=torch.empty_like(x1), h2=torch.empty_like(x1),
            logits=torch.empty((T, NE), dtype=torch.float32, device=dev),
            gate=torch.empty((T,), dtype=torch.float32, device=dev),
            partial=torch.empty((T, H), dtype=torch.float32, device=dev),
            ids=torch.empty((T, top_k), dtype=torch.int32, device=dev),
            rw=torch.empty((T, top_k), dtype=torch.float32, device=dev))
    base, h2, logits = bufs["base"], bufs["h2"], bufs["logits"]
    out = torch.empty_like(x1) if out is None else out
    if overlap and _one_call_ok(x1, w, top_k):
        _lib.run("moe.block", x1=x1, ln2=w["ln2"], w_router=w["w_router"], w_shg=w["w_shg"].reshape(-1),
                 w_gate=w["w_gate"], w_up=w["w_up"], w_down=w["w_down"], s_gate_up_tiled=w["s_gate_up_tiled"],
                 s_down_tiled=w["s_down_tiled"], e_gw=_u8(w["e_gw"]), e_dw=_u8(w["e_dw"]), e_gs_tiled=w["e_gs_tiled"],
                 e_ds_tiled=w["e_ds_tiled"], out=out, ids=bufs["ids"], rw=bufs["rw"], logits_out=logits, h2_out=h2)
        return out, bufs["ids"], bufs["rw"], logits
    if not overlap:
        moe_pre(x1, w["ln2"], w["w_gate"], w["s_gate"], w["w_up"], w["s_up"], w["w_down"], w["s_down"], w["w_router"],
                w["w_shg"], base, h2, logits)
        ids, rw = route(logits, top_k, bufs["ids"], bufs["rw"])
        moe_experts(h2, base, ids, rw, w["e_gw"], w["e_gs"], w["e_dw"], w["e_ds"], out)
        return out, ids, rw, logits
    _lib.run("moe.norm_router", x1=x1, ln2=w["ln2"], w_router=w["w_router"], w_shg=w["w_shg"].reshape(-1), h2_out=h2,
             logits_out=logits, gate_out=bufs["gate"])
    main, side = torch.cuda.current_stream(dev), _side_stream(dev)
    side.wait_stream(main)
    with torch.cuda.stream(side):
        _lib.run("moe.shared", x1=x1, h2=h2, gate=bufs["gate"], w_gate=w["w_gate"], s_gate=_u8(w["s_gate"]),
                 w_up=w["w_up"], s_up=_u8(w["s_up"]), w_down=w["w_down"], s_down=_u8(w["s_down"]), out=base)
    ids, rw = route(logits, top_k, bufs["ids"], bufs["rw"])
    _lib.run("moe.experts", h2=h2, ids=ids, rw=rw, e_gw=_u8(w["e_gw"]), e_gs=_u8(w["e_gs"]), e_dw=_u8(w["e_dw"]),
             e_ds=_u8(w["e_ds"]), partial_out=bufs["partial"])
    main.wait_stream(side)
    _lib.run("moe.finish", base=base, partial=bufs["partial"], out=out)
    return out, ids, rw, logits


def linear(x, w, s, out=None, bias=None, out_dtype=torch.bfloat16, row_div=None, residual=None, s2=None):
    """x [T, K] bf16 times a quantised weight [N, K]: MXFP4 (uint8 [N, K/2] + E8M0 [N, K/32]), MXFP8 (e4m3 [N, K] +
    E8M0), FP8 per-row (e4m3 [N, K] + fp32 [N]; fp8_gemm with scale_a = 1,
    models/qwen35_35b_a3b/sgl/python/sgl_kernel_axera/gemm.py:457-466) or NVFP4 (uint8 [N, K/2] + float8_e4m3fn scales
    [N, K/16] + the fp32 tensor scale s2 [1]; quantize_nvfp4, .../sgl_kernel_axera/quantization.py:8-37)."""
    T, N = x.shape[0], w.shape[0]
    out = torch.empty((T, N), dtype=out_dtype, device=x.device) if out is None else out
    kw = dict(x=x, w=w, s=s if s.dtype in (torch.float32, torch.float8_e4m3fn) else _u8(s), out=out)
    if s2 is not None:
        kw["s2"] = s2
    if bias is not None:
        kw["bias"] = bias
    if row_div is not None:  # per-token divisor applied to the bf16-rounded product (folded RMSNorm of the GDN sublayer)
        kw["row_div"] = row_div
    if residual is not None:  # out = residual + bf16(product)
        kw["residual"] = residual
    _lib.run("linear", **kw)
    return out


def linear_multi(x, w, s, sizes, row_div=None, bias=None, out_dtype=torch.bfloat16):
    """Several projections of one input as ONE launch sequence (one quantisation of x, one pass over the weights, one
    reduction): w / s are the projections' weights and scales concatenated by rows, sizes their row counts in that
    order.  Returns one [T, N_i] tensor per projection.  The reference fuses the same rows into one weight (w_qkv of
    its GDN kernels, models/qwen35_35b_a3b/qwen35_35b_a3b.manifest.json `prefill64.gdn`)."""
    if len(sizes) > 8 or sum(sizes) != w.shape[0]:
        raise ValueError("linear_multi: at most 8 projections whose rows add up to the weight's")
    T = x.shape[0]
    outs = [torch.empty((T, n), dtype=out_dtype, device=x.device) for n in sizes]
    kw = dict(x=x, w=w, s=s if s.dtype in (torch.float32, torch.float8_e4m3fn) else _u8(s))
    kw.update({f"out{i}": o for i, o in enumerate(outs)})
    if row_div is not None:
        kw["row_div"] = row_div
    if bias is not None:
        kw["bias"] = bias
    _lib.run("linear.multi", **kw)
    return outs


def fuse_rows(weights, names, fused):
    """adds `w_<fused>`, `s_<fused>` (rows of the projections `names` concatenated, one copy made at load time) and
    `n_<fused>` (their row counts) to a weight dict and drops the separate entries.  No-op when the projections differ
    in format or one is missing."""
    ws, ss = [weights.get("w_" + n) for n in names], [weights.get("s_" + n) for n in names]
    if any(t is None for t in ws + ss) or len({t.dtype for t in ws}) != 1 or len({t.dtype for t in ss}) != 1 or \
            len({t.shape[1] for t in ws}) != 1 or len({t.dim() for t in ss}) != 1:
        return weights
    weights["w_" + fused] = torch.cat(ws, 0).contiguous()
    weights["s_" + fused] = torch.cat(ss, 0).contiguous()
    weights["n_" + fused] = [int(t.shape[0]) for t in ws]
    for n in names:
        del weights["w_" + n], weights["s_" + n]
    return weights


def lm_head(x, w, s, logits=None, token=None, want_logits=True, want_token=True):
    """MXFP4 output projection: fp32 logits [T, N] and / or the greedy token [T] (first index of the row maximum).
    Reference: mul_mat_mx4 (models/qwen35_2b/whole/src/q35_layer_mc.py:741-758), golden torch_logits
    (models/qwen38_27b/head/mx4_common.py:62-69).  K must be a multiple of 512."""
    T, N = x.shape[0], w.shape[0]
    kw = dict(x=x, w=w, s=_u8(s))
    if want_logits or logits is not None:
        logits = torch.empty((T, N), dtype=torch.float32, device=x.device) if logits is None else logits
        kw["logits"] = logits
    if want_token or token is not None:
        token = torch.empty((T,), dtype=torch.int32, device=x.device) if token is None else token
        kw["token"] = token
    _lib.run("lm_head", **kw)
    return logits, token


# ---------------------------------------------------------------------------------------------------------------
# The sgl line's one-call entry point, by the names of its `inputs` object
# (models/qwen35_35b_a3b/sgl/python/sgl_kernel_axera/moe/m_qwen3.py:3607-3795).
_MOE_MODES = ("expert_parallel", "token_parallel")
_prepared = {}


def _inp(inputs, name, default=None):
    if isinstance(inputs, dict):
        return inputs.get(name, default)
    return getattr(inputs, name, default)


def _mx4_pair(inputs, name, what):
    w, s = _inp(inputs, "w_" + name), _inp(inputs, "w_scale_" + name)
    if w is None or s is None:
        raise ValueError(f"qwen3_moe inputs must provide w_{name} and w_scale_{name}")
    if _inp(inputs, "w_zeropoint_" + name) is not None:
        raise ValueError("qwen3_moe: AWQ INT4 experts (zero points) are not supported on this device path")
    if s.element_size() != 1 or s.dtype == torch.float8_e4m3fn or w.shape[-1] * 2 != s.shape[-1] * 32:
        raise ValueError(f"qwen3_moe: {what} must be MXFP4 (E2M1 pairs [.., K / 2] bytes with one E8M0 scale per 32 "
                         "inputs); NVFP4 (E4M3 scales per 16 + scale2) and MXFP8 experts are not supported on this "
                         "device path")
    return _u8(w), _u8(s)


def qwen3_moe(inputs, output=None, *, mode="auto", core_num=1, chunk_size=None, resident_weights=False):
    """The MoE block by the reference's one-call contract: `output = x + moe(post_attention_layernorm(x))` with
    `inputs.w_norm` in the Qwen3.5 zero-centred form (the multiplier is 1 + w_norm).  inputs (mapping or object): x (or
    hidden_states) [..., H] bf16, w_norm [H], norm_eps, w_route [E, H] bf16, w_gate / w_up [E, I, H / 2] and w_down
    [E, H, I / 2] MXFP4 bytes with w_scale_* E8M0 (w_gate may already hold gate and up rows, [E, 2 I, H / 2], with w_up
    absent or the same tensor), shared_expert_gate [H], w_shared_expert_mlp_{gate, up, down} with their
    w_scale_shared_expert_mlp_*, top_k, norm_topk_prob.  mode: "auto", "expert_parallel", "token_parallel" are accepted
    and run the same kernels (they name how the reference spreads work over NPU cores); core_num and chunk_size are
    accepted for the same reason and unused.  Weights are bound, not copied, except that separate gate and up planes are
    joined once per weight set (the kernels read one gate-up plane per expert) and the E8M0 scales are re-tiled once.

    Arithmetic is that of the q35 block (fp32 router logits, routing weights applied after the down projection); the
    reference's sgl kernel computes router logits in bf16 and, for long prefills, scales the activation before the down
    projection -- same results within the block's tolerance, not bit for bit."""
    x = _inp(inputs, "x")
    if x is None:
        x = _inp(inputs, "hidden_states")
    if x is None:
        raise ValueError("qwen3_moe inputs must provide x")
    if x.dim() < 2:
        raise ValueError("qwen3_moe hidden states must have rank >= 2")
    if output is None:
        output = torch.empty_like(x)
    elif tuple(output.shape) != tuple(x.shape) or output.dtype != x.dtype:
        raise ValueError(f"output {tuple(output.shape)} {output.dtype} must match hidden_states {tuple(x.shape)} {x.dtype}")
    if mode != "auto" and mode not in _MOE_MODES:
        raise ValueError(f"unsupported qwen3_moe mode {mode!r}; expected one of: {', '.join(_MOE_MODES)}, auto")
    if not x.is_cuda:
        raise TypeError("qwen3_moe: tensors must be on the GPU (there is no CPU path)")
    if not bool(_inp(inputs, "norm_topk_prob", True)):
        raise ValueError("qwen3_moe: norm_topk_prob=False is not supported (the routing kernel normalises the top-k "
                         "weights, as Qwen3.5 does)")
    w_norm = _inp(inputs, "w_norm")
    if w_norm is None:
        raise ValueError("qwen3_moe: inputs.w_norm is required (the fused x + moe(norm(x)) contract)")
    if _inp(inputs, "shared_expert_gate") is None:
        raise ValueError("qwen3_moe: the block without a shared expert is not supported on this device path")
    eps = _inp(inputs, "norm_eps")
    if eps is not None and abs(float(eps) - 1e-6) > 1e-12:
        raise ValueError("qwen3_moe: norm_eps other than 1e-6 is not supported")
    H = x.shape[-1]
    key = tuple(int(t.data_ptr()) for t in (w_norm, _inp(inputs, "w_gate"), _inp(inputs, "w_down"),
                                            _inp(inputs, "w_route")) if t is not None)
    w = _prepared.get(key)
    if w is None:
        if resident_weights and (_inp(inputs, "w_gate").dtype == torch.bfloat16):
            raise ValueError("qwen3_moe: resident bf16 / per-row FP8 expert weights are not supported; bind MXFP4 planes")
        gw, gs = _mx4_pair(inputs, "gate", "expert weights")
        dw, ds = _mx4_pair(inputs, "down", "expert weights")
        up = _inp(inputs, "w_up")
        if up is not None and up.data_ptr() != _inp(inputs, "w_gate").data_ptr():
            uw, us = _mx4_pair(inputs, "up", "expert weights")
            gw, gs = torch.cat([gw, uw], 1).contiguous(), torch.cat([gs, us], 1).contiguous()
        route_w = _inp(inputs, "w_route")
        if route_w is None or route_w.dtype != torch.bfloat16:
            raise ValueError("qwen3_moe: w_route must be a bf16 [E, H] matrix")
        w = dict(ln2=(w_norm.float().reshape(-1) + 1.0).contiguous(), w_router=route_w,
                 w_shg=_inp(inputs, "shared_expert_gate").to(torch.bfloat16).reshape(1, H).contiguous(),
                 e_gw=gw, e_gs=gs, e_dw=dw, e_ds=ds)
        for ours, theirs in (("gate", "shared_expert_mlp_gate"), ("up", "shared_expert_mlp_up"),
                             ("down", "shared_expert_mlp_down")):
            w["w_" + ours], w["s_" + ours] = _mx4_pair(inputs, theirs, "shared expert weights")
        if w["ln2"].numel() != H:
            raise ValueError(f"qwen3_moe w_norm shape {tuple(w_norm.shape)} must match hidden size {H}")
        prepare_moe_weights(w)
        _prepared[key] = w
    top_k = _inp(inputs, "top_k")
    if top_k is None:
        raise ValueError("qwen3_moe inputs must provide top_k")
    moe_block(x.reshape(-1, H), w, int(top_k), output.reshape(-1, H))
    return output
