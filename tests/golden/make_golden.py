"""Generates the golden fixtures in this directory from the reference's OWN torch goldens.

Run where the reference checkout is available, with its path in the environment variable REF:
    REF=<reference checkout> python tests/golden/make_golden.py
The reference's kernels need its NPU DSL package `axnn`, which is not installable; its pure-torch golden functions do
not, so `axnn` (and `onnx`, imported by a board helper) are replaced by inert stub modules and the golden functions
are imported and called unchanged.  Outputs: small .npz files (bf16 tensors stored as their int16 bit patterns with a
`__bf16` suffix, fp8 as uint8 with `__e4m3`).  The tests only read the .npz files; nothing reads the reference at
test time.  Two fixtures need no reference source but the `transformers` package, whose Qwen3.5 decoder layers are the
ground truth the reference compares its layer kernels with: `--only-hf-layer` (MoE decoder layers) and
`--only-hf-stack` (the dense text model with its cache).
"""
import importlib.abc
import importlib.machinery
import json
import os
import sys
import tempfile
from unittest.mock import MagicMock

import numpy as np
import torch

REF = os.environ.get("REF", "")
HERE = os.path.dirname(os.path.abspath(__file__))


class _Mod(MagicMock):
    __path__ = []
    __all__ = []


def _builder(*a, **k):
    return lambda fn: fn


class _Finder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    def find_spec(self, name, path, target=None):
        if name.split(".")[0] in ("axnn", "onnx"):
            return importlib.machinery.ModuleSpec(name, self, is_package=True)
        return None

    def create_module(self, spec):
        m = _Mod()
        m.__name__, m.__spec__, m.builder = spec.name, spec, _builder
        return m

    def exec_module(self, module):
        pass


def pack(d):
    out = {}
    for k, v in d.items():
        if isinstance(v, torch.Tensor):
            if v.dtype == torch.bfloat16:
                out[k + "__bf16"] = v.contiguous().view(torch.int16).numpy()
            elif v.dtype == torch.float8_e4m3fn:
                out[k + "__e4m3"] = v.contiguous().view(torch.uint8).numpy()
            elif v.dtype in (torch.float8_e8m0fnu, torch.float4_e2m1fn_x2):
                out[k] = v.contiguous().view(torch.uint8).numpy()
            else:
                out[k] = v.contiguous().numpy()
        else:
            out[k] = np.asarray(v)
    return out


def save(name, d):
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **pack(d))
    print("wrote", name, {k: tuple(np.asarray(v).shape) for k, v in pack(d).items()})


def lm_head():
    """7. MXFP4 output projection: head-variant codec and logits golden (models/qwen38_27b/head/mx4_common.py:11-69)"""
    sys.path.insert(0, os.path.join(REF, "models/qwen38_27b/head"))
    import mx4_common as hc
    g = torch.Generator().manual_seed(21)
    w = torch.randn((160, 512), generator=g) * 0.02
    w[5, :32] = 0                      # a zero block: exponent 0 -> byte 127
    w[6] *= 2.0 ** 100                 # large: clamps nowhere near 254 but exercises big exponents
    w[7, 32:64] = 3e-39                # amax below the reference's floor of 1e-30: scale byte 25
    pk, sc = hc.quantize_mxfp4(w)
    x = torch.randn((3, 512), generator=g).to(torch.bfloat16)
    logits = hc.torch_logits(x.float(), pk, sc)
    save("lm_head", dict(w=w, packed=pk, scale=sc, dequant=hc.dequantize_mxfp4(pk, sc), x=x, logits=logits,
                         token=logits.argmax(-1).to(torch.int32)))


def manifest_roles():
    """8. the roles of the reference's 35B manifest that map onto single roles of the library (IO metadata only), plus
    the first entries of decode.group as an example of a role that does not"""
    m = json.load(open(os.path.join(REF, "models/qwen35_35b_a3b/qwen35_35b_a3b.manifest.json")))
    keep = {k: v for k, v in m["kernels"].items() if k.startswith("moe.") or k in ("lm_head", "decode.group")}
    g = keep["decode.group"]
    keep["decode.group"] = {"file": g["file"], "in": g["in"][:6], "out": g["out"][:2]}
    out = {k: m[k] for k in ("format", "model", "context", "cores")}
    out["params"] = {"experts": m["params"]["experts"]}
    out["kernels"] = keep
    json.dump(out, open(os.path.join(HERE, "manifest_35b_roles.json"), "w"), indent=0)
    print("wrote manifest_35b_roles.json", list(keep))


def mrope():
    """9. M-RoPE table mixing (attn_utils/common.py:304-345): T / H / W rows of the cos / sin tables mixed by channel masks,
    sections (11, 11, 10) of the 32 rotary pairs, chunked and interleaved"""
    sys.meta_path.insert(0, _Finder())
    sys.path.insert(0, os.path.join(REF, "models/qwen35_35b_a3b/sgl/python"))
    from sgl_kernel_axera.attention.attn_utils import common as cm
    g = torch.Generator().manual_seed(31)
    rot, theta, T = 64, 1e7, 9
    pos = torch.randint(0, 5000, (3, T), generator=g)
    inv = 1.0 / (theta ** (torch.arange(0, rot, 2, dtype=torch.int64).float() / rot))
    table = torch.arange(5000).float().reshape(-1, 1) * inv.reshape(1, -1)
    cos_t, sin_t = table.cos(), table.sin()
    d = dict(position_ids=pos.to(torch.int32), inv_freq=inv)
    for name, inter in (("chunked", False), ("interleaved", True)):
        m = cm.mrope_channel_masks((11, 11, 10), interleaved=inter)
        d[f"mask_{name}"] = torch.tensor(np.stack(m))
        d[f"cos_{name}"] = cm.mix_mrope_tables(cos_t[pos[0]], cos_t[pos[1]], cos_t[pos[2]], (11, 11, 10), interleaved=inter)
        d[f"sin_{name}"] = cm.mix_mrope_tables(sin_t[pos[0]], sin_t[pos[1]], sin_t[pos[2]], (11, 11, 10), interleaved=inter)
    save("mrope", d)


def mtp():
    """10. the MTP block of the speculative-decode group (mtp_step, models/qwen38_27b/mtp/mtp_ref.py:202-239) at a reduced
    width (the module's size constants are set before its functions run): MXFP4 projections made and dequantised by
    the module's own codec, three chained rows (the hidden fed back) appending to the block's own paged KV"""
    sys.path.insert(0, os.path.join(REF, "models/qwen38_27b/mtp"))
    import mtp_ref as mr
    mr.H, mr.F, mr.HQ, mr.HKV, mr.D = 256, 512, 2, 1, 128
    W = mr.MtpWeights("", random=True)
    packed, deq = mr.mtp_args(W, quantized=True)
    g = torch.Generator().manual_seed(41)
    rows = 3
    e = (torch.randn((rows, mr.H), generator=g) * 0.5).to(torch.bfloat16)
    h0 = (torch.randn((mr.H,), generator=g) * 0.5).to(torch.bfloat16)
    kv = torch.zeros((1, 2, 256, mr.HKV * mr.D), dtype=torch.bfloat16)
    h, hn_all, y_all = h0.float(), [], []
    for pos in range(rows):
        hn, y = mr.mtp_step(e[pos].float(), h, pos, kv, deq)
        hn_all.append(hn.reshape(-1))
        y_all.append(y.reshape(-1))
        h = hn.reshape(-1).to(torch.bfloat16).float()  # the next row takes the hidden as the kernels pass it: bf16
    d = dict(e=e, h0=h0, h_next=torch.stack(hn_all), y=torch.stack(y_all), kv=kv,
             dims=torch.tensor([mr.H, mr.F, mr.HQ, mr.HKV, mr.D, mr.ROT]))
    for n, t in packed.items():
        d["w." + n] = t.view(torch.uint8) if t.dtype in (torch.float4_e2m1fn_x2, torch.float8_e8m0fnu) else t
    save("mtp", d)


def hf_layer():
    """The end-to-end ground truth the reference checks its layer kernels against: transformers'
    Qwen3_5MoeDecoderLayer in fp32, eager attention, with the routed experts' weights passed through the MXFP4 round
    trip (hf_layer / hf_out, models/qwen35_2b/whole/src/q35_moe.py:300-324).  A small configuration of the same
    architecture, seeded random weights rounded to bf16, one GDN layer and one attention layer on a 6-token prefill.
    Needs the `transformers` package (no reference source)."""
    from transformers.models.qwen3_5_moe.configuration_qwen3_5_moe import Qwen3_5MoeTextConfig
    from transformers.models.qwen3_5_moe.modeling_qwen3_5_moe import (Qwen3_5MoeDecoderLayer,
                                                                       Qwen3_5MoeTextRotaryEmbedding)
    sys.path.insert(0, os.path.join(HERE, "..", ".."))
    from oracle import codecs
    dims = dict(hidden_size=256, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=64,
                shared_expert_intermediate_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                layer_types=["linear_attention", "full_attention"], num_hidden_layers=2, linear_num_key_heads=2,
                linear_num_value_heads=4, linear_key_head_dim=32, linear_value_head_dim=32, linear_conv_kernel_dim=4,
                rms_norm_eps=1e-6, vocab_size=1000)
    hc = Qwen3_5MoeTextConfig(**dims)
    hc._attn_implementation = "eager"
    rot = Qwen3_5MoeTextRotaryEmbedding(hc)
    g = torch.Generator().manual_seed(77)
    P, H, NE, FE = 6, dims["hidden_size"], dims["num_experts"], dims["moe_intermediate_size"]
    out = dict(rope_theta=float(hc.rope_parameters["rope_theta"]),
               partial_rotary_factor=float(hc.rope_parameters["partial_rotary_factor"]))
    for kind, il in (("gdn", 0), ("attn", 1)):
        layer = Qwen3_5MoeDecoderLayer(hc, il).float().eval()
        sd = {}
        for name, t in layer.state_dict().items():
            if name.endswith("layernorm.weight") or name.endswith("_norm.weight"):  # stored as w - 1
                v = torch.randn(t.shape, generator=g) * 0.1
            elif name.endswith("linear_attn.norm.weight"):
                v = 1.0 + torch.randn(t.shape, generator=g) * 0.1
            elif name.endswith("A_log"):
                v = torch.randn(t.shape, generator=g) * 0.5
            elif name.endswith("dt_bias"):
                v = torch.randn(t.shape, generator=g) * 0.5
            elif name.endswith("conv1d.weight"):
                v = torch.randn(t.shape, generator=g) * 0.3
            else:
                v = torch.randn(t.shape, generator=g) * (t.shape[-1] ** -0.5)
            sd[name] = v.to(torch.bfloat16).float()
        packs = {}
        for name in ("mlp.experts.gate_up_proj", "mlp.experts.down_proj"):  # the MXFP4 round trip, expert by expert
            w = sd[name]
            pk, sc = zip(*[codecs.quant_mxfp4(w[e]) for e in range(NE)])
            packs[name] = (torch.stack(pk), torch.stack(sc))
            sd[name] = torch.stack([codecs.dequant_mxfp4(a, b) for a, b in zip(pk, sc)])
        layer.load_state_dict(sd, strict=True)
        x = (torch.randn((1, P, H), generator=g) * 0.5).to(torch.bfloat16)
        pos = torch.arange(P).reshape(1, P)
        mask = None
        if kind == "attn":  # additive causal mask: key j is visible to query i when j <= i
            visible = pos.reshape(P, 1) >= pos.reshape(1, P)
            mask = torch.zeros((P, P)).masked_fill(~visible, float("-inf")).reshape(1, 1, P, P)
        probs = []

        def keep_router_output(module, args, output):
            probs.append(output[0])  # the router's first output: softmax over all experts, fp32

        handle = layer.mlp.gate.register_forward_hook(keep_router_output)
        with torch.no_grad():
            y = layer(x.float(), position_embeddings=rot(x.float(), pos), attention_mask=mask, position_ids=pos)
        handle.remove()
        if isinstance(y, tuple):
            y = y[0]
        out[kind + ".x"] = x
        out[kind + ".y"] = y.reshape(P, H).float()
        out[kind + ".router_probs"] = probs[0].reshape(P, NE).float()
        for name, t in sd.items():
            if name in packs:
                out[f"{kind}.{name}.packed"], out[f"{kind}.{name}.scale"] = packs[name]
            else:
                out[f"{kind}.{name}"] = t.to(torch.bfloat16)
    cos, sin = rot(torch.zeros((1, P, H)), torch.arange(P)[None])
    out["rope_cos"], out["rope_sin"] = cos.reshape(P, -1).float(), sin.reshape(P, -1).float()
    for k, v in dims.items():
        if isinstance(v, (int, float)):
            out["cfg." + k] = v
    save("hf_layer", out)


def hf_stack():
    """The dense hybrid stack (layers g g g a, SwiGLU block after every token mixer) as transformers' Qwen3_5TextModel
    runs it in fp32 with its own cache: a 7-token prefill, then two single-token decode steps; the hidden state after
    every decoder layer of each call.  The layer loop this stands for:
    models/qwen35_2b/whole/src/q35_step.py:438-470.  Needs the `transformers` package (no reference source)."""
    from transformers.models.qwen3_5.configuration_qwen3_5 import Qwen3_5TextConfig
    from transformers.models.qwen3_5.modeling_qwen3_5 import Qwen3_5TextModel
    dims = dict(hidden_size=128, intermediate_size=256, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                layer_types=["linear_attention"] * 3 + ["full_attention"], num_hidden_layers=4, linear_num_key_heads=2,
                linear_num_value_heads=4, linear_key_head_dim=16, linear_value_head_dim=16, linear_conv_kernel_dim=4,
                rms_norm_eps=1e-6, vocab_size=64)
    hc = Qwen3_5TextConfig(**dims)
    hc._attn_implementation = "eager"
    model = Qwen3_5TextModel(hc).float().eval()
    g = torch.Generator().manual_seed(91)
    sd = {}
    for name, t in model.state_dict().items():
        if name.endswith("layernorm.weight") or name.endswith("_norm.weight") or name == "norm.weight":
            v = torch.randn(t.shape, generator=g) * 0.1  # stored as w - 1
        elif name.endswith("linear_attn.norm.weight"):
            v = 1.0 + torch.randn(t.shape, generator=g) * 0.1
        elif name.endswith("A_log") or name.endswith("dt_bias"):
            v = torch.randn(t.shape, generator=g) * 0.5
        elif name.endswith("conv1d.weight"):
            v = torch.randn(t.shape, generator=g) * 0.3
        else:
            v = torch.randn(t.shape, generator=g) * (t.shape[-1] ** -0.5)
        sd[name] = v.to(torch.bfloat16).float()
    model.load_state_dict(sd, strict=True)
    T, H = 7, dims["hidden_size"]
    xs = (torch.randn((1, T + 2, H), generator=g) * 0.5).to(torch.bfloat16)
    seen = []
    hooks = [layer.register_forward_hook(lambda m, i, o: seen.append(o[0] if isinstance(o, tuple) else o))
             for layer in model.layers]
    with torch.no_grad():
        r = model(inputs_embeds=xs[:, :T].float(), use_cache=True)
        cache = r.past_key_values
        for t in range(T, T + 2):
            r = model(inputs_embeds=xs[:, t:t + 1].float(), past_key_values=cache, use_cache=True)
            cache = r.past_key_values
    for h in hooks:
        h.remove()
    L = len(model.layers)  # seen: the L layers' outputs of the prefill, then of each decode step
    out = dict(x=xs, y_prefill=torch.stack([t.reshape(T, H) for t in seen[:L]]).float(),
               y_decode0=torch.stack([t.reshape(1, H) for t in seen[L:2 * L]]).float(),
               y_decode1=torch.stack([t.reshape(1, H) for t in seen[2 * L:3 * L]]).float(),
               rope_theta=float(hc.rope_parameters["rope_theta"]),
               partial_rotary_factor=float(hc.rope_parameters["partial_rotary_factor"]))
    for name, t in sd.items():
        if name.startswith("layers."):
            out[name] = t.to(torch.bfloat16)
    for k, v in dims.items():
        if isinstance(v, (int, float)):
            out["cfg." + k] = v
    save("hf_stack", out)


def main():
    if "--only-hf-layer" in sys.argv:
        return hf_layer()
    if "--only-hf-stack" in sys.argv:
        return hf_stack()
    if not os.path.isdir(REF):
        sys.exit("set REF to the reference checkout")
    if "--only-lm-head" in sys.argv:
        return lm_head()
    if "--only-manifest" in sys.argv:
        return manifest_roles()
    if "--only-mrope" in sys.argv:
        return mrope()
    if "--only-mtp" in sys.argv:
        return mtp()
    sys.meta_path.insert(0, _Finder())
    sgl = os.path.join(REF, "models/qwen35_35b_a3b/sgl")
    sys.path[:0] = [os.path.join(sgl, "python"), os.path.join(sgl, "tests"),
                    os.path.join(REF, "models/qwen35_2b/whole/src")]
    cfg_dir = tempfile.mkdtemp()
    json.dump({"text_config": {
        "hidden_size": 2048, "num_experts": 256, "num_experts_per_tok": 8, "moe_intermediate_size": 512,
        "shared_expert_intermediate_size": 512, "num_attention_heads": 16, "num_key_value_heads": 2, "head_dim": 256,
        "rope_parameters": {"partial_rotary_factor": 0.25, "rope_theta": 1e7},
        "layer_types": ["linear_attention"] * 3 + ["full_attention"], "num_hidden_layers": 4,
        "linear_num_key_heads": 16, "linear_num_value_heads": 32, "linear_key_head_dim": 128,
        "linear_value_head_dim": 128, "linear_conv_kernel_dim": 4, "rms_norm_eps": 1e-6, "vocab_size": 248320}},
        open(os.path.join(cfg_dir, "config.json"), "w"))
    os.environ["MODEL"] = cfg_dir
    os.environ["WFMT"] = "mx8"
    os.chdir(cfg_dir)
    import q35_moe as mo  # models/qwen35_2b/whole/src/q35_moe.py
    import q35_mx_build as mb  # models/qwen35_2b/whole/src/q35_mx_build.py
    import test_gdn_attn as tg  # models/qwen35_35b_a3b/sgl/tests/test_gdn_attn.py

    # 1. MXFP4 codec (q35_moe.py:46-63): random rows, a zero block, exact rounding ties, big/small magnitudes
    g = torch.Generator().manual_seed(11)
    w = torch.randn((12, 128), generator=g) * 0.02
    w[1, :32] = 0
    w[2, :8] = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -5.0])  # midpoints between E2M1 values
    w[3] *= 1e4
    w[4] *= 1e-6
    pk, sc = mo.quant_mxfp4(w)
    save("mxfp4_codec", dict(w=w, packed=pk, scale=sc, dequant=mo.dequant_mxfp4(pk, sc)))

    # 2. MXFP8 (q35_mx_build.py:60-72) and NVFP4 (:168-186) codecs
    w = torch.randn((6, 96), generator=g) * 0.05
    w[0, :32] *= 1e3
    q8, s8 = mb.quant_mxfp8(w)
    save("mxfp8_codec", dict(w=w, q8=q8, scale=s8.view(torch.uint8), dequant=mb.dequant(q8, s8)))
    w = torch.randn((6, 64), generator=g) * 0.02
    p4, s4, t4 = mb.quant_nvfp4(w)
    save("nvfp4_codec", dict(w=w, packed=p4.view(torch.uint8), scale=s4, scale2=t4,
                             dequant=mb.dequant_nvfp4(p4, s4, t4)))

    # 3. router (q35_moe.py:293-297), one token per call as the reference does
    logits = torch.randn((24, 256), generator=g)
    logits[3, 10] = logits[3, 200] = logits[3].max() + 1.0  # an exact tie at the top
    logits[4, 7] = logits[4, 99] = torch.sort(logits[4], descending=True).values[7]  # a tie across the top-8 edge
    ids, rws = [], []
    for t in range(logits.shape[0]):
        i, r = mo.route(logits[t])
        ids.append(i)
        rws.append(r.reshape(-1))
    save("route", dict(logits=logits, ids=torch.tensor(ids, dtype=torch.int32), rw=torch.stack(rws)))

    # 4. causal conv1d + SiLU (test_gdn_attn.py:241-257)
    x = tg.bf16_randn((2, 9, 24), 0.5)
    cw = tg.bf16_randn((24, 4), 0.2)
    st = tg.bf16_randn((2, 3, 24), 0.3)
    y, so = tg.causal_conv1d_silu_reference(x, cw, st)
    save("conv1d", dict(x=x, weight=cw, state_in=st, y=y, state_out=so))

    # 5. GDN core recurrence (gdn_reference, test_gdn_attn.py:260-296)
    torch.manual_seed(5)
    T, NK, NV, DK, DV = 10, 2, 4, 16, 16
    q, k = tg.bf16_randn((1, T, NK, DK), 1.0), tg.bf16_randn((1, T, NK, DK), 1.0)
    v = tg.bf16_randn((1, T, NV, DV), 1.0)
    a, b = tg.bf16_randn((1, T, NV), 1.0), tg.bf16_randn((1, T, NV), 1.0)
    a_log, dt_bias = torch.randn(NV) * 0.5, tg.bf16_randn((NV,), 0.5)
    s0 = torch.randn((1, NV, DK, DV)) * 0.03
    o, s1 = tg.gdn_reference(q, k, v, a, b, a_log, dt_bias, s0)
    save("gdn_core", dict(q=q, k=k, v=v, a=a, b=b, a_log=a_log, dt_bias=dt_bias, state_in=s0, o=o, state_out=s1))

    # 6. whole GDN sublayer (reference(), test_gdn_attn.py:427-474) on the fixture shape, seq 7
    case = tg.random_case(7)
    fused, st_out, cv_out = tg.reference(case, input_norm_eps=2e-6, o_norm_eps=3e-6)
    hs, res, wts, ts, cs = case
    d = dict(hidden=hs, residual=res, temporal_state=ts, conv_state=cs, fused=fused, state_out=st_out, conv_out=cv_out)
    d.update({"w." + n: t for n, t in wts.items()})
    save("gdn_sublayer", d)
    lm_head()
    manifest_roles()
    mrope()
    mtp()
    hf_layer()
    hf_stack()


if __name__ == "__main__":
    main()
