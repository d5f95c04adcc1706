"""The CPU oracle's whole decoder layer (GDN or attention sublayer + MoE block) against the ground truth the reference
checks its layer kernels with: transformers' Qwen3_5MoeDecoderLayer in fp32, experts through the MXFP4 round trip
(hf_layer / hf_out, models/qwen35_2b/whole/src/q35_moe.py:300-324).  The fixture (tests/golden/hf_layer.npz, made by
tests/golden/make_golden.py --only-hf-layer) holds a small configuration of the same architecture with seeded weights.
The oracle rounds to bf16 where the reference's kernels do and the Hugging Face layer does not round at all, so the
comparison is the reference's own kind -- cosine and error against RMS -- not bit for bit: it pins the structure (norm
convention, projection splits, head order, RoPE pairing, gates, residuals, router rule, expert layout).  Checkpoint
weights become kernel inputs as the reference's loader makes them: the layer norms and the q / k norms as 1 + w, the
gated norm of the GDN output as it is (models/qwen35_2b/whole/src/q35_step.py:347, 370-401)."""
import torch

from oracle import attention as oattn
from oracle import codecs, gdn, moe, stack


def _cos(a, b):
    a, b = a.float().reshape(-1), b.float().reshape(-1)
    return float(a @ b / (a.norm() * b.norm()))


def _moe_weights(f, kind):
    g = lambda n: f[f"{kind}.{n}"]  # noqa: E731
    return dict(ln2=1.0 + g("post_attention_layernorm.weight").float(),  # Qwen3.5 stores norm weights as w - 1
                sh_gate=g("mlp.shared_expert.gate_proj.weight").float(), sh_up=g("mlp.shared_expert.up_proj.weight").float(),
                sh_down=g("mlp.shared_expert.down_proj.weight").float(), w_router=g("mlp.gate.weight"),
                w_shg=g("mlp.shared_expert_gate.weight").reshape(-1),
                e_gw=g("mlp.experts.gate_up_proj.packed"), e_gs=g("mlp.experts.gate_up_proj.scale"),
                e_dw=g("mlp.experts.down_proj.packed"), e_ds=g("mlp.experts.down_proj.scale"))


def _finish(f, kind, x1, top_k):
    """MoE block on the sublayer's output; checks the router against the Hugging Face probabilities"""
    w = _moe_weights(f, kind)
    out, ids, rw, logits = moe.moe_block(x1, w["ln2"], w["sh_gate"], w["sh_up"], w["sh_down"], w["w_router"], w["w_shg"],
                                         w["e_gw"], w["e_gs"], w["e_dw"], w["e_ds"], top_k)
    probs = f[f"{kind}.router_probs"]
    assert _cos(torch.softmax(logits.float(), -1), probs) > 0.9995
    top = torch.topk(probs, top_k, -1)
    for t in range(ids.shape[0]):
        margin = float(top.values[t, -1] - torch.topk(probs[t], top_k + 1).values[-1])
        if margin > 1e-2:  # a clear k-th place: the same experts, the same renormalised weights
            assert sorted(ids[t].tolist()) == sorted(top.indices[t].tolist()), (t, ids[t], top.indices[t])
            ref_w = dict(zip(top.indices[t].tolist(), (top.values[t] / top.values[t].sum()).tolist()))
            for e, wv in zip(ids[t].tolist(), rw[t].tolist()):
                assert abs(wv - ref_w[e]) < 2e-2
    return out


def _check(out, ref, worst_limit=0.1):
    """bf16 rounding at every step of the oracle against no rounding at all: error of the whole output against its RMS
    within 2e-2, cosine above 0.9998 (the reference logs the cosine, q35_moe.py:353-355), no element off by worst_limit RMS"""
    rms = ref.square().mean().sqrt()
    d = out.float() - ref
    rel, worst = float(d.square().mean().sqrt() / rms), float(d.abs().max() / rms)
    assert _cos(out, ref) > 0.9998 and rel < 2e-2 and worst < worst_limit, (_cos(out, ref), rel, worst)


def test_gdn_layer_with_moe_block_matches_the_transformers_layer(golden):
    f = golden("hf_layer")
    g = lambda n: f["gdn." + n]  # noqa: E731
    NK, NV = int(f["cfg.linear_num_key_heads"]), int(f["cfg.linear_num_value_heads"])
    DK, DV = int(f["cfg.linear_key_head_dim"]), int(f["cfg.linear_value_head_dim"])
    kd, vd = NK * DK, NV * DV
    qkv = g("linear_attn.in_proj_qkv.weight")  # rows: q | k | v
    conv = g("linear_attn.conv1d.weight").reshape(2 * kd + vd, -1)  # [channels, taps], oldest tap first
    w = dict(input_norm_w=1.0 + g("input_layernorm.weight").float(), w_q=qkv[:kd], w_k=qkv[kd:2 * kd], w_v=qkv[2 * kd:],
             w_z=g("linear_attn.in_proj_z.weight"), w_a=g("linear_attn.in_proj_a.weight"),
             w_b=g("linear_attn.in_proj_b.weight"), w_q_conv=conv[:kd], w_k_conv=conv[kd:2 * kd], w_v_conv=conv[2 * kd:],
             a_log=g("linear_attn.A_log").float(), dt_bias=g("linear_attn.dt_bias"),
             o_norm_w=g("linear_attn.norm.weight").float(), w_o=g("linear_attn.out_proj.weight"))
    x = g("x")
    T = x.shape[1]
    x1, _, _ = gdn.gdn_sublayer(x, torch.zeros_like(x), w, torch.zeros((1, NV, DK, DV)),
                                torch.zeros((1, conv.shape[1] - 1, 2 * kd + vd), dtype=torch.bfloat16))
    out = _finish(f, "gdn", x1.reshape(T, -1), int(f["cfg.num_experts_per_tok"]))
    _check(out, g("y"))


def test_attention_layer_with_moe_block_matches_the_transformers_layer(golden):
    f = golden("hf_layer")
    g = lambda n: f["attn." + n]  # noqa: E731
    heads, kv_heads, hd = int(f["cfg.num_attention_heads"]), int(f["cfg.num_key_value_heads"]), int(f["cfg.head_dim"])
    rot = int(round(hd * float(f["partial_rotary_factor"])))
    w = dict(ln1=1.0 + g("input_layernorm.weight").float(), w_q=g("self_attn.q_proj.weight"),
             w_k=g("self_attn.k_proj.weight"), w_v=g("self_attn.v_proj.weight"), w_o=g("self_attn.o_proj.weight"),
             q_norm=1.0 + g("self_attn.q_norm.weight").float(), k_norm=1.0 + g("self_attn.k_norm.weight").float())
    x = g("x")
    T = x.shape[1]
    cos, sin = oattn.rope_cos_sin(torch.arange(T), rot, float(f["rope_theta"]))
    # the oracle's table against the rotary embedding module's (which repeats the rot / 2 frequencies twice)
    torch.testing.assert_close(cos.float(), f["rope_cos"][:, :rot // 2], rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(sin.float(), f["rope_sin"][:, :rot // 2], rtol=1e-5, atol=1e-6)
    P = 8
    cache = torch.zeros((1, 2, P, kv_heads, hd), dtype=torch.bfloat16)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32)  # noqa: E731
    x1 = stack.attn_sublayer(x.reshape(T, -1), w, cache, i32([0, 1]), i32([0]), i32([T]), cos, sin, heads=heads,
                             kv_heads=kv_heads, head_dim=hd, rot=rot, gated=True, qo_indptr=i32([0, T]))
    out = _finish(f, "attn", x1, int(f["cfg.num_experts_per_tok"]))
    _check(out, g("y"))
    assert codecs.GROUP == 32


def test_dense_hybrid_stack_prefill_then_decode_matches_the_transformers_model(golden):
    """oracle.stack.HybridStack (g g g a with a SwiGLU block per layer; the stack the GPU stack drivers are checked
    against) on a 7-token prefill and two decode steps, against transformers' Qwen3_5TextModel with its own cache
    (tests/golden/hf_stack.npz, make_golden.py --only-hf-stack): the decode steps go through the recurrent state, the
    conv state and the paged KV cache the prefill left behind."""
    f = golden("hf_stack")
    NK, NV = int(f["cfg.linear_num_key_heads"]), int(f["cfg.linear_num_value_heads"])
    DK, DV = int(f["cfg.linear_key_head_dim"]), int(f["cfg.linear_value_head_dim"])
    kd, vd = NK * DK, NV * DV
    heads, kv_heads, hd = int(f["cfg.num_attention_heads"]), int(f["cfg.num_key_value_heads"]), int(f["cfg.head_dim"])
    rot = int(round(hd * float(f["partial_rotary_factor"])))
    kinds, layers = ["g", "g", "g", "a"], []
    for i, kind in enumerate(kinds):
        g = lambda n: f[f"layers.{i}.{n}"]  # noqa: E731,B023
        w = dict(ln2=1.0 + g("post_attention_layernorm.weight").float(), w_gate=g("mlp.gate_proj.weight"),
                 w_up=g("mlp.up_proj.weight"), w_down=g("mlp.down_proj.weight"))
        if kind == "g":
            qkv = g("linear_attn.in_proj_qkv.weight")
            conv = g("linear_attn.conv1d.weight").reshape(2 * kd + vd, -1)
            w.update(input_norm_w=1.0 + g("input_layernorm.weight").float(), w_q=qkv[:kd], w_k=qkv[kd:2 * kd],
                     w_v=qkv[2 * kd:], w_z=g("linear_attn.in_proj_z.weight"), w_a=g("linear_attn.in_proj_a.weight"),
                     w_b=g("linear_attn.in_proj_b.weight"), w_q_conv=conv[:kd], w_k_conv=conv[kd:2 * kd],
                     w_v_conv=conv[2 * kd:], a_log=g("linear_attn.A_log").float(), dt_bias=g("linear_attn.dt_bias"),
                     o_norm_w=g("linear_attn.norm.weight").float(), w_o=g("linear_attn.out_proj.weight"))
        else:
            w.update(ln1=1.0 + g("input_layernorm.weight").float(), w_q=g("self_attn.q_proj.weight"),
                     w_k=g("self_attn.k_proj.weight"), w_v=g("self_attn.v_proj.weight"), w_o=g("self_attn.o_proj.weight"),
                     q_norm=1.0 + g("self_attn.q_norm.weight").float(), k_norm=1.0 + g("self_attn.k_norm.weight").float())
        layers.append(w)
    cfg = dict(heads=heads, kv_heads=kv_heads, head_dim=hd, rot=rot, theta=float(f["rope_theta"]), page_size=4, max_tokens=16,
               gated=True)
    x = f["x"][0]
    T = f["y_prefill"].shape[1]
    calls = [(x[:T], f["y_prefill"]), (x[T:T + 1], f["y_decode0"]), (x[T + 1:T + 2], f["y_decode1"])]
    # every layer by itself, fed what the transformers layer was fed, its own state carried from call to call
    for i, kind in enumerate(kinds):
        one = stack.HybridStack(layers[i:i + 1], [kind], **cfg)
        for xin, ys in calls:
            _check(one.forward(xin if i == 0 else ys[i - 1].to(torch.bfloat16)), ys[i], worst_limit=0.15)
    # the four layers chained: the rounding of one layer is the input noise of the next
    st = stack.HybridStack(layers, kinds, **cfg)
    for xin, ys in calls:
        out, ref = st.forward(xin), ys[-1]
        assert _cos(out, ref) > 0.999 and float((out.float() - ref).square().mean().sqrt() / ref.square().mean().sqrt()) < 5e-2
