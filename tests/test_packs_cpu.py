"""Weight packs, phase banks and load-time conversions (ax_dsl_kernels_b200/packs.py) on the CPU: the `.layout` text
form, members in and out of packs (plain, column strips, column blocks), the tiled -> grouped value-head order, the GGUF
MXFP4 block form, and a reduced `decode.group` role bound through packs and banks."""
import torch

from ax_dsl_kernels_b200 import packs
from oracle import codecs
from _cases import stack_case

LAYOUT = """pf - 0 448
ps - 0 128
p4 - 0 4096
L0.ln1 pf 0 128
L0.s_b ps 0 48
L0.w_down p4 0 2048 blk 16 128 32
L1.ln1 pf 128 128
L1.w_down p4 2048 2048 16 128 64:128,0:64
L1.q_norm pf 256 192
"""


def test_layout_text_round_trip_and_manifest_form():
    pk, members = packs.parse_layout(LAYOUT)
    assert pk == {"pf": 448, "ps": 128, "p4": 4096}
    assert [m["name"] for m in members] == ["L0.ln1", "L0.s_b", "L0.w_down", "L1.ln1", "L1.w_down", "L1.q_norm"]
    assert members[0] == {"name": "L0.ln1", "pack": "pf", "offset": 0, "bytes": 128, "layer": 0, "param": "ln1"}
    assert members[2]["strips"] == [16, 128, 32]
    assert members[4]["blocks"] == {"rows": 16, "row_bytes": 128, "ranges": [[64, 128], [0, 64]]}
    assert packs.format_layout(pk, members) == LAYOUT
    assert packs.bank_input(6, "attn_w_q") == ("k_b2_attn_w_q", 1)
    assert packs.pack_base("pf_1") == "pf"


def test_members_in_and_out_of_packs():
    pk, members = packs.parse_layout(LAYOUT)
    g = torch.Generator().manual_seed(0)
    bound = packs.new_packs(pk)
    vals = {}
    for m in members:
        t = torch.randint(0, 256, (m["bytes"],), generator=g, dtype=torch.uint8)
        vals[m["name"]] = t
        packs.write_member(bound, m, t)
    for m in members:
        got = packs.read_member(bound, m, dtype=torch.uint8)
        assert torch.equal(got.reshape(-1), vals[m["name"]]), m["name"]
    # strips: [cols / width * rows, width] in storage (q35_layer_pk.blocked); ranges: the given order
    w = vals["L0.w_down"].reshape(16, 128)
    stored = bound["p4"][0:2048]
    assert torch.equal(stored, torch.cat([w[:, a:a + 32].reshape(-1) for a in range(0, 128, 32)]))
    w1 = vals["L1.w_down"].reshape(16, 128)
    assert torch.equal(bound["p4"][2048:4096], torch.cat([w1[:, 64:128].reshape(-1), w1[:, 0:64].reshape(-1)]))
    # plain members are views of the pack, typed by the pack
    ln = packs.read_member(bound, members[0])
    assert ln.dtype == torch.float32 and ln.numel() == 32 and ln.data_ptr() == bound["pf"].data_ptr()
    ln.zero_()
    assert int(bound["pf"][:128].sum()) == 0


def test_plan_layout_aligns_members_like_the_reference():
    a = torch.zeros(5, dtype=torch.float32)
    b = torch.zeros((3, 40), dtype=torch.uint8)
    pk, members = packs.plan_layout([{"ln1": ("pf", a), "w_o": ("p4", b)}, {"ln1": ("pf", a)}],
                                    blocks={"w_o": [(20, 40), (0, 20)]})
    assert [(m["name"], m["offset"], m["bytes"]) for m in members] == [("L0.ln1", 0, 20), ("L0.w_o", 0, 120),
                                                                       ("L1.ln1", 64, 20)]
    assert pk == {"pf": 128, "p4": 128}
    assert members[1]["blocks"] == {"rows": 3, "row_bytes": 40, "ranges": [[20, 40], [0, 20]]}


def test_value_head_order_tiled_to_grouped():
    VH, KH, hd = 6, 2, 3
    REP = VH // KH
    first = 4
    tiled = torch.arange(first + VH * hd)
    got = packs.apply_vperm(tiled, f"rows:{first}:{VH}:{KH}")
    assert torch.equal(got[:first], torch.arange(first))
    for k in range(KH):
        for r in range(REP):  # grouped head k * REP + r sits at tiled r * KH + k
            src = first + (r * KH + k) * hd
            dst = first + (k * REP + r) * hd
            assert torch.equal(got[dst:dst + hd], torch.arange(src, src + hd))
    cols = torch.arange(2 * VH * hd).reshape(2, VH * hd)
    gc = packs.apply_vperm(cols, f"cols:{VH}:{KH}")
    assert torch.equal(gc[0], packs.apply_vperm(cols[0].clone(), f"rows:0:{VH}:{KH}"))
    assert torch.equal(gc[1], gc[0] + VH * hd)


def test_conversions_against_the_oracle_codecs():
    g = torch.Generator().manual_seed(5)
    w = torch.randn((24, 128), generator=g) * torch.exp2(torch.randint(-6, 3, (24, 1), generator=g).float())
    w[3, 32:64] = 0
    pk, sc = packs.quant_mxfp4(w)
    rpk, rsc = codecs.quant_mxfp4(w)
    assert torch.equal(pk, rpk) and torch.equal(sc, rsc)
    q8, s8 = packs.quant_mxfp8(w)
    r8, rs8 = codecs.quant_mxfp8(w)
    assert torch.equal(q8.view(torch.uint8), r8.view(torch.uint8)) and torch.equal(s8, rs8)
    # GGUF block form of the same weight: exponent byte, then value j | value (j + 16) << 4
    code = torch.stack([pk & 15, pk >> 4], -1).reshape(24, 4, 32)
    blocks = torch.cat([sc.reshape(24, 4, 1), code[..., :16] | (code[..., 16:] << 4)], -1)
    planar, scales = packs.convert("mxfp4_planar_codes", blocks)
    assert torch.equal(planar, pk) and torch.equal(scales, sc)
    assert torch.equal(codecs.dequant_mxfp4(planar, scales), codecs.dequant_mxfp4(rpk, rsc))
    a = -torch.exp(torch.randn(6, generator=g))
    assert torch.allclose(packs.convert("log_neg", a), torch.log(-a))
    taps = torch.randn((8, 4), generator=g)
    assert torch.equal(packs.convert("bf16_taps_reversed", taps), taps.flip(-1).to(torch.bfloat16))
    assert packs.convert("tensor", taps) is taps


def reference_form_group(kernel_layers, kinds, NK, NV):
    """The layers of stack_case() laid out as the reference binds a decode group: small parameters in packs
    (`L<j>.<name>`), projections in phase banks k_b<j % 4>_<bank> [blocks, rows, cols], value heads in tiled order,
    conv taps reversed, GDN conv weights as one [2 KD + VD, 4] member.  Returns (manifest, tensors)."""
    G = len(kinds)
    blocks = (G + 3) // 4
    rep = NV // NK
    tiled = lambda t: (t.reshape(NK, rep, -1, *t.shape[1:]).transpose(0, 1).reshape(t.shape).contiguous())  # noqa: E731

    def tiled_cols(t):
        hd = t.shape[-1] // NV
        return t.reshape(t.shape[0], NK, rep, hd).transpose(1, 2).reshape(t.shape).contiguous()

    per_layer, banks, params = [], {}, {"gdn": {}, "attn": {}}

    def bank(j, kind, name, t):
        bname, blk = packs.bank_input(j, packs.BANK_OF[kind][name])
        if bname not in banks:
            banks[bname] = torch.zeros((blocks, *t.shape), dtype=t.dtype)
        banks[bname][blk] = t

    def entry(kind, name, t, vperm=None):
        e = {"bytes": t.numel() * t.element_size(), "dtype": {torch.float32: 3, torch.bfloat16: 9}.get(t.dtype, 1),
             "shape": list(t.shape)}
        if vperm:
            e["vperm"] = vperm
        params[kind][name] = e

    for j, (w, kd) in enumerate(zip(kernel_layers, kinds)):
        kind = "gdn" if kd == "g" else "attn"
        small = {}
        for n in ("gate", "up", "down"):
            bank(j, kind, "w_" + n, w["w_" + n])
            small["s_" + n] = ("pf", w["s_" + n])
            entry(kind, "s_" + n, w["s_" + n])
        small["ln2"] = ("pf", w["ln2"])
        entry(kind, "ln2", w["ln2"])
        if kd == "a":
            for n in ("ln1", "q_norm", "k_norm"):
                small[n] = ("pf", w[n])
                entry(kind, n, w[n])
            for n in ("q", "k", "v", "o"):
                bank(j, kind, "w_" + n, w["w_" + n])
                small["s_" + n] = ("pf", w["s_" + n])
                entry(kind, "s_" + n, w["s_" + n])
        else:
            rows = f"rows:0:{NV}:{NK}"
            ln1 = w["input_norm_w"].float()
            small["ln1"] = ("pf", ln1)
            entry(kind, "ln1", ln1)
            for ours, theirs, t in (("q", "gq", False), ("k", "gk", False), ("v", "gv", True), ("z", "z", True),
                                    ("a", "a", True), ("b", "b", True)):
                bank(j, kind, "w_" + theirs, tiled(w["w_" + ours]) if t else w["w_" + ours])
                s = tiled(w["s_" + ours]) if t else w["s_" + ours]
                small["s_" + theirs] = ("pf", s)
                entry(kind, "s_" + theirs, s, rows if t else None)
            bank(j, kind, "w_out", tiled_cols(w["w_o"]))
            small["s_out"] = ("pf", w["s_o"])  # per-row scales of the output projection: no value-head axis
            entry(kind, "s_out", w["s_o"])
            conv = torch.cat([w["w_q_conv"], w["w_k_conv"], tiled(w["w_v_conv"])]).flip(-1).contiguous()
            small["conv_w"] = ("pb", conv)
            entry(kind, "conv_w", conv, f"rows:{2 * w['w_q_conv'].shape[0]}:{NV}:{NK}")
            for n, src in (("a_log", w["a_log"]), ("dt_bias", w["dt_bias"].float())):
                small[n] = ("pf", tiled(src))
                entry(kind, n, src, rows)
            nw = w["o_norm_w"].float()
            small["norm_w"] = ("pf", nw)
            entry(kind, "norm_w", nw)
        per_layer.append(small)
    pk, members = packs.plan_layout(per_layer)
    for m in members:
        m["kind"] = "gdn" if kinds[m["layer"]] == "g" else "attn"
    bound = packs.new_packs(pk)
    for m in members:
        packs.write_member(bound, m, per_layer[m["layer"]][m["param"]][1])
    tensors = {p: t.view(packs.PACK_DTYPE[p]) for p, t in bound.items()}
    tensors.update(banks)
    ins = [{"name": n, "bytes": t.numel() * t.element_size(), "dtype": 1, "shape": list(t.shape)}
           for n, t in tensors.items()]
    manifest = {"format": 1, "model": "reduced", "context": 256, "cores": 4, "params": params,
                "kernels": {"decode.group": {"file": "reduced", "in": ins, "out": [], "packs": pk,
                                             "members": members}}}
    return manifest, tensors


def test_decode_group_bound_through_packs_and_banks_recovers_every_weight():
    kinds = "gggaggga"
    NK, NV = 2, 4
    kw, _ = stack_case(kinds, seed=9, NK=NK, NV=NV)
    manifest, tensors = reference_form_group(kw, kinds, NK, NV)
    assert set(n for n in tensors if n.startswith("k_b")) >= {"k_b0_attn_w_q", "k_b3_mlp_w3", "k_b3_attn_w_o"}
    assert tensors["k_b0_mlp_w1"].shape[0] == 2  # layers 0 and 4 live in blocks 0 and 1 of phase 0
    layers, got_kinds = packs.group_layers(manifest, "decode.group", tensors)
    assert "".join(got_kinds) == kinds
    for j, (got, ref) in enumerate(zip(layers, kw)):
        assert set(got) == set(ref), (j, set(got) ^ set(ref))
        for n, t in ref.items():
            g = got[n]
            assert g.shape == t.shape, (j, n, g.shape, t.shape)
            assert torch.equal(g.float() if g.dtype != torch.uint8 else g, t.float() if t.dtype != torch.uint8 else t), (j, n)
    # bank blocks of layers whose value heads need no reorder are views of the bound inputs, not copies
    assert layers[3]["w_q"].data_ptr() == tensors["k_b3_attn_w_q"][0].data_ptr()
    assert layers[4]["w_gate"].data_ptr() == tensors["k_b0_mlp_w1"][1].data_ptr()
