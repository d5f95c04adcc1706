"""Weight packs, phase banks and load-time conversions of the reference's kernel manifests.

The reference's fused layer kernels do not take one input per weight: small parameters travel in one PACK per dtype
(`p4` E2M1 pairs, `pw` E4M3, `ps` E8M0 / E4M3 scales, `pf` fp32, `pb` bf16; set s > 0 of a split pack is `<pack>_<s>`),
each member at a 64-byte aligned offset, described by a `.layout` file next to the kernel ("member pack offset bytes"
per line, the pack itself as "pack - 0 bytes"; models/qwen35_2b/whole/src/q35_layer_pk.py:5-10,143-161,273-280) and by
the `packs` / `members` entries of a manifest role (tools/manifest/mkmanifest.py:254-277,313-324).  A member that the
NPU cores slice by columns is stored column-blocked: `blk rows cols width` = strips of `width` bytes of every row
stacked one after the other (q35_layer_pk.py:90-105), or `rows row_bytes a:b,c:d,...` = the byte ranges of a row in
storage order, each [rows, b - a] contiguous (models/qwen38_27b/decode/q35_layer_mc.py:1269-1313).  The large
row-split projections of the decode group are not packed at all: they are the prefill kernel's PHASE BANKS
`[blocks, rows, cols]`, bound a second time under the names `k_b<phase>_<bank>`, layer j of the group in block j // 4
of phase j % 4 (models/qwen38_27b/decode/q35_group.py:73-99).

This module reads and writes those forms on the host and turns a bound role into the per-layer weight dictionaries
layers.py takes.  Plain members and bank blocks are zero-copy views of the caller's tensors; column-blocked members and
members whose value heads are stored in the GGUF's tiled order are copied once into row-major / grouped order (this
library's kernels index `key_head = value_head // ratio`), which is load-time work outside the decode step.

`convert()` implements the conversions a manifest's `params.<kind>.<name>.convert` names (mkmanifest.py:224-251,
330-336): they describe how the backend fills the packs from a GGUF file once.
"""
import re

import torch

ALIGN = 64
PACK_DTYPE = {"p4": torch.uint8, "pw": torch.float8_e4m3fn, "ps": torch.uint8, "pf": torch.float32,
              "pb": torch.bfloat16}
E2M1 = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def pack_base(name):
    """`pf_1` -> `pf` (set 1 of a pack split to stay under the runtime's IO size limit)"""
    return name.split("_")[0]


# ------------------------------------------------------------------------------------------------- .layout text
def parse_layout(text):
    """(.layout text) -> (packs {name: bytes}, members [dict]) in the manifest's form (mkmanifest.py:254-277)"""
    packs, members = {}, []
    for line in text.splitlines():
        f = line.split()
        if len(f) < 4:
            continue
        name, pack, off, nbytes = f[0], f[1], int(f[2]), int(f[3])
        if pack == "-":
            packs[name] = nbytes
            continue
        m = {"name": name, "pack": pack, "offset": off, "bytes": nbytes}
        lm = re.match(r"L(\d+)\.(.+)", name)
        if lm:
            m["layer"], m["param"] = int(lm.group(1)), lm.group(2)
        else:
            m["param"] = name
        rest = f[4:]
        if rest[:1] == ["blk"]:
            m["strips"] = [int(x) for x in rest[1:4]]
        elif len(rest) >= 3:
            m["blocks"] = {"rows": int(rest[0]), "row_bytes": int(rest[1]),
                           "ranges": [[int(a), int(b)] for a, b in (r.split(":") for r in rest[2].split(","))]}
        members.append(m)
    return packs, members


def format_layout(packs, members):
    """inverse of parse_layout"""
    lines = [f"{p} - 0 {n}" for p, n in packs.items()]
    for m in members:
        s = f"{m['name']} {m['pack']} {m['offset']} {m['bytes']}"
        if "strips" in m:
            s += " blk " + " ".join(str(v) for v in m["strips"])
        elif "blocks" in m:
            b = m["blocks"]
            s += f" {b['rows']} {b['row_bytes']} " + ",".join(f"{a}:{c}" for a, c in b["ranges"])
        lines.append(s)
    return "\n".join(lines) + "\n"


def plan_layout(layers, blocks=None, align=ALIGN):
    """Places parameters in packs as the reference's layout() does: `layers` = [{param: (pack, tensor)}] per layer (or
    one dict for a single-layer kernel), members in the given order, every offset rounded up to `align` bytes.
    blocks: {param: [(a, b), ...]} byte ranges of a row for members stored column-blocked.  Returns (packs, members)."""
    single = isinstance(layers, dict)
    used, members = {}, []
    for j, layer in enumerate([layers] if single else layers):
        for param, (pack, t) in layer.items():
            nbytes = t.numel() * t.element_size()
            off = (used.get(pack, 0) + align - 1) // align * align
            m = {"name": param if single else f"L{j}.{param}", "pack": pack, "offset": off, "bytes": nbytes,
                 "param": param}
            if not single:
                m["layer"] = j
            if blocks and param in blocks:
                rows = t.shape[0]
                m["blocks"] = {"rows": rows, "row_bytes": nbytes // rows, "ranges": [list(r) for r in blocks[param]]}
            members.append(m)
            used[pack] = off + nbytes
    packs = {p: max(1, (n + align - 1) // align * align) for p, n in used.items()}
    return packs, members


# ------------------------------------------------------------------------------------------------- members <-> packs
def _bytes(t):
    return t.contiguous().reshape(-1).view(torch.uint8)


def _pack_bytes(tensors, pack):
    if pack not in tensors:
        raise KeyError(f"pack {pack} is not bound")
    return _bytes(tensors[pack]) if tensors[pack].dtype != torch.uint8 or tensors[pack].dim() != 1 else tensors[pack]


def _ranges(m):
    """byte ranges of a row in storage order, rows, row bytes -- for both column-blocked forms"""
    if "strips" in m:
        rows, cols, bw = m["strips"]
        return [(a, a + bw) for a in range(0, cols, bw)], rows, cols
    b = m["blocks"]
    return [tuple(r) for r in b["ranges"]], b["rows"], b["row_bytes"]


def read_member(tensors, m, dtype=None, shape=None):
    """The member's tensor.  Plain members are views of the pack's memory; column-blocked ones are gathered into a
    new row-major [rows, row_bytes] tensor."""
    raw = _pack_bytes(tensors, m["pack"])[m["offset"]:m["offset"] + m["bytes"]]
    if raw.numel() != m["bytes"]:
        raise ValueError(f"{m['name']}: pack {m['pack']} is shorter than offset + bytes")
    if "strips" in m or "blocks" in m:
        ranges, rows, row_bytes = _ranges(m)
        if sum(b - a for a, b in ranges) != row_bytes or rows * row_bytes != m["bytes"]:
            raise ValueError(f"{m['name']}: column blocks do not cover the member")
        out = torch.empty((rows, row_bytes), dtype=torch.uint8, device=raw.device)
        o = 0
        for a, b in ranges:
            n = rows * (b - a)
            out[:, a:b] = raw[o:o + n].reshape(rows, b - a)
            o += n
        raw = out.reshape(-1)
    dtype = dtype or PACK_DTYPE[pack_base(m["pack"])]
    t = raw.view(dtype)
    return t.reshape(shape) if shape is not None else t


def write_member(tensors, m, t):
    """copies t into its place in the pack (the backend's one-time fill)"""
    dst = _pack_bytes(tensors, m["pack"])
    src = _bytes(t)
    if src.numel() != m["bytes"]:
        raise ValueError(f"{m['name']}: {src.numel()} bytes given, the layout says {m['bytes']}")
    if "strips" in m or "blocks" in m:
        ranges, rows, row_bytes = _ranges(m)
        src2 = src.reshape(rows, row_bytes)
        src = torch.cat([src2[:, a:b].reshape(-1) for a, b in ranges])
    dst[m["offset"]:m["offset"] + m["bytes"]] = src


def new_packs(packs, device="cpu"):
    """zero-filled byte tensors of the packs' sizes"""
    return {p: torch.zeros(n, dtype=torch.uint8, device=device) for p, n in packs.items()}


def stored_shape(entry):
    """shape of a `params` entry in stored elements: a logical FP4 tensor (dtype code 15) holds two values per byte"""
    shape = list(entry["shape"])
    if int(entry["dtype"]) == 15:
        shape[-1] //= 2
    return shape


def unpack(kernel, tensors, params=None):
    """{layer (None for single-layer kernels): {param: tensor}} of a manifest role's `members`.  params: the manifest's
    `params` table ({kind: {name: entry}}); with it every member gets its entry's shape, without it members stay flat."""
    out = {}
    for m in kernel.get("members", []):
        shape = None
        if params is not None:
            kinds = [m["kind"]] if "kind" in m else list(params)
            for k in kinds:
                e = params.get(k, {}).get(m["param"])
                if e is not None and int(e["bytes"]) == m["bytes"]:
                    shape = stored_shape(e)
                    break
        out.setdefault(m.get("layer"), {})[m["param"]] = read_member(tensors, m, shape=shape)
    return out


# ------------------------------------------------------------------------------------------------- phase banks
def bank_input(layer, bank):
    """name of the decode group's input that holds `bank` for group layer `layer`, and the block inside it"""
    return f"k_b{layer % 4}_{bank}", layer // 4


def bank_view(tensors, layer, bank):
    name, blk = bank_input(layer, bank)
    if name not in tensors:
        raise KeyError(f"bank input {name} is not bound")
    return tensors[name][blk]


# member of a layer kind -> bank (without the k_b<phase>_ prefix), the naming of the 27B decode group
# (models/qwen38_27b/decode/q35_group.py:76-99; the w_down / w_out / w_o entries are its KSTRIDE form)
BANK_OF = {
    "gdn": {"w_gq": "attn_w_q", "s_gq": "attn_w_q_scale", "w_gk": "attn_w_k", "s_gk": "attn_w_k_scale",
            "w_gv": "attn_w_v", "s_gv": "attn_w_v_scale", "w_z": "attn_w_z", "s_z": "attn_w_z_scale",
            "w_a": "attn_w_a", "w_b": "attn_w_b", "w_gate": "mlp_w1", "s_gate": "mlp_w_scale1",
            "w_up": "mlp_w2", "s_up": "mlp_w_scale2", "w_down": "mlp_w3", "s_down": "mlp_w_scale3",
            "w_out": "attn_w_o", "s_out": "attn_w_o_scale"},
    "attn": {"w_q": "attn_w_q", "s_q": "attn_w_scale_q", "w_k": "attn_w_k", "s_k": "attn_w_scale_k",
             "w_v": "attn_w_v", "s_v": "attn_w_scale_v", "w_gate": "mlp_w1", "s_gate": "mlp_w_scale1",
             "w_up": "mlp_w2", "s_up": "mlp_w_scale2", "w_down": "mlp_w3", "s_down": "mlp_w_scale3",
             "w_o": "attn_w_o", "s_o": "attn_w_scale_o"},
}


# ------------------------------------------------------------------------------------------------- value-head order
def vperm_index(spec, length):
    """Index tensor that takes a dimension of `length` from the GGUF's TILED value-head order (head (k, r) at
    r * KH + k) to the grouped order (k * REP + r) -- `rows:<first>:<VH>:<KH>` (entries before `first` stay) or
    `cols:<VH>:<KH>` (tools/manifest/mkmanifest.py:202-219; models/qwen38_27b/prefill/check27.py:57-60)."""
    f = spec.split(":")
    first, vh, kh = (int(f[1]), int(f[2]), int(f[3])) if f[0] == "rows" else (0, int(f[1]), int(f[2]))
    hd, rem = divmod(length - first, vh)
    if rem or vh % kh:
        raise ValueError(f"vperm {spec}: {length - first} entries are not {vh} heads")
    idx = torch.arange(vh * hd).reshape(vh // kh, kh, hd).transpose(0, 1).reshape(-1) + first
    return torch.cat([torch.arange(first), idx])


def apply_vperm(t, spec):
    """t with its value heads taken from tiled to grouped order (rows of dimension 0, or equal groups of stored columns
    of the last dimension: FP4 pairs and block scales keep whole heads together)"""
    if spec.startswith("rows"):
        return t[vperm_index(spec, t.shape[0]).to(t.device)].contiguous()
    f = spec.split(":")
    vh = int(f[1])
    cols = t.shape[-1]
    hd = cols // vh  # stored columns per head
    idx = vperm_index(f"cols:{vh}:{f[2]}", vh)  # permutation of heads
    return t.reshape(*t.shape[:-1], vh, hd)[..., idx.to(t.device), :].reshape(t.shape).contiguous()


# ------------------------------------------------------------------------------------------------- conversions
def quant_mxfp4(w):
    """[N, K] float -> (E2M1 pairs [N, K / 2] u8, low nibble = even k; E8M0 [N, K / 32] u8): per 32 inputs
    e = floor(log2 amax) - 2 (0 for an all-zero block), codes = nearest of {0, .5, 1, 1.5, 2, 3, 4, 6}, ties to the lower
    code (models/qwen35_2b/whole/src/q35_moe.py:43-58)"""
    n, k = w.shape
    g = w.float().reshape(n, k // 32, 32)
    amax = g.abs().amax(-1, keepdim=True)
    e = torch.where(amax > 0, torch.floor(torch.log2(amax.clamp_min(1e-30))) - 2, torch.zeros_like(amax))
    x = (g / torch.exp2(e)).reshape(n, k)
    lut = torch.tensor(E2M1, device=w.device)
    code = ((x.abs().unsqueeze(-1) - lut).abs().argmin(-1) | ((x < 0).long() << 3)).to(torch.uint8)
    return (code[:, 0::2] | (code[:, 1::2] << 4)).contiguous(), (e.squeeze(-1) + 127).to(torch.uint8).contiguous()


def quant_mxfp8(w):
    """[N, K] float -> (E4M3 [N, K], E8M0 [N, K / 32] u8): e = ceil(log2(amax / 448)) per 32 inputs
    (models/qwen35_2b/whole/src/q35_mx_build.py:60-72)"""
    n, k = w.shape
    g = w.float().reshape(n, k // 32, 32)
    amax = g.abs().amax(-1, keepdim=True).clamp_min(2.0 ** -120)
    e = torch.ceil(torch.log2(amax / 448.0)).clamp(-127, 127)
    q = (g / torch.exp2(e)).reshape(n, k).to(torch.float8_e4m3fn)
    return q.contiguous(), (e.squeeze(-1) + 127).to(torch.uint8).contiguous()


def ggml_mxfp4_planes(blocks):
    """GGUF MXFP4 rows [..., K / 32, 17] u8 (byte 0 = E8M0 exponent, bytes 1..16: value j in the low nibble of byte j,
    value j + 16 in the high nibble -- ggml's block_mxfp4) -> (codes [..., K / 2] with value 2i in the low nibble of
    byte i, scales [..., K / 32]): the manifest's `mxfp4_planar_codes` / `mxfp4_planar_scales`."""
    if blocks.dtype != torch.uint8 or blocks.shape[-1] != 17:
        raise ValueError("ggml_mxfp4_planes: expected uint8 blocks of 17 bytes")
    qs = blocks[..., 1:]
    codes = torch.cat([qs & 15, qs >> 4], dim=-1)  # values 0..31 of the block
    packed = codes[..., 0::2] | (codes[..., 1::2] << 4)
    return packed.reshape(*blocks.shape[:-2], -1).contiguous(), blocks[..., 0].contiguous()


def convert(kind, src):
    """One `params.*.convert` conversion.  src: the GGUF tensor as torch (float for tensor / log_neg / mxfp* of an
    unquantised source, [.., K / 32, 17] u8 blocks for a GGUF MXFP4 source).  Returns the kernel-form tensor, or the
    (elements, scales) pair for the mxfp* kinds (the `<kind>_scales` entry of the same weight is its second half)."""
    if kind == "tensor":
        return src
    if kind == "log_neg":  # GGUF ssm_a = -exp(A_log)
        return torch.log(-src.float())
    if kind == "bf16_taps_reversed":  # kernel tap 0 multiplies the current token; GGUF / torch conv1d: the last tap
        return src.flip(-1).to(torch.bfloat16).contiguous()
    if kind in ("mxfp4", "mxfp4_scales", "mxfp4_planar_codes", "mxfp4_planar_scales"):
        pair = ggml_mxfp4_planes(src) if src.dtype == torch.uint8 else quant_mxfp4(src)
        return pair
    if kind in ("mxfp8", "mxfp8_scales"):
        return quant_mxfp8(src)
    raise ValueError(f"unknown conversion {kind}")


# ------------------------------------------------------------------------------------------------- a bound decode group
def _take(tensors, members, kind, j, name):
    """member `name` of group layer j: from the packs if the layout holds it, else from its phase bank"""
    if name in members.get(j, {}):
        return members[j][name]
    bank = BANK_OF[kind].get(name)
    if bank is None:
        raise KeyError(f"L{j}.{name}: neither a pack member nor a bank")
    return bank_view(tensors, j, bank)


def group_layers(manifest, role, tensors, kinds=None):
    """Per-layer weight dictionaries (the names layers.gdn / layers.attention / layers.mlp_residual take) of a manifest
    role that binds a group of layers through packs and phase banks (`decode.group`).  tensors: the role's inputs by
    the manifest's names (packs, `k_b<phase>_<bank>` banks), on the GPU.  kinds: "g" / "a" per layer; default: from the
    members' `kind` entries.  Returns (layers, kinds).  Value heads come out in grouped order."""
    k = manifest["kernels"][role]
    params = manifest.get("params", {})
    members = unpack(k, tensors, params)
    if kinds is None:
        kind_of = {}
        for m in k.get("members", []):
            if "layer" in m and "kind" in m:
                kind_of[m["layer"]] = "g" if m["kind"] == "gdn" else "a"
        kinds = [kind_of[j] for j in sorted(kind_of)]
    layers = []
    for j, kd in enumerate(kinds):
        kind = "gdn" if kd == "g" else "attn"
        P = params.get(kind, {})
        get = lambda n: _take(tensors, members, kind, j, n)  # noqa: E731
        w = {"ln2": get("ln2").reshape(-1)}
        for n in ("gate", "up", "down"):
            w["w_" + n], w["s_" + n] = get("w_" + n), get("s_" + n)
        if kind == "attn":
            w.update(ln1=get("ln1").reshape(-1), q_norm=get("q_norm").reshape(-1), k_norm=get("k_norm").reshape(-1))
            for n in ("q", "k", "v", "o"):
                w["w_" + n], w["s_" + n] = get("w_" + n), get("s_" + n)
        else:
            w["input_norm_w"] = get("ln1").reshape(-1)
            nv = P["a_log"]["shape"][0] if "a_log" in P else get("a_log").numel()
            tiled = P.get("a_log", {}).get("vperm")
            heads = (lambda t: apply_vperm(t, tiled)) if tiled else (lambda t: t)  # noqa: E731
            w["a_log"], w["dt_bias"] = heads(get("a_log").reshape(-1)), heads(get("dt_bias").reshape(-1))
            w["o_norm_w"] = get("norm_w").reshape(-1)
            for ours, theirs in (("q", "gq"), ("k", "gk")):
                w["w_" + ours], w["s_" + ours] = get("w_" + theirs), get("s_" + theirs)
            for ours, theirs in (("v", "gv"), ("z", "z"), ("a", "a"), ("b", "b")):
                w["w_" + ours], w["s_" + ours] = heads(get("w_" + theirs)), heads(get("s_" + theirs))
            wo, so = get("w_out"), get("s_out")
            if tiled:  # input columns of the output projection; per-row scales (1-D) have no such axis
                spec = f"cols:{nv}:{tiled.split(':')[-1]}"
                wo, so = apply_vperm(wo, spec), (apply_vperm(so, spec) if so.dim() == 2 else so)
            w["w_o"], w["s_o"] = wo, so
            conv = get("conv_w")  # [2 KD + VD, 4] bf16, tap 0 = current token, value channels tiled
            kd2 = conv.shape[0] - w["w_v"].shape[0]
            conv = conv.flip(-1)
            w["w_q_conv"] = conv[:kd2 // 2].contiguous()
            w["w_k_conv"] = conv[kd2 // 2:kd2].contiguous()
            w["w_v_conv"] = heads(conv[kd2:])
        layers.append(w)
    return layers, kinds
