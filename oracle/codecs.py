"""Numeric formats of the runtime weights and the FP8 KV cache (CPU oracle; test infrastructure only).

Bytes are what the kernels receive: uint8 tensors for FP4 pairs and E8M0 scales, float8_e4m3fn for FP8.
"""
import torch

GROUP = 32  # MX block: one E8M0 scale per 32 input channels
NVG = 16  # NVFP4 block
E2M1 = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
FP4_LUT = torch.tensor([0, 0.5, 1, 1.5, 2, 3, 4, 6, -0.0, -0.5, -1, -1.5, -2, -3, -4, -6])


def quant_mxfp4(w):
    """[N, K] float -> (FP4 pairs [N, K/2] uint8, low nibble = even k; E8M0 [N, K/32] uint8).

    models/qwen35_2b/whole/src/q35_moe.py:46-57: scale 2^(floor(log2 amax) - 2) per 32 inputs (0 when the block
    is all zero), elements to the nearest E2M1 magnitude (argmin: ties go to the smaller code), sign in bit 3.
    """
    n, k = w.shape
    g = w.float().reshape(n, k // GROUP, GROUP)
    amax = g.abs().amax(-1, keepdim=True)
    e = torch.where(amax > 0, torch.floor(torch.log2(amax.clamp_min(1e-30))) - 2, torch.zeros_like(amax))
    x = (g / torch.exp2(e)).reshape(n, k)
    code = (x.abs().unsqueeze(-1) - E2M1).abs().argmin(-1) | ((x < 0).long() << 3)
    code = code.to(torch.uint8)
    packed = code[:, 0::2] | (code[:, 1::2] << 4)
    return packed.contiguous(), (e.squeeze(-1) + 127).to(torch.uint8).contiguous()


def dequant_mxfp4(packed, scale):
    """models/qwen35_2b/whole/src/q35_moe.py:60-63. Leading dims are kept: [..., N, K/2] -> [..., N, K] fp32."""
    packed = packed.view(torch.uint8)
    scale = scale.view(torch.uint8)
    lead = packed.shape[:-1]
    code = torch.stack([packed & 15, packed >> 4], -1).reshape(*lead, -1).long()
    v = E2M1[code & 7] * torch.where(code >= 8, -1.0, 1.0)
    s = torch.exp2(scale.float() - 127).unsqueeze(-1)
    return (v.reshape(*lead, -1, GROUP) * s).reshape(*lead, -1)


def random_mxfp4(shape, gen, exp_lo=-8, exp_hi=0):
    """Packed weights drawn directly in code space (codes uniform over the 16 values, E8M0 exponent uniform in
    [exp_lo, exp_hi]); same idea as random_mxfp4_weights in
    models/qwen35_35b_a3b/sgl/tests/test_gdn_attn.py:218-238. shape = logical [..., N, K]."""
    *lead, n, k = shape
    packed = torch.randint(0, 256, (*lead, n, k // 2), generator=gen, dtype=torch.int32).to(torch.uint8)
    scale = torch.randint(127 + exp_lo, 127 + exp_hi + 1, (*lead, n, k // GROUP), generator=gen,
                          dtype=torch.int32).to(torch.uint8)
    return packed, scale


def quant_mxfp8(w):
    """[N, K] -> (e4m3 [N, K], E8M0 [N, K/32] uint8); models/qwen35_2b/whole/src/q35_mx_build.py:60-67."""
    g = w.float().reshape(w.shape[0], -1, GROUP)
    amax = g.abs().amax(-1, keepdim=True).clamp_min(2.0 ** -126)
    e = torch.ceil(torch.log2(amax / 448.0)).clamp(-127, 127)
    q8 = (g / torch.exp2(e)).to(torch.float8_e4m3fn).reshape(w.shape)
    return q8.contiguous(), (e.squeeze(-1) + 127).to(torch.uint8).contiguous()


def dequant_mxfp8(q8, scale):
    """models/qwen35_2b/whole/src/q35_mx_build.py:70-72."""
    s = torch.exp2(scale.view(torch.uint8).float() - 127).repeat_interleave(GROUP, dim=-1)
    return q8.float() * s


def quant_fp8_rowwise(w):
    """[N, K] -> (e4m3 [N, K], fp32 scale [N] = amax_row / 448): the per-row form consumed by fp8_gemm
    (models/qwen35_35b_a3b/sgl/python/sgl_kernel_axera/gemm.py:137-145: operand * scale[:, None])."""
    s = (w.float().abs().amax(-1) / 448.0).clamp_min(2.0 ** -126)
    return (w.float() / s[:, None]).to(torch.float8_e4m3fn).contiguous(), s.float().contiguous()


def dequant_fp8_rowwise(q8, s):
    return q8.float() * s.float()[:, None]


def fp8_gemm(a, b_t, scale_a, scale_b, out_dtype=torch.bfloat16, bias=None):
    """out = (a * sa[:, None]) @ (b_t * sb[:, None]).T + bias; operands are scaled into the OUTPUT dtype first,
    products accumulate in fp32, one cast at the end (gemm.py:143-151)."""
    a_s = (a.float() * scale_a.float()[:, None]).to(out_dtype).float()
    b_s = (b_t.float() * scale_b.float()[:, None]).to(out_dtype).float()
    out = a_s @ b_s.T
    if bias is not None:
        out = out + bias.float()[None, :]
    return out.to(out_dtype)


def quant_nvfp4(w):
    """models/qwen35_2b/whole/src/q35_mx_build.py:168-179 (E2M1 pairs, E4M3 scale per 16, fp32 global scale)."""
    n, k = w.shape
    s2 = (w.float().abs().max() / (6.0 * 448.0)).clamp_min(2.0 ** -126)
    g = w.float().reshape(n, k // NVG, NVG)
    sc = (g.abs().amax(-1, keepdim=True) / 6.0 / s2).to(torch.float8_e4m3fn)
    d = sc.float() * s2
    x = torch.where(d > 0, g / d, torch.zeros_like(g)).reshape(n, k)
    code = ((x.abs().unsqueeze(-1) - E2M1).abs().argmin(-1) | ((x < 0).long() << 3)).to(torch.uint8)
    pk = (code[:, 0::2] | (code[:, 1::2] << 4)).contiguous()
    return pk, sc.reshape(n, k // NVG).contiguous(), s2.reshape(1).float()


def dequant_nvfp4(pk, sc, s2):
    """models/qwen35_2b/whole/src/q35_mx_build.py:182-186."""
    code = pk.view(torch.uint8)
    code = torch.stack([code & 15, code >> 4], -1).reshape(code.shape[0], -1).long()
    v = E2M1[code & 7] * torch.where(code >= 8, -1.0, 1.0)
    return (v.reshape(v.shape[0], -1, NVG) * (sc.float() * s2).unsqueeze(-1)).reshape(v.shape[0], -1)


KV8_SCALE = 8.0  # models/qwen38_27b/decode/q35_group.py:48-54: cache holds e4m3(8 x), consumers multiply by 1/8


def kv_quant_fp8(x, scale=None):
    """bf16/fp32 rows -> e4m3.  scale None: the reference's constant form e4m3(x * 8)
    (models/qwen38_27b/decode/q35_group.py:244-249).  scale [HKV] (per KV head, fp32): e4m3(x / scale_h) with x
    [..., HKV, D] -- the per-head form of the paged-decode config; the reference has no exact counterpart (its other
    variant is int8 with a per-row-per-head scale, q35_group.py:198-205)."""
    if scale is None:
        return (x.float() * KV8_SCALE).to(torch.float8_e4m3fn)
    return (x.float() / scale.float().reshape(*([1] * (x.dim() - 2)), -1, 1)).to(torch.float8_e4m3fn)


def kv_quant_int8_rows(x):
    """[..., HKV, D] bf16 -> (int8 [..., HKV, D], bf16 scale [..., HKV]): amax per head (at least 1e-5), s = bf16(amax *
    bf16(1 / 127)), q = round(bf16(x * bf16(1 / s))) -- kv_quant_row (models/qwen38_27b/decode/q35_group.py:198-205),
    every product rounded to bf16 as the reference's bf16 ops do.  Parity unpinned: the reference has these lines only
    as kernel DSL (no torch function to import, no inline golden), so this restates their operation sequence."""
    bf = lambda t: t.to(torch.bfloat16).float()  # noqa: E731
    xb = x.to(torch.bfloat16).float()
    amax = torch.maximum(xb.abs().amax(-1, keepdim=True), bf(torch.tensor(1e-5)))
    sc = bf(amax * bf(torch.tensor(1.0 / 127)))
    q = torch.round(bf(xb * bf(1.0 / sc))).clamp(-127, 127).to(torch.int8)
    return q, sc.squeeze(-1).to(torch.bfloat16)


def kv_dequant_int8_rows(q, sc):
    """bf16(int8 * scale) as the reference's page dequantisation (kv_page, q35_group.py:208-222), returned as fp32"""
    return (q.float() * sc.float().unsqueeze(-1)).to(torch.bfloat16).float()


def kv_dequant_fp8(c, scale=None):
    if scale is None:
        return c.float() / KV8_SCALE
    return c.float() * scale.float().reshape(*([1] * (c.dim() - 2)), -1, 1)


def quant_mxfp4_head(w):
    """MXFP4 as the output-projection tools pack it (models/qwen38_27b/head/mx4_common.py:11-36): the same rule as
    quant_mxfp4 with the scale byte clamped to [0, 254] (0xFF is the E8M0 NaN)."""
    w = w.float()
    n, k = w.shape
    g = w.reshape(n, k // 32, 32)
    amax = g.abs().amax(-1)
    e = torch.where(amax > 0, torch.floor(torch.log2(amax.clamp_min(1e-30))) - 2, torch.zeros_like(amax))
    x = g / torch.exp2(e).unsqueeze(-1)
    lut = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
    best = (x.abs().unsqueeze(-1) - lut).abs().argmin(-1).to(torch.uint8)  # ties go to the lower code
    code = best | ((x < 0).to(torch.uint8) << 3)
    packed = (code[..., 0::2] | (code[..., 1::2] << 4)).reshape(n, k // 2)
    return packed.contiguous(), (e + 127).clamp(0, 254).to(torch.uint8).contiguous()


def lm_head_logits(x, packed, scale):
    """fp32 logits x @ dequant(w)^T and the greedy token (first index of the maximum): torch_logits,
    models/qwen38_27b/head/mx4_common.py:62-69; the kernel role is mul_mat_mx4
    (models/qwen35_2b/whole/src/q35_layer_mc.py:741-758)."""
    logits = torch.empty((x.shape[0], packed.shape[0]), dtype=torch.float32)
    for r0 in range(0, packed.shape[0], 8192):  # row chunks, as the reference does, to keep the temporaries small
        logits[:, r0:r0 + 8192] = x.float() @ dequant_mxfp4(packed[r0:r0 + 8192], scale[r0:r0 + 8192]).T
    return logits, logits.argmax(-1).to(torch.int32)
