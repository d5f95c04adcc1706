// Small per-row kernels that sit between the projections and the core kernels of a decoder layer: RMSNorm (plain and
// the folded form of the GDN sublayer), q / k norm + RoPE, GDN gates and L2 norms, gated output norm, sigmoid gate,
// SiLU * up.  All are a few bytes per token next to the weight and state streams; one block per row.
// Rounding points follow the reference's torch goldens (cited at each kernel).
#include "abi.h"
#include "common.cuh"

namespace q35 {

__device__ __forceinline__ float block_sum(float v, float* red) {  // blockDim.x <= 1024, red[32]
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = 0.f;
  const int nw = (blockDim.x + 31) >> 5;
  for (int i = 0; i < nw; ++i) t += red[i];
  return t;
}

__device__ __forceinline__ float load_w(const void* w, int w_bf16, int i) {
  return w_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(w)[i]) : static_cast<const float*>(w)[i];
}

// norm.rms.  base = bf16(x + residual) when a residual is bound.
//   plain : y = bf16(base * rsqrt(mean base^2 + eps) * w)        (attn_utils/common.py:216-228)
//   folded: y = bf16(base * w), xsqrt[t] = sqrt(mean base^2 + eps): the projections are divided by it afterwards
//           (golden reference(), models/qwen35_35b_a3b/sgl/tests/test_gdn_attn.py:437-442)
__global__ void __launch_bounds__(256) rms_kernel(const __nv_bfloat16* __restrict__ x,
                                                  const __nv_bfloat16* __restrict__ residual, const void* w, int w_bf16,
                                                  __nv_bfloat16* __restrict__ y, __nv_bfloat16* base_out,
                                                  float* xsqrt_out, int H, const float* eps_ptr, int folded) {
  __shared__ float red[32];
  const int t = blockIdx.x;
  // rows of up to 8192 channels in multiples of 8, 16-byte aligned: every thread keeps its (at most four) 16-byte
  // pieces of the row in registers, so the row is read once and all loads of a thread are in flight together -- a
  // decode step normalises a handful of rows and the latency of a load chain is all this kernel costs
  const bool vec = (H & 7) == 0 && H <= 8 * 256 * RMS_MAX_PIECES && blockDim.x == 256 &&
                   ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(residual) |
                     reinterpret_cast<uintptr_t>(base_out) | reinterpret_cast<uintptr_t>(w)) & 15) == 0;
  if (vec) {
    RmsPieces p, r;
    rms_load(x + size_t(t) * H, H, threadIdx.x, p);
    if (residual) {
      rms_load(residual + size_t(t) * H, H, threadIdx.x, r);
#pragma unroll
      for (int c = 0; c < RMS_MAX_PIECES; ++c) {
        uint32_t* pv = reinterpret_cast<uint32_t*>(&p.v[c]);
        const uint32_t* rv = reinterpret_cast<const uint32_t*>(&r.v[c]);
#pragma unroll
        for (int u = 0; u < 4; ++u) pv[u] = pack_bf16(bf16lo(pv[u]) + bf16lo(rv[u]), bf16hi(pv[u]) + bf16hi(rv[u]));
      }
    }
    const float tot = block_sum(rms_sumsq(p), red);
    const float var = tot / float(H) + (eps_ptr ? eps_ptr[0] : 1e-6f);
    const float rs = folded ? 1.f : rsqrtf(var);
    if (folded && threadIdx.x == 0) xsqrt_out[t] = sqrtf(var);
#pragma unroll
    for (int c = 0; c < RMS_MAX_PIECES; ++c) {
      const int i = (threadIdx.x + 256 * c) * 8;
      if (i >= H) break;
      if (base_out) *reinterpret_cast<uint4*>(base_out + size_t(t) * H + i) = p.v[c];
      float wv[8];
      if (w_bf16) {
        const uint4 wq = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(w) + i);
        const uint32_t ww[4] = {wq.x, wq.y, wq.z, wq.w};
#pragma unroll
        for (int u = 0; u < 4; ++u) { wv[2 * u] = bf16lo(ww[u]); wv[2 * u + 1] = bf16hi(ww[u]); }
      } else {
        const float4 w0 = *reinterpret_cast<const float4*>(static_cast<const float*>(w) + i);
        const float4 w1 = *reinterpret_cast<const float4*>(static_cast<const float*>(w) + i + 4);
        wv[0] = w0.x; wv[1] = w0.y; wv[2] = w0.z; wv[3] = w0.w; wv[4] = w1.x; wv[5] = w1.y; wv[6] = w1.z; wv[7] = w1.w;
      }
      const uint32_t pv[4] = {p.v[c].x, p.v[c].y, p.v[c].z, p.v[c].w};
      uint32_t o[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float a = bf16lo(pv[u]), b = bf16hi(pv[u]);
        o[u] = folded ? pack_bf16(a * wv[2 * u], b * wv[2 * u + 1]) : pack_bf16(a * rs * wv[2 * u], b * rs * wv[2 * u + 1]);
      }
      *reinterpret_cast<uint4*>(y + size_t(t) * H + i) = make_uint4(o[0], o[1], o[2], o[3]);
    }
    return;
  }
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = __bfloat162float(x[size_t(t) * H + i]);
    if (residual) v = round_bf16(v + __bfloat162float(residual[size_t(t) * H + i]));
    ss += v * v;
  }
  const float tot = block_sum(ss, red);
  const float var = tot / float(H) + (eps_ptr ? eps_ptr[0] : 1e-6f);
  const float rs = rsqrtf(var);
  if (folded && threadIdx.x == 0) xsqrt_out[t] = sqrtf(var);
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = __bfloat162float(x[size_t(t) * H + i]);
    if (residual) v = round_bf16(v + __bfloat162float(residual[size_t(t) * H + i]));
    if (base_out) base_out[size_t(t) * H + i] = __float2bfloat16_rn(v);
    const float wv = load_w(w, w_bf16, i);
    y[size_t(t) * H + i] = __float2bfloat16_rn(folded ? v * wv : v * rs * wv);
  }
}

int run_norm_rms(Call& c) {
  Tensor x, res, w, y, base, rstd, eps;
  Q35_TRY(c.get("x", M(Q35_BF16), &x));
  Q35_TRY(c.get("residual", M(Q35_BF16), &res, false));
  Q35_TRY(c.get("w", M(Q35_F32) | M(Q35_BF16), &w));
  Q35_TRY(c.get("y", M(Q35_BF16), &y));
  Q35_TRY(c.get("base_out", M(Q35_BF16), &base, false));
  Q35_TRY(c.get("xsqrt_out", M(Q35_F32), &rstd, false));
  Q35_TRY(c.get("eps", M(Q35_F32), &eps, false));
  Q35_REQUIRE(x.nd >= 1, Q35_ERR_SHAPE, "norm.rms: x [T, H]");
  const int64_t H = x.s[x.nd - 1], T = x.numel() / (H ? H : 1);
  Q35_REQUIRE(w.numel() == H && y.numel() == x.numel(), Q35_ERR_SHAPE, "norm.rms: w [H], y like x");
  Q35_REQUIRE(!res.present || res.numel() == x.numel(), Q35_ERR_SHAPE, "norm.rms: residual like x");
  Q35_REQUIRE(!base.present || base.numel() == x.numel(), Q35_ERR_SHAPE, "norm.rms: base_out like x");
  Q35_REQUIRE(!rstd.present || rstd.numel() == T, Q35_ERR_SHAPE, "norm.rms: xsqrt_out [T]");
  c.ws_need = 0;
  if (c.dry || T == 0) return 0;
  rms_kernel<<<unsigned(T), 256, 0, c.stream>>>(x.as<__nv_bfloat16>(), res.present ? res.as<__nv_bfloat16>() : nullptr,
                                                w.p, w.dtype == Q35_BF16, y.as<__nv_bfloat16>(),
                                                base.present ? base.as<__nv_bfloat16>() : nullptr,
                                                rstd.present ? rstd.as<float>() : nullptr, int(H),
                                                eps.present ? eps.as<float>() : nullptr,
                                                rstd.present ? 1 : 0);
  Q35_CUDA_LAUNCH_CHECK("norm.rms");
  return 0;
}

// gdn.prep: per token, per head: q = bf16(bf16(q / sqrt(sum q^2 + 1e-6)) * dk^-0.5), k = bf16(k / sqrt(sum k^2 + 1e-6)),
// g = -exp(A_log) * softplus(a + dt_bias) (fp32), beta = bf16(sigmoid(b))
// (gdn_reference, models/qwen35_35b_a3b/sgl/tests/test_gdn_attn.py:260-270; kernels gdn.py:919-949, 1631-1632)
__global__ void __launch_bounds__(128) gdn_prep_kernel(const __nv_bfloat16* __restrict__ q,
                                                       const __nv_bfloat16* __restrict__ k,
                                                       const __nv_bfloat16* __restrict__ a,
                                                       const __nv_bfloat16* __restrict__ b,
                                                       const float* __restrict__ a_log, const void* dt_bias, int dt_bf16,
                                                       __nv_bfloat16* __restrict__ qn, __nv_bfloat16* __restrict__ kn,
                                                       float* __restrict__ g, __nv_bfloat16* __restrict__ beta, int NK,
                                                       int NV, int DK) {
  const int row = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float qscale = rsqrtf(float(DK));
  // heads of q then heads of k, one per warp: blockIdx.y spreads them over CTAs (a decode step has few rows)
  for (int h = warp + 4 * blockIdx.y; h < 2 * NK; h += 4 * gridDim.y) {
    const bool is_k = h >= NK;
    const __nv_bfloat16* src = (is_k ? k : q) + (size_t(row) * NK + (is_k ? h - NK : h)) * DK;
    __nv_bfloat16* dst = (is_k ? kn : qn) + (size_t(row) * NK + (is_k ? h - NK : h)) * DK;
    float ss = 0.f;
    for (int i = lane; i < DK; i += 32) { const float v = __bfloat162float(src[i]); ss += v * v; }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss + 1e-6f);
    for (int i = lane; i < DK; i += 32) {
      float v = round_bf16(__bfloat162float(src[i]) * inv);
      if (!is_k) v = v * qscale;
      dst[i] = __float2bfloat16_rn(v);
    }
  }
  if (blockIdx.y != 0) return;
  for (int h = threadIdx.x; h < NV; h += blockDim.x) {
    const float av = __bfloat162float(a[size_t(row) * NV + h]) + load_w(dt_bias, dt_bf16, h);
    const float sp = av > 20.f ? av : log1pf(expf(av));
    g[size_t(row) * NV + h] = -expf(a_log[h]) * sp;
    beta[size_t(row) * NV + h] = __float2bfloat16_rn(1.0f / (1.0f + expf(-__bfloat162float(b[size_t(row) * NV + h]))));
  }
}

int run_gdn_prep(Call& c) {
  Tensor q, k, a, b, alog, dtb, qn, kn, g, beta;
  Q35_TRY(c.get("q", M(Q35_BF16), &q));
  Q35_TRY(c.get("k", M(Q35_BF16), &k));
  Q35_TRY(c.get("a", M(Q35_BF16), &a));
  Q35_TRY(c.get("b", M(Q35_BF16), &b));
  Q35_TRY(c.get("a_log", M(Q35_F32), &alog));
  Q35_TRY(c.get("dt_bias", M(Q35_F32) | M(Q35_BF16), &dtb));
  Q35_TRY(c.get("q_out", M(Q35_BF16), &qn));
  Q35_TRY(c.get("k_out", M(Q35_BF16), &kn));
  Q35_TRY(c.get("g", M(Q35_F32), &g));
  Q35_TRY(c.get("beta", M(Q35_BF16), &beta));
  Q35_REQUIRE(q.nd >= 3, Q35_ERR_SHAPE, "gdn.prep: q [.., NK, DK]");
  const int64_t DK = q.s[q.nd - 1], NK = q.s[q.nd - 2], R = q.numel() / (NK * DK), NV = alog.numel();
  Q35_REQUIRE(k.numel() == q.numel() && qn.numel() == q.numel() && kn.numel() == q.numel(), Q35_ERR_SHAPE, "gdn.prep: q / k");
  Q35_REQUIRE(a.numel() == R * NV && b.numel() == R * NV && g.numel() == R * NV && beta.numel() == R * NV &&
                  dtb.numel() == NV, Q35_ERR_SHAPE, "gdn.prep: a / b / g / beta [R, NV], dt_bias [NV]");
  c.ws_need = 0;
  if (c.dry || R == 0) return 0;
  gdn_prep_kernel<<<dim3(unsigned(R), unsigned((2 * NK + 3) / 4)), 128, 0, c.stream>>>(q.as<__nv_bfloat16>(), k.as<__nv_bfloat16>(), a.as<__nv_bfloat16>(),
                                                     b.as<__nv_bfloat16>(), alog.as<float>(), dtb.p, dtb.dtype == Q35_BF16,
                                                     qn.as<__nv_bfloat16>(), kn.as<__nv_bfloat16>(), g.as<float>(),
                                                     beta.as<__nv_bfloat16>(), int(NK), int(NV), int(DK));
  Q35_CUDA_LAUNCH_CHECK("gdn.prep");
  return 0;
}

// gdn.out_norm: per (token, value head): n = bf16(core * rsqrt(mean core^2 + eps) * w); y = bf16(n * bf16(silu(z)))
// (reference(), models/qwen35_35b_a3b/sgl/tests/test_gdn_attn.py:466-469)
__global__ void __launch_bounds__(128) gdn_out_norm_kernel(const __nv_bfloat16* __restrict__ core,
                                                           const __nv_bfloat16* __restrict__ z, const void* w, int w_bf16,
                                                           __nv_bfloat16* __restrict__ y, int heads, int DV, const float* eps_ptr) {
  const int row = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float eps = eps_ptr ? eps_ptr[0] : 1e-6f;
  for (int h = warp + 4 * blockIdx.y; h < heads; h += 4 * gridDim.y) {  // one head per warp, heads over blockIdx.y
    const size_t o = (size_t(row) * heads + h) * DV;
    float ss = 0.f;
    for (int i = lane; i < DV; i += 32) { const float v = __bfloat162float(core[o + i]); ss += v * v; }
    ss = warp_sum(ss);
    const float rs = rsqrtf(ss / float(DV) + eps);
    for (int i = lane; i < DV; i += 32) {
      const float n = round_bf16(__bfloat162float(core[o + i]) * rs * load_w(w, w_bf16, i));
      const float zv = __bfloat162float(z[o + i]);
      y[o + i] = __float2bfloat16_rn(n * round_bf16(zv / (1.0f + expf(-zv))));
    }
  }
}

int run_gdn_out_norm(Call& c) {
  Tensor core, z, w, y, eps;
  Q35_TRY(c.get("eps", M(Q35_F32), &eps, false));
  Q35_TRY(c.get("core", M(Q35_BF16), &core));
  Q35_TRY(c.get("z", M(Q35_BF16), &z));
  Q35_TRY(c.get("w", M(Q35_F32) | M(Q35_BF16), &w));
  Q35_TRY(c.get("y", M(Q35_BF16), &y));
  Q35_REQUIRE(core.nd >= 3, Q35_ERR_SHAPE, "gdn.out_norm: core [.., NV, DV]");
  const int64_t DV = core.s[core.nd - 1], NV = core.s[core.nd - 2], R = core.numel() / (NV * DV);
  Q35_REQUIRE(z.numel() == core.numel() && y.numel() == core.numel() && w.numel() == DV, Q35_ERR_SHAPE, "gdn.out_norm: shapes");
  c.ws_need = 0;
  if (c.dry || R == 0) return 0;
  gdn_out_norm_kernel<<<dim3(unsigned(R), unsigned((NV + 3) / 4)), 128, 0, c.stream>>>(core.as<__nv_bfloat16>(), z.as<__nv_bfloat16>(), w.p,
                                                         w.dtype == Q35_BF16, y.as<__nv_bfloat16>(), int(NV), int(DV),
                                                         eps.present ? eps.as<float>() : nullptr);
  Q35_CUDA_LAUNCH_CHECK("gdn.out_norm");
  return 0;
}

// attn.qk_prep: per token: split q | gate per head (when gated), RMSNorm of q and k heads, NeoX RoPE on the first
// `rot` channels (golden: models/qwen35_35b_a3b/sgl/tests/test_qwen35_runtime.py:57-72; kernel q35_step.py:192-200)
__global__ void __launch_bounds__(256) attn_qk_prep_kernel(const __nv_bfloat16* __restrict__ qg,
                                                           const __nv_bfloat16* __restrict__ k,
                                                           const float* __restrict__ qw, const float* __restrict__ kw,
                                                           const float* __restrict__ cosv, const float* __restrict__ sinv,
                                                           __nv_bfloat16* __restrict__ q_out,
                                                           __nv_bfloat16* __restrict__ k_out,
                                                           __nv_bfloat16* __restrict__ gate_out, int HQ, int HKV, int D,
                                                           int rot, int gated, const float* eps_ptr) {
  const int row = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int half = rot / 2;
  const float eps = eps_ptr ? eps_ptr[0] : 1e-6f;
  for (int h = warp + 8 * blockIdx.y; h < HQ + HKV; h += 8 * gridDim.y) {  // one head per warp, heads over blockIdx.y
    const bool is_k = h >= HQ;
    const int hh = is_k ? h - HQ : h;
    const __nv_bfloat16* src = is_k ? k + (size_t(row) * HKV + hh) * D : qg + (size_t(row) * HQ + hh) * (gated ? 2 * D : D);
    __nv_bfloat16* dst = is_k ? k_out + (size_t(row) * HKV + hh) * D : q_out + (size_t(row) * HQ + hh) * D;
    const float* w = is_k ? kw : qw;
    float ss = 0.f;
    for (int i = lane; i < D; i += 32) { const float v = __bfloat162float(src[i]); ss += v * v; }
    ss = warp_sum(ss);
    const float rs = rsqrtf(ss / float(D) + eps);
    for (int i = lane; i < D; i += 32) {
      const float n = round_bf16(__bfloat162float(src[i]) * rs * w[i]);
      float o = n;
      if (i < rot) {  // partner channel normalised the same way
        const int j = i < half ? i + half : i - half;
        const float pn = round_bf16(__bfloat162float(src[j]) * rs * w[j]);
        const float cs = cosv[size_t(row) * half + (i < half ? i : i - half)];
        const float sn = sinv[size_t(row) * half + (i < half ? i : i - half)];
        o = i < half ? n * cs - pn * sn : n * cs + pn * sn;
      }
      dst[i] = __float2bfloat16_rn(o);
    }
    if (!is_k && gated)
      for (int i = lane; i < D; i += 32) gate_out[(size_t(row) * HQ + hh) * D + i] = src[D + i];
  }
}

int run_attn_qk_prep(Call& c) {
  Tensor qg, k, qw, kw, cs, sn, qo, ko, go, eps;
  Q35_TRY(c.get("eps", M(Q35_F32), &eps, false));
  Q35_TRY(c.get("qg", M(Q35_BF16), &qg));
  Q35_TRY(c.get("k", M(Q35_BF16), &k));
  Q35_TRY(c.get("q_norm", M(Q35_F32), &qw));
  Q35_TRY(c.get("k_norm", M(Q35_F32), &kw));
  Q35_TRY(c.get("cos", M(Q35_F32), &cs));
  Q35_TRY(c.get("sin", M(Q35_F32), &sn));
  Q35_TRY(c.get("q_out", M(Q35_BF16), &qo));
  Q35_TRY(c.get("k_out", M(Q35_BF16), &ko));
  Q35_TRY(c.get("gate_out", M(Q35_BF16), &go, false));
  Q35_REQUIRE(qo.nd == 3 && ko.nd == 3, Q35_ERR_SHAPE, "attn.qk_prep: q_out [R, HQ, D], k_out [R, HKV, D]");
  const int64_t R = qo.s[0], HQ = qo.s[1], D = qo.s[2], HKV = ko.s[1];
  const bool gated = go.present;
  Q35_REQUIRE(qg.numel() == R * HQ * D * (gated ? 2 : 1) && k.numel() == R * HKV * D && ko.s[0] == R && ko.s[2] == D,
              Q35_ERR_SHAPE, "attn.qk_prep: qg [R, HQ, D or 2D], k [R, HKV, D]");
  Q35_REQUIRE(qw.numel() == D && kw.numel() == D && cs.numel() == sn.numel() && cs.numel() % (R ? R : 1) == 0,
              Q35_ERR_SHAPE, "attn.qk_prep: norms [D], cos / sin [R, rot/2]");
  const int64_t rot = R ? 2 * cs.numel() / R : 0;
  Q35_REQUIRE(rot <= D && rot % 2 == 0 && (!gated || go.numel() == R * HQ * D), Q35_ERR_SHAPE, "attn.qk_prep: rot / gate_out");
  c.ws_need = 0;
  if (c.dry || R == 0) return 0;
  attn_qk_prep_kernel<<<dim3(unsigned(R), unsigned((HQ + HKV + 7) / 8)), 256, 0, c.stream>>>(
      qg.as<__nv_bfloat16>(), k.as<__nv_bfloat16>(), qw.as<float>(), kw.as<float>(), cs.as<float>(), sn.as<float>(),
      qo.as<__nv_bfloat16>(), ko.as<__nv_bfloat16>(), gated ? go.as<__nv_bfloat16>() : nullptr, int(HQ), int(HKV),
      int(D), int(rot), gated, eps.present ? eps.as<float>() : nullptr);
  Q35_CUDA_LAUNCH_CHECK("attn.qk_prep");
  return 0;
}

// act: elementwise pairs.  mode 0: y = bf16(silu(a) * b) (SwiGLU, q35_step.py:131-133); mode 1: y = bf16(a * sigmoid(b))
// (attention output gate, test_qwen35_runtime.py:86-87)
__global__ void act_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                           __nv_bfloat16* __restrict__ y, long long n, int mode) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float av = __bfloat162float(a[i]), bv = __bfloat162float(b[i]);
  y[i] = __float2bfloat16_rn(mode == 0 ? av / (1.0f + expf(-av)) * bv : av / (1.0f + expf(-bv)));
}

static int run_act(Call& c, int mode, const char* what) {
  Tensor a, b, y;
  Q35_TRY(c.get("a", M(Q35_BF16), &a));
  Q35_TRY(c.get("b", M(Q35_BF16), &b));
  Q35_TRY(c.get("y", M(Q35_BF16), &y));
  Q35_REQUIRE(b.numel() == a.numel() && y.numel() == a.numel(), Q35_ERR_SHAPE, "%s: a, b, y of equal size", what);
  c.ws_need = 0;
  if (c.dry || a.numel() == 0) return 0;
  act_kernel<<<unsigned((a.numel() + 255) / 256), 256, 0, c.stream>>>(a.as<__nv_bfloat16>(), b.as<__nv_bfloat16>(),
                                                                     y.as<__nv_bfloat16>(), a.numel(), mode);
  Q35_CUDA_LAUNCH_CHECK(what);
  return 0;
}
int run_act_silu_mul(Call& c) { return run_act(c, 0, "act.silu_mul"); }
int run_act_sigmoid_gate(Call& c) { return run_act(c, 1, "act.sigmoid_gate"); }

}  // namespace q35
