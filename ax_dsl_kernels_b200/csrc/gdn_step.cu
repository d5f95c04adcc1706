// Gated delta net, decode: recurrent state update for one token per sequence, and the causal conv1d + SiLU front end.
//
// Reference semantics: gdn_recurrent_step (models/qwen35_35b_a3b/sgl/python/sgl_kernel_axera/attention/gdn.py:952-989)
// and its golden loop (models/qwen35_35b_a3b/sgl/tests/test_gdn_attn.py:272-296):
//   S *= exp(g); p = bf16(k . S); err = bf16(bf16(v - p) * beta); S += k (x) err; o = bf16(q . S)
// per (sequence, value head); key head = value head / (NV / NK) (grouped order).
//
// HBM-bound: the fp32 state [DK, DV] = 64 KB per head is read once and written once; everything else is noise.
// One CTA of 128 threads owns one head's state entirely in registers (each thread a 32-row x 4-column patch), so
// every state byte crosses HBM exactly twice and all 64 KB of loads are in flight before the first use.
#include "abi.h"
#include "common.cuh"

namespace q35 {

constexpr int GD = 128;  // DK = DV = 128 for every Qwen3.5 / 3.8 configuration

__global__ void __launch_bounds__(128) gdn_step_kernel(const __nv_bfloat16* __restrict__ q,
                                                      const __nv_bfloat16* __restrict__ k,
                                                      const __nv_bfloat16* __restrict__ v, const float* __restrict__ g,
                                                      const __nv_bfloat16* __restrict__ beta, const float* state_in,
                                                      __nv_bfloat16* __restrict__ o, float* state_out, int NK, int NV) {
  pdl_wait();
  pdl_launch();
  const int bh = blockIdx.x;  // b * NV + vh
  const int b = bh / NV, vh = bh % NV;
  const int kh = vh / (NV / NK);
  const int tid = threadIdx.x;
  const int cq = tid & 31;   // column quad: columns 4 cq .. 4 cq + 3
  const int slab = tid >> 5; // rows 32 slab .. 32 slab + 31

  __shared__ float s_k[GD], s_q[GD];
  __shared__ float s_part[4][GD];

  // all state loads first: 32 independent 16-byte loads per thread
  const float4* sin = reinterpret_cast<const float4*>(state_in + size_t(bh) * GD * GD);
  float4 S[32];
#pragma unroll
  for (int r = 0; r < 32; ++r) S[r] = __ldcs(&sin[(slab * 32 + r) * (GD / 4) + cq]);

  s_k[tid] = __bfloat162float(k[(size_t(b) * NK + kh) * GD + tid]);
  s_q[tid] = __bfloat162float(q[(size_t(b) * NK + kh) * GD + tid]);
  const float decay = expf(g[bh]);
  const float bt = __bfloat162float(beta[bh]);
  const uint2 vraw = *reinterpret_cast<const uint2*>(v + size_t(bh) * GD + cq * 4);
  __syncthreads();

  float4 p = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int r = 0; r < 32; ++r) {
    const float kr = s_k[slab * 32 + r];
    S[r].x *= decay; S[r].y *= decay; S[r].z *= decay; S[r].w *= decay;
    p.x = fmaf(kr, S[r].x, p.x); p.y = fmaf(kr, S[r].y, p.y);
    p.z = fmaf(kr, S[r].z, p.z); p.w = fmaf(kr, S[r].w, p.w);
  }
  *reinterpret_cast<float4*>(&s_part[slab][cq * 4]) = p;
  __syncthreads();
  float e[4];
  {
    const float vv[4] = {bf16lo(vraw.x), bf16hi(vraw.x), bf16lo(vraw.y), bf16hi(vraw.y)};
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int col = cq * 4 + c;
      const float pred = round_bf16(s_part[0][col] + s_part[1][col] + s_part[2][col] + s_part[3][col]);
      e[c] = round_bf16(round_bf16(vv[c] - pred) * bt);
    }
  }
  __syncthreads();  // s_part is reused for the output partials
  float4 op = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int r = 0; r < 32; ++r) {
    const float kr = s_k[slab * 32 + r], qr = s_q[slab * 32 + r];
    S[r].x = fmaf(kr, e[0], S[r].x); S[r].y = fmaf(kr, e[1], S[r].y);
    S[r].z = fmaf(kr, e[2], S[r].z); S[r].w = fmaf(kr, e[3], S[r].w);
    op.x = fmaf(qr, S[r].x, op.x); op.y = fmaf(qr, S[r].y, op.y);
    op.z = fmaf(qr, S[r].z, op.z); op.w = fmaf(qr, S[r].w, op.w);
  }
  float4* sout = reinterpret_cast<float4*>(state_out + size_t(bh) * GD * GD);
#pragma unroll
  for (int r = 0; r < 32; ++r) __stcs(&sout[(slab * 32 + r) * (GD / 4) + cq], S[r]);
  *reinterpret_cast<float4*>(&s_part[slab][cq * 4]) = op;
  __syncthreads();
  if (tid < GD) {
    const float ov = s_part[0][tid] + s_part[1][tid] + s_part[2][tid] + s_part[3][tid];
    o[size_t(bh) * GD + tid] = __float2bfloat16_rn(ov);
  }
}

int run_gdn_step(Call& c) {
  Tensor q, k, v, g, beta, sin, o, sout;
  Q35_TRY(c.get("q", M(Q35_BF16), &q));
  Q35_TRY(c.get("k", M(Q35_BF16), &k));
  Q35_TRY(c.get("v", M(Q35_BF16), &v));
  Q35_TRY(c.get("g", M(Q35_F32), &g));
  Q35_TRY(c.get("beta", M(Q35_BF16), &beta));
  Q35_TRY(c.get("state_in", M(Q35_F32), &sin));
  Q35_TRY(c.get("o", M(Q35_BF16), &o));
  Q35_TRY(c.get("state_out", M(Q35_F32), &sout));
  Q35_REQUIRE(q.nd == 3 && k.nd == 3 && v.nd == 3, Q35_ERR_SHAPE, "gdn.step: q, k, v must be [B, heads, dim]");
  const int64_t B = q.s[0], NK = q.s[1], NV = v.s[1];
  Q35_REQUIRE(q.s[2] == GD && v.s[2] == GD, Q35_ERR_UNSUPPORTED, "gdn.step: head dims must be 128 (got %lld, %lld)",
              (long long)q.s[2], (long long)v.s[2]);
  Q35_REQUIRE(k.s[0] == B && k.s[1] == NK && k.s[2] == GD && v.s[0] == B, Q35_ERR_SHAPE, "gdn.step: k / v shape");
  Q35_REQUIRE(NK > 0 && NV % NK == 0, Q35_ERR_SHAPE, "gdn.step: NV %lld not a multiple of NK %lld", (long long)NV,
              (long long)NK);
  Q35_REQUIRE(g.numel() == B * NV && beta.numel() == B * NV, Q35_ERR_SHAPE, "gdn.step: g / beta must be [B, NV]");
  Q35_REQUIRE(sin.numel() == B * NV * GD * GD && sout.numel() == sin.numel(), Q35_ERR_SHAPE,
              "gdn.step: state must be [B, NV, 128, 128]");
  Q35_REQUIRE(o.numel() == B * NV * GD, Q35_ERR_SHAPE, "gdn.step: o must be [B, NV, 128]");
  c.ws_need = 0;
  if (c.dry || B * NV == 0) return 0;
  Q35_REQUIRE(aligned16(sin.p) && aligned16(sout.p) && aligned16(v.p), Q35_ERR_ALIGN, "gdn.step: 16-byte alignment");
  launch_pdl(gdn_step_kernel, dim3(unsigned(B * NV)), dim3(128), 0, c.stream, q.as<__nv_bfloat16>(),
             k.as<__nv_bfloat16>(), v.as<__nv_bfloat16>(), g.as<float>(), beta.as<__nv_bfloat16>(), sin.as<float>(),
             o.as<__nv_bfloat16>(), sout.as<float>(), int(NK), int(NV));
  Q35_CUDA_LAUNCH_CHECK("gdn.step");
  return 0;
}

// ---------------------------------------------------------------------------------------------------------------
// causal depthwise conv1d (kernel KW <= 8) + SiLU with state, T >= 1 tokens.
// Golden: causal_conv1d_silu_reference (models/qwen35_35b_a3b/sgl/tests/test_gdn_attn.py:241-257): taps in
// checkpoint order (column KW-1 multiplies the current token), accumulated newest tap first with a bf16 rounding
// after every tap, SiLU in fp32, new state = last KW-1 rows of [state; x].
template <int KW>
__global__ void gdn_conv_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                const __nv_bfloat16* conv_in, __nv_bfloat16* __restrict__ y, __nv_bfloat16* conv_out,
                                int T, int C, int t_chunk) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int b = blockIdx.z;
  if (c >= C) return;
  const int t0 = blockIdx.y * t_chunk;
  const int t1 = min(T, t0 + t_chunk);
  constexpr int SL = KW - 1;
  float wt[KW];
#pragma unroll
  for (int j = 0; j < KW; ++j) wt[j] = __bfloat162float(w[size_t(c) * KW + j]);
  const __nv_bfloat16* xb = x + size_t(b) * T * C;
  const __nv_bfloat16* sb = conv_in + size_t(b) * SL * C;
  // window[j] = input at time t - (KW - 1) + j
  float win[KW];
#pragma unroll
  for (int j = 0; j < KW; ++j) {
    const int ti = t0 - SL + j;  // time index, negative = state rows
    win[j] = (j == KW - 1) ? 0.f
             : (ti >= 0 ? __bfloat162float(xb[size_t(ti) * C + c]) : __bfloat162float(sb[size_t(ti + SL) * C + c]));
  }
  for (int t = t0; t < t1; ++t) {
    win[KW - 1] = __bfloat162float(xb[size_t(t) * C + c]);
    float acc = 0.f;
#pragma unroll
    for (int off = 0; off < KW; ++off) acc = round_bf16(acc + win[KW - 1 - off] * wt[KW - 1 - off]);
    const float s = acc / (1.0f + expf(-acc));
    y[(size_t(b) * T + t) * C + c] = __float2bfloat16_rn(s);
#pragma unroll
    for (int j = 0; j < KW - 1; ++j) win[j] = win[j + 1];
  }
  if (t1 == T) {  // the chunk that ends the sequence writes the new state (may alias conv_in: own column only,
                  // and every read of the old state by this column's other chunks ... see launcher note)
    for (int j = 0; j < SL; ++j) {
      const int ti = T - SL + j;
      const __nv_bfloat16 val = ti >= 0 ? xb[size_t(ti) * C + c] : sb[size_t(ti + SL) * C + c];
      conv_out[(size_t(b) * SL + j) * C + c] = val;
    }
  }
}

int run_gdn_conv(Call& c) {
  Tensor x, w, ci, y, co;
  Q35_TRY(c.get("x", M(Q35_BF16), &x));
  Q35_TRY(c.get("conv_w", M(Q35_BF16), &w));
  Q35_TRY(c.get("conv_in", M(Q35_BF16), &ci));
  Q35_TRY(c.get("y", M(Q35_BF16), &y));
  Q35_TRY(c.get("conv_out", M(Q35_BF16), &co));
  Q35_REQUIRE(x.nd == 3 && w.nd >= 2, Q35_ERR_SHAPE, "gdn.conv: x [B, T, C], conv_w [C, KW]");
  const int64_t B = x.s[0], T = x.s[1], C = x.s[2];
  const int64_t KW = w.s[w.nd - 1];
  Q35_REQUIRE(w.numel() == C * KW && KW >= 1 && KW <= 8, Q35_ERR_SHAPE, "gdn.conv: conv_w must be [C, KW<=8]");
  Q35_REQUIRE(ci.numel() == B * (KW - 1) * C && co.numel() == ci.numel(), Q35_ERR_SHAPE,
              "gdn.conv: conv state must be [B, KW-1, C]");
  Q35_REQUIRE(y.numel() == x.numel(), Q35_ERR_SHAPE, "gdn.conv: y shape");
  c.ws_need = 0;
  if (c.dry || x.numel() == 0) return 0;
  // In-place state (conv_out == conv_in) is only safe when one chunk covers the sequence: otherwise a later chunk
  // could still be reading old state rows.  Chunks only read state rows when t0 < KW - 1, i.e. the first chunk; the
  // state is written by the last chunk.  With more than one chunk and aliasing we fall back to a single chunk.
  int t_chunk = 64;
  if (ci.p == co.p || T <= 64) t_chunk = int(T);
  const dim3 grid{unsigned((C + 127) / 128), unsigned((T + t_chunk - 1) / t_chunk), unsigned(B)};
#define Q35_CONV_CASE(kw)                                                                                   \
  case kw:                                                                                                  \
    gdn_conv_kernel<kw><<<grid, 128, 0, c.stream>>>(x.as<__nv_bfloat16>(), w.as<__nv_bfloat16>(),           \
                                                    ci.as<__nv_bfloat16>(), y.as<__nv_bfloat16>(),          \
                                                    co.as<__nv_bfloat16>(), int(T), int(C), t_chunk);       \
    break;
  switch (int(KW)) {
    Q35_CONV_CASE(1) Q35_CONV_CASE(2) Q35_CONV_CASE(3) Q35_CONV_CASE(4)
    Q35_CONV_CASE(5) Q35_CONV_CASE(6) Q35_CONV_CASE(7) Q35_CONV_CASE(8)
  }
#undef Q35_CONV_CASE
  Q35_CUDA_LAUNCH_CHECK("gdn.conv");
  return 0;
}

}  // namespace q35
