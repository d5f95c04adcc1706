// Gated delta net, prefill: chunked (WY) evaluation of the delta rule, chunk = 64 tokens.
//
// Reference: gdn_stable_chunk and its driver (models/qwen35_35b_a3b/sgl/python/sgl_kernel_axera/attention/gdn.py:
// 1122-1212, 1654-1705); golden = the token-by-token loop of gdn_reference
// (models/qwen35_35b_a3b/sgl/tests/test_gdn_attn.py:272-296).  Per value head, with G the running sum of the log
// decay g inside the chunk and S0 the state entering the chunk:
//   A[j,l] = beta_j e^{G_j-G_l} (k_j.k_l)  (l < j),      T = (I + A)^-1                       (fp32 substitution)
//   W  = T (beta e^G K),   U~ = T (beta V),   M[i,j] = e^{G_i-G_j} (q_i.k_j)  (j <= i),   Kd = e^{G_C-G} K
//   U  = U~ - W S0,        O = e^G (Q S0) + M U,        S_C = e^{G_C} S0 + Kd^T U
// Everything on the first two lines is independent of the state: `gdn_chunk_prep_kernel` computes it for all chunks
// and heads at once on the tensor cores (mma.sync bf16, fp32 accumulate).  `gdn_chunk_scan_kernel` then walks the
// chunks in order; the state columns are independent, so each value head is split over 4 CTAs of 32 columns whose
// slice of S stays in registers as mma accumulators for the whole sequence.
#include "abi.h"
#include "common.cuh"

namespace q35 {

constexpr int GC = 64;    // chunk length
constexpr int GDK = 128;  // key / value head dim
constexpr int GSL = 32;   // state columns per scan CTA

__device__ __forceinline__ void cp_async_16_zfill(uint32_t smem_addr, const void* gptr, bool valid) {
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr), "l"(gptr), "r"(n));
}
// byte offset of 16-byte chunk `ch` of row `row` in a swizzled row-major tile
__device__ __forceinline__ uint32_t sw256(int row, int ch) { return row * 256 + ((ch ^ (row & 7)) << 4); }  // 128 bf16
__device__ __forceinline__ uint32_t sw128(int row, int ch) { return row * 128 + ((ch ^ (row & 7)) << 4); }  // 64 bf16
__device__ __forceinline__ uint32_t sw64(int row, int ch) { return row * 64 + ((ch ^ ((row >> 1) & 3)) << 4); }  // 32 bf16

struct GdnChunkArgs {
  const __nv_bfloat16 *q, *k, *v, *beta;
  const float* g;
  const float* state_in;
  float* state_out;
  __nv_bfloat16* o;
  int B, T, NK, NV, n_chunks, Tpad;
  // workspace
  __nv_bfloat16 *W, *Ut, *Kd, *M;  // [BV, Tpad, 128] x3, [BV, n_chunks, 64, 64]
  float *EG, *EGL;                 // [BV, Tpad], [BV, n_chunks]
};

// ---------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) gdn_chunk_prep_kernel(const GdnChunkArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int r = lane >> 2, c = lane & 3;
  const int chunk = blockIdx.x, bv = blockIdx.y;
  const int b = bv / a.NV, vh = bv % a.NV, kh = vh / (a.NV / a.NK);
  const int t0 = chunk * GC;
  uint8_t* sK = smem;                 // [64][128] bf16, swizzled
  uint8_t* sQ = smem + 16384;         // Q, later K' = beta e^G K
  uint8_t* sV = smem + 32768;         // V, later V' = beta V
  uint8_t* sT = smem + 49152;         // [64][64] bf16, swizzled
  float* sA = reinterpret_cast<float*>(smem + 57344);  // [64][65]
  float* sg = sA + 64 * 65;           // G (cumulative log decay)
  float* sb = sg + 64;                // beta
  const uint32_t uK = smem_u32(sK), uQ = smem_u32(sQ), uV = smem_u32(sV), uT = smem_u32(sT);

  for (int idx = tid; idx < 64 * 16; idx += 128) {
    const int row = idx >> 4, ch = idx & 15;
    const int t = t0 + row;
    uint4 kv = make_uint4(0, 0, 0, 0), qv = kv, vv = kv;
    if (t < a.T) {
      kv = *reinterpret_cast<const uint4*>(a.k + ((size_t(b) * a.T + t) * a.NK + kh) * GDK + ch * 8);
      qv = *reinterpret_cast<const uint4*>(a.q + ((size_t(b) * a.T + t) * a.NK + kh) * GDK + ch * 8);
      vv = *reinterpret_cast<const uint4*>(a.v + ((size_t(b) * a.T + t) * a.NV + vh) * GDK + ch * 8);
    }
    *reinterpret_cast<uint4*>(sK + sw256(row, ch)) = kv;
    *reinterpret_cast<uint4*>(sQ + sw256(row, ch)) = qv;
    *reinterpret_cast<uint4*>(sV + sw256(row, ch)) = vv;
  }
  if (warp == 0) {  // inclusive scan of g over the chunk, two tokens per lane
    const int ta = t0 + 2 * lane, tb = ta + 1;
    const float ga = ta < a.T ? a.g[(size_t(b) * a.T + ta) * a.NV + vh] : 0.f;
    const float gb = tb < a.T ? a.g[(size_t(b) * a.T + tb) * a.NV + vh] : 0.f;
    float s = ga + gb;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float nbr = __shfl_up_sync(0xffffffffu, s, o);
      if (lane >= o) s += nbr;
    }
    sg[2 * lane] = s - gb;
    sg[2 * lane + 1] = s;
    sb[2 * lane] = ta < a.T ? __bfloat162float(a.beta[(size_t(b) * a.T + ta) * a.NV + vh]) : 0.f;
    sb[2 * lane + 1] = tb < a.T ? __bfloat162float(a.beta[(size_t(b) * a.T + tb) * a.NV + vh]) : 0.f;
  }
  __syncthreads();

  // KK = K K^T and QK = Q K^T for this warp's 16 rows
  float kk[8][4], qk[8][4];
#pragma unroll
  for (int nt = 0; nt < 8; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) kk[nt][i] = qk[nt][i] = 0.f;
  {
    const int arow = warp * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      uint32_t ak[4], aq[4];
      ldmatrix_x4(uK + sw256(arow, 2 * ks + (lane >> 4)), ak[0], ak[1], ak[2], ak[3]);
      ldmatrix_x4(uQ + sw256(arow, 2 * ks + (lane >> 4)), aq[0], aq[1], aq[2], aq[3]);
#pragma unroll
      for (int np = 0; np < 4; ++np) {  // pairs of 8-key column tiles
        const int brow = np * 16 + (lane & 7) + ((lane >> 4) << 3);
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(uK + sw256(brow, 2 * ks + ((lane >> 3) & 1)), b0, b1, b2, b3);
        mma_bf16_16816(kk[2 * np], ak[0], ak[1], ak[2], ak[3], b0, b1);
        mma_bf16_16816(kk[2 * np + 1], ak[0], ak[1], ak[2], ak[3], b2, b3);
        mma_bf16_16816(qk[2 * np], aq[0], aq[1], aq[2], aq[3], b0, b1);
        mma_bf16_16816(qk[2 * np + 1], aq[0], aq[1], aq[2], aq[3], b2, b3);
      }
    }
  }
  __nv_bfloat16* Mg = a.M + (size_t(bv) * a.n_chunks + chunk) * GC * GC;
#pragma unroll
  for (int nt = 0; nt < 8; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int row = warp * 16 + r + ((i >> 1) << 3), col = nt * 8 + 2 * c + (i & 1);
      const float dec = __expf(sg[row] - sg[col]);
      sA[row * 65 + col] = col < row ? sb[row] * dec * kk[nt][i] : 0.f;
      Mg[row * GC + col] = __float2bfloat16_rn(col <= row ? dec * qk[nt][i] : 0.f);
    }
  __syncthreads();

  if (tid < 64) {
    // column `tid` of T = (I + A)^-1 by forward substitution, kept in registers
    float t[64];
#pragma unroll
    for (int j = 0; j < 64; ++j) {
      float acc = (j == tid) ? 1.f : 0.f;
#pragma unroll
      for (int l = 0; l < j; ++l) acc = fmaf(-sA[j * 65 + l], t[l], acc);
      t[j] = acc;
    }
#pragma unroll
    for (int j = 0; j < 64; ++j)
      *reinterpret_cast<__nv_bfloat16*>(sT + sw128(j, tid >> 3) + (tid & 7) * 2) = __float2bfloat16_rn(t[j]);
  } else {
    // meanwhile: K' = beta e^G K (into the Q tile), V' = beta V (in place), Kd = e^{G_C - G} K and e^G to global
    const int u = tid - 64;
    const float g_last = sg[63];
    for (int idx = u; idx < 64 * 16; idx += 64) {
      const int row = idx >> 4, ch = idx & 15;
      const float bt = sb[row], eg = __expf(sg[row]), ed = __expf(g_last - sg[row]);
      const uint4 kv = *reinterpret_cast<const uint4*>(sK + sw256(row, ch));
      const uint4 vv = *reinterpret_cast<const uint4*>(sV + sw256(row, ch));
      const uint32_t kw[4] = {kv.x, kv.y, kv.z, kv.w}, vw[4] = {vv.x, vv.y, vv.z, vv.w};
      uint32_t k1[4], v1[4], kd[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float klo = bf16lo(kw[i]), khi = bf16hi(kw[i]);
        k1[i] = pack_bf16(bt * eg * klo, bt * eg * khi);
        kd[i] = pack_bf16(ed * klo, ed * khi);
        v1[i] = pack_bf16(bt * bf16lo(vw[i]), bt * bf16hi(vw[i]));
      }
      *reinterpret_cast<uint4*>(sQ + sw256(row, ch)) = make_uint4(k1[0], k1[1], k1[2], k1[3]);
      *reinterpret_cast<uint4*>(sV + sw256(row, ch)) = make_uint4(v1[0], v1[1], v1[2], v1[3]);
      *reinterpret_cast<uint4*>(a.Kd + (size_t(bv) * a.Tpad + t0 + row) * GDK + ch * 8) =
          make_uint4(kd[0], kd[1], kd[2], kd[3]);
    }
    a.EG[size_t(bv) * a.Tpad + t0 + u] = __expf(sg[u]);
    if (u == 0) a.EGL[size_t(bv) * a.n_chunks + chunk] = __expf(g_last);
  }
  __syncthreads();

  // W = T K', U~ = T V' for this warp's 16 rows
#pragma unroll 1
  for (int which = 0; which < 2; ++which) {
    const uint32_t uB = which ? uV : uQ;
    float acc[16][4];
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
    const int arow = warp * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      uint32_t a0, a1, a2, a3;
      ldmatrix_x4(uT + sw128(arow, 2 * ks + (lane >> 4)), a0, a1, a2, a3);
      const int brow = ks * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
#pragma unroll
      for (int np = 0; np < 8; ++np) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(uB + sw256(brow, 2 * np + (lane >> 4)), b0, b1, b2, b3);
        mma_bf16_16816(acc[2 * np], a0, a1, a2, a3, b0, b1);
        mma_bf16_16816(acc[2 * np + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    __nv_bfloat16* dst = (which ? a.Ut : a.W) + (size_t(bv) * a.Tpad + t0) * GDK;
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) {
      const int row = warp * 16 + r, col = nt * 8 + 2 * c;
      *reinterpret_cast<uint32_t*>(dst + size_t(row) * GDK + col) = pack_bf16(acc[nt][0], acc[nt][1]);
      *reinterpret_cast<uint32_t*>(dst + size_t(row + 8) * GDK + col) = pack_bf16(acc[nt][2], acc[nt][3]);
    }
  }
}

constexpr int GDN_PREP_SMEM = 57344 + (64 * 65 + 128) * 4;

// ---------------------------------------------------------------------------------------------------------------
// sequential pass: one CTA per (value head, 32-column slice of the state)
constexpr int SCAN_BUF = 16384 * 3 + 8192 + 4096 + 512;  // W, Q, Kd tiles, M, U~ slice, e^G (+ pad)
constexpr int GDN_SCAN_SMEM = 2 * SCAN_BUF + 8192 + 4096;

__global__ void __launch_bounds__(128, 1) gdn_chunk_scan_kernel(const GdnChunkArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int r = lane >> 2, c = lane & 3;
  const int slice = blockIdx.x, bv = blockIdx.y;
  const int b = bv / a.NV, vh = bv % a.NV, kh = vh / (a.NV / a.NK);
  uint8_t* sS = smem + 2 * SCAN_BUF;  // [128][32] bf16 state slice
  uint8_t* sU = sS + 8192;            // [64][32] bf16
  const uint32_t uS = smem_u32(sS), uU = smem_u32(sU);

  // state slice as accumulators: warp owns rows 32 w .. 32 w + 31 (2 m-tiles) x 32 columns (4 n-tiles)
  float S[2][4][4];
  {
    const float* sin = a.state_in + size_t(bv) * GDK * GDK + slice * GSL;
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int row = warp * 32 + mt * 16 + r + ((i >> 1) << 3), col = nt * 8 + 2 * c + (i & 1);
          S[mt][nt][i] = sin[size_t(row) * GDK + col];
        }
  }

  auto issue = [&](int ch) {
    if (ch < a.n_chunks) {
      const uint32_t base = smem_u32(smem) + (ch & 1) * SCAN_BUF;
      const int t0 = ch * GC;
      const __nv_bfloat16* Wg = a.W + (size_t(bv) * a.Tpad + t0) * GDK;
      const __nv_bfloat16* Kg = a.Kd + (size_t(bv) * a.Tpad + t0) * GDK;
      const __nv_bfloat16* Ug = a.Ut + (size_t(bv) * a.Tpad + t0) * GDK + slice * GSL;
      const __nv_bfloat16* Mg = a.M + (size_t(bv) * a.n_chunks + ch) * GC * GC;
      for (int idx = tid; idx < 64 * 16; idx += 128) {
        const int row = idx >> 4, cc = idx & 15;
        cp_async_16(base + sw256(row, cc), Wg + size_t(row) * GDK + cc * 8);
        const int t = t0 + row;
        cp_async_16_zfill(base + 16384 + sw256(row, cc),
                          a.q + ((size_t(b) * a.T + min(t, a.T - 1)) * a.NK + kh) * GDK + cc * 8, t < a.T);
        cp_async_16(base + 32768 + sw256(row, cc), Kg + size_t(row) * GDK + cc * 8);
      }
      for (int idx = tid; idx < 64 * 8; idx += 128) {
        const int row = idx >> 3, cc = idx & 7;
        cp_async_16(base + 49152 + sw128(row, cc), Mg + size_t(row) * GC + cc * 8);
      }
      for (int idx = tid; idx < 64 * 4; idx += 128) {
        const int row = idx >> 2, cc = idx & 3;
        cp_async_16(base + 57344 + sw64(row, cc), Ug + size_t(row) * GDK + cc * 8);
      }
      if (tid < 16) cp_async_16(base + 61440 + tid * 16, a.EG + size_t(bv) * a.Tpad + t0 + tid * 4);
    }
    cp_async_commit();
  };

  issue(0);
  for (int ch = 0; ch < a.n_chunks; ++ch) {
    issue(ch + 1);
    // the state as the bf16 B operand of this chunk
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        const int row = warp * 32 + mt * 16 + r;
        *reinterpret_cast<uint32_t*>(sS + sw64(row, nt) + c * 4) = pack_bf16(S[mt][nt][0], S[mt][nt][1]);
        *reinterpret_cast<uint32_t*>(sS + sw64(row + 8, nt) + c * 4) = pack_bf16(S[mt][nt][2], S[mt][nt][3]);
      }
    cp_async_wait<1>();
    __syncthreads();
    const uint8_t* buf = smem + (ch & 1) * SCAN_BUF;
    const uint32_t uW = smem_u32(buf), uQ = uW + 16384, uKd = uW + 32768, uM = uW + 49152;
    const uint8_t* sUt = buf + 57344;
    const float* sEG = reinterpret_cast<const float*>(buf + 61440);
    const float egl = a.EGL[size_t(bv) * a.n_chunks + ch];

    // P = W S0, R = Q S0 for token rows 16 w .. 16 w + 15
    float P[4][4], R[4][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) P[nt][i] = R[nt][i] = 0.f;
    {
      const int arow = warp * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        uint32_t w0, w1, w2, w3, q0, q1, q2, q3;
        ldmatrix_x4(uW + sw256(arow, 2 * ks + (lane >> 4)), w0, w1, w2, w3);
        ldmatrix_x4(uQ + sw256(arow, 2 * ks + (lane >> 4)), q0, q1, q2, q3);
        const int brow = ks * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
#pragma unroll
        for (int np = 0; np < 2; ++np) {
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4_trans(uS + sw64(brow, 2 * np + (lane >> 4)), b0, b1, b2, b3);
          mma_bf16_16816(P[2 * np], w0, w1, w2, w3, b0, b1);
          mma_bf16_16816(P[2 * np + 1], w0, w1, w2, w3, b2, b3);
          mma_bf16_16816(R[2 * np], q0, q1, q2, q3, b0, b1);
          mma_bf16_16816(R[2 * np + 1], q0, q1, q2, q3, b2, b3);
        }
      }
    }
    // U = U~ - P  -> bf16 tile; O starts as e^G * R
    float O[4][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      const int row = warp * 16 + r;
      const uint32_t u0 = *reinterpret_cast<const uint32_t*>(sUt + sw64(row, nt) + c * 4);
      const uint32_t u1 = *reinterpret_cast<const uint32_t*>(sUt + sw64(row + 8, nt) + c * 4);
      *reinterpret_cast<uint32_t*>(sU + sw64(row, nt) + c * 4) = pack_bf16(bf16lo(u0) - P[nt][0], bf16hi(u0) - P[nt][1]);
      *reinterpret_cast<uint32_t*>(sU + sw64(row + 8, nt) + c * 4) =
          pack_bf16(bf16lo(u1) - P[nt][2], bf16hi(u1) - P[nt][3]);
      const float e0 = sEG[row], e1 = sEG[row + 8];
      O[nt][0] = e0 * R[nt][0]; O[nt][1] = e0 * R[nt][1]; O[nt][2] = e1 * R[nt][2]; O[nt][3] = e1 * R[nt][3];
    }
    __syncthreads();
    // O += M U
    {
      const int arow = warp * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        uint32_t a0, a1, a2, a3;
        ldmatrix_x4(uM + sw128(arow, 2 * ks + (lane >> 4)), a0, a1, a2, a3);
        const int brow = ks * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
#pragma unroll
        for (int np = 0; np < 2; ++np) {
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4_trans(uU + sw64(brow, 2 * np + (lane >> 4)), b0, b1, b2, b3);
          mma_bf16_16816(O[2 * np], a0, a1, a2, a3, b0, b1);
          mma_bf16_16816(O[2 * np + 1], a0, a1, a2, a3, b2, b3);
        }
      }
    }
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      const int t = ch * GC + warp * 16 + r;
      const int col = slice * GSL + nt * 8 + 2 * c;
      if (t < a.T)
        *reinterpret_cast<uint32_t*>(a.o + ((size_t(b) * a.T + t) * a.NV + vh) * GDK + col) = pack_bf16(O[nt][0], O[nt][1]);
      if (t + 8 < a.T)
        *reinterpret_cast<uint32_t*>(a.o + ((size_t(b) * a.T + t + 8) * a.NV + vh) * GDK + col) =
            pack_bf16(O[nt][2], O[nt][3]);
    }
    // S = e^{G_C} S + Kd^T U   (rows of S = key channels 32 w .. 32 w + 31)
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) S[mt][nt][i] *= egl;
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      const int brow = ks * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
      uint32_t bu[2][4];
#pragma unroll
      for (int np = 0; np < 2; ++np)
        ldmatrix_x4_trans(uU + sw64(brow, 2 * np + (lane >> 4)), bu[np][0], bu[np][1], bu[np][2], bu[np][3]);
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        // A = Kd^T: stored [token][channel]; transposed 8x8 blocks give (channel, token pairs)
        const int krow = ks * 16 + (lane & 7) + ((lane >> 4) << 3);
        const int kch = (warp * 32 + mt * 16) / 8 + ((lane >> 3) & 1);
        uint32_t a0, a1, a2, a3;
        ldmatrix_x4_trans(uKd + sw256(krow, kch), a0, a1, a2, a3);
#pragma unroll
        for (int np = 0; np < 2; ++np) {
          mma_bf16_16816(S[mt][2 * np], a0, a1, a2, a3, bu[np][0], bu[np][1]);
          mma_bf16_16816(S[mt][2 * np + 1], a0, a1, a2, a3, bu[np][2], bu[np][3]);
        }
      }
    }
    __syncthreads();  // sS / sU and this chunk's buffer may be overwritten from here on
  }
  cp_async_wait<0>();
  float* sout = a.state_out + size_t(bv) * GDK * GDK + slice * GSL;
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int row = warp * 32 + mt * 16 + r + ((i >> 1) << 3), col = nt * 8 + 2 * c + (i & 1);
        sout[size_t(row) * GDK + col] = S[mt][nt][i];
      }
}

// gdn.chunk_prefill: q, k [B, T, NK, 128] bf16 (L2-normalised, q scaled), v [B, T, NV, 128] bf16, g [B, T, NV] f32,
// beta [B, T, NV] bf16, state_in [B, NV, 128, 128] f32 -> o [B, T, NV, 128] bf16, state_out (may alias state_in)
int run_gdn_chunk_prefill(Call& c) {
  Tensor q, k, v, g, beta, sin, o, sout, ws;
  Q35_TRY(c.get("q", M(Q35_BF16), &q));
  Q35_TRY(c.get("k", M(Q35_BF16), &k));
  Q35_TRY(c.get("v", M(Q35_BF16), &v));
  Q35_TRY(c.get("g", M(Q35_F32), &g));
  Q35_TRY(c.get("beta", M(Q35_BF16), &beta));
  Q35_TRY(c.get("state_in", M(Q35_F32), &sin));
  Q35_TRY(c.get("o", M(Q35_BF16), &o));
  Q35_TRY(c.get("state_out", M(Q35_F32), &sout));
  Q35_REQUIRE(q.nd == 4 && k.nd == 4 && v.nd == 4, Q35_ERR_SHAPE, "gdn.chunk_prefill: q, k, v must be [B, T, heads, 128]");
  const int64_t B = q.s[0], T = q.s[1], NK = q.s[2], NV = v.s[2];
  Q35_REQUIRE(q.s[3] == GDK && v.s[3] == GDK, Q35_ERR_UNSUPPORTED, "gdn.chunk_prefill: head dims must be 128");
  Q35_REQUIRE(k.numel() == q.numel() && v.s[0] == B && v.s[1] == T && NK > 0 && NV % NK == 0, Q35_ERR_SHAPE,
              "gdn.chunk_prefill: head shapes");
  Q35_REQUIRE(g.numel() == B * T * NV && beta.numel() == B * T * NV, Q35_ERR_SHAPE, "gdn.chunk_prefill: g / beta [B, T, NV]");
  Q35_REQUIRE(sin.numel() == B * NV * GDK * GDK && sout.numel() == sin.numel() && o.numel() == v.numel(), Q35_ERR_SHAPE,
              "gdn.chunk_prefill: state [B, NV, 128, 128], o like v");
  const int64_t nch = (T + GC - 1) / GC, Tpad = nch * GC, BV = B * NV;
  int64_t off = 0;
  auto take = [&](int64_t bytes) { const int64_t o2 = off; off = (off + bytes + 255) / 256 * 256; return o2; };
  const int64_t oW = take(BV * Tpad * GDK * 2), oU = take(BV * Tpad * GDK * 2), oK = take(BV * Tpad * GDK * 2),
                oM = take(BV * nch * GC * GC * 2), oE = take(BV * Tpad * 4), oL = take(BV * nch * 4);
  Q35_TRY(c.workspace(off, &ws));
  if (c.dry || BV == 0) return 0;
  if (T == 0) {
    if (sin.p != sout.p) cudaMemcpyAsync(sout.p, sin.p, sin.bytes, cudaMemcpyDeviceToDevice, c.stream);
    return 0;
  }
  Q35_REQUIRE(aligned16(q.p) && aligned16(k.p) && aligned16(v.p) && aligned16(o.p), Q35_ERR_ALIGN,
              "gdn.chunk_prefill: pointers must be 16-byte aligned");
  GdnChunkArgs a{};
  a.q = q.as<__nv_bfloat16>(); a.k = k.as<__nv_bfloat16>(); a.v = v.as<__nv_bfloat16>();
  a.beta = beta.as<__nv_bfloat16>(); a.g = g.as<float>();
  a.state_in = sin.as<float>(); a.state_out = sout.as<float>(); a.o = o.as<__nv_bfloat16>();
  a.B = int(B); a.T = int(T); a.NK = int(NK); a.NV = int(NV); a.n_chunks = int(nch); a.Tpad = int(Tpad);
  uint8_t* w = ws.as<uint8_t>();
  a.W = reinterpret_cast<__nv_bfloat16*>(w + oW); a.Ut = reinterpret_cast<__nv_bfloat16*>(w + oU);
  a.Kd = reinterpret_cast<__nv_bfloat16*>(w + oK); a.M = reinterpret_cast<__nv_bfloat16*>(w + oM);
  a.EG = reinterpret_cast<float*>(w + oE); a.EGL = reinterpret_cast<float*>(w + oL);
  Q35_TRY(ensure_dynamic_smem(reinterpret_cast<const void*>(gdn_chunk_prep_kernel), GDN_PREP_SMEM));
  Q35_TRY(ensure_dynamic_smem(reinterpret_cast<const void*>(gdn_chunk_scan_kernel), GDN_SCAN_SMEM));
  gdn_chunk_prep_kernel<<<dim3{unsigned(nch), unsigned(BV), 1u}, 128, GDN_PREP_SMEM, c.stream>>>(a);
  Q35_CUDA_LAUNCH_CHECK("gdn chunk prep");
  gdn_chunk_scan_kernel<<<dim3{unsigned(GDK / GSL), unsigned(BV), 1u}, 128, GDN_SCAN_SMEM, c.stream>>>(a);
  Q35_CUDA_LAUNCH_CHECK("gdn chunk scan");
  return 0;
}

}  // namespace q35
