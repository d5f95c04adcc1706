// Paged flash-attention decode (one query token per sequence) over a page-table KV cache.
//
// Interface of the reference's sgl line: paged_kv_cache [pages, 2, P, HKV, D], indptr [B+1], indices, last_page_len,
// valid_kv_len = (n_pages - 1) * P + last_page_len
// (models/qwen35_35b_a3b/sgl/python/sgl_kernel_axera/attention/flash_attn.py:1421-1596, 1991-2085, 2354-2358);
// golden: models/qwen35_35b_a3b/sgl/tests/test_qwen35_runtime.py:57-93.  The reference splits the KV blocks of one
// request over its 4 cores and merges [m, l, o] partials (models/qwen35_2b/whole/src/q35_layer_mc.py:308-379); here
// the same split-KV scheme is applied to a whole batch.
//
// Bound: HBM (K and V are read once; 8 query heads share each KV head, so ~8 flop per byte).
// Work = all 64-key tiles of all (sequence, KV head) segments laid end to end; it is cut into equal contiguous
// ranges, one per CTA (one CTA per SM), so every SM streams the same number of bytes whatever the mix of sequence
// lengths.  Inside a CTA each of the 4 warps owns 16 of a tile's 64 keys and runs its own 3-stage cp.async ring
// (16-byte chunks, XOR-swizzled rows), with no block-wide barrier in the loop.  Scores are computed transposed
// (S^T = K Q^T: 16 keys x 8 heads per mma) so the 8 query heads of a KV head fill the n = 8 side exactly and the
// output accumulator O^T [D x 8 heads] costs 64 registers instead of 128.
#include <mutex>
#include "abi.h"
#include "common.cuh"

namespace q35 {

constexpr int AT_TILE = 64;      // keys per tile
constexpr int AT_WKEYS = 16;     // keys per warp per tile
constexpr int AT_GMAX = 8;       // query heads per KV head handled by one mma column block
constexpr float LOG2E = 1.4426950408889634f;

struct AttnPlan {     // header of the workspace, written by the plan kernel
  int total_tiles;    // W
  int tiles_per_cta;  // q
  int pad[62];
};

struct AttnArgs {
  const void* q;        // [B, HQ, D] bf16
  const void* cache;    // [pages, 2, P, HKV, D]
  const int* indptr;
  const int* indices;
  const int* last_page_len;
  const float* sm_scale;   // optional [1]
  const float* kv_scale;   // optional [2, HKV] (FP8 cache)
  const __nv_bfloat16* row_scale;  // int8 cache: [pages, 2, P, HKV] one scale per cached row and head
  const __nv_bfloat16* k_new;  // optional [B, HKV, D]
  const __nv_bfloat16* v_new;
  __nv_bfloat16* out;   // [B, HQ, D]
  // optional: the merged but UNNORMALISED result per (sequence, query head) instead of `out`, for a merge across
  // devices that each hold a part of the keys: maximum (log2 domain), sum of weights, weighted values
  float* lse_m; float* lse_l; float* lse_o;   // [B, HQ], [B, HQ], [B, HQ, D] -- or one packed [B, HQ, D + 2] block
  int lse_os, lse_ms;                         // floats between rows of lse_o, between entries of lse_m / lse_l
  int B, HQ, HKV, G, P, num_pages, n_indices, n_cta;
  int wpc;              // warps per CTA of the decode kernel = partial slots per (segment, CTA)
  // workspace
  AttnPlan* plan;
  int* seg_start;   // [B * HKV + 1]
  int* ctx;         // [B]
  float* part_ml;   // [slots][2][8]
  float* part_o;    // [slots][8][D]
  int* status;
};

// one CTA: context lengths, tiles per segment, exclusive prefix in (b, kvh) order
__global__ void __launch_bounds__(1024) attn_plan_kernel(AttnArgs a) {
  pdl_wait();
  pdl_launch();
  __shared__ int s_part[1024];
  const int tid = threadIdx.x;
  const int per = (a.B + 1023) / 1024;
  const int b0 = tid * per, b1 = min(a.B, b0 + per);
  int local = 0;
  for (int b = b0; b < b1; ++b) {
    const int np = a.indptr[b + 1] - a.indptr[b];
    int ctx = np > 0 ? (np - 1) * a.P + a.last_page_len[b] : 0;
    if (np < 0 || ctx < 0 || a.indptr[b + 1] > a.n_indices || a.last_page_len[b] > a.P) {
      atomicOr(a.status, DS_BAD_PAGE);
      ctx = 0;
    }
    a.ctx[b] = ctx;
    local += (ctx + AT_TILE - 1) / AT_TILE;
  }
  s_part[tid] = local;
  __syncthreads();
  // inclusive scan (Hillis-Steele) over 1024 partials
  for (int o = 1; o < 1024; o <<= 1) {
    const int v = tid >= o ? s_part[tid - o] : 0;
    __syncthreads();
    s_part[tid] += v;
    __syncthreads();
  }
  int run = s_part[tid] - local;  // exclusive prefix of tiles (per KV head) before b0
  for (int b = b0; b < b1; ++b) {
    const int nt = (a.ctx[b] + AT_TILE - 1) / AT_TILE;
    for (int h = 0; h < a.HKV; ++h) a.seg_start[b * a.HKV + h] = run * a.HKV + h * nt;
    run += nt;
  }
  if (tid == 1023) {
    const int W = s_part[1023] * a.HKV;
    a.seg_start[a.B * a.HKV] = W;
    a.plan->total_tiles = W;
    a.plan->tiles_per_cta = max(1, (W + a.n_cta - 1) / a.n_cta);
  }
}

// KVF: cache element format.  0 = bf16, 1 = FP8 E4M3 (one scale per head or the constant 1 / 8), 2 = int8 with a bf16
// scale per cached row and head (kv_quant_row, models/qwen38_27b/decode/q35_group.py:198-205).  The two one-byte
// formats share the byte-wise fragment paths; they differ in the conversion to f16 and in where the scale enters.
// WARPS: 4, or 8 = two groups of four warps that take alternate tiles of the CTA's range.  One warp per scheduler is
// enough while a tile's bytes take longer to arrive than its dependent chain (load fragments, convert, MMA, softmax,
// MMA) takes to run; with one-byte elements the tile arrives in half the time and the chain becomes the limit, so
// those formats run two warps per scheduler with half the stages each (the same bytes in flight).
template <int D, int KVF, int WARPS>
struct AttnCfg {
  static constexpr bool FP8 = KVF != 0;
  static constexpr int ELT = FP8 ? 1 : 2;
  static constexpr int STAGES = (FP8 && WARPS == 4) ? 6 : 3;    // same bytes in flight in every variant
  static constexpr int ROWB = D * ELT;            // bytes of one key row of one head
  static constexpr int CPR = ROWB / 16;           // 16-byte chunks per row
  static constexpr int KV_BYTES = AT_WKEYS * ROWB;  // K (or V) bytes per warp per stage
  static constexpr int STAGE_BYTES = 2 * KV_BYTES;
  static constexpr int WARP_BYTES = STAGES * STAGE_BYTES;
  static constexpr int SMEM = WARPS * WARP_BYTES;
  static constexpr int LD_PER_LANE = AT_WKEYS * CPR / 32;
};

__device__ __forceinline__ uint32_t cvt_e4m3x2_f16x2(uint32_t two_bytes) {
  uint32_t d;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(d) : "h"((unsigned short)two_bytes));
  return d;
}

// two one-byte FP8 cache elements (bytes I0, I1 of x) as f16x2
template <int I0, int I1>
__device__ __forceinline__ uint32_t cvt_kv(uint32_t x) {
  return cvt_e4m3x2_f16x2(__byte_perm(x, 0, 0x4400 | I0 | (I1 << 4)));
}

// int8 bytes I0, I1 of xs (= x ^ 0x80808080) times their rows' scales, rounded to bf16 -- bf16(int8 * scale), the
// reference's page dequantisation (kv_page, models/qwen38_27b/decode/q35_group.py:208-222), exactly: 0x4B000000 | b is
// the float 2^23 + b, the fused multiply-add against -(2^23 + 128) * s leaves (b - 128) * s, a 15-bit product that
// fp32 holds exactly, and one cvt.rn rounds the pair.
template <int I0, int I1>
__device__ __forceinline__ uint32_t cvt_s8x2_bf16x2(uint32_t xs, float s0, float s1) {
  const float f0 = __uint_as_float(__byte_perm(xs, 0x4B000000u, 0x7540 | I0));
  const float f1 = __uint_as_float(__byte_perm(xs, 0x4B000000u, 0x7540 | I1));
  return pack_bf16(fmaf(f0, s0, -8388736.f * s0), fmaf(f1, s1, -8388736.f * s1));
}

template <int D, int KVF, int WARPS>
__global__ void __launch_bounds__(32 * WARPS, 1) attn_decode_kernel(const AttnArgs a) {
  pdl_wait();
  pdl_launch();
  using C = AttnCfg<D, KVF, WARPS>;
  constexpr int TG = WARPS / 4;  // tiles in flight per CTA: warp group wg takes tiles t_begin + wg, + TG, ...
  constexpr bool FP8 = C::FP8;
  constexpr int AT_STAGES = C::STAGES;
  extern __shared__ __align__(128) uint8_t smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int wk = warp & 3, wg = warp >> 2;  // key quarter of a tile, tile group
  const int r = lane >> 2, c = lane & 3;
  const uint32_t sbase = smem_u32(smem) + warp * C::WARP_BYTES;

  const int W = a.plan->total_tiles, q_per = a.plan->tiles_per_cta;
  const int S = a.B * a.HKV;
  int g = blockIdx.x * q_per;
  const int g_end = min(W, g + q_per);
  if (g >= g_end) return;
  // segment containing tile g: last s with seg_start[s] <= g
  int lo = 0, hi = S;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (a.seg_start[mid] <= g) lo = mid; else hi = mid;
  }
  int s = lo;
  const float scale_log2 = (a.sm_scale ? a.sm_scale[0] : rsqrtf(float(D))) * LOG2E;
  const uint8_t* cache = static_cast<const uint8_t*>(a.cache);
  const size_t row_stride = size_t(a.HKV) * C::ROWB;  // bytes between consecutive keys of a page plane

  while (g < g_end) {
    while (a.seg_start[s + 1] <= g) ++s;  // skip empty segments
    const int b = s / a.HKV, kvh = s % a.HKV;
    const int seg0 = a.seg_start[s];
    const int t_begin = g - seg0;
    const int t_end = min(g_end, a.seg_start[s + 1]) - seg0;
    const int t_first = t_begin + wg;  // this warp group's first tile
    const int ctx = a.ctx[b];
    const int page0 = a.indptr[b];

    // query fragments: B operand of S^T = K Q^T, heads on the n side.  bf16 cache: natural k order.  FP8 cache:
    // f16 fragments in the k order the byte-wise K fragments come out in (4 consecutive channels per lane).
    uint32_t qf[D / 16][2];
    float k_mul = 1.f, v_mul = 1.f;  // FP8 dequantisation factors of this KV head
    {
      const __nv_bfloat16* qp = static_cast<const __nv_bfloat16*>(a.q) + (size_t(b) * a.HQ + kvh * a.G + r) * D;
      const bool hv = r < a.G;
      if constexpr (!FP8) {
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          qf[ks][0] = hv ? *reinterpret_cast<const uint32_t*>(qp + ks * 16 + 2 * c) : 0u;
          qf[ks][1] = hv ? *reinterpret_cast<const uint32_t*>(qp + ks * 16 + 8 + 2 * c) : 0u;
        }
      } else {
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          uint2 raw = make_uint2(0u, 0u);
          if (hv) raw = *reinterpret_cast<const uint2*>(qp + ks * 16 + 4 * c);
          if constexpr (KVF == 2) {  // bf16 MMAs: the query stays bf16
            qf[ks][0] = raw.x;
            qf[ks][1] = raw.y;
          } else {
            qf[ks][0] = pack_f16(bf16lo(raw.x), bf16hi(raw.x));
            qf[ks][1] = pack_f16(bf16lo(raw.y), bf16hi(raw.y));
          }
        }
        k_mul = a.kv_scale ? a.kv_scale[kvh] : 0.125f;
        v_mul = a.kv_scale ? a.kv_scale[a.HKV + kvh] : 0.125f;
      }
    }
    if constexpr (KVF == 2) k_mul = v_mul = 1.f;  // the rows are dequantised with their own scales below
    const float seg_scale = scale_log2 * k_mul;
    // int8 cache: the bf16 row scales this lane's fragments need -- K rows r and r + 8 of the warp's 16 keys, V rows
    // 2c, 2c + 1, 2c + 8, 2c + 9 -- fetched two tiles ahead into registers (a plain load at the point of use would
    // stall a warp that has no other work to hide it).  Rows past the context read as scale 0 (their bytes may be
    // anything, and 0 * scale must not become NaN).
    auto load_scales = [&](int t) -> uint3 {
      uint3 v = make_uint3(0u, 0u, 0u);
      if constexpr (KVF == 2) {
        const int kk = t * AT_TILE + wk * AT_WKEYS;
        if (t < t_end && kk < ctx) {
          const int pl = kk / a.P, ro = kk % a.P, valid = ctx - kk;
          int page = a.indices[page0 + pl];
          if (page < 0 || page >= a.num_pages) page = 0;
          const unsigned short* sp = reinterpret_cast<const unsigned short*>(a.row_scale);
          const size_t k0 = ((size_t(page) * 2 + 0) * a.P + ro) * a.HKV + kvh;
          const size_t v0 = ((size_t(page) * 2 + 1) * a.P + ro) * a.HKV + kvh;
          auto at = [&](size_t base, int row) -> uint32_t { return row < valid ? sp[base + size_t(row) * a.HKV] : 0u; };
          v.x = at(k0, r) | (at(k0, r + 8) << 16);
          v.y = at(v0, 2 * c) | (at(v0, 2 * c + 1) << 16);
          v.z = at(v0, 2 * c + 8) | (at(v0, 2 * c + 9) << 16);
        }
      }
      return v;
    };

    float oacc[D / 16][4];
#pragma unroll
    for (int mt = 0; mt < D / 16; ++mt) oacc[mt][0] = oacc[mt][1] = oacc[mt][2] = oacc[mt][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

    auto issue = [&](int t) {  // t: tile index inside the sequence
      const int kk = t * AT_TILE + wk * AT_WKEYS;
      if (t < t_end && kk < ctx) {
        const int pl = kk / a.P, ro = kk % a.P;
        int page = a.indices[page0 + pl];
        if (page < 0 || page >= a.num_pages) {
          if (lane == 0) atomicOr(a.status, DS_BAD_PAGE);
          page = 0;
        }
        const uint8_t* kb = cache + ((size_t(page) * 2 + 0) * a.P + ro) * row_stride + size_t(kvh) * C::ROWB;
        const uint8_t* vb = cache + ((size_t(page) * 2 + 1) * a.P + ro) * row_stride + size_t(kvh) * C::ROWB;
        const uint32_t st = sbase + (((t - t_first) / TG) % AT_STAGES) * C::STAGE_BYTES;
#pragma unroll
        for (int j = 0; j < C::LD_PER_LANE; ++j) {
          const int ci = lane + 32 * j;
          const int key = ci / C::CPR, ch = ci % C::CPR;
          const uint32_t off = key * C::ROWB + ((ch ^ (key & 7)) << 4);
          cp_async_16(st + off, kb + size_t(key) * row_stride + ch * 16);
          cp_async_16(st + C::KV_BYTES + off, vb + size_t(key) * row_stride + ch * 16);
        }
      }
      cp_async_commit();
    };

#pragma unroll
    for (int p = 0; p < AT_STAGES - 1; ++p) issue(t_first + p * TG);
    uint3 rs_cur = load_scales(t_first), rs_n1 = load_scales(t_first + TG), rs_n2 = make_uint3(0u, 0u, 0u);

    for (int t = t_first; t < t_end; t += TG) {
      issue(t + (AT_STAGES - 1) * TG);
      rs_n2 = load_scales(t + 2 * TG);
      cp_async_wait<AT_STAGES - 1>();
      __syncwarp();
      const int kk = t * AT_TILE + wk * AT_WKEYS;
      if (kk < ctx) {
        const int valid = min(AT_WKEYS, ctx - kk);
        const uint32_t st = sbase + (((t - t_first) / TG) % AT_STAGES) * C::STAGE_BYTES;
        if (valid < AT_WKEYS) {  // rows past the context may hold anything (NaN bits included): clear V
          for (int idx = lane; idx < (AT_WKEYS - valid) * C::CPR; idx += 32) {
            const uint32_t addr = st + C::KV_BYTES + (valid + idx / C::CPR) * C::ROWB + ((idx % C::CPR) << 4);
            asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(addr), "r"(0u));
          }
          __syncwarp();
        }
        float sacc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        {
          const int key = (lane & 7) + (((lane >> 3) & 1) << 3);
          const uint32_t rowa = st + key * C::ROWB;
          if constexpr (!FP8) {
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
              const int ch = 2 * ks + (lane >> 4);
              uint32_t a0, a1, a2, a3;
              ldmatrix_x4(rowa + ((ch ^ (key & 7)) << 4), a0, a1, a2, a3);
              mma_bf16_16816(sacc[ks & 1], a0, a1, a2, a3, qf[ks][0], qf[ks][1]);
            }
          } else {
#pragma unroll
            for (int kp = 0; kp < D / 32; ++kp) {  // 32 channels: two mma over bytes taken as b16 pairs
              const int ch = 2 * kp + (lane >> 4);
              uint32_t r0, r1, r2, r3;
              ldmatrix_x4(rowa + ((ch ^ (key & 7)) << 4), r0, r1, r2, r3);
              if constexpr (KVF == 2) {  // rows r (r0, r2) and r + 8 (r1, r3) of the tile, each with its own scale
                const float s0 = bf16lo(rs_cur.x), s1 = bf16hi(rs_cur.x);
                r0 ^= 0x80808080u; r1 ^= 0x80808080u; r2 ^= 0x80808080u; r3 ^= 0x80808080u;
                mma_bf16_16816(sacc[0], cvt_s8x2_bf16x2<0, 1>(r0, s0, s0), cvt_s8x2_bf16x2<0, 1>(r1, s1, s1),
                               cvt_s8x2_bf16x2<2, 3>(r0, s0, s0), cvt_s8x2_bf16x2<2, 3>(r1, s1, s1), qf[2 * kp][0],
                               qf[2 * kp][1]);
                mma_bf16_16816(sacc[1], cvt_s8x2_bf16x2<0, 1>(r2, s0, s0), cvt_s8x2_bf16x2<0, 1>(r3, s1, s1),
                               cvt_s8x2_bf16x2<2, 3>(r2, s0, s0), cvt_s8x2_bf16x2<2, 3>(r3, s1, s1), qf[2 * kp + 1][0],
                               qf[2 * kp + 1][1]);
              } else {
                mma_f16_16816(sacc[0], cvt_kv<0, 1>(r0), cvt_kv<0, 1>(r1), cvt_kv<2, 3>(r0), cvt_kv<2, 3>(r1),
                              qf[2 * kp][0], qf[2 * kp][1]);
                mma_f16_16816(sacc[1], cvt_kv<0, 1>(r2), cvt_kv<0, 1>(r3), cvt_kv<2, 3>(r2), cvt_kv<2, 3>(r3),
                              qf[2 * kp + 1][0], qf[2 * kp + 1][1]);
              }
            }
          }
        }
        float sc[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int key = r + ((i >> 1) << 3);
          sc[i] = key < valid ? (sacc[0][i] + sacc[1][i]) * seg_scale : -INFINITY;
        }
        float mt2[2] = {fmaxf(sc[0], sc[2]), fmaxf(sc[1], sc[3])};
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
          mt2[0] = fmaxf(mt2[0], __shfl_xor_sync(0xffffffffu, mt2[0], o));
          mt2[1] = fmaxf(mt2[1], __shfl_xor_sync(0xffffffffu, mt2[1], o));
        }
        float alpha[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const float mn = fmaxf(m_run[h], mt2[h]);  // finite: key 0 of the tile is always valid
          alpha[h] = exp2f(m_run[h] - mn);
          m_run[h] = mn;
        }
        const float p0 = exp2f(sc[0] - m_run[0]), p1 = exp2f(sc[1] - m_run[1]);
        const float p2 = exp2f(sc[2] - m_run[0]), p3 = exp2f(sc[3] - m_run[1]);
        l_run[0] = l_run[0] * alpha[0] + p0 + p2;
        l_run[1] = l_run[1] * alpha[1] + p1 + p3;
        if (alpha[0] != 1.f || alpha[1] != 1.f) {
#pragma unroll
          for (int mt = 0; mt < D / 16; ++mt) {
            oacc[mt][0] *= alpha[0]; oacc[mt][1] *= alpha[1];
            oacc[mt][2] *= alpha[0]; oacc[mt][3] *= alpha[1];
          }
        }
        if constexpr (!FP8) {
          // P enters the P V product as TWO bf16 terms (p = hi + lo): a single bf16 P carries 2^-9 of relative error
          // into every output element, which on a short or peaked row is as large as the output's own bf16 rounding
          // step; the golden keeps the softmax in fp32.  The kernel is HBM-bound, the second MMA is free.
          const float h0 = round_bf16(p0), h1 = round_bf16(p1), h2 = round_bf16(p2), h3 = round_bf16(p3);
          const uint32_t pb0 = movmatrix_trans(pack_bf16(h0, h1));
          const uint32_t pb1 = movmatrix_trans(pack_bf16(h2, h3));
          const uint32_t pl0 = movmatrix_trans(pack_bf16(p0 - h0, p1 - h1));
          const uint32_t pl1 = movmatrix_trans(pack_bf16(p2 - h2, p3 - h3));
          const int key = (lane & 7) + ((lane >> 4) << 3);
          const uint32_t rowa = st + C::KV_BYTES + key * C::ROWB;
#pragma unroll
          for (int mt = 0; mt < D / 16; ++mt) {
            const int ch = 2 * mt + ((lane >> 3) & 1);
            uint32_t a0, a1, a2, a3;
            ldmatrix_x4_trans(rowa + ((ch ^ (key & 7)) << 4), a0, a1, a2, a3);
            mma_bf16_16816(oacc[mt], a0, a1, a2, a3, pb0, pb1);
            mma_bf16_16816(oacc[mt], a0, a1, a2, a3, pl0, pl1);
          }
        } else {
          // transposed b16 loads keep byte PAIRS (d, d+1) together: a lane gets {V[2c][2r], V[2c][2r+1], V[2c+1][2r],
          // V[2c+1][2r+1]}; bytes (0,2) / (1,3) are the key pairs of channels 2r / 2r+1.  So mma row r holds channel
          // 16 mt + 2r and mma row r + 8 holds channel 16 mt + 2r + 1 (undone when the partial is written).
          // P: f16 for the FP8 cache; for the int8 cache (bf16 MMAs on the rounded rows) two bf16 terms as in the
          // bf16 path
          uint32_t pb0, pb1, pl0 = 0u, pl1 = 0u;
          if constexpr (KVF == 2) {
            const float h0 = round_bf16(p0), h1 = round_bf16(p1), h2 = round_bf16(p2), h3 = round_bf16(p3);
            pb0 = movmatrix_trans(pack_bf16(h0, h1));
            pb1 = movmatrix_trans(pack_bf16(h2, h3));
            pl0 = movmatrix_trans(pack_bf16(p0 - h0, p1 - h1));
            pl1 = movmatrix_trans(pack_bf16(p2 - h2, p3 - h3));
          } else {
            pb0 = movmatrix_trans(pack_f16(p0, p1));
            pb1 = movmatrix_trans(pack_f16(p2, p3));
          }
          const int key = lane & 15;
          const uint32_t rowa = st + C::KV_BYTES + key * C::ROWB;
#pragma unroll
          for (int mp = 0; mp < D / 32; ++mp) {
            const int ch = 2 * mp + (lane >> 4);
            uint32_t r0, r1, r2, r3;  // (keys 0-7, chunk 2mp) (keys 8-15, 2mp) (keys 0-7, 2mp+1) (keys 8-15, 2mp+1)
            ldmatrix_x4_trans(rowa + ((ch ^ (key & 7)) << 4), r0, r1, r2, r3);
            if constexpr (KVF == 2) {  // bytes (0, 2) / (1, 3): keys 2c, 2c + 1 (r0, r2) and 2c + 8, 2c + 9 (r1, r3)
              const float va = bf16lo(rs_cur.y), vb = bf16hi(rs_cur.y), vc = bf16lo(rs_cur.z), vd = bf16hi(rs_cur.z);
              r0 ^= 0x80808080u; r1 ^= 0x80808080u; r2 ^= 0x80808080u; r3 ^= 0x80808080u;
              const uint32_t a0 = cvt_s8x2_bf16x2<0, 2>(r0, va, vb), a1 = cvt_s8x2_bf16x2<1, 3>(r0, va, vb);
              const uint32_t a2 = cvt_s8x2_bf16x2<0, 2>(r1, vc, vd), a3 = cvt_s8x2_bf16x2<1, 3>(r1, vc, vd);
              mma_bf16_16816(oacc[2 * mp], a0, a1, a2, a3, pb0, pb1);
              mma_bf16_16816(oacc[2 * mp], a0, a1, a2, a3, pl0, pl1);
              const uint32_t b0 = cvt_s8x2_bf16x2<0, 2>(r2, va, vb), b1 = cvt_s8x2_bf16x2<1, 3>(r2, va, vb);
              const uint32_t b2 = cvt_s8x2_bf16x2<0, 2>(r3, vc, vd), b3 = cvt_s8x2_bf16x2<1, 3>(r3, vc, vd);
              mma_bf16_16816(oacc[2 * mp + 1], b0, b1, b2, b3, pb0, pb1);
              mma_bf16_16816(oacc[2 * mp + 1], b0, b1, b2, b3, pl0, pl1);
            } else {
              mma_f16_16816(oacc[2 * mp], cvt_kv<0, 2>(r0), cvt_kv<1, 3>(r0), cvt_kv<0, 2>(r1), cvt_kv<1, 3>(r1), pb0, pb1);
              mma_f16_16816(oacc[2 * mp + 1], cvt_kv<0, 2>(r2), cvt_kv<1, 3>(r2), cvt_kv<0, 2>(r3), cvt_kv<1, 3>(r3), pb0,
                            pb1);
            }
          }
        }
      }
      __syncwarp();
      rs_cur = rs_n1;
      rs_n1 = rs_n2;
    }
    cp_async_wait<0>();

    // partial of this (segment, CTA, warp): slot = (s + cta) * WARPS + warp (a warp group without a tile leaves l = 0)
    {
#pragma unroll
      for (int o = 4; o < 32; o <<= 1) {
        l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], o);
        l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], o);
      }
      const size_t slot = size_t(s + blockIdx.x) * WARPS + warp;
      float* ml = a.part_ml + slot * 16;
      if (r == 0) {
        ml[2 * c] = m_run[0]; ml[2 * c + 1] = m_run[1];
        ml[8 + 2 * c] = l_run[0]; ml[8 + 2 * c + 1] = l_run[1];
      }
      float* po = a.part_o + slot * (AT_GMAX * D);
#pragma unroll
      for (int mt = 0; mt < D / 16; ++mt) {
        const int d0 = FP8 ? mt * 16 + 2 * r : mt * 16 + r;      // channel of mma row r
        const int d1 = FP8 ? mt * 16 + 2 * r + 1 : mt * 16 + r + 8;  // channel of mma row r + 8
        po[(2 * c) * D + d0] = oacc[mt][0] * v_mul;
        po[(2 * c + 1) * D + d0] = oacc[mt][1] * v_mul;
        po[(2 * c) * D + d1] = oacc[mt][2] * v_mul;
        po[(2 * c + 1) * D + d1] = oacc[mt][3] * v_mul;
      }
    }
    g = seg0 + t_end;
  }
}

// out[b, h] = merge of the partials of segment (b, h / G) (+ the current token's own k / v) -> bf16
template <int D>
__global__ void __launch_bounds__(D / 2) attn_merge_kernel(const AttnArgs a) {
  pdl_wait();
  pdl_launch();
  const int bh = blockIdx.x;
  const int b = bh / a.HQ, h = bh % a.HQ;
  const int kvh = h / a.G, gq = h % a.G;
  const int s = b * a.HKV + kvh;
  const int tid = threadIdx.x;  // two channels per thread
  const int q_per = a.plan->tiles_per_cta;
  const int seg0 = a.seg_start[s], seg1 = a.seg_start[s + 1];
  float M = -INFINITY, L = 0.f, o0 = 0.f, o1 = 0.f;
  if (seg1 > seg0) {
    // Two passes so that no load waits for arithmetic on the previous one: first the maximum over the segment's
    // partials, then every partial scaled by exp2(m - M) and added (slots: 4 warps of each CTA that touched it).
    const size_t slot0 = (size_t(s) + seg0 / q_per) * a.wpc;
    const int ns = ((seg1 - 1) / q_per - seg0 / q_per + 1) * a.wpc;
#pragma unroll 4
    for (int j = 0; j < ns; ++j) {
      const float m = a.part_ml[(slot0 + j) * 16 + gq];
      const float l = a.part_ml[(slot0 + j) * 16 + 8 + gq];
      if (l > 0.f) M = fmaxf(M, m);
    }
    if (M != -INFINITY) {
#pragma unroll 4
      for (int j = 0; j < ns; ++j) {
        const float m = a.part_ml[(slot0 + j) * 16 + gq];
        const float l = a.part_ml[(slot0 + j) * 16 + 8 + gq];
        const bool on = l > 0.f && m != -INFINITY;
        // an unused slot may hold anything: it is not read, not multiplied by zero
        const float2 po = on ? *reinterpret_cast<const float2*>(a.part_o + (slot0 + j) * (AT_GMAX * D) + gq * D + 2 * tid)
                             : make_float2(0.f, 0.f);
        const float fb = on ? exp2f(m - M) : 0.f;
        L += on ? l * fb : 0.f;
        o0 += po.x * fb;
        o1 += po.y * fb;
      }
    }
  }
  if (a.k_new) {  // the current token, taken from its own k / v row instead of the cache
    const float scale_log2 = (a.sm_scale ? a.sm_scale[0] : rsqrtf(float(D))) * LOG2E;
    const __nv_bfloat16* qp = static_cast<const __nv_bfloat16*>(a.q) + (size_t(b) * a.HQ + h) * D;
    const __nv_bfloat16* kp = a.k_new + (size_t(b) * a.HKV + kvh) * D;
    const __nv_bfloat16* vp = a.v_new + (size_t(b) * a.HKV + kvh) * D;
    float dot = __bfloat162float(qp[2 * tid]) * __bfloat162float(kp[2 * tid]) +
                __bfloat162float(qp[2 * tid + 1]) * __bfloat162float(kp[2 * tid + 1]);
    __shared__ float s_red[32];
    dot = warp_sum(dot);
    if ((tid & 31) == 0) s_red[tid >> 5] = dot;
    __syncthreads();
    float tot = 0.f;
    for (int i = 0; i < (D / 2 + 31) / 32; ++i) tot += s_red[i];
    const float m = tot * scale_log2;
    const float mn = fmaxf(M, m);
    const float fa = exp2f(M - mn), fb = exp2f(m - mn);
    L = L * fa + fb;
    o0 = o0 * fa + __bfloat162float(vp[2 * tid]) * fb;
    o1 = o1 * fa + __bfloat162float(vp[2 * tid + 1]) * fb;
  }
  if (a.lse_o) {
    const size_t row = size_t(b) * a.HQ + h;
    if (tid == 0) { a.lse_m[row * a.lse_ms] = M; a.lse_l[row * a.lse_ms] = L; }
    *reinterpret_cast<float2*>(a.lse_o + row * a.lse_os + 2 * tid) = make_float2(o0, o1);
    return;
  }
  const float inv = L > 0.f ? 1.f / L : 0.f;
  *reinterpret_cast<uint32_t*>(a.out + (size_t(b) * a.HQ + h) * D + 2 * tid) = pack_bf16(o0 * inv, o1 * inv);
}

// attn.lse_merge: out[b, h] = sum_g o_g 2^(m_g - M) / sum_g l_g 2^(m_g - M), M = max_g m_g: the partial results of G
// devices that each attended to a part of the keys (split by pages inside a KV head), all-gathered and merged -- the
// pair scheme of the reference's multi-core attention (models/qwen35_35b_a3b/sgl/python/sgl_kernel_axera/attention/
// flash_attn.py:2393-2474; models/qwen35_2b/whole/src/q35_layer_mc.py:361-379).  Parts with l = 0 hold nothing.
__global__ void attn_lse_merge_kernel(const float* __restrict__ pm, const float* __restrict__ pl,
                                      const float* __restrict__ po, __nv_bfloat16* __restrict__ out, int G, int BH, int D) {
  const int bh = blockIdx.x;
  float M = -INFINITY;
  for (int g = 0; g < G; ++g)
    if (pl[size_t(g) * BH + bh] > 0.f) M = fmaxf(M, pm[size_t(g) * BH + bh]);
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float L = 0.f, o = 0.f;
    for (int g = 0; g < G; ++g) {
      const float l = pl[size_t(g) * BH + bh];
      if (!(l > 0.f)) continue;
      const float f = exp2f(pm[size_t(g) * BH + bh] - M);
      L += l * f;
      o += po[(size_t(g) * BH + bh) * D + d] * f;
    }
    out[size_t(bh) * D + d] = __float2bfloat16_rn(L > 0.f ? o / L : 0.f);
  }
}

// The same merge straight from the all-gathered messages: packed [R, B, Hq, D + 2] holds rank r's unnormalised result
// (o | m | l per row) for ITS Hq query heads; ranks are ordered KV group major (r = group * S + share), so output head
// h = group * Hq + hl merges the S rows (group * S + g, b, hl).
__global__ void attn_lse_merge_packed_kernel(const float* __restrict__ packed, __nv_bfloat16* __restrict__ out, int S,
                                             int B, int Hq, int HQ, int D) {
  const int b = blockIdx.x / HQ, h = blockIdx.x % HQ, grp = h / Hq, hl = h % Hq;
  const size_t W = size_t(D) + 2, rank_stride = size_t(B) * Hq * W;
  const float* base = packed + size_t(grp) * S * rank_stride + (size_t(b) * Hq + hl) * W;
  float M = -INFINITY;
  for (int g = 0; g < S; ++g)
    if (base[g * rank_stride + D + 1] > 0.f) M = fmaxf(M, base[g * rank_stride + D]);
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float L = 0.f, o = 0.f;
    for (int g = 0; g < S; ++g) {
      const float l = base[g * rank_stride + D + 1];
      if (!(l > 0.f)) continue;
      const float f = exp2f(base[g * rank_stride + D] - M);
      L += l * f;
      o += base[g * rank_stride + d] * f;
    }
    out[(size_t(b) * HQ + h) * D + d] = __float2bfloat16_rn(L > 0.f ? o / L : 0.f);
  }
}

int run_attn_lse_merge(Call& c) {
  Tensor pm, pl, po, out, pk;
  Q35_TRY(c.get("packed", M(Q35_F32), &pk, false));
  if (pk.present) {
    Q35_TRY(c.get("out", M(Q35_BF16), &out));
    Q35_REQUIRE(pk.nd == 4 && out.nd == 3, Q35_ERR_SHAPE, "attn.lse_merge: packed [R, B, Hq, D + 2], out [B, HQ, D]");
    const int64_t R = pk.s[0], B = pk.s[1], Hq = pk.s[2], D = pk.s[3] - 2, HQ = out.s[1];
    Q35_REQUIRE(D > 0 && Hq > 0 && out.s[0] == B && out.s[2] == D && HQ % Hq == 0 && R % (HQ / Hq) == 0, Q35_ERR_SHAPE,
                "attn.lse_merge: R ranks must be (HQ / Hq) KV groups times an equal number of page shares");
    c.ws_need = 0;
    if (c.dry || B * HQ == 0) return 0;
    attn_lse_merge_packed_kernel<<<unsigned(B * HQ), 128, 0, c.stream>>>(pk.as<float>(), out.as<__nv_bfloat16>(),
                                                                        int(R / (HQ / Hq)), int(B), int(Hq), int(HQ), int(D));
    Q35_CUDA_LAUNCH_CHECK("attn.lse_merge");
    return 0;
  }
  Q35_TRY(c.get("part_m", M(Q35_F32), &pm));
  Q35_TRY(c.get("part_l", M(Q35_F32), &pl));
  Q35_TRY(c.get("part_o", M(Q35_F32), &po));
  Q35_TRY(c.get("out", M(Q35_BF16), &out));
  Q35_REQUIRE(po.nd == 4 && out.nd == 3, Q35_ERR_SHAPE, "attn.lse_merge: part_o [G, B, HQ, D], out [B, HQ, D]");
  const int64_t G = po.s[0], B = po.s[1], HQ = po.s[2], D = po.s[3];
  Q35_REQUIRE(pm.numel() == G * B * HQ && pl.numel() == G * B * HQ && out.numel() == B * HQ * D, Q35_ERR_SHAPE,
              "attn.lse_merge: part_m / part_l [G, B, HQ]");
  c.ws_need = 0;
  if (c.dry || B * HQ == 0) return 0;
  attn_lse_merge_kernel<<<unsigned(B * HQ), 128, 0, c.stream>>>(pm.as<float>(), pl.as<float>(), po.as<float>(),
                                                               out.as<__nv_bfloat16>(), int(G), int(B * HQ), int(D));
  Q35_CUDA_LAUNCH_CHECK("attn.lse_merge");
  return 0;
}

// attn.kv_write: the current token's K / V rows into the cache at (page, offset)
// (store_paged_kv, flash_attn.py:53-84; FP8: e4m3(8 x), models/qwen38_27b/decode/q35_group.py:244-249, or
// e4m3(x / scale_h) with a per-head scale)
__global__ void attn_kv_write_kernel(const __nv_bfloat16* __restrict__ k_new, const __nv_bfloat16* __restrict__ v_new,
                                     const int* __restrict__ loc, const float* kv_scale, void* cache, int B, int HKV,
                                     int D, int P, int num_pages, int fp8, int* status) {
  const int b = blockIdx.x;
  const int page = loc[2 * b], off = loc[2 * b + 1];
  if (page < 0 || page >= num_pages || off < 0 || off >= P) {
    if (threadIdx.x == 0) atomicOr(status, DS_BAD_PAGE);
    return;
  }
  const int n = HKV * D;
  for (int i = threadIdx.x; i < 2 * n; i += blockDim.x) {
    const int kv = i / n, j = i % n;
    const __nv_bfloat16 val = kv ? v_new[size_t(b) * n + j] : k_new[size_t(b) * n + j];
    const size_t dst = ((size_t(page) * 2 + kv) * P + off) * n + j;
    if (fp8) {
      const float x = __bfloat162float(val);  // per-head form: a true division, as the golden's
      static_cast<__nv_fp8_e4m3*>(cache)[dst] = __nv_fp8_e4m3(kv_scale ? x / kv_scale[kv * HKV + j / D] : x * 8.f);
    } else {
      static_cast<__nv_bfloat16*>(cache)[dst] = val;
    }
  }
}

// int8 rows with one bf16 scale per row and head (kv_quant_row, models/qwen38_27b/decode/q35_group.py:198-205):
// amax over the head's D values (at least 1e-5), s = bf16(amax * bf16(1 / 127)), q = round(bf16(x * bf16(1 / s))).
// One warp per (sequence, K or V, head).
__global__ void attn_kv_write_int8_kernel(const __nv_bfloat16* __restrict__ k_new, const __nv_bfloat16* __restrict__ v_new,
                                          const int* __restrict__ loc, int8_t* cache, __nv_bfloat16* scales, int B,
                                          int HKV, int D, int P, int num_pages, int* status) {
  const int w = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (w >= B * 2 * HKV) return;
  const int b = w / (2 * HKV), kv = (w / HKV) & 1, h = w % HKV;
  const int page = loc[2 * b], off = loc[2 * b + 1];
  if (page < 0 || page >= num_pages || off < 0 || off >= P) {
    if (lane == 0) atomicOr(status, DS_BAD_PAGE);
    return;
  }
  const __nv_bfloat16* src = (kv ? v_new : k_new) + (size_t(b) * HKV + h) * D;
  float amax = 0.f;
  for (int i = lane; i < D; i += 32) amax = fmaxf(amax, fabsf(__bfloat162float(src[i])));
  for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  amax = fmaxf(amax, round_bf16(1e-5f));
  const float sc = round_bf16(amax * round_bf16(1.f / 127.f));
  const float inv = round_bf16(1.f / sc);
  const size_t row = (size_t(page) * 2 + kv) * P + off;
  for (int i = lane; i < D; i += 32) {
    const float qv = rintf(round_bf16(__bfloat162float(src[i]) * inv));
    cache[(row * HKV + h) * D + i] = int8_t(fminf(fmaxf(qv, -127.f), 127.f));
  }
  if (lane == 0) scales[row * HKV + h] = __float2bfloat16_rn(sc);
}

int run_attn_kv_write(Call& c) {
  Tensor k, v, loc, cache, sc;
  Q35_TRY(c.get("k_new", M(Q35_BF16), &k));
  Q35_TRY(c.get("v_new", M(Q35_BF16), &v));
  Q35_TRY(c.get("cache_location", M(Q35_I32), &loc));
  Q35_TRY(c.get("paged_kv_cache", M(Q35_BF16) | M_FP8, &cache));
  Q35_TRY(c.get("kv_scale", M(Q35_F32), &sc, false));
  Q35_REQUIRE(cache.nd == 5 && cache.s[1] == 2 && k.nd == 3, Q35_ERR_SHAPE,
              "attn.kv_write: cache [pages, 2, P, HKV, D], k_new [B, HKV, D]");
  const int64_t B = k.s[0], HKV = cache.s[3], D = cache.s[4], P = cache.s[2];
  Q35_REQUIRE(k.s[1] == HKV && k.s[2] == D && v.numel() == k.numel() && loc.numel() == 2 * B, Q35_ERR_SHAPE,
              "attn.kv_write: shapes");
  Q35_REQUIRE(!sc.present || sc.numel() == 2 * HKV, Q35_ERR_SHAPE, "attn.kv_write: kv_scale [2, HKV]");
  Tensor rsc;
  Q35_TRY(c.get("paged_kv_scale", M(Q35_BF16), &rsc, false));
  Q35_REQUIRE(!rsc.present || (cache.dtype != Q35_BF16 && !sc.present && rsc.numel() == cache.s[0] * 2 * P * HKV),
              Q35_ERR_SHAPE, "attn.kv_write: paged_kv_scale [pages, 2, P, HKV] bf16 goes with an int8 cache");
  c.ws_need = 0;
  if (c.dry || B == 0) return 0;
  if (rsc.present) {
    const int64_t warps = B * 2 * HKV;
    attn_kv_write_int8_kernel<<<unsigned((warps + 3) / 4), 128, 0, c.stream>>>(
        k.as<__nv_bfloat16>(), v.as<__nv_bfloat16>(), loc.as<int>(), static_cast<int8_t*>(cache.p),
        rsc.as<__nv_bfloat16>(), int(B), int(HKV), int(D), int(P), int(cache.s[0]), device_status_ptr());
    Q35_CUDA_LAUNCH_CHECK("attn.kv_write int8");
    return 0;
  }
  attn_kv_write_kernel<<<unsigned(B), 256, 0, c.stream>>>(
      k.as<__nv_bfloat16>(), v.as<__nv_bfloat16>(), loc.as<int>(), sc.present ? sc.as<float>() : nullptr, cache.p,
      int(B), int(HKV), int(D), int(P), int(cache.s[0]), cache.dtype != Q35_BF16, device_status_ptr());
  Q35_CUDA_LAUNCH_CHECK("attn.kv_write");
  return 0;
}

template <int D, int KVF, int WARPS = 4>
static int launch_attn(const AttnArgs& a, cudaStream_t stream) {
  using C = AttnCfg<D, KVF, WARPS>;
  Q35_REQUIRE(a.wpc == WARPS, Q35_ERR_CUDA, "attention decode: partial slots sized for %d warps, kernel has %d", a.wpc, WARPS);
  Q35_TRY(ensure_dynamic_smem(reinterpret_cast<const void*>(attn_decode_kernel<D, KVF, WARPS>), C::SMEM));
  Q35_REQUIRE(a.status != nullptr, Q35_ERR_CUDA, "attention decode: no device status word");
  launch_pdl(attn_plan_kernel, dim3(1), dim3(1024), 0, stream, a);
  Q35_CUDA_LAUNCH_CHECK("attn plan");
  launch_pdl(attn_decode_kernel<D, KVF, WARPS>, dim3(unsigned(a.n_cta)), dim3(32 * WARPS), C::SMEM, stream, a);
  Q35_CUDA_LAUNCH_CHECK("attn decode");
  launch_pdl(attn_merge_kernel<D>, dim3(unsigned(a.B * a.HQ)), dim3(D / 2), 0, stream, a);
  Q35_CUDA_LAUNCH_CHECK("attn merge");
  return 0;
}

int run_attn_paged_decode(Call& c) {
  Tensor q, cache, indptr, indices, lpl, scale, kvs, kn, vn, out, ws;
  Q35_TRY(c.get("q", M(Q35_BF16), &q));
  Q35_TRY(c.get("paged_kv_cache", M(Q35_BF16) | M_FP8, &cache));
  Q35_TRY(c.get("indptr", M(Q35_I32), &indptr));
  Q35_TRY(c.get("indices", M(Q35_I32), &indices));
  Q35_TRY(c.get("last_page_len", M(Q35_I32), &lpl));
  Q35_TRY(c.get("sm_scale", M(Q35_F32), &scale, false));
  Q35_TRY(c.get("kv_scale", M(Q35_F32), &kvs, false));
  Q35_TRY(c.get("k_new", M(Q35_BF16), &kn, false));
  Q35_TRY(c.get("v_new", M(Q35_BF16), &vn, false));
  Tensor lm, ll, lo;
  Q35_TRY(c.get("part_m", M(Q35_F32), &lm, false));
  Q35_TRY(c.get("part_l", M(Q35_F32), &ll, false));
  Q35_TRY(c.get("part_o", M(Q35_F32), &lo, false));
  Q35_REQUIRE(lm.present == lo.present && ll.present == lo.present, Q35_ERR_MISSING,
              "attn.paged_decode: part_m, part_l and part_o go together");
  Tensor lpk;
  Q35_TRY(c.get("part_packed", M(Q35_F32), &lpk, false));
  Q35_REQUIRE(!(lpk.present && lo.present), Q35_ERR_SHAPE, "attn.paged_decode: part_packed or part_m / part_l / part_o");
  const bool partial = lo.present || lpk.present;
  Q35_TRY(c.get("out", M(Q35_BF16), &out, !partial));
  Q35_REQUIRE(q.nd == 3 && cache.nd == 5 && cache.s[1] == 2, Q35_ERR_SHAPE,
              "attn.paged_decode: q [B, HQ, D], paged_kv_cache [pages, 2, P, HKV, D]");
  const int64_t B = q.s[0], HQ = q.s[1], D = q.s[2], P = cache.s[2], HKV = cache.s[3];
  Q35_REQUIRE(cache.s[4] == D && HKV > 0 && HQ % HKV == 0, Q35_ERR_SHAPE, "attn.paged_decode: head shapes");
  const int64_t G = HQ / HKV;
  Q35_REQUIRE(G <= AT_GMAX, Q35_ERR_UNSUPPORTED, "attn.paged_decode: at most 8 query heads per KV head (got %lld)",
              (long long)G);
  Q35_REQUIRE(D == 64 || D == 128 || D == 256, Q35_ERR_UNSUPPORTED, "attn.paged_decode: head_dim must be 64/128/256");
  Q35_REQUIRE(P % 16 == 0 && P >= 16, Q35_ERR_UNSUPPORTED, "attn.paged_decode: page size must be a multiple of 16");
  Q35_REQUIRE(indptr.numel() == B + 1 && lpl.numel() >= B, Q35_ERR_SHAPE, "attn.paged_decode: indptr [B+1], last_page_len [B]");
  Q35_REQUIRE(partial || out.numel() == B * HQ * D, Q35_ERR_SHAPE, "attn.paged_decode: out [B, HQ, D]");
  Q35_REQUIRE(!lpk.present || lpk.numel() == B * HQ * (D + 2), Q35_ERR_SHAPE,
              "attn.paged_decode: part_packed [B, HQ, D + 2]");
  Q35_REQUIRE(!lo.present || (lo.numel() == B * HQ * D && lm.numel() == B * HQ && ll.numel() == B * HQ), Q35_ERR_SHAPE,
              "attn.paged_decode: part_m / part_l [B, HQ], part_o [B, HQ, D]");
  Q35_REQUIRE(kn.present == vn.present, Q35_ERR_MISSING, "attn.paged_decode: k_new and v_new go together");
  Q35_REQUIRE(!kn.present || (kn.numel() == B * HKV * D && vn.numel() == B * HKV * D), Q35_ERR_SHAPE,
              "attn.paged_decode: k_new / v_new [B, HKV, D]");
  Q35_REQUIRE(!kvs.present || kvs.numel() == 2 * HKV, Q35_ERR_SHAPE, "attn.paged_decode: kv_scale [2, HKV]");
  Tensor rsc;
  Q35_TRY(c.get("paged_kv_scale", M(Q35_BF16), &rsc, false));
  const bool fp8 = cache.dtype != Q35_BF16;
  Q35_REQUIRE(!rsc.present || (fp8 && !kvs.present && rsc.numel() == cache.s[0] * 2 * P * HKV), Q35_ERR_SHAPE,
              "attn.paged_decode: paged_kv_scale [pages, 2, P, HKV] bf16 goes with an int8 cache (bound as bytes)");
  Q35_REQUIRE(!fp8 || D == 256 || D == 128, Q35_ERR_UNSUPPORTED, "attn.paged_decode: FP8 cache needs head_dim 128/256");
  const int n_cta = sm_count();
  const int wpc = fp8 ? 8 : 4;  // one-byte formats run two warps per scheduler (see AttnCfg)
  const int64_t S = B * HKV, slots = (S + n_cta) * wpc;
  int64_t off = 0;
  auto take = [&](int64_t bytes) { const int64_t o = off; off = (off + bytes + 255) / 256 * 256; return o; };
  const int64_t o_plan = take(sizeof(AttnPlan)), o_seg = take((S + 1) * 4), o_ctx = take(B * 4),
                o_ml = take(slots * 16 * 4), o_po = take(slots * AT_GMAX * D * 4);
  Q35_TRY(c.workspace(off, &ws));
  if (c.dry || B == 0) return 0;
  Q35_REQUIRE(aligned16(q.p) && aligned16(cache.p) && (lpk.present ? aligned16(lpk.p) : lo.present ? aligned16(lo.p) : aligned16(out.p)), Q35_ERR_ALIGN,
              "attn.paged_decode: pointers must be 16-byte aligned");
  AttnArgs a{};
  a.q = q.p; a.cache = cache.p; a.indptr = indptr.as<int>(); a.indices = indices.as<int>();
  a.last_page_len = lpl.as<int>();
  a.sm_scale = scale.present ? scale.as<float>() : nullptr;
  a.kv_scale = kvs.present ? kvs.as<float>() : nullptr;
  a.k_new = kn.present ? kn.as<__nv_bfloat16>() : nullptr;
  a.v_new = vn.present ? vn.as<__nv_bfloat16>() : nullptr;
  a.out = partial ? nullptr : out.as<__nv_bfloat16>();
  a.lse_m = lo.present ? lm.as<float>() : nullptr;
  a.lse_l = lo.present ? ll.as<float>() : nullptr;
  a.lse_o = lo.present ? lo.as<float>() : nullptr;
  a.lse_os = int(D); a.lse_ms = 1;
  if (lpk.present) {  // one message per rank: o | m | l in every row
    a.lse_o = lpk.as<float>(); a.lse_m = a.lse_o + D; a.lse_l = a.lse_o + D + 1;
    a.lse_os = a.lse_ms = int(D) + 2;
  }
  a.B = int(B); a.HQ = int(HQ); a.HKV = int(HKV); a.G = int(G); a.P = int(P);
  a.num_pages = int(cache.s[0]); a.n_indices = int(indices.numel()); a.n_cta = n_cta;
  uint8_t* w = ws.as<uint8_t>();
  a.plan = reinterpret_cast<AttnPlan*>(w + o_plan);
  a.seg_start = reinterpret_cast<int*>(w + o_seg);
  a.ctx = reinterpret_cast<int*>(w + o_ctx);
  a.part_ml = reinterpret_cast<float*>(w + o_ml);
  a.part_o = reinterpret_cast<float*>(w + o_po);
  a.status = device_status_ptr();
  a.wpc = wpc;
  if (rsc.present) {
    a.row_scale = rsc.as<__nv_bfloat16>();
    return D == 128 ? launch_attn<128, 2, 8>(a, c.stream) : launch_attn<256, 2, 8>(a, c.stream);
  }
  if (fp8) return D == 128 ? launch_attn<128, 1, 8>(a, c.stream) : launch_attn<256, 1, 8>(a, c.stream);
  if (D == 64) return launch_attn<64, 0>(a, c.stream);
  if (D == 128) return launch_attn<128, 0>(a, c.stream);
  return launch_attn<256, 0>(a, c.stream);
}

// ---------------------------------------------------------------------------------------------------------------
// q35_attn_paged_decode_static: paged attention decode for callers that cannot provide a workspace.
//
// Some hosts of these kernels have no way to allocate device memory at call time: an inference runtime whose
// buffers are all planned before the first token and then frozen (the llama.cpp-style backends the reference
// targets work that way), or a caller sitting inside somebody else's memory pool.  q35_run("attn.paged_decode")
// needs a `workspace` tensor for the split-KV partials; this entry point takes none.  The same kernels run, with
// their scratch in the file-scope device array below.
//
// Limits and rules:
//  * the scratch is Q35_ATTN_STATIC_SCRATCH_BYTES (16 MiB) per GPU, held from library load until process exit; a
//    call whose shapes need more is rejected with Q35_ERR_WORKSPACE (need = what q35_workspace_bytes reports for
//    "attn.paged_decode": about (B * HKV + SMs) * 4 * (64 + 32 * D) bytes, e.g. 9.1 MB for batch 64, 2 KV heads,
//    head_dim 256 on 148 SMs);
//  * the first call on a device looks up the array's device address (cudaGetSymbolAddress, with that device
//    current).  That first call should be made outside any stream capture;
//  * nothing here calls cudaMalloc / cudaFree or any allocating library routine;
//  * every call on a GPU uses the same array and finds in it whatever the previous call left.  The kernels write
//    every plan entry and every partial slot before reading it, so nothing has to be cleared, but two calls that
//    overlap on the GPU (different streams, or threads) race on it: serialise them.
constexpr size_t Q35_ATTN_STATIC_SCRATCH_BYTES = size_t(16) << 20;
static __device__ __align__(256) unsigned char g_attn_static_scratch[Q35_ATTN_STATIC_SCRATCH_BYTES];

// In host code `g_attn_static_scratch` is only a host-side handle for the symbol, not an address a kernel can use:
// the device address comes from cudaGetSymbolAddress, once per device.
static int attn_static_scratch(uint8_t** out) {
  constexpr int kMaxDevices = 64;
  static uint8_t* per_device[kMaxDevices] = {nullptr};
  static std::mutex lock;  // host threads may make their first calls at the same time
  std::lock_guard<std::mutex> guard(lock);
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  Q35_REQUIRE(e == cudaSuccess && dev >= 0 && dev < kMaxDevices, Q35_ERR_CUDA, "cudaGetDevice: %s",
              cudaGetErrorString(e));
  if (!per_device[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_attn_static_scratch);
    Q35_REQUIRE(e == cudaSuccess && p != nullptr, Q35_ERR_CUDA, "cudaGetSymbolAddress(static scratch): %s",
                cudaGetErrorString(e));
    per_device[dev] = static_cast<uint8_t*>(p);
  }
  *out = per_device[dev];
  return 0;
}

}  // namespace q35

extern "C" int q35_attn_paged_decode_static(const void* q, const void* paged_kv_cache, int cache_dtype,
                                            const int* indptr, const int* indices, const int* last_page_len,
                                            const float* sm_scale, const float* kv_scale, void* out, int B, int HQ,
                                            int HKV, int D, int P, int num_pages, int n_indices, void* stream) {
  using namespace q35;
  clear_error();
  Q35_REQUIRE(q && paged_kv_cache && indptr && indices && last_page_len && out, Q35_ERR_MISSING,
              "q35_attn_paged_decode_static: null pointer");
  Q35_REQUIRE(cache_dtype == Q35_BF16 || cache_dtype == Q35_E4M3, Q35_ERR_DTYPE,
              "q35_attn_paged_decode_static: cache dtype must be bf16 (9) or e4m3 (11)");
  Q35_REQUIRE(B >= 0 && HKV > 0 && HQ > 0 && HQ % HKV == 0 && HQ / HKV <= AT_GMAX, Q35_ERR_UNSUPPORTED,
              "q35_attn_paged_decode_static: at most 8 query heads per KV head");
  const bool fp8 = cache_dtype == Q35_E4M3;
  Q35_REQUIRE(fp8 ? (D == 128 || D == 256) : (D == 64 || D == 128 || D == 256), Q35_ERR_UNSUPPORTED,
              "q35_attn_paged_decode_static: head_dim %d", D);
  Q35_REQUIRE(P >= 16 && P % 16 == 0 && num_pages > 0 && n_indices >= 0, Q35_ERR_SHAPE,
              "q35_attn_paged_decode_static: page size must be a multiple of 16");
  if (B == 0) return 0;
  Q35_REQUIRE(aligned16(q) && aligned16(paged_kv_cache) && aligned16(out), Q35_ERR_ALIGN,
              "q35_attn_paged_decode_static: pointers must be 16-byte aligned");
  const int n_cta = sm_count();
  const int64_t S = int64_t(B) * HKV, slots = (S + n_cta) * 4;
  int64_t off = 0;
  auto take = [&](int64_t bytes) { const int64_t o = off; off = (off + bytes + 255) / 256 * 256; return o; };
  const int64_t o_plan = take(sizeof(AttnPlan)), o_seg = take((S + 1) * 4), o_ctx = take(int64_t(B) * 4),
                o_ml = take(slots * 16 * 4), o_po = take(slots * AT_GMAX * D * 4);
  Q35_REQUIRE(off <= int64_t(Q35_ATTN_STATIC_SCRATCH_BYTES), Q35_ERR_WORKSPACE,
              "q35_attn_paged_decode_static: these shapes need %lld bytes of scratch, the built-in array holds %lld; "
              "use q35_run(\"attn.paged_decode\") with a workspace",
              (long long)off, (long long)Q35_ATTN_STATIC_SCRATCH_BYTES);
  uint8_t* w = nullptr;
  Q35_TRY(attn_static_scratch(&w));
  AttnArgs a{};
  a.q = q; a.cache = paged_kv_cache; a.indptr = indptr; a.indices = indices; a.last_page_len = last_page_len;
  a.sm_scale = sm_scale; a.kv_scale = kv_scale; a.k_new = nullptr; a.v_new = nullptr;
  a.out = static_cast<__nv_bfloat16*>(out);
  a.B = B; a.HQ = HQ; a.HKV = HKV; a.G = HQ / HKV; a.P = P;
  a.num_pages = num_pages; a.n_indices = n_indices; a.n_cta = n_cta;
  a.wpc = 4;  // every format on four warps here: the built-in scratch holds four partial slots per (segment, CTA)
  a.plan = reinterpret_cast<AttnPlan*>(w + o_plan);
  a.seg_start = reinterpret_cast<int*>(w + o_seg);
  a.ctx = reinterpret_cast<int*>(w + o_ctx);
  a.part_ml = reinterpret_cast<float*>(w + o_ml);
  a.part_o = reinterpret_cast<float*>(w + o_po);
  a.status = device_status_ptr();
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (fp8) return D == 128 ? launch_attn<128, 1>(a, s) : launch_attn<256, 1>(a, s);
  if (D == 64) return launch_attn<64, 0>(a, s);
  if (D == 128) return launch_attn<128, 0>(a, s);
  return launch_attn<256, 0>(a, s);
}
