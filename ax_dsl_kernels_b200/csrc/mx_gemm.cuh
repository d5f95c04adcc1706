// Weight-streaming "skinny" GEMM for decode-sized token counts: out[t, n] = sum_k x[t, k] * W[n, k] with W held in
// HBM as MXFP4 (E2M1 pairs + E8M0 per 32), MXFP8 (E4M3 + E8M0 per 32) or FP8 E4M3 with per-row fp32 scales.
//
// Bound: HBM.  Every weight byte is read once per token group and expanded to bf16 in registers with shifts and one
// bf16x2 multiply per pair (the multiply carries the block scale), then fed to mma.sync m16n8k16 with the weights as
// the 16-row operand and up to 8 tokens as the 8-column operand.  Activations live in shared memory, pre-permuted so
// that the k order of the in-register expansion and of the activation fragments agree.
#pragma once
#include "common.cuh"

namespace q35 {

enum : int { W_MXFP4 = 0, W_MXFP8 = 1, W_FP8ROW = 2, W_NVFP4 = 3 };
// NVFP4: E2M1 pairs as MXFP4, one E4M3 scale per 16 inputs, one fp32 scale for the tensor
// (quantize_nvfp4, models/qwen35_35b_a3b/sgl/python/sgl_kernel_axera/quantization.py:8-37)
constexpr bool fmt_is_fp4(int f) { return f == W_MXFP4 || f == W_NVFP4; }
enum : int { EPI_SILU_MUL = 0, EPI_ROW_SCALE = 1, EPI_SHARED_DOWN = 2, EPI_PLAIN = 3 };

struct SkinnyArgs {
  // two 16-row weight streams per warp (gate rows and up rows, or two neighbouring row tiles of one matrix)
  const uint8_t* w[2];     // weight base of each stream (expert 0)
  const uint8_t* s[2];     // E8M0 scales [rows, K/32] bytes, or fp32 per-row scales (W_FP8ROW)
  long long w_plane, s_plane;  // bytes between consecutive experts
  int K;                   // contraction length
  int roff[2];             // row offset of each stream inside its matrix
  int lim[2];              // first invalid row of each stream (in its matrix)
  int act_rows;            // EPI_SILU_MUL: row stride of act_out (= intermediate size)
  int tile_rows, warp_rows;  // stream row base = tile * tile_rows + warp * warp_rows (+ roff)
  // activations
  const __nv_bfloat16* x;
  int x_stride;            // elements between rows of x
  const int* src;          // destination row -> row of x (nullptr: identity)
  // groups (nullptr g_n: one dense group of n_dense rows on plane 0)
  const int* g_expert; const int* g_n; const int* g_row0;
  int n_dense;
  int n_planes;
  // epilogue
  __nv_bfloat16* act_out;  // EPI_SILU_MUL: [dest row, rows]
  float* f_out;            // EPI_ROW_SCALE / EPI_PLAIN(f32): [dest row, out_stride]
  __nv_bfloat16* b_out;    // EPI_SHARED_DOWN / EPI_PLAIN(bf16)
  int out_stride;
  const float* rw_row;     // EPI_ROW_SCALE: weight per destination row
  const __nv_bfloat16* resid;  // EPI_SHARED_DOWN: residual [T, out_stride]
  const float* gate;       // EPI_SHARED_DOWN: pre-sigmoid gate per token
  const float* bias;       // EPI_PLAIN: optional per-row bias
  const float* tensor_scale;  // W_NVFP4: the weight's fp32 scale [1]
  const float* row_div;    // EPI_PLAIN: optional per-token divisor applied to the bf16-rounded product (folded RMSNorm)
  const __nv_bfloat16* resid2;  // EPI_PLAIN: optional residual [T, out_stride] added to the bf16-rounded product
  int* status;
};

constexpr int SK_KC = 1024;  // activation chunk (elements of k) staged in shared memory

template <int FMT> struct WTraits;
template <> struct WTraits<W_MXFP4> { static constexpr int KIT = 256, PAD_UNITS = 4, BIAS = 63; };
template <> struct WTraits<W_MXFP8> { static constexpr int KIT = 128, PAD_UNITS = 1, BIAS = 57; };
template <> struct WTraits<W_FP8ROW> { static constexpr int KIT = 128, PAD_UNITS = 1, BIAS = 57; };
template <> struct WTraits<W_NVFP4> { static constexpr int KIT = 256, PAD_UNITS = 4, BIAS = 63; };

__device__ __forceinline__ uint32_t bf16x2_mul(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// physical 16-byte unit of logical unit u inside an activation row (bank-conflict-free fragment reads)
template <int FMT>
__device__ __forceinline__ int swz_unit(int u) {
  if constexpr (fmt_is_fp4(FMT)) return u ^ ((u >> 3) & 3);
  else return u ^ (((u >> 3) & 1) << 1);
}

template <int FMT, int EPI, int NT>
__global__ void __launch_bounds__(128) skinny_gemm_kernel(const SkinnyArgs a) {
  using TR = WTraits<FMT>;
  constexpr int KIT = TR::KIT;                    // k per main-loop iteration
  constexpr int ROW_UNITS = SK_KC / 8 + TR::PAD_UNITS;  // 16-byte units per staged activation row
  constexpr int UPL = KIT / 4 / 8;                // activation units per lane per iteration (8 for fp4, 4 for fp8)
  extern __shared__ uint4 s_x[];                  // [NT * 8][ROW_UNITS]

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int r = lane >> 2, c = lane & 3;
  const int grp = blockIdx.y;
  int n, plane, row0;
  if (a.g_n) {
    n = a.g_n[grp];
    plane = a.g_expert[grp];
    row0 = a.g_row0[grp];
    if (plane < 0 || plane >= a.n_planes) {
      if (tid == 0) atomicOr(a.status, DS_BAD_EXPERT);
      n = 0;
    }
  } else {
    n = a.n_dense; plane = 0; row0 = 0;
  }
  if (n <= 0) return;

  const int row_base = blockIdx.x * a.tile_rows + warp * a.warp_rows;
  const int wrow_bytes = fmt_is_fp4(FMT) ? a.K / 2 : a.K;
  const int srow = FMT == W_NVFP4 ? a.K / 16 : a.K / 32;
  // rows this lane streams: [stream][half]; out-of-range rows are clamped for loads and masked at the end
  int rows_l[2][2];
  bool rok[2][2];
  const uint8_t* wptr[2][2];
  const uint8_t* sptr[2][2];
  const uint8_t* sp[2];
#pragma unroll
  for (int st = 0; st < 2; ++st) {
    const uint8_t* wp = a.w[st] + (long long)plane * a.w_plane;
    sp[st] = a.s[st] + (long long)plane * a.s_plane;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      rows_l[st][h] = row_base + a.roff[st] + r + 8 * h;
      rok[st][h] = rows_l[st][h] < a.lim[st];
      const int rr = rok[st][h] ? rows_l[st][h] : 0;
      wptr[st][h] = wp + (long long)rr * wrow_bytes + c * 32;
      if constexpr (FMT == W_MXFP4) sptr[st][h] = sp[st] + (long long)rr * srow + c * 2;
      else if constexpr (FMT == W_NVFP4) sptr[st][h] = sp[st] + (long long)rr * srow + c * 4;
      else if constexpr (FMT == W_MXFP8) sptr[st][h] = sp[st] + (long long)rr * srow + c;
      else sptr[st][h] = sp[st];
    }
  }

  const int n_groups = (n + NT * 8 - 1) / (NT * 8);
  const int n_it = a.K / KIT;
  for (int tg = 0; tg < n_groups; ++tg) {
    const int t_base = tg * NT * 8;
    float acc[2][NT][4];
#pragma unroll
    for (int st = 0; st < 2; ++st)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[st][nt][i] = 0.f;

    uint4 wcur[2][2][2], wnxt[2][2][2];
    uint32_t scur[2][2], snxt[2][2];
    auto load_w = [&](int it, uint4 (&wd)[2][2][2], uint32_t (&sd)[2][2]) {
#pragma unroll
      for (int st = 0; st < 2; ++st)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const uint8_t* p = wptr[st][h] + (long long)it * 128;
          wd[st][h][0] = ldg_nc_16(p);
          wd[st][h][1] = ldg_nc_16(p + 16);
          if constexpr (FMT == W_MXFP4) sd[st][h] = *reinterpret_cast<const unsigned short*>(sptr[st][h] + it * 8);
          else if constexpr (FMT == W_NVFP4) sd[st][h] = *reinterpret_cast<const uint32_t*>(sptr[st][h] + it * 16);
          else if constexpr (FMT == W_MXFP8) sd[st][h] = *(sptr[st][h] + it * 4);
          else sd[st][h] = 127;
        }
    };
    load_w(0, wcur, scur);

    for (int kc = 0; kc < a.K; kc += SK_KC) {
      const int kc_len = min(SK_KC, a.K - kc);
      __syncthreads();
      // stage activations of this chunk: permuted inside each unit, scaled by 2^63
      const int units = kc_len / 8;
      for (int idx = tid; idx < NT * 8 * units; idx += 128) {
        const int tkn = idx / units, u = idx % units;
        const int t = t_base + tkn;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (t < n) {
          const int dst = row0 + t;
          const long long xr = a.src ? a.src[dst] : dst;
          v = *reinterpret_cast<const uint4*>(a.x + xr * a.x_stride + kc + u * 8);
          uint4 o;
          if constexpr (fmt_is_fp4(FMT)) {
            o.x = __byte_perm(v.x, v.z, 0x5410); o.y = __byte_perm(v.x, v.z, 0x7632);
            o.z = __byte_perm(v.y, v.w, 0x5410); o.w = __byte_perm(v.y, v.w, 0x7632);
          } else {
            o.x = __byte_perm(v.x, v.y, 0x5410); o.y = __byte_perm(v.x, v.y, 0x7632);
            o.z = __byte_perm(v.z, v.w, 0x5410); o.w = __byte_perm(v.z, v.w, 0x7632);
          }
          const uint32_t two63 = 0x5F005F00u;
          v.x = bf16x2_mul(o.x, two63); v.y = bf16x2_mul(o.y, two63);
          v.z = bf16x2_mul(o.z, two63); v.w = bf16x2_mul(o.w, two63);
        }
        s_x[tkn * ROW_UNITS + swz_unit<FMT>(u)] = v;
      }
      __syncthreads();

      const int it0 = kc / KIT, it1 = (kc + kc_len) / KIT;
      for (int it = it0; it < it1; ++it) {
        if (it + 1 < n_it) load_w(it + 1, wnxt, snxt);
        // per-block multipliers: 2^(s - 127) folded with the exponent re-bias of the bit trick
        uint32_t mult[2][2][FMT == W_NVFP4 ? 4 : 2];
#pragma unroll
        for (int st = 0; st < 2; ++st)
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            if constexpr (FMT == W_NVFP4) {
              // four E4M3 scales (k 0-15, 16-31, 32-47, 48-63 of this lane's 64 inputs) times the 2^63 of the bit trick
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const __half_raw hr = __nv_cvt_fp8_to_halfraw(__nv_fp8_storage_t((scur[st][h] >> (8 * j)) & 0xff), __NV_E4M3);
                const float f = __half2float(*reinterpret_cast<const __half*>(&hr)) * 9223372036854775808.f;
                mult[st][h][j] = uint32_t(__bfloat16_as_ushort(__float2bfloat16_rn(f))) * 0x00010001u;
              }
            } else if constexpr (FMT == W_MXFP4) {
              mult[st][h][0] = (((scur[st][h] & 0xff) + TR::BIAS) << 7) * 0x00010001u;
              mult[st][h][1] = (((scur[st][h] >> 8) + TR::BIAS) << 7) * 0x00010001u;
            } else {
              mult[st][h][0] = mult[st][h][1] = ((scur[st][h] + TR::BIAS) << 7) * 0x00010001u;
            }
          }
        const int ubase = (it - it0) * (KIT / 8) + c * UPL;
#pragma unroll
        for (int q = 0; q < 2; ++q) {          // the two 16-byte loads of this iteration
#pragma unroll
          for (int wi = 0; wi < 4; ++wi) {     // words of the load
            if constexpr (fmt_is_fp4(FMT)) {
              const int j = q * 4 + wi;        // activation unit of this word (8 nibbles = 8 k)
              uint4 bx[NT];
#pragma unroll
              for (int nt = 0; nt < NT; ++nt) bx[nt] = s_x[(nt * 8 + r) * ROW_UNITS + swz_unit<FMT>(ubase + j)];
#pragma unroll
              for (int st = 0; st < 2; ++st) {
                const uint32_t w0 = reinterpret_cast<const uint32_t*>(&wcur[st][0][q])[wi];
                const uint32_t w1 = reinterpret_cast<const uint32_t*>(&wcur[st][1][q])[wi];
                const int mi = FMT == W_NVFP4 ? q * 2 + (wi >> 1) : q;  // NVFP4: a scale per 16 inputs = two words
                const uint32_t m0 = mult[st][0][mi], m1 = mult[st][1][mi];
                const uint32_t p0 = bf16x2_mul(((w0 << 6) & 0x01C001C0u) | ((w0 << 12) & 0x80008000u), m0);
                const uint32_t p1 = bf16x2_mul(((w0 << 2) & 0x01C001C0u) | ((w0 << 8) & 0x80008000u), m0);
                const uint32_t p2 = bf16x2_mul(((w0 >> 2) & 0x01C001C0u) | ((w0 << 4) & 0x80008000u), m0);
                const uint32_t p3 = bf16x2_mul(((w0 >> 6) & 0x01C001C0u) | (w0 & 0x80008000u), m0);
                const uint32_t q0 = bf16x2_mul(((w1 << 6) & 0x01C001C0u) | ((w1 << 12) & 0x80008000u), m1);
                const uint32_t q1 = bf16x2_mul(((w1 << 2) & 0x01C001C0u) | ((w1 << 8) & 0x80008000u), m1);
                const uint32_t q2 = bf16x2_mul(((w1 >> 2) & 0x01C001C0u) | ((w1 << 4) & 0x80008000u), m1);
                const uint32_t q3 = bf16x2_mul(((w1 >> 6) & 0x01C001C0u) | (w1 & 0x80008000u), m1);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                  mma_bf16_16816(acc[st][nt], p0, q0, p1, q1, bx[nt].x, bx[nt].y);
                  mma_bf16_16816(acc[st][nt], p2, q2, p3, q3, bx[nt].z, bx[nt].w);
                }
              }
            } else {
              const int j = q * 2 + (wi >> 1);  // activation unit (8 k) holding this word's 4 k
              uint2 bx[NT];
#pragma unroll
              for (int nt = 0; nt < NT; ++nt) {
                const uint4 full = s_x[(nt * 8 + r) * ROW_UNITS + swz_unit<FMT>(ubase + j)];
                bx[nt] = (wi & 1) ? make_uint2(full.z, full.w) : make_uint2(full.x, full.y);
              }
#pragma unroll
              for (int st = 0; st < 2; ++st) {
                const uint32_t w0 = reinterpret_cast<const uint32_t*>(&wcur[st][0][q])[wi];
                const uint32_t w1 = reinterpret_cast<const uint32_t*>(&wcur[st][1][q])[wi];
                const uint32_t m0 = mult[st][0][0], m1 = mult[st][1][0];
                const uint32_t p0 = bf16x2_mul(((w0 << 4) & 0x07F007F0u) | ((w0 << 8) & 0x80008000u), m0);
                const uint32_t p1 = bf16x2_mul(((w0 >> 4) & 0x07F007F0u) | (w0 & 0x80008000u), m0);
                const uint32_t q0 = bf16x2_mul(((w1 << 4) & 0x07F007F0u) | ((w1 << 8) & 0x80008000u), m1);
                const uint32_t q1 = bf16x2_mul(((w1 >> 4) & 0x07F007F0u) | (w1 & 0x80008000u), m1);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) mma_bf16_16816(acc[st][nt], p0, q0, p1, q1, bx[nt].x, bx[nt].y);
              }
            }
          }
        }
        if (it + 1 < n_it) {
#pragma unroll
          for (int st = 0; st < 2; ++st)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              wcur[st][h][0] = wnxt[st][h][0];
              wcur[st][h][1] = wnxt[st][h][1];
              scur[st][h] = snxt[st][h];
            }
        }
      }
    }

    // epilogue: acc[st][nt][i]: row = (i < 2 ? r : r + 8) of the stream, token = t_base + nt * 8 + 2 c + (i & 1)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int t = t_base + nt * 8 + 2 * c + (i & 1);
        if (t >= n) continue;
        const int h = i >> 1;
        const int dst = row0 + t;
        if constexpr (EPI == EPI_SILU_MUL) {
          if (!rok[0][h]) continue;
          const float g = round_bf16(acc[0][nt][i]), u = round_bf16(acc[1][nt][i]);
          const float sg = g / (1.0f + expf(-g));
          a.act_out[(long long)dst * a.act_rows + rows_l[0][h]] = __float2bfloat16_rn(sg * u);
        } else {
#pragma unroll
          for (int st = 0; st < 2; ++st) {
            if (!rok[st][h]) continue;
            const int row = rows_l[st][h];
            float v = acc[st][nt][i];
            if constexpr (FMT == W_FP8ROW) v *= reinterpret_cast<const float*>(sp[st])[row];
            if constexpr (FMT == W_NVFP4) v *= a.tensor_scale ? a.tensor_scale[0] : 1.f;
            if constexpr (EPI == EPI_ROW_SCALE) {
              v *= a.rw_row[dst];
              if (a.f_out) a.f_out[(long long)dst * a.out_stride + row] = v;
              else a.b_out[(long long)dst * a.out_stride + row] = __float2bfloat16_rn(v);
            } else if constexpr (EPI == EPI_SHARED_DOWN) {
              const float sig = 1.0f / (1.0f + expf(-a.gate[dst]));
              const float res = __bfloat162float(a.resid[(long long)dst * a.out_stride + row]);
              a.b_out[(long long)dst * a.out_stride + row] = __float2bfloat16_rn(res + v * sig);
            } else {
              if (a.bias) v += a.bias[row];
              if (a.row_div) v = round_bf16(v) / a.row_div[dst];
              if (a.resid2) v = round_bf16(v) + __bfloat162float(a.resid2[(long long)dst * a.out_stride + row]);
              if (a.f_out) a.f_out[(long long)dst * a.out_stride + row] = v;
              else a.b_out[(long long)dst * a.out_stride + row] = __float2bfloat16_rn(v);
            }
          }
        }
      }
  }
}

template <int FMT, int NT>
constexpr int skinny_smem_bytes() {
  return NT * 8 * (SK_KC / 8 + WTraits<FMT>::PAD_UNITS) * 16;
}

}  // namespace q35
