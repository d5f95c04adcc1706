// Host-side interface of the block-scaled tensor-core GEMM (tc_gemm.cu), shared with the MoE launchers.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace q35 {

// 2D row-major tensor [rows, cols] of bytes (fp4 = false) or packed FP4 codes (fp4 = true: cols counts codes, the
// pitch is in bytes) with a [box_rows, 128-element] box and 128-byte swizzle; cached per (device, address, shape)
int tc_make_map(CUtensorMap* m, bool fp4, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch_bytes,
                uint32_t box_rows, const char* what);

struct TcArgs;

struct TcWeights {            // the two 64-row halves of a tile may come from different matrices (gate / up)
  const uint8_t* w[2];        // packed FP4 [rows_total, K/2]
  uint64_t rows_total[2];     // rows of each matrix over all expert planes
};

struct TcQuant {              // activations as two E4M3 terms + UE8M0 block-32 scales, rows in destination order
  uint8_t *qh, *ql;           // [R, K]
  uint8_t *sh, *sl;           // [R, K/32]
  int R, K;
};

int64_t tc_quant_bytes(int64_t R, int64_t K);
TcQuant tc_quant_carve(uint8_t* base, int64_t R, int64_t K);
// src (optional): row r of the result quantises x[src[r]]; ids outside [0, x_rows) read row 0
int tc_quantize(const __nv_bfloat16* x, int x_stride, const int* src, int x_rows, int R, int K, const TcQuant& q,
                cudaStream_t stream);

// active[0] = number of groups with rows, active[1 ..] = their indices; `active` holds groups + 1 ints
int tc_build_active(const int* g_n, int groups, int* active, cudaStream_t stream);

// out[t, n] = x[t, :] . dequant(w[n, :]) on the tensor cores, the epilogue of the `linear` role:
// v = acc (* s[n] for FP8 per-row) + bias[n]; with row_div: v = bf16(v) / row_div[t]; with resid2: v = bf16(v) + resid2[t, n]
struct TcLinear {
  const void* w;      // [N, K/2] MXFP4 pairs (fmt 0) or [N, K] E4M3 (fmt 1, 2)
  const void* s;      // E8M0 [N, K/32] (fmt 0, 1) or fp32 [N] (fmt 2)
  int fmt;            // 0 MXFP4, 1 MXFP8, 2 FP8 with per-row scales
  const float* bias; const float* row_div; const __nv_bfloat16* resid2;
  float* f_out; __nv_bfloat16* b_out;   // one of the two
};
// K a multiple of 128; qws = tc_linear_bytes(T, N, K) bytes of scratch (quantised activations + split-K planes)
int64_t tc_linear_bytes(int64_t T, int64_t N, int64_t K);
int tc_linear(const __nv_bfloat16* x, int64_t T, int64_t N, int64_t K, const TcLinear& p, uint8_t* qws,
              cudaStream_t stream);

// the same product with the weight's rows cut into up to 8 consecutive segments, each written to a tensor of its own
// ([T, rows of the segment], bf16 or fp32): several projections of one input as ONE quantisation and ONE pass over a
// row-concatenated weight.  Decode-sized T only (the sums always go through the fp32 planes of the split-K form).
struct TcSegments {
  int n;
  int n0[9];       // segment i = weight rows [n0[i], n0[i + 1])
  void* out[8];
  int f32[8];      // 1: out[i] is fp32, 0: bf16
};
int64_t tc_linear_multi_bytes(int64_t T, int64_t N, int64_t K);
int tc_linear_multi(const __nv_bfloat16* x, int64_t T, int64_t N, int64_t K, const TcLinear& p, const TcSegments& segs,
                    uint8_t* qws, cudaStream_t stream);

template <int EPI>
int tc_launch(const TcWeights& w, const TcQuant& q, TcArgs a, int nb, int tiles, int groups, cudaStream_t stream);

}  // namespace q35
