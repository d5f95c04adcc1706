// Paged flash-attention prefill: T new tokens per sequence attend causally to the sequence's paged KV cache, which
// already holds their own K / V rows (written with attn.kv_write / attn.kv_write_rows).
//
// Reference: paged_flash_attention (models/qwen35_35b_a3b/sgl/python/sgl_kernel_axera/attention/flash_attn.py:
// 471-610: history pages plus the causal current tile) and attn_layer_prefill
// (models/qwen35_2b/whole/src/q35_prefill.py:250-318: G * P query rows per KV head against the cache with a causal
// mask).  Same arithmetic as the decode golden with a causal mask: softmax(q k^T * scale) v per query head.
//
// One CTA = 16 query tokens x the (up to 8) query heads of one KV head = 128 rows of the score tile, 8 warps of 16
// rows, so a K / V tile fetched once serves all heads of the group.  Keys stream in tiles of 64 through a 2-stage
// cp.async ring (XOR-swizzled rows); S = Q K^T and O += P V on mma.sync bf16 with fp32 accumulation and an online
// softmax in the log2 domain.  Tensor-bound for long prompts (4 T^2 / 2 * HQ * D flop against T * 2 KB of KV).
//
// FP8 cache (E4M3 rows holding x * 8, or x / scale_h with a per-head scale; models/qwen38_27b/prefill/
// sgl_kv8_kvf8.patch, models/qwen38_27b/decode/q35_group.py:244-249): a tile's bytes land in a staging ring, are
// expanded to bf16 (exact: E4M3 has 3 mantissa bits) into the tile the MMAs read, the K scale is folded into the
// softmax scale and the V scale into the final normalisation -- the reference's "constant MX scale on K, block
// weighted values x 1 / 8".  The rows of this call are quantised as they are written, so the call's own tokens are
// attended to in their stored precision, as the reference's cache reads do.
#include "abi.h"
#include "common.cuh"

namespace q35 {

constexpr int PF_TOK = 16;    // query tokens per CTA
constexpr int PF_KEYS = 64;   // keys per tile
constexpr float PF_LOG2E = 1.4426950408889634f;

struct PrefillArgs {
  const __nv_bfloat16* q;      // [Ttot, HQ, D]
  const void* cache;           // [pages, 2, P, HKV, D] bf16 or e4m3
  const float* kv_scale;       // FP8 cache: [2, HKV] per-head scales, or null = the constant form (stored x * 8)
  const __nv_bfloat16* row_scale;  // int8 cache: [pages, 2, P, HKV], one scale per cached row and head
  const int* qo_indptr;        // [B + 1] token ranges of the sequences inside q
  const int* indptr; const int* indices; const int* last_page_len;  // page table incl. the new tokens
  const float* sm_scale;
  __nv_bfloat16* out;          // [Ttot, HQ, D]
  int B, HQ, HKV, G, P, num_pages, n_indices;
  int* status;
};

// KVF: 0 bf16 cache, 1 FP8 E4M3, 2 int8 with a bf16 scale per row and head (kv_quant_row,
// models/qwen38_27b/decode/q35_group.py:198-222): the one-byte formats share the staging ring; int8 rows become
// bf16(int8 x scale) element by element, the reference's page dequantisation, on their way into the MMA tile.
template <int D, int KVF>
__global__ void __launch_bounds__(256, 1) attn_prefill_kernel(const PrefillArgs a) {
  constexpr bool FP8 = KVF != 0;
  constexpr int ROWB = D * 2, CPR = ROWB / 16, TILE_BYTES = PF_KEYS * ROWB;
  // FP8: [K tile | V tile] bf16 work tiles, then two staging stages of raw bytes (K rows then V rows, D bytes each)
  constexpr int RAWB = D, RCPR = RAWB / 16, RAW_TILE = PF_KEYS * RAWB;
  extern __shared__ __align__(128) uint8_t smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int r = lane >> 2, c = lane & 3;
  const int b = blockIdx.z, kvh = blockIdx.y;
  const int q0 = a.qo_indptr[b], q1 = a.qo_indptr[b + 1];
  const int tq = q1 - q0;                       // new tokens of this sequence
  const int tok0 = blockIdx.x * PF_TOK;
  if (tok0 >= tq) return;
  const int np = a.indptr[b + 1] - a.indptr[b];
  int kv_len = np > 0 ? (np - 1) * a.P + a.last_page_len[b] : 0;
  if (kv_len < tq || a.indptr[b + 1] > a.n_indices) {  // the cache must already contain the new tokens
    if (tid == 0) atomicOr(a.status, DS_BAD_PAGE);
    kv_len = max(kv_len, tq);
    return;
  }
  const int hist = kv_len - tq;                 // tokens before this call
  const int page0 = a.indptr[b];
  const float k_deq = KVF != 1 ? 1.f : a.kv_scale ? a.kv_scale[kvh] : 0.125f;
  const float v_deq = KVF != 1 ? 1.f : a.kv_scale ? a.kv_scale[a.HKV + kvh] : 0.125f;
  const float scale_log2 = (a.sm_scale ? a.sm_scale[0] : rsqrtf(float(D))) * PF_LOG2E * k_deq;

  // this thread's two rows: row m = warp * 16 + r (+ 8); token = m / 8, head = m % 8
  const int m0 = warp * 16 + r, m1 = m0 + 8;
  const int tk0 = tok0 + (m0 >> 3), tk1 = tok0 + (m1 >> 3);
  const int h0 = m0 & 7, h1 = m1 & 7;  // equal (r and r + 8 differ by one token), kept for clarity
  const bool v0 = tk0 < tq && h0 < a.G, v1 = tk1 < tq && h1 < a.G;
  const int pos0 = hist + tk0, pos1 = hist + tk1;  // last visible key of each row

  // Q fragments (A operand): a0 = (row m0, d 2c..), a1 = (row m1, ..), a2 = (m0, d + 8), a3 = (m1, d + 8)
  uint32_t qf[D / 16][4];
  {
    const __nv_bfloat16* p0 = a.q + (size_t(q0 + min(tk0, tq - 1)) * a.HQ + kvh * a.G + min(h0, a.G - 1)) * D;
    const __nv_bfloat16* p1 = a.q + (size_t(q0 + min(tk1, tq - 1)) * a.HQ + kvh * a.G + min(h1, a.G - 1)) * D;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      qf[ks][0] = v0 ? *reinterpret_cast<const uint32_t*>(p0 + ks * 16 + 2 * c) : 0u;
      qf[ks][1] = v1 ? *reinterpret_cast<const uint32_t*>(p1 + ks * 16 + 2 * c) : 0u;
      qf[ks][2] = v0 ? *reinterpret_cast<const uint32_t*>(p0 + ks * 16 + 8 + 2 * c) : 0u;
      qf[ks][3] = v1 ? *reinterpret_cast<const uint32_t*>(p1 + ks * 16 + 8 + 2 * c) : 0u;
    }
  }
  float o[D / 8][4];
#pragma unroll
  for (int nt = 0; nt < D / 8; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f;
  float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.f, 0.f};

  const int last_pos = hist + min(tok0 + PF_TOK, tq) - 1;  // last key any row of this CTA may see
  const int n_tiles = last_pos / PF_KEYS + 1;
  const size_t row_stride = size_t(a.HKV) * (FP8 ? RAWB : ROWB);
  const uint8_t* cbase = reinterpret_cast<const uint8_t*>(a.cache);
  const uint32_t sbase = smem_u32(smem);

  auto issue = [&](int t) {
    if (t < n_tiles) {
      const int kk = t * PF_KEYS;
      const int pl = kk / a.P, ro = kk % a.P;
      int page = a.indices[page0 + min(pl, np - 1)];
      if (page < 0 || page >= a.num_pages) {
        if (tid == 0) atomicOr(a.status, DS_BAD_PAGE);
        page = 0;
      }
      const uint8_t* kb = cbase + ((size_t(page) * 2 + 0) * a.P + ro) * row_stride + size_t(kvh) * (FP8 ? RAWB : ROWB);
      const uint8_t* vb = cbase + ((size_t(page) * 2 + 1) * a.P + ro) * row_stride + size_t(kvh) * (FP8 ? RAWB : ROWB);
      if constexpr (FP8) {
        const uint32_t st = sbase + 2 * TILE_BYTES + (t & 1) * 2 * RAW_TILE;
        for (int idx = tid; idx < PF_KEYS * RCPR; idx += 256) {
          const int key = idx / RCPR, ch = idx % RCPR;
          cp_async_16(st + key * RAWB + ch * 16, kb + size_t(key) * row_stride + ch * 16);
          cp_async_16(st + RAW_TILE + key * RAWB + ch * 16, vb + size_t(key) * row_stride + ch * 16);
        }
      } else {
        const uint32_t st = sbase + (t & 1) * 2 * TILE_BYTES;
        for (int idx = tid; idx < PF_KEYS * CPR; idx += 256) {
          const int key = idx / CPR, ch = idx % CPR;
          const uint32_t off = key * ROWB + ((ch ^ (key & 7)) << 4);
          cp_async_16(st + off, kb + size_t(key) * row_stride + ch * 16);
          cp_async_16(st + TILE_BYTES + off, vb + size_t(key) * row_stride + ch * 16);
        }
      }
    }
    cp_async_commit();
  };

  issue(0);
  for (int t = 0; t < n_tiles; ++t) {
    issue(t + 1);
    cp_async_wait<1>();
    __syncthreads();
    const uint32_t sK = FP8 ? sbase : sbase + (t & 1) * 2 * TILE_BYTES, sV = sK + TILE_BYTES;
    const int kk = t * PF_KEYS;
    if constexpr (FP8) {  // raw bytes -> the swizzled bf16 tiles (16 bytes in, two 16-byte chunks out)
      const uint8_t* raw = smem + 2 * TILE_BYTES + (t & 1) * 2 * RAW_TILE;
      float* s_rs = reinterpret_cast<float*>(smem + 2 * TILE_BYTES + 4 * RAW_TILE);  // int8: [2][64] row scales
      if constexpr (KVF == 2) {
        if (tid < 2 * PF_KEYS) {  // this tile's K and V row scales; rows past the cached length count as 0
          const int kv = tid / PF_KEYS, key = tid % PF_KEYS, pos = kk + key;
          float sc = 0.f;
          if (pos < kv_len) {
            int page = a.indices[page0 + min(pos / a.P, np - 1)];
            if (page < 0 || page >= a.num_pages) page = 0;
            sc = __bfloat162float(a.row_scale[((size_t(page) * 2 + kv) * a.P + pos % a.P) * a.HKV + kvh]);
          }
          s_rs[tid] = sc;
        }
        __syncthreads();
      }
      for (int idx = tid; idx < 2 * PF_KEYS * RCPR; idx += 256) {
        const int kv = idx / (PF_KEYS * RCPR), rem = idx % (PF_KEYS * RCPR), key = rem / RCPR, ch = rem % RCPR;
        const uint4 in = *reinterpret_cast<const uint4*>(raw + kv * RAW_TILE + key * RAWB + ch * 16);
        const uint32_t w[4] = {in.x, in.y, in.z, in.w};
        uint32_t o8[8];
        if constexpr (KVF == 2) {
          // bf16(int8 x scale), exact: 0x4B000000 | (b ^ 0x80) is the float 2^23 + 128 + b; the fused multiply-add
          // leaves b x scale (a 15-bit product), one rounding to bf16 follows
          const float sc = s_rs[kv * PF_KEYS + key], off = -8388736.f * sc;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t xs = w[j] ^ 0x80808080u;
            const float f0 = __uint_as_float(__byte_perm(xs, 0x4B000000u, 0x7540));
            const float f1 = __uint_as_float(__byte_perm(xs, 0x4B000000u, 0x7541));
            const float f2 = __uint_as_float(__byte_perm(xs, 0x4B000000u, 0x7542));
            const float f3 = __uint_as_float(__byte_perm(xs, 0x4B000000u, 0x7543));
            o8[2 * j] = pack_bf16(fmaf(f0, sc, off), fmaf(f1, sc, off));
            o8[2 * j + 1] = pack_bf16(fmaf(f2, sc, off), fmaf(f3, sc, off));
          }
        } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2(__nv_fp8x2_storage_t(w[j] & 0xffffu), __NV_E4M3);
          const __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2(__nv_fp8x2_storage_t(w[j] >> 16), __NV_E4M3);
          const float2 fl = __half22float2(*reinterpret_cast<const __half2*>(&lo));
          const float2 fh = __half22float2(*reinterpret_cast<const __half2*>(&hi));
          o8[2 * j] = pack_bf16(fl.x, fl.y);
          o8[2 * j + 1] = pack_bf16(fh.x, fh.y);
        }
        }
        const uint32_t dst = sK + kv * TILE_BYTES + key * ROWB;
        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst + (((2 * ch) ^ (key & 7)) << 4)), "r"(o8[0]),
                     "r"(o8[1]), "r"(o8[2]), "r"(o8[3]));
        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst + (((2 * ch + 1) ^ (key & 7)) << 4)), "r"(o8[4]),
                     "r"(o8[5]), "r"(o8[6]), "r"(o8[7]));
      }
      __syncthreads();
    }
    if (kk + PF_KEYS > kv_len) {  // rows past the cached length may hold anything (NaN bits): clear V there
      const int first = kv_len - kk;
      for (int idx = tid; idx < (PF_KEYS - first) * CPR; idx += 256) {
        const uint32_t addr = sV + (first + idx / CPR) * ROWB + ((idx % CPR) << 4);
        asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(addr), "r"(0u));
      }
      __syncthreads();
    }
    // S = Q K^T: 16 rows x 64 keys per warp
    float s[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
      for (int np2 = 0; np2 < 4; ++np2) {
        const int brow = np2 * 16 + (lane & 7) + ((lane >> 4) << 3);
        const int ch = 2 * ks + ((lane >> 3) & 1);
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(sK + brow * ROWB + ((ch ^ (brow & 7)) << 4), b0, b1, b2, b3);
        mma_bf16_16816(s[2 * np2], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b0, b1);
        mma_bf16_16816(s[2 * np2 + 1], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b2, b3);
      }
    }
    // causal mask, online softmax (rows m0: regs 0,1; m1: regs 2,3)
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int key = kk + nt * 8 + 2 * c + (i & 1);
        const int pos = (i >> 1) ? pos1 : pos0;
        s[nt][i] = key <= pos ? s[nt][i] * scale_log2 : -INFINITY;
        mx[i >> 1] = fmaxf(mx[i >> 1], s[nt][i]);
      }
    float alpha[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      const float mn = fmaxf(mrow[h], mx[h]);
      alpha[h] = mn == -INFINITY ? 1.f : exp2f(mrow[h] - mn);
      mrow[h] = mn;
    }
    // P stays in fp32 in the score registers and enters the P V product as TWO bf16 terms (p = hi + lo): a single
    // bf16 P carries 2^-9 of relative error into every output element -- on a row with few or peaked keys as much as
    // the output's own bf16 rounding step -- while the golden keeps the softmax in fp32.
    float ls[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      s[nt][0] = mrow[0] == -INFINITY ? 0.f : exp2f(s[nt][0] - mrow[0]);
      s[nt][1] = mrow[0] == -INFINITY ? 0.f : exp2f(s[nt][1] - mrow[0]);
      s[nt][2] = mrow[1] == -INFINITY ? 0.f : exp2f(s[nt][2] - mrow[1]);
      s[nt][3] = mrow[1] == -INFINITY ? 0.f : exp2f(s[nt][3] - mrow[1]);
      ls[0] += s[nt][0] + s[nt][1]; ls[1] += s[nt][2] + s[nt][3];
    }
    lrow[0] = lrow[0] * alpha[0] + ls[0];
    lrow[1] = lrow[1] * alpha[1] + ls[1];
    if (alpha[0] != 1.f || alpha[1] != 1.f) {
#pragma unroll
      for (int nt = 0; nt < D / 8; ++nt) {
        o[nt][0] *= alpha[0]; o[nt][1] *= alpha[0]; o[nt][2] *= alpha[1]; o[nt][3] *= alpha[1];
      }
    }
    // O += P V: A = P (score accumulators reused as fragments), B = V tile [key][d] read transposed
#pragma unroll
    for (int ks = 0; ks < PF_KEYS / 16; ++ks) {
      uint32_t ah[4], al[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {  // fragments a0..a3 = (tile 2ks: rows m0 | m1), (tile 2ks + 1: rows m0 | m1)
        const float x = s[2 * ks + (u >> 1)][2 * (u & 1)], y = s[2 * ks + (u >> 1)][2 * (u & 1) + 1];
        const float xh = round_bf16(x), yh = round_bf16(y);
        ah[u] = pack_bf16(xh, yh);
        al[u] = pack_bf16(x - xh, y - yh);
      }
      const int brow = ks * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
#pragma unroll
      for (int np2 = 0; np2 < D / 16; ++np2) {
        const int ch = 2 * np2 + (lane >> 4);
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(sV + brow * ROWB + ((ch ^ (brow & 7)) << 4), b0, b1, b2, b3);
        mma_bf16_16816(o[2 * np2], ah[0], ah[1], ah[2], ah[3], b0, b1);
        mma_bf16_16816(o[2 * np2 + 1], ah[0], ah[1], ah[2], ah[3], b2, b3);
        mma_bf16_16816(o[2 * np2], al[0], al[1], al[2], al[3], b0, b1);
        mma_bf16_16816(o[2 * np2 + 1], al[0], al[1], al[2], al[3], b2, b3);
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    lrow[h] += __shfl_xor_sync(0xffffffffu, lrow[h], 1);
    lrow[h] += __shfl_xor_sync(0xffffffffu, lrow[h], 2);
  }
  const float inv0 = lrow[0] > 0.f ? v_deq / lrow[0] : 0.f, inv1 = lrow[1] > 0.f ? v_deq / lrow[1] : 0.f;
  __nv_bfloat16* d0 = a.out + (size_t(q0 + tk0) * a.HQ + kvh * a.G + h0) * D;
  __nv_bfloat16* d1 = a.out + (size_t(q0 + tk1) * a.HQ + kvh * a.G + h1) * D;
#pragma unroll
  for (int nt = 0; nt < D / 8; ++nt) {
    if (v0) *reinterpret_cast<uint32_t*>(d0 + nt * 8 + 2 * c) = pack_bf16(o[nt][0] * inv0, o[nt][1] * inv0);
    if (v1) *reinterpret_cast<uint32_t*>(d1 + nt * 8 + 2 * c) = pack_bf16(o[nt][2] * inv1, o[nt][3] * inv1);
  }
}

// attn.kv_write_rows: K / V rows of T new tokens per sequence into the paged cache at positions hist .. hist + T - 1
// (store_paged_kv for a prefill tile, flash_attn.py:53-84)
__global__ void attn_kv_write_rows_kernel(const __nv_bfloat16* __restrict__ k_new, const __nv_bfloat16* __restrict__ v_new,
                                          const int* __restrict__ qo_indptr, const int* __restrict__ indptr,
                                          const int* __restrict__ indices, const int* __restrict__ last_page_len,
                                          void* cache, const float* kv_scale, __nv_bfloat16* row_scale, int fp8, int B,
                                          int HKV, int D, int P, int num_pages, int* status) {
  const int tok = blockIdx.x;  // global token index
  int b = 0;
  while (b + 1 < B && qo_indptr[b + 1] <= tok) ++b;
  if (tok < qo_indptr[b] || tok >= qo_indptr[b + 1]) return;
  const int tq = qo_indptr[b + 1] - qo_indptr[b];
  const int np = indptr[b + 1] - indptr[b];
  const int kv_len = np > 0 ? (np - 1) * P + last_page_len[b] : 0;
  const int pos = kv_len - tq + (tok - qo_indptr[b]);
  if (pos < 0 || pos / P >= np) { if (threadIdx.x == 0) atomicOr(status, DS_BAD_PAGE); return; }
  const int page = indices[indptr[b] + pos / P];
  if (page < 0 || page >= num_pages) { if (threadIdx.x == 0) atomicOr(status, DS_BAD_PAGE); return; }
  const int n = HKV * D;
  const size_t krow = ((size_t(page) * 2 + 0) * P + pos % P) * n, vrow = ((size_t(page) * 2 + 1) * P + pos % P) * n;
  if (row_scale) {  // int8 rows with a bf16 scale per row and head: the arithmetic of attn.kv_write's int8 form
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int8_t* c8 = static_cast<int8_t*>(cache);
    for (int item = warp; item < 2 * HKV; item += blockDim.x >> 5) {
      const int kv = item / HKV, h = item % HKV;
      const __nv_bfloat16* src = (kv ? v_new : k_new) + size_t(tok) * n + size_t(h) * D;
      float amax = 0.f;
      for (int i = lane; i < D; i += 32) amax = fmaxf(amax, fabsf(__bfloat162float(src[i])));
      for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      amax = fmaxf(amax, round_bf16(1e-5f));
      const float sc = round_bf16(amax * round_bf16(1.f / 127.f)), inv = round_bf16(1.f / sc);
      const size_t row = (size_t(page) * 2 + kv) * P + pos % P;
      for (int i = lane; i < D; i += 32) {
        const float qv = rintf(round_bf16(__bfloat162float(src[i]) * inv));
        c8[(row * HKV + h) * D + i] = int8_t(fminf(fmaxf(qv, -127.f), 127.f));
      }
      if (lane == 0) row_scale[row * HKV + h] = __float2bfloat16_rn(sc);
    }
    return;
  }
  if (fp8) {  // e4m3(x * 8), or e4m3(x / scale_h) with per-head scales: the arithmetic of attn.kv_write
    __nv_fp8_e4m3* c8 = static_cast<__nv_fp8_e4m3*>(cache);
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const float k = __bfloat162float(k_new[size_t(tok) * n + i]), v = __bfloat162float(v_new[size_t(tok) * n + i]);
      c8[krow + i] = __nv_fp8_e4m3(kv_scale ? k / kv_scale[i / D] : k * 8.f);  // a true division, as the golden's
      c8[vrow + i] = __nv_fp8_e4m3(kv_scale ? v / kv_scale[HKV + i / D] : v * 8.f);
    }
    return;
  }
  __nv_bfloat16* cb = static_cast<__nv_bfloat16*>(cache);
  for (int i = threadIdx.x * 8; i < n; i += blockDim.x * 8) {
    *reinterpret_cast<uint4*>(cb + krow + i) = *reinterpret_cast<const uint4*>(k_new + size_t(tok) * n + i);
    *reinterpret_cast<uint4*>(cb + vrow + i) = *reinterpret_cast<const uint4*>(v_new + size_t(tok) * n + i);
  }
}

template <int D, int KVF>
static int launch_prefill(const PrefillArgs& a, dim3 grid, cudaStream_t stream) {
  constexpr int smem = KVF ? 2 * PF_KEYS * D * 2 + 4 * PF_KEYS * D + 2 * PF_KEYS * 4 : 4 * PF_KEYS * D * 2;
  Q35_TRY(ensure_dynamic_smem(reinterpret_cast<const void*>(attn_prefill_kernel<D, KVF>), smem));
  attn_prefill_kernel<D, KVF><<<grid, 256, smem, stream>>>(a);
  Q35_CUDA_LAUNCH_CHECK("attn.paged_prefill");
  return 0;
}

int run_attn_paged_prefill(Call& c) {
  Tensor q, cache, qo, indptr, indices, lpl, scale, kvs, kn, vn, out;
  Q35_TRY(c.get("q", M(Q35_BF16), &q));
  Q35_TRY(c.get("paged_kv_cache", M(Q35_BF16) | M_FP8, &cache));
  Q35_TRY(c.get("qo_indptr", M(Q35_I32), &qo));
  Q35_TRY(c.get("indptr", M(Q35_I32), &indptr));
  Q35_TRY(c.get("indices", M(Q35_I32), &indices));
  Q35_TRY(c.get("last_page_len", M(Q35_I32), &lpl));
  Q35_TRY(c.get("sm_scale", M(Q35_F32), &scale, false));
  Q35_TRY(c.get("kv_scale", M(Q35_F32), &kvs, false));
  Q35_TRY(c.get("k_new", M(Q35_BF16), &kn, false));
  Q35_TRY(c.get("v_new", M(Q35_BF16), &vn, false));
  Q35_TRY(c.get("out", M(Q35_BF16), &out));
  Q35_REQUIRE(q.nd == 3 && cache.nd == 5 && cache.s[1] == 2, Q35_ERR_SHAPE,
              "attn.paged_prefill: q [T, HQ, D], paged_kv_cache [pages, 2, P, HKV, D]");
  const int64_t T = q.s[0], HQ = q.s[1], D = q.s[2], P = cache.s[2], HKV = cache.s[3], B = qo.numel() - 1;
  const bool fp8 = cache.dtype != Q35_BF16;
  Q35_REQUIRE(cache.s[4] == D && HKV > 0 && HQ % HKV == 0 && HQ / HKV <= 8, Q35_ERR_UNSUPPORTED,
              "attn.paged_prefill: at most 8 query heads per KV head");
  Q35_REQUIRE(D == 128 || D == 256, Q35_ERR_UNSUPPORTED, "attn.paged_prefill: head_dim must be 128 or 256");
  Q35_REQUIRE(P % 64 == 0, Q35_ERR_UNSUPPORTED, "attn.paged_prefill: page size must be a multiple of 64");
  Q35_REQUIRE(B >= 1 && indptr.numel() == B + 1 && lpl.numel() >= B && out.numel() == q.numel(), Q35_ERR_SHAPE,
              "attn.paged_prefill: qo_indptr / indptr [B+1], last_page_len [B], out like q");
  Q35_REQUIRE(kn.present == vn.present && (!kn.present || (kn.numel() == T * HKV * D && vn.numel() == T * HKV * D)),
              Q35_ERR_SHAPE, "attn.paged_prefill: k_new / v_new [T, HKV, D]");
  Q35_REQUIRE(!kvs.present || (fp8 && kvs.numel() == 2 * HKV), Q35_ERR_SHAPE,
              "attn.paged_prefill: kv_scale [2, HKV] goes with an FP8 cache");
  Tensor rsc;
  Q35_TRY(c.get("paged_kv_scale", M(Q35_BF16), &rsc, false));
  Q35_REQUIRE(!rsc.present || (fp8 && !kvs.present && rsc.numel() == cache.s[0] * 2 * P * HKV), Q35_ERR_SHAPE,
              "attn.paged_prefill: paged_kv_scale [pages, 2, P, HKV] bf16 goes with an int8 cache (bound as bytes)");
  c.ws_need = 0;
  if (c.dry || T == 0) return 0;
  Q35_REQUIRE(aligned16(q.p) && aligned16(cache.p) && aligned16(out.p), Q35_ERR_ALIGN, "attn.paged_prefill: alignment");
  if (kn.present) {
    attn_kv_write_rows_kernel<<<unsigned(T), 128, 0, c.stream>>>(
        kn.as<__nv_bfloat16>(), vn.as<__nv_bfloat16>(), qo.as<int>(), indptr.as<int>(), indices.as<int>(),
        lpl.as<int>(), cache.p, kvs.present ? kvs.as<float>() : nullptr,
        rsc.present ? rsc.as<__nv_bfloat16>() : nullptr, fp8, int(B), int(HKV), int(D), int(P), int(cache.s[0]),
        device_status_ptr());
    Q35_CUDA_LAUNCH_CHECK("attn.kv_write_rows");
  }
  PrefillArgs a{};
  a.q = q.as<__nv_bfloat16>(); a.cache = cache.p; a.qo_indptr = qo.as<int>();
  a.kv_scale = kvs.present ? kvs.as<float>() : nullptr;
  a.indptr = indptr.as<int>(); a.indices = indices.as<int>(); a.last_page_len = lpl.as<int>();
  a.sm_scale = scale.present ? scale.as<float>() : nullptr;
  a.out = out.as<__nv_bfloat16>();
  a.B = int(B); a.HQ = int(HQ); a.HKV = int(HKV); a.G = int(HQ / HKV); a.P = int(P);
  a.num_pages = int(cache.s[0]); a.n_indices = int(indices.numel());
  a.status = device_status_ptr();
  // the longest sequence is not known on the host: the grid covers T tokens for every sequence, CTAs past a
  // sequence's own length leave at once
  const dim3 grid{unsigned((T + PF_TOK - 1) / PF_TOK), unsigned(HKV), unsigned(B)};
  if (rsc.present) {
    a.row_scale = rsc.as<__nv_bfloat16>();
    return D == 256 ? launch_prefill<256, 2>(a, grid, c.stream) : launch_prefill<128, 2>(a, grid, c.stream);
  }
  if (D == 256) return fp8 ? launch_prefill<256, 1>(a, grid, c.stream) : launch_prefill<256, 0>(a, grid, c.stream);
  return fp8 ? launch_prefill<128, 1>(a, grid, c.stream) : launch_prefill<128, 0>(a, grid, c.stream);
}

}  // namespace q35
