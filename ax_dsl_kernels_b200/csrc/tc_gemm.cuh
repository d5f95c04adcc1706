// Block-scaled tensor-core GEMM for the MoE block (sm_100a): out[token, row] = sum_k W[row, k] * x[token, k] with
//   W  : MXFP4 in HBM (E2M1 pairs + E8M0 per 32), fed to tcgen05.mma kind::mxf8f6f4 as the 128-row A operand straight
//        from TMA (CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B unpacks the nibbles into the padded shared-memory form),
//        its E8M0 scales copied smem -> tensor memory with tcgen05.cp;
//   x  : bf16 activations split into two E4M3 terms with UE8M0 block-32 scales (x = hi + lo exactly up to 2^-9 of
//        the block maximum), both terms columns of the B operand; the epilogue adds the two accumulator columns.
// Why two terms: the reference multiplies bf16 activations by the dequantised weights (golden
// models/qwen35_2b/whole/src/q35_moe.py:235-238); a single E4M3 term misses the 2e-2 tolerance by a factor 6.
//
// Work item = (group, 128-row weight tile, NB-token tile).  One CTA of 192 threads per (group, row tile): warp 0
// issues TMA, warp 1 owns tensor memory and issues the MMAs, warps 2-5 gather scale factors and run the epilogue.
// 4-stage mbarrier ring, K = 128 per stage (4 MMAs of K = 32), accumulators [128 lanes x 2 NB columns] in TMEM.
#pragma once
#include "tc_ptx.cuh"

namespace q35 {

enum : int { TC_EPI_SILU_MUL = 0, TC_EPI_ROW_SCALE = 1, TC_EPI_SHARED_DOWN = 2, TC_EPI_PLAIN = 3 };

struct TcArgs {
  // groups: nullptr g_n = one dense group of n_dense rows on plane 0
  const int* g_expert; const int* g_n; const int* g_row0;
  int n_dense, n_planes;
  int K;                    // contraction length, multiple of 128
  int plane_rows[2];        // rows per expert plane in each half's weight tensor map (y = plane * plane_rows + row)
  int roff[2];              // row offset of each 64-row half inside its matrix
  int lim[2];               // first invalid row of each half
  int tile_rows;            // rows a tile advances by (64: gate/up pairing, 128: plain matrix)
  const uint8_t* sw[2];     // E8M0 weight scales [rows, K/32] of each half
  long long s_plane;        // bytes between expert planes in sw
  const uint8_t* sfh; const uint8_t* sfl;  // activation scales [R, K/32] of the hi / lo term
  int total_rows;           // R: rows of the quantised activation planes
  // epilogue
  int act_rows;             // TC_EPI_SILU_MUL: row stride of act_out
  __nv_bfloat16* act_out;
  float* f_out; __nv_bfloat16* b_out; int out_stride;
  const float* rw_row; const __nv_bfloat16* resid; const float* gate; const float* bias;
  int* status;
};

template <int NB>
struct TcCfg {
  static constexpr int STAGES = 4;
  static constexpr int N = 2 * NB;                         // MMA N: hi columns then lo columns
  static constexpr int A_BYTES = 128 * 128;                // 128 rows x 128 unpacked FP4 bytes
  static constexpr int B_BYTES = N * 128;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  // bytes the TMA unit reports per stage: the FP4 loads count their PACKED source bytes (128 rows x 64 B), measured on
  // B200: with the unpacked size the barrier never completes
  static constexpr int STAGE_TX = 128 * 64 + B_BYTES;
  static constexpr int TMEM_COLS = (N + 8) <= 32 ? 32 : (N + 8) <= 64 ? 64 : (N + 8) <= 128 ? 128 : 256;
  static constexpr int SFA_COL = N, SFB_COL = N + 4;
  static constexpr int smem_bytes(int K) {                 // + 1024 for manual alignment
    return 1024 + STAGES * STAGE_BYTES + (K / 128) * 1024 + 256;
  }
};

template <int NB, int EPI>
__global__ void __launch_bounds__(192) tc_gemm_kernel(const __grid_constant__ CUtensorMap wmap0,
                                                      const __grid_constant__ CUtensorMap wmap1,
                                                      const __grid_constant__ CUtensorMap xmap_hi,
                                                      const __grid_constant__ CUtensorMap xmap_lo, const TcArgs a) {
  using C = TcCfg<NB>;
  using namespace tc;
  extern __shared__ uint8_t smem_raw[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int grp = blockIdx.y, tile = blockIdx.x;
  int n, plane, row0;
  if (a.g_n) {
    n = a.g_n[grp]; plane = a.g_expert[grp]; row0 = a.g_row0[grp];
    if (plane < 0 || plane >= a.n_planes) {
      if (tid == 0 && n > 0) atomicOr(a.status, DS_BAD_EXPERT);
      n = 0;
    }
  } else {
    n = a.n_dense; plane = 0; row0 = 0;
  }
  if (n <= 0) return;

  const int KS = a.K / 128;
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sgen = smem_raw + (sbase - smem_u32(smem_raw));
  const uint32_t s_stage = sbase;
  const uint32_t s_atomA = sbase + C::STAGES * C::STAGE_BYTES;
  const uint32_t s_atomB = s_atomA + KS * 512;
  const uint32_t s_bar = s_atomB + KS * 512;                  // full[4], empty[4], tmem_full
  uint32_t* g_atomA = reinterpret_cast<uint32_t*>(sgen + C::STAGES * C::STAGE_BYTES);
  uint32_t* g_atomB = g_atomA + KS * 128;
  volatile uint32_t* g_slot = reinterpret_cast<volatile uint32_t*>(sgen + C::STAGES * C::STAGE_BYTES + KS * 1024 + 128);
  const uint32_t s_slot = s_bar + 128;
  auto full_bar = [&](int s) { return s_bar + 8 * s; };
  auto empty_bar = [&](int s) { return s_bar + 32 + 8 * s; };
  const uint32_t tfull_bar = s_bar + 64;

  const int rowh[2] = {tile * a.tile_rows + a.roff[0], tile * a.tile_rows + a.roff[1]};

  if (tid == 0) {
    for (int s = 0; s < C::STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    mbar_init(tfull_bar, 1);
    fence_barrier_init();
    tma_prefetch_desc(&wmap0); tma_prefetch_desc(&wmap1); tma_prefetch_desc(&xmap_hi); tma_prefetch_desc(&xmap_lo);
  }
  if (warp == 1) { tmem_alloc(s_slot, C::TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *g_slot;

  // weight scale atoms: word (row r = r0 + 32 r1, stage ks) -> atomA[ks][r0 * 4 + r1], the 32 x 16-byte block that
  // tcgen05.cp replicates over the four lane quadrants
  {
    const int chunks = a.K / 32 / 16;  // 16-byte chunks per scale row (16 k-blocks = 4 stages each)
    for (int idx = tid; idx < 128 * chunks; idx += 192) {
      const int r = idx / chunks, ch = idx % chunks;
      const int h = r >> 6;
      const int row = rowh[h] + (r & 63);
      uint4 v = make_uint4(0x7f7f7f7fu, 0x7f7f7f7fu, 0x7f7f7f7fu, 0x7f7f7f7fu);
      if (row < a.lim[h])
        v = *reinterpret_cast<const uint4*>(a.sw[h] + (long long)plane * a.s_plane + (long long)row * (a.K / 32) + ch * 16);
      const int w = (r & 31) * 4 + (r >> 5);
      g_atomA[(ch * 4 + 0) * 128 + w] = v.x; g_atomA[(ch * 4 + 1) * 128 + w] = v.y;
      g_atomA[(ch * 4 + 2) * 128 + w] = v.z; g_atomA[(ch * 4 + 3) * 128 + w] = v.w;
    }
  }

  uint32_t it = 0;  // k-stages issued so far (ring position), identical in every role
  int item = 0;
  for (int t0 = 0; t0 < n; t0 += NB, ++item) {
    // activation scale atoms of this token tile: columns [0, NB) = hi term, [NB, 2 NB) = lo term
    {
      const int chunks = a.K / 32 / 16;
      for (int idx = tid; idx < C::N * chunks; idx += 192) {
        const int col = idx / chunks, ch = idx % chunks;
        const int t = t0 + (col < NB ? col : col - NB);
        const int row = row0 + t;
        uint4 v = make_uint4(0x7f7f7f7fu, 0x7f7f7f7fu, 0x7f7f7f7fu, 0x7f7f7f7fu);
        if (t < n && row < a.total_rows)
          v = *reinterpret_cast<const uint4*>((col < NB ? a.sfh : a.sfl) + (long long)row * (a.K / 32) + ch * 16);
        const int w = (col & 31) * 4 + (col >> 5);
        g_atomB[(ch * 4 + 0) * 128 + w] = v.x; g_atomB[(ch * 4 + 1) * 128 + w] = v.y;
        g_atomB[(ch * 4 + 2) * 128 + w] = v.z; g_atomB[(ch * 4 + 3) * 128 + w] = v.w;
      }
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    if (warp == 0) {
      if (elect_one()) {
        for (int ks = 0; ks < KS; ++ks) {
          const uint32_t s = (it + ks) % C::STAGES, ph = ((it + ks) / C::STAGES) & 1;
          if (!mbar_wait(empty_bar(s), ph ^ 1)) { atomicOr(a.status, DS_WAIT_TIMEOUT | 0x10); break; }
          mbar_expect_tx(full_bar(s), C::STAGE_TX);
          const uint32_t sa = s_stage + s * C::STAGE_BYTES, sb = sa + C::A_BYTES;
          tma_load_2d(sa, &wmap0, full_bar(s), ks * 128, plane * a.plane_rows[0] + rowh[0]);
          tma_load_2d(sa + 8192, &wmap1, full_bar(s), ks * 128, plane * a.plane_rows[1] + rowh[1]);
          tma_load_2d(sb, &xmap_hi, full_bar(s), ks * 128, row0 + t0);
          tma_load_2d(sb + NB * 128, &xmap_lo, full_bar(s), ks * 128, row0 + t0);
        }
      }
      __syncwarp();
    } else if (warp == 1) {
      if (elect_one()) {
        bool ok = true;
        for (int ks = 0; ks < KS && ok; ++ks) {
          const uint32_t s = (it + ks) % C::STAGES, ph = ((it + ks) / C::STAGES) & 1;
          if (!mbar_wait(full_bar(s), ph)) { atomicOr(a.status, DS_WAIT_TIMEOUT | 0x20 | (ks << 8)); ok = false; break; }
          tc_fence_after();
          tc_cp_32x128b_warpx4(tmem + C::SFA_COL, smem_desc(s_atomA + ks * 512, 0, 128, 0));
          tc_cp_32x128b_warpx4(tmem + C::SFB_COL, smem_desc(s_atomB + ks * 512, 0, 128, 0));
          const uint32_t sa = s_stage + s * C::STAGE_BYTES, sb = sa + C::A_BYTES;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            tc_mma_mxf8f6f4(tmem, smem_desc(sa + k * 32, 16, 1024, 2), smem_desc(sb + k * 32, 16, 1024, 2),
                            idesc_mxf8f6f4(FMT_E2M1, FMT_E4M3, 128, C::N, k, k), tmem + C::SFA_COL,
                            tmem + C::SFB_COL, (ks | k) != 0);
          }
          tc_commit(empty_bar(s));
        }
        tc_commit(tfull_bar);  // also on failure: the epilogue's wait must not be left hanging
      }
      __syncwarp();
    } else {
      // epilogue warps 2..5 own lane quadrants (warp % 4): rows 32 q .. 32 q + 31 of the tile
      const int q = warp & 3;
      const bool ok = mbar_wait(tfull_bar, item & 1);
      if (!ok && lane == 0) atomicOr(a.status, DS_WAIT_TIMEOUT | 0x40);
      tc_fence_after();
      const int r = q * 32 + lane;        // row of the 128-row tile
      const int h = r >> 6;
      const int row = rowh[h] + (r & 63);
      const bool rvalid = row < a.lim[h];
      float* xch = reinterpret_cast<float*>(sgen);  // stage memory is free once the accumulator is complete
      for (int c0 = 0; c0 < NB; c0 += 16) {  // runs even after a timed-out wait: the named barriers below must pair up
        float hi[16], lo[16];
        tmem_ld_x16(tmem + (uint32_t(q * 32) << 16) + c0, hi);
        tmem_ld_x16(tmem + (uint32_t(q * 32) << 16) + NB + c0, lo);
#pragma unroll
        for (int j = 0; j < 16; ++j) hi[j] += lo[j];
        if constexpr (EPI == TC_EPI_SILU_MUL) {
          // rows 64..127 (up) hand their values to rows 0..63 (gate) through shared memory
          if (h == 1) {
#pragma unroll
            for (int j = 0; j < 16; ++j) xch[(c0 + j) * 64 + (r & 63)] = hi[j];
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (h == 0) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int t = t0 + c0 + j;
              if (t < n && rvalid) {
                const float g = round_bf16(hi[j]), u = round_bf16(xch[(c0 + j) * 64 + r]);
                a.act_out[(long long)(row0 + t) * a.act_rows + row] = __float2bfloat16_rn(g / (1.0f + expf(-g)) * u);
              }
            }
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int t = t0 + c0 + j;
            if (t >= n || !rvalid) continue;
            const long long dst = row0 + t;
            float v = hi[j];
            if constexpr (EPI == TC_EPI_ROW_SCALE) {
              v *= a.rw_row[dst];
              if (a.f_out) a.f_out[dst * a.out_stride + row] = v;
              else a.b_out[dst * a.out_stride + row] = __float2bfloat16_rn(v);
            } else if constexpr (EPI == TC_EPI_SHARED_DOWN) {
              const float sig = 1.0f / (1.0f + expf(-a.gate[dst]));
              const float res = __bfloat162float(a.resid[dst * a.out_stride + row]);
              a.b_out[dst * a.out_stride + row] = __float2bfloat16_rn(res + v * sig);
            } else {
              if (a.bias) v += a.bias[row];
              if (a.f_out) a.f_out[dst * a.out_stride + row] = v;
              else a.b_out[dst * a.out_stride + row] = __float2bfloat16_rn(v);
            }
          }
        }
      }
    }
    it += KS;
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
  }
  if (warp == 1) tmem_dealloc(tmem, C::TMEM_COLS);
}

}  // namespace q35
