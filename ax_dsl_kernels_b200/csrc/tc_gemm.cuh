// Block-scaled tensor-core GEMM for the MoE block (sm_100a): out[token, row] = sum_k W[row, k] * x[token, k] with
//   W  : MXFP4 in HBM (E2M1 pairs + E8M0 per 32), fed to tcgen05.mma kind::mxf8f6f4 as the 128-row A operand straight
//        from TMA (CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B unpacks the nibbles into the padded shared-memory form),
//        its E8M0 scales copied smem -> tensor memory with tcgen05.cp;
//   x  : bf16 activations split into two E4M3 terms with UE8M0 block-32 scales (x = hi + lo exactly up to 2^-9 of
//        the block maximum), both terms columns of the B operand; the epilogue adds the two accumulator columns.
// Why two terms: the reference multiplies bf16 activations by the dequantised weights (golden
// models/qwen35_2b/whole/src/q35_moe.py:235-238); a single E4M3 term misses the 2e-2 tolerance by a factor 6.
//
// Work item = (group, 128-row weight tile, NB-token tile).  Persistent kernel (320 or 448 threads, two CTAs per SM for small
// token tiles), items dealt round-robin over the compacted list of non-empty groups.  Warp-specialised and decoupled:
//   warp 0    TMA producer: weight and activation tiles into a ring of stages (K = 128 per stage), running ahead
//             across item boundaries;
//   warp 1    owns tensor memory, copies the stage's scale blocks into TMEM (tcgen05.cp) and issues 4 MMAs of K = 32;
//   warps 2-5 epilogue: tcgen05.ld of a finished accumulator while the next item accumulates into the other buffer
//             (prefill-sized MoE tiles: a second epilogue group, warps 10-13, one group per accumulator buffer);
//   warps 6-9 gather the E8M0 scales from global memory into 32 x 16-byte blocks (the layout tcgen05.cp wants), four
//             stages (K = 512, 16 scale bytes of a row) at a time, in a two-deep ring of their own, with the loads of
//             four granules in flight in registers.  Measured alternatives, all slower: the same per stage (a proxy
//             fence and a barrier per stage in a serial chain, -15 %); scales written straight to tensor memory with
//             tcgen05.st (cheap by itself, but it leaves too few registers to keep enough loads in flight with two
//             CTAs per SM); asking the TMA unit to prefetch weight tiles into L2 ahead of the ring (-20 %).
//             Also measured and dropped: quantising the SiLU x up activation for the down projection inside this
//             kernel's epilogue instead of in a pass of its own made the decode step 18 us slower.
// Accumulators [128 lanes x 2 NB columns] are double-buffered; every hand-over is an mbarrier.  A stage carries only
// 8 KB of HBM bytes (the unpacked FP4 tile takes 16 KB of shared memory), so the ring is made as deep as shared memory
// allows.  Without the scale path the same pipeline streams weights at 6.3 TB/s; with it, 5.4 TB/s.
#pragma once
#include "tc_ptx.cuh"

namespace q35 {

enum : int { TC_EPI_SILU_MUL = 0, TC_EPI_ROW_SCALE = 1, TC_EPI_SHARED_DOWN = 2, TC_EPI_PLAIN = 3 };

struct TcArgs {
  // groups: nullptr g_n = one dense group of n_dense rows on plane 0
  const int* g_expert; const int* g_n; const int* g_row0;
  int n_dense, n_planes;
  int dense_rows;           // dense form: rows per virtual group (set by the launcher)
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
  // TC_EPI_PLAIN extras (the `linear` role): v = acc * row_scale[row] + bias[row]; then, when bound,
  // v = bf16(v) / row_div[token] and v = bf16(v) + resid2[token, row]
  const float* row_scale; const float* row_div; const __nv_bfloat16* resid2;
  int w_fp8;                // 0: weights are MXFP4 pairs; 1: E4M3 bytes (MXFP8 with E8M0 scales, or FP8 per-row: sw null)
  int a_fmt;                // set by the launcher from w_fp8: FMT_E2M1 or FMT_E4M3
  int stage_tx;             // bytes the TMA unit reports per stage (FP4 tiles count their packed bytes)
  const int* active; const int* n_active;  // compacted list of groups with rows (nullptr: dense)
  int n_tiles;              // row tiles per group
  // split K (dense launches whose row tiles alone leave most CTAs idle): the stages are cut into k_slices ranges of
  // slice_stages each, an item is (group, tile, slice), and every slice's fp32 sums go to its own plane of `part`
  // ([k_slices][rows of x][out_stride]) for a reduction kernel that also applies the epilogue
  int k_slices, slice_stages;
  int raw;                  // 1: raw sums to `part` even with one slice (the reduction kernel owns the epilogue)
  float* part; long long part_plane;
  int* status;
};

template <int NB>
struct TcCfg {
  static constexpr int N = 2 * NB;                         // MMA N: hi columns then lo columns
  static constexpr int A_BYTES = 128 * 128;                // 128 rows x 128 unpacked FP4 bytes
  static constexpr int B_BYTES = N * 128;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int SF_GRAN = 4;                        // stages per scale granule (16 scale bytes of a row)
  static constexpr int SF_RING = 2;
  static constexpr int SF_BYTES = SF_GRAN * 1024;          // per stage: weights' block (512 B), activations' block
  // bytes the TMA unit reports per stage: the FP4 loads count their PACKED source bytes (128 rows x 64 B), measured on
  // B200: with the unpacked size the barrier never completes
  static constexpr int STAGE_TX = 128 * 64 + B_BYTES;
  static constexpr int CTAS_PER_SM = NB <= 32 ? 2 : 1;
  static constexpr int STAGES = NB <= 16 ? 5 : NB <= 32 ? 4 : 6;
  static constexpr int TMEM_COLS = (2 * N + 8) <= 128 ? 128 : (2 * N + 8) <= 256 ? 256 : 512;
  static constexpr int SFA_COL = 2 * N, SFB_COL = 2 * N + 4;
  static constexpr int EPI_GROUPS = NB == 64 ? 2 : 1;      // epilogue warpgroups the shared memory is laid out for
  static constexpr int XCH_BYTES = 16 * 64 * 2 * EPI_GROUPS;  // per group: gate/up exchange of one 16-column chunk (bf16)
  static constexpr int smem_bytes(int) {                   // + 1024 for manual alignment
    return 1024 + STAGES * STAGE_BYTES + SF_RING * SF_BYTES + XCH_BYTES + 256;
  }
};


// Threads of a CTA.  Prefill-sized token tiles (NB = 64) of the MoE epilogues run TWO epilogue warpgroups, one per
// accumulator buffer (warps 2-5 take the even token tiles, warps 10-13 the odd ones): with the whole pipeline
// switched off part by part, the epilogue alone accounted for 0.47 ms of a 1.55 ms prefill block -- a tile's
// tcgen05.ld round trips, exchange through shared memory and stores are a chain of latencies that one warp per
// scheduler cannot hide, and a second accumulator in flight only helps if somebody is free to drain it.  (The plain
// epilogue of the `linear` role keeps one group: its 168 registers do not fit 448 threads.)
template <int NB, int EPI>
__host__ __device__ constexpr int tc_threads() { return (NB == 64 && EPI != TC_EPI_PLAIN) ? 448 : 320; }

struct TcItem {
  int plane, row0, n, tile, slice;
};

// Work items are read one ahead of their use: tc_load_item only issues the loads (no branch on what they return), so
// the two dependent reads of a grouped item (active list, then the group's row count / expert / first row) are in
// flight while the previous item is being worked on.  tc_check_item validates at the point of use; every role walks
// the items through these two functions and therefore skips the same ones.
__device__ __forceinline__ void tc_load_item(const TcArgs& a, int j, TcItem* it) {
  if (a.g_n) {
    const int grp = a.active[j / a.n_tiles];
    it->n = a.g_n[grp]; it->plane = a.g_expert[grp]; it->row0 = a.g_row0[grp];
  } else {  // one dense matrix: the rows are cut into virtual groups of dense_rows so that the work spreads over the
            // CTAs (small for decode-sized inputs, whose weights then come out of L2 for all but the first group)
    const int per = a.n_tiles * a.k_slices, jj = j % per;
    it->row0 = (j / per) * a.dense_rows;
    it->n = min(a.dense_rows, a.n_dense - it->row0);
    it->plane = 0;
    it->tile = jj % a.n_tiles;
    it->slice = jj / a.n_tiles;
    return;
  }
  it->tile = j % a.n_tiles;
  it->slice = 0;
}

__device__ __forceinline__ bool tc_check_item(const TcArgs& a, TcItem* it) {
  if (it->plane < 0 || it->plane >= a.n_planes) {
    atomicOr(a.status, DS_BAD_EXPERT);
    it->n = 0;
  }
  return it->n > 0;
}

// for (TcItemWalk w(a, n_items); w.next(&im);) { ... }: items blockIdx.x, blockIdx.x + gridDim.x, ...
struct TcItemWalk {
  const TcArgs& a;
  int n_items, jn;
  TcItem nxt;
  __device__ __forceinline__ TcItemWalk(const TcArgs& args, int n) : a(args), n_items(n), jn(int(blockIdx.x)) {
    if (jn < n_items) tc_load_item(a, jn, &nxt);
  }
  __device__ __forceinline__ bool next(TcItem* im) {
    while (jn < n_items) {
      *im = nxt;
      jn += int(gridDim.x);
      if (jn < n_items) tc_load_item(a, jn, &nxt);
      if (tc_check_item(a, im)) return true;
    }
    return false;
  }
};

template <int NB, int EPI>
__global__ void __launch_bounds__(tc_threads<NB, EPI>(), TcCfg<NB>::CTAS_PER_SM) tc_gemm_kernel(const __grid_constant__ CUtensorMap wmap0,
                                                         const __grid_constant__ CUtensorMap wmap1,
                                                         const __grid_constant__ CUtensorMap xmap_hi,
                                                         const __grid_constant__ CUtensorMap xmap_lo, const TcArgs a) {
  using C = TcCfg<NB>;
  using namespace tc;
  extern __shared__ uint8_t smem_raw[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // stages of K = 128, rounded up to whole scale granules of four: the stages past the real K load out-of-range boxes,
  // which the TMA unit fills with zeros (weights and activations), so they add nothing
  const int KS = (a.K / 128 + C::SF_GRAN - 1) / C::SF_GRAN * C::SF_GRAN;
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sgen = smem_raw + (sbase - smem_u32(smem_raw));
  const uint32_t s_stage = sbase;
  const uint32_t s_sf = sbase + C::STAGES * C::STAGE_BYTES;        // [SF_RING][SF_GRAN][weights 512 B | activations 512 B]
  const uint32_t s_xch = s_sf + C::SF_RING * C::SF_BYTES;
  const uint32_t s_bar = s_xch + C::XCH_BYTES;
  uint8_t* g_sf = sgen + C::STAGES * C::STAGE_BYTES;
  __nv_bfloat16* g_xch = reinterpret_cast<__nv_bfloat16*>(g_sf + C::SF_RING * C::SF_BYTES);
  volatile uint32_t* g_slot = reinterpret_cast<volatile uint32_t*>(g_sf + C::SF_RING * C::SF_BYTES + C::XCH_BYTES + 192);
  const uint32_t s_slot = s_bar + 192;
  auto full_bar = [&](int s) { return s_bar + 8 * s; };            // [0, 64): up to 8 stages
  auto empty_bar = [&](int s) { return s_bar + 64 + 8 * s; };      // [64, 128)
  auto sf_full = [&](int g) { return s_bar + 128 + 8 * g; };
  auto sf_empty = [&](int g) { return s_bar + 144 + 8 * g; };
  auto acc_full = [&](int b) { return s_bar + 160 + 8 * b; };
  auto acc_empty = [&](int b) { return s_bar + 176 + 8 * b; };

  if (tid == 0) {
    for (int s = 0; s < C::STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int b = 0; b < 2; ++b) {
      mbar_init(sf_full(b), 1); mbar_init(sf_empty(b), 1); mbar_init(acc_full(b), 1); mbar_init(acc_empty(b), 1);
    }
    fence_barrier_init();
    tma_prefetch_desc(&wmap0); tma_prefetch_desc(&wmap1); tma_prefetch_desc(&xmap_hi); tma_prefetch_desc(&xmap_lo);
  }
  if (warp == 1) { tmem_alloc(s_slot, C::TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *g_slot;
  // everything above touches only this CTA's shared and tensor memory and may overlap the previous kernel's tail
  pdl_wait();
  pdl_launch();
  // a CTA without work walks empty loops and falls through to the release of its tensor memory
  const int n_items = a.g_n ? a.n_active[0] * a.n_tiles
                            : (a.n_dense + a.dense_rows - 1) / a.dense_rows * a.n_tiles * a.k_slices;
  // stage range of an item: all of K, or its slice (slices start on scale-granule boundaries)
  auto ks_begin = [&](const TcItem& im) { return im.slice * a.slice_stages; };
  auto ks_end = [&](const TcItem& im) { return min(KS, (im.slice + 1) * a.slice_stages); };

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (elect_one()) {
      uint32_t it = 0;
      bool dead = false;
      TcItem im;
      for (TcItemWalk walk(a, n_items); !dead && walk.next(&im);) {
        const int r0 = im.tile * a.tile_rows + a.roff[0], r1 = im.tile * a.tile_rows + a.roff[1];
        const int ks0 = ks_begin(im), ks1 = ks_end(im);
        for (int t0 = 0; t0 < im.n && !dead; t0 += NB) {
          for (int ks = ks0; ks < ks1; ++ks, ++it) {
            const uint32_t s = it % C::STAGES, ph = (it / C::STAGES) & 1;
            if (!mbar_wait(empty_bar(s), ph ^ 1)) { atomicOr(a.status, DS_WAIT_TIMEOUT | 0x10); dead = true; break; }
            mbar_expect_tx(full_bar(s), uint32_t(a.stage_tx));
            const uint32_t sa = s_stage + s * C::STAGE_BYTES, sb = sa + C::A_BYTES;
            tma_load_2d(sa, &wmap0, full_bar(s), ks * 128, im.plane * a.plane_rows[0] + r0);
            tma_load_2d(sa + 8192, &wmap1, full_bar(s), ks * 128, im.plane * a.plane_rows[1] + r1);
            tma_load_2d(sb, &xmap_hi, full_bar(s), ks * 128, im.row0 + t0);
            tma_load_2d(sb + NB * 128, &xmap_lo, full_bar(s), ks * 128, im.row0 + t0);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      uint32_t it = 0, q = 0;
      bool dead = false;
      TcItem im;
      for (TcItemWalk walk(a, n_items); !dead && walk.next(&im);) {
        for (int t0 = 0; t0 < im.n && !dead; t0 += NB, ++q) {
          const uint32_t b = q & 1, bph = (q >> 1) & 1;
          if (!mbar_wait(acc_empty(b), bph ^ 1)) {
            atomicOr(a.status, DS_WAIT_TIMEOUT | 0x20);
            dead = true;
            break;
          }
          tc_fence_after();
          const uint32_t acc = tmem + b * C::N;
          const int ks0 = ks_begin(im), ks1 = ks_end(im);
          for (int ks = ks0; ks < ks1; ++ks, ++it) {
            const uint32_t s = it % C::STAGES, ph = (it / C::STAGES) & 1;
            const uint32_t g = (it / C::SF_GRAN) % C::SF_RING, gph = (it / (C::SF_GRAN * C::SF_RING)) & 1;
            if ((ks % C::SF_GRAN) == 0 && !mbar_wait(sf_full(g), gph)) {
              atomicOr(a.status, DS_WAIT_TIMEOUT | 0x200); dead = true; break;
            }
            if (!mbar_wait(full_bar(s), ph)) { atomicOr(a.status, DS_WAIT_TIMEOUT | 0x40); dead = true; break; }
            tc_fence_after();
            const uint32_t sa = s_stage + s * C::STAGE_BYTES, sb = sa + C::A_BYTES;
            const uint32_t ssf = s_sf + g * C::SF_BYTES + (ks % C::SF_GRAN) * 1024;
            tc_cp_32x128b_warpx4(tmem + C::SFA_COL, smem_desc(ssf, 0, 128, 0));
            tc_cp_32x128b_warpx4(tmem + C::SFB_COL, smem_desc(ssf + 512, 0, 128, 0));
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              tc_mma_mxf8f6f4(acc, smem_desc(sa + k * 32, 16, 1024, 2), smem_desc(sb + k * 32, 16, 1024, 2),
                              idesc_mxf8f6f4(uint32_t(a.a_fmt), FMT_E4M3, 128, C::N, k, k), tmem + C::SFA_COL,
                              tmem + C::SFB_COL, ((ks - ks0) | k) != 0);
            }
            tc_commit(empty_bar(s));
            if ((ks % C::SF_GRAN) == C::SF_GRAN - 1) tc_commit(sf_empty(g));
          }
          tc_commit(acc_full(b));  // also after a failed wait: the epilogue must not be left waiting
        }
      }
    }
    __syncwarp();
  } else if (warp >= 6 && warp < 10) {
    // ---------------------------------------------------------------- scale gather (128 threads: one tile row each)
    // A unit = one granule (four stages, K = 512) of one (item, token tile): 16 scale bytes of weight row gt and of
    // activation column gt.  Four units are kept in flight in registers, so the loads' latency is off the chain.
    const int gt = tid - 192;
    const int srow = a.K / 32;          // scale bytes per row
    const int hh = gt >> 6;
    int t0 = 0, kg = 0, kg0 = 0, kg1 = 0;  // granules [kg0, kg1) of the item's stage range
    bool have_item = false;
    TcItem im{};
    TcItemWalk walk(a, n_items);
    const uint8_t *wsc = nullptr, *xsc = nullptr;
    auto advance = [&]() -> bool {
      if (have_item) {
        if (++kg < kg1) return true;
        kg = kg0; t0 += NB;
        if (t0 >= im.n) have_item = false;
      }
      if (!have_item) {
        if (!walk.next(&im)) return false;
        kg0 = ks_begin(im) / C::SF_GRAN; kg1 = ks_end(im) / C::SF_GRAN;
        have_item = true; t0 = 0; kg = kg0;
        const int wrow = im.tile * a.tile_rows + a.roff[hh] + (gt & 63);
        wsc = (a.sw[hh] && wrow < a.lim[hh]) ? a.sw[hh] + (long long)im.plane * a.s_plane + (long long)wrow * srow : nullptr;
      }
      const int tcol = t0 + (gt < NB ? gt : gt - NB);  // column gt of the MMA's N: hi terms, then lo terms
      const long long xrow = im.row0 + tcol;
      xsc = (gt < C::N && tcol < im.n && xrow < a.total_rows) ? (gt < NB ? a.sfh : a.sfl) + xrow * srow : nullptr;
      return true;
    };
    const uint4 ones = make_uint4(0x7f7f7f7fu, 0x7f7f7f7fu, 0x7f7f7f7fu, 0x7f7f7f7fu);
    // 16 scale bytes of a row = one granule; the last granule of a K that is not a multiple of 512 holds fewer
    // (4 per real stage): the rest reads as scale 1 (it multiplies zeros)
    auto load_g = [&](const uint8_t* p) -> uint4 {
      if ((srow & 15) == 0) return ldg_nc_16(p + kg * 16);  // K a multiple of 512: whole, aligned granules
      const int rem = srow - kg * 16;                       // rows are only 4-byte aligned: word loads
      uint4 v = ones;
      if (rem > 0) v.x = ldg_nc_4(p + kg * 16);
      if (rem > 4) v.y = ldg_nc_4(p + kg * 16 + 4);
      if (rem > 8) v.z = ldg_nc_4(p + kg * 16 + 8);
      if (rem > 12) v.w = ldg_nc_4(p + kg * 16 + 12);
      return v;
    };
    auto load1 = [&](uint4& va, uint4& vb) {
      va = wsc ? load_g(wsc) : ones;
      vb = xsc ? load_g(xsc) : ones;
    };
    uint32_t gi = 0;
    bool dead = false;
    // word of row r = r0 + 32 r1 goes to [r0 * 4 + r1]: the 32 x 16-byte block tcgen05.cp replicates over the four lane
    // quadrants
    const int widx = (gt & 31) * 4 + (gt >> 5);
    auto put = [&](const uint4& va, const uint4& vb) {
      const uint32_t g = gi % C::SF_RING, gph = (gi / C::SF_RING) & 1;
      if (!dead && !mbar_wait(sf_empty(g), gph ^ 1)) {
        if (gt == 0) atomicOr(a.status, DS_WAIT_TIMEOUT | 0x80);
        dead = true;
      }
      uint32_t* blk = reinterpret_cast<uint32_t*>(g_sf + g * C::SF_BYTES);
      blk[widx] = va.x; blk[128 + widx] = vb.x;
      blk[256 + widx] = va.y; blk[384 + widx] = vb.y;
      blk[512 + widx] = va.z; blk[640 + widx] = vb.z;
      blk[768 + widx] = va.w; blk[896 + widx] = vb.w;
      fence_proxy_async();
      asm volatile("bar.sync 2, 128;" ::: "memory");
      if (gt == 0) mbar_arrive(sf_full(g));
      ++gi;
    };
    constexpr int DEPTH = 4;
    uint4 qa[DEPTH], qb[DEPTH];
    bool qv[DEPTH];
#pragma unroll
    for (int d = 0; d < DEPTH; ++d) {
      qv[d] = advance();
      if (qv[d]) load1(qa[d], qb[d]);
    }
    bool more = true;
    while (more) {
#pragma unroll
      for (int d = 0; d < DEPTH; ++d) {
        if (more && !qv[d]) more = false;  // units are used in order: the first empty slot ends the walk
        if (more) {
          put(qa[d], qb[d]);
          qv[d] = advance();
          if (qv[d]) load1(qa[d], qb[d]);
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue: warps 2..5 (and 10..13) own lane
    // quadrant warp % 4; with two groups, group eg drains accumulator buffer eg (token tiles of that parity)
    constexpr bool TWO = tc_threads<NB, EPI>() == 448;
    const int eg = TWO && warp >= 10 ? 1 : 0;
    const int ebase = eg ? 320 : 64;                 // first thread of this group
    const uint32_t bar_x = eg ? 4u : 1u, bar_acc = eg ? 5u : 3u;  // named barriers of this group
    __nv_bfloat16* const xch = g_xch + eg * (16 * 64);
    const int qd = warp & 3;
    const int r = qd * 32 + lane;  // row of the 128-row tile
    const int h = r >> 6;
    uint32_t q = 0;
    bool dead = false;
    // bf16 output whose 128 tile rows are 128 consecutive output columns (every epilogue but SiLU x up)
    const bool staged = EPI != TC_EPI_SILU_MUL && a.b_out != nullptr && a.f_out == nullptr && a.tile_rows == 128 &&
                        a.roff[1] == a.roff[0] + 64 && (a.lim[0] & 7) == 0 && (a.out_stride & 7) == 0;
    TcItem im;
    for (TcItemWalk walk(a, n_items); walk.next(&im);) {
      const int row = im.tile * a.tile_rows + a.roff[h] + (r & 63);
      const bool rvalid = row < a.lim[h];
      for (int t0 = 0; t0 < im.n; t0 += NB, ++q) {
        if (TWO && int(q & 1) != eg) continue;
        const uint32_t b = q & 1, bph = (q >> 1) & 1;
        if (!dead && !mbar_wait(acc_full(b), bph)) {
          if (lane == 0) atomicOr(a.status, DS_WAIT_TIMEOUT | 0x100);
          dead = true;  // keep walking the loops so that the named barriers below still pair up
        }
        tc_fence_after();
        const uint32_t acc = tmem + b * C::N + (uint32_t(qd * 32) << 16);
        const int ncols = min(NB, im.n - t0);  // columns past the group's last row hold nothing anyone reads
        for (int c0 = 0; c0 < ncols; c0 += 16) {
          float hi[16], lo[16];
          tmem_ld_x16(acc + c0, hi);
          tmem_ld_x16(acc + NB + c0, lo);
          if (c0 + 16 >= ncols) {
            // the last columns are in registers: hand the accumulator back before the global loads and stores below,
            // so that the MMA warp is never held up by their latency
            tc_fence_before();
            asm volatile("bar.sync %0, 128;" ::"r"(bar_acc) : "memory");
            if (tid == ebase) mbar_arrive(acc_empty(b));
          }
#pragma unroll
          for (int jj = 0; jj < 16; ++jj) hi[jj] += lo[jj];
          if (EPI == TC_EPI_PLAIN && (a.k_slices > 1 || a.raw)) {  // split K: raw sums of this slice, the epilogue runs after the reduction
            float* pp = a.part + (long long)im.slice * a.part_plane;
#pragma unroll
            for (int jj = 0; jj < 16; ++jj) {
              const int t = t0 + c0 + jj;
              if (t < im.n && rvalid) pp[(long long)(im.row0 + t) * a.out_stride + row] = hi[jj];
            }
            continue;
          }
          if constexpr (EPI == TC_EPI_SILU_MUL) {
            // Row p of the gate half and row p of the up half make one output element.  The gate rows' threads finish
            // columns 0..7 of the chunk, the up rows' threads columns 8..15; each side hands the other the eight
            // values it needs through shared memory (already rounded to bf16, as the golden rounds gate and up).
            const int p = r & 63;
            const int orow = im.tile * a.tile_rows + a.roff[0] + p;  // the pair's row in the activation
            const bool ovalid = orow < a.lim[0];
#pragma unroll
            for (int jj = 0; jj < 8; ++jj) {
              const int col = h ? jj : jj + 8;
              xch[col * 64 + p] = __float2bfloat16_rn(h ? hi[jj] : hi[jj + 8]);  // static indices: hi stays in registers
            }
            asm volatile("bar.sync %0, 128;" ::"r"(bar_x) : "memory");
#pragma unroll
            for (int jj = 0; jj < 8; ++jj) {
              const int col = h ? jj + 8 : jj;
              const int t = t0 + c0 + col;
              if (t < im.n && ovalid) {
                const float mine = round_bf16(h ? hi[jj + 8] : hi[jj]), other = __bfloat162float(xch[col * 64 + p]);
                const float g = h ? other : mine, u = h ? mine : other;
                a.act_out[(long long)(im.row0 + t) * a.act_rows + orow] = __float2bfloat16_rn(g / (1.0f + expf(-g)) * u);
              }
            }
            asm volatile("bar.sync %0, 128;" ::"r"(bar_x) : "memory");
          } else {
            // every global load of the chunk goes out before the first store: the output may alias the residual, so
            // the compiler cannot move a load above a store, and one round trip per column would be paid otherwise
            float aux[16];
            uint32_t res2[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};  // residual, two bf16 per register
            const float bias = (EPI == TC_EPI_PLAIN && a.bias && rvalid) ? a.bias[row] : 0.f;
            const float rscale = (EPI == TC_EPI_PLAIN && a.row_scale && rvalid) ? a.row_scale[row] : 1.f;
#pragma unroll
            for (int jj = 0; jj < 16; ++jj) {
              const int t = t0 + c0 + jj;
              const bool ok = t < im.n && rvalid;
              const long long dst = im.row0 + t;
              aux[jj] = 0.f;
              if constexpr (EPI == TC_EPI_ROW_SCALE) {
                if (ok) aux[jj] = a.rw_row[dst];
              } else if constexpr (EPI == TC_EPI_SHARED_DOWN) {
                if (ok) {
                  aux[jj] = a.gate[dst];
                  const uint32_t rb = *reinterpret_cast<const unsigned short*>(a.resid + dst * a.out_stride + row);
                  res2[jj >> 1] |= rb << (16 * (jj & 1));
                }
              } else if constexpr (EPI == TC_EPI_PLAIN) {
                if (ok && a.row_div) aux[jj] = a.row_div[dst];
                if (ok && a.resid2) {
                  const uint32_t rb = *reinterpret_cast<const unsigned short*>(a.resid2 + dst * a.out_stride + row);
                  res2[jj >> 1] |= rb << (16 * (jj & 1));
                }
              }
            }
            float o[16];
#pragma unroll
            for (int jj = 0; jj < 16; ++jj) {
              float v = hi[jj];
              if constexpr (EPI == TC_EPI_ROW_SCALE) {
                v *= aux[jj];
              } else if constexpr (EPI == TC_EPI_SHARED_DOWN) {
                const float sig = 1.0f / (1.0f + expf(-aux[jj]));
                v = ((jj & 1) ? bf16hi(res2[jj >> 1]) : bf16lo(res2[jj >> 1])) + v * sig;
              } else {
                v = v * rscale + bias;
                if (a.row_div) v = round_bf16(v) / aux[jj];
                if (a.resid2) v = round_bf16(v) + ((jj & 1) ? bf16hi(res2[jj >> 1]) : bf16lo(res2[jj >> 1]));
              }
              o[jj] = v;
            }
            if (staged) {
              // bf16 output of a full-width tile: 2-byte stores of one row per lane reach about 1 TB/s; the values go
              // through shared memory instead (8 columns at a time) and leave as 16-byte stores, 16 lanes per token row
#pragma unroll
              for (int half = 0; half < 2; ++half) {
#pragma unroll
                for (int jj = 0; jj < 8; ++jj) xch[jj * 128 + r] = __float2bfloat16_rn(o[half * 8 + jj]);
                asm volatile("bar.sync %0, 128;" ::"r"(bar_x) : "memory");
                const int e = tid - ebase, tt = e >> 4, part = e & 15;
                const int t = t0 + c0 + half * 8 + tt;
                const int rowg = im.tile * 128 + a.roff[0] + part * 8;
                if (t < im.n && rowg < a.lim[0])
                  *reinterpret_cast<uint4*>(a.b_out + (long long)(im.row0 + t) * a.out_stride + rowg) =
                      *reinterpret_cast<const uint4*>(xch + tt * 128 + part * 8);
                asm volatile("bar.sync %0, 128;" ::"r"(bar_x) : "memory");
              }
            } else {
#pragma unroll
              for (int jj = 0; jj < 16; ++jj) {
                const int t = t0 + c0 + jj;
                if (t >= im.n || !rvalid) continue;
                const long long dst = im.row0 + t;
                if (a.f_out) a.f_out[dst * a.out_stride + row] = o[jj];
                else a.b_out[dst * a.out_stride + row] = __float2bfloat16_rn(o[jj]);
              }
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem, C::TMEM_COLS);
}

}  // namespace q35
