// Decode-sized MoE block in four launches on one stream (role "moe.block"), and the load-time re-layout of E8M0
// scales it reads (roles "mx.tile_scales.paired" / "mx.tile_scales.plain").
//
// Arithmetic: models/qwen35_2b/whole/src/q35_moe.py:73-85,123-137 (moe_pre, moe_experts), golden :227-238, routing
// :293-297.  What the block computes per token t:
//   h2 = RMSNorm(x1) * ln2;  logits = h2 @ w_router^T (fp32);  ids, rw = top-k of softmax(logits), renormalised
//   base = bf16(x1 + sigmoid(h2 . w_shg) * shared_expert(h2));  out = bf16(base + sum_i rw_i * expert_{ids_i}(h2))
//   expert(h) = down(bf16(silu(bf16(gate h)) * bf16(up h)))
//
// Launches:
//   1. moe_front_kernel         RMSNorm, router logits and the shared-expert gate dot, a CTA per (token, expert slice);
//                               the last CTA of a token does its softmax / top-k, the last CTA of all the routing plan:
//                               per expert the tokens that chose it (bitmaps, ranks by popcount), row blocks of 16 per
//                               group, the shared expert as extra groups of 16 tokens
//   2. moe_decode_quant_kernel  h2 rows gathered into the groups' row blocks as two E4M3 terms + UE8M0 block scales
//   3. moe_decode_kernel        ONE persistent tcgen05 kernel for gate-up AND down of every group (below)
//   4. moe_block_combine_kernel out = bf16(bf16(x1 + sigmoid(gate) * shared row) + sum_i rw_i * routed row_i), fp32
//
// moe_decode_kernel.  Work items: (group, 128-row tile of gate|up rows) for all groups, then (group, 128-row tile of
// down rows); dealt round-robin to persistent CTAs (192 threads, two per SM).  A down item needs the group's whole
// activation row, i.e. all of the group's gate-up items, which other CTAs may own: every gate-up item ends by adding
// one to the group's counter in global memory, and the loader of a down item polls (bounded) until the counter is
// full.  All gate-up items precede all down items in every CTA's list and every CTA of the grid is resident (the grid
// is sized from the occupancy query), so a counter a CTA waits for is always being worked on by a running CTA.
// Gate-up and down therefore stream the expert weights back to back in one launch: no second ramp-up, no kernel
// boundary, and the quantisation of the activation happens in the gate-up epilogue.
//   warp 0    loader: per stage (K = 128) two TMA tiles of FP4 weights (CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B unpacks
//             them), two TMA tiles of E4M3 activations (hi, lo), and two 512-byte bulk copies of scale blocks that are
//             already in the layout tcgen05.cp wants -- the weights' from the tiled scale tensors made at load time,
//             the activations' written that way by launch 2 / by the gate-up epilogue.  One mbarrier per stage.
//   warp 1    owns tensor memory; per stage: tcgen05.cp of the two scale blocks, four tcgen05.mma
//             kind::mxf8f6f4.block_scale of K = 32 into a double-buffered accumulator [128 rows x (16 hi + 16 lo)]
//   warps 2-5 epilogue: gate-up: SiLU(gate) * up per row pair (the two 64-row halves of a tile), rounded to bf16, split
//             into two E4M3 terms with block scales over the warp's 32 rows (= 32 consecutive down inputs), written as
//             the down phase's operand; down: fp32 rows.  Only the group's real tokens are touched.
// Every wait is bounded and reports through the status word.
#include <algorithm>
#include <cstdlib>
#include <mutex>
#include "abi.h"
#include "common.cuh"
#include "tc_host.h"
#include "tc_ptx.cuh"

namespace q35 {

constexpr int MD_NB = 16;                                   // tokens per token tile
constexpr int MD_N = 2 * MD_NB;                             // MMA N: hi columns then lo columns
constexpr int MD_A_BYTES = 128 * 128;                       // 128 rows x 128 unpacked FP4 codes
constexpr int MD_B_BYTES = MD_N * 128;
constexpr int MD_SF_BYTES = 512;                            // one tcgen05.cp block: 32 rows x 16 bytes
constexpr int MD_STAGE_BYTES = MD_A_BYTES + MD_B_BYTES + 2 * MD_SF_BYTES;  // 21504 = 21 x 1024
constexpr int MD_STAGE_TX = 128 * 64 + MD_B_BYTES + 2 * MD_SF_BYTES;       // FP4 tiles count their packed bytes
constexpr int MD_STAGES = 5;
constexpr int MD_THREADS = 192;
constexpr int MD_TMEM_COLS = 128;                           // 2 x 32 accumulator columns + 8 scale columns
constexpr int MD_SFA_COL = 2 * MD_N, MD_SFB_COL = 2 * MD_N + 4;
constexpr int MD_XCH_BYTES = 16 * 64 * 2;
constexpr int MD_SMEM = 1024 + MD_STAGES * MD_STAGE_BYTES + MD_XCH_BYTES + 256;
constexpr int MD_MAX_ITEMS = 128;                           // work items one CTA can hold
constexpr uint32_t MD_READY_POLLS = 1u << 22;
constexpr int MD_MAX_PAIRS = 4096, MD_MAX_WORDS = 4096;

struct MdArgs {
  const int* g_plane; const int* g_n; const int* g_row0;    // per group: expert plane, rows, first row (multiple of 16)
  const int* active;                                         // [0] = groups with rows, [1..] their indices
  int* ready;                                                // per group: gate-up tiles finished
  int n_planes;                                              // routed planes; plane == n_planes = the shared expert
  int H, FE;
  int ratio;                                                 // bytes of a gate-up item / bytes of a down item (H / FE)
  const uint8_t* gs_t; const uint8_t* ds_t;                  // tiled scales of the routed experts
  const uint8_t* sgs_t; const uint8_t* sds_t;                // ... of the shared expert (nullptr: none)
  const uint8_t* sfb1;                                       // activation scale blocks, gate-up phase
  uint8_t* q2h; uint8_t* q2l; uint8_t* sfb2;                 // gate-up output = down operand
  float* sout;                                               // [rows, H] fp32
  int* status;
};

__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ int ld_acquire(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(MD_THREADS, 2)
moe_decode_kernel(const __grid_constant__ CUtensorMap m_wg, const __grid_constant__ CUtensorMap m_wd,
                  const __grid_constant__ CUtensorMap m_sg, const __grid_constant__ CUtensorMap m_su,
                  const __grid_constant__ CUtensorMap m_sd, const __grid_constant__ CUtensorMap m_x1h,
                  const __grid_constant__ CUtensorMap m_x1l, const __grid_constant__ CUtensorMap m_x2h,
                  const __grid_constant__ CUtensorMap m_x2l, const MdArgs a) {
  using namespace tc;
  extern __shared__ uint8_t smem_raw[];
  __shared__ int4 s_item[MD_MAX_ITEMS];   // x plane, y first row, z rows, w tile | phase << 16
  __shared__ int s_grp[MD_MAX_ITEMS];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sgen = smem_raw + (sbase - smem_u32(smem_raw));
  const uint32_t s_stage = sbase;
  const uint32_t s_xch = sbase + MD_STAGES * MD_STAGE_BYTES;
  const uint32_t s_bar = s_xch + MD_XCH_BYTES;
  __nv_bfloat16* g_xch = reinterpret_cast<__nv_bfloat16*>(sgen + MD_STAGES * MD_STAGE_BYTES);
  volatile uint32_t* g_slot = reinterpret_cast<volatile uint32_t*>(sgen + MD_STAGES * MD_STAGE_BYTES + MD_XCH_BYTES + 192);
  const uint32_t s_slot = s_bar + 192;
  auto full_bar = [&](int s) { return s_bar + 8 * s; };
  auto empty_bar = [&](int s) { return s_bar + 64 + 8 * s; };
  auto acc_full = [&](int b) { return s_bar + 128 + 8 * b; };
  auto acc_empty = [&](int b) { return s_bar + 144 + 8 * b; };

  // The plan (groups, rows, list of groups with rows) was written by the kernel before the one ahead of this one, which
  // had completed when this kernel was allowed to start: the item table is built before the wait, under the tail of
  // the kernel ahead.
  const int n_act = a.active[0];
  const int T1 = a.FE / 64, T2 = a.H / 128;
  const int items1 = n_act * T1, total = items1 + n_act * T2;
  // Dealing.  A gate-up item streams a.ratio times the bytes of a down item.  Gate-up items go round-robin; the CTAs
  // that got one fewer of them first receive a.ratio down items each (round-robin among themselves, lowest groups
  // first: those are ready first), the rest of the down items go round-robin over all CTAs.  Every CTA's gate-up items
  // come before its down items.
  const int G = int(gridDim.x), cta = int(blockIdx.x);
  const int items2 = total - items1;
  const int n1 = cta < items1 ? (items1 - cta + G - 1) / G : 0;
  const int rem = items1 % G, late = G - rem;  // CTAs rem .. G - 1 hold one gate-up item fewer
  const int E = rem == 0 ? 0 : min(items2, a.ratio * late);
  const int ne = (cta >= rem && cta - rem < E) ? (E - (cta - rem) + late - 1) / late : 0;
  const int rest = items2 - E;
  const int nr = cta < rest ? (rest - cta + G - 1) / G : 0;
  int n_mine = n1 + ne + nr;
  if (n_mine > MD_MAX_ITEMS) {  // the launcher sizes the grid so that this cannot happen
    if (tid == 0) atomicOr(a.status, DS_BAD_TOKEN);
    n_mine = MD_MAX_ITEMS;
  }
  if (tid < n_mine) {
    int j, phase = 0, tiles = T1;
    if (tid < n1) {
      j = cta + tid * G;
    } else {
      phase = 1; tiles = T2;
      j = tid < n1 + ne ? (cta - rem) + (tid - n1) * late : E + cta + (tid - n1 - ne) * G;
    }
    const int grp = a.active[1 + j / tiles];
    int4 im;
    im.x = a.g_plane[grp]; im.y = a.g_row0[grp]; im.z = a.g_n[grp]; im.w = (j % tiles) | (phase << 16);
    const int max_plane = a.sgs_t ? a.n_planes : a.n_planes - 1;
    if (im.x < 0 || im.x > max_plane || (im.y & 15)) {
      atomicOr(a.status, DS_BAD_EXPERT);
      im.z = 0;
    }
    s_item[tid] = im;
    s_grp[tid] = grp;
  }
  if (tid == 0) {
    for (int s = 0; s < MD_STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(acc_full(b), 1); mbar_init(acc_empty(b), 1); }
    fence_barrier_init();
    tma_prefetch_desc(&m_wg); tma_prefetch_desc(&m_wd); tma_prefetch_desc(&m_x1h); tma_prefetch_desc(&m_x1l);
    tma_prefetch_desc(&m_x2h); tma_prefetch_desc(&m_x2l);
  }
  if (warp == 1) { tmem_alloc(s_slot, MD_TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *g_slot;
  // everything above may overlap the previous kernel's tail
  pdl_wait();
  pdl_launch();

  const int KS1 = a.H / 128, KS2 = a.FE / 128;

  if (warp == 0) {
    // ---------------------------------------------------------------- loader
    if (elect_one()) {
      uint32_t it = 0;
      bool dead = false;
      for (int i = 0; i < n_mine && !dead; ++i) {
        const int4 im = s_item[i];
        if (im.z <= 0) continue;
        const int tile = im.w & 0xffff, phase = im.w >> 16;
        const bool shared = im.x == a.n_planes;
        const int KS = phase ? KS2 : KS1;
        const CUtensorMap *w0, *w1, *xh, *xl;
        int y0, y1;
        const uint8_t *sfa, *sfb;
        if (!phase) {
          w0 = shared ? &m_sg : &m_wg; w1 = shared ? &m_su : &m_wg;
          y0 = (shared ? 0 : im.x * 2 * a.FE) + tile * 64;
          y1 = shared ? tile * 64 : y0 + a.FE;
          sfa = (shared ? a.sgs_t : a.gs_t + size_t(im.x) * T1 * KS1 * MD_SF_BYTES) + size_t(tile) * KS1 * MD_SF_BYTES;
          xh = &m_x1h; xl = &m_x1l; sfb = a.sfb1;
        } else {
          w0 = w1 = shared ? &m_sd : &m_wd;
          y0 = (shared ? 0 : im.x * a.H) + tile * 128;
          y1 = y0 + 64;
          sfa = (shared ? a.sds_t : a.ds_t + size_t(im.x) * T2 * KS2 * MD_SF_BYTES) + size_t(tile) * KS2 * MD_SF_BYTES;
          xh = &m_x2h; xl = &m_x2l; sfb = a.sfb2;
          // the group's activation rows are complete when all of its gate-up tiles have reported
          const int* flag = a.ready + s_grp[i];
          uint32_t polls = 0;
          while (ld_acquire(flag) < T1) {
            if (++polls > MD_READY_POLLS) { atomicOr(a.status, DS_WAIT_TIMEOUT | 0x400); dead = true; break; }
          }
          if (dead) break;
          asm volatile("fence.proxy.async;" ::: "memory");  // rows written with plain stores, read by the TMA unit
        }
        for (int t0 = 0; t0 < im.z && !dead; t0 += MD_NB) {
          const uint8_t* sfb_t = sfb + size_t((im.y + t0) >> 4) * KS * MD_SF_BYTES;
          for (int ks = 0; ks < KS; ++ks, ++it) {
            const uint32_t s = it % MD_STAGES, ph = (it / MD_STAGES) & 1;
            if (!mbar_wait(empty_bar(s), ph ^ 1)) { atomicOr(a.status, DS_WAIT_TIMEOUT | 0x10); dead = true; break; }
            mbar_expect_tx(full_bar(s), MD_STAGE_TX);
            const uint32_t sa = s_stage + s * MD_STAGE_BYTES, sb = sa + MD_A_BYTES, ssf = sb + MD_B_BYTES;
            tma_load_2d(sa, w0, full_bar(s), ks * 128, y0);
            tma_load_2d(sa + 8192, w1, full_bar(s), ks * 128, y1);
            tma_load_2d(sb, xh, full_bar(s), ks * 128, im.y + t0);
            tma_load_2d(sb + MD_NB * 128, xl, full_bar(s), ks * 128, im.y + t0);
            bulk_load(ssf, sfa + size_t(ks) * MD_SF_BYTES, MD_SF_BYTES, full_bar(s));
            bulk_load(ssf + MD_SF_BYTES, sfb_t + size_t(ks) * MD_SF_BYTES, MD_SF_BYTES, full_bar(s));
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
      for (int i = 0; i < n_mine && !dead; ++i) {
        const int4 im = s_item[i];
        if (im.z <= 0) continue;
        const int KS = (im.w >> 16) ? KS2 : KS1;
        for (int t0 = 0; t0 < im.z && !dead; t0 += MD_NB, ++q) {
          const uint32_t b = q & 1, bph = (q >> 1) & 1;
          if (!mbar_wait(acc_empty(b), bph ^ 1)) { atomicOr(a.status, DS_WAIT_TIMEOUT | 0x20); dead = true; break; }
          tc_fence_after();
          const uint32_t acc = tmem + b * MD_N;
          for (int ks = 0; ks < KS; ++ks, ++it) {
            const uint32_t s = it % MD_STAGES, ph = (it / MD_STAGES) & 1;
            if (!mbar_wait(full_bar(s), ph)) { atomicOr(a.status, DS_WAIT_TIMEOUT | 0x40); dead = true; break; }
            tc_fence_after();
            const uint32_t sa = s_stage + s * MD_STAGE_BYTES, sb = sa + MD_A_BYTES, ssf = sb + MD_B_BYTES;
            tc_cp_32x128b_warpx4(tmem + MD_SFA_COL, smem_desc(ssf, 0, 128, 0));
            tc_cp_32x128b_warpx4(tmem + MD_SFB_COL, smem_desc(ssf + MD_SF_BYTES, 0, 128, 0));
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              tc_mma_mxf8f6f4(acc, smem_desc(sa + k * 32, 16, 1024, 2), smem_desc(sb + k * 32, 16, 1024, 2),
                              idesc_mxf8f6f4(FMT_E2M1, FMT_E4M3, 128, MD_N, k, k), tmem + MD_SFA_COL,
                              tmem + MD_SFB_COL, (ks | k) != 0);
            }
            tc_commit(empty_bar(s));
          }
          tc_commit(acc_full(b));  // also after a failed wait: the epilogue must not be left waiting
        }
      }
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- epilogue: warps 2..5 own lane quadrant warp % 4
    const int qd = warp & 3;
    const int r = qd * 32 + lane;  // row of the 128-row tile
    const int h = r >> 6, p = r & 63;
    uint32_t q = 0;
    bool dead = false;
    for (int i = 0; i < n_mine; ++i) {
      const int4 im = s_item[i];
      if (im.z <= 0) continue;
      const int tile = im.w & 0xffff, phase = im.w >> 16;
      for (int t0 = 0; t0 < im.z; t0 += MD_NB, ++q) {
        const uint32_t b = q & 1, bph = (q >> 1) & 1;
        if (!dead && !mbar_wait(acc_full(b), bph)) {
          if (lane == 0) atomicOr(a.status, DS_WAIT_TIMEOUT | 0x100);
          dead = true;  // keep walking the loops so that the named barriers below still pair up
        }
        tc_fence_after();
        const uint32_t acc = tmem + b * MD_N + (uint32_t(qd * 32) << 16);
        float v[16], lo[16];
        tmem_ld_x16(acc, v);
        tmem_ld_x16(acc + MD_NB, lo);
        // the accumulator goes back before any global access, so the MMA warp is never held up by their latency
        tc_fence_before();
        asm volatile("bar.sync 3, 128;" ::: "memory");
        if (tid == 64) mbar_arrive(acc_empty(b));
#pragma unroll
        for (int jj = 0; jj < 16; ++jj) v[jj] += lo[jj];
        const int ncols = min(MD_NB, im.z - t0);
        if (!phase) {
          // Row p of the gate half and row p of the up half make one activation element.  The gate rows' threads
          // finish tokens 0..7 of the tile, the up rows' threads tokens 8..15; each side hands the other the eight
          // values it needs through shared memory (already rounded to bf16, as the golden rounds gate and up).
#pragma unroll
          for (int jj = 0; jj < 8; ++jj) {
            const int col = h ? jj : jj + 8;
            g_xch[col * 64 + p] = __float2bfloat16_rn(h ? v[jj] : v[jj + 8]);
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
          const int col_fe = tile * 64 + p;  // input index of the down projection
#pragma unroll
          for (int jj = 0; jj < 8; ++jj) {
            const int t = (h ? 8 : 0) + jj;   // uniform over the warp
            if (t < ncols) {
              const float mine = round_bf16(h ? v[jj + 8] : v[jj]), other = __bfloat162float(g_xch[t * 64 + p]);
              const float g = h ? other : mine, u = h ? mine : other;
              const float act = round_bf16(g / (1.0f + expf(-g)) * u);
              // two E4M3 terms with UE8M0 scales over the warp's 32 consecutive inputs (same split as launch 2)
              const int eh = e8m0_for(warp_max(fabsf(act)));
              const __nv_fp8_e4m3 hq(act * pow2_int(-eh));
              const float rem = act - float(hq) * pow2_int(eh);
              const int el = e8m0_for(warp_max(fabsf(rem)));
              const __nv_fp8_e4m3 lq(rem * pow2_int(-el));
              const long long row = im.y + t0 + t;
              a.q2h[row * a.FE + col_fe] = *reinterpret_cast<const uint8_t*>(&hq);
              a.q2l[row * a.FE + col_fe] = *reinterpret_cast<const uint8_t*>(&lq);
              if (lane == 0) {
                uint8_t* blk = a.sfb2 + (size_t(row >> 4) * KS2 + (col_fe >> 7)) * MD_SF_BYTES;
                const int n = int(row & 15), kb = (col_fe >> 5) & 3;
                blk[n * 16 + kb] = uint8_t(eh + 127);
                blk[(MD_NB + n) * 16 + kb] = uint8_t(el + 127);
              }
            }
          }
          if (t0 + MD_NB >= im.z) {  // last token tile of the item: publish it
            __threadfence();
            asm volatile("fence.proxy.async;" ::: "memory");  // plain stores, read by another CTA's TMA unit
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (tid == 64) atomicAdd(a.ready + s_grp[i], 1);
          } else {
            asm volatile("bar.sync 1, 128;" ::: "memory");  // the exchange buffer is reused by the next token tile
          }
        } else {
          const int row_out = tile * 128 + r;
#pragma unroll
          for (int jj = 0; jj < 16; ++jj)
            if (jj < ncols) a.sout[size_t(im.y + t0 + jj) * a.H + row_out] = v[jj];
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem, MD_TMEM_COLS);
}

// ---------------------------------------------------------------------------------------------------------------
// launch 1: RMSNorm, router logits, shared-expert gate dot, routing and the routing plan in ONE launch.
// Grid (token groups, slices), 256 threads.  A CTA normalises its (up to four) tokens into shared memory (h2 =
// bf16(x1 * rsqrt(mean x1^2 + eps) * ln2)) and takes a slice of the NE + 1 rows (router rows, then the gate vector): a
// warp per row, the row's loads in flight together and used for every token of the group (the router matrix is read
// T / 4 times from L2 instead of T times); logits in fp32 (bf16 products are exact in fp32), in the same order of
// operations as rmsnorm_kernel + router_kernel of the role-by-role path, so both give the same bits.
// The LAST CTA of a token group to finish (a counter per group) routes its tokens, a warp each: softmax over all
// experts, top-K by logit with ties to the lower id, weights renormalised (the rule of moe.route).  The LAST CTA of the
// grid (a counter for all groups) then builds the plan.  Nobody waits for anybody: whoever arrives last does the work.
// Plan: every expert keeps a bitmap of the tokens that chose it; its row count is the number of set bits, a pair's
// rank the number of set bits below its token (tokens ascending = the stable order).  Groups get whole blocks of 16
// rows (the token tile of the GEMM), so a tile never spans two groups and the activations' scale blocks can be
// fetched as they lie.  The shared expert, when present, takes every token: one group per 16 tokens (groups NE, NE + 1,
// ...: every work item of the GEMM is then one token tile), rows in token order, listed FIRST among the groups with
// rows.  The counters are zero on entry (the launcher clears them) and on exit.
constexpr int NR_MAX_H = 8192;
constexpr int NR_TOK = 4;  // tokens per CTA at most (NR_MAX_H / H of them fit the shared-memory row buffer)

__device__ __forceinline__ uint32_t orderable(float f) {  // monotone map of floats onto unsigned integers
  const uint32_t b = __float_as_uint(f);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

template <int PER>
__global__ void __launch_bounds__(256, 4) moe_front_kernel(const __nv_bfloat16* __restrict__ x1,
                                                        const float* __restrict__ ln2,
                                                        const __nv_bfloat16* __restrict__ w_router,
                                                        const __nv_bfloat16* __restrict__ w_shg,
                                                        __nv_bfloat16* __restrict__ h2, float* logits, float* gate, int H,
                                                        int NE, float eps, int T, int K, int has_shared, int tok_per,
                                                        int* ids, float* rw, int* counters, int* g_plane, int* g_n,
                                                        int* g_row0, int* active, int* ready, int* loc) {
  pdl_wait();
  pdl_launch();
  __shared__ __align__(16) __nv_bfloat16 s_h2[NR_MAX_H];   // tok_per rows of H; the plan reuses these 16 KB as bitmaps
  __shared__ float s_red[8 * 4];
  __shared__ short s_raw[MD_MAX_PAIRS];
  __shared__ int s_row0[1024];
  __shared__ int s_warp[8];
  __shared__ int s_flag, s_flag_all, s_tot;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int t0 = int(blockIdx.x) * tok_per, nt = min(tok_per, T - t0);
  const int rows = NE + 1, per = (rows + int(gridDim.y) - 1) / int(gridDim.y);
  const int e0 = int(blockIdx.y) * per, e1 = min(rows, e0 + per);
  // Everything the CTA will need is requested at once: the tokens' rows as loads, ln2 and this warp's router rows as
  // prefetches into L2 (they cost no registers; the loads that follow find the lines there or on their way).
  for (int e = e0 + warp; e < e1; e += 8) {
    const __nv_bfloat16* wr = e < NE ? w_router + size_t(e) * H : w_shg;
    for (int b = lane * 128; b < H * 2; b += 32 * 128) prefetch_l2(reinterpret_cast<const char*>(wr) + b);
  }
  for (int b = tid * 128; b < H * 4; b += 256 * 128) prefetch_l2(reinterpret_cast<const char*>(ln2) + b);
  {
    // tok_per * ceil(H / 2048) <= 4 pieces of 16 bytes a thread: piece q = token q / ppt, chunk q % ppt
    const int ppt = (H + 2047) / 2048;
    uint4 xp[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int j = q / ppt, i = (tid + 256 * (q % ppt)) * 8;
      xp[q] = (j < nt && i < H) ? *reinterpret_cast<const uint4*>(x1 + size_t(t0 + j) * H + i) : make_uint4(0u, 0u, 0u, 0u);
    }
    float ssq[4];  // per piece, elements in order (the order rms_sumsq takes them in)
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const uint32_t w[4] = {xp[q].x, xp[q].y, xp[q].z, xp[q].w};
      float ss = 0.f;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float a = bf16lo(w[u]), b = bf16hi(w[u]);
        ss += a * a;
        ss += b * b;
      }
      ssq[q] = ss;
    }
    for (int j = 0; j < nt; ++j) {
      // a token's pieces in chunk order: continue one running sum, as rms_sumsq does over a thread's pieces
      float ss = 0.f;
#pragma unroll
      for (int q = 0; q < 4; ++q)
        if (q / ppt == j) ss = (q % ppt == 0) ? ssq[q] : rms_chain(ss, xp[q]);
      ss = warp_sum(ss);
      if (lane == 0) s_red[j * 8 + warp] = ss;
    }
    __syncthreads();
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int j = q / ppt, i = (tid + 256 * (q % ppt)) * 8;
      if (j >= nt || i >= H) continue;
      float tot = 0.f;
#pragma unroll
      for (int u = 0; u < 8; ++u) tot += s_red[j * 8 + u];
      const float rs = rsqrtf(tot / float(H) + eps);
      const float4 w0 = *reinterpret_cast<const float4*>(ln2 + i), w1 = *reinterpret_cast<const float4*>(ln2 + i + 4);
      uint4 o;
      o.x = pack_bf16(bf16lo(xp[q].x) * rs * w0.x, bf16hi(xp[q].x) * rs * w0.y);
      o.y = pack_bf16(bf16lo(xp[q].y) * rs * w0.z, bf16hi(xp[q].y) * rs * w0.w);
      o.z = pack_bf16(bf16lo(xp[q].z) * rs * w1.x, bf16hi(xp[q].z) * rs * w1.y);
      o.w = pack_bf16(bf16lo(xp[q].w) * rs * w1.z, bf16hi(xp[q].w) * rs * w1.w);
      *reinterpret_cast<uint4*>(s_h2 + j * H + i) = o;
      if (blockIdx.y == 0) *reinterpret_cast<uint4*>(h2 + size_t(t0 + j) * H + i) = o;
    }
  }
  __syncthreads();
  for (int e = e0 + warp; e < e1; e += 8) {
    const __nv_bfloat16* wr = e < NE ? w_router + size_t(e) * H : w_shg;
    float acc[NR_TOK] = {0.f, 0.f, 0.f, 0.f};
    for (int k0 = lane * 8; k0 < H; k0 += 2048) {  // eight 16-byte loads of the row in flight
      uint4 wv[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (k0 + u * 256 < H) wv[u] = ldg_nc_16(wr + k0 + u * 256);
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (k0 + u * 256 >= H) break;
#pragma unroll
        for (int j = 0; j < NR_TOK; ++j) {
          if (j >= nt) break;
          const uint4 xv = *reinterpret_cast<const uint4*>(s_h2 + j * H + k0 + u * 256);
          float a = acc[j];
          a = fmaf(bf16lo(xv.x), bf16lo(wv[u].x), a); a = fmaf(bf16hi(xv.x), bf16hi(wv[u].x), a);
          a = fmaf(bf16lo(xv.y), bf16lo(wv[u].y), a); a = fmaf(bf16hi(xv.y), bf16hi(wv[u].y), a);
          a = fmaf(bf16lo(xv.z), bf16lo(wv[u].z), a); a = fmaf(bf16hi(xv.z), bf16hi(wv[u].z), a);
          a = fmaf(bf16lo(xv.w), bf16lo(wv[u].w), a); a = fmaf(bf16hi(xv.w), bf16hi(wv[u].w), a);
          acc[j] = a;
        }
      }
    }
#pragma unroll
    for (int j = 0; j < NR_TOK; ++j) {
      if (j >= nt) break;
      const float a = warp_sum(acc[j]);
      if (lane == 0) {
        if (e < NE) logits[size_t(t0 + j) * NE + e] = a;
        else gate[t0 + j] = a;
      }
    }
  }
  // ---- the last CTA of this token group routes its tokens
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    s_flag = atomicAdd(counters + 1 + blockIdx.x, 1) == int(gridDim.y) - 1;
    s_flag_all = 0;
  }
  __syncthreads();
  if (!s_flag) return;
  __threadfence();
  if (warp < nt) {
    const int t = t0 + warp;
    const float* row = logits + size_t(t) * NE;
    float v[PER];
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int e = lane + 32 * j;
      v[j] = e < NE ? __ldcg(row + e) : -INFINITY;
    }
    float mx = v[0];
#pragma unroll
    for (int j = 1; j < PER; ++j) mx = fmaxf(mx, v[j]);
    mx = warp_max(mx);
    float z = 0.f;
#pragma unroll
    for (int j = 0; j < PER; ++j) z += (lane + 32 * j < NE) ? expf(v[j] - mx) : 0.f;
    z = warp_sum(z);
    unsigned taken = 0;
    float my_p = 0.f, sel_sum = 0.f;
    int my_id = 0;
    for (int k = 0; k < K; ++k) {
      // this lane's best remaining expert, then the warp's: the largest logit (one integer max-reduction over a
      // monotone image of the floats), and among the lanes that hold it the lowest expert id (one min-reduction)
      float bv = -INFINITY;
      int bi = 0x7fffffff;
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        const int e = lane + 32 * j;
        const bool ok = e < NE && !((taken >> j) & 1u);
        if (ok && (v[j] > bv || (v[j] == bv && e < bi))) { bv = v[j]; bi = e; }
      }
      const uint32_t key = bi != 0x7fffffff ? orderable(bv) : 0u;
      const uint32_t kmax = __reduce_max_sync(0xffffffffu, key);
      const int win = __reduce_min_sync(0xffffffffu, (key == kmax && bi != 0x7fffffff) ? bi : 0x7fffffff);
      const float wv = __shfl_sync(0xffffffffu, bv, win & 31);  // the winner's lane is its id modulo 32
      if (win != 0x7fffffff && (win & 31) == lane) taken |= 1u << (win >> 5);
      const float p = win != 0x7fffffff ? expf(wv - mx) / z : 0.f;
      sel_sum += p;
      if (lane == k) { my_p = p; my_id = win != 0x7fffffff ? win : 0; }
    }
    if (lane < K) {
      ids[size_t(t) * K + lane] = my_id;
      rw[size_t(t) * K + lane] = my_p / sel_sum;
    }
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    counters[1 + blockIdx.x] = 0;
    s_flag_all = atomicAdd(counters, 1) == int(gridDim.x) - 1;
  }
  __syncthreads();
  if (!s_flag_all) return;
  // ---- the last CTA of the grid builds the plan
  __threadfence();
  uint32_t* s_bits = reinterpret_cast<uint32_t*>(s_h2);  // 4096 words
  const int P = T * K, W = (T + 31) / 32;
  for (int i = tid; i < NE * W; i += 256) s_bits[i] = 0u;
  for (int p = tid; p < P; p += 256) s_raw[p] = short(__ldcg(ids + p));
  __syncthreads();
  for (int p = tid; p < P; p += 256) {
    const int tk = p / K;
    atomicOr(&s_bits[int(s_raw[p]) * W + (tk >> 5)], 1u << (tk & 31));
  }
  __syncthreads();
  // exclusive scan over the experts of (row blocks, has rows) packed as blocks | on << 16; four experts per thread
  const int n_sh = has_shared ? (T + MD_NB - 1) / MD_NB : 0;  // groups of the shared expert
  int cnt[4], v4[4], mine = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int e = tid * 4 + j;
    cnt[j] = 0;
    if (e < NE)
      for (int w = 0; w < W; ++w) cnt[j] += __popc(s_bits[e * W + w]);
    v4[j] = ((cnt[j] + MD_NB - 1) / MD_NB) | (cnt[j] > 0 ? 1 << 16 : 0);
    mine += v4[j];
  }
  int inc = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int n = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += n;
  }
  if (lane == 31) s_warp[warp] = inc;
  __syncthreads();
  int before = 0;
  for (int w = 0; w < warp; ++w) before += s_warp[w];
  int exc = before + inc - mine;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int e = tid * 4 + j;
    if (e < NE) {
      s_row0[e] = (exc & 0xffff) * MD_NB;
      g_plane[e] = e; g_n[e] = cnt[j]; g_row0[e] = (exc & 0xffff) * MD_NB;
      ready[e] = 0;
      if (cnt[j] > 0) active[1 + n_sh + (exc >> 16)] = e;
    }
    exc += v4[j];
  }
  if (tid == 255) {  // exc is now the grand total
    s_tot = (exc & 0xffff) * MD_NB;  // first row of the shared expert's groups
    active[0] = (exc >> 16) + n_sh;
    counters[0] = 0;
  }
  __syncthreads();
  for (int j = tid; j < n_sh; j += 256) {
    g_plane[NE + j] = NE; g_n[NE + j] = min(MD_NB, T - j * MD_NB); g_row0[NE + j] = s_tot + j * MD_NB;
    ready[NE + j] = 0;
    active[1 + j] = NE + j;
  }
  for (int p = tid; p < P; p += 256) {
    const int tk = p / K, k = p % K, id = s_raw[p];
    int rank = __popc(s_bits[id * W + (tk >> 5)] & ((1u << (tk & 31)) - 1u));
    for (int w = 0; w < (tk >> 5); ++w) rank += __popc(s_bits[id * W + w]);
    loc[size_t(k) * T + tk] = s_row0[id] + rank;
  }
  if (has_shared)
    for (int tk = tid; tk < T; tk += 256) loc[size_t(K) * T + tk] = s_tot + tk;
}

// ---------------------------------------------------------------------------------------------------------------
// launch 2: row loc[j, t] of the operand = h2[t] as two E4M3 terms with UE8M0 block-32 scales (x = hi 2^eh + lo 2^el),
// the scales written straight into the 512-byte blocks the GEMM copies to tensor memory: block (row / 16, k / 128),
// byte [(row % 16) * 16 + (k / 32) % 4] for the hi term, 256 bytes further for the lo term.
__global__ void __launch_bounds__(256) moe_decode_quant_kernel(const __nv_bfloat16* __restrict__ x,
                                                               const int* __restrict__ loc, int n_pairs, int T, int H,
                                                               uint8_t* __restrict__ qh, uint8_t* __restrict__ ql,
                                                               uint8_t* __restrict__ sfb) {
  pdl_wait();
  pdl_launch();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;  // index of the 8-element piece
  const int per_row = H / 8;
  const bool in = i < (long long)n_pairs * per_row;  // whole quads are in or out together (H is a multiple of 32)
  const int pair = in ? int(i / per_row) : 0, c8 = in ? int(i % per_row) : 0;
  const int row = in ? loc[pair] : -1;
  const bool on = row >= 0;
  uint4 raw = make_uint4(0u, 0u, 0u, 0u);
  if (on) raw = *reinterpret_cast<const uint4*>(x + size_t(pair % T) * H + c8 * 8);
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  float v[8];
#pragma unroll
  for (int u = 0; u < 4; ++u) { v[2 * u] = bf16lo(w[u]); v[2 * u + 1] = bf16hi(w[u]); }
  const TwoTerm8 t = quant_two_terms8(v);
  if (!on) return;
  const long long o = (long long)row * H + c8 * 8;
  *reinterpret_cast<uint2*>(qh + o) = t.hi;
  *reinterpret_cast<uint2*>(ql + o) = t.lo;
  if ((c8 & 3) == 0) {
    uint8_t* blk = sfb + (size_t(row >> 4) * (H / 128) + (c8 >> 4)) * MD_SF_BYTES;
    const int n = row & 15, kb = (c8 >> 2) & 3;
    blk[n * 16 + kb] = uint8_t(t.eh + 127);
    blk[(MD_NB + n) * 16 + kb] = uint8_t(t.el + 127);
  }
}

// ---------------------------------------------------------------------------------------------------------------
// launch 4: out[t] = bf16(base + sum_i rw[t, i] * row_i), base = bf16(x1[t] + sigmoid(gate[t]) * shared row) -- the
// golden's order: the shared expert closes the dense part in bf16, the routed terms are added to it in fp32 one by one
// (rw * d rounded, then added: no fused multiply-add, as torch computes them).
__global__ void __launch_bounds__(256) moe_block_combine_kernel(const __nv_bfloat16* __restrict__ x1,
                                                                const float* __restrict__ gate,
                                                                const float* __restrict__ rw,
                                                                const int* __restrict__ loc,
                                                                const float* __restrict__ sout,
                                                                __nv_bfloat16* __restrict__ out, int T, int H, int K,
                                                                int has_shared) {
  // x1, gate, rw and loc were written by kernels that completed before the kernel ahead of this one passed its own
  // wait (every kernel of the chain waits before it lets its successor start), so they may be read before this
  // kernel's wait: their latency then hides behind the tail of the GEMM.  Only the rows need the wait.
  const int t = blockIdx.x;
  const int h = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
  const bool on = h < H;
  uint2 xb = make_uint2(0u, 0u);
  int rix[8], rsh = -1;
  float wts[8], sg = 0.f;
  const int kmax = K < 8 ? K : 8;
  if (on) {
    xb = *reinterpret_cast<const uint2*>(x1 + size_t(t) * H + h);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      rix[k] = k < kmax ? loc[size_t(k) * T + t] : -1;
      wts[k] = k < kmax ? rw[size_t(t) * K + k] : 0.f;
    }
    if (has_shared) {
      rsh = loc[size_t(K) * T + t];
      sg = 1.0f / (1.0f + expf(-gate[t]));
    }
  }
  pdl_wait();
  pdl_launch();
  if (!on) return;
  float acc[4] = {bf16lo(xb.x), bf16hi(xb.x), bf16lo(xb.y), bf16hi(xb.y)};
  float4 rows[8];
  float4 sh = make_float4(0.f, 0.f, 0.f, 0.f);
  // all row loads go out before the first use; K <= 8 here, the general loop below takes the rest
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    rows[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (rix[k] >= 0) rows[k] = *reinterpret_cast<const float4*>(sout + size_t(rix[k]) * H + h);
    else wts[k] = 0.f;
  }
  if (rsh >= 0) sh = *reinterpret_cast<const float4*>(sout + size_t(rsh) * H + h);
  if (has_shared) {
    acc[0] = round_bf16(acc[0] + sh.x * sg); acc[1] = round_bf16(acc[1] + sh.y * sg);
    acc[2] = round_bf16(acc[2] + sh.z * sg); acc[3] = round_bf16(acc[3] + sh.w * sg);
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    acc[0] = __fadd_rn(acc[0], __fmul_rn(wts[k], rows[k].x)); acc[1] = __fadd_rn(acc[1], __fmul_rn(wts[k], rows[k].y));
    acc[2] = __fadd_rn(acc[2], __fmul_rn(wts[k], rows[k].z)); acc[3] = __fadd_rn(acc[3], __fmul_rn(wts[k], rows[k].w));
  }
  for (int k = 8; k < K; ++k) {
    const int r = loc[size_t(k) * T + t];
    if (r < 0) continue;
    const float4 d = *reinterpret_cast<const float4*>(sout + size_t(r) * H + h);
    const float wk = rw[size_t(t) * K + k];
    acc[0] = __fadd_rn(acc[0], __fmul_rn(wk, d.x)); acc[1] = __fadd_rn(acc[1], __fmul_rn(wk, d.y));
    acc[2] = __fadd_rn(acc[2], __fmul_rn(wk, d.z)); acc[3] = __fadd_rn(acc[3], __fmul_rn(wk, d.w));
  }
  uint2 o;
  o.x = pack_bf16(acc[0], acc[1]);
  o.y = pack_bf16(acc[2], acc[3]);
  *reinterpret_cast<uint2*>(out + size_t(t) * H + h) = o;
}

// ---------------------------------------------------------------------------------------------------------------
// mx.tile_scales.*: E8M0 scales [planes, rows, K/32] re-laid into the 512-byte blocks tcgen05.cp copies to tensor
// memory, one block per (plane, 128-row tile, K = 128): byte [l * 16 + c * 4 + b] = scale of tile row l + 32 c for the
// inputs 128 s + 32 b .. + 31.  A load-time conversion of the weights (the reference converts weights at load as its
// manifests' `convert` kinds say, tools/manifest/mkmanifest.py:202-251): the bytes are the same, only their order
// changes, so the GEMM's loader can fetch a stage's scales with one bulk copy.
//   paired: tile i = rows 64 i .. + 63 (gate) followed by rows rows/2 + 64 i .. + 63 (up)     [gate | up planes]
//   plain : tile i = rows 128 i .. + 127
__global__ void tile_scales_kernel(const uint8_t* __restrict__ s, uint8_t* __restrict__ out, int rows, int KB,
                                   int paired, long long n_words) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;  // one 4-byte word of the output
  if (i >= n_words) return;
  const int KS = KB / 4, tiles = rows / 128;
  const int c = int(i & 3), l = int((i >> 2) & 31);
  const long long blk = i >> 7;
  const int st = int(blk % KS);
  const int tile = int((blk / KS) % tiles);
  const long long plane = blk / KS / tiles;
  const int m = l + 32 * c;
  const int row = paired ? (m < 64 ? tile * 64 + m : rows / 2 + tile * 64 + (m - 64)) : tile * 128 + m;
  reinterpret_cast<uint32_t*>(out)[i] =
      *reinterpret_cast<const uint32_t*>(s + (plane * rows + row) * KB + st * 4);
}

static int run_tile_scales(Call& c, int paired) {
  Tensor s, out;
  Q35_TRY(c.get("s", M(Q35_U8), &s));
  Q35_TRY(c.get("out", M(Q35_U8), &out));
  Q35_REQUIRE(s.nd == 2 || s.nd == 3, Q35_ERR_SHAPE, "mx.tile_scales: s [planes, rows, K/32] or [rows, K/32]");
  const int64_t KB = s.s[s.nd - 1], rows = s.s[s.nd - 2], planes = s.nd == 3 ? s.s[0] : 1;
  Q35_REQUIRE(KB % 4 == 0 && rows % 128 == 0, Q35_ERR_UNSUPPORTED,
              "mx.tile_scales: K must be a multiple of 128 and rows a multiple of 128");
  Q35_REQUIRE(out.numel() == s.numel(), Q35_ERR_SHAPE, "mx.tile_scales: out must hold as many bytes as s");
  c.ws_need = 0;
  if (c.dry || s.numel() == 0) return 0;
  Q35_REQUIRE((reinterpret_cast<uintptr_t>(s.p) & 3) == 0 && aligned16(out.p), Q35_ERR_ALIGN, "mx.tile_scales: alignment");
  const long long n_words = s.numel() / 4;
  tile_scales_kernel<<<unsigned((n_words + 255) / 256), 256, 0, c.stream>>>(s.as<uint8_t>(), out.as<uint8_t>(), int(rows),
                                                                           int(KB), paired, n_words);
  Q35_CUDA_LAUNCH_CHECK("mx.tile_scales");
  (void)planes;
  return 0;
}
int run_tile_scales_paired(Call& c) { return run_tile_scales(c, 1); }
int run_tile_scales_plain(Call& c) { return run_tile_scales(c, 0); }

// ---------------------------------------------------------------------------------------------------------------
static int md_grid(int* grid) {  // CTAs that are resident at once: the kernel's items wait on one another
  static std::mutex lock;
  static int per_device[64] = {0};
  int dev = 0;
  Q35_REQUIRE(cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64, Q35_ERR_CUDA, "cudaGetDevice");
  std::lock_guard<std::mutex> guard(lock);
  if (!per_device[dev]) {
    Q35_TRY(ensure_dynamic_smem(reinterpret_cast<const void*>(moe_decode_kernel), MD_SMEM));
    cudaFuncSetAttribute(moe_decode_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    // CTAs per SM from the kernel's own figures: shared memory (static + dynamic + the per-block reserve) and registers.
    // (The runtime's occupancy query answers 1 for this kernel whatever its shared memory size -- measured; it seems
    // to budget all of tensor memory for a kernel that allocates any -- while two CTAs of 128 columns each do run
    // side by side.  Should only one be resident after all, the bounded waits report it instead of hanging.)
    cudaFuncAttributes fa{};
    cudaError_t e = cudaFuncGetAttributes(&fa, moe_decode_kernel);
    Q35_REQUIRE(e == cudaSuccess, Q35_ERR_CUDA, "cudaFuncGetAttributes: %s", cudaGetErrorString(e));
    int smem_sm = 0, resv = 0, regs_sm = 0;
    cudaDeviceGetAttribute(&smem_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev);
    cudaDeviceGetAttribute(&resv, cudaDevAttrReservedSharedMemoryPerBlock, dev);
    cudaDeviceGetAttribute(&regs_sm, cudaDevAttrMaxRegistersPerMultiprocessor, dev);
    const long long per_cta = (long long)fa.sharedSizeBytes + MD_SMEM + resv;
    const long long regs_cta = (long long)((fa.numRegs + 7) / 8 * 8) * MD_THREADS;
    int occ = int(std::min<long long>(smem_sm / per_cta, regs_sm / (regs_cta > 0 ? regs_cta : 1)));
    Q35_REQUIRE(occ >= 1, Q35_ERR_CUDA, "the decode MoE kernel does not fit an SM (%lld bytes of shared memory)", per_cta);
    per_device[dev] = sm_count() * (occ > 2 ? 2 : occ);
  }
  *grid = per_device[dev];
  return 0;
}

struct WsCut {
  uint8_t* base;
  int64_t off = 0;
  template <class T> T* take(int64_t count) {
    T* p = base ? reinterpret_cast<T*>(base + off) : nullptr;
    off = (off + count * int64_t(sizeof(T)) + 255) / 256 * 256;
    return p;
  }
};

// ---------------------------------------------------------------------------------------------------------------
// Routed experts alone on given ids (role moe.experts with tiled scales bound): the expert-parallel form, where the
// tokens of all ranks were gathered and every rank runs ITS experts.  Plan from the caller's ids (one CTA; ids
// outside [base, base + NE) belong to other ranks and get loc = -1; an expert a token lists twice gets one row that
// both listings point at, so its two weights are both applied), then the same quantise / GEMM launches as moe.block,
// then the weighted sum of each token's rows: out = bf16(base + sum) or, without a base, the fp32 partial sum.
__global__ void __launch_bounds__(1024) moe_plan_kernel(const int* __restrict__ ids, const int* __restrict__ base, int T,
                                                        int K, int NE, int* g_plane, int* g_n, int* g_row0, int* active,
                                                        int* ready, int* loc, int* status) {
  pdl_wait();
  pdl_launch();
  __shared__ short s_raw[MD_MAX_PAIRS];
  __shared__ uint32_t s_bits[MD_MAX_WORDS];
  __shared__ int s_row0[1024];
  __shared__ int s_warp[32];
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  const int P = T * K, W = (T + 31) / 32;
  const int first = base ? base[0] : 0;
  for (int p = tid; p < P; p += 1024) {
    int id = ids[p] - first;
    if (id >= NE) {
      if (!base) atomicOr(status, DS_BAD_EXPERT);
      id = -1;
    }
    s_raw[p] = short(id < 0 ? -1 : id);  // negative: not on this rank
  }
  for (int i = tid; i < NE * W; i += 1024) s_bits[i] = 0u;
  __syncthreads();
  for (int p = tid; p < P; p += 1024) {
    const int t = p / K, id = s_raw[p];
    if (id >= 0) atomicOr(&s_bits[id * W + (t >> 5)], 1u << (t & 31));
  }
  __syncthreads();
  int cnt = 0;
  if (tid < NE)
    for (int w = 0; w < W; ++w) cnt += __popc(s_bits[tid * W + w]);
  const int v = ((cnt + MD_NB - 1) / MD_NB) | (cnt > 0 ? 1 << 16 : 0);
  int inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int n = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += n;
  }
  if (lane == 31) s_warp[wid] = inc;
  __syncthreads();
  if (wid == 0) {
    int w = s_warp[lane], winc = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, winc, o);
      if (lane >= o) winc += n;
    }
    s_warp[lane] = winc - w;
  }
  __syncthreads();
  const int exc = s_warp[wid] + inc - v;
  if (tid < NE) {
    s_row0[tid] = (exc & 0xffff) * MD_NB;
    g_plane[tid] = tid; g_n[tid] = cnt; g_row0[tid] = (exc & 0xffff) * MD_NB;
    ready[tid] = 0;
    if (cnt > 0) active[1 + (exc >> 16)] = tid;
  }
  if (tid == 1023) active[0] = (exc + v) >> 16;
  __syncthreads();
  for (int p = tid; p < P; p += 1024) {
    const int t = p / K, k = p % K, id = s_raw[p];
    int row = -1;
    if (id >= 0) {
      int rank = __popc(s_bits[id * W + (t >> 5)] & ((1u << (t & 31)) - 1u));
      for (int w = 0; w < (t >> 5); ++w) rank += __popc(s_bits[id * W + w]);
      row = s_row0[id] + rank;
    }
    loc[size_t(k) * T + t] = row;
  }
}

// out[t] = bf16(base[t] + sum_k rw[t, k] * row(loc[k, t])) in fp32, k ascending, product rounded before the add (the
// golden's acc += rw * d, models/qwen35_2b/whole/src/q35_moe.py:235-238); without base / out: partial[t] = the sum
__global__ void __launch_bounds__(256) moe_rows_combine_kernel(const __nv_bfloat16* __restrict__ base,
                                                               const float* __restrict__ rw,
                                                               const int* __restrict__ loc,
                                                               const float* __restrict__ sout,
                                                               __nv_bfloat16* __restrict__ out,
                                                               float* __restrict__ partial, int T, int H, int K) {
  const int t = blockIdx.x;
  const int h = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
  const bool on = h < H;
  int rix[8];
  float wts[8];
  const int kmax = K < 8 ? K : 8;
  if (on) {  // the plan and the routing weights were complete before the kernel ahead of this one could start
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      rix[k] = k < kmax ? loc[size_t(k) * T + t] : -1;
      wts[k] = k < kmax ? rw[size_t(t) * K + k] : 0.f;
    }
  }
  pdl_wait();
  pdl_launch();
  if (!on) return;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  if (base) {
    const uint2 xb = *reinterpret_cast<const uint2*>(base + size_t(t) * H + h);
    acc[0] = bf16lo(xb.x); acc[1] = bf16hi(xb.x); acc[2] = bf16lo(xb.y); acc[3] = bf16hi(xb.y);
  }
  float4 rows[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    rows[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (rix[k] >= 0) rows[k] = *reinterpret_cast<const float4*>(sout + size_t(rix[k]) * H + h);
    else wts[k] = 0.f;
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    acc[0] = __fadd_rn(acc[0], __fmul_rn(wts[k], rows[k].x)); acc[1] = __fadd_rn(acc[1], __fmul_rn(wts[k], rows[k].y));
    acc[2] = __fadd_rn(acc[2], __fmul_rn(wts[k], rows[k].z)); acc[3] = __fadd_rn(acc[3], __fmul_rn(wts[k], rows[k].w));
  }
  for (int k = 8; k < K; ++k) {
    const int r = loc[size_t(k) * T + t];
    if (r < 0) continue;
    const float4 d = *reinterpret_cast<const float4*>(sout + size_t(r) * H + h);
    const float wk = rw[size_t(t) * K + k];
    acc[0] = __fadd_rn(acc[0], __fmul_rn(wk, d.x)); acc[1] = __fadd_rn(acc[1], __fmul_rn(wk, d.y));
    acc[2] = __fadd_rn(acc[2], __fmul_rn(wk, d.z)); acc[3] = __fadd_rn(acc[3], __fmul_rn(wk, d.w));
  }
  if (partial) {
    *reinterpret_cast<float4*>(partial + size_t(t) * H + h) = make_float4(acc[0], acc[1], acc[2], acc[3]);
  } else {
    uint2 o;
    o.x = pack_bf16(acc[0], acc[1]);
    o.y = pack_bf16(acc[2], acc[3]);
    *reinterpret_cast<uint2*>(out + size_t(t) * H + h) = o;
  }
}

bool moe_experts_tiled_ok(int64_t T, int64_t K, int64_t NE, int64_t H, int64_t FE) {
  return T >= 1 && T * K <= MD_MAX_PAIRS && NE <= 1024 && NE * ((T + 31) / 32) <= MD_MAX_WORDS && H % 512 == 0 &&
         FE % 512 == 0;
}

int moe_experts_tiled(Call& c, const Tensor& h2, const Tensor& base, const Tensor& ids, const Tensor& rw,
                      const Tensor& egw, const Tensor& edw, const Tensor& egs, const Tensor& eds, const Tensor& ebase,
                      const Tensor& out, const Tensor& partial) {
  const int64_t NE = egw.s[0], FE = egw.s[1] / 2, H = egw.s[2] * 2, T = ids.s[0], K = ids.s[1], P = T * K;
  Q35_REQUIRE(egs.numel() == NE * 2 * FE * (H / 32) && eds.numel() == NE * H * (FE / 32), Q35_ERR_SHAPE,
              "moe.experts: tiled scale tensors must hold as many bytes as the scales they were made from");
  const int64_t max_blocks = (NE < P ? NE : P) + P / MD_NB + 1, R = max_blocks * MD_NB;
  auto carve = [&](WsCut& w, int*& g_plane, int*& g_n, int*& g_row0, int*& active, int*& ready, int*& loc,
                   uint8_t*& q1h, uint8_t*& q1l, uint8_t*& sfb1, uint8_t*& q2h, uint8_t*& q2l, uint8_t*& sfb2, float*& sout) {
    g_plane = w.take<int>(NE); g_n = w.take<int>(NE); g_row0 = w.take<int>(NE);
    active = w.take<int>(NE + 1); ready = w.take<int>(NE); loc = w.take<int>(K * T);
    q1h = w.take<uint8_t>(R * H); q1l = w.take<uint8_t>(R * H);
    sfb1 = w.take<uint8_t>(max_blocks * (H / 128) * MD_SF_BYTES);
    q2h = w.take<uint8_t>(R * FE); q2l = w.take<uint8_t>(R * FE);
    sfb2 = w.take<uint8_t>(max_blocks * (FE / 128) * MD_SF_BYTES);
    sout = w.take<float>(R * H);
  };
  int *g_plane, *g_n, *g_row0, *active, *ready, *loc;
  uint8_t *q1h, *q1l, *sfb1, *q2h, *q2l, *sfb2;
  float* sout;
  WsCut cut{nullptr};
  carve(cut, g_plane, g_n, g_row0, active, ready, loc, q1h, q1l, sfb1, q2h, q2l, sfb2, sout);
  Tensor ws;
  Q35_TRY(c.workspace(cut.off, &ws));
  if (c.dry || T == 0) return 0;
  Q35_REQUIRE(aligned16(h2.p) && (uintptr_t(egw.p) & 31) == 0 && (uintptr_t(edw.p) & 31) == 0 && aligned16(egs.p) &&
                  aligned16(eds.p) && (partial.present ? aligned16(partial.p) : aligned16(base.p) && aligned16(out.p)),
              Q35_ERR_ALIGN, "moe.experts: pointers must be 16-byte aligned (FP4 planes 32)");
  WsCut wc{ws.as<uint8_t>()};
  carve(wc, g_plane, g_n, g_row0, active, ready, loc, q1h, q1l, sfb1, q2h, q2l, sfb2, sout);
  cudaStream_t st = c.stream;
  launch_pdl(moe_plan_kernel, dim3(1), dim3(1024), 0, st, (const int*)ids.as<int>(),
             (const int*)(ebase.present ? ebase.as<int>() : nullptr), int(T), int(K), int(NE), g_plane, g_n, g_row0, active,
             ready, loc, device_status_ptr());
  Q35_CUDA_LAUNCH_CHECK("moe.experts plan");
  const long long pieces = (long long)P * (H / 8);
  launch_pdl(moe_decode_quant_kernel, dim3(unsigned((pieces + 255) / 256)), dim3(256), 0, st,
             (const __nv_bfloat16*)h2.as<__nv_bfloat16>(), (const int*)loc, int(P), int(T), int(H), q1h, q1l, sfb1);
  Q35_CUDA_LAUNCH_CHECK("moe.experts quantise");
  CUtensorMap m_wg, m_wd, m_x1h, m_x1l, m_x2h, m_x2l;
  Q35_TRY(tc_make_map(&m_wg, true, egw.p, uint64_t(NE * 2 * FE), uint64_t(H), uint64_t(H / 2), 64, "e_gw"));
  Q35_TRY(tc_make_map(&m_wd, true, edw.p, uint64_t(NE * H), uint64_t(FE), uint64_t(FE / 2), 64, "e_dw"));
  Q35_TRY(tc_make_map(&m_x1h, false, q1h, uint64_t(R), uint64_t(H), uint64_t(H), MD_NB, "activations"));
  Q35_TRY(tc_make_map(&m_x1l, false, q1l, uint64_t(R), uint64_t(H), uint64_t(H), MD_NB, "activations"));
  Q35_TRY(tc_make_map(&m_x2h, false, q2h, uint64_t(R), uint64_t(FE), uint64_t(FE), MD_NB, "activations"));
  Q35_TRY(tc_make_map(&m_x2l, false, q2l, uint64_t(R), uint64_t(FE), uint64_t(FE), MD_NB, "activations"));
  MdArgs a{};
  a.g_plane = g_plane; a.g_n = g_n; a.g_row0 = g_row0; a.active = active; a.ready = ready;
  a.n_planes = int(NE); a.H = int(H); a.FE = int(FE);
  a.ratio = int(H / FE) < 1 ? 1 : int(H / FE);
  a.gs_t = egs.as<uint8_t>(); a.ds_t = eds.as<uint8_t>();
  a.sfb1 = sfb1; a.q2h = q2h; a.q2l = q2l; a.sfb2 = sfb2; a.sout = sout; a.status = device_status_ptr();
  int grid = 0;
  Q35_TRY(md_grid(&grid));
  // a group may hold more than one token tile here, but every CTA's item count is what matters for the table
  const int64_t max_items = NE * (FE / 64 + H / 128);
  Q35_REQUIRE((max_items + grid - 1) / grid + a.ratio + 2 <= MD_MAX_ITEMS, Q35_ERR_UNSUPPORTED,
              "moe.experts: %lld work items over %d CTAs exceed the per-CTA item table", (long long)max_items, grid);
  launch_pdl(moe_decode_kernel, dim3(unsigned(grid)), dim3(MD_THREADS), size_t(MD_SMEM), st, m_wg, m_wd, m_wg, m_wg, m_wd,
             m_x1h, m_x1l, m_x2h, m_x2l, a);
  Q35_CUDA_LAUNCH_CHECK("moe.experts gate-up + down");
  launch_pdl(moe_rows_combine_kernel, dim3(unsigned(T), unsigned((H / 4 + 255) / 256)), dim3(256), 0, st,
             (const __nv_bfloat16*)(partial.present ? nullptr : base.as<__nv_bfloat16>()), (const float*)rw.as<float>(),
             (const int*)loc, (const float*)sout, partial.present ? nullptr : out.as<__nv_bfloat16>(),
             partial.present ? partial.as<float>() : nullptr, int(T), int(H), int(K));
  Q35_CUDA_LAUNCH_CHECK("moe.experts combine");
  return 0;
}

// moe.front: the head of the block on a decode-sized batch in ONE launch -- RMSNorm, router logits, shared-expert gate
// dot, softmax, top-k, routing weights (moe_pre's first half + route, models/qwen35_2b/whole/src/q35_moe.py:123-137,
// 293-297) -- for hosts that put something of their own between routing and the experts (the expert-parallel step
// exchanges rows between GPUs there).  The same kernel as moe.block's first launch; its slot plan goes to scratch.
int run_moe_front(Call& c) {
  Tensor x1, ln2, wr, wshg, h2o, lg, gt, ids, rw, ws;
  Q35_TRY(c.get("x1", M(Q35_BF16), &x1));
  Q35_TRY(c.get("ln2", M(Q35_F32), &ln2));
  Q35_TRY(c.get("w_router", M(Q35_BF16), &wr));
  Q35_TRY(c.get("w_shg", M(Q35_BF16), &wshg, false));
  Q35_TRY(c.get("h2_out", M(Q35_BF16), &h2o));
  Q35_TRY(c.get("logits_out", M(Q35_F32), &lg));
  Q35_TRY(c.get("gate_out", M(Q35_F32), &gt, false));
  Q35_TRY(c.get("ids", M(Q35_I32), &ids));
  Q35_TRY(c.get("rw", M(Q35_F32), &rw));
  Q35_REQUIRE(x1.nd == 2 && wr.nd == 2 && ids.nd == 2, Q35_ERR_SHAPE, "moe.front: x1 [T, H], w_router [NE, H], ids [T, K]");
  const int64_t T = x1.s[0], H = x1.s[1], NE = wr.s[0], K = ids.s[1];
  const bool has_shared = wshg.present;
  Q35_REQUIRE(wr.s[1] == H && ln2.numel() == H && h2o.numel() == T * H && lg.numel() == T * NE && ids.s[0] == T &&
                  rw.numel() == T * K && (!has_shared || (wshg.numel() == H && gt.present && gt.numel() == T)),
              Q35_ERR_SHAPE, "moe.front: shapes (w_shg [H] goes with gate_out [T])");
  Q35_REQUIRE(H % 512 == 0 && H <= NR_MAX_H && K >= 1 && K <= 32 && K <= NE && NE + 1 <= 1024, Q35_ERR_UNSUPPORTED,
              "moe.front: H a multiple of 512 up to 8192, K <= 32, NE < 1024");
  const int64_t P = T * K, W = (T + 31) / 32;
  Q35_REQUIRE(T >= 1 && P <= MD_MAX_PAIRS && NE * W <= MD_MAX_WORDS, Q35_ERR_UNSUPPORTED,
              "moe.front: decode-sized batches only (T * K <= 4096)");
  const int64_t groups = NE + (T + MD_NB - 1) / MD_NB;
  WsCut cut{nullptr};
  int *counters, *g_plane, *g_n, *g_row0, *active, *ready, *loc;
  float* gate;
  auto carve = [&](WsCut& w) {
    counters = w.take<int>(T + 1);
    g_plane = w.take<int>(groups); g_n = w.take<int>(groups); g_row0 = w.take<int>(groups);
    active = w.take<int>(groups + 1); ready = w.take<int>(groups); loc = w.take<int>((K + 1) * T);
    gate = w.take<float>(T);
  };
  carve(cut);
  Q35_TRY(c.workspace(cut.off, &ws));
  if (c.dry) return 0;
  Q35_REQUIRE(aligned16(x1.p) && aligned16(wr.p) && aligned16(ln2.p) && aligned16(h2o.p) &&
                  (!has_shared || aligned16(wshg.p)), Q35_ERR_ALIGN, "moe.front: pointers must be 16-byte aligned");
  WsCut wc{ws.as<uint8_t>()};
  carve(wc);
  if (gt.present) gate = gt.as<float>();
  const int tok_per = NR_TOK / int((H + 2047) / 2048);
  const int tgroups = int((T + tok_per - 1) / tok_per);
  cudaMemsetAsync(counters, 0, size_t(tgroups + 1) * sizeof(int), c.stream);
  const int max_slices = int((NE + 1 + 7) / 8);
  int slices = (4 * sm_count() + tgroups - 1) / tgroups;
  slices = slices < 1 ? 1 : slices > max_slices ? max_slices : slices;
#define Q35_FRONT(PER)                                                                                                \
  launch_pdl(moe_front_kernel<PER>, dim3(unsigned(tgroups), unsigned(slices)), dim3(256), 0, c.stream,                 \
             x1.as<__nv_bfloat16>(), ln2.as<float>(), wr.as<__nv_bfloat16>(),                                          \
             has_shared ? wshg.as<__nv_bfloat16>() : wr.as<__nv_bfloat16>(), h2o.as<__nv_bfloat16>(), lg.as<float>(),  \
             gate, int(H), int(NE), 1e-6f, int(T), int(K), int(has_shared), tok_per, ids.as<int>(), rw.as<float>(),    \
             counters, g_plane, g_n, g_row0, active, ready, loc)
  if (NE <= 256) Q35_FRONT(8);
  else Q35_FRONT(32);
#undef Q35_FRONT
  Q35_CUDA_LAUNCH_CHECK("moe.front");
  return 0;
}

// moe.block: the whole block on a decode-sized batch.  Needs the tiled scale tensors (mx.tile_scales.*) of the routed
// and, when bound, the shared expert; MXFP4 everywhere; H and FE multiples of 512; shared intermediate size == FE.
int run_moe_block(Call& c) {
  Tensor x1, ln2, wr, wshg, wg, wu, wd, sgs, sds, egw, edw, egs, eds, out, ids, rw, lg, h2o, ws;
  Q35_TRY(c.get("x1", M(Q35_BF16), &x1));
  Q35_TRY(c.get("ln2", M(Q35_F32), &ln2));
  Q35_TRY(c.get("w_router", M(Q35_BF16), &wr));
  Q35_TRY(c.get("w_shg", M(Q35_BF16), &wshg, false));
  Q35_TRY(c.get("w_gate", M_BYTES, &wg, false));
  Q35_TRY(c.get("w_up", M_BYTES, &wu, false));
  Q35_TRY(c.get("w_down", M_BYTES, &wd, false));
  Q35_TRY(c.get("s_gate_up_tiled", M(Q35_U8), &sgs, false));
  Q35_TRY(c.get("s_down_tiled", M(Q35_U8), &sds, false));
  Q35_TRY(c.get("e_gw", M_BYTES, &egw));
  Q35_TRY(c.get("e_dw", M_BYTES, &edw));
  Q35_TRY(c.get("e_gs_tiled", M(Q35_U8), &egs));
  Q35_TRY(c.get("e_ds_tiled", M(Q35_U8), &eds));
  Q35_TRY(c.get("out", M(Q35_BF16), &out));
  Q35_TRY(c.get("ids", M(Q35_I32), &ids));
  Q35_TRY(c.get("rw", M(Q35_F32), &rw));
  Q35_TRY(c.get("logits_out", M(Q35_F32), &lg, false));
  Q35_TRY(c.get("h2_out", M(Q35_BF16), &h2o, false));
  Q35_REQUIRE(x1.nd == 2 && wr.nd == 2 && egw.nd == 3 && edw.nd == 3 && ids.nd == 2, Q35_ERR_SHAPE,
              "moe.block: x1 [T, H], w_router [NE, H], e_gw [NE, 2FE, H/2], e_dw [NE, H, FE/2], ids [T, K]");
  const int64_t T = x1.s[0], H = x1.s[1], NE = wr.s[0], FE = egw.s[1] / 2, K = ids.s[1];
  const bool has_shared = wg.present;
  Q35_REQUIRE(wr.s[1] == H && ln2.numel() == H && egw.s[0] == NE && egw.s[2] == H / 2 && edw.s[0] == NE &&
                  edw.s[1] == H && edw.s[2] == FE / 2,
              Q35_ERR_SHAPE, "moe.block: expert plane shapes");
  Q35_REQUIRE(egs.numel() == NE * 2 * FE * (H / 32) && eds.numel() == NE * H * (FE / 32), Q35_ERR_SHAPE,
              "moe.block: tiled scale tensors must hold as many bytes as the scales they were made from");
  Q35_REQUIRE(out.numel() == T * H && ids.s[0] == T && rw.numel() == T * K, Q35_ERR_SHAPE, "moe.block: out [T, H], ids / rw [T, K]");
  Q35_REQUIRE(!lg.present || lg.numel() == T * NE, Q35_ERR_SHAPE, "moe.block: logits_out [T, NE]");
  Q35_REQUIRE(!h2o.present || h2o.numel() == T * H, Q35_ERR_SHAPE, "moe.block: h2_out [T, H]");
  if (has_shared) {
    Q35_REQUIRE(wu.present && wd.present && sgs.present && sds.present && wshg.present, Q35_ERR_MISSING,
                "moe.block: the shared expert needs w_gate, w_up, w_down, s_gate_up_tiled, s_down_tiled and w_shg");
    Q35_REQUIRE(wg.nd == 2 && wg.s[0] == FE && wg.s[1] == H / 2 && wu.numel() == wg.numel() && wd.nd == 2 &&
                    wd.s[0] == H && wd.s[1] == FE / 2 && wshg.numel() == H,
                Q35_ERR_UNSUPPORTED, "moe.block: the shared expert must have the routed experts' shape (FS == FE)");
    Q35_REQUIRE(sgs.numel() == 2 * FE * (H / 32) && sds.numel() == H * (FE / 32), Q35_ERR_SHAPE,
                "moe.block: tiled shared-expert scales");
  }
  Q35_REQUIRE(H % 512 == 0 && FE % 512 == 0 && H <= NR_MAX_H, Q35_ERR_UNSUPPORTED,
              "moe.block: H and FE must be multiples of 512 (H <= 8192)");
  Q35_REQUIRE(K >= 1 && K <= 32 && K <= NE && NE + 1 <= 1024, Q35_ERR_UNSUPPORTED, "moe.block: K / NE out of range");
  const int64_t P = T * K, W = (T + 31) / 32;
  Q35_REQUIRE(T >= 1 && P <= MD_MAX_PAIRS && NE * W <= MD_MAX_WORDS, Q35_ERR_UNSUPPORTED,
              "moe.block: decode-sized batches only (T * K <= 4096); larger ones take moe.pre / moe.experts");
  const int64_t groups = NE + (T + MD_NB - 1) / MD_NB;  // routed experts + the shared expert's 16-token groups
  const int64_t max_blocks = (NE < P ? NE : P) + P / MD_NB + (T + MD_NB - 1) / MD_NB + 1;
  const int64_t R = max_blocks * MD_NB;
  const int64_t n_pairs = (K + (has_shared ? 1 : 0)) * T;
  WsCut cut{nullptr};
  int* counters = nullptr;
  auto carve = [&](WsCut& w, int*& g_plane, int*& g_n, int*& g_row0, int*& active, int*& ready, int*& loc, float*& gate,
                   float*& logits, __nv_bfloat16*& h2, uint8_t*& q1h, uint8_t*& q1l, uint8_t*& sfb1, uint8_t*& q2h,
                   uint8_t*& q2l, uint8_t*& sfb2, float*& sout) {
    counters = w.take<int>(T + 1);
    g_plane = w.take<int>(groups); g_n = w.take<int>(groups); g_row0 = w.take<int>(groups);
    active = w.take<int>(groups + 1); ready = w.take<int>(groups); loc = w.take<int>((K + 1) * T);
    gate = w.take<float>(T); logits = w.take<float>(T * NE); h2 = w.take<__nv_bfloat16>(T * H);
    q1h = w.take<uint8_t>(R * H); q1l = w.take<uint8_t>(R * H);
    sfb1 = w.take<uint8_t>(max_blocks * (H / 128) * MD_SF_BYTES);
    q2h = w.take<uint8_t>(R * FE); q2l = w.take<uint8_t>(R * FE);
    sfb2 = w.take<uint8_t>(max_blocks * (FE / 128) * MD_SF_BYTES);
    sout = w.take<float>(R * H);
  };
  int *g_plane, *g_n, *g_row0, *active, *ready, *loc;
  float *gate, *logits, *sout;
  __nv_bfloat16* h2;
  uint8_t *q1h, *q1l, *sfb1, *q2h, *q2l, *sfb2;
  carve(cut, g_plane, g_n, g_row0, active, ready, loc, gate, logits, h2, q1h, q1l, sfb1, q2h, q2l, sfb2, sout);
  Q35_TRY(c.workspace(cut.off, &ws));
  if (c.dry) return 0;
  Q35_REQUIRE(aligned16(x1.p) && aligned16(out.p) && aligned16(wr.p) && aligned16(ln2.p) && (uintptr_t(egw.p) & 31) == 0 &&
                  (uintptr_t(edw.p) & 31) == 0 && aligned16(egs.p) && aligned16(eds.p) &&
                  (!has_shared || ((uintptr_t(wg.p) & 31) == 0 && (uintptr_t(wu.p) & 31) == 0 &&
                                   (uintptr_t(wd.p) & 31) == 0 && aligned16(sgs.p) && aligned16(sds.p) && aligned16(wshg.p))),
              Q35_ERR_ALIGN, "moe.block: pointers must be 16-byte aligned (FP4 planes 32)");
  WsCut wc{ws.as<uint8_t>()};
  carve(wc, g_plane, g_n, g_row0, active, ready, loc, gate, logits, h2, q1h, q1l, sfb1, q2h, q2l, sfb2, sout);
  if (lg.present) logits = lg.as<float>();
  if (h2o.present) h2 = h2o.as<__nv_bfloat16>();
  cudaStream_t st = c.stream;

  // 1. norm + router + route + plan
  const int tok_per = NR_TOK / int((H + 2047) / 2048);  // four 16-byte pieces a thread hold the CTA's token rows
  const int tgroups = int((T + tok_per - 1) / tok_per);
  cudaMemsetAsync(counters, 0, size_t(tgroups + 1) * sizeof(int), st);  // the "who finishes last" counters start at zero
  const int max_slices = int((NE + 1 + 7) / 8);  // at least eight rows (one per warp) per CTA
  int slices = (4 * sm_count() + tgroups - 1) / tgroups;
  slices = slices < 1 ? 1 : slices > max_slices ? max_slices : slices;
#define Q35_FRONT(PER)                                                                                                \
  launch_pdl(moe_front_kernel<PER>, dim3(unsigned(tgroups), unsigned(slices)), dim3(256), 0, st,                       \
             x1.as<__nv_bfloat16>(), ln2.as<float>(), wr.as<__nv_bfloat16>(),                                          \
             has_shared ? wshg.as<__nv_bfloat16>() : wr.as<__nv_bfloat16>(), h2, logits, gate, int(H), int(NE), 1e-6f, \
             int(T), int(K), int(has_shared), tok_per, ids.as<int>(), rw.as<float>(), counters, g_plane, g_n, g_row0,   \
             active, ready, loc)
  if (NE <= 256) Q35_FRONT(8);
  else Q35_FRONT(32);
#undef Q35_FRONT
  Q35_CUDA_LAUNCH_CHECK("moe.block norm + router + route + plan");
  // 2. gather + quantise
  const long long pieces = (long long)n_pairs * (H / 8);
  launch_pdl(moe_decode_quant_kernel, dim3(unsigned((pieces + 255) / 256)), dim3(256), 0, st, (const __nv_bfloat16*)h2,
             (const int*)loc, int(n_pairs), int(T), int(H), q1h, q1l, sfb1);
  Q35_CUDA_LAUNCH_CHECK("moe.block quantise");
  // 3. gate-up + down
  CUtensorMap m_wg, m_wd, m_sg, m_su, m_sd, m_x1h, m_x1l, m_x2h, m_x2l;
  Q35_TRY(tc_make_map(&m_wg, true, egw.p, uint64_t(NE * 2 * FE), uint64_t(H), uint64_t(H / 2), 64, "e_gw"));
  Q35_TRY(tc_make_map(&m_wd, true, edw.p, uint64_t(NE * H), uint64_t(FE), uint64_t(FE / 2), 64, "e_dw"));
  if (has_shared) {
    Q35_TRY(tc_make_map(&m_sg, true, wg.p, uint64_t(FE), uint64_t(H), uint64_t(H / 2), 64, "w_gate"));
    Q35_TRY(tc_make_map(&m_su, true, wu.p, uint64_t(FE), uint64_t(H), uint64_t(H / 2), 64, "w_up"));
    Q35_TRY(tc_make_map(&m_sd, true, wd.p, uint64_t(H), uint64_t(FE), uint64_t(FE / 2), 64, "w_down"));
  } else {
    m_sg = m_su = m_wg; m_sd = m_wd;
  }
  Q35_TRY(tc_make_map(&m_x1h, false, q1h, uint64_t(R), uint64_t(H), uint64_t(H), MD_NB, "activations"));
  Q35_TRY(tc_make_map(&m_x1l, false, q1l, uint64_t(R), uint64_t(H), uint64_t(H), MD_NB, "activations"));
  Q35_TRY(tc_make_map(&m_x2h, false, q2h, uint64_t(R), uint64_t(FE), uint64_t(FE), MD_NB, "activations"));
  Q35_TRY(tc_make_map(&m_x2l, false, q2l, uint64_t(R), uint64_t(FE), uint64_t(FE), MD_NB, "activations"));
  MdArgs a{};
  a.g_plane = g_plane; a.g_n = g_n; a.g_row0 = g_row0; a.active = active; a.ready = ready;
  a.n_planes = int(NE); a.H = int(H); a.FE = int(FE);
  a.ratio = int(H / FE) < 1 ? 1 : int(H / FE);
  a.gs_t = egs.as<uint8_t>(); a.ds_t = eds.as<uint8_t>();
  a.sgs_t = has_shared ? sgs.as<uint8_t>() : nullptr; a.sds_t = has_shared ? sds.as<uint8_t>() : nullptr;
  a.sfb1 = sfb1; a.q2h = q2h; a.q2l = q2l; a.sfb2 = sfb2; a.sout = sout; a.status = device_status_ptr();
  int grid = 0;
  Q35_TRY(md_grid(&grid));
  const int64_t max_items = groups * (FE / 64 + H / 128);
  Q35_REQUIRE((max_items + grid - 1) / grid + a.ratio + 2 <= MD_MAX_ITEMS, Q35_ERR_UNSUPPORTED,
              "moe.block: %lld work items over %d CTAs exceed the per-CTA item table", (long long)max_items, grid);
  launch_pdl(moe_decode_kernel, dim3(unsigned(grid)), dim3(MD_THREADS), size_t(MD_SMEM), st, m_wg, m_wd, m_sg, m_su, m_sd,
             m_x1h, m_x1l, m_x2h, m_x2l, a);
  Q35_CUDA_LAUNCH_CHECK("moe.block experts");
  // 4. combine
  launch_pdl(moe_block_combine_kernel, dim3(unsigned(T), unsigned((H / 4 + 255) / 256)), dim3(256), 0, st,
             x1.as<__nv_bfloat16>(), (const float*)gate, (const float*)rw.as<float>(), (const int*)loc, (const float*)sout,
             out.as<__nv_bfloat16>(), int(T), int(H), int(K), int(has_shared));
  Q35_CUDA_LAUNCH_CHECK("moe.block combine");
  return 0;
}

}  // namespace q35
