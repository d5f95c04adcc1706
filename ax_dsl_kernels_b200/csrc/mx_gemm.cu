// Launchers of the weight-streaming GEMM: routed experts (decode and slot form), the dense part of the MoE block
// (RMSNorm, shared expert, router), and plain quantised projections.
#include "abi.h"
#include "common.cuh"
#include "moe_group.cuh"
#include "mx_gemm.cuh"
#include "tc_gemm.cuh"
#include "tc_host.h"

namespace q35 {

static inline int64_t align_up(int64_t x, int64_t a) { return (x + a - 1) / a * a; }

struct WsCarver {
  uint8_t* base;
  int64_t off = 0;
  template <class T> T* take(int64_t count) {
    T* p = base ? reinterpret_cast<T*>(base + off) : nullptr;
    off = align_up(off + count * int64_t(sizeof(T)), 256);
    return p;
  }
};

template <int FMT, int EPI>
static int launch_skinny(const SkinnyArgs& a, int nt, int tiles, int groups, cudaStream_t stream) {
  const dim3 grid{unsigned(tiles), unsigned(groups), 1u};
#define Q35_SK(NTV)                                                                                         \
  {                                                                                                         \
    constexpr int smem = skinny_smem_bytes<FMT, NTV>();                                                     \
    Q35_TRY(ensure_dynamic_smem(reinterpret_cast<const void*>(skinny_gemm_kernel<FMT, EPI, NTV>), smem));  \
    skinny_gemm_kernel<FMT, EPI, NTV><<<grid, 128, smem, stream>>>(a);                                      \
  }
  if (nt <= 1) Q35_SK(1)
  else if (nt == 2) Q35_SK(2)
  else Q35_SK(4)
#undef Q35_SK
  Q35_CUDA_LAUNCH_CHECK("skinny gemm");
  return 0;
}

static int pick_nt(int64_t rows_per_group) { return rows_per_group <= 8 ? 1 : rows_per_group <= 16 ? 2 : 4; }

// ---------------------------------------------------------------------------------------------------------------
// Routed experts on the tensor cores: quantise the gathered activation rows, gate-up GEMM with SiLU * up epilogue,
// quantise the bf16 activations, down GEMM scaled by the routing weight.  Used when H and FE are multiples of 512
// (every Qwen3.5 MoE shape); other shapes take the CUDA-core weight-streaming kernel.
struct ExpertPlanes {
  const uint8_t *gw, *gs, *dw, *ds;
  int64_t NE, FE, H;
};

static bool tc_shapes_ok(int64_t H, int64_t FE) { return H % 512 == 0 && FE % 512 == 0; }

static int64_t tc_routed_bytes(int64_t R, int64_t H, int64_t FE, int64_t groups = 0) {
  return tc_quant_bytes(R, H) + tc_quant_bytes(R, FE) + (groups + 1) * 4 + 256;
}

// [0] = number of groups with rows, [1..] = their indices in group order
static int* tc_routed_active(uint8_t* qws, int64_t R, int64_t H, int64_t FE) {
  return reinterpret_cast<int*>(qws + (tc_quant_bytes(R, H) + tc_quant_bytes(R, FE) + 255) / 256 * 256);
}

static int tc_routed(const ExpertPlanes& e, const __nv_bfloat16* x, int x_rows, const int* src, int R, int groups,
                     const int* g_expert, const int* g_n, const int* g_row0, int nb, __nv_bfloat16* act,
                     uint8_t* qws, float* f_out, __nv_bfloat16* b_out, const float* rw_row, cudaStream_t stream,
                     bool active_ready = false) {
  const TcQuant q1 = tc_quant_carve(qws, R, e.H);
  const TcQuant q2 = tc_quant_carve(qws + tc_quant_bytes(R, e.H), R, e.FE);
  int* active = tc_routed_active(qws, R, e.H, e.FE);
  if (!active_ready) Q35_TRY(tc_build_active(g_n, groups, active, stream));
  Q35_TRY(tc_quantize(x, int(e.H), src, x_rows, R, int(e.H), q1, stream));
  TcArgs a{};
  a.n_active = active; a.active = active + 1;
  a.g_expert = g_expert; a.g_n = g_n; a.g_row0 = g_row0; a.n_planes = int(e.NE);
  a.K = int(e.H);
  a.plane_rows[0] = a.plane_rows[1] = int(2 * e.FE);
  a.roff[0] = 0; a.roff[1] = int(e.FE); a.lim[0] = int(e.FE); a.lim[1] = int(2 * e.FE); a.tile_rows = 64;
  a.sw[0] = a.sw[1] = e.gs; a.s_plane = 2 * e.FE * (e.H / 32);
  a.act_rows = int(e.FE); a.act_out = act;
  const TcWeights wg{{e.gw, e.gw}, {uint64_t(e.NE * 2 * e.FE), uint64_t(e.NE * 2 * e.FE)}};
  Q35_TRY(tc_launch<TC_EPI_SILU_MUL>(wg, q1, a, nb, int(e.FE / 64), groups, stream));
  Q35_TRY(tc_quantize(act, int(e.FE), nullptr, R, R, int(e.FE), q2, stream));
  TcArgs d{};
  d.n_active = active; d.active = active + 1;
  d.g_expert = g_expert; d.g_n = g_n; d.g_row0 = g_row0; d.n_planes = int(e.NE);
  d.K = int(e.FE);
  d.plane_rows[0] = d.plane_rows[1] = int(e.H);
  d.roff[0] = 0; d.roff[1] = 64; d.lim[0] = d.lim[1] = int(e.H); d.tile_rows = 128;
  d.sw[0] = d.sw[1] = e.ds; d.s_plane = e.H * (e.FE / 32);
  d.f_out = f_out; d.b_out = b_out; d.out_stride = int(e.H); d.rw_row = rw_row;
  const TcWeights wd{{e.dw, e.dw}, {uint64_t(e.NE * e.H), uint64_t(e.NE * e.H)}};
  return tc_launch<TC_EPI_ROW_SCALE>(wd, q2, d, nb, int(e.H / 128), groups, stream);
}

// ---------------------------------------------------------------------------------------------------------------
// moe.experts: decode form of the routed experts with planar expert tensors.
// Reference: moe_experts_gu (models/qwen35_2b/whole/src/q35_moe.py:101-112) per token; golden :227-238; experts
// picked from planes by id as moe_full does (models/qwen35_2b/whole/src/q35_layer_mc.py:863-885).
// A token that lists the same expert twice gets ONE row for it, weighted by the sum of the two routing weights (the
// golden adds rw_i * d_i for every listed pair, models/qwen35_2b/whole/src/q35_moe.py:235-238: the same value up to
// fp32 rounding); the later listing's loc stays -1.  The one-CTA plan below follows the same rule.
__global__ void __launch_bounds__(256) experts_build_rows_kernel(const int* __restrict__ counts,
                                                                 const int* __restrict__ list,
                                                                 const int* __restrict__ ids,
                                                                 const int* __restrict__ base,
                                                                 const float* __restrict__ rw, int T, int K, int NE,
                                                                 int* g_expert, int* g_n, int* g_row0, int* src,
                                                                 float* rw_row, int* loc) {
  const int e = blockIdx.x, tid = threadIdx.x;
  __shared__ int s_red[256];
  int mine = 0;
  for (int i = tid; i < e; i += 256) mine += counts[i];
  s_red[tid] = mine;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (tid < o) s_red[tid] += s_red[tid + o];
    __syncthreads();
  }
  const int row0 = s_red[0];
  const int n = counts[e];
  if (tid == 0) { g_expert[e] = e; g_n[e] = n; g_row0[e] = row0; }
  for (int j = tid; j < n; j += 256) {
    const int p = list[size_t(e) * T + j];
    const int t = p / K, k = p % K;
    float wsum = rw[p];
    const int want = e + (base ? base[0] : 0);
    for (int kk = k + 1; kk < K; ++kk)
      if (ids[size_t(t) * K + kk] == want) wsum += rw[size_t(t) * K + kk];
    src[row0 + j] = t;
    rw_row[row0 + j] = wsum;
    loc[size_t(k) * T + t] = row0 + j;
  }
}

// Small form of the grouping (at most 4096 pairs, 1024 experts, experts x ceil(T / 32) <= 4096): one CTA does the count,
// the stable ranks, the row tables and the list of experts with rows that the tensor-core GEMM walks.  Same result as
// moe_group_count_kernel + experts_build_rows_kernel + the active-group scan; pairs without a local expert get loc -1.
// Every expert keeps a bitmap of the tokens that chose it; a pair's rank inside its expert is the number of set bits
// below its token (tokens ascending = the stable order), its expert's row count the number of set bits.
constexpr int PLAN_MAX_PAIRS = 4096, PLAN_MAX_WORDS = 4096;
__global__ void __launch_bounds__(1024) experts_plan_small_kernel(const int* __restrict__ ids,
                                                                  const int* __restrict__ base,
                                                                  const float* __restrict__ rw, int T, int K, int NE,
                                                                  int* g_expert, int* g_n, int* g_row0, int* src,
                                                                  float* rw_row, int* loc, int* active, int* status) {
  pdl_wait();
  pdl_launch();
  __shared__ short s_raw[PLAN_MAX_PAIRS];
  __shared__ uint32_t s_bits[PLAN_MAX_WORDS];
  __shared__ int s_row0[1024];
  __shared__ int s_warp[32];
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  const int P = T * K, W = (T + 31) / 32;
  const int first = base ? base[0] : 0;  // first global id of this rank's planes
  for (int p = tid; p < P; p += 1024) {
    int id = ids[p] - first;
    if (id >= NE) {
      if (!base) atomicOr(status, DS_BAD_EXPERT);
      id = -1;
    }
    s_raw[p] = short(id < 0 ? -1 : id);  // negative ids mean "not on this rank"
  }
  for (int i = tid; i < NE * W; i += 1024) s_bits[i] = 0u;
  __syncthreads();
  int myid[PLAN_MAX_PAIRS / 1024];
#pragma unroll
  for (int i = 0; i < PLAN_MAX_PAIRS / 1024; ++i) {
    const int p = tid + i * 1024;
    int id = -1;
    if (p < P) {
      const int t = p / K, k = p % K;
      id = s_raw[p];
      for (int kk = 0; kk < k && id >= 0; ++kk)
        if (s_raw[t * K + kk] == id) id = -1;  // listed twice: one row, the weights are summed on the first listing
      if (id >= 0) atomicOr(&s_bits[id * W + (t >> 5)], 1u << (t & 31));
    }
    myid[i] = id;
  }
  __syncthreads();
  // exclusive scan over the experts of (rows, has rows) packed as rows | on << 16
  int cnt = 0;
  if (tid < NE)
    for (int w = 0; w < W; ++w) cnt += __popc(s_bits[tid * W + w]);
  int v = cnt | (cnt > 0 ? 1 << 16 : 0);
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
    s_row0[tid] = exc & 0xffff;
    g_expert[tid] = tid; g_n[tid] = cnt; g_row0[tid] = exc & 0xffff;
    if (active && cnt > 0) active[1 + (exc >> 16)] = tid;
  }
  if (active && tid == 1023) active[0] = (exc + v) >> 16;
  __syncthreads();
#pragma unroll
  for (int i = 0; i < PLAN_MAX_PAIRS / 1024; ++i) {
    const int p = tid + i * 1024;
    if (p >= P) continue;
    const int t = p / K, k = p % K, id = myid[i];
    int row = -1;
    if (id >= 0) {
      int rank = __popc(s_bits[id * W + (t >> 5)] & ((1u << (t & 31)) - 1u));
      for (int w = 0; w < (t >> 5); ++w) rank += __popc(s_bits[id * W + w]);
      row = s_row0[id] + rank;
      float wsum = rw[p];
      for (int kk = k + 1; kk < K; ++kk)
        if (s_raw[t * K + kk] == id) wsum += rw[t * K + kk];
      src[row] = t;
      rw_row[row] = wsum;
    }
    loc[size_t(k) * T + t] = row;
  }
}

int run_moe_experts(Call& c) {
  Tensor h2, base, ids, rw, gw, gs, dw, ds, out, partial, ebase, ws;
  Q35_TRY(c.get("h2", M(Q35_BF16), &h2));
  Q35_TRY(c.get("partial_out", M(Q35_F32), &partial, false));  // expert-parallel form: fp32 sums, no base
  Q35_TRY(c.get("expert_base", M(Q35_I32), &ebase, false));    // ids are global, the planes start at this id
  Q35_TRY(c.get("base", M(Q35_BF16), &base, !partial.present));
  Q35_TRY(c.get("ids", M(Q35_I32), &ids));
  Q35_TRY(c.get("rw", M(Q35_F32), &rw));
  Tensor gs_t, ds_t;
  Q35_TRY(c.get("e_gs_tiled", M(Q35_U8), &gs_t, false));  // mx.tile_scales.* of the scales: the one-kernel decode form
  Q35_TRY(c.get("e_ds_tiled", M(Q35_U8), &ds_t, false));
  const bool tiled = gs_t.present && ds_t.present;
  Q35_TRY(c.get("e_gw", M_BYTES, &gw));
  Q35_TRY(c.get("e_gs", M(Q35_U8), &gs, !tiled));
  Q35_TRY(c.get("e_dw", M_BYTES, &dw));
  Q35_TRY(c.get("e_ds", M(Q35_U8), &ds, !tiled));
  Q35_TRY(c.get("out", M(Q35_BF16), &out, !partial.present));
  Q35_REQUIRE(gw.nd == 3 && dw.nd == 3 && ids.nd == 2, Q35_ERR_SHAPE, "moe.experts: expert planes must be rank 3, ids rank 2");
  if (tiled && moe_experts_tiled_ok(ids.s[0], ids.s[1], gw.s[0], gw.s[2] * 2, gw.s[1] / 2)) {
    const int64_t NE_ = gw.s[0], FE_ = gw.s[1] / 2, H_ = gw.s[2] * 2, T_ = ids.s[0], K_ = ids.s[1];
    Q35_REQUIRE(h2.numel() == T_ * H_ && rw.numel() == T_ * K_ && dw.s[0] == NE_ && dw.s[1] == H_ && dw.s[2] == FE_ / 2 &&
                    (partial.present ? partial.numel() == T_ * H_ : base.numel() == T_ * H_ && out.numel() == T_ * H_),
                Q35_ERR_SHAPE, "moe.experts: shapes");
    return moe_experts_tiled(c, h2, base, ids, rw, gw, dw, gs_t, ds_t, ebase, out, partial);
  }
  Q35_REQUIRE(gs.present && ds.present, Q35_ERR_MISSING, "moe.experts: e_gs / e_ds are needed for this shape");
  Q35_REQUIRE(gs.nd == 3 && ds.nd == 3, Q35_ERR_SHAPE, "moe.experts: scale planes must be rank 3");
  const int64_t NE = gw.s[0], FE2 = gw.s[1], H = gw.s[2] * 2, FE = FE2 / 2;
  const int64_t T = ids.s[0], K = ids.s[1];
  Q35_REQUIRE(h2.numel() == T * H, Q35_ERR_SHAPE, "moe.experts: h2 must be [T=%lld, H=%lld]", (long long)T, (long long)H);
  if (partial.present) {
    Q35_REQUIRE(partial.numel() == T * H, Q35_ERR_SHAPE, "moe.experts: partial_out must be [T, H]");
  } else {
    Q35_REQUIRE(base.numel() == T * H && out.numel() == T * H, Q35_ERR_SHAPE, "moe.experts: base / out must be [T, H]");
  }
  Q35_REQUIRE(rw.numel() == T * K, Q35_ERR_SHAPE, "moe.experts: rw must be [T, K]");
  Q35_REQUIRE(gs.s[0] == NE && gs.s[1] == FE2 && gs.s[2] == H / 32, Q35_ERR_SHAPE, "moe.experts: e_gs [NE, 2FE, H/32]");
  Q35_REQUIRE(dw.s[0] == NE && dw.s[1] == H && dw.s[2] == FE / 2, Q35_ERR_SHAPE, "moe.experts: e_dw [NE, H, FE/2]");
  Q35_REQUIRE(ds.s[0] == NE && ds.s[1] == H && ds.s[2] == FE / 32, Q35_ERR_SHAPE, "moe.experts: e_ds [NE, H, FE/32]");
  Q35_REQUIRE(H % 256 == 0 && FE % 256 == 0, Q35_ERR_UNSUPPORTED, "moe.experts: H and FE must be multiples of 256");
  const int64_t P = T * K;
  const bool use_tc = tc_shapes_ok(H, FE);
  uint8_t* qws = nullptr;
  WsCarver w{nullptr};
  auto carve = [&](WsCarver& cw, int*& counts, int*& list, int*& g_expert, int*& g_n, int*& g_row0, int*& src,
                   float*& rw_row, int*& loc, __nv_bfloat16*& act, float*& sout) {
    counts = cw.take<int>(NE); list = cw.take<int>(NE * T);
    g_expert = cw.take<int>(NE); g_n = cw.take<int>(NE); g_row0 = cw.take<int>(NE);
    src = cw.take<int>(P); rw_row = cw.take<float>(P); loc = cw.take<int>(P);
    act = cw.take<__nv_bfloat16>(P * FE); sout = cw.take<float>(P * H);
    qws = use_tc ? cw.take<uint8_t>(tc_routed_bytes(P, H, FE, NE)) : nullptr;
  };
  int *counts, *list, *g_expert, *g_n, *g_row0, *src, *loc;
  float *rw_row, *sout;
  __nv_bfloat16* act;
  carve(w, counts, list, g_expert, g_n, g_row0, src, rw_row, loc, act, sout);
  Q35_TRY(c.workspace(w.off, &ws));
  if (c.dry || T == 0) return 0;
  Q35_REQUIRE(aligned16(h2.p) && (partial.present ? aligned16(partial.p) : aligned16(base.p) && aligned16(out.p)) &&
                  aligned16(gw.p) && aligned16(dw.p) &&
                  (uintptr_t(gs.p) & 1) == 0 && (uintptr_t(ds.p) & 1) == 0,
              Q35_ERR_ALIGN, "moe.experts: pointers must be 16-byte aligned");
  WsCarver wr{ws.as<uint8_t>()};
  carve(wr, counts, list, g_expert, g_n, g_row0, src, rw_row, loc, act, sout);

  const bool small = P <= PLAN_MAX_PAIRS && NE <= 1024 && NE * ((T + 31) / 32) <= PLAN_MAX_WORDS;
  if (small) {
    launch_pdl(experts_plan_small_kernel, dim3(1), dim3(1024), 0, c.stream, ids.as<int>(),
               ebase.present ? ebase.as<int>() : nullptr, rw.as<float>(), int(T), int(K), int(NE), g_expert, g_n, g_row0,
               src, rw_row, loc, use_tc ? tc_routed_active(qws, P, H, FE) : nullptr, device_status_ptr());
    Q35_CUDA_LAUNCH_CHECK("moe.experts plan");
  } else {
    // pairs of other ranks, out-of-range ids and second listings of an expert: loc = -1 (moe.combine skips them)
    cudaMemsetAsync(loc, 0xff, size_t(P) * 4, c.stream);
    Q35_TRY(launch_group_count(ids.as<int>(), ebase.present ? ebase.as<int>() : nullptr, int(T), int(K), int(NE), counts,
                               list, c.stream));
    experts_build_rows_kernel<<<unsigned(NE), 256, 0, c.stream>>>(counts, list, ids.as<int>(),
                                                                  ebase.present ? ebase.as<int>() : nullptr,
                                                                  rw.as<float>(), int(T), int(K), int(NE), g_expert, g_n,
                                                                  g_row0, src, rw_row, loc);
    Q35_CUDA_LAUNCH_CHECK("moe.experts rows");
  }
  if (use_tc) {
    const ExpertPlanes ep{gw.as<uint8_t>(), gs.as<uint8_t>(), dw.as<uint8_t>(), ds.as<uint8_t>(), NE, FE, H};
    // Prefill-sized: the weighted expert rows are kept in bf16, as the reference's slot kernels emit them
    // (moe_slots_px out [S, G, H] bf16, models/qwen35_2b/whole/src/q35_moe_prefill.py:150-166), which halves the
    // largest write of the block; decode-sized calls keep the fp32 rows of the decode golden.
    const bool rows_f32 = P <= 4096;
    Q35_TRY(tc_routed(ep, h2.as<__nv_bfloat16>(), int(T), src, int(P), int(NE), g_expert, g_n, g_row0,
                      int((P + NE - 1) / NE), act, qws, rows_f32 ? sout : nullptr,
                      rows_f32 ? nullptr : reinterpret_cast<__nv_bfloat16*>(sout), rw_row, c.stream, small));
    if (partial.present)
      return launch_partial_sum(loc, sout, rows_f32, partial.as<float>(), int(T), int(H), int(K), int(P), c.stream);
    return launch_combine(base.as<__nv_bfloat16>(), loc, sout, rows_f32, out.as<__nv_bfloat16>(), int(T), int(H), int(K),
                          int(P), c.stream);
  }
  const int nt = pick_nt((P + NE - 1) / NE);
  SkinnyArgs a{};
  a.status = device_status_ptr();
  a.g_expert = g_expert; a.g_n = g_n; a.g_row0 = g_row0; a.n_planes = int(NE);
  // gate-up + SiLU * up -> act
  a.w[0] = a.w[1] = gw.as<uint8_t>(); a.s[0] = a.s[1] = gs.as<uint8_t>();
  a.w_plane = FE2 * (H / 2); a.s_plane = FE2 * (H / 32);
  a.K = int(H); a.roff[0] = 0; a.roff[1] = int(FE); a.lim[0] = int(FE); a.lim[1] = int(FE2);
  a.act_rows = int(FE); a.tile_rows = 64; a.warp_rows = 16;
  a.x = h2.as<__nv_bfloat16>(); a.x_stride = int(H); a.src = src; a.act_out = act;
  Q35_TRY((launch_skinny<W_MXFP4, EPI_SILU_MUL>(a, nt, int(FE / 64), int(NE), c.stream)));
  // down, scaled by the routing weight -> sout (fp32)
  SkinnyArgs d{};
  d.status = a.status;
  d.g_expert = g_expert; d.g_n = g_n; d.g_row0 = g_row0; d.n_planes = int(NE);
  d.w[0] = d.w[1] = dw.as<uint8_t>(); d.s[0] = d.s[1] = ds.as<uint8_t>();
  d.w_plane = H * (FE / 2); d.s_plane = H * (FE / 32);
  d.K = int(FE); d.roff[0] = 0; d.roff[1] = 16; d.lim[0] = d.lim[1] = int(H);
  d.tile_rows = 128; d.warp_rows = 32;
  d.x = act; d.x_stride = int(FE); d.src = nullptr;
  d.f_out = sout; d.out_stride = int(H); d.rw_row = rw_row;
  Q35_TRY((launch_skinny<W_MXFP4, EPI_ROW_SCALE>(d, nt, int((H + 127) / 128), int(NE), c.stream)));
  if (partial.present)
    return launch_partial_sum(loc, sout, true, partial.as<float>(), int(T), int(H), int(K), int(P), c.stream);
  return launch_combine(base.as<__nv_bfloat16>(), loc, sout, true, out.as<__nv_bfloat16>(), int(T), int(H), int(K),
                        int(P), c.stream);
}

// ---------------------------------------------------------------------------------------------------------------
// moe.slots: slot-grouped routed experts of a prefill group, reading rows out of h2 by token id
// (moe_slots_px, models/qwen35_2b/whole/src/q35_moe_prefill.py:150-166; golden :239-246).
__global__ void slots_build_groups_kernel(const int* __restrict__ tok, const int* n_slots, int S, int G, int T, int NE,
                                          int* g_expert, int* g_n, int* g_row0, int* src, int* status) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= S * G) return;
  const int s = idx / G, j = idx % G;
  int t = tok[size_t(s) * (1 + G) + 1 + j];
  if (t < 0 || t >= T) { atomicOr(status, DS_BAD_TOKEN); t = 0; }
  src[idx] = t;
  if (j == 0) {
    const bool used = !n_slots || s < n_slots[0];
    g_expert[s] = tok[size_t(s) * (1 + G)];
    g_n[s] = used ? G : 0;
    g_row0[s] = s * G;
  }
}

int run_moe_slots(Call& c) {
  Tensor h2, tok, rw, gw, gs, dw, ds, out, ns, ws;
  Q35_TRY(c.get("h2", M(Q35_BF16), &h2));
  Q35_TRY(c.get("tok", M(Q35_I32), &tok));
  Q35_TRY(c.get("rw", M(Q35_F32), &rw));
  Q35_TRY(c.get("e_gw", M_BYTES, &gw));
  Q35_TRY(c.get("e_gs", M(Q35_U8), &gs));
  Q35_TRY(c.get("e_dw", M_BYTES, &dw));
  Q35_TRY(c.get("e_ds", M(Q35_U8), &ds));
  Q35_TRY(c.get("out", M(Q35_BF16) | M(Q35_F32), &out));
  Q35_TRY(c.get("n_slots", M(Q35_I32), &ns, false));
  Q35_REQUIRE(gw.nd == 3 && gs.nd == 3 && dw.nd == 3 && ds.nd == 3 && tok.nd == 2 && h2.nd == 2, Q35_ERR_SHAPE,
              "moe.slots: ranks");
  const int64_t NE = gw.s[0], FE2 = gw.s[1], H = gw.s[2] * 2, FE = FE2 / 2;
  const int64_t S = tok.s[0], G = tok.s[1] - 1, T = h2.s[0];
  Q35_REQUIRE(G >= 1 && rw.numel() == S * G && out.numel() == S * G * H && h2.s[1] == H, Q35_ERR_SHAPE,
              "moe.slots: tok [S, 1+G], rw [S, G], out [S, G, H], h2 [T, H]");
  Q35_REQUIRE(gs.s[0] == NE && gs.s[1] == FE2 && gs.s[2] == H / 32 && dw.s[0] == NE && dw.s[1] == H &&
                  dw.s[2] == FE / 2 && ds.s[0] == NE && ds.s[1] == H && ds.s[2] == FE / 32,
              Q35_ERR_SHAPE, "moe.slots: expert plane shapes");
  Q35_REQUIRE(H % 256 == 0 && FE % 256 == 0, Q35_ERR_UNSUPPORTED, "moe.slots: H and FE must be multiples of 256");
  const bool use_tc = tc_shapes_ok(H, FE);
  uint8_t* qws = nullptr;
  WsCarver w{nullptr};
  auto carve = [&](WsCarver& cw, int*& g_expert, int*& g_n, int*& g_row0, int*& src, __nv_bfloat16*& act) {
    g_expert = cw.take<int>(S); g_n = cw.take<int>(S); g_row0 = cw.take<int>(S);
    src = cw.take<int>(S * G); act = cw.take<__nv_bfloat16>(S * G * FE);
    qws = use_tc ? cw.take<uint8_t>(tc_routed_bytes(S * G, H, FE, S)) : nullptr;
  };
  int *g_expert, *g_n, *g_row0, *src;
  __nv_bfloat16* act;
  carve(w, g_expert, g_n, g_row0, src, act);
  Q35_TRY(c.workspace(w.off, &ws));
  if (c.dry || S == 0) return 0;
  Q35_REQUIRE(aligned16(h2.p) && aligned16(out.p) && aligned16(gw.p) && aligned16(dw.p), Q35_ERR_ALIGN,
              "moe.slots: pointers must be 16-byte aligned");
  WsCarver wr{ws.as<uint8_t>()};
  carve(wr, g_expert, g_n, g_row0, src, act);
  if (ns.present) cudaMemsetAsync(out.p, 0, out.bytes, c.stream);  // rows of unused slots
  slots_build_groups_kernel<<<unsigned((S * G + 255) / 256), 256, 0, c.stream>>>(
      tok.as<int>(), ns.present ? ns.as<int>() : nullptr, int(S), int(G), int(T), int(NE), g_expert, g_n, g_row0, src,
      device_status_ptr());
  Q35_CUDA_LAUNCH_CHECK("moe.slots groups");
  if (use_tc) {
    const ExpertPlanes ep{gw.as<uint8_t>(), gs.as<uint8_t>(), dw.as<uint8_t>(), ds.as<uint8_t>(), NE, FE, H};
    return tc_routed(ep, h2.as<__nv_bfloat16>(), int(T), src, int(S * G), int(S), g_expert, g_n, g_row0, int(G), act, qws,
                     out.dtype == Q35_F32 ? out.as<float>() : nullptr,
                     out.dtype == Q35_F32 ? nullptr : out.as<__nv_bfloat16>(), rw.as<float>(), c.stream);
  }
  const int nt = pick_nt(G);
  SkinnyArgs a{};
  a.status = device_status_ptr();
  a.g_expert = g_expert; a.g_n = g_n; a.g_row0 = g_row0; a.n_planes = int(NE);
  a.w[0] = a.w[1] = gw.as<uint8_t>(); a.s[0] = a.s[1] = gs.as<uint8_t>();
  a.w_plane = FE2 * (H / 2); a.s_plane = FE2 * (H / 32);
  a.K = int(H); a.roff[0] = 0; a.roff[1] = int(FE); a.lim[0] = int(FE); a.lim[1] = int(FE2);
  a.act_rows = int(FE); a.tile_rows = 64; a.warp_rows = 16;
  a.x = h2.as<__nv_bfloat16>(); a.x_stride = int(H); a.src = src; a.act_out = act;
  Q35_TRY((launch_skinny<W_MXFP4, EPI_SILU_MUL>(a, nt, int(FE / 64), int(S), c.stream)));
  SkinnyArgs d{};
  d.status = a.status;
  d.g_expert = g_expert; d.g_n = g_n; d.g_row0 = g_row0; d.n_planes = int(NE);
  d.w[0] = d.w[1] = dw.as<uint8_t>(); d.s[0] = d.s[1] = ds.as<uint8_t>();
  d.w_plane = H * (FE / 2); d.s_plane = H * (FE / 32);
  d.K = int(FE); d.roff[0] = 0; d.roff[1] = 16; d.lim[0] = d.lim[1] = int(H);
  d.tile_rows = 128; d.warp_rows = 32;
  d.x = act; d.x_stride = int(FE); d.src = nullptr;
  if (out.dtype == Q35_F32) d.f_out = out.as<float>(); else d.b_out = out.as<__nv_bfloat16>();
  d.out_stride = int(H); d.rw_row = rw.as<float>();
  return launch_skinny<W_MXFP4, EPI_ROW_SCALE>(d, nt, int((H + 127) / 128), int(S), c.stream);
}

// ---------------------------------------------------------------------------------------------------------------
// moe.pre: dense part of the MoE block (moe_pre, models/qwen35_2b/whole/src/q35_moe.py:123-137):
// h2 = RMSNorm(x1) * ln2; base = bf16(x1 + sigmoid(h2 . w_shg) * shared_expert(h2)); logits = h2 @ w_router^T (fp32).
__global__ void __launch_bounds__(256) rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w,
                                                      __nv_bfloat16* __restrict__ y, int H, float eps) {
  pdl_wait();
  pdl_launch();
  const int t = blockIdx.x, tid = threadIdx.x;
  const __nv_bfloat16* xr = x + size_t(t) * H;
  __shared__ float s_red[8];
  const bool pieces = H <= 256 * 8 * RMS_MAX_PIECES && H % 8 == 0;  // the row fits the threads' registers
  RmsPieces p;
  float ss = 0.f;
  if (pieces) {
    rms_load(xr, H, tid, p);
    ss = rms_sumsq(p);
  } else {
    for (int i = tid; i < H; i += 256) { const float v = __bfloat162float(xr[i]); ss += v * v; }
  }
  ss = warp_sum(ss);
  if ((tid & 31) == 0) s_red[tid >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += s_red[i];
  const float rs = rsqrtf(tot / float(H) + eps);
  if (pieces) {
    rms_apply(p, H, tid, rs, w, y + size_t(t) * H, nullptr);
  } else {
    for (int i = tid; i < H; i += 256) y[size_t(t) * H + i] = __float2bfloat16_rn(__bfloat162float(xr[i]) * rs * w[i]);
  }
}

// logits[t, e] = sum_k h2[t, k] * w_router[e, k] in fp32 (bf16 products are exact in fp32); row NE is the shared-
// expert gate vector.  One warp per (t, e); lanes stride k so the order of the sum is fixed.
__global__ void __launch_bounds__(256) router_kernel(const __nv_bfloat16* __restrict__ h2,
                                                     const __nv_bfloat16* __restrict__ w_router,
                                                     const __nv_bfloat16* __restrict__ w_shg,
                                                     float* __restrict__ logits, float* __restrict__ gate, int H, int NE) {
  pdl_wait();
  pdl_launch();
  const int t = blockIdx.y;
  const int e = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (e > NE) return;
  const __nv_bfloat16* wr = e < NE ? w_router + size_t(e) * H : w_shg;
  const __nv_bfloat16* xr = h2 + size_t(t) * H;
  float acc = 0.f;
  for (int k = lane * 8; k < H; k += 256) {
    const uint4 xv = *reinterpret_cast<const uint4*>(xr + k);
    const uint4 wv = *reinterpret_cast<const uint4*>(wr + k);
    acc = fmaf(bf16lo(xv.x), bf16lo(wv.x), acc); acc = fmaf(bf16hi(xv.x), bf16hi(wv.x), acc);
    acc = fmaf(bf16lo(xv.y), bf16lo(wv.y), acc); acc = fmaf(bf16hi(xv.y), bf16hi(wv.y), acc);
    acc = fmaf(bf16lo(xv.z), bf16lo(wv.z), acc); acc = fmaf(bf16hi(xv.z), bf16hi(wv.z), acc);
    acc = fmaf(bf16lo(xv.w), bf16lo(wv.w), acc); acc = fmaf(bf16hi(xv.w), bf16hi(wv.w), acc);
  }
  acc = warp_sum(acc);
  if (lane == 0) {
    if (e < NE) logits[size_t(t) * NE + e] = acc;
    else gate[t] = acc;
  }
}

// Prefill-sized router: the same logits [T, NE] (+ the shared-expert gate dot as column NE) as a bf16 tensor-core GEMM
// with fp32 accumulation -- bf16 products are exact in fp32, so only the order of the sum differs from router_kernel.
// CTA = 64 tokens x 64 router rows, 4 warps of 16 tokens each, K in chunks of 64 through a two-stage cp.async ring with
// XOR-swizzled 128-byte rows.
__global__ void __launch_bounds__(128) router_mma_kernel(const __nv_bfloat16* __restrict__ h2,
                                                         const __nv_bfloat16* __restrict__ w_router,
                                                         const __nv_bfloat16* __restrict__ w_shg,
                                                         float* __restrict__ logits, float* __restrict__ gate, int T,
                                                         int H, int NE) {
  pdl_wait();
  pdl_launch();
  __shared__ __align__(128) __nv_bfloat16 sA[2][64 * 64];
  __shared__ __align__(128) __nv_bfloat16 sB[2][64 * 64];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int t0 = blockIdx.x * 64, e0 = blockIdx.y * 64;
  auto stage_load = [&](int st, int k0) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int c = tid + i * 128, row = c >> 3, ch = c & 7;
      const int t = min(t0 + row, T - 1), e = e0 + row;  // rows past the end repeat a valid row and are not stored
      const __nv_bfloat16* wrow = e < NE ? w_router + size_t(e) * H : w_shg;
      const int dst = row * 64 + ((ch ^ (row & 7)) << 3);
      cp_async_16(smem_u32(&sA[st][dst]), h2 + size_t(t) * H + k0 + ch * 8);
      cp_async_16(smem_u32(&sB[st][dst]), wrow + k0 + ch * 8);
    }
    cp_async_commit();
  };
  float acc[8][4];
#pragma unroll
  for (int j = 0; j < 8; ++j) { acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f; }
  const int nk = H / 64;
  stage_load(0, 0);
  for (int kc = 0; kc < nk; ++kc) {
    if (kc + 1 < nk) { stage_load((kc + 1) & 1, (kc + 1) * 64); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
    __syncthreads();
    const __nv_bfloat16* A = sA[kc & 1];
    const __nv_bfloat16* B = sB[kc & 1];
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      uint32_t a0, a1, a2, a3;
      {
        const int row = warp * 16 + (lane & 15), ch = kk * 2 + (lane >> 4);
        ldmatrix_x4(smem_u32(A + row * 64 + ((ch ^ (row & 7)) << 3)), a0, a1, a2, a3);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {  // 16 router rows per ldmatrix: two n-tiles
        uint32_t b0, b1, b2, b3;
        const int row = j * 16 + (lane & 7) + ((lane >> 4) << 3), ch = kk * 2 + ((lane >> 3) & 1);
        ldmatrix_x4(smem_u32(B + row * 64 + ((ch ^ (row & 7)) << 3)), b0, b1, b2, b3);
        mma_bf16_16816(acc[2 * j], a0, a1, a2, a3, b0, b1);
        mma_bf16_16816(acc[2 * j + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    __syncthreads();
  }
  const int gid = lane >> 2, tig = lane & 3;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int t = t0 + warp * 16 + gid + 8 * h;
      if (t >= T) continue;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int e = e0 + 8 * j + 2 * tig + c;
        const float v = acc[j][2 * h + c];
        if (e < NE) logits[size_t(t) * NE + e] = v;
        else if (e == NE) gate[t] = v;
      }
    }
  }
}

static int weight_format(const Tensor& w, const Tensor& s, int64_t K, int* fmt) {
  if (s.present && s.dtype == Q35_F32) { *fmt = W_FP8ROW; return 0; }
  Q35_REQUIRE(s.present, Q35_ERR_MISSING, "quantised weight without scales");
  const int64_t inner = w.s[w.nd - 1];
  if (s.dtype == Q35_E4M3 && inner == K / 2) { *fmt = W_NVFP4; return 0; }  // E4M3 scales per 16 inputs
  if (inner == K / 2 && w.dtype == Q35_U8) { *fmt = W_MXFP4; return 0; }
  if (inner == K) { *fmt = W_MXFP8; return 0; }
  return fail(Q35_ERR_SHAPE, "weight inner dim %lld matches neither K/2 (MXFP4) nor K (FP8) for K=%lld",
              (long long)inner, (long long)K);
}

// mode 0: the whole dense part (moe.pre); 1: RMSNorm + router logits + shared-expert gate dot only (moe.norm_router);
// 2: the shared expert on given h2 / gate (moe.shared).  Modes 1 and 2 let a host overlap the shared expert with the
// routed experts on a second stream.
static int moe_pre_impl(Call& c, int mode) {
  const bool do_norm = mode != 2, do_shared = mode != 1;
  Tensor x1, ln2, wg, sg, wu, su, wd, sd, wr, wshg, out, h2o, lgo, gate_t, ws;
  Q35_TRY(c.get("x1", M(Q35_BF16), &x1));
  Q35_REQUIRE(x1.nd >= 2, Q35_ERR_SHAPE, "moe.pre: x1 [T, H]");
  const int64_t H = x1.s[x1.nd - 1], T = x1.numel() / H;
  int64_t NE = 0, FS = 0;
  int f1 = W_MXFP4;
  if (do_norm) {
    Q35_TRY(c.get("ln2", M(Q35_F32), &ln2));
    Q35_TRY(c.get("w_router", M(Q35_BF16), &wr));
    Q35_TRY(c.get("w_shg", M(Q35_BF16), &wshg));
    Q35_TRY(c.get("h2_out", M(Q35_BF16), &h2o));
    Q35_TRY(c.get("logits_out", M(Q35_F32), &lgo));
    Q35_REQUIRE(wr.nd == 2, Q35_ERR_SHAPE, "moe.pre: w_router [NE, H]");
    NE = wr.s[0];
    Q35_REQUIRE(ln2.numel() == H && wr.s[1] == H && wshg.numel() == H, Q35_ERR_SHAPE, "moe.pre: ln2 / w_router / w_shg");
    Q35_REQUIRE(h2o.numel() == T * H && lgo.numel() == T * NE, Q35_ERR_SHAPE, "moe.pre: h2_out / logits_out");
  } else {
    Q35_TRY(c.get("h2", M(Q35_BF16), &h2o));
    Q35_REQUIRE(h2o.numel() == T * H, Q35_ERR_SHAPE, "moe.shared: h2 [T, H]");
  }
  if (mode != 0) {  // the gate dot products travel between the two halves as a tensor
    Q35_TRY(c.get(mode == 1 ? "gate_out" : "gate", M(Q35_F32), &gate_t));
    Q35_REQUIRE(gate_t.numel() == T, Q35_ERR_SHAPE, "moe.pre: gate [T]");
  }
  if (do_shared) {
    Q35_TRY(c.get("w_gate", M_BYTES | M(Q35_E4M3), &wg));
    Q35_TRY(c.get("s_gate", M(Q35_U8), &sg));
    Q35_TRY(c.get("w_up", M_BYTES | M(Q35_E4M3), &wu));
    Q35_TRY(c.get("s_up", M(Q35_U8), &su));
    Q35_TRY(c.get("w_down", M_BYTES | M(Q35_E4M3), &wd));
    Q35_TRY(c.get("s_down", M(Q35_U8), &sd));
    Q35_TRY(c.get("out", M(Q35_BF16), &out));
    Q35_REQUIRE(wg.nd == 2 && wd.nd == 2, Q35_ERR_SHAPE, "moe.pre: shared expert ranks");
    FS = wg.s[0];
    Q35_REQUIRE(out.numel() == T * H && wu.s[0] == FS && wd.s[0] == H, Q35_ERR_SHAPE, "moe.pre: shared expert shapes");
    int f2, f3;
    Q35_TRY(weight_format(wg, sg, H, &f1));
    Q35_TRY(weight_format(wu, su, H, &f2));
    Q35_TRY(weight_format(wd, sd, FS, &f3));
    Q35_REQUIRE(f1 == f2 && f1 == f3 && f1 != W_FP8ROW && f1 != W_NVFP4, Q35_ERR_UNSUPPORTED,
                "moe.pre: shared expert must be MXFP4 or MXFP8");
    Q35_REQUIRE(sg.numel() == FS * (H / 32) && su.numel() == FS * (H / 32) && sd.numel() == H * (FS / 32),
                Q35_ERR_SHAPE, "moe.pre: scale shapes");
    Q35_REQUIRE(FS % 256 == 0, Q35_ERR_UNSUPPORTED, "moe.pre: FS must be a multiple of 256");
  }
  Q35_REQUIRE(H % 256 == 0, Q35_ERR_UNSUPPORTED, "moe.pre: H must be a multiple of 256");
  const bool use_tc = do_shared && f1 == W_MXFP4 && tc_shapes_ok(H, FS);
  WsCarver w{nullptr};
  __nv_bfloat16* act = w.take<__nv_bfloat16>(T * FS);
  float* gate = w.take<float>(T);
  uint8_t* qws = use_tc ? w.take<uint8_t>(tc_routed_bytes(T, H, FS)) : nullptr;
  Q35_TRY(c.workspace(w.off, &ws));
  if (c.dry || T == 0) return 0;
  Q35_REQUIRE(aligned16(x1.p) && aligned16(h2o.p) && (!do_shared || (aligned16(out.p) && aligned16(wg.p) &&
                  aligned16(wu.p) && aligned16(wd.p))) && (!do_norm || (aligned16(wr.p) && aligned16(wshg.p) && aligned16(ln2.p))),
              Q35_ERR_ALIGN, "moe.pre: pointers must be 16-byte aligned");
  WsCarver wc{ws.as<uint8_t>()};
  act = wc.take<__nv_bfloat16>(T * FS);
  gate = wc.take<float>(T);
  qws = use_tc ? wc.take<uint8_t>(tc_routed_bytes(T, H, FS)) : nullptr;
  if (mode != 0) gate = gate_t.as<float>();
  if (do_norm) {
    // eps is a constant of the model family (1e-6 for every Qwen3.5 config)
    const float eps = 1e-6f;
    launch_pdl(rmsnorm_kernel, dim3(unsigned(T)), dim3(256), 0, c.stream, x1.as<__nv_bfloat16>(), ln2.as<float>(),
               h2o.as<__nv_bfloat16>(), int(H), eps);
    Q35_CUDA_LAUNCH_CHECK("moe.pre rmsnorm");
    if (T >= 256 && H % 64 == 0) {  // prefill-sized: tensor cores
      launch_pdl(router_mma_kernel, dim3(unsigned((T + 63) / 64), unsigned((NE + 1 + 63) / 64)), dim3(128), 0, c.stream,
                 h2o.as<__nv_bfloat16>(), wr.as<__nv_bfloat16>(), wshg.as<__nv_bfloat16>(), lgo.as<float>(), gate, int(T),
                 int(H), int(NE));
    } else {
      launch_pdl(router_kernel, dim3(unsigned((NE + 1 + 7) / 8), unsigned(T)), dim3(256), 0, c.stream,
                 h2o.as<__nv_bfloat16>(), wr.as<__nv_bfloat16>(), wshg.as<__nv_bfloat16>(), lgo.as<float>(), gate, int(H),
                 int(NE));
    }
    Q35_CUDA_LAUNCH_CHECK("moe.pre router");
  }
  if (!do_shared) return 0;
  if (use_tc) {  // shared expert on the tensor cores: one dense group of T rows
    const TcQuant q1 = tc_quant_carve(qws, T, H);
    const TcQuant q2 = tc_quant_carve(qws + tc_quant_bytes(T, H), T, FS);
    Q35_TRY(tc_quantize(h2o.as<__nv_bfloat16>(), int(H), nullptr, int(T), int(T), int(H), q1, c.stream));
    TcArgs ta{};
    ta.n_dense = int(T); ta.n_planes = 1; ta.K = int(H);
    ta.plane_rows[0] = ta.plane_rows[1] = int(FS);
    ta.roff[0] = ta.roff[1] = 0; ta.lim[0] = ta.lim[1] = int(FS); ta.tile_rows = 64;
    ta.sw[0] = sg.as<uint8_t>(); ta.sw[1] = su.as<uint8_t>(); ta.s_plane = 0;
    ta.act_rows = int(FS); ta.act_out = act;
    const TcWeights wgu{{wg.as<uint8_t>(), wu.as<uint8_t>()}, {uint64_t(FS), uint64_t(FS)}};
    Q35_TRY(tc_launch<TC_EPI_SILU_MUL>(wgu, q1, ta, int(T), int(FS / 64), 1, c.stream));
    Q35_TRY(tc_quantize(act, int(FS), nullptr, int(T), int(T), int(FS), q2, c.stream));
    TcArgs td{};
    td.n_dense = int(T); td.n_planes = 1; td.K = int(FS);
    td.plane_rows[0] = td.plane_rows[1] = int(H);
    td.roff[0] = 0; td.roff[1] = 64; td.lim[0] = td.lim[1] = int(H); td.tile_rows = 128;
    td.sw[0] = td.sw[1] = sd.as<uint8_t>(); td.s_plane = 0;
    td.b_out = out.as<__nv_bfloat16>(); td.out_stride = int(H); td.resid = x1.as<__nv_bfloat16>(); td.gate = gate;
    const TcWeights wdn{{wd.as<uint8_t>(), wd.as<uint8_t>()}, {uint64_t(H), uint64_t(H)}};
    return tc_launch<TC_EPI_SHARED_DOWN>(wdn, q2, td, int(T), int(H / 128), 1, c.stream);
  }
  const int nt = pick_nt(T);
  SkinnyArgs a{};
  a.status = device_status_ptr();
  a.n_dense = int(T); a.n_planes = 1;
  a.w[0] = wg.as<uint8_t>(); a.w[1] = wu.as<uint8_t>(); a.s[0] = sg.as<uint8_t>(); a.s[1] = su.as<uint8_t>();
  a.K = int(H); a.roff[0] = a.roff[1] = 0; a.lim[0] = a.lim[1] = int(FS);
  a.act_rows = int(FS); a.tile_rows = 64; a.warp_rows = 16;
  a.x = h2o.as<__nv_bfloat16>(); a.x_stride = int(H); a.act_out = act;
  SkinnyArgs d{};
  d.status = a.status;
  d.n_dense = int(T); d.n_planes = 1;
  d.w[0] = d.w[1] = wd.as<uint8_t>(); d.s[0] = d.s[1] = sd.as<uint8_t>();
  d.K = int(FS); d.roff[0] = 0; d.roff[1] = 16; d.lim[0] = d.lim[1] = int(H);
  d.tile_rows = 128; d.warp_rows = 32;
  d.x = act; d.x_stride = int(FS);
  d.b_out = out.as<__nv_bfloat16>(); d.out_stride = int(H); d.resid = x1.as<__nv_bfloat16>(); d.gate = gate;
  if (f1 == W_MXFP4) {
    Q35_TRY((launch_skinny<W_MXFP4, EPI_SILU_MUL>(a, nt, int(FS / 64), 1, c.stream)));
    return launch_skinny<W_MXFP4, EPI_SHARED_DOWN>(d, nt, int((H + 127) / 128), 1, c.stream);
  }
  Q35_TRY((launch_skinny<W_MXFP8, EPI_SILU_MUL>(a, nt, int(FS / 64), 1, c.stream)));
  return launch_skinny<W_MXFP8, EPI_SHARED_DOWN>(d, nt, int((H + 127) / 128), 1, c.stream);
}

int run_moe_pre(Call& c) { return moe_pre_impl(c, 0); }
int run_moe_norm_router(Call& c) { return moe_pre_impl(c, 1); }
int run_moe_shared(Call& c) { return moe_pre_impl(c, 2); }

// moe.finish: out = bf16(base + partial): closes the block when the routed experts were summed separately
// (the fp32 accumulation `acc = base; acc += rw_i * d_i` of moe_experts, models/qwen35_2b/whole/src/q35_moe.py:73-85,
// with the routed terms added first)
__global__ void moe_finish_kernel(const __nv_bfloat16* __restrict__ base, const float* __restrict__ partial,
                                  __nv_bfloat16* __restrict__ out, long long n) {
  pdl_wait();
  pdl_launch();
  const long long i = (long long)(blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i >= n) return;
  const uint2 b = *reinterpret_cast<const uint2*>(base + i);
  const float4 p = *reinterpret_cast<const float4*>(partial + i);
  uint2 o;
  o.x = pack_bf16(bf16lo(b.x) + p.x, bf16hi(b.x) + p.y);
  o.y = pack_bf16(bf16lo(b.y) + p.z, bf16hi(b.y) + p.w);
  *reinterpret_cast<uint2*>(out + i) = o;
}

int run_moe_finish(Call& c) {
  Tensor base, partial, out;
  Q35_TRY(c.get("base", M(Q35_BF16), &base));
  Q35_TRY(c.get("partial", M(Q35_F32), &partial));
  Q35_TRY(c.get("out", M(Q35_BF16), &out));
  const int64_t n = base.numel();
  Q35_REQUIRE(partial.numel() == n && out.numel() == n && n % 4 == 0, Q35_ERR_SHAPE, "moe.finish: base, partial, out [T, H]");
  c.ws_need = 0;
  if (c.dry || n == 0) return 0;
  Q35_REQUIRE(aligned16(base.p) && aligned16(partial.p) && aligned16(out.p), Q35_ERR_ALIGN, "moe.finish: alignment");
  launch_pdl(moe_finish_kernel, dim3(unsigned((n / 4 + 255) / 256)), dim3(256), 0, c.stream, base.as<__nv_bfloat16>(),
             partial.as<float>(), out.as<__nv_bfloat16>(), n);
  Q35_CUDA_LAUNCH_CHECK("moe.finish");
  return 0;
}

// ---------------------------------------------------------------------------------------------------------------
// linear: out[t, n] = x[t, :] . dequant(w[n, :]) (+ bias): the quantised projections of the layer kernels.
// MXFP4 / MXFP8: linear(x, w, s) of the reference's q35 line (models/qwen35_2b/whole/src/q35_mx_build.py:100-115);
// FP8 with per-row fp32 scales: fp8_gemm with scale_a = 1
// (models/qwen35_35b_a3b/sgl/python/sgl_kernel_axera/gemm.py:123-153, 457-466).
int run_linear(Call& c) {
  Tensor x, w, s, bias, out, rdiv, resid;
  Q35_TRY(c.get("row_div", M(Q35_F32), &rdiv, false));
  Q35_TRY(c.get("residual", M(Q35_BF16), &resid, false));
  Q35_TRY(c.get("x", M(Q35_BF16), &x));
  Q35_TRY(c.get("w", M_BYTES | M(Q35_E4M3), &w));
  Q35_TRY(c.get("s", M(Q35_U8) | M(Q35_F32) | M(Q35_E4M3), &s));
  Tensor s2;
  Q35_TRY(c.get("s2", M(Q35_F32), &s2, false));
  Q35_TRY(c.get("bias", M(Q35_F32), &bias, false));
  Q35_TRY(c.get("out", M(Q35_BF16) | M(Q35_F32), &out));
  Q35_REQUIRE(x.nd >= 2 && w.nd == 2, Q35_ERR_SHAPE, "linear: x [T, K], w [N, K or K/2]");
  const int64_t K = x.s[x.nd - 1], T = x.numel() / K, N = w.s[0];
  int fmt;
  Q35_TRY(weight_format(w, s, K, &fmt));
  Q35_REQUIRE(out.numel() == T * N, Q35_ERR_SHAPE, "linear: out must be [T, N]");
  Q35_REQUIRE(fmt == W_FP8ROW ? s.numel() == N : fmt == W_NVFP4 ? s.numel() == N * (K / 16) : s.numel() == N * (K / 32),
              Q35_ERR_SHAPE, "linear: scale shape");
  Q35_REQUIRE(!s2.present || (fmt == W_NVFP4 && s2.numel() == 1), Q35_ERR_SHAPE,
              "linear: s2 [1] is the tensor scale of an NVFP4 weight (E4M3 scales [N, K/16])");
  Q35_REQUIRE(!bias.present || bias.numel() == N, Q35_ERR_SHAPE, "linear: bias [N]");
  Q35_REQUIRE((!rdiv.present || rdiv.numel() == T) && (!resid.present || resid.numel() == T * N), Q35_ERR_SHAPE,
              "linear: row_div [T], residual [T, N]");
  Q35_REQUIRE(K % 128 == 0, Q35_ERR_UNSUPPORTED, "linear: K must be a multiple of 128");
  // With a workspace bound, the projection runs on the tensor cores (tcgen05 block-scaled MMA:
  // E2M1 or E4M3 weights straight from TMA, activations as two E4M3 terms); without a workspace on the CUDA-core
  // weight-streaming kernel, which takes K in multiples of 256 only.  Same results within the tolerance of the role.
  const bool tc_shape = fmt != W_NVFP4;  // the block-scaled MMA kind used here takes E8M0 scales per 32 only
  const int64_t need = tc_shape ? tc_linear_bytes(T, N, K) : 0;
  Tensor ws;
  c.ws_need = need;
  if (!c.dry) Q35_TRY(c.get("workspace", M(Q35_U8), &ws, false));
  if (c.dry || T == 0 || N == 0) return 0;
  Q35_REQUIRE(aligned16(x.p) && aligned16(w.p), Q35_ERR_ALIGN, "linear: pointers must be 16-byte aligned");
  if (tc_shape && ws.present && int64_t(ws.bytes) >= need && (reinterpret_cast<uintptr_t>(ws.p) & 255) == 0 &&
      (reinterpret_cast<uintptr_t>(w.p) & 31) == 0 && aligned16(s.p)) {
    TcLinear p{};
    p.w = w.p; p.s = s.p; p.fmt = fmt == W_MXFP4 ? 0 : fmt == W_MXFP8 ? 1 : 2;
    p.bias = bias.present ? bias.as<float>() : nullptr;
    p.row_div = rdiv.present ? rdiv.as<float>() : nullptr;
    p.resid2 = resid.present ? resid.as<__nv_bfloat16>() : nullptr;
    p.f_out = out.dtype == Q35_F32 ? out.as<float>() : nullptr;
    p.b_out = out.dtype == Q35_F32 ? nullptr : out.as<__nv_bfloat16>();
    return tc_linear(x.as<__nv_bfloat16>(), T, N, K, p, ws.as<uint8_t>(), c.stream);
  }
  Q35_REQUIRE(K % 256 == 0, Q35_ERR_UNSUPPORTED,
              "linear: K that is not a multiple of 256 needs the tensor-core path (an aligned workspace of "
              "q35_workspace_bytes)");
  SkinnyArgs d{};
  d.status = device_status_ptr();
  d.n_dense = int(T); d.n_planes = 1;
  d.w[0] = d.w[1] = w.as<uint8_t>(); d.s[0] = d.s[1] = s.as<uint8_t>();
  d.K = int(K); d.roff[0] = 0; d.roff[1] = 16; d.lim[0] = d.lim[1] = int(N);
  d.tile_rows = 128; d.warp_rows = 32;
  d.x = x.as<__nv_bfloat16>(); d.x_stride = int(K);
  if (out.dtype == Q35_F32) d.f_out = out.as<float>(); else d.b_out = out.as<__nv_bfloat16>();
  d.out_stride = int(N);
  d.bias = bias.present ? bias.as<float>() : nullptr;
  d.row_div = rdiv.present ? rdiv.as<float>() : nullptr;
  d.resid2 = resid.present ? resid.as<__nv_bfloat16>() : nullptr;
  const int nt = pick_nt(T), tiles = int((N + 127) / 128);
  if (fmt == W_MXFP4) return launch_skinny<W_MXFP4, EPI_PLAIN>(d, nt, tiles, 1, c.stream);
  if (fmt == W_MXFP8) return launch_skinny<W_MXFP8, EPI_PLAIN>(d, nt, tiles, 1, c.stream);
  if (fmt == W_NVFP4) {
    d.tensor_scale = s2.present ? s2.as<float>() : nullptr;
    return launch_skinny<W_NVFP4, EPI_PLAIN>(d, nt, tiles, 1, c.stream);
  }
  return launch_skinny<W_FP8ROW, EPI_PLAIN>(d, nt, tiles, 1, c.stream);
}

// linear.multi: several projections of one input in one pass -- w is the row-wise concatenation of their weights
// (the reference's fused w_qkv rows, models/qwen35_35b_a3b/qwen35_35b_a3b.manifest.json `prefill64.gdn`), out0 ..
// out7 the projections' own tensors [T, N_i] in that order.  One activation quantisation, one pass over the weights,
// one reduction that applies bias / per-row scale / per-token divisor and scatters the segments.
int run_linear_multi(Call& c) {
  Tensor x, w, s, bias, rdiv, ws;
  Q35_TRY(c.get("x", M(Q35_BF16), &x));
  Q35_TRY(c.get("row_div", M(Q35_F32), &rdiv, false));
  Q35_TRY(c.get("w", M_BYTES | M(Q35_E4M3), &w));
  Q35_TRY(c.get("s", M(Q35_U8) | M(Q35_F32), &s));
  Q35_TRY(c.get("bias", M(Q35_F32), &bias, false));
  Q35_REQUIRE(x.nd >= 2 && w.nd == 2, Q35_ERR_SHAPE, "linear.multi: x [T, K], w [N, K or K/2]");
  const int64_t K = x.s[x.nd - 1], T = x.numel() / K, N = w.s[0];
  int fmt;
  Q35_TRY(weight_format(w, s, K, &fmt));
  Q35_REQUIRE(fmt != W_NVFP4, Q35_ERR_UNSUPPORTED, "linear.multi: NVFP4 weights take the one-projection role");
  Q35_REQUIRE(fmt == W_FP8ROW ? s.numel() == N : s.numel() == N * (K / 32), Q35_ERR_SHAPE, "linear.multi: scale shape");
  Q35_REQUIRE((!bias.present || bias.numel() == N) && (!rdiv.present || rdiv.numel() == T), Q35_ERR_SHAPE,
              "linear.multi: bias [N], row_div [T]");
  Q35_REQUIRE(K % 128 == 0, Q35_ERR_UNSUPPORTED, "linear.multi: K must be a multiple of 128");
  TcSegments segs{};
  int64_t rows = 0;
  static const char* const names[8] = {"out0", "out1", "out2", "out3", "out4", "out5", "out6", "out7"};
  for (int i = 0; i < 8; ++i) {
    Tensor o;
    Q35_TRY(c.get(names[i], M(Q35_BF16) | M(Q35_F32), &o, i == 0));
    if (!o.present) break;
    Q35_REQUIRE(T > 0 && o.numel() % T == 0 && o.numel() > 0, Q35_ERR_SHAPE, "linear.multi: %s must be [T, N_i]", names[i]);
    segs.n0[i] = int(rows);
    segs.out[i] = o.p;
    segs.f32[i] = o.dtype == Q35_F32;
    rows += o.numel() / T;
    segs.n = i + 1;
  }
  segs.n0[segs.n] = int(rows);
  Q35_REQUIRE(rows == N, Q35_ERR_SHAPE, "linear.multi: the outputs hold %lld rows, the weight %lld", (long long)rows,
              (long long)N);
  Q35_TRY(c.workspace(tc_linear_multi_bytes(T, N, K), &ws));
  if (c.dry || T == 0) return 0;
  Q35_REQUIRE(aligned16(x.p) && (reinterpret_cast<uintptr_t>(w.p) & 31) == 0 && aligned16(s.p), Q35_ERR_ALIGN,
              "linear.multi: x, s 16-byte and w 32-byte aligned");
  TcLinear p{};
  p.w = w.p; p.s = s.p; p.fmt = fmt == W_MXFP4 ? 0 : fmt == W_MXFP8 ? 1 : 2;
  p.bias = bias.present ? bias.as<float>() : nullptr;
  p.row_div = rdiv.present ? rdiv.as<float>() : nullptr;
  return tc_linear_multi(x.as<__nv_bfloat16>(), T, N, K, p, segs, ws.as<uint8_t>(), c.stream);
}

}  // namespace q35
