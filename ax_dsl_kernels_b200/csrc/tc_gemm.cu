// Host side of the block-scaled tensor-core GEMM: tensor maps, activation quantisation, launch.
#include <mutex>
#include <unordered_map>
#include "abi.h"
#include "common.cuh"
#include "tc_gemm.cuh"
#include "tc_host.h"

namespace q35 {

// ---------------------------------------------------------------------------------------------------------------
// cuTensorMapEncodeTiled is taken from the driver at run time, so the library links against the runtime only.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// Encoded tensor maps are kept per (device, address, shape, box): weights, and the workspace the quantised activations
// live in, do not move between the steps of a decode loop, so every launch after the first finds its maps here
// instead of asking the driver again (about a microsecond each, four per GEMM).
struct MapKey {
  int dev; bool fp4; const void* base; uint64_t rows, cols, pitch; uint32_t box_rows;
  bool operator==(const MapKey& o) const {
    return dev == o.dev && fp4 == o.fp4 && base == o.base && rows == o.rows && cols == o.cols && pitch == o.pitch &&
           box_rows == o.box_rows;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    uint64_t h = reinterpret_cast<uintptr_t>(k.base) * 0x9E3779B97F4A7C15ull;
    h ^= (k.rows + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2));
    h ^= (k.cols * 31 + k.pitch * 17 + k.box_rows * 7 + uint64_t(k.dev) * 3 + (k.fp4 ? 1 : 0)) + (h << 6) + (h >> 2);
    return size_t(h);
  }
};
static std::mutex g_map_mutex;
static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_map_cache;
constexpr size_t MAP_CACHE_MAX = 4096;  // entries (128 B each); emptied when full

static int encode_map(CUtensorMap* m, bool fp4, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch_bytes,
                      uint32_t box_rows, const char* what);

// 2D row-major tensor [rows, cols] with a [box_rows, 128-element] box and 128-byte swizzle
static int make_map(CUtensorMap* m, bool fp4, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch_bytes,
                    uint32_t box_rows, const char* what) {
  MapKey key{0, fp4, base, rows, cols, pitch_bytes, box_rows};
  if (cudaGetDevice(&key.dev) != cudaSuccess) key.dev = -1;
  {
    std::lock_guard<std::mutex> lock(g_map_mutex);
    auto it = g_map_cache.find(key);
    if (it != g_map_cache.end()) { *m = it->second; return 0; }
  }
  Q35_TRY(encode_map(m, fp4, base, rows, cols, pitch_bytes, box_rows, what));
  std::lock_guard<std::mutex> lock(g_map_mutex);
  if (g_map_cache.size() >= MAP_CACHE_MAX) g_map_cache.clear();
  g_map_cache.emplace(key, *m);
  return 0;
}

static int encode_map(CUtensorMap* m, bool fp4, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch_bytes,
                      uint32_t box_rows, const char* what) {
  EncodeTiledFn fn = encode_fn();
  Q35_REQUIRE(fn != nullptr, Q35_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {pitch_bytes};
  const cuuint32_t box[2] = {128, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(m, fp4 ? CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2,
                        const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  Q35_REQUIRE(r == CUDA_SUCCESS, Q35_ERR_CUDA, "tensor map for %s rejected by the driver (CUresult %d)", what, int(r));
  return 0;
}

// ---------------------------------------------------------------------------------------------------------------
// x (bf16) -> two E4M3 terms with UE8M0 block-32 scales: x = hi * 2^eh + lo * 2^el;
// rows gathered through `src` (destination row -> source row; nullptr = identity).
// Eight elements per piece (one 16-byte load), four threads per 32-block.  A thread takes PP pieces, 256 apart, and
// has the row ids and then the 16-byte loads of all of them in flight before it converts the first: with one piece per
// thread a prefill-sized call (millions of pieces, two dependent loads each) ran at the loads' latency, not at the
// bandwidth of its stores.
template <int PP>
__global__ void __launch_bounds__(256) tc_quant_kernel(const __nv_bfloat16* __restrict__ x, int x_stride,
                                                       const int* __restrict__ src, int x_rows, int R, int K,
                                                       uint8_t* __restrict__ qh, uint8_t* __restrict__ ql,
                                                       uint8_t* __restrict__ sh, uint8_t* __restrict__ sl) {
  pdl_wait();
  pdl_launch();
  const int per_row = K / 8;
  const long long n_pieces = (long long)R * per_row;
  const long long i0 = (long long)blockIdx.x * (256 * PP) + threadIdx.x;  // index of the first 8-element piece
  bool on[PP];
  int row[PP], c8[PP];
  long long srow[PP];
#pragma unroll
  for (int j = 0; j < PP; ++j) {
    const long long i = i0 + j * 256;
    on[j] = i < n_pieces;  // whole quads are on or off together (K is a multiple of 32)
    row[j] = on[j] ? int(i / per_row) : 0;
    c8[j] = on[j] ? int(i % per_row) : 0;
    srow[j] = row[j];
    if (src) srow[j] = src[row[j]];
  }
  uint4 raw[PP];
#pragma unroll
  for (int j = 0; j < PP; ++j) {
    // rows past the filled part of a grouped list hold stale ids: read row 0 instead, nobody uses the result
    if (srow[j] < 0 || srow[j] >= x_rows) srow[j] = 0;
    raw[j] = make_uint4(0u, 0u, 0u, 0u);
    if (on[j]) raw[j] = *reinterpret_cast<const uint4*>(x + srow[j] * x_stride + c8[j] * 8);
  }
#pragma unroll
  for (int j = 0; j < PP; ++j) {
    const uint32_t w[4] = {raw[j].x, raw[j].y, raw[j].z, raw[j].w};
    float v[8];
#pragma unroll
    for (int u = 0; u < 4; ++u) { v[2 * u] = bf16lo(w[u]); v[2 * u + 1] = bf16hi(w[u]); }
    const TwoTerm8 t = quant_two_terms8(v);
    if (!on[j]) continue;
    const long long o = (long long)row[j] * K + c8[j] * 8;
    *reinterpret_cast<uint2*>(qh + o) = t.hi;
    *reinterpret_cast<uint2*>(ql + o) = t.lo;
    if ((c8[j] & 3) == 0) {
      sh[(long long)row[j] * (K / 32) + c8[j] / 4] = uint8_t(t.eh + 127);
      sl[(long long)row[j] * (K / 32) + c8[j] / 4] = uint8_t(t.el + 127);
    }
  }
}

int tc_quantize(const __nv_bfloat16* x, int x_stride, const int* src, int x_rows, int R, int K, const TcQuant& q,
                cudaStream_t stream) {
  const long long pieces = (long long)R * (K / 8);
  if (pieces == 0) return 0;
  Q35_REQUIRE(K % 32 == 0 && x_stride % 8 == 0 && (uintptr_t(x) & 15) == 0, Q35_ERR_ALIGN,
              "tc quantize: rows must start on 16-byte boundaries");
  // several pieces per thread once there are enough pieces to fill every SM several times over
  if (pieces >= 4ll * 256 * 8 * sm_count())
    launch_pdl(tc_quant_kernel<4>, dim3(unsigned((pieces + 1023) / 1024)), dim3(256), 0, stream, x, x_stride, src, x_rows,
               R, K, q.qh, q.ql, q.sh, q.sl);
  else
    launch_pdl(tc_quant_kernel<1>, dim3(unsigned((pieces + 255) / 256)), dim3(256), 0, stream, x, x_stride, src, x_rows, R,
               K, q.qh, q.ql, q.sh, q.sl);
  Q35_CUDA_LAUNCH_CHECK("tc quantize");
  return 0;
}

int64_t tc_quant_bytes(int64_t R, int64_t K) { return 2 * (R * K + 256) + 2 * (R * (K / 32) + 256) + 1024; }

TcQuant tc_quant_carve(uint8_t* base, int64_t R, int64_t K) {
  auto up = [](int64_t v) { return (v + 255) / 256 * 256; };
  TcQuant q;
  q.qh = base;
  q.ql = q.qh + up(R * K);
  q.sh = q.ql + up(R * K);
  q.sl = q.sh + up(R * (K / 32));
  q.R = int(R);
  q.K = int(K);
  return q;
}

// ---------------------------------------------------------------------------------------------------------------
// compacted list of the groups that have rows, in group order (one CTA; groups <= a few thousand)
__global__ void __launch_bounds__(1024) tc_active_kernel(const int* __restrict__ g_n, int G, int* __restrict__ active,
                                                         int* __restrict__ n_active) {
  __shared__ int s_warp[32];
  __shared__ int s_base;
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  if (tid == 0) s_base = 0;
  __syncthreads();
  for (int g0 = 0; g0 < G; g0 += 1024) {
    const int g = g0 + tid;
    const bool on = g < G && g_n[g] > 0;
    const unsigned m = __ballot_sync(0xffffffffu, on);
    if (lane == 0) s_warp[wid] = __popc(m);
    __syncthreads();
    int before = s_base;
    for (int w = 0; w < wid; ++w) before += s_warp[w];
    if (on) active[before + __popc(m & ((1u << lane) - 1))] = g;
    __syncthreads();
    if (tid == 0) {
      int tot = 0;
      for (int w = 0; w < 32; ++w) tot += s_warp[w];
      s_base += tot;
    }
    __syncthreads();
  }
  if (tid == 0) n_active[0] = s_base;
}

int tc_build_active(const int* g_n, int groups, int* active, cudaStream_t stream) {
  tc_active_kernel<<<1, 1024, 0, stream>>>(g_n, groups, active + 1, active);
  Q35_CUDA_LAUNCH_CHECK("tc active groups");
  return 0;
}

int tc_make_map(CUtensorMap* m, bool fp4, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch_bytes,
                uint32_t box_rows, const char* what) {
  return make_map(m, fp4, base, rows, cols, pitch_bytes, box_rows, what);
}

template <int NB, int EPI>
static int launch_nb(const CUtensorMap& w0, const CUtensorMap& w1, const CUtensorMap& xh, const CUtensorMap& xl,
                     const TcArgs& a, int tiles, int groups, cudaStream_t stream) {
  const int smem = TcCfg<NB>::smem_bytes(a.K);
  Q35_TRY(ensure_dynamic_smem(reinterpret_cast<const void*>(tc_gemm_kernel<NB, EPI>), smem));
  const long long items = (long long)tiles * (a.g_n ? groups : (a.n_dense + a.dense_rows - 1) / a.dense_rows * a.k_slices);
  const long long slots = (long long)sm_count() * TcCfg<NB>::CTAS_PER_SM;
  const unsigned grid = unsigned(items < slots ? items : slots);
  launch_pdl(tc_gemm_kernel<NB, EPI>, dim3(grid), dim3(tc_threads<NB, EPI>()), size_t(smem), stream, w0, w1, xh, xl, a);
  Q35_CUDA_LAUNCH_CHECK("tc gemm");
  return 0;
}

template <int EPI>
int tc_launch(const TcWeights& w, const TcQuant& q, TcArgs a, int nb, int tiles, int groups, cudaStream_t stream) {
  Q35_REQUIRE(a.K % 128 == 0 && a.K == q.K, Q35_ERR_UNSUPPORTED, "tc gemm: K must be a multiple of 128");
  Q35_REQUIRE((uintptr_t(a.sw[0]) & 15) == 0 && (uintptr_t(a.sw[1]) & 15) == 0 &&
                  (a.s_plane & (a.K % 512 == 0 ? 15 : 3)) == 0,
              Q35_ERR_ALIGN, "tc gemm: scale tensors must be 16-byte aligned");
  Q35_REQUIRE((a.sw[0] == nullptr) == (a.sw[1] == nullptr), Q35_ERR_MISSING, "tc gemm: scales of one half only");
  CUtensorMap w0, w1, xh, xl;
  const bool fp4 = a.w_fp8 == 0;
  a.a_fmt = fp4 ? int(tc::FMT_E2M1) : int(tc::FMT_E4M3);
  Q35_TRY(make_map(&w0, fp4, w.w[0], w.rows_total[0], a.K, fp4 ? a.K / 2 : a.K, 64, "weights"));
  Q35_TRY(make_map(&w1, fp4, w.w[1], w.rows_total[1], a.K, fp4 ? a.K / 2 : a.K, 64, "weights"));
  if (!a.g_n) {
    // dense: the rows are cut into virtual groups.  Every group streams the whole weight matrix, so groups are only
    // made smaller than 256 rows while the row tiles alone leave CTAs idle (decode-sized inputs on small matrices,
    // whose repeated reads then come out of L2).
    const int want = (2 * sm_count() + tiles - 1) / tiles;
    int rows = ((a.n_dense + want - 1) / want + 15) / 16 * 16;
    a.dense_rows = rows < 16 ? 16 : rows > 256 ? 256 : rows;
    nb = nb < a.dense_rows ? nb : a.dense_rows;
  }
  nb = nb <= 16 ? 16 : nb <= 32 ? 32 : 64;
  if (a.k_slices < 1 || a.g_n || a.part == nullptr) a.k_slices = 1;
  {
    const int ks_total = (a.K / 128 + 3) / 4 * 4;
    a.slice_stages = ((ks_total / 4 + a.k_slices - 1) / a.k_slices) * 4;
    a.k_slices = (ks_total + a.slice_stages - 1) / a.slice_stages;  // no empty slice
  }
  Q35_TRY(make_map(&xh, false, q.qh, q.R, a.K, a.K, nb, "activations"));
  Q35_TRY(make_map(&xl, false, q.ql, q.R, a.K, a.K, nb, "activations"));
  a.sfh = q.sh; a.sfl = q.sl; a.total_rows = q.R;
  a.n_tiles = tiles;
  Q35_REQUIRE(a.g_n == nullptr || (a.active != nullptr && a.n_active != nullptr), Q35_ERR_WORKSPACE,
              "tc gemm: grouped launch without an active-group list");
  a.status = device_status_ptr();
  a.stage_tx = (fp4 ? 128 * 64 : 128 * 128) + 2 * nb * 128;
  if (nb == 16) return launch_nb<16, EPI>(w0, w1, xh, xl, a, tiles, groups, stream);
  if (nb == 32) return launch_nb<32, EPI>(w0, w1, xh, xl, a, tiles, groups, stream);
  return launch_nb<64, EPI>(w0, w1, xh, xl, a, tiles, groups, stream);
}

template int tc_launch<TC_EPI_SILU_MUL>(const TcWeights&, const TcQuant&, TcArgs, int, int, int, cudaStream_t);
template int tc_launch<TC_EPI_ROW_SCALE>(const TcWeights&, const TcQuant&, TcArgs, int, int, int, cudaStream_t);
template int tc_launch<TC_EPI_SHARED_DOWN>(const TcWeights&, const TcQuant&, TcArgs, int, int, int, cudaStream_t);
template int tc_launch<TC_EPI_PLAIN>(const TcWeights&, const TcQuant&, TcArgs, int, int, int, cudaStream_t);

// ---------------------------------------------------------------------------------------------------------------
// linear.tc: out[t, n] = x[t, :] . dequant_mxfp4(w[n, :]) on the tensor cores (same contract as `linear` with MXFP4
// weights; reference: linear(x, w, s) of the MX projections, models/qwen35_2b/whole/src/q35_mx_build.py:100-115)
// shared by linear.tc and lm_head: quantise x into the workspace and run the plain-epilogue GEMM
// split-K slices of a dense launch: only for decode-sized inputs (one group of token rows) whose row tiles leave more
// than half of the CTAs without work; as many slices as bring the items up to the CTA count, in whole scale granules
int tc_linear_slices(int64_t T, int64_t N, int64_t K) {
  if (T > 16) return 1;
  const int64_t tiles = (N + 127) / 128, slots = 2 * int64_t(sm_count()), granules = (K / 128 + 3) / 4;
  if (tiles * 2 > slots) return 1;
  int64_t s = slots / tiles;
  s = s > granules ? granules : s;
  s = s > 16 ? 16 : s < 1 ? 1 : s;
  const int64_t per = (granules + s - 1) / s;  // granules a slice; no slice is left empty
  return int((granules + per - 1) / per);
}

int64_t tc_linear_bytes(int64_t T, int64_t N, int64_t K) {
  const int s = tc_linear_slices(T, N, K);
  return (tc_quant_bytes(T, K) + 255) / 256 * 256 + (s > 1 ? int64_t(s) * T * N * 4 : 0);
}

// sums the slices' fp32 planes and applies the epilogue of the `linear` role
__global__ void __launch_bounds__(256) tc_linear_reduce_kernel(const float* __restrict__ part, long long plane, int slices,
                                                               int T, int N, const float* __restrict__ row_scale,
                                                               const float* __restrict__ bias,
                                                               const float* __restrict__ row_div,
                                                               const __nv_bfloat16* __restrict__ resid2, float* f_out,
                                                               __nv_bfloat16* b_out) {
  pdl_wait();
  pdl_launch();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)T * N) return;
  const int t = int(i / N), n = int(i % N);
  float v = 0.f;
  for (int s = 0; s < slices; ++s) v += part[s * plane + i];
  v = v * (row_scale ? row_scale[n] : 1.f) + (bias ? bias[n] : 0.f);
  if (row_div) v = round_bf16(v) / row_div[t];
  if (resid2) v = round_bf16(v) + __bfloat162float(resid2[i]);
  if (f_out) f_out[i] = v;
  else b_out[i] = __float2bfloat16_rn(v);
}

// the reduction with the rows cut into segments, each with an output tensor of its own
__global__ void __launch_bounds__(256) tc_linear_reduce_multi_kernel(const float* __restrict__ part, long long plane,
                                                                     int slices, int T, int N,
                                                                     const float* __restrict__ row_scale,
                                                                     const float* __restrict__ bias,
                                                                     const float* __restrict__ row_div, TcSegments segs) {
  pdl_wait();
  pdl_launch();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)T * N) return;
  const int t = int(i / N), n = int(i % N);
  float v = 0.f;
  for (int s = 0; s < slices; ++s) v += part[s * plane + i];
  v = v * (row_scale ? row_scale[n] : 1.f) + (bias ? bias[n] : 0.f);
  if (row_div) v = round_bf16(v) / row_div[t];
  int g = 0;
  while (g + 1 < segs.n && n >= segs.n0[g + 1]) ++g;
  const long long o = (long long)t * (segs.n0[g + 1] - segs.n0[g]) + (n - segs.n0[g]);
  if (segs.f32[g]) static_cast<float*>(segs.out[g])[o] = v;
  else static_cast<__nv_bfloat16*>(segs.out[g])[o] = __float2bfloat16_rn(v);
}

int64_t tc_linear_multi_bytes(int64_t T, int64_t N, int64_t K) {
  const int s = tc_linear_slices(T, N, K);
  return (tc_quant_bytes(T, K) + 255) / 256 * 256 + int64_t(s) * T * N * 4;
}

static int tc_linear_impl(const __nv_bfloat16* x, int64_t T, int64_t N, int64_t K, const TcLinear& p,
                          const TcSegments* segs, uint8_t* qws, cudaStream_t stream) {
  const TcQuant q = tc_quant_carve(qws, T, K);
  const int slices = tc_linear_slices(T, N, K);
  float* part = (slices > 1 || segs) ? reinterpret_cast<float*>(qws + (tc_quant_bytes(T, K) + 255) / 256 * 256) : nullptr;
  Q35_TRY(tc_quantize(x, int(K), nullptr, int(T), int(T), int(K), q, stream));
  const uint8_t* w = static_cast<const uint8_t*>(p.w);
  TcWeights tw{{w, w}, {uint64_t(N), uint64_t(N)}};
  TcArgs a{};
  a.n_dense = int(T); a.n_planes = 1; a.K = int(K);
  a.plane_rows[0] = a.plane_rows[1] = int(N);
  a.roff[0] = 0; a.roff[1] = 64; a.lim[0] = a.lim[1] = int(N); a.tile_rows = 128;
  a.w_fp8 = p.fmt == 0 ? 0 : 1;
  // block scales: E8M0 [N, K/32] for the MX formats; FP8 per-row has none (block scale 1) and a fp32 scale per row
  a.sw[0] = a.sw[1] = p.fmt == 2 ? nullptr : static_cast<const uint8_t*>(p.s);
  a.row_scale = p.fmt == 2 ? static_cast<const float*>(p.s) : nullptr;
  a.s_plane = 0;
  a.f_out = p.f_out; a.b_out = p.b_out;
  a.out_stride = int(N);
  a.bias = p.bias; a.row_div = p.row_div; a.resid2 = p.resid2;
  a.k_slices = slices; a.part = part; a.part_plane = (long long)T * N;
  a.raw = segs ? 1 : 0;
  Q35_TRY(tc_launch<TC_EPI_PLAIN>(tw, q, a, int(T), int((N + 127) / 128), 1, stream));
  if (segs) {
    launch_pdl(tc_linear_reduce_multi_kernel, dim3(unsigned((T * N + 255) / 256)), dim3(256), 0, stream,
               (const float*)part, (long long)T * N, slices, int(T), int(N), a.row_scale, p.bias, p.row_div, *segs);
    Q35_CUDA_LAUNCH_CHECK("tc linear reduce (segments)");
    return 0;
  }
  if (slices > 1) {
    launch_pdl(tc_linear_reduce_kernel, dim3(unsigned((T * N + 255) / 256)), dim3(256), 0, stream, (const float*)part,
               (long long)T * N, slices, int(T), int(N), a.row_scale, p.bias, p.row_div, p.resid2, p.f_out, p.b_out);
    Q35_CUDA_LAUNCH_CHECK("tc linear reduce");
  }
  return 0;
}

int tc_linear(const __nv_bfloat16* x, int64_t T, int64_t N, int64_t K, const TcLinear& p, uint8_t* qws,
              cudaStream_t stream) {
  return tc_linear_impl(x, T, N, K, p, nullptr, qws, stream);
}

int tc_linear_multi(const __nv_bfloat16* x, int64_t T, int64_t N, int64_t K, const TcLinear& p, const TcSegments& segs,
                    uint8_t* qws, cudaStream_t stream) {
  return tc_linear_impl(x, T, N, K, p, &segs, qws, stream);
}

// shared by linear.tc and lm_head: quantise x into the workspace and run the plain-epilogue GEMM
static int linear_tc_impl(const Tensor& x, const Tensor& w, const Tensor& s, const float* bias, float* f_out,
                          __nv_bfloat16* b_out, uint8_t* qws, int64_t T, int64_t N, int64_t K, cudaStream_t stream) {
  TcLinear p{};
  p.w = w.p; p.s = s.p; p.fmt = 0; p.bias = bias; p.f_out = f_out; p.b_out = b_out;
  return tc_linear(x.as<__nv_bfloat16>(), T, N, K, p, qws, stream);
}

int run_linear_tc(Call& c) {
  Tensor x, w, s, bias, out, ws;
  Q35_TRY(c.get("x", M(Q35_BF16), &x));
  Q35_TRY(c.get("w", M_BYTES, &w));
  Q35_TRY(c.get("s", M(Q35_U8), &s));
  Q35_TRY(c.get("bias", M(Q35_F32), &bias, false));
  Q35_TRY(c.get("out", M(Q35_BF16) | M(Q35_F32), &out));
  Q35_REQUIRE(x.nd >= 2 && w.nd == 2, Q35_ERR_SHAPE, "linear.tc: x [T, K], w [N, K/2]");
  const int64_t K = x.s[x.nd - 1], T = x.numel() / K, N = w.s[0];
  Q35_REQUIRE(w.s[1] == K / 2 && s.numel() == N * (K / 32) && out.numel() == T * N, Q35_ERR_SHAPE, "linear.tc: shapes");
  Q35_REQUIRE(K % 128 == 0, Q35_ERR_UNSUPPORTED, "linear.tc: K must be a multiple of 128");
  Q35_TRY(c.workspace(tc_linear_bytes(T, N, K), &ws));
  if (c.dry || T == 0 || N == 0) return 0;
  Q35_REQUIRE((uintptr_t(w.p) & 31) == 0 && aligned16(x.p) && aligned16(s.p), Q35_ERR_ALIGN, "linear.tc: alignment");
  return linear_tc_impl(x, w, s, bias.present ? bias.as<float>() : nullptr,
                        out.dtype == Q35_F32 ? out.as<float>() : nullptr,
                        out.dtype == Q35_F32 ? nullptr : out.as<__nv_bfloat16>(), ws.as<uint8_t>(), T, N, K, c.stream);
}

// ---------------------------------------------------------------------------------------------------------------
// lm_head: fp32 logits of the MXFP4 output projection and / or the greedy token per row.
// Reference: mul_mat_mx4 (models/qwen35_2b/whole/src/q35_layer_mc.py:741-758: x [1, K] bf16 x w [N, K] fp4 + s -> f32
// logits), golden torch_logits (models/qwen38_27b/head/mx4_common.py:62-69); the token is the first index of the
// row's maximum, as torch.argmax gives the reference's host code.
__global__ void __launch_bounds__(1024) argmax_rows_kernel(const float* __restrict__ logits, int N, int* __restrict__ token) {
  pdl_wait();
  pdl_launch();
  const float* row = logits + size_t(blockIdx.x) * N;
  float best = -INFINITY;
  int at = 0x7fffffff;
  for (int i = threadIdx.x; i < N; i += 1024) {  // ascending i per thread: strict > keeps the first maximum
    const float v = row[i];
    if (v > best || (v == best && i < at)) { best = v; at = i; }
  }
  __shared__ float s_v[32];
  __shared__ int s_i[32];
  auto merge = [](float& v, int& i, float ov, int oi) {
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
  };
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    merge(best, at, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, at, o));
  if ((threadIdx.x & 31) == 0) { s_v[threadIdx.x >> 5] = best; s_i[threadIdx.x >> 5] = at; }
  __syncthreads();
  if (threadIdx.x < 32) {
    best = s_v[threadIdx.x]; at = s_i[threadIdx.x];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
      merge(best, at, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, at, o));
    if (threadIdx.x == 0) token[blockIdx.x] = at == 0x7fffffff ? 0 : at;  // a row of NaNs: token 0
  }
}

int run_lm_head(Call& c) {
  Tensor x, w, s, logits, token, ws;
  Q35_TRY(c.get("x", M(Q35_BF16), &x));
  Q35_TRY(c.get("w", M_BYTES, &w));
  Q35_TRY(c.get("s", M(Q35_U8), &s));
  Q35_TRY(c.get("logits", M(Q35_F32), &logits, false));
  if (!logits.present) Q35_TRY(c.get("out", M(Q35_F32), &logits, false));  // the name in the reference's manifests
  Q35_TRY(c.get("token", M(Q35_I32), &token, false));
  Q35_REQUIRE(logits.present || token.present, Q35_ERR_MISSING, "lm_head: give logits, token or both");
  Q35_REQUIRE(x.nd >= 2 && w.nd == 2, Q35_ERR_SHAPE, "lm_head: x [T, K], w [N, K/2]");
  const int64_t K = x.s[x.nd - 1], T = x.numel() / K, N = w.s[0];
  Q35_REQUIRE(w.s[1] == K / 2 && s.numel() == N * (K / 32), Q35_ERR_SHAPE, "lm_head: w [N, K/2], s [N, K/32]");
  Q35_REQUIRE((!logits.present || logits.numel() == T * N) && (!token.present || token.numel() == T), Q35_ERR_SHAPE,
              "lm_head: logits [T, N], token [T]");
  Q35_REQUIRE(K % 512 == 0, Q35_ERR_UNSUPPORTED, "lm_head: K must be a multiple of 512");
  const int64_t qb = (tc_linear_bytes(T, N, K) + 255) / 256 * 256;
  Q35_TRY(c.workspace(qb + (logits.present ? 0 : T * N * 4), &ws));
  if (c.dry || T == 0 || N == 0) return 0;
  Q35_REQUIRE((uintptr_t(w.p) & 31) == 0 && aligned16(x.p) && aligned16(s.p), Q35_ERR_ALIGN, "lm_head: alignment");
  float* lg = logits.present ? logits.as<float>() : reinterpret_cast<float*>(ws.as<uint8_t>() + qb);
  Q35_TRY(linear_tc_impl(x, w, s, nullptr, lg, nullptr, ws.as<uint8_t>(), T, N, K, c.stream));
  if (token.present) {
    launch_pdl(argmax_rows_kernel, dim3(unsigned(T)), dim3(1024), 0, c.stream, lg, int(N), token.as<int>());
    Q35_CUDA_LAUNCH_CHECK("lm_head argmax");
  }
  return 0;
}

// ---------------------------------------------------------------------------------------------------------------
// debug.wait_probe: the bounded-wait reporting path on its own.  One thread waits, with the caller's poll limit, on an
// mbarrier that nothing ever arrives at -- the same mbar_wait the GEMM's roles use -- records DS_WAIT_TIMEOUT in the
// status word when the wait gives up, writes how it ended to `result` (1 = gave up, 0 = the barrier completed, which
// cannot happen) and returns.  Nothing faults and nothing hangs: the wait is the loop bound.
__global__ void wait_probe_kernel(const int* __restrict__ polls, int* __restrict__ result, int* status) {
  __shared__ __align__(8) uint64_t bar;
  if (threadIdx.x == 0) {
    const uint32_t b = smem_u32(&bar);
    tc::mbar_init(b, 1);
    tc::fence_barrier_init();
    int limit = polls[0];
    limit = limit < 1 ? 1 : limit > (1 << 20) ? (1 << 20) : limit;
    const bool ok = tc::mbar_wait(b, 0, uint32_t(limit));
    if (!ok) atomicOr(status, DS_WAIT_TIMEOUT);
    result[0] = ok ? 0 : 1;
  }
}

// ---------------------------------------------------------------------------------------------------------------
// debug.tc_peak: what the block-scaled tensor-core path can do with operands that are already in shared memory: every
// CTA (one per SM) issues `iters` x 4 tcgen05.mma kind::mxf8f6f4.block_scale of 128 x 256 x 32 (E2M1 x E4M3, the
// formats of the MoE GEMMs) on a fixed pseudo-random tile, nothing is loaded or stored.  The host times the launch:
// FLOP = CTAs x iters x 4 x 2 x 128 x 256 x 32.  This is the denominator "FP4 / FP8 tensor peak" of the prefill numbers.
__global__ void __launch_bounds__(128, 1) tc_peak_kernel(const int* __restrict__ iters_p, int* __restrict__ done,
                                                         int* status) {
  using namespace tc;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar;
  __shared__ uint32_t slot;
  const int tid = threadIdx.x, warp = tid >> 5;
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sgen = smem_raw + (sbase - smem_u32(smem_raw));
  for (int i = tid; i < (16384 + 32768) / 4; i += 128)  // operand tiles: A 128 x 128 bytes, B 256 x 128 bytes
    reinterpret_cast<uint32_t*>(sgen)[i] = (uint32_t(i) * 2654435761u) & 0x37373737u;  // small finite E4M3 / E2M1 codes
  if (tid == 0) { mbar_init(smem_u32(&bar), 1); fence_barrier_init(); }
  if (warp == 0) { tmem_alloc(smem_u32(&slot), 512); tmem_relinquish(); }
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(&slot);
  const int iters = iters_p[0];
  if (tid == 0) {
    const uint32_t sa = sbase, sb = sbase + 16384;
    for (int i = 0; i < iters; ++i) {
#pragma unroll
      for (int k = 0; k < 4; ++k)
        tc_mma_mxf8f6f4(tmem, smem_desc(sa + k * 32, 16, 1024, 2), smem_desc(sb + k * 32, 16, 1024, 2),
                        idesc_mxf8f6f4(FMT_E2M1, FMT_E4M3, 128, 256, k, k), tmem + 256, tmem + 264, (i | k) != 0);
    }
    tc_commit(smem_u32(&bar));
    if (!mbar_wait(smem_u32(&bar), 0, 1u << 28)) atomicOr(status, DS_WAIT_TIMEOUT);
    if (blockIdx.x == 0) done[0] = iters;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

int run_debug_tc_peak(Call& c) {
  Tensor iters, done;
  Q35_TRY(c.get("iters", M(Q35_I32), &iters));
  Q35_TRY(c.get("done", M(Q35_I32), &done));
  Q35_REQUIRE(iters.numel() == 1 && done.numel() == 1, Q35_ERR_SHAPE, "debug.tc_peak: iters [1], done [1]");
  c.ws_need = 0;
  if (c.dry) return 0;
  const int smem = 1024 + 16384 + 32768;
  Q35_TRY(ensure_dynamic_smem(reinterpret_cast<const void*>(tc_peak_kernel), smem));
  tc_peak_kernel<<<unsigned(sm_count()), 128, smem, c.stream>>>(iters.as<int>(), done.as<int>(), device_status_ptr());
  Q35_CUDA_LAUNCH_CHECK("debug.tc_peak");
  return 0;
}

int run_debug_wait_probe(Call& c) {
  Tensor polls, result;
  Q35_TRY(c.get("polls", M(Q35_I32), &polls));
  Q35_TRY(c.get("result", M(Q35_I32), &result));
  Q35_REQUIRE(polls.numel() == 1 && result.numel() == 1, Q35_ERR_SHAPE, "debug.wait_probe: polls [1], result [1]");
  c.ws_need = 0;
  if (c.dry) return 0;
  wait_probe_kernel<<<1, 32, 0, c.stream>>>(polls.as<int>(), result.as<int>(), device_status_ptr());
  Q35_CUDA_LAUNCH_CHECK("debug.wait_probe");
  return 0;
}

}  // namespace q35
