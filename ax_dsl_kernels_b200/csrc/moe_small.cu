// Small kernels of the MoE block: router (softmax / top-k / renormalise), token -> expert grouping, combine.
#include "abi.h"
#include "common.cuh"
#include "moe_group.cuh"

namespace q35 {

// ---------------------------------------------------------------------------------------------------------------
// moe.route: reference host router `route` (models/qwen35_2b/whole/src/q35_moe.py:293-297) batched on device:
// softmax fp32 over all experts, top-K, weights / their sum.  Order: descending, exact ties to the lower expert id
// (the rule of models/qwen35_2b/whole/src/q35_layer_mc.py:1494-1499).  Selection compares the logits themselves
// (the probabilities are a monotone function of them), the weights are computed from the full softmax as the
// reference does.  One warp per token; lane i holds experts i, i + 32, ...
template <int PER>
__global__ void moe_route_kernel(const float* __restrict__ logits, int* __restrict__ ids, float* __restrict__ rw,
                                 int T, int NE, int K) {
  pdl_wait();
  pdl_launch();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= T) return;
  const float* row = logits + size_t(warp) * NE;
  float v[PER];
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int e = lane + 32 * j;
    v[j] = e < NE ? row[e] : -INFINITY;
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
  float my_p = 0.f;  // lane k keeps the k-th selected probability
  int my_id = 0;
  float sel_sum = 0.f;
  for (int k = 0; k < K; ++k) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int e = lane + 32 * j;
      const bool ok = e < NE && !((taken >> j) & 1u);
      if (ok && (v[j] > bv || (v[j] == bv && e < bi))) { bv = v[j]; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (bi != 0x7fffffff && (bi & 31) == lane) taken |= 1u << (bi >> 5);
    const float p = bi != 0x7fffffff ? expf(bv - mx) / z : 0.f;
    sel_sum += p;  // same order on every lane
    if (lane == k) { my_p = p; my_id = bi != 0x7fffffff ? bi : 0; }
  }
  if (lane < K) {
    ids[size_t(warp) * K + lane] = my_id;
    rw[size_t(warp) * K + lane] = my_p / sel_sum;
  }
}

int run_moe_route(Call& c) {
  Tensor lg, ids, rw;
  Q35_TRY(c.get("logits", M(Q35_F32), &lg));
  Q35_TRY(c.get("ids", M(Q35_I32), &ids));
  Q35_TRY(c.get("rw", M(Q35_F32), &rw));
  Q35_REQUIRE(lg.nd >= 2 && ids.nd >= 2, Q35_ERR_SHAPE, "moe.route: logits [T, NE], ids [T, K]");
  const int64_t NE = lg.s[lg.nd - 1], T = lg.numel() / (NE ? NE : 1), K = ids.s[ids.nd - 1];
  Q35_REQUIRE(NE >= 1 && NE <= 1024, Q35_ERR_UNSUPPORTED, "moe.route: NE %lld outside [1, 1024]", (long long)NE);
  Q35_REQUIRE(K >= 1 && K <= 32 && K <= NE, Q35_ERR_SHAPE, "moe.route: K %lld", (long long)K);
  Q35_REQUIRE(ids.numel() == T * K && rw.numel() == T * K, Q35_ERR_SHAPE, "moe.route: ids / rw must be [T, K]");
  c.ws_need = 0;
  if (c.dry || T == 0) return 0;
  const int per = int((NE + 31) / 32);
  const unsigned blocks = unsigned((T + 3) / 4);
#define Q35_ROUTE(P) \
  launch_pdl(moe_route_kernel<P>, dim3(blocks), dim3(128), 0, c.stream, lg.as<float>(), ids.as<int>(), rw.as<float>(), \
             int(T), int(NE), int(K))
  if (per <= 1) Q35_ROUTE(1);
  else if (per <= 2) Q35_ROUTE(2);
  else if (per <= 4) Q35_ROUTE(4);
  else if (per <= 8) Q35_ROUTE(8);
  else if (per <= 16) Q35_ROUTE(16);
  else Q35_ROUTE(32);
#undef Q35_ROUTE
  Q35_CUDA_LAUNCH_CHECK("moe.route");
  return 0;
}

// ---------------------------------------------------------------------------------------------------------------
// Grouping of (token, k) pairs by expert: a counting sort that is stable in token index.  One CTA per expert scans
// the ids in token order and compacts the pairs that chose it, so the result does not depend on scheduling.
// counts[e] = number of pairs, list[e * T + j] = pair index t * K + k of the j-th token (ascending t) of expert e.
// base (optional): first global expert id of this rank's planes; ids outside [base, base + NE) belong to other ranks.
// A thread takes four consecutive tokens of every 1024 (their ids as 16-byte loads when K allows, all in flight), so
// a prefill-sized call pays one block-wide hand-over per 1024 tokens.
__global__ void __launch_bounds__(256) moe_group_count_kernel(const int* __restrict__ ids, const int* __restrict__ base,
                                                              int T, int K, int NE, int* __restrict__ counts,
                                                              int* __restrict__ list, int* status) {
  const int e = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  const int first = base ? base[0] : 0;
  __shared__ int s_warp[8];
  __shared__ int s_base;
  if (tid == 0) s_base = 0;
  __syncthreads();
  const bool vec = (K & 3) == 0 && (reinterpret_cast<uintptr_t>(ids) & 15) == 0;
  bool bad = false;
  for (int t0 = 0; t0 < T; t0 += 1024) {
    int hit[4] = {-1, -1, -1, -1};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int t = t0 + tid * 4 + j;
      if (t >= T) continue;
      const int* row = ids + size_t(t) * K;
      if (vec) {
        for (int k = 0; k < K; k += 4) {
          const int4 v = *reinterpret_cast<const int4*>(row + k);
          const int id4[4] = {v.x - first, v.y - first, v.z - first, v.w - first};
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            if (id4[u] == e && hit[j] < 0) hit[j] = k + u;
            bad |= id4[u] >= NE;
          }
        }
      } else {
        for (int k = 0; k < K; ++k) {
          const int id = row[k] - first;
          if (id == e && hit[j] < 0) hit[j] = k;
          bad |= id >= NE;
        }
      }
    }
    const int cnt = (hit[0] >= 0) + (hit[1] >= 0) + (hit[2] >= 0) + (hit[3] >= 0);
    int inc = cnt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += n;
    }
    if (lane == 31) s_warp[wid] = inc;
    __syncthreads();
    int at = s_base + inc - cnt;
    for (int w = 0; w < wid; ++w) at += s_warp[w];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (hit[j] >= 0) list[size_t(e) * T + at++] = (t0 + tid * 4 + j) * K + hit[j];
    __syncthreads();
    if (tid == 0) {
      int tot = 0;
      for (int w = 0; w < 8; ++w) tot += s_warp[w];
      s_base += tot;
    }
    __syncthreads();
  }
  if (e == 0 && !base && bad) atomicOr(status, DS_BAD_EXPERT);  // with a base, foreign ids mean "not on this rank"
  if (tid == 0) counts[e] = s_base;
}

int launch_group_count(const int* ids, const int* base, int T, int K, int NE, int* counts, int* list,
                       cudaStream_t stream) {
  moe_group_count_kernel<<<unsigned(NE), 256, 0, stream>>>(ids, base, T, K, NE, counts, list, device_status_ptr());
  Q35_CUDA_LAUNCH_CHECK("moe group count");
  return 0;
}

// moe.permute: slot tables of the prefill kernels (reference: rule at
// models/qwen35_2b/whole/src/q35_moe_prefill.py:150-152,194-195; the permutation itself is host code of the
// reference's adapter).  Experts in id order, each expert's tokens in index order, ceil(n / G) slots per expert.
__global__ void __launch_bounds__(256) moe_permute_fill_kernel(const int* __restrict__ counts,
                                                               const int* __restrict__ list,
                                                               const float* __restrict__ rw, int T, int K, int NE, int G,
                                                               int S, int* __restrict__ tok, float* __restrict__ srw,
                                                               int* __restrict__ loc, int* __restrict__ n_slots) {
  const int e = blockIdx.x;
  const int tid = threadIdx.x;
  __shared__ int s_red[256];
  int mine = 0, total = 0;
  for (int i = tid; i < NE; i += 256) {
    const int sl = (counts[i] + G - 1) / G;
    total += sl;
    if (i < e) mine += sl;
  }
  s_red[tid] = mine;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (tid < o) s_red[tid] += s_red[tid + o];
    __syncthreads();
  }
  const int slot0 = s_red[0];
  __syncthreads();
  s_red[tid] = total;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (tid < o) s_red[tid] += s_red[tid + o];
    __syncthreads();
  }
  const int used = s_red[0];
  const int n = counts[e];
  const int my_slots = (n + G - 1) / G;
  for (int j = tid; j < my_slots * G; j += 256) {
    const int slot = slot0 + j / G, col = j % G;
    if (slot >= S) continue;  // table too small: reported through n_slots > S
    if (j < n) {
      const int p = list[size_t(e) * T + j];
      const int t = p / K, k = p % K;
      tok[size_t(slot) * (1 + G) + 1 + col] = t;
      srw[size_t(slot) * G + col] = rw[p];
      loc[size_t(k) * T + t] = slot * G + col;
    } else {
      tok[size_t(slot) * (1 + G) + 1 + col] = 0;
      srw[size_t(slot) * G + col] = 0.f;
    }
    if (col == 0) tok[size_t(slot) * (1 + G)] = e;
  }
  if (e == 0) {
    if (tid == 0) n_slots[0] = used;
    for (int j = used * G + tid; j < S * G; j += 256) {  // unused slots: expert 0, token 0, weight 0
      const int slot = j / G, col = j % G;
      tok[size_t(slot) * (1 + G) + 1 + col] = 0;
      srw[size_t(slot) * G + col] = 0.f;
      if (col == 0) tok[size_t(slot) * (1 + G)] = 0;
    }
  }
}

int run_moe_permute(Call& c) {
  Tensor ids, rw, tok, srw, loc, ns, counts, ws;
  Q35_TRY(c.get("ids", M(Q35_I32), &ids));
  Q35_TRY(c.get("rw", M(Q35_F32), &rw));
  Q35_TRY(c.get("tok", M(Q35_I32), &tok));
  Q35_TRY(c.get("srw", M(Q35_F32), &srw));
  Q35_TRY(c.get("loc", M(Q35_I32), &loc));
  Q35_TRY(c.get("n_slots", M(Q35_I32), &ns));
  Q35_TRY(c.get("counts", M(Q35_I32), &counts));
  Q35_REQUIRE(ids.nd == 2 && tok.nd == 2 && srw.nd == 2 && loc.nd == 2, Q35_ERR_SHAPE, "moe.permute: ranks");
  const int64_t T = ids.s[0], K = ids.s[1], S = tok.s[0], G = tok.s[1] - 1, NE = counts.numel();
  Q35_REQUIRE(G >= 1 && srw.s[0] == S && srw.s[1] == G, Q35_ERR_SHAPE, "moe.permute: tok [S, 1+G], srw [S, G]");
  Q35_REQUIRE(rw.numel() == T * K && loc.s[0] == K && loc.s[1] == T && ns.numel() >= 1 && NE >= 1, Q35_ERR_SHAPE,
              "moe.permute: rw [T, K], loc [K, T], n_slots [1], counts [NE]");
  Q35_TRY(c.workspace(NE * T * 4, &ws));
  if (c.dry || T == 0) return 0;
  Q35_TRY(launch_group_count(ids.as<int>(), nullptr, int(T), int(K), int(NE), counts.as<int>(), ws.as<int>(), c.stream));
  moe_permute_fill_kernel<<<unsigned(NE), 256, 0, c.stream>>>(counts.as<int>(), ws.as<int>(), rw.as<float>(), int(T),
                                                              int(K), int(NE), int(G), int(S), tok.as<int>(),
                                                              srw.as<float>(), loc.as<int>(), ns.as<int>());
  Q35_CUDA_LAUNCH_CHECK("moe.permute");
  return 0;
}

// ---------------------------------------------------------------------------------------------------------------
// moe.combine: out[t] = bf16(base[t] + sum_k sout[loc[k, t]]), fp32, k ascending
// (models/qwen35_2b/whole/src/q35_moe_prefill.py:201-214).  One thread per 8 channels.
// expert-parallel form: partial[t] = sum over the pairs present on this rank (loc >= 0) of sout[loc[k, t]], fp32
template <typename ST>
__global__ void __launch_bounds__(256) moe_partial_sum_kernel(const int* __restrict__ loc, const ST* __restrict__ sout,
                                                              float* __restrict__ partial, int T, int H, int K, int R) {
  pdl_wait();
  pdl_launch();
  const int t = blockIdx.x;
  const int h = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
  if (h >= H) return;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int k0 = 0; k0 < K; k0 += 8) {  // the loads of eight pairs go out together; the sum keeps the order of k
    float4 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int r = k0 + u < K ? loc[size_t(k0 + u) * T + t] : -1;
      v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (r >= 0 && r < R) {
        if constexpr (sizeof(ST) == 4) {
          v[u] = *reinterpret_cast<const float4*>(sout + size_t(r) * H + h);
        } else {
          const uint2 b = *reinterpret_cast<const uint2*>(sout + size_t(r) * H + h);
          v[u] = make_float4(bf16lo(b.x), bf16hi(b.x), bf16lo(b.y), bf16hi(b.y));
        }
      }
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) { acc.x += v[u].x; acc.y += v[u].y; acc.z += v[u].z; acc.w += v[u].w; }
  }
  *reinterpret_cast<float4*>(partial + size_t(t) * H + h) = acc;
}

int launch_partial_sum(const int* loc, const void* sout, bool sout_f32, float* partial, int T, int H, int K, int R,
                       cudaStream_t stream) {
  const dim3 grid(unsigned(T), unsigned((H / 4 + 255) / 256));
  if (sout_f32)
    launch_pdl(moe_partial_sum_kernel<float>, grid, dim3(256), 0, stream, loc, static_cast<const float*>(sout), partial, T,
               H, K, R);
  else
    launch_pdl(moe_partial_sum_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, loc,
               static_cast<const __nv_bfloat16*>(sout), partial, T, H, K, R);
  Q35_CUDA_LAUNCH_CHECK("moe partial sum");
  return 0;
}

template <typename ST>
__global__ void __launch_bounds__(256) moe_combine_kernel(const __nv_bfloat16* __restrict__ base,
                                                          const int* __restrict__ loc, const ST* __restrict__ sout,
                                                          __nv_bfloat16* __restrict__ out, int T, int H, int K, int R,
                                                          int* status) {
  const int t = blockIdx.x;
  for (int h = threadIdx.x * 8; h < H; h += blockDim.x * 8) {
    float acc[8];
    {
      const uint4 b = *reinterpret_cast<const uint4*>(base + size_t(t) * H + h);
      acc[0] = bf16lo(b.x); acc[1] = bf16hi(b.x); acc[2] = bf16lo(b.y); acc[3] = bf16hi(b.y);
      acc[4] = bf16lo(b.z); acc[5] = bf16hi(b.z); acc[6] = bf16lo(b.w); acc[7] = bf16hi(b.w);
    }
    for (int k = 0; k < K; ++k) {
      const int r = loc[size_t(k) * T + t];
      if (r < 0) continue;  // no row: a pair of another rank, a bad expert id (reported by the plan), a second listing
      if (r >= R) {
        if (h == 0) atomicOr(status, DS_BAD_TOKEN);
        continue;
      }
      if constexpr (sizeof(ST) == 4) {
        const float4 a = *reinterpret_cast<const float4*>(sout + size_t(r) * H + h);
        const float4 b = *reinterpret_cast<const float4*>(sout + size_t(r) * H + h + 4);
        acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
        acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
      } else {
        const uint4 b = *reinterpret_cast<const uint4*>(sout + size_t(r) * H + h);
        acc[0] += bf16lo(b.x); acc[1] += bf16hi(b.x); acc[2] += bf16lo(b.y); acc[3] += bf16hi(b.y);
        acc[4] += bf16lo(b.z); acc[5] += bf16hi(b.z); acc[6] += bf16lo(b.w); acc[7] += bf16hi(b.w);
      }
    }
    uint4 o;
    o.x = pack_bf16(acc[0], acc[1]); o.y = pack_bf16(acc[2], acc[3]);
    o.z = pack_bf16(acc[4], acc[5]); o.w = pack_bf16(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(out + size_t(t) * H + h) = o;
  }
}

int launch_combine(const __nv_bfloat16* base, const int* loc, const void* sout, bool sout_f32, __nv_bfloat16* out,
                   int T, int H, int K, int R, cudaStream_t stream) {
  if (sout_f32)
    moe_combine_kernel<float><<<unsigned(T), 256, 0, stream>>>(base, loc, static_cast<const float*>(sout), out, T, H, K,
                                                               R, device_status_ptr());
  else
    moe_combine_kernel<__nv_bfloat16><<<unsigned(T), 256, 0, stream>>>(
        base, loc, static_cast<const __nv_bfloat16*>(sout), out, T, H, K, R, device_status_ptr());
  Q35_CUDA_LAUNCH_CHECK("moe.combine");
  return 0;
}

int run_moe_combine(Call& c) {
  Tensor base, loc, sout, out;
  Q35_TRY(c.get("base", M(Q35_BF16), &base));
  Q35_TRY(c.get("loc", M(Q35_I32), &loc));
  Q35_TRY(c.get("sout", M(Q35_BF16) | M(Q35_F32), &sout));
  Q35_TRY(c.get("out", M(Q35_BF16), &out));
  Q35_REQUIRE(base.nd == 2 && loc.nd == 2 && sout.nd == 2, Q35_ERR_SHAPE, "moe.combine: base [T,H], loc [K,T], sout [R,H]");
  const int64_t T = base.s[0], H = base.s[1], K = loc.s[0], R = sout.s[0];
  Q35_REQUIRE(loc.s[1] == T && sout.s[1] == H && out.numel() == T * H, Q35_ERR_SHAPE, "moe.combine: shapes");
  Q35_REQUIRE(H % 8 == 0, Q35_ERR_UNSUPPORTED, "moe.combine: H must be a multiple of 8");
  c.ws_need = 0;
  if (c.dry || T == 0) return 0;
  Q35_REQUIRE(aligned16(base.p) && aligned16(sout.p) && aligned16(out.p), Q35_ERR_ALIGN, "moe.combine: alignment");
  return launch_combine(base.as<__nv_bfloat16>(), loc.as<int>(), sout.p, sout.dtype == Q35_F32,
                        out.as<__nv_bfloat16>(), int(T), int(H), int(K), int(R), c.stream);
}

}  // namespace q35
