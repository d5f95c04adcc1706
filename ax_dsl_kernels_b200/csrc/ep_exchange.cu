// Expert-parallel decode exchange over peer memory (NVLink / NVSwitch): the two exchanges of the expert-parallel MoE
// step -- every rank's post-norm rows, expert ids and routing weights to all ranks before the experts, and every
// rank's fp32 partial sums of MY tokens back to me after them -- done by this library's own kernels with plain peer
// stores and peer loads instead of an all-gather and a reduce-scatter.  In the reference the same two exchanges cross
// the NPU cores' shared on-chip memory inside the layer kernel (pub / sub of logits and partial sums,
// models/qwen35_2b/whole/src/q35_layer_mc.py:830-886).
//
// Every rank owns one EXCHANGE buffer of the same layout, mapped into every other rank's address space (the host
// passes the table of the ranks' base addresses):
//   [0]    epoch (u32): number of exchanges this rank has started      [4]  arrival counter of the publish kernel
//   [256]  gather flags (u32 per source rank): "rank p's rows of exchange e are in my buffer"
//   [512]  done flags   (u32 per source rank): "rank p's partial sums of exchange e are in ITS buffer"
//   then the caller's regions, addressed by their offset from the base: h2_all [N, T, H], ids_all [N, T, K],
//   rw_all [N, T, K] (written by the peers), partial [N * T, H] fp32 (written by this rank, read by the peers).
// Flags only grow (they hold epochs), nothing is ever reset, and the step's own data dependencies order the reuse of
// the regions: a peer can start exchange e + 1 (and overwrite its slice of my gather regions, or expect my new partial
// sums) only after its reduce of exchange e, which waited for my done flag of e, which I raise after my experts of e
// have read the gather regions; and I overwrite my partial sums in exchange e + 1 only after every peer's publish of
// e + 1 arrived, which it issues after its reduce of e has read them.
//
// No kernel here waits on another kernel of the same GPU; the waits are on flags that kernels of OTHER GPUs raise,
// every wait is bounded (about a second), and a wait that runs out records DS_WAIT_TIMEOUT with its site in the
// status word and lets the kernel finish (the output of that step is then wrong and the host sees the status).
// Plain loads and stores only: no multimem, no TMA on peer memory.
#include <algorithm>

#include "abi.h"
#include "common.cuh"

namespace q35 {

constexpr int EP_MAX_RANKS = 16;
constexpr int EP_HDR_BYTES = 1024;
constexpr uint32_t EP_WAIT_POLLS = 1u << 20;  // about a second of polling

// the ranks' exchange buffer addresses as this process maps them: a table in device memory, read by the kernels
// (nothing of it is read on the host, so a call can be captured from its first use on)
struct EpPeers {
  const unsigned long long* tab;
  const int* rank_ptr;
  uint8_t* self;  // the `exchange` argument of the call: must be entry `rank` of the table
  // a table that does not name `self` at `rank` (a stale or foreign table) is recorded and the kernel does nothing
  __device__ __forceinline__ bool bound(int N, int* status) const {
    const int r = rank_ptr[0];
    if (r >= 0 && r < N && reinterpret_cast<uint8_t*>(tab[r]) == self) return true;
    if (threadIdx.x == 0 && blockIdx.x == 0) atomicOr(status, 0x4000);
    return false;
  }
  __device__ __forceinline__ uint8_t* base(int p) const { return reinterpret_cast<uint8_t*>(tab[p]); }
  __device__ __forceinline__ int rank() const { return rank_ptr[0]; }
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// waits until every one of the first n flags has reached `epoch`; false when the poll budget ran out.  Once a wait has
// run out on this GPU (the bit stays in the status word until the host reads it) later waits give up at once: a rank
// that is gone costs the others one timeout, not one per kernel of every following step.
__device__ __forceinline__ bool ep_wait_flags(const uint32_t* flags, int n, uint32_t epoch, const int* status) {
  for (int p = 0; p < n; ++p) {
    uint32_t polls = 0;
    if (int32_t(ld_acquire_sys(flags + p) - epoch) >= 0) continue;
    if (*reinterpret_cast<const volatile int*>(status) & DS_WAIT_TIMEOUT) return false;
    // (epochs wrap after 2^32 exchanges; the signed difference keeps the comparison right across the wrap)
    while (int32_t(ld_acquire_sys(flags + p) - epoch) < 0) {
      if (++polls > EP_WAIT_POLLS) return false;
      __nanosleep(20);
    }
  }
  return true;
}

// ep.publish: my rows -> slice `rank` of every rank's gather regions; the last CTA raises my gather flag everywhere
// and (wait_all) waits for everybody else's, which saves the launch of ep.wait.
__global__ void __launch_bounds__(256) ep_publish_kernel(const uint4* __restrict__ h2, const uint4* __restrict__ ids,
                                                         const uint4* __restrict__ rw, EpPeers peers, int N,
                                                         long long off_h2, long long off_ids, long long off_rw,
                                                         int n_h2, int n_ids, int n_rw,  // counts of 16-byte units
                                                         int wait_all, int* status) {
  pdl_wait();
  pdl_launch();
  if (!peers.bound(N, status)) return;
  const int rank = peers.rank();
  uint8_t* mine = peers.base(rank);
  const int per_peer = n_h2 + n_ids + n_rw;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < (long long)N * per_peer;
       i += (long long)gridDim.x * blockDim.x) {
    const int q = int(i / per_peer);
    int j = int(i % per_peer);
    uint8_t* dst = peers.base(q);
    if (j < n_h2) {
      reinterpret_cast<uint4*>(dst + off_h2)[(long long)rank * n_h2 + j] = h2[j];
    } else if ((j -= n_h2) < n_ids) {
      reinterpret_cast<uint4*>(dst + off_ids)[(long long)rank * n_ids + j] = ids[j];
    } else {
      j -= n_ids;
      reinterpret_cast<uint4*>(dst + off_rw)[(long long)rank * n_rw + j] = rw[j];
    }
  }
  __threadfence_system();  // every thread: its own peer stores are performed before the CTA reports in
  __syncthreads();
  __shared__ bool last;
  uint32_t* hdr = reinterpret_cast<uint32_t*>(mine);
  if (threadIdx.x == 0) last = atomicAdd(hdr + 1, 1u) == gridDim.x - 1;
  __syncthreads();
  if (last) {
    if (threadIdx.x == 0) hdr[1] = 0;
    const uint32_t epoch = hdr[0] + 1;  // only this CTA touches the epoch, once per launch
    __threadfence_system();
    if (threadIdx.x < N)
      st_release_sys(reinterpret_cast<uint32_t*>(peers.base(threadIdx.x) + 256) + rank, epoch);
    __syncthreads();
    if (threadIdx.x == 0) { hdr[0] = epoch; __threadfence(); }
    // ... and waits for everybody's rows of this exchange (one thread per source rank), so that the kernels that follow
    // in the stream find the gather regions complete
    if (wait_all && threadIdx.x < N &&
        !ep_wait_flags(reinterpret_cast<const uint32_t*>(mine + 256) + threadIdx.x, 1, epoch, status))
      atomicOr(status, DS_WAIT_TIMEOUT | 0x800);
  }
}

// ep.wait: until every rank's rows of the current exchange are in my gather regions
__global__ void ep_wait_gather_kernel(EpPeers peers, int N, int* status) {
  pdl_wait();
  pdl_launch();
  if (!peers.bound(N, status)) return;
  uint8_t* mine = peers.self;
  if (threadIdx.x < N) {  // one thread per source rank
    const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(mine);
    if (!ep_wait_flags(reinterpret_cast<const uint32_t*>(mine + 256) + threadIdx.x, 1, epoch, status))
      atomicOr(status, DS_WAIT_TIMEOUT | 0x800);
  }
}

// ep.reduce: raise my done flag everywhere (my partial sums were written by the previous kernel of this stream), wait
// for everybody's, then out[t] = bf16(base[t] + sum over ranks p, in rank order, of partial_p[rank * T + t]).
__global__ void __launch_bounds__(256) ep_reduce_kernel(const __nv_bfloat16* __restrict__ base, EpPeers peers, int N,
                                                        long long off_partial, int T, int H,
                                                        __nv_bfloat16* __restrict__ out, int* status) {
  pdl_wait();
  pdl_launch();
  if (!peers.bound(N, status)) return;
  const int rank = peers.rank();
  uint8_t* mine = peers.base(rank);
  __shared__ bool ok;
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(mine);
  // one thread per peer raises my done flag there (N round trips side by side, not one after the other) ...
  if (blockIdx.x == 0 && threadIdx.x < N)
    st_release_sys(reinterpret_cast<uint32_t*>(peers.base(threadIdx.x) + 512) + rank, epoch);
  // ... and one thread per peer waits for that peer's flag here
  if (threadIdx.x == 0) ok = true;
  __syncthreads();
  if (threadIdx.x < N && !ep_wait_flags(reinterpret_cast<const uint32_t*>(mine + 512) + threadIdx.x, 1, epoch, status)) {
    ok = false;
    atomicOr(status, DS_WAIT_TIMEOUT | 0x1000);
  }
  __syncthreads();
  const int vec = H / 4;  // float4 per row
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < T * vec; i += gridDim.x * blockDim.x) {
    const int t = i / vec, c = i % vec;
    const uint2 b2 = *reinterpret_cast<const uint2*>(base + size_t(t) * H + 4 * c);
    float4 acc = make_float4(bf16lo(b2.x), bf16hi(b2.x), bf16lo(b2.y), bf16hi(b2.y));
    // every rank's load goes out before the first sum (a peer load is a round trip over NVLink; one after the other
    // they would add up), the sums then run in rank order.  The same peer addresses are read every step: never from
    // a cached line.
    float4 v[EP_MAX_RANKS];
    const size_t o = off_partial + (size_t(rank) * T + t) * H * 4 + size_t(c) * 16;
#pragma unroll
    for (int p = 0; p < EP_MAX_RANKS; ++p)
      if (p < N) v[p] = __ldcv(reinterpret_cast<const float4*>(peers.base(p) + o));
#pragma unroll
    for (int p = 0; p < EP_MAX_RANKS; ++p)
      if (p < N) { acc.x += v[p].x; acc.y += v[p].y; acc.z += v[p].z; acc.w += v[p].w; }
    *reinterpret_cast<uint2*>(out + size_t(t) * H + 4 * c) = make_uint2(pack_bf16(acc.x, acc.y), pack_bf16(acc.z, acc.w));
  }
}

// ar.oneshot: sum over the ranks of an fp32 tensor of a few hundred kilobytes -- the all-reduce after every sublayer's
// output projection in the tensor-parallel decode group (reduce(), models/qwen38_27b/decode/q35_group.py:128-137; the
// NPU cores add their partial sums through shared memory) -- in ONE kernel: every rank stores its tensor into slot
// `rank` of every rank's buffer, raises its flag everywhere, waits for everybody's flag and adds the N slots in rank
// order (the same order on every rank: bit-identical results).  Slots are double-buffered by the parity of the exchange
// count: a rank can be at most one exchange ahead of another (it cannot finish exchange e + 1 without the other's flag
// of e + 1, raised after that rank is done reading exchange e).  Layout: the 1 KB header as above (epoch, counter, flags
// at 256), then [2 parities][N ranks][bytes of the tensor, rounded up to 256].
__global__ void __launch_bounds__(256) ar_oneshot_kernel(const float4* __restrict__ x, EpPeers peers, int N,
                                                         int n_vec, long long slot_bytes, float4* __restrict__ out,
                                                         int* status) {
  pdl_wait();
  pdl_launch();
  if (!peers.bound(N, status)) return;
  const int rank = peers.rank();
  uint8_t* mine = peers.base(rank);
  uint32_t* hdr = reinterpret_cast<uint32_t*>(mine);
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(hdr) + 1;  // (updated by the last CTA, after every CTA read it)
  const long long par = (long long)(epoch & 1u) * N * slot_bytes;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += gridDim.x * blockDim.x) {
    const float4 v = x[i];
#pragma unroll
    for (int q = 0; q < EP_MAX_RANKS; ++q)
      if (q < N) reinterpret_cast<float4*>(peers.base(q) + EP_HDR_BYTES + par + rank * slot_bytes)[i] = v;
  }
  __threadfence_system();
  __syncthreads();
  __shared__ bool last;
  if (threadIdx.x == 0) last = atomicAdd(hdr + 1, 1u) == gridDim.x - 1;
  __syncthreads();
  if (last) {
    __threadfence_system();
    if (threadIdx.x < N) st_release_sys(reinterpret_cast<uint32_t*>(peers.base(threadIdx.x) + 256) + rank, epoch);
    if (threadIdx.x == 0) { hdr[1] = 0; hdr[0] = epoch; }
  }
  if (threadIdx.x < N && !ep_wait_flags(reinterpret_cast<const uint32_t*>(mine + 256) + threadIdx.x, 1, epoch, status))
    atomicOr(status, DS_WAIT_TIMEOUT | 0x2000);
  __syncthreads();
  const uint8_t* slots = mine + EP_HDR_BYTES + par;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += gridDim.x * blockDim.x) {
    float4 v[EP_MAX_RANKS];
#pragma unroll
    for (int p = 0; p < EP_MAX_RANKS; ++p)
      if (p < N) v[p] = __ldcv(reinterpret_cast<const float4*>(slots + p * slot_bytes) + i);  // written by peers: not cached
    float4 acc = v[0];
#pragma unroll
    for (int p = 1; p < EP_MAX_RANKS; ++p)
      if (p < N) { acc.x += v[p].x; acc.y += v[p].y; acc.z += v[p].z; acc.w += v[p].w; }
    out[i] = acc;
  }
}

// ---------------------------------------------------------------------------------------------------------------
static int ep_common(Call& c, const char* role, Tensor* ex, EpPeers* peers, int* N) {
  Tensor pt, rk;
  Q35_TRY(c.get("exchange", M(Q35_U8), ex));
  Q35_TRY(c.get("peers", M(Q35_U8), &pt));
  Q35_TRY(c.get("rank", M(Q35_I32), &rk));
  Q35_REQUIRE(pt.bytes % 8 == 0 && pt.bytes >= 8 && pt.bytes <= 8 * EP_MAX_RANKS, Q35_ERR_SHAPE,
              "%s: peers = one 8-byte address per rank (at most %d ranks)", role, EP_MAX_RANKS);
  *N = int(pt.bytes / 8);
  Q35_REQUIRE(rk.numel() >= 1, Q35_ERR_SHAPE, "%s: rank [1]", role);
  Q35_REQUIRE(ex->bytes >= EP_HDR_BYTES && (reinterpret_cast<uintptr_t>(ex->p) & 255) == 0 &&
                  (reinterpret_cast<uintptr_t>(pt.p) & 7) == 0, Q35_ERR_ALIGN,
              "%s: exchange must be 256-byte aligned and hold the 1 KB header; peers 8-byte aligned", role);
  // peers[rank] must be this rank's own buffer, `exchange`: the kernels check it and record 0x4000 otherwise
  peers->tab = static_cast<const unsigned long long*>(pt.p);
  peers->rank_ptr = rk.as<int>();
  peers->self = ex->as<uint8_t>();
  return 0;
}

static int region_offset(const char* role, const Tensor& ex, const Tensor& t, const char* name, long long* off) {
  const long long o = static_cast<const uint8_t*>(t.p) - static_cast<const uint8_t*>(ex.p);
  Q35_REQUIRE(o >= EP_HDR_BYTES && o + (long long)t.bytes <= (long long)ex.bytes && (o & 15) == 0, Q35_ERR_SHAPE,
              "%s: %s must be a 16-byte aligned region of `exchange` past its 1 KB header", role, name);
  *off = o;
  return 0;
}

int run_ep_publish(Call& c) {
  Tensor ex, h2, ids, rw, h2a, idsa, rwa;
  EpPeers peers{};
  int N = 0;
  Q35_TRY(c.get("h2", M(Q35_BF16), &h2));
  Q35_TRY(c.get("ids", M(Q35_I32), &ids));
  Q35_TRY(c.get("rw", M(Q35_F32), &rw));
  Q35_TRY(c.get("h2_all", M(Q35_BF16), &h2a));
  Q35_TRY(c.get("ids_all", M(Q35_I32), &idsa));
  Q35_TRY(c.get("rw_all", M(Q35_F32), &rwa));
  Tensor nowait;  // bound (any i32 [1]): return after publishing; the host calls ep.wait later, with work in between
  Q35_TRY(c.get("no_wait", M(Q35_I32), &nowait, false));
  Q35_TRY(ep_common(c, "ep.publish", &ex, &peers, &N));
  Q35_REQUIRE(h2a.bytes == h2.bytes * N && idsa.bytes == ids.bytes * N && rwa.bytes == rw.bytes * N, Q35_ERR_SHAPE,
              "ep.publish: the *_all regions hold one slice per rank");
  Q35_REQUIRE(h2.bytes % 16 == 0 && ids.bytes % 16 == 0 && rw.bytes % 16 == 0 && aligned16(h2.p) && aligned16(ids.p) &&
                  aligned16(rw.p), Q35_ERR_ALIGN, "ep.publish: slices in multiples of 16 bytes, 16-byte aligned");
  c.ws_need = 0;
  if (c.dry) return 0;
  long long o1, o2, o3;
  Q35_TRY(region_offset("ep.publish", ex, h2a, "h2_all", &o1));
  Q35_TRY(region_offset("ep.publish", ex, idsa, "ids_all", &o2));
  Q35_TRY(region_offset("ep.publish", ex, rwa, "rw_all", &o3));
  const int n1 = int(h2.bytes / 16), n2 = int(ids.bytes / 16), n3 = int(rw.bytes / 16);
  const long long units = (long long)N * (n1 + n2 + n3);
  const unsigned grid = unsigned(std::min<long long>((units + 255) / 256, 2 * sm_count()));
  launch_pdl(ep_publish_kernel, dim3(grid), dim3(256), 0, c.stream, static_cast<const uint4*>(h2.p),
             static_cast<const uint4*>(ids.p), static_cast<const uint4*>(rw.p), peers, N, o1, o2, o3, n1, n2, n3,
             nowait.present ? 0 : 1, device_status_ptr());
  Q35_CUDA_LAUNCH_CHECK("ep.publish");
  return 0;
}

int run_ep_wait(Call& c) {
  Tensor ex;
  EpPeers peers{};
  int N = 0;
  Q35_TRY(ep_common(c, "ep.wait", &ex, &peers, &N));
  c.ws_need = 0;
  if (c.dry) return 0;
  launch_pdl(ep_wait_gather_kernel, dim3(1), dim3(32), 0, c.stream, peers, N, device_status_ptr());
  Q35_CUDA_LAUNCH_CHECK("ep.wait");
  return 0;
}

int run_ep_reduce(Call& c) {
  Tensor ex, base, partial, out;
  EpPeers peers{};
  int N = 0;
  Q35_TRY(c.get("base", M(Q35_BF16), &base));
  Q35_TRY(c.get("partial", M(Q35_F32), &partial));
  Q35_TRY(c.get("out", M(Q35_BF16), &out));
  Q35_TRY(ep_common(c, "ep.reduce", &ex, &peers, &N));
  Q35_REQUIRE(base.nd == 2 && out.numel() == base.numel(), Q35_ERR_SHAPE, "ep.reduce: base, out [T, H]");
  const int64_t T = base.s[0], H = base.s[1];
  Q35_REQUIRE(partial.numel() == int64_t(N) * T * H && H % 4 == 0, Q35_ERR_SHAPE, "ep.reduce: partial [N * T, H], H % 4 == 0");
  c.ws_need = 0;
  if (c.dry || T == 0) return 0;
  long long off;
  Q35_TRY(region_offset("ep.reduce", ex, partial, "partial", &off));
  Q35_REQUIRE(aligned16(base.p) && aligned16(out.p), Q35_ERR_ALIGN, "ep.reduce: base, out 16-byte aligned");
  const unsigned grid = unsigned(std::min<int64_t>((T * (H / 4) + 255) / 256, 2 * sm_count()));
  launch_pdl(ep_reduce_kernel, dim3(grid), dim3(256), 0, c.stream, base.as<__nv_bfloat16>(), peers, N, off,
             int(T), int(H), out.as<__nv_bfloat16>(), device_status_ptr());
  Q35_CUDA_LAUNCH_CHECK("ep.reduce");
  return 0;
}

int run_ar_oneshot(Call& c) {
  Tensor ex, x, out;
  EpPeers peers{};
  int N = 0;
  Q35_TRY(c.get("x", M(Q35_F32), &x));
  Q35_TRY(c.get("out", M(Q35_F32), &out));
  Q35_TRY(ep_common(c, "ar.oneshot", &ex, &peers, &N));
  Q35_REQUIRE(out.numel() == x.numel() && x.numel() % 4 == 0, Q35_ERR_SHAPE, "ar.oneshot: out like x, a multiple of 4 elements");
  const long long slot = (long long)(x.bytes + 255) / 256 * 256;
  Q35_REQUIRE((long long)ex.bytes >= EP_HDR_BYTES + 2 * N * slot, Q35_ERR_WORKSPACE,
              "ar.oneshot: exchange must hold the 1 KB header and 2 x %d slots of %lld bytes", N, slot);
  c.ws_need = 0;
  if (c.dry || x.numel() == 0) return 0;
  Q35_REQUIRE(aligned16(x.p) && aligned16(out.p), Q35_ERR_ALIGN, "ar.oneshot: x, out 16-byte aligned");
  const int n_vec = int(x.numel() / 4);
  // every CTA waits for the peers' flags: the grid must be resident at once
  const unsigned grid = unsigned(std::min<long long>((n_vec + 255) / 256, sm_count()));
  launch_pdl(ar_oneshot_kernel, dim3(grid), dim3(256), 0, c.stream, static_cast<const float4*>(x.p), peers, N, n_vec,
             slot, static_cast<float4*>(out.p), device_status_ptr());
  Q35_CUDA_LAUNCH_CHECK("ar.oneshot");
  return 0;
}

}  // namespace q35
