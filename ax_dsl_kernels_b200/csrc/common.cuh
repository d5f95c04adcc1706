// Device helpers shared by the kernels (sm_100a).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace q35 {

// bits recorded in the device status word
enum : int { DS_BAD_PAGE = 1, DS_BAD_EXPERT = 2, DS_WAIT_TIMEOUT = 4, DS_BAD_TOKEN = 8 };

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t lo16) { return __uint_as_float(lo16 << 16); }
__device__ __forceinline__ float bf16lo(uint32_t pair) { return __uint_as_float(pair << 16); }
__device__ __forceinline__ float bf16hi(uint32_t pair) { return __uint_as_float(pair & 0xffff0000u); }
__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ uint32_t pack_f16(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Programmatic dependent launch (see launch_pdl in abi.h).  pdl_wait: returns once the previous kernel of the stream
// has completed and its writes are visible; nothing in global memory may be touched before it.  pdl_launch: lets the
// next kernel's CTAs become resident (they stop at their own pdl_wait until THIS grid has completed).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ uint4 ldg_nc_16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint2 ldg_nc_8(const void* p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t ldg_nc_4(const void* p) {
  uint32_t v;
  asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void cp_async_16(uint32_t smem_addr, const void* gptr) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr), "l"(gptr));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                                  uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
  return d;
}

// D(16x8, f32) += A(16x16, bf16 row) * B(16x8, bf16 col)
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_f16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + __expf(-x)); }

// E8M0 byte -> 2^(s - 127) as fp32 (s = 0 gives 2^-127, a denormal; s = 255 is NaN in the format)
__device__ __forceinline__ float e8m0_to_f32(uint32_t s) {
  return s == 0 ? __uint_as_float(0x00400000u) : __uint_as_float(s << 23);
}

// RMSNorm of a row by a block of 256 threads, H a multiple of 8 and at most 8192: thread `tid` holds the 16-byte pieces
// tid, tid + 256, ... of the row (at most four), all loaded before the first use.  The sum of squares is taken per
// thread over its elements in order, then over the warp (warp_sum), then over the eight warp sums in order: every
// kernel that normalises through these helpers produces the same bits.
constexpr int RMS_MAX_PIECES = 4;
struct RmsPieces { uint4 v[RMS_MAX_PIECES]; };
__device__ __forceinline__ void rms_load(const __nv_bfloat16* xr, int H, int tid, RmsPieces& p) {
#pragma unroll
  for (int c = 0; c < RMS_MAX_PIECES; ++c) {
    const int i = (tid + 256 * c) * 8;
    p.v[c] = i < H ? *reinterpret_cast<const uint4*>(xr + i) : make_uint4(0u, 0u, 0u, 0u);
  }
}
__device__ __forceinline__ float rms_sumsq(const RmsPieces& p) {
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < RMS_MAX_PIECES; ++c) {
    const uint32_t w[4] = {p.v[c].x, p.v[c].y, p.v[c].z, p.v[c].w};
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const float a = bf16lo(w[u]), b = bf16hi(w[u]);
      ss += a * a;
      ss += b * b;
    }
  }
  return ss;
}
// the running sum of squares continued over one more piece (same element order as rms_sumsq)
__device__ __forceinline__ float rms_chain(float ss, const uint4& v) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const float a = bf16lo(w[u]), b = bf16hi(w[u]);
    ss += a * a;
    ss += b * b;
  }
  return ss;
}
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

// y = bf16(x * rs * w) for this thread's pieces; dst0 / dst1 (either may be null) receive the row
__device__ __forceinline__ void rms_apply(const RmsPieces& p, int H, int tid, float rs, const float* __restrict__ w,
                                          __nv_bfloat16* dst0, __nv_bfloat16* dst1) {
#pragma unroll
  for (int c = 0; c < RMS_MAX_PIECES; ++c) {
    const int i = (tid + 256 * c) * 8;
    if (i >= H) break;
    const float4 w0 = *reinterpret_cast<const float4*>(w + i), w1 = *reinterpret_cast<const float4*>(w + i + 4);
    uint4 o;
    o.x = pack_bf16(bf16lo(p.v[c].x) * rs * w0.x, bf16hi(p.v[c].x) * rs * w0.y);
    o.y = pack_bf16(bf16lo(p.v[c].y) * rs * w0.z, bf16hi(p.v[c].y) * rs * w0.w);
    o.z = pack_bf16(bf16lo(p.v[c].z) * rs * w1.x, bf16hi(p.v[c].z) * rs * w1.y);
    o.w = pack_bf16(bf16lo(p.v[c].w) * rs * w1.z, bf16hi(p.v[c].w) * rs * w1.w);
    if (dst0) *reinterpret_cast<uint4*>(dst0 + i) = o;
    if (dst1) *reinterpret_cast<uint4*>(dst1 + i) = o;
  }
}

// exponent of the UE8M0 block scale of an E4M3 block: the smallest e with amax * 2^-e <= 448 (= 1.75 * 2^8)
__device__ __forceinline__ int e8m0_for(float amax) {
  if (amax == 0.f) return -127;
  const uint32_t b = __float_as_uint(amax);
  const int E = int(b >> 23) - 127;
  const uint32_t mant = b & 0x7fffffu;
  int e = E - 8 + (mant > 0x600000u ? 1 : 0);  // mantissa above 1.75 needs one more octave
  return max(-127, min(127, e));
}

// 2^e as a float for the exponents a UE8M0 scale can name (-127 is the subnormal 2^-127): no special-function unit
__device__ __forceinline__ float pow2_int(int e) {
  return __uint_as_float(e > -127 ? uint32_t(e + 127) << 23 : 0x00400000u);
}

// Eight consecutive values of a block of 32 that four neighbouring lanes hold -> two E4M3 terms with UE8M0 block
// exponents: v = hi * 2^eh + lo * 2^el up to 2^-9 of the block's maximum.  Every lane of the warp calls (shuffles).
// Conversions go two at a time (cvt.rn.satfinite.e4m3x2.f32 and cvt.rn.f16x2.e4m3x2): the conversion unit is the
// narrow one, and a prefill-sized quantisation is bound by it.
struct TwoTerm8 {
  uint2 hi, lo;  // eight E4M3 bytes each, element u in byte u
  int eh, el;
};
__device__ __forceinline__ TwoTerm8 quant_two_terms8(const float (&v)[8]) {
  TwoTerm8 t;
  float amax = 0.f;
#pragma unroll
  for (int u = 0; u < 8; ++u) amax = fmaxf(amax, fabsf(v[u]));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  t.eh = e8m0_for(amax);
  const float dn = pow2_int(-t.eh), up = pow2_int(t.eh);
  uint32_t hw[4], lw[4];
  float rem[8];
  float rmax = 0.f;
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const __nv_fp8x2_storage_t h2 =
        __nv_cvt_float2_to_fp8x2(make_float2(v[2 * u] * dn, v[2 * u + 1] * dn), __NV_SATFINITE, __NV_E4M3);
    const float2 back = __half22float2(__half2(__nv_cvt_fp8x2_to_halfraw2(h2, __NV_E4M3)));
    hw[u] = h2;
    rem[2 * u] = v[2 * u] - back.x * up;
    rem[2 * u + 1] = v[2 * u + 1] - back.y * up;
    rmax = fmaxf(rmax, fmaxf(fabsf(rem[2 * u]), fabsf(rem[2 * u + 1])));
  }
  rmax = fmaxf(rmax, __shfl_xor_sync(0xffffffffu, rmax, 1));
  rmax = fmaxf(rmax, __shfl_xor_sync(0xffffffffu, rmax, 2));
  t.el = e8m0_for(rmax);
  const float dl = pow2_int(-t.el);
#pragma unroll
  for (int u = 0; u < 4; ++u)
    lw[u] = __nv_cvt_float2_to_fp8x2(make_float2(rem[2 * u] * dl, rem[2 * u + 1] * dl), __NV_SATFINITE, __NV_E4M3);
  t.hi = make_uint2(hw[0] | hw[1] << 16, hw[2] | hw[3] << 16);
  t.lo = make_uint2(lw[0] | lw[1] << 16, lw[2] | lw[3] << 16);
  return t;
}

}  // namespace q35
