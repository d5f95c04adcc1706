// Host-side plumbing shared by the kernel launchers: tensors bound by name, contract checks, error text.
#pragma once
#include <utility>
#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include "../../include/q35b200.h"

namespace q35 {

int fail(int code, const char* fmt, ...);

struct Tensor {
  void* p = nullptr;
  size_t bytes = 0;
  int dtype = 0;
  int nd = 0;
  int64_t s[Q35_MAX_DIMS] = {0, 0, 0, 0, 0, 0};
  bool present = false;
  int64_t numel() const {
    int64_t n = 1;
    for (int i = 0; i < nd; ++i) n *= s[i];
    return n;
  }
  template <class T> T* as() const { return reinterpret_cast<T*>(p); }
};

constexpr unsigned M(int dtype) { return 1u << dtype; }
constexpr unsigned M_BYTES = M(Q35_U8) | M(Q35_FP4);   // FP4 pairs / E8M0 scales
constexpr unsigned M_FP8 = M(Q35_E4M3) | M(Q35_U8);

// One q35_run / q35_workspace_bytes invocation.
struct Call {
  const q35_io* ios;
  int n;
  cudaStream_t stream;
  bool dry;            // workspace query: validate shapes, launch nothing
  int64_t ws_need;     // set by the launcher
  // Finds `name`; checks dtype against the mask and bytes against the shape.  FP4 logical tensors are normalised
  // to their byte view (last dim halved).  Returns 0 or a q35_status.
  int get(const char* name, unsigned dtype_mask, Tensor* out, bool required = true) const;
  // Workspace handling: records the need; when running, checks the bound `workspace` tensor is big enough.
  int workspace(int64_t need, Tensor* ws);
};

struct RoleDef {
  const char* name;
  const char* io_json;  // symbolic IO table
  int (*run)(Call&);
};

int elem_bits(int dtype);

// Per-device state.  One process may drive several GPUs (and several host threads may call in at once), so nothing
// about "the" device is cached process-wide: the address of the device status word, the SM count and the "dynamic
// shared memory limit already raised" marks are kept per device ordinal, filled under a lock on first use with that
// device current.
struct DeviceInfo {
  int* status;    // device address of this GPU's status word (see q35_device_status)
  int sm_count;
};
// state of the CURRENT device; nullptr (and the error text set) when the CUDA runtime refuses
const DeviceInfo* device_info();
int* device_status_ptr();   // device_info()->status, nullptr on failure
int sm_count();             // device_info()->sm_count, 148 when it cannot be read
// cudaFuncSetAttribute(func, MaxDynamicSharedMemorySize, bytes) once per (device, function, size); 0 or Q35_ERR_CUDA
int ensure_dynamic_smem(const void* func, int bytes);
void clear_error();

#define Q35_REQUIRE(cond, code, ...) \
  do {                               \
    if (!(cond)) return ::q35::fail(code, __VA_ARGS__); \
  } while (0)
#define Q35_TRY(expr)        \
  do {                       \
    int _st = (expr);        \
    if (_st) return _st;     \
  } while (0)
// every kernel launch of the library is followed by this check, which also counts it (q35_launch_count)
void count_launch();
#define Q35_CUDA_LAUNCH_CHECK(what)                                                        \
  do {                                                                                     \
    ::q35::count_launch();                                                                 \
    cudaError_t _e = cudaGetLastError();                                                   \
    if (_e != cudaSuccess) return ::q35::fail(Q35_ERR_CUDA, "%s: %s", what, cudaGetErrorString(_e)); \
  } while (0)

// Launch with programmatic dependent launch allowed: the kernel's CTAs may become resident while the previous kernel
// of the stream drains, and run up to their `pdl_wait()` (common.cuh) -- which EVERY kernel launched this way executes
// before its first global memory access.  After anything that is not such a kernel the launch serialises as usual.
// An error of the launch is left for Q35_CUDA_LAUNCH_CHECK.
template <typename... KArgs, typename... Args>
inline void launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                       Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  cudaLaunchKernelEx(&cfg, kernel, KArgs(std::forward<Args>(args))...);
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// launchers (one per role), defined next to their kernels
int run_moe_route(Call&);
int run_moe_pre(Call&);
int run_moe_norm_router(Call&);
int run_moe_shared(Call&);
int run_moe_finish(Call&);
int run_moe_experts(Call&);
int run_moe_slots(Call&);
int run_moe_combine(Call&);
int run_moe_permute(Call&);
int run_attn_paged_decode(Call&);
int run_attn_kv_write(Call&);
int run_attn_lse_merge(Call&);
int run_attn_paged_prefill(Call&);
int run_gdn_step(Call&);
int run_gdn_conv(Call&);
int run_gdn_chunk_prefill(Call&);
int run_linear(Call&);
int run_norm_rms(Call&);
int run_gdn_prep(Call&);
int run_gdn_out_norm(Call&);
int run_attn_qk_prep(Call&);
int run_act_silu_mul(Call&);
int run_act_sigmoid_gate(Call&);
int run_linear_tc(Call&);
int run_linear_multi(Call&);
int run_ep_publish(Call&);
int run_ep_wait(Call&);
int run_ep_reduce(Call&);
int run_ar_oneshot(Call&);
int run_moe_front(Call&);
int run_lm_head(Call&);
int run_debug_wait_probe(Call&);
int run_debug_tc_peak(Call&);
int run_moe_block(Call&);
bool moe_experts_tiled_ok(int64_t T, int64_t K, int64_t NE, int64_t H, int64_t FE);
int moe_experts_tiled(Call& c, const Tensor& h2, const Tensor& base, const Tensor& ids, const Tensor& rw, const Tensor& egw,
                      const Tensor& edw, const Tensor& egs_t, const Tensor& eds_t, const Tensor& ebase, const Tensor& out,
                      const Tensor& partial);
int run_tile_scales_paired(Call&);
int run_tile_scales_plain(Call&);

}  // namespace q35
