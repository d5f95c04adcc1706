// C ABI of the library: role registry, by-name binding, validation (see include/q35b200.h).
#include "abi.h"
#include <atomic>
#include <mutex>
#include <string>
#include <unordered_map>

namespace q35 {

static thread_local std::string g_err;

int fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  g_err = buf;
  return code;
}

int elem_bits(int dtype) {
  switch (dtype) {
    case Q35_U8: case Q35_E4M3: return 8;
    case Q35_F32: case Q35_I32: return 32;
    case Q35_BF16: case Q35_F16: return 16;
    case Q35_FP4: return 4;
    default: return 0;
  }
}

int Call::get(const char* name, unsigned dtype_mask, Tensor* out, bool required) const {
  *out = Tensor();
  for (int i = 0; i < n; ++i) {
    const q35_io& io = ios[i];
    if (!io.name || strcmp(io.name, name) != 0) continue;
    int bits = elem_bits(io.dtype);
    Q35_REQUIRE(bits != 0, Q35_ERR_DTYPE, "%s: unknown dtype code %d", name, io.dtype);
    Q35_REQUIRE((dtype_mask >> io.dtype) & 1u, Q35_ERR_DTYPE, "%s: dtype code %d not accepted here (mask 0x%x)", name,
                io.dtype, dtype_mask);
    Q35_REQUIRE(io.ndim >= 0 && io.ndim <= Q35_MAX_DIMS, Q35_ERR_SHAPE, "%s: ndim %d", name, io.ndim);
    out->nd = io.ndim;
    int64_t numel = 1;
    for (int d = 0; d < io.ndim; ++d) {
      Q35_REQUIRE(io.shape[d] >= 0, Q35_ERR_SHAPE, "%s: negative dim", name);
      out->s[d] = io.shape[d];
      numel *= io.shape[d];
    }
    Q35_REQUIRE((numel * bits) % 8 == 0 && size_t(numel * bits / 8) == io.bytes, Q35_ERR_BYTES,
                "%s: %zu bytes bound, shape needs %lld", name, io.bytes, (long long)(numel * bits / 8));
    out->dtype = io.dtype;
    if (io.dtype == Q35_FP4) {  // logical FP4 [.., K] -> byte view [.., K/2]
      Q35_REQUIRE(io.ndim >= 1 && io.shape[io.ndim - 1] % 2 == 0, Q35_ERR_SHAPE, "%s: odd FP4 inner dim", name);
      out->s[io.ndim - 1] /= 2;
      out->dtype = Q35_U8;
    }
    out->p = io.ptr;
    out->bytes = io.bytes;
    out->present = true;
    Q35_REQUIRE(dry || io.ptr != nullptr || io.bytes == 0, Q35_ERR_MISSING, "%s: null pointer", name);
    return 0;
  }
  Q35_REQUIRE(!required, Q35_ERR_MISSING, "tensor '%s' is not bound", name);
  return 0;
}

int Call::workspace(int64_t need, Tensor* ws) {
  ws_need = need;
  *ws = Tensor();
  if (dry) return 0;
  Q35_TRY(get("workspace", M(Q35_U8), ws, need > 0));
  Q35_REQUIRE(need == 0 || int64_t(ws->bytes) >= need, Q35_ERR_WORKSPACE, "workspace: %zu bytes bound, %lld needed",
              ws->bytes, (long long)need);
  Q35_REQUIRE(need == 0 || (reinterpret_cast<uintptr_t>(ws->p) & 255) == 0, Q35_ERR_ALIGN,
              "workspace must be 256-byte aligned");
  return 0;
}

void clear_error() { g_err.clear(); }

static std::atomic<long long> g_launches{0};
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

__device__ int g_device_status;

namespace {
constexpr int kMaxDevices = 64;
struct DeviceSlot {
  bool ready = false;
  DeviceInfo info{nullptr, 0};
  std::unordered_map<const void*, int> smem_limit;  // kernel -> dynamic shared memory limit already set
};
std::mutex g_dev_mutex;
DeviceSlot g_dev[kMaxDevices];

// the slot of the current device, filled on first use; call with g_dev_mutex held
DeviceSlot* current_slot() {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    fail(Q35_ERR_CUDA, "cudaGetDevice: %s (device %d)", cudaGetErrorString(e), dev);
    return nullptr;
  }
  DeviceSlot& s = g_dev[dev];
  if (!s.ready) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_device_status);  // in host code the symbol is only a handle: ask for its address
    if (e != cudaSuccess || !p) {
      fail(Q35_ERR_CUDA, "cudaGetSymbolAddress(status word) on device %d: %s", dev, cudaGetErrorString(e));
      return nullptr;
    }
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    s.info.status = static_cast<int*>(p);
    s.info.sm_count = n;
    s.ready = true;
  }
  return &s;
}
}  // namespace

const DeviceInfo* device_info() {
  std::lock_guard<std::mutex> lock(g_dev_mutex);
  DeviceSlot* s = current_slot();
  return s ? &s->info : nullptr;
}

int* device_status_ptr() {
  const DeviceInfo* d = device_info();
  return d ? d->status : nullptr;
}

int sm_count() {  // also used by shape-only queries that may run without a usable device: falls back silently
  const std::string keep = g_err;
  const DeviceInfo* d = device_info();
  if (!d) g_err = keep;
  return d ? d->sm_count : 148;
}

int ensure_dynamic_smem(const void* func, int bytes) {
  if (bytes <= 48 * 1024) return 0;  // within the default limit
  std::lock_guard<std::mutex> lock(g_dev_mutex);
  DeviceSlot* s = current_slot();
  if (!s) return Q35_ERR_CUDA;
  int& have = s->smem_limit[func];
  if (bytes > have) {
    const cudaError_t e = cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    Q35_REQUIRE(e == cudaSuccess, Q35_ERR_CUDA, "cudaFuncSetAttribute(%d bytes of dynamic shared memory): %s", bytes,
                cudaGetErrorString(e));
    have = bytes;
  }
  return 0;
}

static const RoleDef kRoles[] = {
    {"moe.route",
     R"({"in":[["logits","f32","[T,NE]"]],"out":[["ids","i32","[T,K]"],["rw","f32","[T,K]"]]})", run_moe_route},
    {"moe.pre",
     R"({"in":[["x1","bf16","[T,H]"],["ln2","f32","[H]"],["w_gate","u8|e4m3","[FS,H/2]|[FS,H]"],["s_gate","u8","[FS,H/32]"],["w_up","u8|e4m3","[FS,H/2]|[FS,H]"],["s_up","u8","[FS,H/32]"],["w_down","u8|e4m3","[H,FS/2]|[H,FS]"],["s_down","u8","[H,FS/32]"],["w_router","bf16","[NE,H]"],["w_shg","bf16","[H]"],["workspace","u8","[*]"]],"out":[["out","bf16","[T,H]"],["h2_out","bf16","[T,H]"],["logits_out","f32","[T,NE]"]]})",
     run_moe_pre},
    {"moe.norm_router",
     R"({"in":[["x1","bf16","[T,H]"],["ln2","f32","[H]"],["w_router","bf16","[NE,H]"],["w_shg","bf16","[H]"]],"out":[["h2_out","bf16","[T,H]"],["logits_out","f32","[T,NE]"],["gate_out","f32","[T]"]]})",
     run_moe_norm_router},
    {"moe.shared",
     R"({"in":[["x1","bf16","[T,H]"],["h2","bf16","[T,H]"],["gate","f32","[T]"],["w_gate","u8|e4m3","[FS,H/2]|[FS,H]"],["s_gate","u8","[FS,H/32]"],["w_up","u8|e4m3","[FS,H/2]|[FS,H]"],["s_up","u8","[FS,H/32]"],["w_down","u8|e4m3","[H,FS/2]|[H,FS]"],["s_down","u8","[H,FS/32]"],["workspace","u8","[*]"]],"out":[["out","bf16","[T,H]"]]})",
     run_moe_shared},
    {"moe.finish",
     R"({"in":[["base","bf16","[T,H]"],["partial","f32","[T,H]"]],"out":[["out","bf16","[T,H]"]]})",
     run_moe_finish},
    {"moe.experts",
     R"({"in":[["h2","bf16","[T,H]"],["base","bf16","[T,H]"],["ids","i32","[T,K]"],["rw","f32","[T,K]"],["e_gw","u8","[NE,2FE,H/2]"],["e_gs","u8","[NE,2FE,H/32]"],["e_dw","u8","[NE,H,FE/2]"],["e_ds","u8","[NE,H,FE/32]"],["expert_base","i32","[1] optional: ids are global and the planes start at this id"],["e_gs_tiled","u8","optional with e_ds_tiled: mx.tile_scales.paired / .plain of the scales; decode-sized batches then run as one persistent kernel"],["e_ds_tiled","u8","optional"],["workspace","u8","[*]"]],"out":[["out","bf16","[T,H]"],["partial_out","f32","[T,H] instead of base/out: sums of the pairs with ids >= 0"]]})",
     run_moe_experts},
    {"moe.permute",
     R"({"in":[["ids","i32","[T,K]"],["rw","f32","[T,K]"],["workspace","u8","[*]"]],"out":[["tok","i32","[S,1+G]"],["srw","f32","[S,G]"],["loc","i32","[K,T]"],["n_slots","i32","[1]"],["counts","i32","[NE]"]]})",
     run_moe_permute},
    {"moe.slots",
     R"({"in":[["h2","bf16","[T,H]"],["tok","i32","[S,1+G]"],["rw","f32","[S,G]"],["e_gw","u8","[NE,2FE,H/2]"],["e_gs","u8","[NE,2FE,H/32]"],["e_dw","u8","[NE,H,FE/2]"],["e_ds","u8","[NE,H,FE/32]"],["n_slots","i32","[1] optional"],["workspace","u8","[*]"]],"out":[["out","bf16|f32","[S,G,H]"]]})",
     run_moe_slots},
    {"moe.combine",
     R"({"in":[["base","bf16","[T,H]"],["loc","i32","[K,T]"],["sout","bf16|f32","[R,H]"]],"out":[["out","bf16","[T,H]"]]})",
     run_moe_combine},
    {"attn.paged_decode",
     R"({"in":[["q","bf16","[B,HQ,D]"],["paged_kv_cache","bf16|e4m3","[pages,2,P,HKV,D]"],["indptr","i32","[B+1]"],["indices","i32","[N]"],["last_page_len","i32","[B]"],["sm_scale","f32","[1] optional"],["kv_scale","f32","[2,HKV] optional"],["paged_kv_scale","bf16","[pages,2,P,HKV] optional: int8 cache bound as bytes, one scale per row and head"],["k_new","bf16","[B,HKV,D] optional"],["v_new","bf16","[B,HKV,D] optional"],["workspace","u8","[*]"]],"out":[["out","bf16","[B,HQ,D]"],["part_m","f32","[B,HQ] optional with part_l, part_o instead of out: the unnormalised result for attn.lse_merge"],["part_l","f32","[B,HQ]"],["part_o","f32","[B,HQ,D]"],["part_packed","f32","[B,HQ,D+2] optional instead of the three: o, m, l of a row side by side, one message per rank"]]})",
     run_attn_paged_decode},
    {"attn.lse_merge",
     R"({"in":[["part_m","f32","[G,B,HQ] optional"],["part_l","f32","[G,B,HQ] optional"],["part_o","f32","[G,B,HQ,D] optional"],["packed","f32","[R,B,Hq,D+2] optional instead of the three: the all-gathered part_packed blocks of R ranks, KV group major"]],"out":[["out","bf16","[B,HQ,D]"]]})",
     run_attn_lse_merge},
    {"attn.kv_write",
     R"({"in":[["k_new","bf16","[B,HKV,D]"],["v_new","bf16","[B,HKV,D]"],["cache_location","i32","[B,2]"],["kv_scale","f32","[2,HKV] optional"]],"out":[["paged_kv_cache","bf16|e4m3","[pages,2,P,HKV,D]"],["paged_kv_scale","bf16","[pages,2,P,HKV] optional: int8 cache bound as bytes, the rows' scales land here"]]})",
     run_attn_kv_write},
    {"attn.paged_prefill",
     R"({"in":[["q","bf16","[T,HQ,D]"],["paged_kv_cache","bf16|e4m3","[pages,2,P,HKV,D]"],["qo_indptr","i32","[B+1]"],["indptr","i32","[B+1]"],["indices","i32","[N]"],["last_page_len","i32","[B]"],["sm_scale","f32","[1] optional"],["kv_scale","f32","[2,HKV] optional: FP8 cache with per-head scales; absent: the stored x 8 form"],["paged_kv_scale","bf16","[pages,2,P,HKV] optional: int8 cache bound as bytes, one scale per row and head; new rows' scales are written"],["k_new","bf16","[T,HKV,D] optional: written into the cache first"],["v_new","bf16","[T,HKV,D] optional"]],"out":[["out","bf16","[T,HQ,D]"]]})",
     run_attn_paged_prefill},
    {"gdn.step",
     R"({"in":[["q","bf16","[B,NK,DK]"],["k","bf16","[B,NK,DK]"],["v","bf16","[B,NV,DV]"],["g","f32","[B,NV]"],["beta","bf16","[B,NV]"],["state_in","f32","[B,NV,DK,DV]"]],"out":[["o","bf16","[B,NV,DV]"],["state_out","f32","[B,NV,DK,DV]"]]})",
     run_gdn_step},
    {"gdn.conv",
     R"({"in":[["x","bf16","[B,T,C]"],["conv_w","bf16","[C,KW]"],["conv_in","bf16","[B,KW-1,C]"]],"out":[["y","bf16","[B,T,C]"],["conv_out","bf16","[B,KW-1,C]"]]})",
     run_gdn_conv},
    {"gdn.chunk_prefill",
     R"({"in":[["q","bf16","[B,T,NK,128]"],["k","bf16","[B,T,NK,128]"],["v","bf16","[B,T,NV,128]"],["g","f32","[B,T,NV]"],["beta","bf16","[B,T,NV]"],["state_in","f32","[B,NV,128,128]"],["workspace","u8","[*]"]],"out":[["o","bf16","[B,T,NV,128]"],["state_out","f32","[B,NV,128,128]"]]})",
     run_gdn_chunk_prefill},
    {"linear",
     R"({"in":[["x","bf16","[T,K]"],["w","u8|e4m3|bf16","[N,K/2]|[N,K]"],["s","u8|f32|e4m3","[N,K/32]|[N]|[N,K/16], the last with E4M3 scales per 16 inputs: NVFP4"],["s2","f32","[1] optional: tensor scale of an NVFP4 weight"],["bias","f32","[N] optional"],["row_div","f32","[T] optional"],["residual","bf16","[T,N] optional"],["workspace","u8","[*] optional: with it (and K a multiple of 512) the tensor-core path runs"]],"out":[["out","bf16|f32","[T,N]"]]})",
     run_linear},
    {"linear.multi",
     R"({"in":[["x","bf16","[T,K]"],["w","u8|e4m3","[N,K/2]|[N,K]: the projections' weights, rows concatenated"],["s","u8|f32","[N,K/32]|[N]"],["bias","f32","[N] optional"],["row_div","f32","[T] optional"],["workspace","u8","[*]"]],"out":[["out0","bf16|f32","[T,N_0]"],["out1","bf16|f32","[T,N_1] optional, and so on up to out7; the N_i add up to N"],["out2","bf16|f32","optional"],["out3","bf16|f32","optional"],["out4","bf16|f32","optional"],["out5","bf16|f32","optional"],["out6","bf16|f32","optional"],["out7","bf16|f32","optional"]]})",
     run_linear_multi},
    {"moe.front",
     R"({"in":[["x1","bf16","[T,H]"],["ln2","f32","[H]"],["w_router","bf16","[NE,H]"],["w_shg","bf16","[H] optional: shared-expert gate vector"],["workspace","u8","[*]"]],"out":[["h2_out","bf16","[T,H]"],["logits_out","f32","[T,NE]"],["gate_out","f32","[T] with w_shg"],["ids","i32","[T,K]"],["rw","f32","[T,K]"]]})",
     run_moe_front},
    {"ep.publish",
     R"({"in":[["h2","bf16","[T,H]"],["ids","i32","[T,K]"],["rw","f32","[T,K]"],["peers","u8","[8 N]: the ranks' exchange buffer addresses as mapped here, peers[rank] = exchange; the kernels read the table"],["rank","i32","[1]: read by the kernels"],["no_wait","i32","[1] optional: return after publishing instead of waiting for every rank's rows; ep.wait does that later"]],"out":[["exchange","u8","[*]: this rank's exchange buffer, 1 KB header first"],["h2_all","bf16","[N,T,H] region of exchange"],["ids_all","i32","[N,T,K] region of exchange"],["rw_all","f32","[N,T,K] region of exchange"]]})",
     run_ep_publish},
    {"ep.wait",
     R"({"in":[["peers","u8","[8 N]"],["rank","i32","[1]"]],"out":[["exchange","u8","[*]: returns when every rank's rows of the current exchange have arrived, or records a wait timeout"]]})",
     run_ep_wait},
    {"ep.reduce",
     R"({"in":[["base","bf16","[T,H]"],["partial","f32","[N T,H] region of exchange: this rank's sums for every rank's tokens"],["peers","u8","[8 N]"],["rank","i32","[1]"],["exchange","u8","[*]"]],"out":[["out","bf16","[T,H]: base + the ranks' partial sums of this rank's tokens, added in rank order"]]})",
     run_ep_reduce},
    {"ar.oneshot",
     R"({"in":[["x","f32","[*]: this rank's addend, a multiple of 4 elements"],["peers","u8","[8 N]"],["rank","i32","[1]"],["exchange","u8","[1024 + 2 N slot]: slot = bytes of x rounded up to 256"]],"out":[["out","f32","like x: the sum over the ranks, added in rank order"]]})",
     run_ar_oneshot},
    {"norm.rms",
     R"({"in":[["x","bf16","[T,H]"],["residual","bf16","[T,H] optional"],["w","f32|bf16","[H]"],["eps","f32","[1] optional"]],"out":[["y","bf16","[T,H]"],["base_out","bf16","[T,H] optional"],["xsqrt_out","f32","[T] optional: folded form"]]})",
     run_norm_rms},
    {"gdn.prep",
     R"({"in":[["q","bf16","[R,NK,DK]"],["k","bf16","[R,NK,DK]"],["a","bf16","[R,NV]"],["b","bf16","[R,NV]"],["a_log","f32","[NV]"],["dt_bias","f32|bf16","[NV]"]],"out":[["q_out","bf16","[R,NK,DK]"],["k_out","bf16","[R,NK,DK]"],["g","f32","[R,NV]"],["beta","bf16","[R,NV]"]]})",
     run_gdn_prep},
    {"gdn.out_norm",
     R"({"in":[["core","bf16","[R,NV,DV]"],["z","bf16","[R,NV,DV]"],["w","f32|bf16","[DV]"],["eps","f32","[1] optional"]],"out":[["y","bf16","[R,NV,DV]"]]})",
     run_gdn_out_norm},
    {"attn.qk_prep",
     R"({"in":[["qg","bf16","[R,HQ,D|2D]"],["k","bf16","[R,HKV,D]"],["q_norm","f32","[D]"],["k_norm","f32","[D]"],["cos","f32","[R,rot/2]"],["sin","f32","[R,rot/2]"],["eps","f32","[1] optional"]],"out":[["q_out","bf16","[R,HQ,D]"],["k_out","bf16","[R,HKV,D]"],["gate_out","bf16","[R,HQ,D] optional"]]})",
     run_attn_qk_prep},
    {"act.silu_mul",
     R"({"in":[["a","bf16","[*]"],["b","bf16","[*]"]],"out":[["y","bf16","[*]"]]})", run_act_silu_mul},
    {"act.sigmoid_gate",
     R"({"in":[["a","bf16","[*]"],["b","bf16","[*]"]],"out":[["y","bf16","[*]"]]})", run_act_sigmoid_gate},
    {"linear.tc",
     R"({"in":[["x","bf16","[T,K]"],["w","u8","[N,K/2]"],["s","u8","[N,K/32]"],["bias","f32","[N] optional"],["workspace","u8","[*]"]],"out":[["out","bf16|f32","[T,N]"]]})",
     run_linear_tc},
    {"lm_head",
     R"({"in":[["x","bf16","[T,K]"],["w","u8","[N,K/2]"],["s","u8","[N,K/32]"],["workspace","u8","[*]"]],"out":[["logits","f32","[T,N] optional; also accepted under the name out"],["token","i32","[T] optional: first index of the row maximum"]]})",
     run_lm_head},
    {"moe.block",
     R"({"in":[["x1","bf16","[T,H]"],["ln2","f32","[H]"],["w_router","bf16","[NE,H]"],["w_shg","bf16","[H] with the shared expert"],["w_gate","u8","[FE,H/2] optional: shared expert, MXFP4"],["w_up","u8","[FE,H/2]"],["w_down","u8","[H,FE/2]"],["s_gate_up_tiled","u8","mx.tile_scales.paired of s_gate rows followed by s_up rows"],["s_down_tiled","u8","mx.tile_scales.plain of s_down"],["e_gw","u8","[NE,2FE,H/2]"],["e_dw","u8","[NE,H,FE/2]"],["e_gs_tiled","u8","mx.tile_scales.paired of e_gs"],["e_ds_tiled","u8","mx.tile_scales.plain of e_ds"],["workspace","u8","[*]"]],"out":[["out","bf16","[T,H]"],["ids","i32","[T,K]"],["rw","f32","[T,K]"],["logits_out","f32","[T,NE] optional"],["h2_out","bf16","[T,H] optional"]]})",
     run_moe_block},
    {"mx.tile_scales.paired",
     R"({"in":[["s","u8","[planes,rows,K/32] E8M0, rows = gate rows then up rows"]],"out":[["out","u8","[planes,rows/128,K/128,512]"]]})",
     run_tile_scales_paired},
    {"mx.tile_scales.plain",
     R"({"in":[["s","u8","[planes,rows,K/32] E8M0"]],"out":[["out","u8","[planes,rows/128,K/128,512]"]]})",
     run_tile_scales_plain},
    {"debug.tc_peak",
     R"({"in":[["iters","i32","[1] MMA groups of K = 128 per CTA"]],"out":[["done","i32","[1]"]]})", run_debug_tc_peak},
    {"debug.wait_probe",
     R"({"in":[["polls","i32","[1] poll limit of the wait, clamped to 1 .. 2^20"]],"out":[["result","i32","[1] 1 = the wait gave up and the status word got its bit"]]})",
     run_debug_wait_probe},
};
static const int kNumRoles = int(sizeof(kRoles) / sizeof(kRoles[0]));

static const RoleDef* find_role(const char* role) {
  if (!role) return nullptr;
  for (int i = 0; i < kNumRoles; ++i)
    if (strcmp(kRoles[i].name, role) == 0) return &kRoles[i];
  return nullptr;
}

}  // namespace q35

using namespace q35;

extern "C" {

int q35_run(const char* role, const q35_io* ios, int n_io, void* stream) {
  g_err.clear();
  const RoleDef* r = find_role(role);
  if (!r) return fail(Q35_ERR_ROLE, "unknown role '%s'", role ? role : "(null)");
  if (n_io < 0 || (n_io > 0 && !ios)) return fail(Q35_ERR_MISSING, "bad io table");
  // the launchers hand kernels the status word's address: resolve this device's state first, so that a failure is
  // a status code here and never a null pointer inside a kernel
  if (!device_info()) return Q35_ERR_CUDA;
  Call c{ios, n_io, static_cast<cudaStream_t>(stream), false, 0};
  return r->run(c);
}

int64_t q35_workspace_bytes(const char* role, const q35_io* ios, int n_io) {
  g_err.clear();
  const RoleDef* r = find_role(role);
  if (!r) return -int64_t(fail(Q35_ERR_ROLE, "unknown role '%s'", role ? role : "(null)"));
  Call c{ios, n_io, nullptr, true, 0};
  int st = r->run(c);
  if (st) return -int64_t(st);
  return c.ws_need;
}

int q35_io_table(const char* role, char* buf, size_t cap) {
  const RoleDef* r = find_role(role);
  if (!r) return -fail(Q35_ERR_ROLE, "unknown role '%s'", role ? role : "(null)");
  size_t len = strlen(r->io_json);
  if (buf && cap) {
    size_t ncopy = len < cap - 1 ? len : cap - 1;
    memcpy(buf, r->io_json, ncopy);
    buf[ncopy] = 0;
  }
  return int(len);
}

int q35_role_count(void) { return kNumRoles; }
const char* q35_role_name(int i) { return (i >= 0 && i < kNumRoles) ? kRoles[i].name : nullptr; }
const char* q35_last_error(void) { return g_err.c_str(); }

int q35_device_status(void* stream) {
  int* p = device_status_ptr();
  int v = 0, zero = 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (!p) return -1;
  if (cudaMemcpyAsync(&v, p, sizeof v, cudaMemcpyDeviceToHost, s) != cudaSuccess) return -1;
  if (cudaMemcpyAsync(p, &zero, sizeof zero, cudaMemcpyHostToDevice, s) != cudaSuccess) return -1;
  if (cudaStreamSynchronize(s) != cudaSuccess) return -1;
  return v;
}

int q35_version(void) { return 2; }

long long q35_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

}  // extern "C"
