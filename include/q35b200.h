/*
 * q35b200 -- C ABI of the B200 (sm_100a) implementation of the Qwen3.5 decoder hot path:
 * MoE block, paged flash attention, gated delta net.
 *
 * The boundary mirrors how the reference's host drives one of its kernels: a kernel ("role") has a table of
 * named inputs and outputs, the caller owns every buffer, fills the table in any order and issues one
 * synchronous-looking run call that returns an int status
 *   (reference: tools/board/axrun.cc:55-110 -- GetIOInfo gives names and sizes, the caller fills
 *    AX_ENGINE_IO_BUFFER_T[] and calls AX_ENGINE_RunSync; tools/board/iojson.c dumps the IO table;
 *    tools/manifest/mkmanifest.py:1-15 -- manifest entries are [name, bytes, dtype, shape]).
 * Here the buffers are device pointers and the call is enqueued on a CUDA stream.
 *
 * Nothing in this interface allocates device memory (reference contract: "No allocation, conversion, padding,
 * copy, or output slicing occurs here", models/qwen35_35b_a3b/sgl/python/sgl_kernel_axera/attention/flash_attn.py:
 * 2573-2587).  Kernels that need scratch take it as a named input `workspace`; q35_workspace_bytes() tells its size.
 * Outputs may alias inputs where the reference keeps state in place (state_out == state_in, KV cache rows).
 */
#ifndef Q35B200_H
#define Q35B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element type codes: the AX engine codes the reference's IO tables use (tools/manifest/onnx_io.py:21-32) */
enum q35_dtype {
  Q35_U8 = 1,    /* raw bytes: FP4 pairs (low nibble = even k), E8M0 scales */
  Q35_F32 = 3,
  Q35_I32 = 6,
  Q35_BF16 = 9,
  Q35_F16 = 10,
  Q35_E4M3 = 11,
  Q35_FP4 = 15   /* logical FP4 shape [.., K]: bytes = elements / 2 (same bytes as the U8 [.., K/2] view) */
};

#define Q35_MAX_DIMS 6

/* one bound tensor: what AX_ENGINE_IO_BUFFER_T + the IO-info entry carry (tools/board/axrun.cc:61-75) */
typedef struct q35_io {
  const char* name;
  void* ptr;       /* device pointer */
  size_t bytes;    /* storage bytes; must equal the product of shape times the element size */
  int dtype;       /* enum q35_dtype */
  int ndim;
  int64_t shape[Q35_MAX_DIMS];
} q35_io;

/* status codes (0 = ok); q35_last_error() gives the text */
enum q35_status {
  Q35_OK = 0,
  Q35_ERR_ROLE = 1,      /* unknown role */
  Q35_ERR_MISSING = 2,   /* a required tensor is not bound */
  Q35_ERR_DTYPE = 3,
  Q35_ERR_SHAPE = 4,
  Q35_ERR_BYTES = 5,
  Q35_ERR_WORKSPACE = 6, /* workspace missing or too small */
  Q35_ERR_CUDA = 7,      /* a CUDA runtime call failed */
  Q35_ERR_UNSUPPORTED = 8,
  Q35_ERR_ALIGN = 9      /* a pointer is not aligned as the kernel needs (16 bytes) */
};

/* Run one kernel role with tensors bound by name on `stream` (a cudaStream_t; NULL = default stream).
 * Replaces AX_ENGINE_RunSync(handle, &io) (tools/board/axrun.cc:104-110) and the Python launch
 * kernel[cores](*[case[n] for n in order(fn)]) (models/qwen35_2b/whole/src/q35_layer_mc.py:915-916).
 * Validates names, dtypes, byte counts and shapes before anything is enqueued; returns a q35_status. */
int q35_run(const char* role, const q35_io* ios, int n_io, void* stream);

/* Scratch bytes the role needs for these shapes (0 if none); negative q35_status on a contract error.
 * Only shapes are read, pointers may be NULL. */
int64_t q35_workspace_bytes(const char* role, const q35_io* ios, int n_io);

/* The role's IO table as JSON {"in":[[name,dtype,"shape"],...],"out":[...]} with symbolic shapes: the analogue
 * of tools/board/iojson.c.  Returns the length needed (excluding NUL); writes at most cap bytes. */
int q35_io_table(const char* role, char* buf, size_t cap);

int q35_role_count(void);
const char* q35_role_name(int index);

/* Text of the calling thread's last error ("" if none). */
const char* q35_last_error(void);

/* Device-side status word (one per GPU): kernels record (and skip) out-of-range page ids, expert ids and waits that
 * ran out instead of faulting or hanging.  Reads and clears the current device's word (synchronises the stream);
 * 0 = clean, negative = the CUDA runtime refused.  Bits:
 *   0x001 page id / page table entry out of range      0x002 expert id out of range
 *   0x004 a bounded device-side wait gave up           0x008 token / row index out of range
 * and, with 0x004, which wait of the tensor-core GEMM it was:
 *   0x010 loader waiting for a free ring stage         0x020 MMA issuer waiting for a free accumulator
 *   0x040 MMA issuer waiting for a stage's data        0x080 scale path waiting for a free scale slot
 *   0x100 epilogue waiting for a finished accumulator  0x200 MMA issuer waiting for a stage's scales
 *   0x400 a work item waiting for the rows another item produces
 *   0x800 ep.wait: another rank's rows did not arrive   0x1000 ep.reduce: another rank's partial sums did not
 *   0x2000 ar.oneshot: another rank's addend did not arrive
 *   0x4000 ep.* / ar.oneshot: entry `rank` of `peers` is not `exchange` (the call did nothing)
 * The role "debug.wait_probe" makes one such wait run out on purpose (a barrier nobody arrives at, a poll limit the
 * caller gives) so that a host can check this reporting path; it touches nothing else. */
int q35_device_status(void* stream);

int q35_version(void);

/* Kernels this library has launched in this process so far (all threads, all devices; launches recorded into a CUDA
 * graph count once, at capture).  A diagnostic with no counterpart in the reference: a host can difference it around
 * a step to see how many kernels the step costs. */
long long q35_launch_count(void);

/* Paged attention decode without any caller-provided scratch.  No counterpart in the reference: it exists for hosts
 * that cannot allocate device memory when they call in (runtimes whose buffers are planned up front and frozen, callers
 * living inside another component's memory pool).  Same computation and argument meaning as the role
 * "attn.paged_decode" (q [B, HQ, D] bf16; paged_kv_cache [num_pages, 2, P, HKV, D] of cache_dtype Q35_BF16 or Q35_E4M3;
 * indptr [B + 1], indices [n_indices], last_page_len [B]; sm_scale / kv_scale device pointers or NULL; out [B, HQ, D]
 * bf16), but the split-KV scratch is a 16 MiB array built into the library (held on every GPU that loads it).
 * Shapes that need more return Q35_ERR_WORKSPACE.  Calls nothing that allocates.  The first call on a device resolves
 * the array's device address and should happen outside stream capture.  All calls on a GPU share the array: calls that
 * overlap on the GPU race, so keep them on one stream or otherwise ordered. */
int q35_attn_paged_decode_static(const void* q, const void* paged_kv_cache, int cache_dtype, const int* indptr,
                                 const int* indices, const int* last_page_len, const float* sm_scale,
                                 const float* kv_scale, void* out, int B, int HQ, int HKV, int D, int P, int num_pages,
                                 int n_indices, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* Q35B200_H */
