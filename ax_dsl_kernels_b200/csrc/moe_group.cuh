// Entry points shared between the MoE translation units.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace q35 {
int launch_group_count(const int* ids, const int* base, int T, int K, int NE, int* counts, int* list,
                       cudaStream_t stream);
int launch_combine(const __nv_bfloat16* base, const int* loc, const void* sout, bool sout_f32, __nv_bfloat16* out,
                   int T, int H, int K, int R, cudaStream_t stream);
int launch_partial_sum(const int* loc, const void* sout, bool sout_f32, float* partial, int T, int H, int K, int R,
                       cudaStream_t stream);
}  // namespace q35
