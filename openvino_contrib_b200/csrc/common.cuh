// Shared device helpers of the attention kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "b2a.h"

namespace b2a {

template <typename T>
__device__ __forceinline__ float to_f32(T x);
template <>
__device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T>
__device__ __forceinline__ T from_f32(float x);
template <>
__device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ void report(int32_t* status, uint32_t bits) {
    if (status != nullptr) atomicOr(reinterpret_cast<unsigned int*>(status), bits);
}

// The four int32 tables of a paged step plus the pool geometry.
struct PagedTables {
    const int32_t* past_lens;
    const int32_t* subsequence_begins;
    const int32_t* block_indices;
    const int32_t* block_indices_begins;
    int32_t num_seqs, num_tokens, num_blocks_total, block_size;
};

// Layout of one u8 chunk [block_size*D values | block_size f16 scales | block_size f16 zero-points].
__host__ __device__ __forceinline__ size_t u8_chunk_bytes(int block_size, int d) {
    return static_cast<size_t>(block_size) * (d + 4);
}

constexpr float kLog2e = 1.4426950408889634f;

// Programmatic dependent launch: a kernel launched with launch_overlapped may be scheduled while the kernel before
// it on the stream is still running (as soon as that one has executed grid_launch_dependents in every CTA, or has
// finished), so that its launch latency and set-up hide behind the predecessor's tail.  It must call
// grid_dependency_wait before it reads or writes anything an earlier kernel on the stream touches: the wait
// returns when the predecessor grid has completed and its memory operations are visible.  EVERY kernel launched
// this way calls the wait (a kernel that skipped it could finish before its predecessor and let ITS successor
// overtake that one).  Both calls are no-ops in a kernel launched the ordinary way.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KernelArgs, typename... Args>
inline cudaError_t launch_overlapped(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                     Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KernelArgs(args)...);
}

}  // namespace b2a
