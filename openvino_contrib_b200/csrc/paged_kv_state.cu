// Kernels of the stateful-model bridge (host/kv_pool_state.hpp): between the dense [B, Hkv, T, D] tensors in which a
// ReadValue / Assign model sees its KV cache and the paged pool.
//
//   bhsd_to_rows   positions t0 .. t0+q-1 of a [B, Hkv, T, D] tensor -> [B*q, Hkv*D]: the new rows of a step in the
//                  token-major layout the KV store takes (row b*q + i = token i of sequence b); a plain transposing
//                  copy of 2- or 4-byte elements.
//   kv_export      pool -> [B, Hkv, T, D] in f32 / f16 / bf16: the first T positions of every sequence, read through
//                  the block table and, for a u8 pool, de-quantised as (code - zp) * scale in float32 - the values the
//                  attention kernels compute with.
// Both are slow-path helpers (state import / export, the Concat + Assign of a multi-token step); neither is on the
// path of a decode step, whose [B, Hkv, 1, D] rows are token-major already.
#include "launch.cuh"

namespace b2a {
namespace {

template <typename E>
__global__ void __launch_bounds__(256) bhsd_to_rows_kernel(const E* __restrict__ src, E* __restrict__ dst, int B, int H,
                                                          int q, int D, int src_T, int t0) {
    grid_dependency_wait();
    grid_launch_dependents();
    const long long total = static_cast<long long>(B) * H * q * D;
    for (long long i = blockIdx.x * 256LL + threadIdx.x; i < total; i += 256LL * gridDim.x) {
        const int d = static_cast<int>(i % D);
        const int h = static_cast<int>((i / D) % H);
        const int t = static_cast<int>((i / (static_cast<long long>(D) * H)) % q);
        const int b = static_cast<int>(i / (static_cast<long long>(D) * H * q));
        dst[i] = src[((static_cast<long long>(b) * H + h) * src_T + t0 + t) * D + d];  // dst index i is [b][t][h][d]
    }
}

template <typename TOut>
__global__ void __launch_bounds__(256) kv_export_kernel(const uint8_t* __restrict__ cache, const int32_t* block_indices,
                                                        const int32_t* block_indices_begins, int num_blocks_total,
                                                        int B, int H, int T, int D, int bs, int kv_dtype,
                                                        TOut* __restrict__ out, int32_t* status) {
    grid_dependency_wait();
    grid_launch_dependents();
    const long long total = static_cast<long long>(B) * H * T * D;
    const size_t chunk = kv_dtype == B2A_U8 ? u8_chunk_bytes(bs, D) : static_cast<size_t>(bs) * D * 2;
    for (long long i = blockIdx.x * 256LL + threadIdx.x; i < total; i += 256LL * gridDim.x) {
        const int d = static_cast<int>(i % D);
        const int t = static_cast<int>((i / D) % T);
        const int h = static_cast<int>((i / (static_cast<long long>(D) * T)) % H);
        const int b = static_cast<int>(i / (static_cast<long long>(D) * T * H));
        const int lb = t / bs, slot = t % bs;
        float x = 0.f;
        const int b0 = block_indices_begins[b], b1 = block_indices_begins[b + 1];
        const int phys = lb < b1 - b0 ? block_indices[b0 + lb] : -1;
        if (phys < 0 || phys >= num_blocks_total) {
            if (d == 0) report(status, lb < b1 - b0 ? B2A_DEV_BAD_BLOCK : B2A_DEV_BAD_LEN);
        } else {
            const uint8_t* c = cache + (static_cast<size_t>(phys) * H + h) * chunk;
            if (kv_dtype == B2A_U8) {
                const __half* meta = reinterpret_cast<const __half*>(c + static_cast<size_t>(bs) * D);
                const float sc = __half2float(meta[slot]), zp = __half2float(meta[bs + slot]);
                x = __fmul_rn(__fsub_rn(static_cast<float>(c[slot * D + d]), zp), sc);
            } else if (kv_dtype == B2A_F16) {
                x = __half2float(reinterpret_cast<const __half*>(c)[slot * D + d]);
            } else {
                x = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(c)[slot * D + d]);
            }
        }
        out[i] = from_f32<TOut>(x);
    }
}

unsigned grid_for(long long total) {
    const long long blocks = (total + 255) / 256;
    return static_cast<unsigned>(blocks < 1 ? 1 : (blocks > 148 * 16 ? 148 * 16 : blocks));
}

}  // namespace

int kv_rows_from_bhsd_launch(int dtype, const void* src, void* dst, int B, int H, int q, int D, int src_T, int t0,
                             cudaStream_t stream) {
    const long long total = static_cast<long long>(B) * H * q * D;
    if (total == 0) return B2A_OK;
    cudaError_t e;
    if (dtype == B2A_F32)
        e = launch_overlapped(bhsd_to_rows_kernel<uint32_t>, dim3(grid_for(total)), dim3(256), 0, stream,
                              static_cast<const uint32_t*>(src), static_cast<uint32_t*>(dst), B, H, q, D, src_T, t0);
    else if (dtype == B2A_F16 || dtype == B2A_BF16)
        e = launch_overlapped(bhsd_to_rows_kernel<uint16_t>, dim3(grid_for(total)), dim3(256), 0, stream,
                              static_cast<const uint16_t*>(src), static_cast<uint16_t*>(dst), B, H, q, D, src_T, t0);
    else
        return B2A_ERR_DTYPE;
    return e == cudaSuccess ? B2A_OK : B2A_ERR_CUDA;
}

int kv_export_launch(int kv_dtype, int out_dtype, const void* cache, const int32_t* block_indices,
                     const int32_t* block_indices_begins, int num_blocks_total, int B, int H, int T, int D, int bs,
                     void* out, int32_t* status, cudaStream_t stream) {
    const long long total = static_cast<long long>(B) * H * T * D;
    if (total == 0) return B2A_OK;
    const dim3 grid(grid_for(total)), block(256);
    const uint8_t* c = static_cast<const uint8_t*>(cache);
    cudaError_t e;
    switch (out_dtype) {
        case B2A_F32:
            e = launch_overlapped(kv_export_kernel<float>, grid, block, 0, stream, c, block_indices, block_indices_begins,
                                  num_blocks_total, B, H, T, D, bs, kv_dtype, static_cast<float*>(out), status);
            break;
        case B2A_F16:
            e = launch_overlapped(kv_export_kernel<__half>, grid, block, 0, stream, c, block_indices, block_indices_begins,
                                  num_blocks_total, B, H, T, D, bs, kv_dtype, static_cast<__half*>(out), status);
            break;
        case B2A_BF16:
            e = launch_overlapped(kv_export_kernel<__nv_bfloat16>, grid, block, 0, stream, c, block_indices,
                                  block_indices_begins, num_blocks_total, B, H, T, D, bs, kv_dtype,
                                  static_cast<__nv_bfloat16*>(out), status);
            break;
        default: return B2A_ERR_DTYPE;
    }
    return e == cudaSuccess ? B2A_OK : B2A_ERR_CUDA;
}

}  // namespace b2a
