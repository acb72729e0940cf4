// Append this step's K/V rows to the block pools through the block table.
//
// One warp per (token, KV head, K-or-V): it finds the token's sequence by bisection of subsequence_begins, its
// cache position past_lens[s] + offset, the physical block from the block table, and writes the row.  For a u8
// cache the row is quantised per token, asymmetrically, with the scale and zero-point rounded to f16 BEFORE the
// values are quantised, every step a single round-to-nearest-even binary32 operation:
//     s  = f16((max - min) / 255)  (1.0 when that is 0 or not finite)
//     zp = f16(-min / s)
//     q  = clamp(rint(x / s + zp), 0, 255)
// so the bytes and the two f16 values are reproducible bit for bit on a CPU.
#include "launch.cuh"

namespace b2a {
namespace {

constexpr int kWarpsPerCta = 8;

struct StoreParams {
    const void* key;
    const void* value;
    uint8_t* k_cache;
    uint8_t* v_cache;
    PagedTables t;
    int Hkv, D, Dv, kv_dtype;
    int32_t* status;
};

template <typename T>
__global__ void __launch_bounds__(kWarpsPerCta * 32) paged_kv_store_kernel(const StoreParams p) {
    const int lane = threadIdx.x & 31;
    const long long item = static_cast<long long>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
    const long long total = 2LL * p.t.num_tokens * p.Hkv;
    if (item >= total) return;
    const int which = static_cast<int>(item % 2);  // 0 = key, 1 = value
    const int hk = static_cast<int>((item / 2) % p.Hkv);
    const int tok = static_cast<int>(item / (2LL * p.Hkv));
    const int D = which ? p.Dv : p.D;

    // sequence of this token: last s with subsequence_begins[s] <= tok
    int lo = 0, hi = p.t.num_seqs;  // invariant: begins[lo] <= tok < begins[hi]
    if (tok >= p.t.subsequence_begins[p.t.num_seqs] || tok < p.t.subsequence_begins[0]) return;  // not scheduled
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (p.t.subsequence_begins[mid] <= tok) lo = mid; else hi = mid;
    }
    const int seq = lo;
    const int pos = p.t.past_lens[seq] + (tok - p.t.subsequence_begins[seq]);
    const int bs = p.t.block_size;
    const int nblk_seq = p.t.block_indices_begins[seq + 1] - p.t.block_indices_begins[seq];
    if (pos < 0 || pos / bs >= nblk_seq) {
        if (lane == 0) report(p.status, B2A_DEV_BAD_LEN);
        return;
    }
    const int blk = p.t.block_indices[p.t.block_indices_begins[seq] + pos / bs];
    if (blk < 0 || blk >= p.t.num_blocks_total) {
        if (lane == 0) report(p.status, B2A_DEV_BAD_BLOCK);
        return;
    }
    const int slot = pos % bs;
    const T* src = reinterpret_cast<const T*>(which ? p.value : p.key) + (static_cast<size_t>(tok) * p.Hkv + hk) * D;
    uint8_t* cache = which ? p.v_cache : p.k_cache;

    if (p.kv_dtype != B2A_U8) {
        // plain [block_size, D] chunk of f16 / bf16
        uint16_t* dst = reinterpret_cast<uint16_t*>(cache) +
                        ((static_cast<size_t>(blk) * p.Hkv + hk) * bs + slot) * D;
        for (int d = lane; d < D; d += 32) {
            const float x = to_f32<T>(src[d]);
            dst[d] = p.kv_dtype == B2A_F16 ? __half_as_ushort(__float2half_rn(x))
                                           : __bfloat16_as_ushort(__float2bfloat16_rn(x));
        }
        return;
    }

    uint8_t* chunk = cache + (static_cast<size_t>(blk) * p.Hkv + hk) * u8_chunk_bytes(bs, D);
    uint8_t* row = chunk + slot * D;
    // D == 128 with 16-bit inputs: each lane keeps its 4 consecutive values in registers (one 8-byte load, one
    // 4-byte store); other sizes take the strided loops below.  Same arithmetic either way.
    const bool vec = (D == 128) && sizeof(T) == 2 && ((reinterpret_cast<uintptr_t>(src) & 7) == 0);
    float xv[4];
    float mn = INFINITY, mx = -INFINITY;
    if (vec) {
        const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(src) + 4 * lane);
        const T* h = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            xv[i] = to_f32<T>(h[i]);
            mn = fminf(mn, xv[i]);
            mx = fmaxf(mx, xv[i]);
        }
    } else {
        for (int d = lane; d < D; d += 32) {
            const float x = to_f32<T>(src[d]);
            mn = fminf(mn, x);
            mx = fmaxf(mx, x);
        }
    }
    mx = warp_max(mx);
    mn = -warp_max(-mn);
    __half s16 = __float2half_rn(__fdiv_rn(__fsub_rn(mx, mn), 255.0f));
    float sf = __half2float(s16);
    if (sf == 0.f || isinf(sf) || isnan(sf)) {
        s16 = __float2half_rn(1.0f);
        sf = 1.0f;
    }
    const __half z16 = __float2half_rn(__fdiv_rn(-mn, sf));
    const float zf = __half2float(z16);
    if (vec) {
        uint32_t packed = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float t = rintf(__fadd_rn(__fdiv_rn(xv[i], sf), zf));
            packed |= static_cast<uint32_t>(fminf(fmaxf(t, 0.f), 255.f)) << (8 * i);
        }
        reinterpret_cast<uint32_t*>(row)[lane] = packed;
    } else {
        for (int d = lane; d < D; d += 32) {
            const float x = to_f32<T>(src[d]);
            const float t = rintf(__fadd_rn(__fdiv_rn(x, sf), zf));
            row[d] = static_cast<uint8_t>(fminf(fmaxf(t, 0.f), 255.f));
        }
    }
    if (lane == 0) {
        __half* meta = reinterpret_cast<__half*>(chunk + bs * D);
        meta[slot] = s16;
        meta[bs + slot] = z16;
    }
}

}  // namespace

int paged_kv_store_launch(const b2a_paged_desc& d, const void* key, const void* value, void* k_cache, void* v_cache,
                          const PagedTables& t, int32_t* status, cudaStream_t stream) {
    if (d.num_tokens == 0) return B2A_OK;
    StoreParams p{key, value, static_cast<uint8_t*>(k_cache), static_cast<uint8_t*>(v_cache), t,
                  d.Hkv, d.D, d.Dv, d.kv_dtype, status};
    const long long total = 2LL * d.num_tokens * d.Hkv;
    const unsigned grid = static_cast<unsigned>((total + kWarpsPerCta - 1) / kWarpsPerCta);
    switch (d.q_dtype) {
        case B2A_F32: paged_kv_store_kernel<float><<<grid, kWarpsPerCta * 32, 0, stream>>>(p); break;
        case B2A_F16: paged_kv_store_kernel<__half><<<grid, kWarpsPerCta * 32, 0, stream>>>(p); break;
        case B2A_BF16: paged_kv_store_kernel<__nv_bfloat16><<<grid, kWarpsPerCta * 32, 0, stream>>>(p); break;
        default: return B2A_ERR_DTYPE;
    }
    return cudaGetLastError() == cudaSuccess ? B2A_OK : B2A_ERR_CUDA;
}

}  // namespace b2a
