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
//
// Rotary position embedding can be applied to the key rows on the way (b2a_paged_kv_store_rope): the first
// rotary_dim values of a key row, at cache position p, are rotated in pairs (i, i + rotary_dim/2) -
//     x'[i]         = x[i] * cos[p][i] - x[i + r/2] * sin[p][i]
//     x'[i + r/2]   = x[i + r/2] * cos[p][i] + x[i] * sin[p][i]            (r = rotary_dim, i < r/2)
// each product and the sum single round-to-nearest binary32 operations (no fused multiply-add), and the rotated
// float32 values are what is quantised (or rounded to the cache's 16-bit type).  A model then feeds the un-rotated
// key projection to the store and saves the pass that rotates K in memory; queries are rotated by their producer.
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
    // rotary embedding of the key rows (rotary_dim == 0: none): f32 tables [positions][rotary_dim / 2]
    const float* rope_cos;
    const float* rope_sin;
    int rotary_dim, rope_positions;
};

// x[d] of a key row at cache position `pos`, rotated; `own` is x[d], `partner` is x[d +- rotary_dim/2]
__device__ __forceinline__ float rope_value(const StoreParams& p, int pos, int d, float own, float partner) {
    const int half = p.rotary_dim >> 1;
    const int i = d < half ? d : d - half;
    const float c = p.rope_cos[static_cast<size_t>(pos) * half + i], s = p.rope_sin[static_cast<size_t>(pos) * half + i];
    return d < half ? __fsub_rn(__fmul_rn(own, c), __fmul_rn(partner, s)) : __fadd_rn(__fmul_rn(own, c), __fmul_rn(partner, s));
}

// Sequence of token `tok`: the last s with subsequence_begins[s] <= tok, found by the whole warp - every round the 32
// lanes probe 32 evenly spaced entries of the remaining range and a ballot picks the segment, so 65535 sequences take
// four dependent loads instead of sixteen.  Returns -1 for a token outside the scheduled range.
__device__ __forceinline__ int find_sequence(const PagedTables& t, int tok, int lane) {
    if (tok >= t.subsequence_begins[t.num_seqs] || tok < t.subsequence_begins[0]) return -1;
    int lo = 0, hi = t.num_seqs;  // invariant: begins[lo] <= tok < begins[hi]
    while (hi - lo > 1) {
        const int step = (hi - lo + 31) / 32;
        const int probe = lo + lane * step;  // lane 0 probes lo itself
        const bool le = probe < hi && t.subsequence_begins[probe] <= tok;
        const unsigned m = __ballot_sync(0xffffffffu, le);  // a prefix of the lanes (begins are non-decreasing)
        const int last = 31 - __clz(static_cast<int>(m));
        const int nlo = lo + last * step;
        hi = min(hi, nlo + step);
        lo = nlo;
    }
    return lo;
}

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

    const int seq = find_sequence(p.t, tok, lane);
    if (seq < 0) return;  // not scheduled
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
    const bool rope = which == 0 && p.rotary_dim > 0;
    if (rope && pos >= p.rope_positions) {  // no table row for this position
        if (lane == 0) report(p.status, B2A_DEV_BAD_LEN);
        return;
    }
    auto value_at = [&](int d) {
        const float x = to_f32<T>(src[d]);
        if (!rope || d >= p.rotary_dim) return x;
        const int half = p.rotary_dim >> 1;
        return rope_value(p, pos, d, x, to_f32<T>(src[d < half ? d + half : d - half]));
    };

    if (p.kv_dtype != B2A_U8) {
        // plain [block_size, D] chunk of f16 / bf16
        uint16_t* dst = reinterpret_cast<uint16_t*>(cache) +
                        ((static_cast<size_t>(blk) * p.Hkv + hk) * bs + slot) * D;
        for (int d = lane; d < D; d += 32) {
            const float x = value_at(d);
            dst[d] = p.kv_dtype == B2A_F16 ? __half_as_ushort(__float2half_rn(x))
                                           : __bfloat16_as_ushort(__float2bfloat16_rn(x));
        }
        return;
    }

    uint8_t* chunk = cache + (static_cast<size_t>(blk) * p.Hkv + hk) * u8_chunk_bytes(bs, D);
    uint8_t* row = chunk + slot * D;
    // D == 128 with 16-bit inputs: each lane keeps its 4 consecutive values in registers (one 8-byte load, one
    // 4-byte store); other sizes take the strided loops below.  Same arithmetic either way.
    const bool vec = !rope && (D == 128) && sizeof(T) == 2 && ((reinterpret_cast<uintptr_t>(src) & 7) == 0);
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
            const float x = value_at(d);
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
            const float x = value_at(d);
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

// The common geometry (u8 cache, D = Dv = 128, 16-bit rows) with one warp per TOKEN: the walk through the step tables
// is paid once for the token's 2*Hkv rows, and a row is handled by EIGHT lanes (16 values each: two 16-byte loads,
// one 16-byte store of codes), so one pass of the warp quantises four rows - the per-row work (min/max reduction,
// now three shuffle steps, the two scalar divisions, addressing) is issued once for four rows.  Same arithmetic as
// above, operation for operation, except that x / s for the row's values uses one reciprocal (see below).
template <typename T>
__device__ __forceinline__ float bits_to_f32(uint32_t h16);
template <>
__device__ __forceinline__ float bits_to_f32<__half>(uint32_t h16) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(h16)));
}
template <>
__device__ __forceinline__ float bits_to_f32<__nv_bfloat16>(uint32_t h16) {
    return __uint_as_float(h16 << 16);
}

// kRope: the key rows are rotated over all 128 values (rotary_dim == 128): a value's partner, 64 further on or back,
// sits at the same place in the registers of the lane four lanes away; rotated values are arbitrary float32
// numbers, for which the reciprocal shortcut below is not proved, so those rows take the division itself.
template <typename T, bool kRope>
__global__ void __launch_bounds__(kWarpsPerCta * 32) paged_kv_store_rows128_kernel(const StoreParams p) {
    constexpr int D = 128;
    const int lane = threadIdx.x & 31, l8 = lane & 7, rg = lane >> 3;
    const int tok = static_cast<int>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
    grid_dependency_wait();  // the new key/value rows (and the pool's previous readers) belong to earlier kernels
    grid_launch_dependents();
    if (tok >= p.t.num_tokens) return;
    const int seq = find_sequence(p.t, tok, lane);
    if (seq < 0) return;  // not scheduled
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
    if (kRope && pos >= p.rope_positions) {  // no table row for this position
        if (lane == 0) report(p.status, B2A_DEV_BAD_LEN);
        return;
    }
    const size_t chunk_bytes = u8_chunk_bytes(bs, D);
    const int rows = 2 * p.Hkv;  // row r: head r >> 1, key (0) or value (1)
    for (int r0 = 0; r0 < rows; r0 += 4) {
        const int r = r0 + rg;
        const bool live = r < rows;  // whole 8-lane groups are live or not: the shuffles below stay inside a group
        uint4 raw0 = make_uint4(0u, 0u, 0u, 0u), raw1 = raw0;
        if (live) {
            const uint4* src = reinterpret_cast<const uint4*>(
                reinterpret_cast<const T*>((r & 1) ? p.value : p.key) + (static_cast<size_t>(tok) * p.Hkv + (r >> 1)) * D);
            raw0 = src[2 * l8];
            raw1 = src[2 * l8 + 1];
        }
        const uint32_t w[8] = {raw0.x, raw0.y, raw0.z, raw0.w, raw1.x, raw1.y, raw1.z, raw1.w};
        float xv[16];
        float mn = INFINITY, mx = -INFINITY;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            xv[2 * i] = bits_to_f32<T>(w[i] & 0xffffu);
            xv[2 * i + 1] = bits_to_f32<T>(w[i] >> 16);
        }
        const bool rotated = kRope && (r & 1) == 0;  // key rows
        if constexpr (kRope) {
            // lane l8 holds values 16*l8 .. +15: partners are in lane l8 ^ 4 (every lane takes part in the exchange)
#pragma unroll
            for (int e = 0; e < 16; ++e) {
                const float partner = __shfl_xor_sync(0xffffffffu, xv[e], 4);
                if (rotated) xv[e] = rope_value(p, pos, 16 * l8 + e, xv[e], partner);
            }
        }
#pragma unroll
        for (int e = 0; e < 16; ++e) {
            mn = fminf(mn, xv[e]);
            mx = fmaxf(mx, xv[e]);
        }
#pragma unroll
        for (int o = 1; o <= 4; o <<= 1) {
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
        }
        __half s16 = __float2half_rn(__fdiv_rn(__fsub_rn(mx, mn), 255.0f));
        float sf = __half2float(s16);
        if (sf == 0.f || isinf(sf) || isnan(sf)) {
            s16 = __float2half_rn(1.0f);
            sf = 1.0f;
        }
        const __half z16 = __float2half_rn(__fdiv_rn(-mn, sf));
        const float zf = __half2float(z16);
        // x / s for the row's values with ONE reciprocal: q0 = x * r, then one Newton step in fused arithmetic.
        // For a scale that is an f16 value and x an f16 or bf16 value this equals the correctly rounded quotient in
        // every case except |x| below 2^-116, which take the division itself (checked exhaustively on the CPU by
        // oracle/div_by_scale_check.c).
        const float rs = __frcp_rn(sf);
        uint32_t packed[4] = {0u, 0u, 0u, 0u};
#pragma unroll
        for (int e = 0; e < 16; ++e) {
            float q;
            if (rotated || fabsf(xv[e]) < 1e-30f) {
                q = __fdiv_rn(xv[e], sf);
            } else {
                const float q0 = __fmul_rn(xv[e], rs);
                q = fabsf(q0) < INFINITY ? __fmaf_rn(__fmaf_rn(-sf, q0, xv[e]), rs, q0) : q0;
            }
            const float t = rintf(__fadd_rn(q, zf));
            packed[e >> 2] |= static_cast<uint32_t>(fminf(fmaxf(t, 0.f), 255.f)) << (8 * (e & 3));
        }
        if (live) {
            uint8_t* chunk = ((r & 1) ? p.v_cache : p.k_cache) + (static_cast<size_t>(blk) * p.Hkv + (r >> 1)) * chunk_bytes;
            reinterpret_cast<uint4*>(chunk + slot * D)[l8] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            if (l8 == 0) {
                __half* meta = reinterpret_cast<__half*>(chunk + bs * D);
                meta[slot] = s16;
                meta[bs + slot] = z16;
            }
        }
    }
}

}  // namespace

int paged_kv_store_launch(const b2a_paged_desc& d, const void* key, const void* value, void* k_cache, void* v_cache,
                          const PagedTables& t, int32_t* status, cudaStream_t stream, const RopeTables* rope) {
    if (d.num_tokens == 0) return B2A_OK;
    StoreParams p{key, value, static_cast<uint8_t*>(k_cache), static_cast<uint8_t*>(v_cache), t,
                  d.Hkv, d.D, d.Dv, d.kv_dtype, status, nullptr, nullptr, 0, 0};
    if (rope != nullptr && rope->rotary_dim > 0) {
        p.rope_cos = rope->cos;
        p.rope_sin = rope->sin;
        p.rotary_dim = rope->rotary_dim;
        p.rope_positions = rope->positions;
    }
    const bool rope_all = p.rotary_dim == 128;
    auto al8 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
    if (d.kv_dtype == B2A_U8 && d.D == 128 && d.Dv == 128 && (d.q_dtype == B2A_F16 || d.q_dtype == B2A_BF16) &&
        al8(key) && al8(value) && (p.rotary_dim == 0 || rope_all)) {
        const unsigned grid_t = static_cast<unsigned>((d.num_tokens + kWarpsPerCta - 1) / kWarpsPerCta);
        const dim3 block(kWarpsPerCta * 32);
        cudaError_t e;
        if (d.q_dtype == B2A_F16)
            e = rope_all ? launch_overlapped(paged_kv_store_rows128_kernel<__half, true>, dim3(grid_t), block, 0, stream, p)
                         : launch_overlapped(paged_kv_store_rows128_kernel<__half, false>, dim3(grid_t), block, 0, stream, p);
        else
            e = rope_all ? launch_overlapped(paged_kv_store_rows128_kernel<__nv_bfloat16, true>, dim3(grid_t), block, 0, stream, p)
                         : launch_overlapped(paged_kv_store_rows128_kernel<__nv_bfloat16, false>, dim3(grid_t), block, 0, stream, p);
        return e == cudaSuccess ? B2A_OK : B2A_ERR_CUDA;
    }
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
