// General attention kernel: any head size up to 256, any mask, any stride, f32 / f16 / bf16, contiguous or paged
// K/V.  It is the path for the shapes the specialised kernels (tcgen05 prefill, split-K decode) do not take:
// f32 tensors, explicit masks, odd head sizes, multi-token rows over a paged cache.
//
// One CTA of 256 threads owns 32 query rows of one query head and walks the keys 32 at a time with an online
// (running max / running sum) softmax, all arithmetic in float32:
//   phase 1  S[i][j] = q_i . k_j            thread = (4 rows of its warp) x (key = lane)
//   phase 2  row max / sum by warp shuffle, P = exp(S - m) into shared memory
//   phase 3  O[i][:] = O[i][:]*alpha + P[i][:] . V     thread = (4 rows of its warp) x (columns lane, lane+32, ..)
// A warp owns the same 4 rows in all phases, so the softmax state lives in registers.
#include "launch.cuh"

namespace b2a {
namespace {

constexpr int kBM = 32;       // query rows per CTA
constexpr int kBN = 32;       // keys per step
constexpr int kThreads = 256;
constexpr int kRowsPerWarp = 4;
constexpr int kMaxD = 256;

struct GenericParams {
    // geometry
    int B, Hq, Hkv, Sq, Skv, D, Dv;
    int causal;
    float scale;
    // contiguous mode
    const void* q;
    const void* k;
    const void* v;
    void* o;
    int64_t qs[4], ks[4], vs[4], os[4];
    const void* mask;
    int mask_kind;
    int64_t ms[4];
    // paged mode
    int paged;     // 0 = contiguous, 1 = paged
    int kv_dtype;  // paged only
    int sliding_window;
    PagedTables t;
    const uint8_t* k_cache;
    const uint8_t* v_cache;
    int32_t* status;
};

template <typename T>
__device__ __forceinline__ float load_cache_elem(const uint8_t* chunk, int kv_dtype, int bs, int d_total, int slot,
                                                 int d) {
    if (kv_dtype == B2A_U8) {
        const float qv = static_cast<float>(chunk[slot * d_total + d]);
        const __half* meta = reinterpret_cast<const __half*>(chunk + bs * d_total);
        const float sc = __half2float(meta[slot]);
        const float zp = __half2float(meta[bs + slot]);
        return __fmul_rn(__fsub_rn(qv, zp), sc);
    } else if (kv_dtype == B2A_F16) {
        return __half2float(reinterpret_cast<const __half*>(chunk)[slot * d_total + d]);
    } else {
        return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(chunk)[slot * d_total + d]);
    }
}

template <typename T>
__global__ void __launch_bounds__(kThreads) attn_generic_kernel(const GenericParams p) {
    extern __shared__ float smem[];
    const int D = p.D, Dv = p.Dv;
    float* sQ = smem;                    // [32][D]
    float* sK = sQ + kBM * D;            // [32][D+1]
    float* sV = sK + kBN * (D + 1);      // [32][Dv]
    float* sP = sV + kBN * Dv;           // [32][33]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.y;
    const int g = p.Hq / p.Hkv;
    const int hk = h / g;

    // Row range of this CTA and the key horizon of each row.
    int row0, nrows, kv_len, pos0;  // pos0: cache position of row 0 of the tile (paged) / row index (contiguous)
    int b = 0, seq = 0;
    int tok0 = 0;
    if (p.paged) {
        seq = blockIdx.z;
        const int sb = p.t.subsequence_begins[seq], se = p.t.subsequence_begins[seq + 1];
        const int qlen = se - sb;
        row0 = blockIdx.x * kBM;
        if (row0 >= qlen) return;
        nrows = min(kBM, qlen - row0);
        const int past = p.t.past_lens[seq];
        kv_len = past + qlen;
        pos0 = past + row0;
        tok0 = sb + row0;
        if (qlen < 0 || past < 0 || se > p.t.num_tokens) {
            if (tid == 0) report(p.status, B2A_DEV_BAD_LEN);
            return;
        }
    } else {
        b = blockIdx.z;
        row0 = blockIdx.x * kBM;
        nrows = min(kBM, p.Sq - row0);
        kv_len = p.Skv;
        pos0 = row0;
    }
    const bool causal = p.paged || p.causal;
    // keys beyond the last row's horizon are never needed
    const int k_end = causal ? min(kv_len, pos0 + nrows) : kv_len;
    int k_begin = 0;
    if (p.paged && p.sliding_window > 0) k_begin = max(0, pos0 - p.sliding_window + 1);
    k_begin = (k_begin / kBN) * kBN;

    // ---- load the query tile (zero rows beyond nrows)
    const T* qbase;
    int64_t q_row_stride;
    if (p.paged) {
        qbase = reinterpret_cast<const T*>(p.q) + static_cast<int64_t>(tok0) * p.Hq * D + static_cast<int64_t>(h) * D;
        q_row_stride = static_cast<int64_t>(p.Hq) * D;
    } else {
        qbase = reinterpret_cast<const T*>(p.q) + b * p.qs[0] + h * p.qs[1] + row0 * p.qs[2];
        q_row_stride = p.qs[2];
    }
    for (int idx = tid; idx < kBM * D; idx += kThreads) {
        const int r = idx / D, d = idx - r * D;
        sQ[idx] = r < nrows ? to_f32<T>(qbase[r * q_row_stride + d]) : 0.f;
    }

    float m_run[kRowsPerWarp], l_run[kRowsPerWarp];
    float acc[kRowsPerWarp][kMaxD / 32];
#pragma unroll
    for (int i = 0; i < kRowsPerWarp; ++i) {
        m_run[i] = -INFINITY;
        l_run[i] = 0.f;
#pragma unroll
        for (int c = 0; c < kMaxD / 32; ++c) acc[i][c] = 0.f;
    }
    const int ncol = (Dv + 31) / 32;

    const int32_t* btab = p.paged ? p.t.block_indices + p.t.block_indices_begins[seq] : nullptr;
    const size_t chunk_k = p.paged ? (p.kv_dtype == B2A_U8 ? u8_chunk_bytes(p.t.block_size, D)
                                                           : static_cast<size_t>(p.t.block_size) * D * 2)
                                   : 0;
    const size_t chunk_v = p.paged ? (p.kv_dtype == B2A_U8 ? u8_chunk_bytes(p.t.block_size, Dv)
                                                           : static_cast<size_t>(p.t.block_size) * Dv * 2)
                                   : 0;

    for (int j0 = k_begin; j0 < k_end; j0 += kBN) {
        __syncthreads();  // previous tile fully consumed (also orders the sQ fill before first use)
        // ---- stage K and V rows j0 .. j0+31 as float32
        if (!p.paged) {
            const T* kb = reinterpret_cast<const T*>(p.k) + b * p.ks[0] + hk * p.ks[1];
            const T* vb = reinterpret_cast<const T*>(p.v) + b * p.vs[0] + hk * p.vs[1];
            for (int idx = tid; idx < kBN * D; idx += kThreads) {
                const int r = idx / D, d = idx - r * D;
                const int j = j0 + r;
                sK[r * (D + 1) + d] = j < k_end ? to_f32<T>(kb[j * p.ks[2] + d]) : 0.f;
            }
            for (int idx = tid; idx < kBN * Dv; idx += kThreads) {
                const int r = idx / Dv, d = idx - r * Dv;
                const int j = j0 + r;
                sV[idx] = j < k_end ? to_f32<T>(vb[j * p.vs[2] + d]) : 0.f;
            }
        } else {
            const int bs = p.t.block_size;
            for (int idx = tid; idx < kBN * D; idx += kThreads) {
                const int r = idx / D, d = idx - r * D;
                const int j = j0 + r;
                float x = 0.f;
                if (j < k_end) {
                    const int blk = btab[j / bs];
                    if (blk < 0 || blk >= p.t.num_blocks_total) {
                        report(p.status, B2A_DEV_BAD_BLOCK);
                    } else {
                        const uint8_t* chunk = p.k_cache + (static_cast<size_t>(blk) * p.Hkv + hk) * chunk_k;
                        x = load_cache_elem<T>(chunk, p.kv_dtype, bs, D, j % bs, d);
                    }
                }
                sK[r * (D + 1) + d] = x;
            }
            for (int idx = tid; idx < kBN * Dv; idx += kThreads) {
                const int r = idx / Dv, d = idx - r * Dv;
                const int j = j0 + r;
                float x = 0.f;
                if (j < k_end) {
                    const int blk = btab[j / bs];
                    if (blk >= 0 && blk < p.t.num_blocks_total) {
                        const uint8_t* chunk = p.v_cache + (static_cast<size_t>(blk) * p.Hkv + hk) * chunk_v;
                        x = load_cache_elem<T>(chunk, p.kv_dtype, bs, Dv, j % bs, d);
                    }
                }
                sV[idx] = x;
            }
        }
        __syncthreads();

        // ---- phase 1: scores of rows warp*4+i against key j0+lane
        float s[kRowsPerWarp] = {0.f, 0.f, 0.f, 0.f};
        {
            const float* kr = sK + lane * (D + 1);
            const float* qr = sQ + (warp * kRowsPerWarp) * D;
            for (int d = 0; d < D; ++d) {
                const float kv = kr[d];
#pragma unroll
                for (int i = 0; i < kRowsPerWarp; ++i) s[i] = fmaf(qr[i * D + d], kv, s[i]);
            }
        }
        const int j = j0 + lane;
        // ---- phase 2: mask, online softmax
#pragma unroll
        for (int i = 0; i < kRowsPerWarp; ++i) {
            const int r = warp * kRowsPerWarp + i;
            float sv = s[i] * p.scale;
            bool keep = (j < k_end) && (r < nrows);
            if (causal) keep = keep && (j <= pos0 + r);
            if (p.paged && p.sliding_window > 0) keep = keep && (pos0 + r - j < p.sliding_window);
            if (!p.paged && !p.causal && p.mask_kind != B2A_MASK_NONE && keep) {
                const int64_t mo = b * p.ms[0] + h * p.ms[1] + static_cast<int64_t>(row0 + r) * p.ms[2] + j * p.ms[3];
                if (p.mask_kind == B2A_MASK_BOOL) {
                    keep = reinterpret_cast<const uint8_t*>(p.mask)[mo] != 0;
                } else {
                    sv += to_f32<T>(reinterpret_cast<const T*>(p.mask)[mo]);
                }
            }
            if (!keep) sv = -INFINITY;
            const float tile_max = warp_max(sv);
            const float m_new = fmaxf(m_run[i], tile_max);
            float alpha, pv;
            if (m_new == -INFINITY) {  // nothing kept so far
                alpha = 1.f;
                pv = 0.f;
            } else {
                alpha = expf(m_run[i] - m_new);  // exp(-inf) = 0 on the first kept tile
                pv = expf(sv - m_new);
            }
            const float tile_sum = warp_sum(pv);
            l_run[i] = l_run[i] * alpha + tile_sum;
            m_run[i] = m_new;
            sP[r * (kBN + 1) + lane] = pv;
#pragma unroll
            for (int c = 0; c < kMaxD / 32; ++c) acc[i][c] *= alpha;
        }
        __syncwarp();
        // ---- phase 3: O += P . V
        for (int jj = 0; jj < kBN; ++jj) {
            float pr[kRowsPerWarp];
#pragma unroll
            for (int i = 0; i < kRowsPerWarp; ++i) pr[i] = sP[(warp * kRowsPerWarp + i) * (kBN + 1) + jj];
#pragma unroll
            for (int c = 0; c < kMaxD / 32; ++c) {
                if (c < ncol) {
                    const int d = lane + 32 * c;
                    const float vv = d < Dv ? sV[jj * Dv + d] : 0.f;
#pragma unroll
                    for (int i = 0; i < kRowsPerWarp; ++i) acc[i][c] = fmaf(pr[i], vv, acc[i][c]);
                }
            }
        }
        __syncwarp();
    }

    // ---- normalise and store
#pragma unroll
    for (int i = 0; i < kRowsPerWarp; ++i) {
        const int r = warp * kRowsPerWarp + i;
        if (r >= nrows) continue;
        const float inv = l_run[i] > 0.f ? 1.f / l_run[i] : 0.f;
        T* orow;
        if (p.paged) {
            orow = reinterpret_cast<T*>(p.o) + static_cast<int64_t>(tok0 + r) * p.Hq * Dv + static_cast<int64_t>(h) * Dv;
        } else {
            orow = reinterpret_cast<T*>(p.o) + b * p.os[0] + h * p.os[1] + static_cast<int64_t>(row0 + r) * p.os[2];
        }
#pragma unroll
        for (int c = 0; c < kMaxD / 32; ++c) {
            const int d = lane + 32 * c;
            if (c < ncol && d < Dv) orow[d] = from_f32<T>(acc[i][c] * inv);
        }
    }
}

size_t generic_smem_bytes(int D, int Dv) {
    return sizeof(float) * (static_cast<size_t>(kBM) * D + kBN * (D + 1) + kBN * Dv + kBM * (kBN + 1));
}

template <typename T>
int launch_generic_t(const GenericParams& p, dim3 grid, cudaStream_t stream) {
    const size_t smem = generic_smem_bytes(p.D, p.Dv);
    auto kern = attn_generic_kernel<T>;
    static bool configured[64] = {};  // per device, per element type (this function is a template)
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return B2A_ERR_CUDA;
    if (smem > 48 * 1024 && (dev < 0 || dev >= 64 || !configured[dev])) {
        // An attribute of the function, not a stream operation: legal while a stream is being captured.
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 120 * 1024) != cudaSuccess)
            return B2A_ERR_CUDA;
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    kern<<<grid, kThreads, smem, stream>>>(p);
    return cudaGetLastError() == cudaSuccess ? B2A_OK : B2A_ERR_CUDA;
}

int launch_generic(int dtype, const GenericParams& p, dim3 grid, cudaStream_t stream) {
    switch (dtype) {
        case B2A_F32: return launch_generic_t<float>(p, grid, stream);
        case B2A_F16: return launch_generic_t<__half>(p, grid, stream);
        case B2A_BF16: return launch_generic_t<__nv_bfloat16>(p, grid, stream);
        default: return B2A_ERR_DTYPE;
    }
}

}  // namespace

int sdpa_generic_launch(const b2a_sdpa_desc& d, const int64_t (&qs)[4], const int64_t (&ks)[4],
                        const int64_t (&vs)[4], const int64_t (&os)[4], const void* q, const void* k, const void* v,
                        const void* mask, void* o, int32_t* status, cudaStream_t stream) {
    if (d.D > kMaxD || d.Dv > kMaxD) return B2A_ERR_UNSUPPORTED;
    GenericParams p{};
    p.B = d.B; p.Hq = d.Hq; p.Hkv = d.Hkv; p.Sq = d.Sq; p.Skv = d.Skv; p.D = d.D; p.Dv = d.Dv;
    p.causal = d.causal;
    p.scale = d.scale;
    p.q = q; p.k = k; p.v = v; p.o = o;
    for (int i = 0; i < 4; ++i) {
        p.qs[i] = qs[i]; p.ks[i] = ks[i]; p.vs[i] = vs[i]; p.os[i] = os[i]; p.ms[i] = d.mask_strides[i];
    }
    p.mask = mask;
    p.mask_kind = d.causal ? B2A_MASK_NONE : d.mask_kind;
    p.paged = 0;
    p.status = status;
    dim3 grid((d.Sq + kBM - 1) / kBM, d.Hq, d.B);
    return launch_generic(d.dtype, p, grid, stream);
}

int paged_generic_launch(const b2a_paged_desc& d, const void* query, const void* k_cache, const void* v_cache,
                         const PagedTables& t, void* out, int32_t* status, cudaStream_t stream) {
    if (d.D > kMaxD || d.Dv > kMaxD) return B2A_ERR_UNSUPPORTED;
    GenericParams p{};
    p.Hq = d.Hq; p.Hkv = d.Hkv; p.D = d.D; p.Dv = d.Dv;
    p.scale = d.scale;
    p.q = query; p.o = out;
    p.paged = 1;
    p.kv_dtype = d.kv_dtype;
    p.sliding_window = d.sliding_window;
    p.t = t;
    p.k_cache = static_cast<const uint8_t*>(k_cache);
    p.v_cache = static_cast<const uint8_t*>(v_cache);
    p.status = status;
    dim3 grid((d.max_q_len + kBM - 1) / kBM, d.Hq, d.num_seqs);
    return launch_generic(d.q_dtype, p, grid, stream);
}

}  // namespace b2a
