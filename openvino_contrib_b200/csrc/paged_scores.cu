// Score output of the paged attention: for every sequence of a step, the attention probabilities of its LAST query
// token over the sequence's cached keys, summed over the query heads - what a cache-eviction policy accumulates to
// decide which tokens to keep (the reference's policy consumes exactly such per-key sums of attention weights:
// modules/genai_optimizations/genai_opt/token_eviction.py:154-183, `attn_w.sum(dim=(0, 2))` then `.sum(0)` over heads).
// OpenVINO's PagedAttentionExtension carries it as its second output; the reference plugin has no paged attention,
// so there is no kernel there to compare with.
//
// u8 cache, D = 128, 16-token blocks, at most eight query heads per KV head.  Only K is read.  Two passes over K
// (each at the speed of the decode kernel's K stream: the same per-warp cp.async pipeline, the same QK^T on
// mma.sync with the codes unscaled), because a probability needs the row's final maximum and sum:
//   pass 0: per (sequence, chunk of blocks) the running (max, sum) of every head -> one partial per chunk;
//           a small kernel merges the chunks into lse[h] = max + log2(sum)  (base-2, of the scaled scores);
//   pass 1: p = 2^(s - lse[h]) for every key, summed over the heads, written once per key (no atomics: a CTA walks
//           ALL KV heads of its blocks - a block's chunks of the eight KV heads are adjacent in the pool - and keeps
//           the per-key sums in shared memory).
// The output is flat: sequence s occupies [score_begins[s], score_begins[s+1]) with one float per context position
// (positions outside a sliding window get 0); score_begins is written by the first kernel.
#include <algorithm>

#include "launch.cuh"

namespace b2a {
namespace {

constexpr int kD = 128;
constexpr int kBS = 16;
constexpr int kChunk = kBS * (kD + 4);  // 2112 bytes: 2048 codes, 16 f16 scales, 16 f16 zero-points
constexpr int kStages = 3;
constexpr int kWarps = 4;
constexpr int kMaxBlocksPerCta = 32 * kWarps;  // a warp keeps the ids of at most 32 blocks
constexpr int kMaxHq = 128;
constexpr float kNegBig = -1.0e30f;
constexpr float kCodeBias = 1024.f;  // the byte permute below yields 1024 + code; the 1024 joins the zero-point

struct ScoreParams {
    const void* query;
    const uint8_t* k_cache;
    PagedTables t;
    int Hq, Hkv, G;
    int blocks_per_cta, max_splits, max_blocks;
    int sliding_window;
    float scale_log2;
    float* ws_ml;          // [num_seqs][max_splits][Hq][2]
    float* ws_lse;         // [num_seqs][Hq]
    int32_t* score_begins; // [num_seqs + 1]
    float* scores;         // flat
    long long capacity;    // floats the caller's score buffer holds
    int32_t* status;
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 r;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "r"(addr));
    return r;
}
__device__ __forceinline__ float lds_h(uint32_t addr) {
    unsigned short r;
    asm volatile("ld.shared.u16 %0, [%1];\n" : "=h"(r) : "r"(addr));
    return __half2float(__ushort_as_half(r));
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
template <int PAIR>
__device__ __forceinline__ uint32_t bytes_to_h2(uint32_t w) {  // (1024 + byte 2*PAIR, 1024 + byte 2*PAIR+1) as f16 pair
    return __byte_perm(w, 0x64646464u, PAIR == 0 ? 0x4140 : 0x4342);
}
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ float h2_lo(uint32_t v) { return __half2float(__ushort_as_half(v & 0xFFFFu)); }
__device__ __forceinline__ float h2_hi(uint32_t v) { return __half2float(__ushort_as_half(v >> 16)); }
template <typename T>
__device__ __forceinline__ uint32_t q_word_to_h2(uint32_t w);
template <>
__device__ __forceinline__ uint32_t q_word_to_h2<__half>(uint32_t w) {
    return w;
}
template <>
__device__ __forceinline__ uint32_t q_word_to_h2<__nv_bfloat16>(uint32_t w) {
    return pack_h2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}

// A sequence as the score kernels see it: its last query token against its whole context.
struct SeqRow {
    int tok, ctx, nblk, bib0, blk_lo, first_pos;
    bool ok;   // has a query token and consistent tables
    bool bad;  // inconsistent tables (to be reported)
};
__device__ __forceinline__ SeqRow seq_row(const ScoreParams& p, int s) {
    SeqRow r;
    const int t0 = p.t.subsequence_begins[s], t1 = p.t.subsequence_begins[s + 1];
    const int past = p.t.past_lens[s];
    r.bib0 = p.t.block_indices_begins[s];
    const int have = p.t.block_indices_begins[s + 1] - r.bib0;
    r.tok = t1 - 1;
    r.ctx = past + (t1 - t0);
    r.nblk = (r.ctx + kBS - 1) / kBS;
    r.first_pos = p.sliding_window > 0 ? max(0, r.ctx - p.sliding_window) : 0;
    r.blk_lo = r.first_pos / kBS;
    const bool has_row = t1 - t0 >= 1;
    r.bad = has_row && (past < 0 || t0 < 0 || t1 > p.t.num_tokens || r.nblk > have || r.nblk > p.max_blocks);
    r.ok = has_row && !r.bad;
    return r;
}

// First kernel: where every sequence's scores start.  A sequence without a query token, or with inconsistent tables
// (reported), gets no entries.  One CTA; sequences are few.
__global__ void __launch_bounds__(256) score_begins_kernel(const ScoreParams p) {
    __shared__ int s_part[256];
    grid_dependency_wait();
    grid_launch_dependents();
    const int tid = threadIdx.x, n = p.t.num_seqs;
    const int per = (n + 255) / 256;
    int mine = 0;
    bool bad = false;
    for (int s = tid * per; s < min(n, (tid + 1) * per); ++s) {
        const SeqRow r = seq_row(p, s);
        mine += r.ok ? r.ctx : 0;
        bad |= r.bad;
    }
    s_part[tid] = mine;
    __syncthreads();
    if (tid == 0) {
        int run = 0;
        for (int i = 0; i < 256; ++i) {
            const int v = s_part[i];
            s_part[i] = run;
            run += v;
        }
        p.score_begins[n] = run;
        if (run > p.capacity) report(p.status, B2A_DEV_BAD_LEN);  // the score buffer is too small: nothing past it is written
    }
    __syncthreads();
    int run = s_part[tid];
    for (int s = tid * per; s < min(n, (tid + 1) * per); ++s) {
        const SeqRow r = seq_row(p, s);
        p.score_begins[s] = run;
        run += r.ok ? r.ctx : 0;
    }
    if (bad) report(p.status, B2A_DEV_BAD_LEN);
}

// One pass over the K chunks of (sequence blockIdx.x, chunk of blocks blockIdx.y), all KV heads.  Warp w takes blocks
// w, w + 4, ... of the chunk; for each KV head in turn it walks its blocks (iteration i = hk * n_w + b), so the query
// fragments and the per-head state change only every n_w iterations.
//   kPass 0: running (max, sum) per head; the warps' results are merged and one partial per head is written.
//   kPass 1: probabilities from the finished lse, summed over the heads into per-key sums in shared memory (a block
//            belongs to one warp for all KV heads, so nobody else touches its sums), written out at the end.
template <typename T, int kPass>
__global__ void __launch_bounds__(kWarps * 32) score_pass_kernel(const ScoreParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ float s_scores[kPass == 1 ? kMaxBlocksPerCta * kBS : 1];
    __shared__ float s_ml[kPass == 0 ? kWarps * kMaxHq * 2 : 1];
    const int seq = blockIdx.x, split = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int gid = lane >> 2, tid4 = lane & 3;
    grid_dependency_wait();
    grid_launch_dependents();

    const SeqRow r = seq_row(p, seq);
    if (!r.ok) return;
    if (r.nblk - r.blk_lo > p.max_splits * p.blocks_per_cta) return;  // (cannot happen: nblk <= max_blocks was checked)
    const int my_lo = r.blk_lo + split * p.blocks_per_cta;
    const int my_hi = min(r.nblk, my_lo + p.blocks_per_cta);
    if (my_lo >= my_hi) return;
    const long long out0 = p.score_begins[seq];
    if (kPass == 1 && out0 + r.ctx > p.capacity) return;  // reported by the first kernel

    const int n_w = max(0, (my_hi - my_lo - warp + kWarps - 1) / kWarps);
    int my_phys = 0;
    if (lane < n_w) {
        my_phys = p.t.block_indices[r.bib0 + my_lo + warp + kWarps * lane];
        if (my_phys < 0 || my_phys >= p.t.num_blocks_total) {
            report(p.status, B2A_DEV_BAD_BLOCK);
            my_phys = -1;
        }
    }
    if constexpr (kPass == 1) {
        for (int i = tid; i < (my_hi - my_lo) * kBS; i += kWarps * 32) s_scores[i] = 0.f;
        __syncthreads();
    }

    const uint32_t smem_warp = static_cast<uint32_t>(__cvta_generic_to_shared(smem)) + warp * (kStages * kChunk);
    const size_t block_stride = static_cast<size_t>(p.Hkv) * kChunk;
    const int iters = p.Hkv * n_w;
    auto issue = [&](int i) {
        const int hk = i / n_w, b = i - hk * n_w;
        const int phys = __shfl_sync(0xffffffffu, my_phys, b & 31);
        if (phys >= 0) {
            const uint8_t* kc = p.k_cache + phys * block_stride + static_cast<size_t>(hk) * kChunk;
            const uint32_t st = smem_warp + (i % kStages) * kChunk;
#pragma unroll
            for (int rr = 0; rr < 4; ++rr) {
                const int piece = rr * 32 + lane;  // 16-byte piece of the 2048 code bytes
                const int row = piece >> 3, col = piece & 7;
                cp_async16(st + row * 128 + ((col ^ (row & 7)) << 4), kc + piece * 16);
            }
            if (lane < 4) cp_async16(st + 2048 + lane * 16, kc + 2048 + lane * 16);
        }
    };
#pragma unroll
    for (int s = 0; s < kStages - 1; ++s) {
        if (s < iters) issue(s);
        cp_async_commit();
    }

    uint32_t qf[8][2];
    float qsum_a = 0.f, qsum_b = 0.f;          // sums of Q over d for heads 2*tid4 and 2*tid4 + 1 of the group
    float m_a = kNegBig, m_b = kNegBig, l_a = 0.f, l_b = 0.f;  // pass 0
    float lse_a = 0.f, lse_b = 0.f;            // pass 1
    const int sw_k = gid & 7;
    const bool head_a = 2 * tid4 < p.G, head_b = 2 * tid4 + 1 < p.G;
    for (int i = 0; i < iters; ++i) {
        const int hk = i / n_w, b = i - hk * n_w;
        if (b == 0) {
            // query fragments of this KV head's group: head gid, elements tid4*32 .. +31
            const T* qrow = reinterpret_cast<const T*>(p.query) + (static_cast<size_t>(r.tok) * p.Hq + hk * p.G) * kD;
            float part = 0.f;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint4 w4 = make_uint4(0u, 0u, 0u, 0u);
                if (gid < p.G) w4 = reinterpret_cast<const uint4*>(qrow + gid * kD + tid4 * 32)[c];
                const uint32_t w[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
                for (int hf = 0; hf < 2; ++hf) {
                    const uint32_t b0 = q_word_to_h2<T>(w[2 * hf]), b1 = q_word_to_h2<T>(w[2 * hf + 1]);
                    qf[2 * c + hf][0] = b0;
                    qf[2 * c + hf][1] = b1;
                    part += h2_lo(b0) + h2_hi(b0) + h2_lo(b1) + h2_hi(b1);
                }
            }
            part += __shfl_xor_sync(0xffffffffu, part, 1);
            part += __shfl_xor_sync(0xffffffffu, part, 2);
            qsum_a = __shfl_sync(0xffffffffu, part, 8 * tid4);
            qsum_b = __shfl_sync(0xffffffffu, part, 8 * tid4 + 4);
            if constexpr (kPass == 0) {
                m_a = m_b = kNegBig;
                l_a = l_b = 0.f;
            } else {
                const float* lse = p.ws_lse + static_cast<size_t>(seq) * p.Hq + hk * p.G;
                lse_a = head_a ? lse[2 * tid4] : 0.f;
                lse_b = head_b ? lse[2 * tid4 + 1] : 0.f;
            }
        }
        if (i + kStages - 1 < iters) issue(i + kStages - 1);
        cp_async_commit();
        cp_async_wait<kStages - 1>();
        __syncwarp();

        const uint32_t sK = smem_warp + (i % kStages) * kChunk;
        const int lb = my_lo + warp + kWarps * b;
        const bool blk_ok = __shfl_sync(0xffffffffu, my_phys, b & 31) >= 0;
        const int pos0 = lb * kBS + gid, pos1 = pos0 + 8;
        const bool ok0 = blk_ok && pos0 < r.ctx && pos0 >= r.first_pos;
        const bool ok1 = blk_ok && pos1 < r.ctx && pos1 >= r.first_pos;
        float sc[4] = {0.f, 0.f, 0.f, 0.f};
        {
            const uint4 x0 = lds128(sK + gid * 128 + (((2 * tid4) ^ sw_k) << 4));
            const uint4 x1 = lds128(sK + gid * 128 + (((2 * tid4 + 1) ^ sw_k) << 4));
            const uint4 y0 = lds128(sK + (gid + 8) * 128 + (((2 * tid4) ^ sw_k) << 4));
            const uint4 y1 = lds128(sK + (gid + 8) * 128 + (((2 * tid4 + 1) ^ sw_k) << 4));
            const uint32_t wl[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
            const uint32_t wh[8] = {y0.x, y0.y, y0.z, y0.w, y1.x, y1.y, y1.z, y1.w};
#pragma unroll
            for (int j = 0; j < 8; ++j)
                mma16816(sc, bytes_to_h2<0>(wl[j]), bytes_to_h2<0>(wh[j]), bytes_to_h2<1>(wl[j]), bytes_to_h2<1>(wh[j]),
                         qf[j][0], qf[j][1]);
        }
        const float sk0 = ok0 ? lds_h(sK + 2048 + 2 * gid) * p.scale_log2 : 0.f;
        const float sk1 = ok1 ? lds_h(sK + 2048 + 2 * (gid + 8)) * p.scale_log2 : 0.f;
        const float zk0 = ok0 ? lds_h(sK + 2048 + 32 + 2 * gid) + kCodeBias : 0.f;
        const float zk1 = ok1 ? lds_h(sK + 2048 + 32 + 2 * (gid + 8)) + kCodeBias : 0.f;
        // scaled scores in base-2 units: token gid x heads (a, b), token gid+8 x heads (a, b)
        const float s0 = ok0 ? (sc[0] - zk0 * qsum_a) * sk0 : -INFINITY;
        const float s1 = ok0 ? (sc[1] - zk0 * qsum_b) * sk0 : -INFINITY;
        const float s2 = ok1 ? (sc[2] - zk1 * qsum_a) * sk1 : -INFINITY;
        const float s3 = ok1 ? (sc[3] - zk1 * qsum_b) * sk1 : -INFINITY;
        if constexpr (kPass == 0) {
            float ta = fmaxf(s0, s2), tb = fmaxf(s1, s3);
#pragma unroll
            for (int o = 4; o <= 16; o <<= 1) {
                ta = fmaxf(ta, __shfl_xor_sync(0xffffffffu, ta, o));
                tb = fmaxf(tb, __shfl_xor_sync(0xffffffffu, tb, o));
            }
            const float na = fmaxf(m_a, ta), nb = fmaxf(m_b, tb);
            l_a = l_a * ex2(m_a - na) + ex2(s0 - na) + ex2(s2 - na);
            l_b = l_b * ex2(m_b - nb) + ex2(s1 - nb) + ex2(s3 - nb);
            m_a = na;
            m_b = nb;
            if (b == n_w - 1) {  // this KV head is done: sums over the eight token rows, parked for the merge of the warps
#pragma unroll
                for (int o = 4; o <= 16; o <<= 1) {
                    l_a += __shfl_xor_sync(0xffffffffu, l_a, o);
                    l_b += __shfl_xor_sync(0xffffffffu, l_b, o);
                }
                if (gid == 0) {
                    float* dst = s_ml + (warp * kMaxHq + hk * p.G) * 2;
                    if (head_a) { dst[4 * tid4] = m_a; dst[4 * tid4 + 1] = l_a; }
                    if (head_b) { dst[4 * tid4 + 2] = m_b; dst[4 * tid4 + 3] = l_b; }
                }
            }
        } else {
            float c0 = (head_a ? ex2(s0 - lse_a) : 0.f) + (head_b ? ex2(s1 - lse_b) : 0.f);  // token gid
            float c1 = (head_a ? ex2(s2 - lse_a) : 0.f) + (head_b ? ex2(s3 - lse_b) : 0.f);  // token gid + 8
            c0 += __shfl_xor_sync(0xffffffffu, c0, 1);
            c1 += __shfl_xor_sync(0xffffffffu, c1, 1);
            c0 += __shfl_xor_sync(0xffffffffu, c0, 2);
            c1 += __shfl_xor_sync(0xffffffffu, c1, 2);
            if (tid4 == 0) {
                float* dst = s_scores + (lb - my_lo) * kBS;
                dst[gid] += c0;
                dst[gid + 8] += c1;
            }
        }
        __syncwarp();  // every lane is done with this stage before it is refilled
    }
    cp_async_wait<0>();
    __syncthreads();

    if constexpr (kPass == 0) {
        // merge the warps (a warp without blocks parked nothing): one (max, sum) per head
        for (int h = tid; h < p.Hq; h += kWarps * 32) {
            float mc = kNegBig;
            for (int w = 0; w < kWarps; ++w)
                if ((my_hi - my_lo - w + kWarps - 1) / kWarps > 0) mc = fmaxf(mc, s_ml[(w * kMaxHq + h) * 2]);
            float l = 0.f;
            for (int w = 0; w < kWarps; ++w)
                if ((my_hi - my_lo - w + kWarps - 1) / kWarps > 0)
                    l += s_ml[(w * kMaxHq + h) * 2 + 1] * ex2(s_ml[(w * kMaxHq + h) * 2] - mc);
            float* dst = p.ws_ml + ((static_cast<size_t>(seq) * p.max_splits + split) * p.Hq + h) * 2;
            dst[0] = mc;
            dst[1] = l;
        }
    } else {
        const int first = my_lo * kBS, count = min(r.ctx, my_hi * kBS) - first;
        for (int i = tid; i < count; i += kWarps * 32) p.scores[out0 + first + i] = s_scores[i];
        // positions below the first block of a sliding window belong to nobody's chunk: the first chunk clears them
        if (split == 0)
            for (int i = tid; i < first; i += kWarps * 32) p.scores[out0 + i] = 0.f;
    }
}

// lse[h] = max + log2(sum) over the chunks of a sequence (base 2, of the scaled scores).
__global__ void __launch_bounds__(128) score_lse_kernel(const ScoreParams p) {
    const int seq = blockIdx.x;
    grid_dependency_wait();
    grid_launch_dependents();
    const SeqRow r = seq_row(p, seq);
    if (!r.ok) return;
    const int nsplit = min(p.max_splits, (r.nblk - r.blk_lo + p.blocks_per_cta - 1) / p.blocks_per_cta);
    for (int h = threadIdx.x; h < p.Hq; h += blockDim.x) {
        const float* ml = p.ws_ml + (static_cast<size_t>(seq) * p.max_splits * p.Hq + h) * 2;
        const size_t stride = static_cast<size_t>(p.Hq) * 2;
        float mc = kNegBig;
        for (int s = 0; s < nsplit; ++s) mc = fmaxf(mc, ml[s * stride]);
        float l = 0.f;
        for (int s = 0; s < nsplit; ++s) l += ml[s * stride + 1] * ex2(ml[s * stride] - mc);
        p.ws_lse[static_cast<size_t>(seq) * p.Hq + h] = mc + log2f(l);
    }
}

}  // namespace

bool paged_scores_supported(const b2a_paged_desc& d) {
    const int g = d.Hkv > 0 ? d.Hq / d.Hkv : 0;
    return d.kv_dtype == B2A_U8 && (d.q_dtype == B2A_F16 || d.q_dtype == B2A_BF16) && d.D == kD && d.block_size == kBS &&
           g >= 1 && g <= 8 && d.Hq <= kMaxHq && d.Hq % d.Hkv == 0;
}

// Chunks: about eight CTAs per SM over the step's sequences, at most 128 blocks each.  The chunks are sized for the
// longest admitted context, so a ragged batch leaves some of them empty: cutting finer than the resident CTAs keeps
// the SMs busy all the same (measured on 64 sequences of 512..8192 tokens: 217 us with four per SM, 148 us with
// eight, 150 us with sixteen; 16 x 32768 tokens: 255 / 225 / 229 us), and a CTA walks its blocks once per KV head, so
// it stays long enough.
ScorePlan paged_scores_plan(const b2a_paged_desc& d, int sm_count) {
    const long long nblk_max = std::max<long long>(1, (static_cast<long long>(d.max_context_len) + kBS - 1) / kBS);
    const long long want = std::max<long long>(1, (8LL * sm_count + d.num_seqs - 1) / std::max(1, d.num_seqs));
    long long bpc = (nblk_max + want - 1) / want;
    bpc = std::min<long long>(kMaxBlocksPerCta, std::max<long long>(kWarps, (bpc + kWarps - 1) / kWarps * kWarps));
    ScorePlan plan;
    plan.blocks_per_cta = static_cast<int>(bpc);
    plan.max_splits = static_cast<int>((nblk_max + bpc - 1) / bpc);
    const size_t ml = static_cast<size_t>(d.num_seqs) * plan.max_splits * d.Hq * 2 * sizeof(float);
    const size_t lse = static_cast<size_t>(d.num_seqs) * d.Hq * sizeof(float);
    plan.workspace_bytes = ((ml + 15) & ~static_cast<size_t>(15)) + ((lse + 15) & ~static_cast<size_t>(15));
    return plan;
}

int paged_scores_launch(const b2a_paged_desc& d, const ScorePlan& plan, const void* query, const void* k_cache,
                        const PagedTables& t, float* scores, long long capacity, int32_t* score_begins, void* workspace,
                        int32_t* status, cudaStream_t stream) {
    ScoreParams p{};
    p.query = query;
    p.k_cache = static_cast<const uint8_t*>(k_cache);
    p.t = t;
    p.Hq = d.Hq;
    p.Hkv = d.Hkv;
    p.G = d.Hq / d.Hkv;
    p.blocks_per_cta = plan.blocks_per_cta;
    p.max_splits = plan.max_splits;
    p.max_blocks = static_cast<int>((static_cast<long long>(d.max_context_len) + kBS - 1) / kBS);
    p.sliding_window = d.sliding_window;
    p.scale_log2 = d.scale * kLog2e;
    const size_t ml = static_cast<size_t>(d.num_seqs) * plan.max_splits * d.Hq * 2 * sizeof(float);
    p.ws_ml = static_cast<float*>(workspace);
    p.ws_lse = reinterpret_cast<float*>(static_cast<char*>(workspace) + ((ml + 15) & ~static_cast<size_t>(15)));
    p.score_begins = score_begins;
    p.scores = scores;
    p.capacity = capacity;
    p.status = status;
    const dim3 grid(d.num_seqs, plan.max_splits), block(kWarps * 32);
    const size_t smem = static_cast<size_t>(kWarps) * kStages * kChunk;
    const bool half = d.q_dtype == B2A_F16;
    if (launch_overlapped(score_begins_kernel, dim3(1), dim3(256), 0, stream, p) != cudaSuccess) return B2A_ERR_CUDA;
    if (launch_overlapped(half ? score_pass_kernel<__half, 0> : score_pass_kernel<__nv_bfloat16, 0>, grid, block, smem,
                          stream, p) != cudaSuccess)
        return B2A_ERR_CUDA;
    if (launch_overlapped(score_lse_kernel, dim3(d.num_seqs), dim3(128), 0, stream, p) != cudaSuccess) return B2A_ERR_CUDA;
    if (launch_overlapped(half ? score_pass_kernel<__half, 1> : score_pass_kernel<__nv_bfloat16, 1>, grid, block, smem,
                          stream, p) != cudaSuccess)
        return B2A_ERR_CUDA;
    return B2A_OK;
}

}  // namespace b2a
