// Split-K paged decode over a u8 KV cache: one query token per sequence, D = Dv = 128, 16-token blocks.
//
// The step is bound by HBM: every cached token costs Hkv * 2 * (128 + 4) bytes and a handful of flops.  With
// grouped-query attention the flops are not free, though: G query heads share each K/V byte, and at G = 8 plain
// FP32 FMAs (2*G*128 per token and KV head for QK^T, as many for PV, plus the u8 conversions) need more issue
// slots than the memory system leaves time for.  So the two small contractions run on the warp-level MMA
// (m16n8k16, f16 in, f32 accumulate) with the u8 codes fed in UNSCALED:
//     S[t][g]  = scale_k[t] * ( sum_d code_k[t][d] * Q[g][d]  -  zp_k[t] * sum_d Q[g][d] )
//     O[g][d]  = sum_t P'[g][t] * code_v[t][d]  -  sum_t P'[g][t] * zp_v[t],      P'[g][t] = p[g][t] * scale_v[t]
// Codes 0..255 (and code + 1024, which is what the byte permute produces for free) are exact in f16, products are
// exact, accumulation is f32: the only roundings are the f32 accumulation itself and one f16 rounding of P'.
//
// Grid = (KV head, sequence, split); a CTA of 4 warps walks `blocks_per_cta` logical blocks of one sequence and KV
// head, warp w taking blocks w, w+4, ...  Each warp runs its own 3-stage cp.async pipeline: a stage holds the K chunk
// and the V chunk of one block (2 x 2112 bytes), copied as 16-byte pieces, 512 contiguous bytes per warp
// instruction, into shared memory with an XOR swizzle of the 16-byte column so that the MMA fragments are read
// with conflict-free 128-bit loads.  Online softmax per warp (row max by warp shuffle), partials of the 4 warps
// merged in shared memory, one (m, l, O[G][128]) partial per CTA into the workspace; a second kernel merges the
// splits.  Lengths and tables are read on the device, the grid depends only on max_context_len, so a captured
// launch stays valid when lengths change.  The split index is the slowest grid dimension (full chunks are dispatched
// before partial ones), the cache copies carry an evict-first L2 policy, and the merge kernel is launched
// programmatically dependent.
//
// With the heads sharded over several GPUs the decode kernel also merges and sends (PeerPush in launch.cuh): the
// last CTA of every (sequence, KV head) to finish - a ticket counter in the shard group's memory - merges that
// group's partials and stores the rows into every rank's memory, either as 8-byte {two values, step number} words
// that a small receiving kernel polls and copies to the caller's output, or in place into the ranks' fixed output
// buffers behind a "step begun" / "step published" flag protocol.  No separate merge launch in either form.
#include <atomic>

#include "launch.cuh"

namespace b2a {
namespace {

constexpr int kD = 128;
constexpr int kBS = 16;
constexpr int kChunk = kBS * (kD + 4);   // 2112 bytes: 2048 codes, 16 f16 scales, 16 f16 zero-points
constexpr int kStage = 2 * kChunk;       // K chunk then V chunk
constexpr int kStages = 3;                // copy stages per warp
// Warps per CTA: 4 when the grid fills every SM four CTAs deep (16 warps per SM hide one another's latencies).  A grid
// of at most two CTAs per SM - a head shard of a step - would leave each warp alone with its chain of dependent
// instructions per block (measured: 5.3 TB/s instead of 7), so its CTAs take 8 warps over the same blocks.
constexpr int kWarpsFew = 4, kWarpsMany = 8;
constexpr int smem_bytes(int warps) { return warps * kStages * kStage; }
constexpr float kNegBig = -1.0e30f;      // finite "minus infinity" for the running max (keeps exp2 arguments NaN-free)

struct DecodeParams {
    const void* query;
    const uint8_t* k_cache;
    const uint8_t* v_cache;
    PagedTables t;
    void* out;
    float* ws_o;   // [num_seqs*Hq][max_splits][128]
    float* ws_ml;  // [num_seqs*Hq][max_splits][2]
    int Hq, Hkv, G;
    int blocks_per_cta, max_splits;
    int sliding_window;
    float scale_log2;  // softmax scale * log2(e)
    int32_t* status;
    int beside_predecessor;      // see paged_decode_launch: no wait for the kernel before this one
    int cache_rows_settled;      // b2a_paged_desc: the kernel before this one writes no cache row but the new tokens'
    cudaEvent_t predecessor_done;  // host side only: completes with that kernel
    PeerPush push;     // world == 0 unless the heads are sharded over several GPUs
};

// The cache is read once per step and is far larger than L2: the copies carry an evict-first policy so that the
// lines they bring in are the first to go and the step's small re-used data (queries, tables, partials) stays.
__device__ __forceinline__ uint64_t evict_first_policy() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;\n" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, uint64_t policy) {
    asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "l"(policy) : "memory");
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
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(d) : "r"(a));
    return d;
}
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
// 0x64XX as f16 is 1024 + XX exactly: the MMAs are fed code + 1024 (one byte permute per register, no subtraction)
// and the 1024 joins the zero-point, which is subtracted after the contraction anyway.
constexpr float kCodeBias = 1024.f;
template <int PAIR>
__device__ __forceinline__ uint32_t bytes_to_h2(uint32_t w) {  // (1024 + byte 2*PAIR, 1024 + byte 2*PAIR+1)
    return __byte_perm(w, 0x64646464u, PAIR == 0 ? 0x4140 : 0x4342);
}
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ float h2_lo(uint32_t v) { return __half2float(__ushort_as_half(v & 0xFFFFu)); }
__device__ __forceinline__ float h2_hi(uint32_t v) { return __half2float(__ushort_as_half(v >> 16)); }

// two consecutive query values, as loaded (f16 or bf16 bits), to half2 bits
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

__device__ __forceinline__ int first_block_of(int ctx, int sliding_window) {
    const int first_pos = sliding_window > 0 ? max(0, ctx - sliding_window) : 0;
    return first_pos / kBS;
}

// What a CTA found when it looked at its (sequence, KV head, split).
enum ChunkState {
    kChunkIdle = 0,     // nothing to do: a split past the end of the context (no partial, no ticket)
    kChunkWorked = 1,   // its partial is in the workspace
    kChunkNotRow = 2,   // the sequence is not a one-token decode row (a mixed step's prefill sequence, an idle slot)
    kChunkInvalid = 3   // inconsistent tables (reported)
};

// The walk over this CTA's chunk of one (sequence, KV head).  On kChunkWorked its partial is in the workspace, `nsplit`
// is the number of CTAs of this sequence that write one and `tok` the sequence's token row.  With kRowIsSeq the
// token row must equal the sequence index (the sharded exchange addresses rows by sequence), else kChunkInvalid.
//
// With `wait_for_predecessor` the kernel was launched programmatically dependent on the kernel before it, and its CTAs
// sit on the SMs while that kernel drains.  The walk uses that time for the first two of its three dependent loads:
// the step's tables and this warp's block ids are read BEFORE the wait (the tables of a step exist before its first
// kernel is launched; nothing on this path writes them), through L2 so that no line cached by an earlier step is
// met; so are the first cache blocks of a CTA that does not hold its sequence's last block.  Everything an earlier
// kernel of the step produces - the query rows, the cache rows of the new tokens, the workspace, the status word, the
// exchange's counters - is touched only after the wait.
template <typename T, int NT, bool kRowIsSeq, int kWarps>
__device__ __forceinline__ ChunkState decode_chunk(const DecodeParams& p, uint8_t* smem, int& nsplit, int& tok_out,
                                                   const bool wait_for_predecessor) {
    const int hk = blockIdx.x, seq = blockIdx.y, split = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int gid = lane >> 2, tid4 = lane & 3;

    // A CTA's start is a chain of dependent global loads (tables -> block ids -> cache rows), and in a step that
    // fills the GPU only once nothing hides it.  So the chain is kept as short as it can be: the five table entries
    // are requested together, then the block ids, then the query rows and the first cache stages; the query
    // fragments are put together while those are in flight.
    const int tok = __ldcg(p.t.subsequence_begins + seq);
    const int tok_end = __ldcg(p.t.subsequence_begins + seq + 1);
    const int past = __ldcg(p.t.past_lens + seq);
    const int bib0 = __ldcg(p.t.block_indices_begins + seq);
    const int bib1 = __ldcg(p.t.block_indices_begins + seq + 1);
    const int ctx = past + 1;  // the query token sits at position `past` and sees 0..past
    const int nblk = (ctx + kBS - 1) / kBS;
    const int first_pos = p.sliding_window > 0 ? max(0, ctx - p.sliding_window) : 0;
    const int blk_lo = first_block_of(ctx, p.sliding_window);
    const int my_lo = blk_lo + split * p.blocks_per_cta;
    const int my_hi = min(nblk, my_lo + p.blocks_per_cta);
    ChunkState state = kChunkWorked;
    if (tok_end - tok != 1) state = kChunkNotRow;  // idle sequences, and multi-token sequences of a mixed step (the prefill kernel's)
    else if (past < 0 || nblk > bib1 - bib0 || tok < 0 || tok >= p.t.num_tokens || (kRowIsSeq && tok != seq) ||
             nblk - blk_lo > p.max_splits * p.blocks_per_cta)  // (last: context longer than the max_context_len the grid was sized for)
        state = kChunkInvalid;
    else if (my_lo >= my_hi) state = kChunkIdle;

    // blocks of this warp: my_lo + warp + kWarps*i, i < n_w  (n_w <= 32 because blocks_per_cta <= 128)
    const int n_w = state == kChunkWorked ? (my_hi - my_lo - warp + kWarps - 1) / kWarps : 0;
    int my_phys = 0;
    if (lane < n_w) my_phys = __ldcg(p.t.block_indices + bib0 + my_lo + warp + kWarps * lane);
    const bool bad_block = lane < n_w && (my_phys < 0 || my_phys >= p.t.num_blocks_total);
    if (bad_block) my_phys = -1;

    const uint32_t smem_warp = static_cast<uint32_t>(__cvta_generic_to_shared(smem)) + warp * (kStages * kStage);
    const size_t head_stride = kChunk;                         // chunks of one block: [Hkv][2112]
    const size_t block_stride = static_cast<size_t>(p.Hkv) * kChunk;

    const uint64_t l2_policy = evict_first_policy();
    auto issue = [&](int i) {
        // stage i % kStages <- block i of this warp; an out-of-range physical index copies nothing
        const int phys = __shfl_sync(0xffffffffu, my_phys, i & 31);
        if (phys >= 0) {
            const uint8_t* kc = p.k_cache + phys * block_stride + hk * head_stride;
            const uint8_t* vc = p.v_cache + phys * block_stride + hk * head_stride;
            const uint32_t st = smem_warp + (i % kStages) * kStage;
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int piece = r * 32 + lane;          // 16-byte piece of the 2048 code bytes
                const int row = piece >> 3, col = piece & 7;
                const uint32_t off = row * 128 + ((col ^ (row & 7)) << 4);
                cp_async16(st + off, kc + piece * 16, l2_policy);
                cp_async16(st + kChunk + off, vc + piece * 16, l2_policy);
            }
            if (lane < 4) cp_async16(st + 2048 + lane * 16, kc + 2048 + lane * 16, l2_policy);
            else if (lane < 8) cp_async16(st + kChunk + 2048 + (lane - 4) * 16, vc + 2048 + (lane - 4) * 16, l2_policy);
        }
    };

    // With the caller's promise that the kernel before this one writes no cache row but the new tokens' (each in
    // its sequence's last block), a CTA whose blocks end before that block reads nothing that kernel changes, so its
    // first copy stages also go out before the wait.
    const bool early = wait_for_predecessor && p.cache_rows_settled && state == kChunkWorked && my_hi < nblk;
    if (early) {
#pragma unroll
        for (int s = 0; s < kStages - 1; ++s) {
            if (s < n_w) issue(s);
            cp_async_commit();
        }
    }

    if (wait_for_predecessor) grid_dependency_wait();
    grid_launch_dependents();  // the next kernel's CTAs may take their seats while this grid drains

    if (state == kChunkNotRow) return state;
    if (state == kChunkInvalid) {
        if (tid == 0 && split == 0) report(p.status, B2A_DEV_BAD_LEN);
        return state;
    }
    nsplit = min(p.max_splits, (nblk - blk_lo + p.blocks_per_cta - 1) / p.blocks_per_cta);
    tok_out = tok;
    if (state == kChunkIdle) return state;

    // ---- query rows of this thread's heads as loaded: head nt*8 + gid, elements tid4*32 .. +31 (64 bytes)
    const T* qrow = reinterpret_cast<const T*>(p.query) + (static_cast<size_t>(tok) * p.Hq + hk * p.G) * kD;
    uint4 qraw[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        const int n = nt * 8 + gid;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            qraw[nt][c] = make_uint4(0u, 0u, 0u, 0u);
            if (n < p.G) qraw[nt][c] = reinterpret_cast<const uint4*>(qrow + n * kD + tid4 * 32)[c];
        }
    }

    if (bad_block) report(p.status, B2A_DEV_BAD_BLOCK);

    // ---- pipeline prologue (unless it went out before the wait): the first stages are on their way before the
    // query fragments are put together
    if (!early) {
#pragma unroll
        for (int s = 0; s < kStages - 1; ++s) {
            if (s < n_w) issue(s);
            cp_async_commit();
        }
    }

    // ---- query fragments (B operand of QK^T) and per-head sums of Q
    uint32_t qf[NT][8][2];
    float qsum_a[NT], qsum_b[NT];  // heads nt*8 + 2*tid4 and + 1
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        float part = 0.f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const uint32_t w[4] = {qraw[nt][c].x, qraw[nt][c].y, qraw[nt][c].z, qraw[nt][c].w};
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {  // j = 2c + hf covers elements 4j .. 4j+3 of the thread's 32
                const uint32_t b0 = q_word_to_h2<T>(w[2 * hf]), b1 = q_word_to_h2<T>(w[2 * hf + 1]);
                qf[nt][2 * c + hf][0] = b0;
                qf[nt][2 * c + hf][1] = b1;
                part += h2_lo(b0) + h2_hi(b0) + h2_lo(b1) + h2_hi(b1);
            }
        }
        part += __shfl_xor_sync(0xffffffffu, part, 1);
        part += __shfl_xor_sync(0xffffffffu, part, 2);  // sum of Q[head nt*8+gid][:]
        qsum_a[nt] = __shfl_sync(0xffffffffu, part, 8 * tid4);
        qsum_b[nt] = __shfl_sync(0xffffffffu, part, 8 * tid4 + 4);
    }

    float acc[NT][8][4];
    float m_a[NT], m_b[NT], l_a[NT], l_b[NT], corr_a[NT], corr_b[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        m_a[nt] = m_b[nt] = kNegBig;
        l_a[nt] = l_b[nt] = corr_a[nt] = corr_b[nt] = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[nt][j][0] = acc[nt][j][1] = acc[nt][j][2] = acc[nt][j][3] = 0.f;
    }

    const int sw_k = (gid & 7);  // swizzle key of rows gid and gid+8
    for (int i = 0; i < n_w; ++i) {
        if (i + kStages - 1 < n_w) issue(i + kStages - 1);
        cp_async_commit();
        cp_async_wait<kStages - 1>();
        __syncwarp();

        const uint32_t sK = smem_warp + (i % kStages) * kStage;
        const uint32_t sV = sK + kChunk;
        const int lb = my_lo + warp + kWarps * i;
        const bool blk_ok = __shfl_sync(0xffffffffu, my_phys, i & 31) >= 0;
        const int pos0 = lb * kBS + gid, pos1 = pos0 + 8;
        const bool ok0 = blk_ok && pos0 < ctx && pos0 >= first_pos;
        const bool ok1 = blk_ok && pos1 < ctx && pos1 >= first_pos;

        // ---- S^T = codes_K . Q^T  (rows = tokens gid, gid+8; columns = heads)
        float sc[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f;
        {
            const uint4 x0 = lds128(sK + gid * 128 + (((2 * tid4) ^ sw_k) << 4));
            const uint4 x1 = lds128(sK + gid * 128 + (((2 * tid4 + 1) ^ sw_k) << 4));
            const uint4 y0 = lds128(sK + (gid + 8) * 128 + (((2 * tid4) ^ sw_k) << 4));
            const uint4 y1 = lds128(sK + (gid + 8) * 128 + (((2 * tid4 + 1) ^ sw_k) << 4));
            const uint32_t wl[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
            const uint32_t wh[8] = {y0.x, y0.y, y0.z, y0.w, y1.x, y1.y, y1.z, y1.w};
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint32_t a0 = bytes_to_h2<0>(wl[j]), a1 = bytes_to_h2<0>(wh[j]);
                const uint32_t a2 = bytes_to_h2<1>(wl[j]), a3 = bytes_to_h2<1>(wh[j]);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) mma16816(sc[nt], a0, a1, a2, a3, qf[nt][j][0], qf[nt][j][1]);
            }
        }
        // per-token scale / zero-point (forced to 0 for tokens outside the context: unused slots may hold anything)
        const float sk0 = ok0 ? lds_h(sK + 2048 + 2 * gid) * p.scale_log2 : 0.f;
        const float sk1 = ok1 ? lds_h(sK + 2048 + 2 * (gid + 8)) * p.scale_log2 : 0.f;
        const float zk0 = ok0 ? lds_h(sK + 2048 + 32 + 2 * gid) + kCodeBias : 0.f;
        const float zk1 = ok1 ? lds_h(sK + 2048 + 32 + 2 * (gid + 8)) + kCodeBias : 0.f;
        const float sv0 = ok0 ? lds_h(sV + 2048 + 2 * gid) : 0.f;
        const float sv1 = ok1 ? lds_h(sV + 2048 + 2 * (gid + 8)) : 0.f;
        const float zv0 = ok0 ? lds_h(sV + 2048 + 32 + 2 * gid) + kCodeBias : 0.f;
        const float zv1 = ok1 ? lds_h(sV + 2048 + 32 + 2 * (gid + 8)) + kCodeBias : 0.f;

        uint32_t pb0[NT], pb1[NT];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const float s0 = ok0 ? (sc[nt][0] - zk0 * qsum_a[nt]) * sk0 : -INFINITY;
            const float s1 = ok0 ? (sc[nt][1] - zk0 * qsum_b[nt]) * sk0 : -INFINITY;
            const float s2 = ok1 ? (sc[nt][2] - zk1 * qsum_a[nt]) * sk1 : -INFINITY;
            const float s3 = ok1 ? (sc[nt][3] - zk1 * qsum_b[nt]) * sk1 : -INFINITY;
            float ta = fmaxf(s0, s2), tb = fmaxf(s1, s3);
#pragma unroll
            for (int o = 4; o <= 16; o <<= 1) {
                ta = fmaxf(ta, __shfl_xor_sync(0xffffffffu, ta, o));
                tb = fmaxf(tb, __shfl_xor_sync(0xffffffffu, tb, o));
            }
            const float na = fmaxf(m_a[nt], ta), nb = fmaxf(m_b[nt], tb);
            const float alpha_a = ex2(m_a[nt] - na), alpha_b = ex2(m_b[nt] - nb);
            m_a[nt] = na;
            m_b[nt] = nb;
            const float p0 = ex2(s0 - na), p1 = ex2(s1 - nb), p2 = ex2(s2 - na), p3 = ex2(s3 - nb);
            l_a[nt] = l_a[nt] * alpha_a + p0 + p2;
            l_b[nt] = l_b[nt] * alpha_b + p1 + p3;
            const uint32_t x0 = pack_h2(p0 * sv0, p1 * sv0);  // token gid:   heads a, b
            const uint32_t x1 = pack_h2(p2 * sv1, p3 * sv1);  // token gid+8: heads a, b
            corr_a[nt] = corr_a[nt] * alpha_a + h2_lo(x0) * zv0 + h2_lo(x1) * zv1;
            corr_b[nt] = corr_b[nt] * alpha_b + h2_hi(x0) * zv0 + h2_hi(x1) * zv1;
            pb0[nt] = movmatrix_trans(x0);  // (P'[head gid][token 2*tid4], P'[head gid][token 2*tid4+1])
            pb1[nt] = movmatrix_trans(x1);  // tokens 2*tid4+8, +9
            // the accumulators only need rescaling when some row maximum of the warp moved, which after the first
            // few blocks of a context is rare: skip the 32 multiplications otherwise (warp-uniform branch)
            if (__any_sync(0xffffffffu, alpha_a != 1.f || alpha_b != 1.f)) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    acc[nt][j][0] *= alpha_a;
                    acc[nt][j][1] *= alpha_b;
                    acc[nt][j][2] *= alpha_a;
                    acc[nt][j][3] *= alpha_b;
                }
            }
        }

        // ---- O^T += codes_V^T . P'^T  (rows = d, columns = heads, contraction over the 16 tokens)
        // ldmatrix.trans over byte PAIRS: an 8x8 "b16" matrix is 8 tokens x one 16-byte chunk; transposed, this lane
        // gets (token 2*tid4, token 2*tid4+1) x bytes (2*gid, 2*gid+1) of the chunk in one register, which is the
        // token pairing the A fragment wants.  M-tile j is chunk j: row gid <-> d = 16j+2gid, row gid+8 <-> d+1.
        {
            const int mrow = lane & 7, mh = (lane >> 3) & 1, mc = lane >> 4;  // row, token half and chunk of "my" matrix row
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                uint32_t r0, r1, r2, r3;  // (tokens 0-7, chunk 2q), (8-15, 2q), (0-7, 2q+1), (8-15, 2q+1)
                const uint32_t addr = sV + (8 * mh + mrow) * 128 + (((2 * q + mc) ^ mrow) << 4);
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                             : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                             : "r"(addr));
#pragma unroll
                for (int jj = 0; jj < 2; ++jj) {
                    const uint32_t lo = jj ? r2 : r0, hi = jj ? r3 : r1;
                    const uint32_t a0 = __byte_perm(lo, 0x64646464u, 0x4240);  // d,   tokens t0, t0+1
                    const uint32_t a1 = __byte_perm(lo, 0x64646464u, 0x4341);  // d+1
                    const uint32_t a2 = __byte_perm(hi, 0x64646464u, 0x4240);  // tokens t0+8, t0+9
                    const uint32_t a3 = __byte_perm(hi, 0x64646464u, 0x4341);
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) mma16816(acc[nt][2 * q + jj], a0, a1, a2, a3, pb0[nt], pb1[nt]);
                }
            }
        }
        __syncwarp();  // every lane is done with this stage before it is refilled
    }
    cp_async_wait<0>();
    __syncwarp();

    // ---- warp partial: reduce l and corr over the 8 token rows, park (O - corr, m, l) in this warp's smem
    float* wbuf = reinterpret_cast<float*>(smem + warp * (kStages * kStage));  // [NT*8][128] O, then [NT*8] m, [NT*8] l
    constexpr int GP = NT * 8;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int o = 4; o <= 16; o <<= 1) {
            l_a[nt] += __shfl_xor_sync(0xffffffffu, l_a[nt], o);
            l_b[nt] += __shfl_xor_sync(0xffffffffu, l_b[nt], o);
            corr_a[nt] += __shfl_xor_sync(0xffffffffu, corr_a[nt], o);
            corr_b[nt] += __shfl_xor_sync(0xffffffffu, corr_b[nt], o);
        }
        const int ga = nt * 8 + 2 * tid4, gb = ga + 1;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int d = 16 * j + 2 * gid;
            *reinterpret_cast<float2*>(wbuf + ga * kD + d) =
                make_float2(acc[nt][j][0] - corr_a[nt], acc[nt][j][2] - corr_a[nt]);
            *reinterpret_cast<float2*>(wbuf + gb * kD + d) =
                make_float2(acc[nt][j][1] - corr_b[nt], acc[nt][j][3] - corr_b[nt]);
        }
        if (gid == 0) {
            wbuf[GP * kD + ga] = m_a[nt];
            wbuf[GP * kD + gb] = m_b[nt];
            wbuf[GP * kD + GP + ga] = l_a[nt];
            wbuf[GP * kD + GP + gb] = l_b[nt];
        }
    }
    __syncthreads();

    // ---- merge the warps: thread = (column d, one of the heads taken per round)
    const int d = tid % kD;
    for (int g = tid / kD; g < p.G; g += kWarps * 32 / kD) {
        float mw[kWarps], mc = kNegBig;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            const float* wb = reinterpret_cast<const float*>(smem + w * (kStages * kStage));
            mw[w] = wb[GP * kD + g];
            mc = fmaxf(mc, mw[w]);
        }
        float o = 0.f, l = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            const float* wb = reinterpret_cast<const float*>(smem + w * (kStages * kStage));
            const float f = ex2(mw[w] - mc);
            o += wb[g * kD + d] * f;
            l += wb[GP * kD + GP + g] * f;
        }
        const size_t slot = (static_cast<size_t>(seq) * p.Hq + hk * p.G + g) * p.max_splits + split;
        p.ws_o[slot * kD + d] = o;
        if (d == 0) {
            p.ws_ml[slot * 2] = mc;
            p.ws_ml[slot * 2 + 1] = l;
        }
    }
    return kChunkWorked;
}

__device__ __forceinline__ void st_release_sys(int32_t* p, int32_t v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int32_t ld_acquire_sys(const int32_t* p) {
    int32_t v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// wall-clock nanoseconds: waits on other GPUs are bounded in real time, whatever the SM clock does
__device__ __forceinline__ long long global_ns() {
    long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

template <typename T>
__device__ __forceinline__ uint32_t pack2(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
    return pack_h2(a, b);
}
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// Bounded wait on `n` flags (one thread per flag) until each shows `epoch`; B2A_DEV_TIMEOUT after `limit_ns`.
__device__ __forceinline__ void wait_flags(const int32_t* flags, int n, int32_t epoch, long long limit_ns, int32_t* status) {
    if (static_cast<int>(threadIdx.x) < n) {
        const int32_t* flag = flags + threadIdx.x;
        const long long t0 = global_ns();
        while (ld_acquire_sys(flag) - epoch < 0) {
            if (global_ns() - t0 > limit_ns) {
                report(status, B2A_DEV_TIMEOUT);
                break;
            }
        }
    }
}

// Merge of the split partials of one (sequence, KV head) by the CTA that finished last, and delivery of the rows.
// kDims consecutive output columns per thread (4: 32 threads per head, four heads per round; 8: 16 threads per head,
// eight heads per round - taken for groups of more than four heads so that one round covers the group).  The
// partials come from L2 (other CTAs wrote them); eight splits are requested at a time before any is used.  The
// arithmetic is that of paged_decode_merge_kernel, operation for operation (maximum over all splits first, then the
// weighted sums in split order, one division per value), so a sharded step gives the bits of the single-GPU path.
//   kLL  : every pair of 16-bit values travels as one 8-byte store {two values, step number} into staging[r][parity]
//          of every rank r; such a store arrives whole or not at all, so the receiver simply polls the word.
//   !kLL : the rows are stored as they are - into staging[r][0] of every rank (the ranks' fixed output buffers), or,
//          without a group, into the caller's output.
template <typename T, int kDims, bool kLL, int kWarps>
__device__ __forceinline__ void merge_and_deliver(const DecodeParams& p, int seq, int hk, int tok, int nsplit,
                                                  int32_t epoch) {
    constexpr int kVec = kDims / 4;            // float4 loads per split
    constexpr int kLanes = kD / kDims;         // threads per head
    constexpr int kHeadsPerRound = (kWarps * 32) / kLanes;
    constexpr int kBatch = 8;
    const int tid = threadIdx.x;
    const int d0 = (tid % kLanes) * kDims;
    for (int g = tid / kLanes; g < p.G; g += kHeadsPerRound) {
        const int h = hk * p.G + g;
        const size_t base = (static_cast<size_t>(seq) * p.Hq + h) * p.max_splits;
        const float2* mlp = reinterpret_cast<const float2*>(p.ws_ml) + base;
        float l = 0.f, o[kDims];
#pragma unroll
        for (int i = 0; i < kDims; ++i) o[i] = 0.f;
        float2 ml[kBatch];
        float4 v[kBatch][kVec];
        auto load_batch = [&](int s0) {
#pragma unroll
            for (int i = 0; i < kBatch; ++i) {
                const int sp = min(s0 + i, nsplit - 1);  // the tail repeats the last split (dropped below)
                ml[i] = __ldcg(mlp + sp);
#pragma unroll
                for (int q = 0; q < kVec; ++q)
                    v[i][q] = __ldcg(reinterpret_cast<const float4*>(p.ws_o + (base + sp) * kD + d0) + q);
            }
        };
        load_batch(0);
        float mc = kNegBig;
#pragma unroll
        for (int i = 0; i < kBatch; ++i) mc = fmaxf(mc, ml[i].x);
#pragma unroll 8
        for (int sp = kBatch; sp < nsplit; ++sp) mc = fmaxf(mc, __ldcg(mlp + sp).x);
        for (int s0 = 0; s0 < nsplit; s0 += kBatch) {
            if (s0 > 0) load_batch(s0);
#pragma unroll
            for (int i = 0; i < kBatch; ++i) {
                if (s0 + i < nsplit) {
                    const float f = ex2(ml[i].x - mc);
                    l += ml[i].y * f;
#pragma unroll
                    for (int q = 0; q < kVec; ++q) {
                        o[4 * q + 0] += v[i][q].x * f;
                        o[4 * q + 1] += v[i][q].y * f;
                        o[4 * q + 2] += v[i][q].z * f;
                        o[4 * q + 3] += v[i][q].w * f;
                    }
                }
            }
        }
        const bool nz = l > 0.f;
        uint32_t w[kDims / 2];
#pragma unroll
        for (int i = 0; i < kDims / 2; ++i) w[i] = pack2<T>(nz ? o[2 * i] / l : 0.f, nz ? o[2 * i + 1] / l : 0.f);
        if constexpr (kLL) {
            const size_t at = (static_cast<size_t>(seq) * p.push.row_elems + p.push.col_offset + h * kD + d0) >> 1;
            const int parity = epoch & 1;
            for (int r = 0; r < p.push.world; ++r) {
                uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint2*>(p.push.staging[r][parity]) + at);
#pragma unroll
                for (int q = 0; q < kDims / 4; ++q)
                    dst[q] = make_uint4(w[2 * q], static_cast<uint32_t>(epoch), w[2 * q + 1], static_cast<uint32_t>(epoch));
            }
        } else if (p.push.world > 0) {
            const size_t at = static_cast<size_t>(tok) * p.push.row_elems + p.push.col_offset + h * kD + d0;
            for (int r = 0; r < p.push.world; ++r) {
                uint2* dst = reinterpret_cast<uint2*>(reinterpret_cast<T*>(p.push.staging[r][0]) + at);
#pragma unroll
                for (int q = 0; q < kDims / 4; ++q) dst[q] = make_uint2(w[2 * q], w[2 * q + 1]);
            }
        } else {
            uint2* dst = reinterpret_cast<uint2*>(reinterpret_cast<T*>(p.out) + (static_cast<size_t>(tok) * p.Hq + h) * kD + d0);
#pragma unroll
            for (int q = 0; q < kDims / 4; ++q) dst[q] = make_uint2(w[2 * q], w[2 * q + 1]);
        }
    }
}

// Low-latency form, a sequence whose row cannot be computed (inconsistent tables: reported): every rank's receiver
// still waits for the row's words, so zeros are sent in their place.
__device__ __forceinline__ void send_zero_row_segment(const DecodeParams& p, int seq, int hk, int32_t epoch) {
    const int words = p.G * kD / 2;  // 8-byte words of this KV head's segment of the row
    const size_t at = (static_cast<size_t>(seq) * p.push.row_elems + p.push.col_offset + hk * p.G * kD) >> 1;
    const uint2 word = make_uint2(0u, static_cast<uint32_t>(epoch));
    for (int r = 0; r < p.push.world; ++r) {
        uint2* dst = reinterpret_cast<uint2*>(p.push.staging[r][epoch & 1]) + at;
        for (int i = threadIdx.x; i < words; i += blockDim.x) dst[i] = word;
    }
}

// Receiving side of the low-latency exchange for one output row: poll every 8-byte word of the row in this rank's
// staging buffer until it carries the step's number (bounded in real time: B2A_DEV_TIMEOUT after push.wait_ns) and
// write the value pairs to the caller's output.  Two words per load (rows are multiples of 256 bytes).
__device__ __forceinline__ void receive_row(const PeerPush& push, uint32_t* out, int row, uint32_t epoch, int32_t* status) {
    const int pairs_per_row = push.row_elems / 2;
    const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const uint2*>(push.staging[push.rank][epoch & 1]) +
                                                      static_cast<size_t>(row) * pairs_per_row);
    uint2* dst = reinterpret_cast<uint2*>(out + static_cast<size_t>(row) * pairs_per_row);
    const long long t0 = global_ns();
    bool gave_up = false;
    for (int i = threadIdx.x; i < pairs_per_row / 2; i += blockDim.x) {
        uint32_t a, ea, b, eb;
        for (;;) {
            asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(a), "=r"(ea), "=r"(b), "=r"(eb)
                         : "l"(src + i)
                         : "memory");
            if ((ea == epoch && eb == epoch) || gave_up) break;
            if (global_ns() - t0 > push.wait_ns) {
                report(status, B2A_DEV_TIMEOUT);
                gave_up = true;
            }
        }
        dst[i] = make_uint2(a, b);
    }
}

// kMode 0: the CTA leaves its partial in the workspace and paged_decode_merge_kernel follows (single GPU).
// kMode 1, 2: the whole step of a head shard in this launch (PeerPush).  After its chunk a CTA takes a ticket of its
// (sequence, KV head); the CTA that gets the last ticket merges the group's partials and delivers the rows to every
// rank - mode 1 as low-latency words for the receiving kernel, mode 2 in place: there the rows land in the ranks'
// fixed output buffers, so a rank first announces that it has begun the step (its readers of the previous output are
// done), nobody stores before every rank has, and the grid's last CTA publishes the step and waits for the other
// ranks' steps, so that the output is complete on this rank when the kernel ends.
template <typename T, int NT, int kMode, int kWarps>
__global__ void __launch_bounds__(kWarps * 32, 16 / kWarps) paged_decode_kernel(const DecodeParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    int nsplit = 0, tok = 0;
    // the cache rows of this step's new tokens and the query come from earlier kernels: decode_chunk waits for them
    // after its table walk (beside the prefill kernel of a mixed step there is nothing to wait for: that kernel waited
    // for them already and is not waited for itself)
    const bool wait_for_predecessor = !p.beside_predecessor;
    if constexpr (kMode == 0) {
        decode_chunk<T, NT, false, kWarps>(p, smem, nsplit, tok, wait_for_predecessor);
    } else {
        constexpr bool kLL = kMode == 1;
        __shared__ int s_role;
        const int tid = threadIdx.x, hk = blockIdx.x, seq = blockIdx.y;
        int32_t epoch = 0;
        if constexpr (!kLL) {
            // in place: the other ranks hold their stores back until this rank says that the readers of its previous
            // step are done, so that is said as early as it is true - before the walk, hence after a wait of its own
            if (wait_for_predecessor) grid_dependency_wait();
            epoch = *reinterpret_cast<volatile int32_t*>(p.push.step_counter) + 1;
            if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && tid < p.push.world)
                st_release_sys(p.push.started[tid] + p.push.rank, epoch);
        }
        const ChunkState state = decode_chunk<T, NT, kLL, kWarps>(p, smem, nsplit, tok, kLL && wait_for_predecessor);
        if constexpr (kLL) epoch = *reinterpret_cast<volatile int32_t*>(p.push.step_counter) + 1;  // (after the walk's wait)
        if (tid == 0) s_role = 0;
        __syncthreads();  // (the role starts cleared for everybody;) every thread's part of the partial is written ...
        if (state == kChunkWorked) {
            if (tid == 0) {
                // ... and, through the barrier, ordered before this thread's ticket: one acquire-release add (the
                // release publishes this CTA's partial, the acquire of the last ticket sees everybody else's)
                int32_t* ctr = p.push.group_counters + seq * p.Hkv + hk;
                int32_t before;
                asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(before) : "l"(ctr) : "memory");
                const bool last = before == nsplit - 1;
                if (last) *ctr = 0;
                s_role = last ? 1 : 0;
            }
            __syncthreads();
            if (s_role == 1) {
                if (!kLL) {
                    wait_flags(p.push.started[p.push.rank], p.push.world, epoch, p.push.wait_ns, p.status);  // every rank has begun this step
                    __syncthreads();
                }
                // columns per thread such that one round covers a group of up to eight heads where the CTA has the threads
                if constexpr (kWarps == kWarpsFew) {
                    if (p.G > 4) merge_and_deliver<T, 8, kLL, kWarps>(p, seq, hk, tok, nsplit, epoch);
                    else merge_and_deliver<T, 4, kLL, kWarps>(p, seq, hk, tok, nsplit, epoch);
                } else {
                    merge_and_deliver<T, 4, kLL, kWarps>(p, seq, hk, tok, nsplit, epoch);
                }
                if (!kLL) __threadfence_system();  // this CTA's peer stores before its arrival below
            }
        } else if (kLL && (state == kChunkInvalid || state == kChunkNotRow) && blockIdx.z == 0) {
            if (state == kChunkNotRow && tid == 0) report(p.status, B2A_DEV_BAD_LEN);
            send_zero_row_segment(p, seq, hk, epoch);
            if (tid == 0) s_role = 1;  // (stands in for the merging CTA of a row that cannot be computed)
            __syncthreads();
        }
        if constexpr (kLL) {
            // One launch for the whole step: the CTA that delivered the first KV head's part of a row also receives
            // the row - it waits for the other KV heads' CTAs of this grid and for the other ranks, which never wait
            // for it, and there are at most as many such CTAs as SMs (the host checks), so every CTA they wait for
            // finds a place to run.  The last receiver counts the step.
            if (p.push.receive_in_kernel && hk == 0 && s_role == 1) {
                receive_row(p.push, static_cast<uint32_t*>(p.out), seq, static_cast<uint32_t>(epoch), p.status);
                __syncthreads();
                if (tid == 0 && atomicAdd(p.push.done_counter, 1) == static_cast<int>(gridDim.y) - 1) {
                    *p.push.done_counter = 0;
                    *reinterpret_cast<volatile int32_t*>(p.push.step_counter) = epoch;
                }
            }
        }
        if constexpr (!kLL) {
            // in place: the grid's last CTA publishes the step on every rank and waits for theirs
            __syncthreads();
            if (tid == 0) {
                const int total = static_cast<int>(gridDim.x * gridDim.y * gridDim.z);
                const bool last = atomicAdd(p.push.done_counter, 1) == total - 1;
                if (last) {
                    *p.push.done_counter = 0;  // every CTA has arrived: ready for the next step
                    *reinterpret_cast<volatile int32_t*>(p.push.step_counter) = epoch;
                    __threadfence_system();
                    for (int r = 0; r < p.push.world; ++r) st_release_sys(p.push.flags[r] + p.push.rank, epoch);
                }
                s_role = last ? 2 : 0;
            }
            __syncthreads();
            if (s_role == 2) wait_flags(p.push.flags[p.push.rank], p.push.world, epoch, p.push.wait_ns, p.status);
        }
        // (low-latency form: nothing to publish - the words carry the step number, and the receiving kernel, which
        // is the step's last, counts the step)
    }
}

// Merge the split partials of one (sequence, query head): out = sum_s O_s 2^(m_s - m) / sum_s l_s 2^(m_s - m) with
// m = max_s m_s.  The (m, l) pairs are read as 8-byte loads and both loops are unrolled so that eight partials are in
// flight per thread (the loads are independent; only the tiny accumulation is a chain).
template <typename T>
__global__ void __launch_bounds__(kD) paged_decode_merge_kernel(const DecodeParams p) {
    const int h = blockIdx.x, seq = blockIdx.y, d = threadIdx.x;
    // the step's tables are read while the decode kernel drains (see decode_chunk), the partials after the wait
    const int tok = __ldcg(p.t.subsequence_begins + seq);
    const int qlen = __ldcg(p.t.subsequence_begins + seq + 1) - tok;
    const int past = __ldcg(p.t.past_lens + seq);
    const int nblk_have = __ldcg(p.t.block_indices_begins + seq + 1) - __ldcg(p.t.block_indices_begins + seq);
    grid_dependency_wait();
    grid_launch_dependents();
    const int ctx = past + 1;
    const int nblk = (ctx + kBS - 1) / kBS;
    const int blk_lo = first_block_of(ctx, p.sliding_window);
    // the same conditions under which the decode kernel wrote partials
    const bool valid = qlen == 1 && past >= 0 && tok >= 0 && tok < p.t.num_tokens && nblk <= nblk_have &&
                       nblk - blk_lo <= p.max_splits * p.blocks_per_cta;
    if (!valid) return;
    const int nsplit = min(p.max_splits, (nblk - blk_lo + p.blocks_per_cta - 1) / p.blocks_per_cta);
    const size_t base = (static_cast<size_t>(seq) * p.Hq + h) * p.max_splits;
    const float2* ml = reinterpret_cast<const float2*>(p.ws_ml) + base;
    // the first sixteen splits (all of them, for the chunk plans in use) are requested at once, (m, l) and values
    // alike, so that the merge costs one trip to L2 instead of two; the arithmetic keeps its order
    constexpr int kFirst = 16;
    float2 mlv[kFirst];
    float ov[kFirst];
#pragma unroll
    for (int i = 0; i < kFirst; ++i) {
        const int sp = min(i, nsplit - 1);  // (the tail repeats the last split: dropped below)
        mlv[i] = ml[sp];
        ov[i] = p.ws_o[(base + sp) * kD + d];
    }
    float mc = kNegBig;
#pragma unroll
    for (int i = 0; i < kFirst; ++i) mc = fmaxf(mc, mlv[i].x);
#pragma unroll 8
    for (int s = kFirst; s < nsplit; ++s) mc = fmaxf(mc, ml[s].x);
    float o = 0.f, l = 0.f;
#pragma unroll
    for (int i = 0; i < kFirst; ++i) {
        if (i < nsplit) {
            const float f = ex2(mlv[i].x - mc);
            o += ov[i] * f;
            l += mlv[i].y * f;
        }
    }
#pragma unroll 8
    for (int s = kFirst; s < nsplit; ++s) {
        const float2 v = ml[s];
        const float f = ex2(v.x - mc);
        o += p.ws_o[(base + s) * kD + d] * f;
        l += v.y * f;
    }
    T* orow = reinterpret_cast<T*>(p.out) + (static_cast<size_t>(tok) * p.Hq + h) * kD;
    orow[d] = from_f32<T>(l > 0.f ? o / l : 0.f);
}

// Receiver of the low-latency exchange as a kernel of its own, one CTA per row, for steps with more rows than the
// decode kernel may hold waiting CTAs for.  It is the last kernel of the step, so its last CTA counts the step: the
// decode kernel before it and this kernel read the same counter value.
__global__ void __launch_bounds__(256) peer_ll_copy_kernel(const PeerPush push, uint32_t* out, int32_t* status) {
    grid_dependency_wait();  // our own decode kernel (its CTAs read the step counter that this kernel advances)
    grid_launch_dependents();
    const uint32_t epoch = static_cast<uint32_t>(*reinterpret_cast<volatile int32_t*>(push.step_counter) + 1);
    receive_row(push, out, blockIdx.x, epoch, status);
    __syncthreads();
    if (threadIdx.x == 0) {
        if (atomicAdd(push.done_counter, 1) == static_cast<int>(gridDim.x) - 1) {
            *push.done_counter = 0;
            *reinterpret_cast<volatile int32_t*>(push.step_counter) = static_cast<int32_t>(epoch);
        }
    }
}

template <typename T, int NT, int kMode, int kWarps>
int launch_kernel_w(const DecodeParams& p, int num_seqs, cudaStream_t stream) {
    auto kern = paged_decode_kernel<T, NT, kMode, kWarps>;
    static std::atomic<bool> configured[64];  // per device; setting the attribute twice is harmless
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return B2A_ERR_CUDA;
    if (dev < 0 || dev >= 64 || !configured[dev].load(std::memory_order_acquire)) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes(kWarps)) != cudaSuccess)
            return B2A_ERR_CUDA;
        if (dev >= 0 && dev < 64) configured[dev].store(true, std::memory_order_release);
    }
    // the split index is the slowest-varying one: every sequence's first chunks (always full) are dispatched before
    // anybody's last chunk (partial or empty), which shortens the tail of a step with uneven contexts
    dim3 grid(p.Hkv, num_seqs, p.max_splits);
    return launch_overlapped(kern, grid, dim3(kWarps * 32), smem_bytes(kWarps), stream, p) == cudaSuccess ? B2A_OK
                                                                                                             : B2A_ERR_CUDA;
}

template <typename T, int NT, int kMode>
int launch_kernel(const DecodeParams& p, int num_seqs, cudaStream_t stream) {
    const long long ctas = static_cast<long long>(p.Hkv) * num_seqs * p.max_splits;
    const int sms = device_sm_count();
    if constexpr (NT == 1) {  // (groups of more than eight query heads keep the one variant)
        if (sms > 0 && ctas <= 2LL * sms) return launch_kernel_w<T, NT, kMode, kWarpsMany>(p, num_seqs, stream);
    }
    return launch_kernel_w<T, NT, kMode, kWarpsFew>(p, num_seqs, stream);
}

template <typename T, int NT>
int launch_t(const DecodeParams& p, int num_seqs, cudaStream_t stream) {
    if (p.push.world > 0) {
        if (!p.push.ll) return launch_kernel<T, NT, 2>(p, num_seqs, stream);
        const int rc = launch_kernel<T, NT, 1>(p, num_seqs, stream);
        if (rc != B2A_OK || p.push.receive_in_kernel) return rc;
        // decode steps carry one token per sequence: row index == sequence index == token index
        return launch_overlapped(peer_ll_copy_kernel, dim3(num_seqs), dim3(256), 0, stream, p.push,
                                 static_cast<uint32_t*>(p.out), p.status) == cudaSuccess
                   ? B2A_OK
                   : B2A_ERR_CUDA;
    }
    const int rc = launch_kernel<T, NT, 0>(p, num_seqs, stream);
    if (rc != B2A_OK) return rc;
    if (p.beside_predecessor) {
        // an ordinary launch behind a wait for the prefill kernel: it starts when the decode kernel AND the kernel it
        // ran beside have completed, which closes the step for whatever comes next on the stream
        if (cudaStreamWaitEvent(stream, p.predecessor_done, 0) != cudaSuccess) return B2A_ERR_CUDA;
        paged_decode_merge_kernel<T><<<dim3(p.Hq, num_seqs), dim3(kD), 0, stream>>>(p);
        return cudaGetLastError() == cudaSuccess ? B2A_OK : B2A_ERR_CUDA;
    }
    return launch_overlapped(paged_decode_merge_kernel<T>, dim3(p.Hq, num_seqs), dim3(kD), 0, stream, p) == cudaSuccess
               ? B2A_OK
               : B2A_ERR_CUDA;
}

}  // namespace

bool paged_decode_geometry_ok(const b2a_paged_desc& d) {
    const int g = d.Hkv > 0 ? d.Hq / d.Hkv : 0;
    return d.kv_dtype == B2A_U8 && (d.q_dtype == B2A_F16 || d.q_dtype == B2A_BF16) && d.D == kD && d.Dv == kD &&
           d.block_size == kBS && g >= 1 && g <= 16;
}

bool paged_decode_supported(const b2a_paged_desc& d) {
    return paged_decode_geometry_ok(d) && d.max_q_len == 1 && d.num_tokens == d.num_seqs;
}

DecodePlan paged_decode_plan(const b2a_paged_desc& d, int sm_count) {
    // Long chunks win (a CTA's pipeline start and its merge are paid once per chunk), so a CTA walks up to 128
    // blocks - 32 per warp, the size of a warp's block-id window.  Only when the whole step is smaller than one
    // wave of 4 CTAs per SM are the chunks shortened, so that every SM still has work.
    const long long nblk_max = (static_cast<long long>(d.max_context_len) + kBS - 1) / kBS;
    const long long total = nblk_max * d.Hkv * d.num_seqs;
    const long long target_ctas = static_cast<long long>(sm_count) * 4;
    long long bpc = (total + target_ctas - 1) / target_ctas;
    bpc = ((bpc + 3) / 4) * 4;
    if (bpc < 96) {
        // A small step (a head shard, say) cannot fill every slot with long chunks.  Short chunks are fine while a
        // sequence is cut into few of them, but every split costs a pipeline start, a partial and merge work:
        // measured on one KV head, 16 x 32768 tokens take 37 us as 37 splits of 56 blocks and 31 us as 16 splits of
        // 128, while 64 ragged sequences of at most 8192 tokens are fastest with their 56-block chunks (10 splits).
        // So a sequence is cut into at most 16 chunks.
        const long long floor_bpc = ((nblk_max + 15) / 16 + 3) / 4 * 4;
        if (bpc < floor_bpc) bpc = floor_bpc;
    }
    if (bpc < 16) bpc = 16;
    if (bpc > 128) bpc = 128;
    DecodePlan plan;
    plan.blocks_per_cta = static_cast<int>(bpc);
    plan.max_splits = static_cast<int>((nblk_max + bpc - 1) / bpc);
    if (plan.max_splits < 1) plan.max_splits = 1;
    plan.workspace_bytes = static_cast<size_t>(d.num_seqs) * d.Hq * plan.max_splits * (kD + 2) * sizeof(float);
    return plan;
}

int paged_decode_launch(const b2a_paged_desc& d, const DecodePlan& plan, const void* query, const void* k_cache,
                        const void* v_cache, const PagedTables& t, void* out, void* workspace, int32_t* status,
                        cudaStream_t stream, const PeerPush* push, cudaEvent_t beside_predecessor) {
    DecodeParams p{};
    if (push != nullptr) p.push = *push;
    // the rows are received by CTAs of the decode kernel itself while there are no more rows than SMs
    if (push != nullptr && p.push.ll) p.push.receive_in_kernel = d.num_seqs <= device_sm_count() ? 1 : 0;
    p.beside_predecessor = beside_predecessor != nullptr && push == nullptr ? 1 : 0;
    p.predecessor_done = beside_predecessor;
    p.query = query;
    p.k_cache = static_cast<const uint8_t*>(k_cache);
    p.v_cache = static_cast<const uint8_t*>(v_cache);
    p.t = t;
    p.out = out;
    const size_t rows = static_cast<size_t>(d.num_seqs) * d.Hq * plan.max_splits;
    p.ws_o = static_cast<float*>(workspace);
    p.ws_ml = p.ws_o + rows * kD;
    p.Hq = d.Hq;
    p.Hkv = d.Hkv;
    p.G = d.Hq / d.Hkv;
    p.blocks_per_cta = plan.blocks_per_cta;
    p.max_splits = plan.max_splits;
    p.sliding_window = d.sliding_window;
    p.cache_rows_settled = d.cache_rows_settled;
    p.scale_log2 = d.scale * kLog2e;
    p.status = status;
    const bool two = p.G > 8;
    if (d.q_dtype == B2A_F16) return two ? launch_t<__half, 2>(p, d.num_seqs, stream) : launch_t<__half, 1>(p, d.num_seqs, stream);
    return two ? launch_t<__nv_bfloat16, 2>(p, d.num_seqs, stream) : launch_t<__nv_bfloat16, 1>(p, d.num_seqs, stream);
}

// ---- decode with built-in scratch ---------------------------------------------------------------------------
//
// Split-K partials for callers that have nowhere to get a workspace from: the array below is part of the
// library image, so every GPU that loads libb2a.so carries these 16 MiB until the process exits, and nothing is
// allocated at call time.  One array per device, shared by every call on that device: two calls that overlap on
// the GPU (different streams, or graph branches) would write each other's partials, so such calls must be ordered.
// Nothing in it has to start at zero: every partial the merge kernel reads is written by the decode kernel of the
// same call, which is why no clearing is issued.
static __device__ __align__(256) unsigned char g_decode_scratch[B2A_BUILTIN_SCRATCH_BYTES];

int paged_decode_launch_builtin_scratch(const b2a_paged_desc& d, const DecodePlan& plan, const void* query,
                                        const void* k_cache, const void* v_cache, const PagedTables& t, void* out,
                                        int32_t* status, cudaStream_t stream) {
    if (plan.workspace_bytes > static_cast<size_t>(B2A_BUILTIN_SCRATCH_BYTES)) return B2A_ERR_SCRATCH_LIMIT;
    // `g_decode_scratch` as written in host code is only a handle for the runtime; the address the kernels can
    // use is looked up once per device, with that device current, and remembered (several host threads may get
    // here at once: they would all store the same value).  The remembered address does not survive a
    // cudaDeviceReset of that device.
    static std::atomic<void*> device_address[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return B2A_ERR_CUDA;
    void* scratch = (dev >= 0 && dev < 64) ? device_address[dev].load(std::memory_order_acquire) : nullptr;
    if (scratch == nullptr) {
        if (cudaGetSymbolAddress(&scratch, g_decode_scratch) != cudaSuccess || scratch == nullptr) return B2A_ERR_CUDA;
        if (dev >= 0 && dev < 64) device_address[dev].store(scratch, std::memory_order_release);
    }
    return paged_decode_launch(d, plan, query, k_cache, v_cache, t, out, scratch, status, stream);
}

}  // namespace b2a
