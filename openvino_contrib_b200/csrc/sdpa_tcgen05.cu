// Fused attention for prefill on the 5th-generation tensor core: S = Q K^T and O = P V as tcgen05.mma with
// accumulators in tensor memory, online softmax in registers.  f16 / bf16, D = Dv = 128, grouped-query heads.
// Three front ends share one kernel body (template parameter kMode):
//   0 dense  (ScaledDotProductAttention): Q, K, V are [B, H, S, 128] tensors, causal or unmasked; K/V tiles are
//     staged by TMA;
//   1 paged, de-quantising in the kernel (PagedAttentionExtension, sequences with two or more new tokens): Q rows
//     come from the step's [tokens, Hq*128] matrix, K/V from the u8 block pool through the block table - a producer
//     warpgroup de-quantises 128-token tiles ((code - zp) * scale in float32, rounded once to f16: queries, keys,
//     values and P are all f16 in the paged modes) straight into the swizzled shared-memory layout the tensor core
//     reads;
//   2 paged, gathered: paged_gather_kernel has de-quantised the contexts of the step's multi-token sequences once
//     into an f16 scratch (a row range per sequence), and K/V tiles are staged from there by TMA like dense ones.
//     Taken when the caller passes the scheduler's bound on those contexts (b2a_paged_desc.prefill_kv_tokens).
//   In the paged modes query token i of a sequence sees cache positions 0 .. past_len + i, or only the last
//   `sliding_window` of them: an item then starts at the first key tile that any of its rows still sees, and key
//   tiles that begin below the window of a tile's last row are masked at their low edge like diagonal tiles at
//   their high edge.
//
// Work is cut into items: TWO 128-row query tiles of one KV head, walked over the keys 128 at a time.  CTAs are
// persistent (one per SM; mode 1 keeps one item per CTA): the items, heaviest first, are dealt in snake order.
//   warps 0-3   softmax of tile A: thread = query row = TMEM lane.  Reads S_A (tcgen05.ld), keeps the running max
//               and sum, writes P_A = exp2(S*c - m) as 16-bit pairs over the first half of S_A's columns
//               (tcgen05.st) and signals the MMA issuer after the first 64 keys and again after all 128; rescales
//               O_A in TMEM when the maximum moved; finally normalises O_A and stores it (dense: through a
//               staging slab per warp - [32 x 64] and one TMA tensor store per slab, to every rank's buffer when the
//               heads are sharded over two ranks; pieces of 16 full rows and one bulk store per rank from four ranks
//               on; paged: row-wise stores).
//   warps 4-7   the same for tile B.
//   warp  8     TMA producer (one lane): the Q tiles of an item as soon as the previous item's last QK^T has
//               completed, and (modes 0, 2) K_j and V_j into two-stage rings that run on across items.
//   warp  9     MMA issuer (one lane): S_X(j) = Q_X K_j^T (A and B from shared memory, K-major, 128-byte swizzle),
//               O_X += P_X(j) V_j (A from TMEM, B from shared memory, MN-major).  Order per step:
//               PV_A(j), QK_A(j+1), PV_B(j), QK_B(j+1) - while one tile's softmax runs, the tensor core works on
//               the other tile.  Descriptors are put together at the point of issue (tcgen05.cuh) so the thread
//               stays within its 56 registers.  The warp also owns the TMEM allocation (all 512 columns: S_A S_B
//               O_A O_B).
//   warps 10-11 complete the service warpgroup whose registers are handed to the softmax groups; in mode 2 with
//               bf16 queries they convert the Q tiles to f16 in shared memory.
//   warps 12-15 mode 1 only: the de-quantising K/V producers.
// The two tiles are consecutive entries of the list (row block, query head of the group), query heads fastest, so
// with an even group size both tiles cover the same rows of two heads that share K/V, and the causal structure of
// the pair is identical.
//
// The maximum used for P is allowed to lag: O and the sum are rescaled only when some row's maximum grew by more
// than 2^8, so P stays below 256 and the result is exact after the final division.
//
// Every mbarrier wait is bounded (tcgen05.cuh); on a timeout the CTA raises an abort flag, all roles leave their
// loops, outstanding copies and MMAs are drained with bounded waits, TMEM is freed and the status word gets
// B2A_DEV_TIMEOUT.  All barrier phases are derived from running counts (K/V ring position, steps of a tile, Q tiles
// loaded) so that they carry over from one item to the next.
#include "launch.cuh"
#include "tcgen05.cuh"

namespace b2a {
namespace {

using namespace tc;

constexpr int kBM = 128;             // query rows per tile = TMEM lanes
constexpr int kBN = 128;             // keys per step
constexpr int kHeadDim = 128;
constexpr int kPanel = 128 * 128;    // bytes of one [128 rows x 64 elements] swizzled panel
constexpr int kTile = 2 * kPanel;    // a [128 x 128] 16-bit tile
constexpr int kThreadsDense = 384;   // 3 warpgroups: softmax A, softmax B, {producer, MMA issuer, 2 idle warps}
constexpr int kThreadsPaged = 512;   // plus the de-quantising producer warpgroup
constexpr int kNumBars = 23;
constexpr int kStageOut = 8 * 4096;  // epilogue staging: one [32 rows x 64 elements] slab per softmax warp
constexpr int kSmemBytes = 6 * kTile + kStageOut + 1024 /* alignment slack */ + 256 /* barriers, TMEM slot, abort flag */;
constexpr float kLazyThreshold = 8.0f;  // log2 units
constexpr int kCacheChunk = 16 * (kHeadDim + 4);  // bytes of one (block, KV head) chunk of the u8 pool

enum Bar { Q_FULL = 0, K_FULL = 2, K_EMPTY = 4, V_FULL = 6, V_EMPTY = 8, S_FULL = 10, P_READY = 12, O_DONE = 14, DRAIN = 16, P_HALF = 17, Q_CONV = 19, Q_EMPTY = 21 };

struct TcParams {
    int B, Hq, Hkv, G, Sq, Skv;
    int causal;
    int window;  // paged modes: a query at position p sees keys p - window + 1 .. p (0: all of them)
    float scale_log2;
    // dense mode with an attention mask (kMask 1: u8, non-zero keeps; 2: additive, the tensors' 16-bit type):
    // logical [B, Hq, Sq, Skv] with element strides mask_strides[0..2] (0 on broadcast dimensions), innermost 1
    const uint8_t* mask;
    int64_t mask_strides[3];
    int32_t* status;
    // paged mode
    const uint8_t* k_cache;
    const uint8_t* v_cache;
    PagedTables t;
    void* out;        // [tokens, Hq*128]
    const int* plan;  // work list built by paged_tc_plan_kernel: plan[0] = count, then (sequence, tile pair) entries
    const int* kv_base;  // gathered K/V: first scratch row of every multi-token sequence
};

// Output side of a head-sharded launch (world == 0: single GPU, the tmO map is the output).
struct TcPeers {
    CUtensorMap out_map[kMaxShardWorld];  // [rank]: that rank's [B, Hq_total, Sq, 128] output buffer
    int32_t* flags[kMaxShardWorld];
    int32_t* done_counter;
    int world, rank, head_offset;
    int32_t step;
    int light_first;  // a CTA takes its items lightest first: their output tiles are on the wire while the heavy ones compute
};

// Work list of the paged front end.  Lengths live on the device, so a one-CTA kernel turns them into the list of
// (sequence, tile pair) items that have work; the attention grid is then sized by a host-side bound on the item
// count (exact when the caller passes the scheduler's hint) instead of max_q_len x num_seqs, which for a step with
// a few long prefills and many decode sequences would be almost all empty CTAs.
constexpr int kPlanHeaderInts = 4;  // [0] items in the list (per KV head), [1] CTAs of the attention kernel that take items
// A mixed step runs its prefill rows (tensor-bound) and its decode rows (HBM-bound) at the same time: the attention
// kernel keeps only as many SMs as its share of the step's work needs and the decode kernel, launched as soon as
// those CTAs are seated, takes the rest (and the others as they come free).  The share is worked out here from the
// tables: item-steps of the work list against cached bytes of the one-token sequences, each divided by what one SM
// gets through per microsecond (measured on a step of eight 1024-token prefills beside 120 decode sequences: about
// 3.4 us per item-step of two 128 x 128 tiles over 128 keys at the efficiency of short items; about 52 bytes per
// nanosecond of u8 cache per SM while the SMs that decode are a minority - a sweep of the share on that step was
// flat within 5 % between 0.59 and 0.70 and best at 0.59).
constexpr float kUsPerItemStep = 3.4f;
constexpr float kDecodeBytesPerNsPerSm = 52.f;
constexpr float kHbmBytesPerNs = 6500.f;
// With `owner` given the kernel also lays out the gathered K/V scratch: every multi-token sequence gets a row range
// of roundup(context, 128) rows (kv_base[seq]; allocation order is whatever the atomics make it), and owner[g] names
// the sequence that 128-row group g belongs to (-1: nobody), which is how paged_gather_kernel finds its work.
__global__ void __launch_bounds__(256) paged_tc_plan_kernel(const PagedTables t, const int G, const int Hkv,
                                                            const int capacity, int* plan, int32_t* status,
                                                            int* kv_base, int* owner, const int owner_groups,
                                                            const int attention_ctas, const int share_with_decode) {
    // The list is sorted by weight (key steps of the pair's later tile, clamped to 255), heaviest first: a counting
    // sort in three passes over the sequences - histogram, bucket offsets, scatter.
    constexpr int kBuckets = 256;
    __shared__ int s_hist[kBuckets], s_count, s_groups, s_steps;
    __shared__ unsigned long long s_decode_blocks;
    // Everything that only reads the step's tables - the histogram of the weights, the counts, the bucket offsets -
    // is done while the kernel in front (the step's store) drains; what this kernel WRITES (list, scratch layout)
    // may still be read by earlier kernels, so the writes come after the wait.  (The tables of a step exist before
    // its kernels are launched.)
    for (int i = threadIdx.x; i < kBuckets; i += blockDim.x) s_hist[i] = 0;
    if (threadIdx.x == 0) {
        s_count = s_groups = s_steps = 0;
        s_decode_blocks = 0ull;
    }
    __syncthreads();
    auto weight = [&](int past, int qlen, int pair) {
        const int tiles = ((qlen + 127) / 128) * G;
        const int tile = min(2 * pair + 1, tiles - 1);  // the pair's later tile
        const int keys = min(past + qlen, past + (tile / G) * 128 + 128);
        return min(kBuckets - 1, max(0, (keys + 127) / 128));
    };
    for (int s = threadIdx.x; s < t.num_seqs; s += blockDim.x) {
        const int qlen = t.subsequence_begins[s + 1] - t.subsequence_begins[s];
        if (qlen == 1 && t.past_lens[s] >= 0)
            atomicAdd(&s_decode_blocks, static_cast<unsigned long long>(t.past_lens[s] / t.block_size + 1));
        if (qlen < 2) continue;
        const int past = max(0, t.past_lens[s]);
        const int pairs = (((qlen + 127) / 128) * G + 1) / 2;
        atomicAdd(&s_count, pairs);
        int steps = 0;
        for (int i = 0; i < pairs; ++i) {
            const int w = weight(past, qlen, i);
            atomicAdd(&s_hist[w], 1);
            steps += w;
        }
        atomicAdd(&s_steps, steps);
    }
    __syncthreads();
    if (threadIdx.x == 0) {  // bucket w starts after all heavier buckets
        int at = 0;
        for (int w = kBuckets - 1; w >= 0; --w) {
            const int n = s_hist[w];
            s_hist[w] = at;
            at += n;
        }
    }
    grid_dependency_wait();
    grid_launch_dependents();
    if (owner != nullptr) {
        for (int g = threadIdx.x; g < owner_groups; g += blockDim.x) owner[g] = -1;
        __syncthreads();
        for (int s = threadIdx.x; s < t.num_seqs; s += blockDim.x) {
            const int qlen = t.subsequence_begins[s + 1] - t.subsequence_begins[s];
            if (qlen < 2) continue;
            const int past = max(0, t.past_lens[s]);
            const int groups = t.past_lens[s] < 0 ? 0 : (past + qlen + 127) / 128;
            const int g0 = atomicAdd(&s_groups, groups);
            kv_base[s] = g0 * 128;
            for (int i = 0; i < groups; ++i)
                if (g0 + i < owner_groups) owner[g0 + i] = s;
        }
    }
    __syncthreads();
    for (int s = threadIdx.x; s < t.num_seqs; s += blockDim.x) {
        const int qlen = t.subsequence_begins[s + 1] - t.subsequence_begins[s];
        if (qlen < 2) continue;
        const int past = max(0, t.past_lens[s]);
        const int pairs = (((qlen + 127) / 128) * G + 1) / 2;
        for (int i = 0; i < pairs; ++i) {
            const int at = atomicAdd(&s_hist[weight(past, qlen, i)], 1);
            if (at < capacity) {
                plan[kPlanHeaderInts + 2 * at] = s;
                plan[kPlanHeaderInts + 2 * at + 1] = i;
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        plan[0] = min(s_count, capacity);
        if (s_count > capacity) {  // the caller's prefill_row_blocks was too small
            report(status, B2A_DEV_BAD_LEN);
            plan[0] = 0;  // a truncated sorted list would drop arbitrary pairs: compute nothing instead
        }
        if (owner != nullptr && s_groups > owner_groups) {        // the caller's prefill_kv_tokens was too small
            report(status, B2A_DEV_BAD_LEN);
            plan[0] = 0;  // nothing is computed from a scratch that does not hold every sequence
        }
        // how many of the attention kernel's CTAs take items (the others leave at once and free their SMs)
        int ctas = attention_ctas;
        if (share_with_decode && s_decode_blocks > 0ull && attention_ctas > 1) {
            const float prefill_sm_us = static_cast<float>(s_steps) * Hkv * kUsPerItemStep;
            const float decode_bytes = static_cast<float>(s_decode_blocks) * Hkv * 2.f * kCacheChunk;
            const float decode_sm_us = decode_bytes / (kDecodeBytesPerNsPerSm * 1000.f);
            const float share = prefill_sm_us / (prefill_sm_us + decode_sm_us);
            ctas = static_cast<int>(ceilf(share * attention_ctas));
            // the decode rows cannot use more SMs than it takes to saturate the memory system
            const int decode_max = static_cast<int>(kHbmBytesPerNs / kDecodeBytesPerNsPerSm);
            ctas = max(ctas, attention_ctas - decode_max);
            ctas = min(max(ctas, 1), attention_ctas);
        }
        plan[1] = ctas;
    }
}

__device__ __forceinline__ float ex2f(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float max3f(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// two float32 lanes in one 64-bit register pair, for the packed f32x2 arithmetic of sm_100
__device__ __forceinline__ uint64_t f2_pack(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void f2_unpack(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
template <bool kBf16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    if constexpr (kBf16) {
        const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<const uint32_t*>(&v);
    } else {
        const __half2 v = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<const uint32_t*>(&v);
    }
}
// time-bounded wait that ignores the abort flag: used only to drain work already in flight
__device__ __forceinline__ void mbar_drain(uint32_t bar, uint32_t parity) {
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (clock64() - t0 > kWaitTicks) return;
    }
}

// De-quantise the 16 codes of one 16-byte piece: (code - zp) * scale in float32, as the decode kernel and the CPU
// restatement compute it - the difference is exact in float32 (an integer below 256 minus an f16 value), the product
// rounds once - and then one rounding to f16, the operand format of the tensor core.  0x4B0000XX is 2^23 + XX as a
// float, so a byte permute and one exact subtraction turn a code into its float value.  scale and zp arrive as the
// raw f16 bits the cache stores; a zero scale with zero codes (positions past the context) gives exact zeros.
__device__ __forceinline__ void dequant16_f16(uint4 w, unsigned short scale_bits, unsigned short zp_bits, uint32_t (&outw)[8]) {
    const uint32_t words[4] = {w.x, w.y, w.z, w.w};
    const float sc = __half2float(__ushort_as_half(scale_bits));
    const float zp = __half2float(__ushort_as_half(zp_bits));
    constexpr float k2p23 = 8388608.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float c0 = __uint_as_float(__byte_perm(words[i], 0x4B000000u, 0x7650)) - k2p23;
        const float c1 = __uint_as_float(__byte_perm(words[i], 0x4B000000u, 0x7651)) - k2p23;
        const float c2 = __uint_as_float(__byte_perm(words[i], 0x4B000000u, 0x7652)) - k2p23;
        const float c3 = __uint_as_float(__byte_perm(words[i], 0x4B000000u, 0x7653)) - k2p23;
        outw[2 * i] = pack2<false>((c0 - zp) * sc, (c1 - zp) * sc);
        outw[2 * i + 1] = pack2<false>((c2 - zp) * sc, (c3 - zp) * sc);
    }
}
// ... and store them as two 16-byte chunks of a swizzled shared-memory tile row
__device__ __forceinline__ void dequant_piece_f16(uint4 w, unsigned short scale_bits, unsigned short zp_bits,
                                                  uint8_t* row, int c16, int token) {
    uint32_t outw[8];
    dequant16_f16(w, scale_bits, zp_bits, outw);
    // the piece covers d = 16*c16 .. +15: chunks 2*c16 and 2*c16+1 of the 128-wide row, 8 chunks per 64-wide panel
    uint8_t* panel = row + (c16 >> 2) * kPanel;
    const int cp = (2 * c16) & 7;
    *reinterpret_cast<uint4*>(panel + ((cp ^ (token & 7)) << 4)) = make_uint4(outw[0], outw[1], outw[2], outw[3]);
    *reinterpret_cast<uint4*>(panel + (((cp + 1) ^ (token & 7)) << 4)) = make_uint4(outw[4], outw[5], outw[6], outw[7]);
}

// De-quantise the contexts of the step's multi-token sequences into the f16 scratch [Hkv][rows][128] (K and V each):
// one CTA per (16 scratch rows, KV head), thread = (token, 16-byte piece) for K and again for V.  Rows past a
// sequence's context (its range is rounded up to 128 rows) become zeros, so a tile that reaches past the context
// holds nothing that could turn 0 * x into NaN.
__global__ void __launch_bounds__(128) paged_gather_kernel(const PagedTables t, const uint8_t* k_cache, const uint8_t* v_cache,
                                                           const int Hkv, const int* kv_base, const int* owner,
                                                           const int scratch_rows, uint16_t* k_out, uint16_t* v_out,
                                                           int32_t* status) {
    const int row0 = blockIdx.x * 16, hk = blockIdx.y;
    grid_dependency_wait();  // the scratch layout (plan kernel) and this step's cache rows (store kernel)
    grid_launch_dependents();
    const int seq = owner[row0 / 128];
    if (seq < 0) return;
    const int tok = threadIdx.x >> 3, c16 = threadIdx.x & 7;
    const int pos = row0 - kv_base[seq] + tok;  // position inside the sequence
    const int qlen = t.subsequence_begins[seq + 1] - t.subsequence_begins[seq];
    const int ctx = t.past_lens[seq] + qlen;
    uint4 wk = make_uint4(0u, 0u, 0u, 0u), wv = wk;
    unsigned short sck = 0, zpk = 0, scv = 0, zpv = 0;
    if (pos < ctx) {
        const int lb = pos >> 4;
        int phys = -1;
        if (lb < t.block_indices_begins[seq + 1] - t.block_indices_begins[seq]) phys = t.block_indices[t.block_indices_begins[seq] + lb];
        if (phys < 0 || phys >= t.num_blocks_total) {
            report(status, B2A_DEV_BAD_BLOCK);
        } else {
            const size_t chunk = (static_cast<size_t>(phys) * Hkv + hk) * kCacheChunk;
            const int tb = pos & 15;
            wk = *reinterpret_cast<const uint4*>(k_cache + chunk + tb * 128 + c16 * 16);
            wv = *reinterpret_cast<const uint4*>(v_cache + chunk + tb * 128 + c16 * 16);
            const unsigned short* mk = reinterpret_cast<const unsigned short*>(k_cache + chunk + 2048);
            const unsigned short* mv = reinterpret_cast<const unsigned short*>(v_cache + chunk + 2048);
            sck = mk[tb];
            zpk = mk[16 + tb];
            scv = mv[tb];
            zpv = mv[16 + tb];
        }
    }
    const size_t at = (static_cast<size_t>(hk) * scratch_rows + row0 + tok) * kHeadDim + c16 * 16;
    uint32_t o[8];
    dequant16_f16(wk, sck, zpk, o);
    *reinterpret_cast<uint4*>(k_out + at) = make_uint4(o[0], o[1], o[2], o[3]);
    *reinterpret_cast<uint4*>(k_out + at + 8) = make_uint4(o[4], o[5], o[6], o[7]);
    dequant16_f16(wv, scv, zpv, o);
    *reinterpret_cast<uint4*>(v_out + at) = make_uint4(o[0], o[1], o[2], o[3]);
    *reinterpret_cast<uint4*>(v_out + at + 8) = make_uint4(o[4], o[5], o[6], o[7]);
}

// kMode: 0 dense tensors; 1 paged, K/V de-quantised by producer warps inside the kernel; 2 paged, K/V de-quantised
// beforehand into per-sequence row ranges of an f16 scratch (paged_gather_kernel) and staged by TMA like dense ones
template <bool kBf16, int kMode, int kMask = 0>
__global__ void __launch_bounds__(kMode == 1 ? kThreadsPaged : kThreadsDense, 1)
attn_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
               const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO, const TcParams p,
               const __grid_constant__ TcPeers peers) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;  // 128-byte swizzle atoms want 1024-byte aligned tiles
    uint8_t* gbase = smem_raw + (base - raw);
    const uint32_t sQ = base, sK = base + 2 * kTile, sV = base + 4 * kTile;
    const uint32_t sOut = base + 6 * kTile;
    const uint32_t bars = base + 6 * kTile + kStageOut;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gbase + 6 * kTile + kStageOut + kNumBars * 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gbase + 6 * kTile + kStageOut + kNumBars * 8 + 8);
    auto BAR = [&](int i) { return bars + 8u * static_cast<uint32_t>(i); };
    constexpr bool kPaged = kMode != 0, kDequant = kMode == 1, kGathered = kMode == 2;
    constexpr bool kKvBf16 = kPaged ? false : kBf16;  // element format of the K/V tiles and of P

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // A kernel launched programmatically dependent on this one (the decode kernel of a mixed step) may take the SMs
    // this grid leaves free as soon as every CTA is seated.
    grid_launch_dependents();

    // ---- work items.  An item is a pair of tiles of one KV head.  Rows are numbered inside the sequence (paged) or
    // the tensor (dense); `pos_base` is the key position the first row of the problem may see up to, `kv_limit` the
    // number of keys that exist.  The CTA is persistent (except with in-kernel de-quantisation: one item per CTA):
    // the items, heaviest first - late row blocks in dense mode, the weight-sorted device-built list in paged mode -
    // are dealt to the CTAs in snake order (round k forwards, round k+1 backwards), which evens out the causal
    // imbalance without any shared counter.  Every role calls get_item for itself, so the per-sequence values
    // below are private to the calling thread and follow its own progress through the items.
    // nkvA, nkvB, nmax count key steps from the item's first key tile kv_tile0 (0 unless a sliding window lets the
    // item skip the tiles that all its rows have left behind)
    struct Item {
        int b, hk, row0A, row0B, headA, headB, nkvA, nkvB, nmax, kv_tile0;
    };
    int seq = 0, tok_base = 0, nrows_total = 0, pos_base = 0, kv_limit = 0;
    bool causal = true;
    int nrb = 0, tiles = 0, pairs = 0, total_items = 0;
    int active_ctas = static_cast<int>(gridDim.x);  // CTAs that take items
    if constexpr (kPaged) {
        total_items = p.plan[0] * p.Hkv;  // the grid is only a bound on the number of items
        if (kDequant && static_cast<int>(blockIdx.x * gridDim.y + blockIdx.y) >= total_items) return;
        if constexpr (kGathered) {
            // the plan kernel decides how many CTAs the prefill rows keep; the others give their SM to the decode rows
            active_ctas = min(max(p.plan[1], 1), static_cast<int>(gridDim.x));
            if (static_cast<int>(blockIdx.x) >= active_ctas) return;
        }
    } else {
        nrows_total = p.Sq;
        kv_limit = p.Skv;
        causal = p.causal != 0;
        nrb = (nrows_total + kBM - 1) / kBM;
        tiles = nrb * p.G;
        pairs = (tiles + 1) / 2;
        total_items = pairs * p.B * p.Hkv;  // the launcher keeps this below 2^31
    }
    auto get_item = [&](int k, Item& it) -> bool {  // the k-th item of this CTA
        int pair;
        if constexpr (kPaged) {
            int idx;
            if constexpr (kDequant) {
                if (k > 0) return false;
                idx = static_cast<int>(blockIdx.x * gridDim.y + blockIdx.y);
            } else {
                const int ctas = active_ctas, me = static_cast<int>(blockIdx.x);
                idx = k * ctas + ((k & 1) ? ctas - 1 - me : me);
            }
            if (idx >= total_items) return false;
            const int e = idx / p.Hkv;
            it.b = 0;
            it.hk = idx - e * p.Hkv;
            seq = p.plan[kPlanHeaderInts + 2 * e];
            pair = p.plan[kPlanHeaderInts + 2 * e + 1];
            tok_base = p.t.subsequence_begins[seq];
            nrows_total = p.t.subsequence_begins[seq + 1] - tok_base;
            pos_base = p.t.past_lens[seq];
            kv_limit = pos_base + nrows_total;
            nrb = (nrows_total + kBM - 1) / kBM;
            tiles = nrb * p.G;
            pairs = (tiles + 1) / 2;
            const int nblk = (kv_limit + 15) / 16;
            if (nrows_total < 2 || pos_base < 0 || tok_base < 0 || tok_base + nrows_total > p.t.num_tokens ||
                nblk > p.t.block_indices_begins[seq + 1] - p.t.block_indices_begins[seq] || pair < 0 || pair >= pairs) {
                // inconsistent tables: an empty item, reported once per item by the producer thread
                if (threadIdx.x == 8 * 32) report(p.status, B2A_DEV_BAD_LEN);
                it.hk = 0;
                it.row0A = it.row0B = it.headA = it.headB = it.nkvA = it.nkvB = it.nmax = it.kv_tile0 = 0;
                return true;
            }
        } else {
            const int ctas = static_cast<int>(gridDim.x), me = static_cast<int>(blockIdx.x);
            // With four or more ranks the step is bound by the exchange of the output tiles, which can only start
            // when the first items end: then a CTA walks the SAME items (the deal below is what balances the CTAs)
            // from its lightest to its heaviest, and the epilogue's stores to the other ranks are on the wire from
            // the first microseconds on.  Measured with four ranks: 0.200 ms a step, against 0.231 ms heaviest
            // first.  (Storing a tile once locally and letting the CTA's two spare warps forward it to the other
            // ranks - so that no softmax warp ever waits for the links - was built and measured as well: 0.207-0.211
            // ms at best, the forwarding stores queue up in the SM's path to memory in front of the K/V loads.)
            if (peers.light_first) {
                const int rounds = total_items / ctas, rem = total_items - rounds * ctas;
                const int mine = rounds + ((((rounds & 1) ? ctas - 1 - me : me) < rem) ? 1 : 0);
                if (k >= mine) return false;
                k = mine - 1 - k;
            }
            const int idx = k * ctas + ((k & 1) ? ctas - 1 - me : me);
            if (idx >= total_items) return false;
            // heaviest row blocks of ALL (batch, KV head) streams first (measured faster than walking one stream
            // after the other, although that keeps fewer K/V streams in flight)
            const int bh = p.B * p.Hkv;
            pair = pairs - 1 - idx / bh;
            const int y = idx % bh;
            it.b = y / p.Hkv;
            it.hk = y % p.Hkv;
        }
        // a tile's rows, its head, the end of its keys (in tiles) and the first key tile any of its rows still sees
        auto tile_of = [&](int t, int& row0, int& head, int& nkv, int& first) {
            const bool present = t < tiles;
            const int rb = present ? t / p.G : 0, g = present ? t % p.G : 0;
            row0 = rb * kBM;
            head = it.hk * p.G + g;
            const int kv_end = causal ? min(kv_limit, pos_base + row0 + kBM) : kv_limit;
            nkv = present ? (kv_end + kBN - 1) / kBN : 0;
            if constexpr (kPaged) {
                first = (p.window > 0 && present) ? max(0, pos_base + row0 - p.window + 1) / kBN : 0;
                if (!present) first = 1 << 30;
            } else {
                first = 0;
            }
        };
        int firstA, firstB;
        tile_of(2 * pair, it.row0A, it.headA, it.nkvA, firstA);
        tile_of(2 * pair + 1, it.row0B, it.headB, it.nkvB, firstB);
        it.kv_tile0 = 0;
        if constexpr (kPaged) {
            // the two tiles walk the same key tiles: both start at the earlier of their first ones (a tile that starts
            // before its window only meets keys its mask removes)
            it.kv_tile0 = min(min(firstA, firstB), max(it.nkvA, it.nkvB));
            it.nkvA = max(0, it.nkvA - it.kv_tile0);
            it.nkvB = max(0, it.nkvB - it.kv_tile0);
        }
        it.nmax = max(it.nkvA, it.nkvB);
        return true;
    };

    // ---- set-up: barriers, TMEM
    if (threadIdx.x == 0) {
        for (int i = 0; i < kNumBars; ++i) {
            uint32_t count = 1;
            if (i == P_READY || i == P_READY + 1 || i == P_HALF || i == P_HALF + 1) count = 128;
            if (i == Q_CONV || i == Q_CONV + 1) count = 128;
            if (i == Q_EMPTY || i == Q_EMPTY + 1) count = 1;
            if (kDequant && (i == K_FULL || i == K_FULL + 1 || i == V_FULL || i == V_FULL + 1)) count = 128;
            if (kGathered && (i == Q_CONV || i == Q_CONV + 1)) count = 64;  // converted by warps 10 and 11
            mbar_init(BAR(i), count);
        }
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 9) {
        tmem_alloc(smem_u32(tmem_slot), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    // Registers follow the work: the service warpgroup keeps 56 per thread, the softmax groups take what is left
    // (dense: 2*128*224 + 128*56 = 384*168; paged: 2*128*168 + 128*56 + 128*112 <= 512*128).
    if (warp >= 8 && warp < 12) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    }
    if (warp >= 12) {
        // =============================== de-quantising K/V producers (paged) ===============================
        if constexpr (kDequant) {
            asm volatile("setmaxnreg.dec.sync.aligned.u32 112;");
            Item item;
            get_item(0, item);  // paged mode: exactly one item per CTA
            const int nkvA = item.nkvA, nkvB = item.nkvB, nmax = item.nmax, hk = item.hk;
            const int tp = static_cast<int>(threadIdx.x) - 384;
            const int tok_in_blk = tp >> 3, c16 = tp & 7;
            const int32_t* btab = p.t.block_indices + p.t.block_indices_begins[seq];
            const int nblk = (kv_limit + 15) / 16;
            bool ok = true;
            if constexpr (kBf16) {
                // bf16 queries: convert the Q tiles to f16 where they lie (the swizzle only permutes 16-byte
                // chunks, so an element-wise pass keeps the layout); magnitudes beyond the f16 range saturate
#pragma unroll
                for (int X = 0; X < 2; ++X) {
                    if ((X ? nkvB : nkvA) > 0) {
                        ok = ok && __all_sync(0xffffffffu, mbar_wait(BAR(Q_FULL + X), 0, abort_flag));
                        if (ok) {
                            uint4* tile = reinterpret_cast<uint4*>(gbase + X * kTile);
                            for (int i = tp; i < kTile / 16; i += 128) {
                                uint4 v = tile[i];
                                uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
                                for (int k = 0; k < 4; ++k) {
                                    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[k]));
                                    w[k] = pack2<false>(fminf(fmaxf(f.x, -65504.f), 65504.f), fminf(fmaxf(f.y, -65504.f), 65504.f));
                                }
                                tile[i] = v;
                            }
                            fence_proxy_async_smem();
                            mbar_arrive(BAR(Q_CONV + X));
                        }
                    }
                }
            }
            // One tile = 8 logical blocks; per block the 128 threads cover 16 tokens x 8 sixteen-byte pieces, so a
            // block's 2048 code bytes are read with fully coalesced 128-bit loads.  Everything a tile needs is
            // requested before anything is converted (one memory latency per tile, not one per block), and the
            // block ids of the next step are fetched while this step is converted.
            int phys[8], phys_next[8];
            const int kv_tile0 = item.kv_tile0;
            auto load_ids = [&](int j, int (&ids)[8]) {
#pragma unroll
                for (int it = 0; it < 8; ++it) {
                    const int lb = (kv_tile0 + j) * 8 + it;
                    int id = -1;
                    if (lb < nblk && lb * 16 + tok_in_blk < kv_limit) {
                        id = btab[lb];
                        if (id < 0 || id >= p.t.num_blocks_total) {
                            report(p.status, B2A_DEV_BAD_BLOCK);
                            id = -1;
                        }
                    }
                    ids[it] = id;
                }
            };
            uint4 w[8];
            unsigned short sc[8], zp[8];  // raw f16 bits: converting here would wait for each load in turn
            auto load_tile = [&](const uint8_t* cache) {
#pragma unroll
                for (int it = 0; it < 8; ++it) {
                    // positions past the context (and unusable blocks) become exact zeros: 0 * anything finite
                    w[it] = make_uint4(0u, 0u, 0u, 0u);
                    sc[it] = 0;
                    zp[it] = 0;
                    if (phys[it] >= 0) {
                        const uint8_t* chunk = cache + (static_cast<size_t>(phys[it]) * p.Hkv + hk) * kCacheChunk;
                        w[it] = *reinterpret_cast<const uint4*>(chunk + tok_in_blk * 128 + c16 * 16);
                        const unsigned short* meta = reinterpret_cast<const unsigned short*>(chunk + 2048);
                        sc[it] = meta[tok_in_blk];
                        zp[it] = meta[16 + tok_in_blk];
                    }
                }
            };
            auto convert_tile = [&](uint8_t* tile) {
#pragma unroll
                for (int it = 0; it < 8; ++it) {
                    const int token = it * 16 + tok_in_blk;
                    dequant_piece_f16(w[it], sc[it], zp[it], tile + token * 128, c16, token);
                }
            };
            load_ids(0, phys_next);
            for (int j = 0; j < nmax; ++j) {
                const int st = j & 1, n = j >> 1;
#pragma unroll
                for (int it = 0; it < 8; ++it) phys[it] = phys_next[it];
                load_tile(p.k_cache);
                if (j + 1 < nmax) load_ids(j + 1, phys_next);
                if (n > 0) ok = __all_sync(0xffffffffu, mbar_wait(BAR(K_EMPTY + st), (n - 1) & 1, abort_flag));
                if (!ok) break;
                convert_tile(gbase + 2 * kTile + st * kTile);
                fence_proxy_async_smem();  // generic-proxy writes must be visible to the tensor core's reads
                mbar_arrive(BAR(K_FULL + st));
                load_tile(p.v_cache);
                if (n > 0) ok = __all_sync(0xffffffffu, mbar_wait(BAR(V_EMPTY + st), (n - 1) & 1, abort_flag));
                if (!ok) break;
                convert_tile(gbase + 4 * kTile + st * kTile);
                fence_proxy_async_smem();
                mbar_arrive(BAR(V_FULL + st));
            }
        }
    } else if (warp >= 10) {
        // idle warps of the service warpgroup; with gathered K/V and bf16 queries they turn the Q tiles into f16 where
        // they lie (the swizzle only permutes 16-byte chunks, so an element-wise pass keeps the layout)
        if constexpr (kGathered && kBf16) {
            Item item;
            const int tp = static_cast<int>(threadIdx.x) - 320;  // 0..63
            bool ok = true;
            int qn[2] = {0, 0};  // Q tiles of each kind seen so far
            for (int kk = 0; ok && get_item(kk, item); ++kk)
#pragma unroll
            for (int X = 0; X < 2; ++X) {
                if ((X ? item.nkvB : item.nkvA) > 0) {
                    ok = ok && __all_sync(0xffffffffu, mbar_wait(BAR(Q_FULL + X), qn[X] & 1, abort_flag));
                    ++qn[X];
                    if (ok) {
                        uint4* tile = reinterpret_cast<uint4*>(gbase + X * kTile);
                        for (int i = tp; i < kTile / 16; i += 64) {
                            uint4 v = tile[i];
                            uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[k]));
                                w[k] = pack2<false>(fminf(fmaxf(f.x, -65504.f), 65504.f), fminf(fmaxf(f.y, -65504.f), 65504.f));
                            }
                            tile[i] = v;
                        }
                        fence_proxy_async_smem();
                        mbar_arrive(BAR(Q_CONV + X));
                    }
                }
            }
        }
    } else if (warp == 8) {
        // =============================== TMA producer ===============================
        if (lane == 0) {
            prefetch_tensormap(&tmQ);
            if constexpr (!kDequant) {
                prefetch_tensormap(&tmK);
                prefetch_tensormap(&tmV);
            }
            // running counts over the items of this CTA: K/V tiles issued (ring position) and Q tiles loaded
            int g = 0, issued_k = 0, issued_v = 0, qn[2] = {0, 0};
            bool ok = true;
            const uint64_t once_policy = l2_evict_first_policy();  // Q tiles are read once
            Item it;
            for (int k = 0; ok && get_item(k, it); ++k) {
                auto load_q = [&](int X) {
                    const int nkvX = X ? it.nkvB : it.nkvA;
                    if (nkvX == 0) return;
                    // the tile's previous occupant is free once its last QK^T has completed
                    if (qn[X] > 0 && !mbar_wait(BAR(Q_EMPTY + X), (qn[X] - 1) & 1, abort_flag)) { ok = false; return; }
                    mbar_expect_tx(BAR(Q_FULL + X), kTile);
                    const int row = tok_base + (X ? it.row0B : it.row0A), head = X ? it.headB : it.headA;
                    tma_load_4d_hint(sQ + X * kTile, &tmQ, BAR(Q_FULL + X), 0, row, head, it.b, once_policy);
                    tma_load_4d_hint(sQ + X * kTile + kPanel, &tmQ, BAR(Q_FULL + X), 64, row, head, it.b, once_policy);
                    ++qn[X];
                };
                load_q(0);
                if (ok) load_q(1);
                if constexpr (!kDequant) {
                    // gathered mode: the sequence's keys start at row kv_row0 of the scratch, which is one [1, Hkv, rows, 128] tensor
                    const int kv_row0 = kGathered ? p.kv_base[seq] + it.kv_tile0 * kBN : 0;
                    for (int j = 0; ok && j < it.nmax; ++j, ++g) {
                        const int st = g & 1, n = g >> 1;
                        if (n > 0 && !mbar_wait(BAR(K_EMPTY + st), (n - 1) & 1, abort_flag)) { ok = false; break; }
                        mbar_expect_tx(BAR(K_FULL + st), kTile);
                        tma_load_4d(sK + st * kTile, &tmK, BAR(K_FULL + st), 0, kv_row0 + j * kBN, it.hk, it.b);
                        tma_load_4d(sK + st * kTile + kPanel, &tmK, BAR(K_FULL + st), 64, kv_row0 + j * kBN, it.hk, it.b);
                        ++issued_k;
                        if (n > 0 && !mbar_wait(BAR(V_EMPTY + st), (n - 1) & 1, abort_flag)) { ok = false; break; }
                        mbar_expect_tx(BAR(V_FULL + st), kTile);
                        tma_load_4d(sV + st * kTile, &tmV, BAR(V_FULL + st), 0, kv_row0 + j * kBN, it.hk, it.b);
                        tma_load_4d(sV + st * kTile + kPanel, &tmV, BAR(V_FULL + st), 64, kv_row0 + j * kBN, it.hk, it.b);
                        ++issued_v;
                    }
                }
            }
            if (*abort_flag) {  // let copies already in flight land before the CTA goes away
                for (int X = 0; X < 2; ++X)
                    if (qn[X] > 0) mbar_drain(BAR(Q_FULL + X), (qn[X] - 1) & 1);
                for (int jj = max(0, issued_k - 2); jj < issued_k; ++jj) mbar_drain(BAR(K_FULL + (jj & 1)), (jj >> 1) & 1);
                for (int jj = max(0, issued_v - 2); jj < issued_v; ++jj) mbar_drain(BAR(V_FULL + (jj & 1)), (jj >> 1) & 1);
            }
        }
    } else if (warp == 9) {
        // =============================== MMA issuer ===============================
        if (lane == 0) {
            // operand formats (A and B of one MMA must agree): dense mode as given; paged mode f16 throughout - the
            // de-quantised values keep 11 significant bits and bf16 queries are converted in shared memory first
            constexpr uint32_t idesc_qk = instr_desc_f16(kKvBf16, false, kBM, kBN);
            constexpr uint32_t idesc_pv = instr_desc_f16(kKvBf16, true, kBM, kHeadDim);
            // descriptors are assembled at the point of issue from (tile address >> 4) plus compile-time parts
            constexpr uint32_t kLoK = desc_lo_sw128(16), kHiK = desc_hi_sw128(1024);        // K-major: Q and K tiles
            constexpr uint32_t kLoV = desc_lo_sw128(kPanel), kHiV = desc_hi_sw128(1024);    // MN-major: V tiles
            const uint32_t q16 = (sQ >> 4) & 0x3FFFu, k16 = (sK >> 4) & 0x3FFFu, v16 = (sV >> 4) & 0x3FFFu;
            auto issue_qk = [&](int X, int st) {  // S_X = Q_X K^T : 8 steps of 16 along D
                const uint32_t d = tmem + static_cast<uint32_t>(X * 128);
                const uint32_t qa = q16 + static_cast<uint32_t>(X * (kTile >> 4)), ka = k16 + static_cast<uint32_t>(st * (kTile >> 4));
#define B2A_QK(ks) \
    mma_ss_c<((((ks) / 4) * kPanel + ((ks) & 3) * 32) / 16), ((((ks) / 4) * kPanel + ((ks) & 3) * 32) / 16), kLoK, kLoK, kHiK, kHiK, \
             idesc_qk>(d, qa, ka, (ks) > 0 ? 1u : 0u)
                B2A_QK(0); B2A_QK(1); B2A_QK(2); B2A_QK(3); B2A_QK(4); B2A_QK(5); B2A_QK(6); B2A_QK(7);
#undef B2A_QK
            };
            // O_X += P_X V : 8 steps of 16 along the keys, issued in two halves as the halves of P arrive
            auto issue_pv = [&](int X, int st, bool acc, int half) {
                const uint32_t d = tmem + static_cast<uint32_t>(256 + X * 128);
                const uint32_t pa = tmem + static_cast<uint32_t>(X * 128 + half * 32);
                const uint32_t va = v16 + static_cast<uint32_t>(st * (kTile >> 4) + half * (4 * 2048 / 16));
#define B2A_PV(ks, accv) mma_ts_c<(ks) * 8, ((ks) * 2048) / 16, kLoV, kHiV, idesc_pv>(d, pa, va, accv)
                B2A_PV(0, acc ? 1u : 0u); B2A_PV(1, 1u); B2A_PV(2, 1u); B2A_PV(3, 1u);
#undef B2A_PV
            };
            bool ok = true;
            constexpr int kQReady = (kPaged && kBf16) ? Q_CONV : Q_FULL;
            // running counts over the items of this CTA: K/V ring position, steps of each tile, Q tiles consumed
            int g0 = 0, sx[2] = {0, 0}, qn[2] = {0, 0};
            Item it;
            for (int k = 0; ok && get_item(k, it); ++k) {
                const int nkvA = it.nkvA, nkvB = it.nkvB, nmax = it.nmax;
                if (nmax == 0) continue;  // an item that was refused (inconsistent tables)
                if (nkvA > 0) ok = ok && mbar_wait(BAR(kQReady + 0), qn[0] & 1, abort_flag);
                if (nkvB > 0) ok = ok && mbar_wait(BAR(kQReady + 1), qn[1] & 1, abort_flag);
                ok = ok && mbar_wait(BAR(K_FULL + (g0 & 1)), (g0 >> 1) & 1, abort_flag);
                if (!ok) break;
                tc_fence_after();
                if (nkvA > 0) {
                    issue_qk(0, g0 & 1);
                    mma_commit(BAR(S_FULL + 0));
                    if (nkvA == 1) mma_commit(BAR(Q_EMPTY + 0));  // last use of this Q tile: the producer may refill it
                }
                if (nkvB > 0) {
                    issue_qk(1, g0 & 1);
                    mma_commit(BAR(S_FULL + 1));
                    if (nkvB == 1) mma_commit(BAR(Q_EMPTY + 1));
                }
                mma_commit(BAR(K_EMPTY + (g0 & 1)));
                for (int j = 0; ok && j < nmax; ++j) {
                    const int g = g0 + j, stv = g & 1;
                    if (!mbar_wait(BAR(V_FULL + stv), (g >> 1) & 1, abort_flag)) { ok = false; break; }
                    bool k_next_ready = false;
#pragma unroll
                    for (int X = 0; X < 2; ++X) {
                        const int nkvX = X ? nkvB : nkvA;
                        if (ok && j < nkvX) {
                            const int par = (sx[X] + j) & 1;
                            if (!mbar_wait(BAR(P_HALF + X), par, abort_flag)) { ok = false; break; }
                            tc_fence_after();
                            issue_pv(X, stv, j > 0, 0);
                            if (!mbar_wait(BAR(P_READY + X), par, abort_flag)) { ok = false; break; }
                            tc_fence_after();
                            issue_pv(X, stv, true, 1);
                            mma_commit(BAR(O_DONE + X));
                        }
                        if (ok && j + 1 < nkvX) {
                            if (!k_next_ready) {
                                if (!mbar_wait(BAR(K_FULL + ((g + 1) & 1)), ((g + 1) >> 1) & 1, abort_flag)) { ok = false; break; }
                                k_next_ready = true;
                                tc_fence_after();
                            }
                            issue_qk(X, (g + 1) & 1);
                            mma_commit(BAR(S_FULL + X));
                            if (j + 2 == nkvX) mma_commit(BAR(Q_EMPTY + X));
                        }
                    }
                    if (!ok) break;
                    mma_commit(BAR(V_EMPTY + stv));
                    if (j + 1 < nmax) mma_commit(BAR(K_EMPTY + ((g + 1) & 1)));
                }
                g0 += nmax;
                sx[0] += nkvA;
                sx[1] += nkvB;
                qn[0] += nkvA > 0;
                qn[1] += nkvB > 0;
            }
            mma_commit(BAR(DRAIN));  // everything issued has completed before TMEM and shared memory are given up
            mbar_drain(BAR(DRAIN), 0);
        }
    } else {
        // =============================== softmax + epilogue of tile X ===============================
        if constexpr (kDequant) {
            asm volatile("setmaxnreg.inc.sync.aligned.u32 168;");
        } else {
            asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
        }
        const int X = warp >> 2;
        const int r = static_cast<int>(threadIdx.x) - X * 128;
        const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const uint32_t tS = tmem + lane_base + static_cast<uint32_t>(X * 128);
        const uint32_t tO = tmem + lane_base + static_cast<uint32_t>(256 + X * 128);
        int sxb = 0;  // steps of this tile in the CTA's earlier items: every per-step barrier is at phase (sxb + j)
        bool ok = true;
        Item item;
        for (int k = 0; ok && get_item(k, item); ++k) {
            const int nkv = X ? item.nkvB : item.nkvA;
            if (nkv == 0) continue;
            const int row_pos0 = pos_base + (X ? item.row0B : item.row0A);
            // first step whose tile touches the end of the keys or the causal diagonal (both conditions only
            // become true as j grows): steps before it need no masking
            int jb;
            {
                const int j_end = kv_limit / kBN;
                const int dgl = row_pos0 - (kBN - 1);
                const int j_diag = dgl < 0 ? 0 : dgl / kBN + 1;
                jb = (causal ? min(j_end, j_diag) : j_end) - (kPaged ? item.kv_tile0 : 0);
            }
            // with a sliding window, key tiles that begin below the window of the tile's LAST row need the mask too
            const int tile0 = kPaged ? item.kv_tile0 : 0;
            const int window = kPaged ? p.window : 0;
            const int low_limit = window > 0 ? row_pos0 + kBM - window : -(1 << 30);  // mask while key0 < low_limit
            const float c = kMask == 2 ? 1.0f : p.scale_log2;  // (additive masks: the block below has scaled the scores)
            float m_used = -1.0e30f, l = 0.f;
            for (int j = 0; j < nkv; ++j) {
                // every lane takes the same decision, so the warp-collective TMEM instructions stay converged
                ok = __all_sync(0xffffffffu, mbar_wait(BAR(S_FULL + X), (sxb + j) & 1, abort_flag));
                if (!ok) break;
                tc_fence_after();
                uint32_t s[4][32];
#pragma unroll
                for (int q = 0; q < 4; ++q) tmem_ld32(tS + 32 * q, s[q]);
                tmem_wait_ld();
                const int key0 = (tile0 + j) * kBN;
                if constexpr (kMask != 0) {
                    // this row's 128 mask values of the step, 32 keys at a time (rows past the end of the tensor read
                    // the last row: their results are dropped; keys past the end are removed below)
                    const int mrow = min(row_pos0 + r, nrows_total - 1);
                    const uint8_t* mbase = p.mask + (static_cast<int64_t>(item.b) * p.mask_strides[0] +
                                                     static_cast<int64_t>(X ? item.headB : item.headA) * p.mask_strides[1] +
                                                     static_cast<int64_t>(mrow) * p.mask_strides[2] + key0) * (kMask == 1 ? 1 : 2);
                    const bool whole = key0 + kBN <= kv_limit;  // else only whole 16-byte pieces inside the row are read
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        if constexpr (kMask == 1) {
                            uint4 m0 = make_uint4(0u, 0u, 0u, 0u), m1 = m0;
                            if (whole || key0 + 32 * q + 16 <= kv_limit) m0 = *reinterpret_cast<const uint4*>(mbase + 32 * q);
                            if (whole || key0 + 32 * q + 32 <= kv_limit) m1 = *reinterpret_cast<const uint4*>(mbase + 32 * q + 16);
                            const uint32_t w[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                                if (((w[i >> 2] >> (8 * (i & 3))) & 0xffu) == 0u) s[q][i] = 0xff800000u;  // -inf
                        } else {
                            // additive: the scores leave this block as S * scale * log2(e) + mask * log2(e)
                            const float c = p.scale_log2;
#pragma unroll
                            for (int h = 0; h < 4; ++h) {
                                uint4 m = make_uint4(0u, 0u, 0u, 0u);
                                if (whole || key0 + 32 * q + 8 * h + 8 <= kv_limit) m = *reinterpret_cast<const uint4*>(mbase + 64 * q + 16 * h);
                                const uint32_t w[4] = {m.x, m.y, m.z, m.w};
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    float lo, hi;
                                    if constexpr (kBf16) {
                                        lo = __uint_as_float(w[i] << 16);
                                        hi = __uint_as_float(w[i] & 0xffff0000u);
                                    } else {
                                        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
                                        lo = f.x;
                                        hi = f.y;
                                    }
                                    const int e = 8 * h + 2 * i;
                                    s[q][e] = __float_as_uint(fmaf(__uint_as_float(s[q][e]), c, lo * kLog2e));
                                    s[q][e + 1] = __float_as_uint(fmaf(__uint_as_float(s[q][e + 1]), c, hi * kLog2e));
                                }
                            }
                        }
                    }
                }
                if (j >= jb || (kPaged && key0 < low_limit)) {
                    const int row_pos = row_pos0 + r;  // last key position this row may see (causal)
                    const int row_low = window > 0 ? row_pos - window + 1 : 0;  // and the first
#pragma unroll
                    for (int q = 0; q < 4; ++q)
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const int key = key0 + q * 32 + i;
                            const bool keep = key < kv_limit && (!causal || key <= row_pos) && (!kPaged || key >= row_low);
                            if (!keep) s[q][i] = 0xff800000u;  // -inf
                        }
                }
                // row maximum: four independent chains of 3-input max (a single chain of 128 would be latency-bound)
                float mq[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    mq[q] = -INFINITY;
#pragma unroll
                    for (int i = 0; i < 32; i += 2)
                        mq[q] = max3f(mq[q], __uint_as_float(s[q][i]), __uint_as_float(s[q][i + 1]));
                }
                const float mx = fmaxf(fmaxf(mq[0], mq[1]), fmaxf(mq[2], mq[3]));
                const float m_cand = mx * c;
                const bool need = (j == 0) || (m_cand > m_used + kLazyThreshold);
                const bool need_any = __any_sync(0xffffffffu, need);
                float alpha = 1.f;
                if (need_any) {
                    const float m_new = fmaxf(m_used, m_cand);
                    alpha = ex2f(m_used - m_new);
                    m_used = m_new;
                    l *= alpha;
                }
                // P = exp2(S*c - m): the scale-and-shift and the row sum run two elements per instruction (f32x2)
                const uint64_t c2 = f2_pack(c, c), nm2 = f2_pack(-m_used, -m_used);
                uint64_t sum2[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    uint32_t pk[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const uint64_t x2 = f2_fma(f2_pack(__uint_as_float(s[q][2 * i]), __uint_as_float(s[q][2 * i + 1])), c2, nm2);
                        float x0, x1;
                        f2_unpack(x2, x0, x1);
                        const float p0 = ex2f(x0), p1 = ex2f(x1);
                        sum2[i & 3] = f2_add(sum2[i & 3], f2_pack(p0, p1));
                        pk[i] = pack2<kKvBf16>(p0, p1);
                    }
                    tmem_st16(tS + 16 * q, pk);  // P over the first 64 columns of S, behind what was already read
                    // first 64 keys of P are in TMEM: PV can start on them, unless O still has to be rescaled
                    if (q == 1 && !(need_any && j > 0)) {
                        tmem_wait_st();
                        tc_fence_before();
                        mbar_arrive(BAR(P_HALF + X));
                    }
                }
                {
                    float a0, a1;
                    f2_unpack(f2_add(f2_add(sum2[0], sum2[1]), f2_add(sum2[2], sum2[3])), a0, a1);
                    l += a0 + a1;
                }
                if (need_any && j > 0) {
                    // O_X still holds the old scale; PV_X(j-1) must have landed before it is touched
                    ok = __all_sync(0xffffffffu, mbar_wait(BAR(O_DONE + X), (sxb + j - 1) & 1, abort_flag));
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        uint32_t o[32];
                        tmem_ld32(tO + 32 * q, o);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        tmem_st32(tO + 32 * q, o);
                    }
                    tmem_wait_st();
                    tc_fence_before();
                    mbar_arrive(BAR(P_HALF + X));
                }
                tmem_wait_st();
                tc_fence_before();
                mbar_arrive(BAR(P_READY + X));
            }
            if (ok) ok = __all_sync(0xffffffffu, mbar_wait(BAR(O_DONE + X), (sxb + nkv - 1) & 1, abort_flag));
            sxb += nkv;
            if (ok) {
                tc_fence_after();
                const float inv = l > 0.f ? 1.f / l : 0.f;
                // where the tile goes: worked out again here rather than kept in registers across the key loop
                if constexpr (!kPaged) {  // (paged items come from tables in global memory: those are kept)
                    int k_again = k;
                    asm volatile("" : "+r"(k_again));
                    get_item(k_again, item);
                }
                const int row0 = X ? item.row0B : item.row0A, head = X ? item.headB : item.headA, b = item.b;
                if constexpr (kPaged) {
                    // row-wise stores: rows past the sequence's end belong to other sequences and are dropped
                    const bool valid = row0 + r < nrows_total;
                    uint4* orow = reinterpret_cast<uint4*>(
                        reinterpret_cast<uint16_t*>(p.out) +
                        (static_cast<size_t>(tok_base + row0 + r) * p.Hq + head) * kHeadDim);
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        uint32_t o[32];
                        tmem_ld32(tO + 32 * q, o);
                        tmem_wait_ld();
                        if (valid) {
#pragma unroll
                            for (int ch = 0; ch < 4; ++ch) {
                                uint4 v;
                                v.x = pack2<kBf16>(__uint_as_float(o[8 * ch + 0]) * inv, __uint_as_float(o[8 * ch + 1]) * inv);
                                v.y = pack2<kBf16>(__uint_as_float(o[8 * ch + 2]) * inv, __uint_as_float(o[8 * ch + 3]) * inv);
                                v.z = pack2<kBf16>(__uint_as_float(o[8 * ch + 4]) * inv, __uint_as_float(o[8 * ch + 5]) * inv);
                                v.w = pack2<kBf16>(__uint_as_float(o[8 * ch + 6]) * inv, __uint_as_float(o[8 * ch + 7]) * inv);
                                orow[q * 4 + ch] = v;
                            }
                        }
                    }
                } else {
                    // two passes of 64 columns through this warp's [32 rows x 128 bytes] staging slab
                    const uint32_t slab = sOut + static_cast<uint32_t>(warp) * 4096u;
                    uint8_t* prow = gbase + 6 * kTile + warp * 4096 + (r & 31) * 128;
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        if (lane == 0) tma_store_wait_read();  // the slab's previous store has read it
                        __syncwarp();
#pragma unroll
                        for (int qq = 0; qq < 2; ++qq) {
                            const int q = 2 * half + qq;
                            uint32_t o[32];
                            tmem_ld32(tO + 32 * q, o);
                            tmem_wait_ld();
#pragma unroll
                            for (int ch = 0; ch < 4; ++ch) {
                                uint4 v;
                                v.x = pack2<kBf16>(__uint_as_float(o[8 * ch + 0]) * inv, __uint_as_float(o[8 * ch + 1]) * inv);
                                v.y = pack2<kBf16>(__uint_as_float(o[8 * ch + 2]) * inv, __uint_as_float(o[8 * ch + 3]) * inv);
                                v.z = pack2<kBf16>(__uint_as_float(o[8 * ch + 4]) * inv, __uint_as_float(o[8 * ch + 5]) * inv);
                                v.w = pack2<kBf16>(__uint_as_float(o[8 * ch + 6]) * inv, __uint_as_float(o[8 * ch + 7]) * inv);
                                const int chunk = qq * 4 + ch;  // 16-byte chunk of the 128-byte row, swizzled like TMA's
                                *reinterpret_cast<uint4*>(prow + ((chunk ^ (r & 7)) << 4)) = v;
                            }
                        }
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            if (peers.world == 0) {
                                tma_store_4d_hint(&tmO, slab, 64 * half, row0 + 32 * (warp & 3), head, b, l2_evict_first_policy());
                            } else {
                                // the same slab into every rank's buffer, the next rank first so that the ranks do
                                // not all write to the same peer at the same time; local copy last
                                for (int i = 1; i <= peers.world; ++i) {
                                    const int dst = (peers.rank + i) % peers.world;
                                    tma_store_4d(&peers.out_map[dst], slab, 64 * half, row0 + 32 * (warp & 3), peers.head_offset + head, b);
                                }
                            }
                            tma_store_commit();
                        }
                    }
                }
            }
        }
        // stores still in flight: their completion (not only the read of shared memory) before the CTA ends
        if (lane == 0) tma_store_wait_all();
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 9) {
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
    if (threadIdx.x == 0 && *abort_flag) report(p.status, B2A_DEV_TIMEOUT);
    if constexpr (!kPaged) {
        if (peers.world > 0 && threadIdx.x == 0) {
            // every storing lane has waited for its writes and passed the barrier above: order them before the
            // arrival, and let the last CTA of the grid publish the step to every rank
            __threadfence_system();
            const int total = static_cast<int>(gridDim.x * gridDim.y);
            if (atomicAdd(peers.done_counter, 1) == total - 1) {
                *peers.done_counter = 0;
                __threadfence_system();
                for (int r = 0; r < peers.world; ++r)
                    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(peers.flags[r] + peers.rank), "r"(peers.step)
                                 : "memory");
            }
        }
    }
}

// Stream-ordered wait for the other ranks of a head-sharded prefill step: returns when every flag shows `step`.
// Bounded in wall-clock time: a peer that never arrives turns into B2A_DEV_TIMEOUT in the status word.
__global__ void __launch_bounds__(32) sdpa_peer_wait_kernel(const int32_t* flags, const int world, const int32_t step,
                                                            const long long wait_ns, int32_t* status) {
    grid_dependency_wait();  // launched while the attention kernel is still running: first let that one finish
    if (static_cast<int>(threadIdx.x) < world) {
        const int32_t* flag = flags + threadIdx.x;
        long long t0;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
        for (;;) {
            int32_t v;
            asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
            if (v - step >= 0) break;
            long long t1;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
            if (t1 - t0 > wait_ns) {
                report(status, B2A_DEV_TIMEOUT);
                break;
            }
        }
    }
}

// ---- host side ---------------------------------------------------------------------------------------------

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            return nullptr;
        return reinterpret_cast<EncodeTiledFn>(ptr);
    }();
    return fn;
}

// [B, H, S, 128] view with element strides st[0..3] (st[3] == 1) as a 4-D map, box = [64 x box_rows x 1 x 1],
// 128-byte swizzle
bool make_map(CUtensorMap* map, const void* ptr, bool bf16, int B, int H, int S, const int64_t (&st)[4], int box_rows) {
    EncodeTiledFn enc = encode_fn();
    if (enc == nullptr) return false;
    const cuuint64_t dims[4] = {static_cast<cuuint64_t>(kHeadDim), static_cast<cuuint64_t>(S),
                                static_cast<cuuint64_t>(H), static_cast<cuuint64_t>(B)};
    // a stride of an extent-1 dimension is never used for addressing but is still validated: give it a legal value
    auto bytes = [](int64_t elems, int extent) { return static_cast<cuuint64_t>(extent == 1 || elems <= 0 ? 256 : elems * 2); };
    const cuuint64_t strides[3] = {bytes(st[2], S), bytes(st[1], H), bytes(st[0], B)};
    const cuuint32_t box[4] = {64, static_cast<cuuint32_t>(box_rows), 1, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    return enc(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
               const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool strides_ok(const int64_t (&st)[4], int B, int H, int S) {
    if (st[3] != 1) return false;
    const int ext[3] = {B, H, S};
    for (int i = 0; i < 3; ++i)
        if (ext[i] > 1 && (st[i] <= 0 || st[i] % 8 != 0)) return false;  // 16-byte multiples
    return true;
}

template <typename Kern>
int configure_once(Kern kern, bool (&done)[64]) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return B2A_ERR_CUDA;
    if (dev < 0 || dev >= 64 || !done[dev]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess)
            return B2A_ERR_CUDA;
        if (dev >= 0 && dev < 64) done[dev] = true;
    }
    return B2A_OK;
}

}  // namespace

bool sdpa_tc_supported(const b2a_sdpa_desc& d, const int64_t (&qs)[4], const int64_t (&ks)[4], const int64_t (&vs)[4],
                       const int64_t (&os)[4], const void* q, const void* k, const void* v, const void* o) {
    if (d.dtype != B2A_F16 && d.dtype != B2A_BF16) return false;
    if (d.D != kHeadDim || d.Dv != kHeadDim) return false;
    if (static_cast<long long>(d.B) * d.Hkv > 65535) return false;
    auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    if (!al(q) || !al(k) || !al(v) || !al(o)) return false;
    if (!strides_ok(qs, d.B, d.Hq, d.Sq) || !strides_ok(ks, d.B, d.Hkv, d.Skv) || !strides_ok(vs, d.B, d.Hkv, d.Skv) ||
        !strides_ok(os, d.B, d.Hq, d.Sq))
        return false;
    return encode_fn() != nullptr;
}

bool sdpa_tc_mask_supported(const b2a_sdpa_desc& d, const void* mask) {
    // the mask is read in 16-byte pieces along the keys: unit stride there, every row start 16-byte aligned, and a
    // key count that is a whole number of pieces
    if (d.mask_kind != B2A_MASK_BOOL && d.mask_kind != B2A_MASK_ADD) return false;
    const int es = d.mask_kind == B2A_MASK_BOOL ? 1 : 2;
    const int per_piece = 16 / es;
    if (d.mask_strides[3] != 1 || d.Skv % per_piece != 0) return false;
    if ((reinterpret_cast<uintptr_t>(mask) & 15) != 0) return false;
    for (int i = 0; i < 3; ++i)
        if (d.mask_strides[i] < 0 || (d.mask_strides[i] * es) % 16 != 0) return false;
    return true;
}

int sdpa_tc_launch(const b2a_sdpa_desc& d, const int64_t (&qs)[4], const int64_t (&ks)[4], const int64_t (&vs)[4],
                   const int64_t (&os)[4], const void* q, const void* k, const void* v, void* o, int32_t* status,
                   cudaStream_t stream, const TcPeerOut* peer_out, const void* mask) {
    const bool bf16 = d.dtype == B2A_BF16;
    CUtensorMap mq, mk, mv, mo;
    if (!make_map(&mq, q, bf16, d.B, d.Hq, d.Sq, qs, 128) || !make_map(&mk, k, bf16, d.B, d.Hkv, d.Skv, ks, 128) ||
        !make_map(&mv, v, bf16, d.B, d.Hkv, d.Skv, vs, 128))
        return B2A_ERR_CUDA;
    TcPeers peers{};
    if (peer_out == nullptr) {
        if (!make_map(&mo, o, bf16, d.B, d.Hq, d.Sq, os, 32)) return B2A_ERR_CUDA;
    } else {
        mo = mq;  // not read
        const int64_t fs[4] = {static_cast<int64_t>(peer_out->hq_total) * d.Sq * kHeadDim,
                               static_cast<int64_t>(d.Sq) * kHeadDim, kHeadDim, 1};
        for (int r = 0; r < peer_out->world; ++r) {
            if (!make_map(&peers.out_map[r], peer_out->out_base[r], bf16, d.B, peer_out->hq_total, d.Sq, fs, 32))
                return B2A_ERR_CUDA;
            peers.flags[r] = peer_out->flags[r];
        }
        peers.done_counter = peer_out->done_counter;
        peers.world = peer_out->world;
        peers.rank = peer_out->rank;
        peers.head_offset = peer_out->head_offset;
        peers.step = peer_out->step;
        peers.light_first = peer_out->world >= 4 ? 1 : 0;
    }
    TcParams p{};
    p.B = d.B; p.Hq = d.Hq; p.Hkv = d.Hkv; p.G = d.Hq / d.Hkv; p.Sq = d.Sq; p.Skv = d.Skv;
    p.causal = d.causal;
    p.scale_log2 = d.scale * kLog2e;
    p.status = status;
    const int nrb = (d.Sq + kBM - 1) / kBM;
    const int pairs = (nrb * p.G + 1) / 2;
    const long long items = static_cast<long long>(pairs) * d.B * d.Hkv;
    if (items >= (1LL << 30)) return B2A_ERR_UNSUPPORTED;
    const int sms = device_sm_count();
    if (sms <= 0) return B2A_ERR_CUDA;
    dim3 grid(static_cast<unsigned>(items < sms ? items : sms));  // persistent CTAs, one per SM
    const int mask_kind = (mask != nullptr && !d.causal) ? d.mask_kind : B2A_MASK_NONE;
    if (mask_kind != B2A_MASK_NONE) {
        p.mask = static_cast<const uint8_t*>(mask);
        for (int i = 0; i < 3; ++i) p.mask_strides[i] = d.mask_strides[i];
    }
    static bool configured[3][2][64] = {};
    auto kern = mask_kind == B2A_MASK_BOOL  ? (bf16 ? attn_tc_kernel<true, 0, 1> : attn_tc_kernel<false, 0, 1>)
                : mask_kind == B2A_MASK_ADD ? (bf16 ? attn_tc_kernel<true, 0, 2> : attn_tc_kernel<false, 0, 2>)
                                            : (bf16 ? attn_tc_kernel<true, 0, 0> : attn_tc_kernel<false, 0, 0>);
    const int rc = configure_once(kern, configured[mask_kind][bf16]);
    if (rc != B2A_OK) return rc;
    kern<<<grid, kThreadsDense, kSmemBytes, stream>>>(mq, mk, mv, mo, p, peers);
    return cudaGetLastError() == cudaSuccess ? B2A_OK : B2A_ERR_CUDA;
}

int sdpa_peer_wait_launch(const int32_t* local_flags, int world, int32_t step, long long wait_ns, int32_t* status,
                          cudaStream_t stream) {
    return launch_overlapped(sdpa_peer_wait_kernel, dim3(1), dim3(32), 0, stream, local_flags, world, step, wait_ns, status) ==
                   cudaSuccess
               ? B2A_OK
               : B2A_ERR_CUDA;
}

bool paged_tc_supported(const b2a_paged_desc& d, const void* query, const void* out) {
    const int g = d.Hkv > 0 ? d.Hq / d.Hkv : 0;
    auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    return d.kv_dtype == B2A_U8 && (d.q_dtype == B2A_F16 || d.q_dtype == B2A_BF16) && d.D == kHeadDim &&
           d.Dv == kHeadDim && d.block_size == 16 && d.max_q_len >= 2 && g >= 1 &&
           d.Hkv <= 65535 && al(query) && al(out) && encode_fn() != nullptr;
}

// upper bound on the (sequence, tile pair) items of a step
static int paged_tc_capacity(const b2a_paged_desc& d) {
    const long long g = d.Hq / d.Hkv;
    const long long rb = d.prefill_row_blocks > 0 ? d.prefill_row_blocks
                                                  : static_cast<long long>(d.num_tokens) / 128 + d.num_seqs;
    const long long cap = (rb * g + 1) / 2 + (rb < d.num_seqs ? rb : d.num_seqs);  // + one round-up per sequence
    return static_cast<int>(cap < 1 ? 1 : cap);
}

// Layout of the prefill kernel's part of the workspace: [work list][kv_base per sequence][owner per 128-row group]
// [K scratch][V scratch]; the last three only when the caller gave prefill_kv_tokens.
namespace {
struct TcWorkspace {
    size_t kv_base_at, owner_at, k_at, v_at, total;
    int rows, groups;
};
TcWorkspace tc_workspace(const b2a_paged_desc& d) {
    auto up = [](size_t x, size_t a) { return (x + a - 1) / a * a; };
    TcWorkspace w{};
    size_t at = up(sizeof(int) * (kPlanHeaderInts + 2 * static_cast<size_t>(paged_tc_capacity(d))), 16);
    if (d.prefill_kv_tokens > 0) {
        w.rows = (d.prefill_kv_tokens + 127) / 128 * 128;
        w.groups = w.rows / 128;
        w.kv_base_at = at;
        at = up(at + sizeof(int) * static_cast<size_t>(d.num_seqs), 16);
        w.owner_at = at;
        at = up(at + sizeof(int) * static_cast<size_t>(w.groups), 256);
        const size_t scratch = static_cast<size_t>(d.Hkv) * w.rows * kHeadDim * 2;
        w.k_at = at;
        w.v_at = at + scratch;
        at += 2 * scratch;
    }
    w.total = at;
    return w;
}
}  // namespace

size_t paged_tc_plan_bytes(const b2a_paged_desc& d) { return tc_workspace(d).total; }

int paged_tc_launch(const b2a_paged_desc& d, const void* query, const void* k_cache, const void* v_cache,
                    const PagedTables& t, void* out, void* plan_ws, int32_t* status, cudaStream_t stream,
                    bool* decode_may_overlap) {
    const bool bf16 = d.q_dtype == B2A_BF16;
    const int capacity = paged_tc_capacity(d);
    const TcWorkspace w = tc_workspace(d);
    const bool gathered = w.rows > 0;
    char* ws = static_cast<char*>(plan_ws);
    int* kv_base = gathered ? reinterpret_cast<int*>(ws + w.kv_base_at) : nullptr;
    int* owner = gathered ? reinterpret_cast<int*>(ws + w.owner_at) : nullptr;
    const int sms = device_sm_count();
    if (sms <= 0) return B2A_ERR_CUDA;
    const long long bound = static_cast<long long>(capacity) * d.Hkv;
    const int attention_ctas = static_cast<int>(bound < sms ? bound : sms);  // persistent CTAs over the sorted list
    // The decode rows may run beside the prefill rows when the attention kernel is the persistent one (one CTA per SM
    // at most, so what it leaves free is whole SMs) and the caller launches the decode kernel right behind it.
    const bool share = gathered && decode_may_overlap != nullptr;
    if (decode_may_overlap != nullptr) *decode_may_overlap = share;
    if (launch_overlapped(paged_tc_plan_kernel, dim3(1), dim3(256), 0, stream, t, d.Hq / d.Hkv, d.Hkv, capacity,
                          static_cast<int*>(plan_ws), status, kv_base, owner, w.groups, attention_ctas,
                          share ? 1 : 0) != cudaSuccess)
        return B2A_ERR_CUDA;
    // the step's query matrix [tokens, Hq*128] as a [1, Hq, tokens, 128] view
    const int64_t qs[4] = {static_cast<int64_t>(d.num_tokens) * d.Hq * kHeadDim, kHeadDim,
                           static_cast<int64_t>(d.Hq) * kHeadDim, 1};
    CUtensorMap mq, mk, mv;
    if (!make_map(&mq, query, bf16, 1, d.Hq, d.num_tokens, qs, 128)) return B2A_ERR_CUDA;
    mk = mv = mq;  // not read unless K/V are gathered
    if (gathered) {
        uint16_t* ks = reinterpret_cast<uint16_t*>(ws + w.k_at);
        uint16_t* vs = reinterpret_cast<uint16_t*>(ws + w.v_at);
        if (launch_overlapped(paged_gather_kernel, dim3(w.rows / 16, d.Hkv), dim3(128), 0, stream, t,
                              static_cast<const uint8_t*>(k_cache), static_cast<const uint8_t*>(v_cache), d.Hkv,
                              static_cast<const int*>(kv_base), static_cast<const int*>(owner), w.rows, ks, vs,
                              status) != cudaSuccess)
            return B2A_ERR_CUDA;
        // the scratch as a [1, Hkv, rows, 128] f16 tensor
        const int64_t ss[4] = {static_cast<int64_t>(d.Hkv) * w.rows * kHeadDim, static_cast<int64_t>(w.rows) * kHeadDim,
                               kHeadDim, 1};
        if (!make_map(&mk, ks, false, 1, d.Hkv, w.rows, ss, 128) || !make_map(&mv, vs, false, 1, d.Hkv, w.rows, ss, 128))
            return B2A_ERR_CUDA;
    }
    TcParams p{};
    p.B = 1; p.Hq = d.Hq; p.Hkv = d.Hkv; p.G = d.Hq / d.Hkv; p.Sq = 0; p.Skv = 0;
    p.causal = 1;
    p.window = d.sliding_window;
    p.scale_log2 = d.scale * kLog2e;
    p.status = status;
    p.k_cache = static_cast<const uint8_t*>(k_cache);
    p.v_cache = static_cast<const uint8_t*>(v_cache);
    p.t = t;
    p.out = out;
    p.plan = static_cast<const int*>(plan_ws);
    p.kv_base = kv_base;
    dim3 grid(capacity, d.Hkv, 1);
    TcPeers peers{};
    if (gathered) {
        grid = dim3(static_cast<unsigned>(attention_ctas));
        static bool configured[2][64] = {};
        auto kern = bf16 ? attn_tc_kernel<true, 2> : attn_tc_kernel<false, 2>;
        const int rc = configure_once(kern, configured[bf16]);
        if (rc != B2A_OK) return rc;
        kern<<<grid, kThreadsDense, kSmemBytes, stream>>>(mq, mk, mv, mq, p, peers);
    } else {
        static bool configured[2][64] = {};
        auto kern = bf16 ? attn_tc_kernel<true, 1> : attn_tc_kernel<false, 1>;
        const int rc = configure_once(kern, configured[bf16]);
        if (rc != B2A_OK) return rc;
        kern<<<grid, kThreadsPaged, kSmemBytes, stream>>>(mq, mq, mq, mq, p, peers);  // only the Q map is read
    }
    return cudaGetLastError() == cudaSuccess ? B2A_OK : B2A_ERR_CUDA;
}

}  // namespace b2a
