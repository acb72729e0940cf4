// Host-side launchers of the kernels, one per .cu file; api.cu validates descriptors and dispatches to these.
#pragma once

#include <type_traits>

#include "common.cuh"

namespace b2a {

// attn_generic.cu
int sdpa_generic_launch(const b2a_sdpa_desc& d, const int64_t (&qs)[4], const int64_t (&ks)[4],
                        const int64_t (&vs)[4], const int64_t (&os)[4], const void* q, const void* k, const void* v,
                        const void* mask, void* o, int32_t* status, cudaStream_t stream);
int paged_generic_launch(const b2a_paged_desc& d, const void* query, const void* k_cache, const void* v_cache,
                         const PagedTables& t, void* out, int32_t* status, cudaStream_t stream);

// paged_kv_store.cu
struct RopeTables {  // rotary embedding of the key rows: f32 tables [positions][rotary_dim / 2] in device memory
    const float* cos;
    const float* sin;
    int rotary_dim, positions;
};
int paged_kv_store_launch(const b2a_paged_desc& d, const void* key, const void* value, void* k_cache, void* v_cache,
                          const PagedTables& t, int32_t* status, cudaStream_t stream, const RopeTables* rope = nullptr);

// Head-sharded decode across the GPUs of a node: where the decode kernel delivers a rank's output columns.
// Every rank owns two full-width staging buffers, flag arrays and counters, all inside one allocation that its peers
// map (shard_group.cu).  The decode kernel of rank r merges the splits of a (sequence, KV head) in the CTA that
// finished last (ticket counters) and stores the rows into the memory of EVERY rank - plain peer stores over NVLink;
// no collective library call is on the path.
constexpr int kMaxShardWorld = 8;
struct PeerPush {
    void* staging[kMaxShardWorld][2];  // [rank][step parity]: that rank's staging buffers as mapped here
    int32_t* flags[kMaxShardWorld];    // [rank]: that rank's "step published" flags (one int per source rank)
    int32_t* step_counter;             // local: number of steps completed so far
    int32_t* done_counter;             // local: CTAs finished in the current step (self-resetting)
    int rank, world;                   // world == 0: not sharded
    int row_elems;                     // elements of one full-width output row (Hq_total * D)
    int col_offset;                    // first column of this rank's heads
    // ll != 0, low-latency form (caller's output buffer; staging buffers twice as large as the output): every pair of
    // 16-bit values travels as one 8-byte store {two values, step number} into staging[r][step parity], which arrives
    // whole or not at all, so the receiving kernel simply polls each word for the step number - no fence, no flag
    // round trip, no rendezvous of whole kernels.
    // ll == 0, in place: the rows go into staging[r][0] of every rank r - the ranks' fixed output buffers, read where
    // they are.  A rank announces in started[r][rank] that it has begun step s, i.e. that its readers of step s-1 are
    // done; nobody stores into a rank's buffer for step s before that; the grid's last CTA publishes the step in
    // flags[r][rank] and waits for the other ranks.
    int ll;
    int receive_in_kernel;             // ll: the decode kernel's CTAs also receive the rows (no second kernel)
    int32_t* group_counters;           // local: one ticket counter per (sequence, KV head), self-resetting
    int32_t* started[kMaxShardWorld];  // [rank]: that rank's array of "rank i has begun step s" (one int per source rank)
    long long wait_ns;                 // bound of every wait on another rank, in nanoseconds of wall-clock time
};

// paged_decode.cu — split-K decode over a u8 cache (D = Dv = 128, block 16, one query token per sequence)
struct DecodePlan {
    int blocks_per_cta;  // logical KV blocks one CTA walks
    int max_splits;      // CTAs per (sequence, KV head)
    size_t workspace_bytes;
};
bool paged_decode_supported(const b2a_paged_desc& d);   // a pure decode step
bool paged_decode_geometry_ok(const b2a_paged_desc& d); // the kernel's shape limits, whatever the step's mix
DecodePlan paged_decode_plan(const b2a_paged_desc& d, int sm_count);
// beside_predecessor != nullptr: the kernel before this launch on the stream is the prefill kernel of the same mixed
// step, which has already waited for everything the decode rows read (cache, tables, query) and writes nothing they
// touch; the event was recorded right behind it.  The decode kernel then starts as soon as that kernel's CTAs are
// seated, on the SMs it leaves free, instead of after it, and does not wait for it.  The merge kernel is launched
// the ordinary way behind a wait on the event, so it - and whatever follows it on the stream - comes after both.
int paged_decode_launch(const b2a_paged_desc& d, const DecodePlan& plan, const void* query, const void* k_cache,
                        const void* v_cache, const PagedTables& t, void* out, void* workspace, int32_t* status,
                        cudaStream_t stream, const PeerPush* push = nullptr, cudaEvent_t beside_predecessor = nullptr);

// Same launch with the split-K partials in the library's built-in device array instead of a caller workspace.
int paged_decode_launch_builtin_scratch(const b2a_paged_desc& d, const DecodePlan& plan, const void* query,
                                        const void* k_cache, const void* v_cache, const PagedTables& t, void* out,
                                        int32_t* status, cudaStream_t stream);

// paged_scores.cu — per-key attention probabilities of every sequence's last query token, summed over the heads
struct ScorePlan {
    int blocks_per_cta, max_splits;
    size_t workspace_bytes;
};
bool paged_scores_supported(const b2a_paged_desc& d);
ScorePlan paged_scores_plan(const b2a_paged_desc& d, int sm_count);
int paged_scores_launch(const b2a_paged_desc& d, const ScorePlan& plan, const void* query, const void* k_cache,
                        const PagedTables& t, float* scores, long long capacity, int32_t* score_begins, void* workspace,
                        int32_t* status, cudaStream_t stream);

// sdpa_tcgen05.cu — TMA + tcgen05 flash prefill (f16 / bf16, D = Dv = 128)
bool sdpa_tc_supported(const b2a_sdpa_desc& d, const int64_t (&qs)[4], const int64_t (&ks)[4],
                       const int64_t (&vs)[4], const int64_t (&os)[4], const void* q, const void* k, const void* v,
                       const void* o);
// Head-sharded prefill: where the kernel's epilogue sends its output tiles.  Every rank owns a full-width
// [B, Hq_total, Sq, 128] output buffer that its peers map; a CTA stores each finished 32-row slab into the buffer of
// EVERY rank with one TMA store per rank (the all-gather happens tile by tile while other CTAs still compute), the
// last CTA of the grid publishes `step` in every rank's flags[rank], and sdpa_peer_wait_launch makes the stream wait
// (bounded) until all ranks have published.
struct TcPeerOut {
    void* out_base[kMaxShardWorld];    // [rank]: that rank's output buffer of this step, as mapped here
    int32_t* flags[kMaxShardWorld];    // [rank]: that rank's flag array (one int per source rank)
    int32_t* done_counter;             // local: CTAs finished in the current step (self-resetting)
    int rank, world;
    int hq_total;                      // heads of the full output
    int head_offset;                   // first head of this rank
    int32_t step;                      // value published when the step is complete (increases by one per step)
    long long wait_ns;                 // bound of the wait for the other ranks, nanoseconds of wall-clock time
};
// mask != nullptr (and d.causal == 0): the attention mask of the descriptor, when sdpa_tc_mask_supported says the
// kernel can read it (16-byte pieces along the keys)
bool sdpa_tc_mask_supported(const b2a_sdpa_desc& d, const void* mask);
int sdpa_tc_launch(const b2a_sdpa_desc& d, const int64_t (&qs)[4], const int64_t (&ks)[4], const int64_t (&vs)[4],
                   const int64_t (&os)[4], const void* q, const void* k, const void* v, void* o, int32_t* status,
                   cudaStream_t stream, const TcPeerOut* peers = nullptr, const void* mask = nullptr);
int sdpa_peer_wait_launch(const int32_t* local_flags, int world, int32_t step, long long wait_ns, int32_t* status,
                          cudaStream_t stream);

// the same kernel body over a paged u8 cache: the multi-token sequences of a step (sequences with one new token are
// left to the decode kernel, which in turn skips the others)
bool paged_tc_supported(const b2a_paged_desc& d, const void* query, const void* out);
size_t paged_tc_plan_bytes(const b2a_paged_desc& d);  // scratch for the device-built work list
// decode_may_overlap (optional, out): true when the attention kernel just launched leaves whole SMs free for the decode
// rows of the same step, which the caller then launches with paged_decode_launch(..., beside_predecessor = true)
int paged_tc_launch(const b2a_paged_desc& d, const void* query, const void* k_cache, const void* v_cache,
                    const PagedTables& t, void* out, void* plan_ws, int32_t* status, cudaStream_t stream,
                    bool* decode_may_overlap = nullptr);

int device_sm_count();

// api.cu — validation of a paged descriptor shared by the entry points (fills the default scale)
int resolve_paged_desc(const b2a_paged_desc* desc, b2a_paged_desc& out);

}  // namespace b2a
