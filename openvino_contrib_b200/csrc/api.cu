// extern "C" entry points of libb2a.so: host-side validation and dispatch, nothing else.
#include <atomic>
#include <cmath>
#include <cstring>

#include "launch.cuh"

namespace b2a {

int device_sm_count() {
    static std::atomic<int> cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (dev >= 0 && dev < 64) {
        const int c = cached[dev].load(std::memory_order_relaxed);
        if (c > 0) return c;
    }
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    if (dev >= 0 && dev < 64) cached[dev].store(n, std::memory_order_relaxed);
    return n;
}

int resolve_paged_desc(const b2a_paged_desc* desc, b2a_paged_desc& d) {
    if (desc == nullptr) return B2A_ERR_NULL;
    d = *desc;
    if (d.q_dtype != B2A_F32 && d.q_dtype != B2A_F16 && d.q_dtype != B2A_BF16) return B2A_ERR_DTYPE;
    if (d.kv_dtype != B2A_U8 && d.kv_dtype != B2A_F16 && d.kv_dtype != B2A_BF16) return B2A_ERR_DTYPE;
    if (d.Hq <= 0 || d.Hkv <= 0 || d.D <= 0 || d.Dv <= 0 || d.block_size <= 0) return B2A_ERR_DIM;
    if (d.Hq % d.Hkv != 0 || d.Hq > 65535) return B2A_ERR_DIM;
    if (d.num_seqs < 0 || d.num_seqs > 65535 || d.num_tokens < 0 || d.num_blocks_total < 0) return B2A_ERR_DIM;
    if (d.max_context_len < 0 || d.max_q_len < 0 || d.sliding_window < 0) return B2A_ERR_DIM;
    if (d.kv_dtype == B2A_U8 && ((d.block_size * d.D) % 2 != 0 || (d.block_size * d.Dv) % 2 != 0)) return B2A_ERR_ALIGN;
    if (!(d.scale >= 0.f) || std::isinf(d.scale)) return B2A_ERR_DIM;
    if (d.scale == 0.f) d.scale = 1.0f / std::sqrt(static_cast<float>(d.D));
    return B2A_OK;
}

namespace {

size_t elem_size(int dtype) {
    switch (dtype) {
        case B2A_F32: return 4;
        case B2A_F16:
        case B2A_BF16: return 2;
        case B2A_U8: return 1;
        default: return 0;
    }
}

bool all_zero(const int64_t (&s)[4]) { return s[0] == 0 && s[1] == 0 && s[2] == 0 && s[3] == 0; }

void contiguous(int64_t (&s)[4], int64_t d0, int64_t d1, int64_t d2, int64_t d3) {
    (void)d0;
    s[3] = 1;
    s[2] = d3;
    s[1] = d2 * d3;
    s[0] = d1 * d2 * d3;
}

struct SdpaResolved {
    b2a_sdpa_desc d;
    int64_t qs[4], ks[4], vs[4], os[4];
};

int resolve_sdpa(const b2a_sdpa_desc* desc, SdpaResolved& r) {
    if (desc == nullptr) return B2A_ERR_NULL;
    r.d = *desc;
    b2a_sdpa_desc& d = r.d;
    if (d.dtype != B2A_F32 && d.dtype != B2A_F16 && d.dtype != B2A_BF16) return B2A_ERR_DTYPE;
    if (d.B <= 0 || d.Hq <= 0 || d.Hkv <= 0 || d.Sq <= 0 || d.Skv <= 0 || d.D <= 0 || d.Dv <= 0) return B2A_ERR_DIM;
    if (d.Hq % d.Hkv != 0) return B2A_ERR_DIM;
    if (d.Hq > 65535 || d.B > 65535) return B2A_ERR_DIM;
    if (d.mask_kind < B2A_MASK_NONE || d.mask_kind > B2A_MASK_ADD) return B2A_ERR_DIM;
    if (!(d.scale >= 0.f) || std::isinf(d.scale)) return B2A_ERR_DIM;
    if (d.scale == 0.f) d.scale = 1.0f / std::sqrt(static_cast<float>(d.D));
    std::memcpy(r.qs, d.q_strides, sizeof r.qs);
    std::memcpy(r.ks, d.k_strides, sizeof r.ks);
    std::memcpy(r.vs, d.v_strides, sizeof r.vs);
    std::memcpy(r.os, d.o_strides, sizeof r.os);
    if (all_zero(r.qs)) contiguous(r.qs, d.B, d.Hq, d.Sq, d.D);
    if (all_zero(r.ks)) contiguous(r.ks, d.B, d.Hkv, d.Skv, d.D);
    if (all_zero(r.vs)) contiguous(r.vs, d.B, d.Hkv, d.Skv, d.Dv);
    if (all_zero(r.os)) contiguous(r.os, d.B, d.Hq, d.Sq, d.Dv);
    if (r.qs[3] != 1 || r.ks[3] != 1 || r.vs[3] != 1 || r.os[3] != 1) return B2A_ERR_ALIGN;
    return B2A_OK;
}

bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// One event per host thread and device, created at the thread's first mixed step on that device and kept: it is
// recorded and waited for within one call, so calls of different threads never share one.
cudaEvent_t step_join_event() {
    thread_local cudaEvent_t events[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (events[dev] == nullptr && cudaEventCreateWithFlags(&events[dev], cudaEventDisableTiming) != cudaSuccess) {
        events[dev] = nullptr;
        (void)cudaGetLastError();
    }
    return events[dev];
}

PagedTables tables_of(const b2a_paged_desc& d, const int32_t* past_lens, const int32_t* subsequence_begins,
                      const int32_t* block_indices, const int32_t* block_indices_begins) {
    return PagedTables{past_lens, subsequence_begins, block_indices, block_indices_begins,
                       d.num_seqs, d.num_tokens, d.num_blocks_total, d.block_size};
}

}  // namespace
}  // namespace b2a

using namespace b2a;

extern "C" {

int b2a_version(void) { return 100; }

const char* b2a_status_string(int status) {
    switch (status) {
        case B2A_OK: return "ok";
        case B2A_ERR_NULL: return "a required pointer is NULL";
        case B2A_ERR_DIM: return "invalid or inconsistent dimension";
        case B2A_ERR_DTYPE: return "unsupported element type";
        case B2A_ERR_ALIGN: return "pointer or stride alignment not supported";
        case B2A_ERR_WORKSPACE: return "workspace missing or too small";
        case B2A_ERR_CUDA: return "CUDA runtime error";
        case B2A_ERR_UNSUPPORTED: return "no kernel for this configuration";
        case B2A_ERR_CAPACITY: return "capacity exceeded";
        case B2A_ERR_NOT_FOUND: return "unknown sequence";
        case B2A_ERR_SCRATCH_LIMIT: return "the step needs more split-K scratch than the library's built-in 16 MiB";
        default: return "unknown status";
    }
}

int b2a_sdpa_workspace_bytes(const b2a_sdpa_desc* desc, int sm_count, size_t* out_bytes) {
    (void)sm_count;
    if (out_bytes == nullptr) return B2A_ERR_NULL;
    SdpaResolved r;
    const int rc = resolve_sdpa(desc, r);
    if (rc != B2A_OK) return rc;
    *out_bytes = 0;  // both SDPA kernels keep their state on chip
    return B2A_OK;
}

int b2a_sdpa_forward(const b2a_sdpa_desc* desc, const void* q, const void* k, const void* v, const void* mask,
                     void* o, void* workspace, size_t workspace_bytes, int32_t* status, b2a_stream_t stream) {
    (void)workspace;
    (void)workspace_bytes;
    SdpaResolved r;
    const int rc = resolve_sdpa(desc, r);
    if (rc != B2A_OK) return rc;
    if (q == nullptr || k == nullptr || v == nullptr || o == nullptr) return B2A_ERR_NULL;
    const bool masked = !r.d.causal && r.d.mask_kind != B2A_MASK_NONE;
    if (masked && mask == nullptr) return B2A_ERR_NULL;
    const size_t es = elem_size(r.d.dtype);
    if (!aligned(q, es) || !aligned(k, es) || !aligned(v, es) || !aligned(o, es)) return B2A_ERR_ALIGN;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    if (sdpa_tc_supported(r.d, r.qs, r.ks, r.vs, r.os, q, k, v, o) && (!masked || sdpa_tc_mask_supported(r.d, mask)))
        return sdpa_tc_launch(r.d, r.qs, r.ks, r.vs, r.os, q, k, v, o, status, s, nullptr, masked ? mask : nullptr);
    return sdpa_generic_launch(r.d, r.qs, r.ks, r.vs, r.os, q, k, v, mask, o, status, s);
}

size_t b2a_paged_chunk_bytes(int32_t kv_dtype, int32_t block_size, int32_t d) {
    if (block_size <= 0 || d <= 0) return 0;
    if (kv_dtype == B2A_U8) return u8_chunk_bytes(block_size, d);
    if (kv_dtype == B2A_F16 || kv_dtype == B2A_BF16) return static_cast<size_t>(block_size) * d * 2;
    return 0;
}

int b2a_paged_workspace_bytes(const b2a_paged_desc* desc, int sm_count, size_t* out_bytes) {
    if (out_bytes == nullptr) return B2A_ERR_NULL;
    b2a_paged_desc d;
    const int rc = resolve_paged_desc(desc, d);
    if (rc != B2A_OK) return rc;
    if (sm_count <= 0) sm_count = device_sm_count();
    if (sm_count <= 0) sm_count = 148;
    // pure decode steps and mixed steps both run the split-K decode kernel for their one-token sequences
    // layout: [split-K partials of the decode kernel, rounded up to 16 bytes][work list of the prefill kernel]
    size_t bytes = 0;
    if (paged_decode_geometry_ok(d)) {
        bytes = (paged_decode_plan(d, sm_count).workspace_bytes + 15) & ~static_cast<size_t>(15);
        if (d.max_q_len >= 2) bytes += paged_tc_plan_bytes(d);
    }
    *out_bytes = bytes;
    return B2A_OK;
}

int b2a_paged_kv_store(const b2a_paged_desc* desc, const void* key, const void* value, void* k_cache, void* v_cache,
                       const int32_t* past_lens, const int32_t* subsequence_begins, const int32_t* block_indices,
                       const int32_t* block_indices_begins, int32_t* status, b2a_stream_t stream) {
    b2a_paged_desc d;
    const int rc = resolve_paged_desc(desc, d);
    if (rc != B2A_OK) return rc;
    if (d.num_tokens == 0 || d.num_seqs == 0) return B2A_OK;
    if (key == nullptr || value == nullptr || k_cache == nullptr || v_cache == nullptr || past_lens == nullptr ||
        subsequence_begins == nullptr || block_indices == nullptr || block_indices_begins == nullptr)
        return B2A_ERR_NULL;
    if (!aligned(k_cache, 16) || !aligned(v_cache, 16)) return B2A_ERR_ALIGN;
    return paged_kv_store_launch(d, key, value, k_cache, v_cache,
                                 tables_of(d, past_lens, subsequence_begins, block_indices, block_indices_begins),
                                 status, reinterpret_cast<cudaStream_t>(stream));
}

int b2a_paged_kv_store_rope(const b2a_paged_desc* desc, const void* key, const void* value, void* k_cache, void* v_cache,
                            const int32_t* past_lens, const int32_t* subsequence_begins, const int32_t* block_indices,
                            const int32_t* block_indices_begins, const float* cos_table, const float* sin_table,
                            int32_t rotary_dim, int32_t table_positions, int32_t* status, b2a_stream_t stream) {
    b2a_paged_desc d;
    const int rc = resolve_paged_desc(desc, d);
    if (rc != B2A_OK) return rc;
    if (d.num_tokens == 0 || d.num_seqs == 0) return B2A_OK;
    if (key == nullptr || value == nullptr || k_cache == nullptr || v_cache == nullptr || past_lens == nullptr ||
        subsequence_begins == nullptr || block_indices == nullptr || block_indices_begins == nullptr ||
        cos_table == nullptr || sin_table == nullptr)
        return B2A_ERR_NULL;
    if (rotary_dim <= 0 || rotary_dim % 2 != 0 || rotary_dim > d.D || table_positions <= 0) return B2A_ERR_DIM;
    if (!aligned(k_cache, 16) || !aligned(v_cache, 16) || !aligned(cos_table, 4) || !aligned(sin_table, 4)) return B2A_ERR_ALIGN;
    const RopeTables rope{cos_table, sin_table, rotary_dim, table_positions};
    return paged_kv_store_launch(d, key, value, k_cache, v_cache,
                                 tables_of(d, past_lens, subsequence_begins, block_indices, block_indices_begins),
                                 status, reinterpret_cast<cudaStream_t>(stream), &rope);
}

int b2a_paged_attention(const b2a_paged_desc* desc, const void* query, const void* k_cache, const void* v_cache,
                        const int32_t* past_lens, const int32_t* subsequence_begins, const int32_t* block_indices,
                        const int32_t* block_indices_begins, void* out, void* workspace, size_t workspace_bytes,
                        int32_t* status, b2a_stream_t stream) {
    b2a_paged_desc d;
    const int rc = resolve_paged_desc(desc, d);
    if (rc != B2A_OK) return rc;
    if (d.num_tokens == 0 || d.num_seqs == 0) return B2A_OK;
    if (query == nullptr || k_cache == nullptr || v_cache == nullptr || out == nullptr || past_lens == nullptr ||
        subsequence_begins == nullptr || block_indices == nullptr || block_indices_begins == nullptr)
        return B2A_ERR_NULL;
    if (d.max_q_len <= 0 || d.max_context_len <= 0) return B2A_ERR_DIM;
    if (!aligned(k_cache, 16) || !aligned(v_cache, 16) || !aligned(query, 16) || !aligned(out, 16)) return B2A_ERR_ALIGN;
    const PagedTables t = tables_of(d, past_lens, subsequence_begins, block_indices, block_indices_begins);
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    if (paged_decode_supported(d)) {
        const int sms = device_sm_count();
        if (sms <= 0) return B2A_ERR_CUDA;
        const DecodePlan plan = paged_decode_plan(d, sms);
        if (workspace == nullptr || workspace_bytes < plan.workspace_bytes) return B2A_ERR_WORKSPACE;
        if (!aligned(workspace, 16)) return B2A_ERR_ALIGN;
        return paged_decode_launch(d, plan, query, k_cache, v_cache, t, out, workspace, status, s);
    }
    if (paged_decode_geometry_ok(d) && paged_tc_supported(d, query, out)) {
        // mixed step: multi-token sequences on the tensor-core kernel, one-token sequences on the decode kernel
        const int sms = device_sm_count();
        if (sms <= 0) return B2A_ERR_CUDA;
        const DecodePlan plan = paged_decode_plan(d, sms);
        const size_t list_at = (plan.workspace_bytes + 15) & ~static_cast<size_t>(15);
        if (workspace == nullptr || workspace_bytes < list_at + paged_tc_plan_bytes(d)) return B2A_ERR_WORKSPACE;
        if (!aligned(workspace, 16)) return B2A_ERR_ALIGN;
        // The persistent prefill kernel leaves whole SMs free for the decode rows, which then run beside it.  An
        // event recorded right behind it lets the step's last kernel wait for it explicitly.
        cudaEvent_t join = step_join_event();
        bool beside = false;
        const int rc2 = paged_tc_launch(d, query, k_cache, v_cache, t, out, static_cast<char*>(workspace) + list_at,
                                        status, s, join != nullptr ? &beside : nullptr);
        if (rc2 != B2A_OK) return rc2;
        if (beside && cudaEventRecord(join, s) != cudaSuccess) return B2A_ERR_CUDA;
        return paged_decode_launch(d, plan, query, k_cache, v_cache, t, out, workspace, status, s, nullptr,
                                   beside ? join : nullptr);
    }
    return paged_generic_launch(d, query, k_cache, v_cache, t, out, status, s);
}

int b2a_paged_attention_noalloc(const b2a_paged_desc* desc, const void* query, const void* k_cache,
                                const void* v_cache, const int32_t* past_lens, const int32_t* subsequence_begins,
                                const int32_t* block_indices, const int32_t* block_indices_begins, void* out,
                                int32_t* status, b2a_stream_t stream) {
    b2a_paged_desc d;
    const int rc = resolve_paged_desc(desc, d);
    if (rc != B2A_OK) return rc;
    if (d.num_tokens == 0 || d.num_seqs == 0) return B2A_OK;
    if (query == nullptr || k_cache == nullptr || v_cache == nullptr || out == nullptr || past_lens == nullptr ||
        subsequence_begins == nullptr || block_indices == nullptr || block_indices_begins == nullptr)
        return B2A_ERR_NULL;
    if (d.max_q_len <= 0 || d.max_context_len <= 0) return B2A_ERR_DIM;
    if (!paged_decode_supported(d)) return B2A_ERR_UNSUPPORTED;
    if (!aligned(k_cache, 16) || !aligned(v_cache, 16) || !aligned(query, 16) || !aligned(out, 16)) return B2A_ERR_ALIGN;
    const int sms = device_sm_count();
    if (sms <= 0) return B2A_ERR_CUDA;
    return paged_decode_launch_builtin_scratch(
        d, paged_decode_plan(d, sms), query, k_cache, v_cache,
        tables_of(d, past_lens, subsequence_begins, block_indices, block_indices_begins), out, status,
        reinterpret_cast<cudaStream_t>(stream));
}

int b2a_paged_scores_workspace_bytes(const b2a_paged_desc* desc, int sm_count, size_t* out_bytes) {
    if (out_bytes == nullptr) return B2A_ERR_NULL;
    b2a_paged_desc d;
    const int rc = resolve_paged_desc(desc, d);
    if (rc != B2A_OK) return rc;
    if (d.max_context_len <= 0) return B2A_ERR_DIM;
    if (!paged_scores_supported(d)) return B2A_ERR_UNSUPPORTED;
    if (sm_count <= 0) sm_count = device_sm_count();
    if (sm_count <= 0) sm_count = 148;
    *out_bytes = paged_scores_plan(d, sm_count).workspace_bytes;
    return B2A_OK;
}

int b2a_paged_last_token_scores(const b2a_paged_desc* desc, const void* query, const void* k_cache,
                                const int32_t* past_lens, const int32_t* subsequence_begins,
                                const int32_t* block_indices, const int32_t* block_indices_begins, float* scores,
                                int64_t scores_capacity, int32_t* score_begins, void* workspace, size_t workspace_bytes,
                                int32_t* status, b2a_stream_t stream) {
    b2a_paged_desc d;
    const int rc = resolve_paged_desc(desc, d);
    if (rc != B2A_OK) return rc;
    if (d.num_seqs == 0) return B2A_OK;
    if (query == nullptr || k_cache == nullptr || scores == nullptr || score_begins == nullptr || past_lens == nullptr ||
        subsequence_begins == nullptr || block_indices == nullptr || block_indices_begins == nullptr)
        return B2A_ERR_NULL;
    if (d.max_context_len <= 0 || scores_capacity < 0) return B2A_ERR_DIM;
    if (!paged_scores_supported(d)) return B2A_ERR_UNSUPPORTED;
    if (!aligned(k_cache, 16) || !aligned(query, 16)) return B2A_ERR_ALIGN;
    const int sms = device_sm_count();
    if (sms <= 0) return B2A_ERR_CUDA;
    const ScorePlan plan = paged_scores_plan(d, sms);
    if (workspace == nullptr || workspace_bytes < plan.workspace_bytes) return B2A_ERR_WORKSPACE;
    if (!aligned(workspace, 16)) return B2A_ERR_ALIGN;
    return paged_scores_launch(d, plan, query, k_cache,
                               tables_of(d, past_lens, subsequence_begins, block_indices, block_indices_begins), scores,
                               scores_capacity, score_begins, workspace, status, reinterpret_cast<cudaStream_t>(stream));
}

}  // extern "C"
