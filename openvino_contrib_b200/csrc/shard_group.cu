// Head-sharded attention across the GPUs of one node without a collective library on the data path.
//
// A shard group is one device allocation per rank, [staging 0 | staging 1 | flags | counters | tickets], which every
// peer maps - through CUDA IPC when the ranks are processes, by pointer when one process drives several ranks.
// b2a_paged_attention_sharded runs the split-K decode on this rank's KV heads; the decode kernel itself merges the
// splits and stores the rank's output columns into every rank's memory over NVLink (PeerPush in launch.cuh, kernels
// in paged_decode.cu).  b2a_sdpa_forward_sharded does the same for prefill: the tensor-core kernel's epilogue stores
// each output tile into every rank's buffer (TcPeerOut in launch.cuh), and the result is read in place.
// The reference never spans devices (one independent plugin configuration per device id,
// modules/nvidia_plugin/src/cuda_plugin.cpp:25-32), so nothing here has a counterpart there.
#include <cmath>
#include <cstring>
#include <new>

#include "launch.cuh"

namespace {
constexpr size_t kFlagsBytes = 256;     // decode: ints 0..7; prefill: ints 16..23; "step begun" of the one-kernel decode: ints 32..39
constexpr size_t kCountersBytes = 256;  // decode step counter at +0, decode done counter at +64, prefill done counter at +128
constexpr int kPrefillFlagOffset = 16;
constexpr int kStartedFlagOffset = 32;
constexpr size_t kGroupCounters = 16384;  // (sequence, KV head) tickets of the one-kernel decode step
enum { kModeUnset = 0, kModeDecode = 1, kModePrefill = 2, kModeDecodeInPlace = 3 };
size_t round_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
}  // namespace

struct b2a_shard_group {
    int rank = 0, world = 1, device = 0;
    size_t staging_bytes = 0;  // one staging buffer
    char* base[b2a::kMaxShardWorld] = {};  // [rank]: that rank's allocation as mapped in this process
    bool ipc_mapped[b2a::kMaxShardWorld] = {};  // base[r] came from cudaIpcOpenMemHandle (closed on destroy)
    bool connected = false;
    long long wait_ns = 1000000000LL;  // bound of every device-side wait on another rank
    int mode = kModeUnset;       // a group serves one kind of step: the two kinds alternate the staging halves differently
    int32_t prefill_step = 0;    // host-side count of prefill steps
    size_t total_bytes() const { return 2 * staging_bytes + kFlagsBytes + kCountersBytes + kGroupCounters * sizeof(int32_t); }
};

extern "C" {

int b2a_shard_group_create(int rank, int world, size_t staging_bytes, b2a_shard_group** out) {
    if (out == nullptr) return B2A_ERR_NULL;
    if (world < 1 || world > b2a::kMaxShardWorld || rank < 0 || rank >= world || staging_bytes == 0) return B2A_ERR_DIM;
    auto* g = new (std::nothrow) b2a_shard_group();
    if (g == nullptr) return B2A_ERR_CAPACITY;
    g->rank = rank;
    g->world = world;
    g->staging_bytes = round_up(staging_bytes, 256);
    void* p = nullptr;
    if (cudaGetDevice(&g->device) != cudaSuccess || cudaMalloc(&p, g->total_bytes()) != cudaSuccess ||
        cudaMemset(p, 0, g->total_bytes()) != cudaSuccess) {
        if (p) cudaFree(p);
        delete g;
        return B2A_ERR_CUDA;
    }
    g->base[rank] = static_cast<char*>(p);
    g->connected = world == 1;
    *out = g;
    return B2A_OK;
}

int b2a_shard_group_handle(const b2a_shard_group* g, unsigned char handle[64]) {
    if (g == nullptr || handle == nullptr) return B2A_ERR_NULL;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, g->base[g->rank]) != cudaSuccess) return B2A_ERR_CUDA;
    std::memcpy(handle, &h, 64);
    return B2A_OK;
}

int b2a_shard_group_connect(b2a_shard_group* g, const unsigned char* handles) {
    if (g == nullptr || handles == nullptr) return B2A_ERR_NULL;
    for (int r = 0; r < g->world; ++r) {
        if (r == g->rank || g->base[r] != nullptr) continue;
        cudaIpcMemHandle_t h;
        std::memcpy(&h, handles + 64 * r, 64);
        void* p = nullptr;
        if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) return B2A_ERR_CUDA;
        g->base[r] = static_cast<char*>(p);
        g->ipc_mapped[r] = true;
    }
    g->connected = true;
    return B2A_OK;
}

int b2a_shard_group_connect_pointers(b2a_shard_group* g, void* const* bases) {
    if (g == nullptr || bases == nullptr) return B2A_ERR_NULL;
    for (int r = 0; r < g->world; ++r) {
        if (r == g->rank) continue;
        if (bases[r] == nullptr) return B2A_ERR_NULL;
        if (g->base[r] != nullptr && g->base[r] != bases[r]) return B2A_ERR_UNSUPPORTED;  // already connected elsewhere
        g->base[r] = static_cast<char*>(bases[r]);
    }
    g->connected = true;
    return B2A_OK;
}

int b2a_shard_group_set_wait_ms(b2a_shard_group* g, int milliseconds) {
    if (g == nullptr) return B2A_ERR_NULL;
    if (milliseconds <= 0) return B2A_ERR_DIM;
    g->wait_ns = static_cast<long long>(milliseconds) * 1000000LL;
    return B2A_OK;
}

int b2a_shard_group_reset(b2a_shard_group* g) {
    if (g == nullptr) return B2A_ERR_NULL;
    int prev = 0;
    if (cudaGetDevice(&prev) != cudaSuccess || cudaSetDevice(g->device) != cudaSuccess) return B2A_ERR_CUDA;
    // everything this rank enqueued has finished (with or without a timeout) before its memory is wiped
    const bool ok = cudaDeviceSynchronize() == cudaSuccess &&
                    cudaMemset(g->base[g->rank], 0, g->total_bytes()) == cudaSuccess &&
                    cudaDeviceSynchronize() == cudaSuccess;
    cudaSetDevice(prev);
    if (!ok) return B2A_ERR_CUDA;
    g->mode = kModeUnset;
    g->prefill_step = 0;
    return B2A_OK;
}

int b2a_shard_group_output(const b2a_shard_group* g, void** out) {
    if (g == nullptr || out == nullptr) return B2A_ERR_NULL;
    *out = g->base[g->rank];
    return B2A_OK;
}

void b2a_shard_group_destroy(b2a_shard_group* g) {
    if (g == nullptr) return;
    for (int r = 0; r < g->world; ++r) {
        if (g->base[r] == nullptr) continue;
        if (r == g->rank) cudaFree(g->base[r]);
        else if (g->ipc_mapped[r]) cudaIpcCloseMemHandle(g->base[r]);
    }
    delete g;
}

int b2a_paged_attention_sharded(b2a_shard_group* g, const b2a_paged_desc* local_desc, const void* query,
                                const void* k_cache, const void* v_cache, const int32_t* past_lens,
                                const int32_t* subsequence_begins, const int32_t* block_indices,
                                const int32_t* block_indices_begins, void* out_full, void* workspace,
                                size_t workspace_bytes, int32_t* status, b2a_stream_t stream) {
    using namespace b2a;
    if (g == nullptr || local_desc == nullptr) return B2A_ERR_NULL;
    if (!g->connected) return B2A_ERR_UNSUPPORTED;
    b2a_paged_desc d;
    const int rc = resolve_paged_desc(local_desc, d);  // the same validation as the single-GPU entry points
    if (rc != B2A_OK) return rc;
    if (d.num_tokens == 0 || d.num_seqs == 0) return B2A_OK;
    if (query == nullptr || k_cache == nullptr || v_cache == nullptr || out_full == nullptr || past_lens == nullptr ||
        subsequence_begins == nullptr || block_indices == nullptr || block_indices_begins == nullptr)
        return B2A_ERR_NULL;
    if (d.max_context_len <= 0) return B2A_ERR_DIM;
    if (!paged_decode_supported(d)) return B2A_ERR_UNSUPPORTED;  // decode steps only
    // out_full == the group's own buffer (b2a_shard_group_output): results are produced in place by one kernel
    const bool in_place = out_full == static_cast<void*>(g->base[g->rank]);
    const int want = in_place ? kModeDecodeInPlace : kModeDecode;
    if (g->mode != kModeUnset && g->mode != want) return B2A_ERR_UNSUPPORTED;
    if (static_cast<size_t>(d.num_seqs) * d.Hkv > kGroupCounters) return B2A_ERR_CAPACITY;
    const size_t row_bytes = static_cast<size_t>(d.Hq) * g->world * d.D * 2;
    // in place: the rows themselves; caller's buffer: every pair of values travels with the step number (8 bytes)
    if ((in_place ? 1 : 2) * static_cast<size_t>(d.num_tokens) * row_bytes > g->staging_bytes) return B2A_ERR_CAPACITY;
    auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    if (!al(k_cache) || !al(v_cache) || !al(query) || !al(out_full) || !al(workspace)) return B2A_ERR_ALIGN;
    const int sms = device_sm_count();
    if (sms <= 0) return B2A_ERR_CUDA;
    const DecodePlan plan = paged_decode_plan(d, sms);
    if (workspace == nullptr || workspace_bytes < plan.workspace_bytes) return B2A_ERR_WORKSPACE;
    PeerPush push{};
    for (int r = 0; r < g->world; ++r) {
        push.staging[r][0] = g->base[r];
        push.staging[r][1] = g->base[r] + g->staging_bytes;
        push.flags[r] = reinterpret_cast<int32_t*>(g->base[r] + 2 * g->staging_bytes);
    }
    char* counters = g->base[g->rank] + 2 * g->staging_bytes + kFlagsBytes;
    push.step_counter = reinterpret_cast<int32_t*>(counters);
    push.done_counter = reinterpret_cast<int32_t*>(counters + 64);
    push.rank = g->rank;
    push.world = g->world;
    push.row_elems = d.Hq * g->world * d.D;
    push.ll = in_place ? 0 : 1;
    push.col_offset = g->rank * d.Hq * d.D;
    push.wait_ns = g->wait_ns;
    push.group_counters = reinterpret_cast<int32_t*>(counters + kCountersBytes);
    const PagedTables t{past_lens, subsequence_begins, block_indices, block_indices_begins,
                        d.num_seqs, d.num_tokens, d.num_blocks_total, d.block_size};
    if (in_place) {
        for (int r = 0; r < g->world; ++r)
            push.started[r] = reinterpret_cast<int32_t*>(g->base[r] + 2 * g->staging_bytes) + kStartedFlagOffset;
    }
    g->mode = want;
    return paged_decode_launch(d, plan, query, k_cache, v_cache, t, out_full, workspace, status,
                               reinterpret_cast<cudaStream_t>(stream), &push);
}

int b2a_sdpa_forward_sharded(b2a_shard_group* g, const b2a_sdpa_desc* local_desc, const void* q, const void* k,
                             const void* v, void** out_full, int32_t* status, b2a_stream_t stream) {
    using namespace b2a;
    if (g == nullptr || local_desc == nullptr || out_full == nullptr) return B2A_ERR_NULL;
    if (!g->connected || (g->mode != kModeUnset && g->mode != kModePrefill)) return B2A_ERR_UNSUPPORTED;
    b2a_sdpa_desc d = *local_desc;
    if (d.dtype != B2A_F16 && d.dtype != B2A_BF16) return B2A_ERR_UNSUPPORTED;
    if (d.B <= 0 || d.Hq <= 0 || d.Hkv <= 0 || d.Sq <= 0 || d.Skv <= 0 || d.Hq % d.Hkv != 0) return B2A_ERR_DIM;
    if (d.B > 65535 || static_cast<long long>(d.Hq) * g->world > 65535) return B2A_ERR_DIM;
    if (d.mask_kind != B2A_MASK_NONE) return B2A_ERR_UNSUPPORTED;
    if (q == nullptr || k == nullptr || v == nullptr) return B2A_ERR_NULL;
    if (!(d.scale >= 0.f) || std::isinf(d.scale)) return B2A_ERR_DIM;
    if (d.scale == 0.f) d.scale = 1.0f / sqrtf(static_cast<float>(d.D));
    auto fill = [](int64_t (&s)[4], int64_t h, int64_t n, int64_t e) {
        if (s[0] == 0 && s[1] == 0 && s[2] == 0 && s[3] == 0) { s[3] = 1; s[2] = e; s[1] = n * e; s[0] = h * n * e; }
    };
    int64_t qs[4], ks[4], vs[4], os[4] = {0, 0, 0, 0};
    std::memcpy(qs, d.q_strides, sizeof qs);
    std::memcpy(ks, d.k_strides, sizeof ks);
    std::memcpy(vs, d.v_strides, sizeof vs);
    fill(qs, d.Hq, d.Sq, d.D);
    fill(ks, d.Hkv, d.Skv, d.D);
    fill(vs, d.Hkv, d.Skv, d.Dv);
    const int hq_total = d.Hq * g->world;
    fill(os, hq_total, d.Sq, d.Dv);
    const size_t out_bytes = static_cast<size_t>(d.B) * hq_total * d.Sq * d.Dv * 2;
    if (out_bytes > g->staging_bytes) return B2A_ERR_CAPACITY;
    const int32_t step = g->prefill_step + 1;
    const size_t half = static_cast<size_t>(step & 1) * g->staging_bytes;
    void* mine = g->base[g->rank] + half;
    if (!sdpa_tc_supported(d, qs, ks, vs, os, q, k, v, mine)) return B2A_ERR_UNSUPPORTED;
    TcPeerOut po{};
    for (int r = 0; r < g->world; ++r) {
        po.out_base[r] = g->base[r] + half;
        po.flags[r] = reinterpret_cast<int32_t*>(g->base[r] + 2 * g->staging_bytes) + kPrefillFlagOffset;
    }
    po.done_counter = reinterpret_cast<int32_t*>(g->base[g->rank] + 2 * g->staging_bytes + kFlagsBytes + 128);
    po.rank = g->rank;
    po.world = g->world;
    po.hq_total = hq_total;
    po.head_offset = g->rank * d.Hq;
    po.step = step;
    po.wait_ns = g->wait_ns;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    int rc = sdpa_tc_launch(d, qs, ks, vs, os, q, k, v, mine, status, s, &po);
    if (rc != B2A_OK) return rc;
    g->mode = kModePrefill;
    g->prefill_step = step;
    rc = sdpa_peer_wait_launch(po.flags[g->rank], g->world, step, g->wait_ns, status, s);
    if (rc != B2A_OK) return rc;
    *out_full = mine;
    return B2A_OK;
}

}  // extern "C"
