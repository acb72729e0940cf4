// Head-sharded decode across the GPUs of one node without a collective library on the data path.
//
// A shard group is one device allocation per rank, [staging 0 | staging 1 | flags | counters], exported with CUDA
// IPC and mapped by every peer.  b2a_paged_attention_sharded runs the split-K decode on this rank's KV heads; its
// merge kernel stores the rank's output columns into every rank's staging buffer over NVLink and publishes the step
// in every rank's flags; peer_wait_copy_kernel then waits (bounded) for all ranks and copies the full-width rows to
// the caller's output (see PeerPush in launch.cuh, kernels in paged_decode.cu).
// The reference never spans devices (one independent plugin configuration per device id,
// modules/nvidia_plugin/src/cuda_plugin.cpp:25-32), so nothing here has a counterpart there.
#include <cstring>
#include <new>

#include "launch.cuh"

namespace {
constexpr size_t kFlagsBytes = 256;     // kMaxShardWorld ints, padded
constexpr size_t kCountersBytes = 256;  // step counter at +0, done counter at +64
size_t round_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
}  // namespace

struct b2a_shard_group {
    int rank = 0, world = 1, device = 0;
    size_t staging_bytes = 0;  // one staging buffer
    char* base[b2a::kMaxShardWorld] = {};  // [rank]: that rank's allocation as mapped in this process
    bool connected = false;
    size_t total_bytes() const { return 2 * staging_bytes + kFlagsBytes + kCountersBytes; }
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
    }
    g->connected = true;
    return B2A_OK;
}

void b2a_shard_group_destroy(b2a_shard_group* g) {
    if (g == nullptr) return;
    for (int r = 0; r < g->world; ++r) {
        if (g->base[r] == nullptr) continue;
        if (r == g->rank) cudaFree(g->base[r]); else cudaIpcCloseMemHandle(g->base[r]);
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
    b2a_paged_desc d = *local_desc;
    if (d.scale == 0.f && d.D > 0) d.scale = 1.0f / sqrtf(static_cast<float>(d.D));
    if (d.num_tokens == 0 || d.num_seqs == 0) return B2A_OK;
    if (query == nullptr || k_cache == nullptr || v_cache == nullptr || out_full == nullptr || past_lens == nullptr ||
        subsequence_begins == nullptr || block_indices == nullptr || block_indices_begins == nullptr)
        return B2A_ERR_NULL;
    if (d.Hq <= 0 || d.Hkv <= 0 || d.Hq % d.Hkv != 0 || d.num_seqs > 65535 || d.max_context_len <= 0) return B2A_ERR_DIM;
    if (!paged_decode_supported(d)) return B2A_ERR_UNSUPPORTED;  // decode steps only
    const size_t row_bytes = static_cast<size_t>(d.Hq) * g->world * d.D * 2;
    if (static_cast<size_t>(d.num_tokens) * row_bytes > g->staging_bytes) return B2A_ERR_CAPACITY;
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
    push.col_offset = g->rank * d.Hq * d.D;
    const PagedTables t{past_lens, subsequence_begins, block_indices, block_indices_begins,
                        d.num_seqs, d.num_tokens, d.num_blocks_total, d.block_size};
    return paged_decode_launch(d, plan, query, k_cache, v_cache, t, out_full, workspace, status,
                               reinterpret_cast<cudaStream_t>(stream), &push);
}

}  // extern "C"
