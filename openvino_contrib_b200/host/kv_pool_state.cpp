#include "kv_pool_state.hpp"

#include <algorithm>
#include <cstring>
#include <new>
#include <stdexcept>
#include <string>

namespace b2a {

// launchers of csrc/paged_kv_state.cu
int kv_rows_from_bhsd_launch(int dtype, const void* src, void* dst, int B, int H, int q, int D, int src_T, int t0,
                             cudaStream_t stream);
int kv_export_launch(int kv_dtype, int out_dtype, const void* cache, const int32_t* block_indices,
                     const int32_t* block_indices_begins, int num_blocks_total, int B, int H, int T, int D, int bs,
                     void* out, int32_t* status, cudaStream_t stream);

namespace {

constexpr int32_t kBlobMagic = 0x4B563161;  // "a1VK"
constexpr size_t kBlobHeaderInts = 8;        // magic, kv_dtype, batch, hkv, d, block_size, length, reserved

size_t size_of(int dtype) {
    switch (dtype) {
        case B2A_F32: return 4;
        case B2A_F16:
        case B2A_BF16: return 2;
        default: return 0;
    }
}

void must(cudaError_t e, const char* what) {
    if (e != cudaSuccess) throw std::runtime_error(std::string("KvPoolState: ") + what + ": " + cudaGetErrorString(e));
}

struct DeviceTemp {  // slow paths only
    void* p = nullptr;
    explicit DeviceTemp(size_t bytes) {
        if (cudaMalloc(&p, std::max<size_t>(bytes, 16)) != cudaSuccess) p = nullptr;
    }
    ~DeviceTemp() {
        if (p) cudaFree(p);
    }
};

}  // namespace

KvPoolState::KvPoolState(int kv_dtype, int x_dtype, int batch, int hkv, int d, int block_size, int num_blocks,
                         int max_step_tokens)
    : kv_dtype_(kv_dtype), x_dtype_(x_dtype), batch_(batch), hkv_(hkv), d_(d), bs_(block_size), num_blocks_(num_blocks),
      max_step_tokens_(max_step_tokens), manager_(num_blocks > 0 ? num_blocks : 1, block_size > 0 ? block_size : 1, 0) {
    x_size_ = size_of(x_dtype);
    chunk_bytes_ = b2a_paged_chunk_bytes(kv_dtype, block_size, d);
    if (x_size_ == 0 || chunk_bytes_ == 0 || batch <= 0 || batch > 65535 || hkv <= 0 || num_blocks <= 0 || max_step_tokens <= 0)
        throw std::invalid_argument("KvPoolState: bad dimensions or element types");
    for (int b = 0; b < batch; ++b) manager_.add_sequence(b);
    const size_t pool = static_cast<size_t>(num_blocks) * hkv * chunk_bytes_;
    const size_t rows = static_cast<size_t>(batch) * max_step_tokens * hkv * d * x_size_;
    tables_ints_ = static_cast<size_t>(batch) + 2 * (static_cast<size_t>(batch) + 1) + static_cast<size_t>(num_blocks);
    must(cudaMalloc(&k_pool_, pool), "cudaMalloc");
    must(cudaMalloc(&v_pool_, pool), "cudaMalloc");
    must(cudaMalloc(&rows_k_, rows), "cudaMalloc");
    must(cudaMalloc(&rows_v_, rows), "cudaMalloc");
    must(cudaMalloc(reinterpret_cast<void**>(&tables_dev_), tables_ints_ * sizeof(int32_t)), "cudaMalloc");
    must(cudaMemset(k_pool_, 0, pool), "cudaMemset");
    must(cudaMemset(v_pool_, 0, pool), "cudaMemset");
    must(cudaMemset(tables_dev_, 0, tables_ints_ * sizeof(int32_t)), "cudaMemset");
    last_.past_lens.assign(static_cast<size_t>(batch), 0);
    last_.subsequence_begins.assign(static_cast<size_t>(batch) + 1, 0);
    last_.block_indices_begins.assign(static_cast<size_t>(batch) + 1, 0);
}

KvPoolState::~KvPoolState() {
    for (void* p : {k_pool_, v_pool_, rows_k_, rows_v_, static_cast<void*>(tables_dev_)})
        if (p) cudaFree(p);
}

int KvPoolState::length() const {
    std::lock_guard<std::mutex> lock(mutex_);
    return manager_.sequence_len(0);
}

b2a_paged_desc KvPoolState::desc(int num_tokens) const {
    b2a_paged_desc d{};
    d.q_dtype = x_dtype_;
    d.kv_dtype = kv_dtype_;
    d.Hq = d.Hkv = hkv_;
    d.D = d.Dv = d_;
    d.block_size = bs_;
    d.num_seqs = batch_;
    d.num_tokens = num_tokens;
    d.num_blocks_total = num_blocks_;
    return d;
}

int KvPoolState::Reset() {
    std::lock_guard<std::mutex> lock(mutex_);
    for (int b = 0; b < batch_; ++b) {
        manager_.free_sequence(b);
        manager_.add_sequence(b);
    }
    last_ = StepTables{};
    last_.past_lens.assign(static_cast<size_t>(batch_), 0);
    last_.subsequence_begins.assign(static_cast<size_t>(batch_) + 1, 0);
    last_.block_indices_begins.assign(static_cast<size_t>(batch_) + 1, 0);
    return B2A_OK;
}

int KvPoolState::upload_tables(const StepTables& t, cudaStream_t stream) {
    // one host -> device copy from ordinary memory: the runtime stages such a copy before it returns, so the vector
    // may change right after
    std::vector<int32_t> all(tables_ints_, 0);
    const size_t B = static_cast<size_t>(batch_);
    if (t.block_indices.size() > static_cast<size_t>(num_blocks_)) return B2A_ERR_CAPACITY;
    std::copy(t.past_lens.begin(), t.past_lens.end(), all.begin());
    std::copy(t.subsequence_begins.begin(), t.subsequence_begins.end(), all.begin() + B);
    std::copy(t.block_indices_begins.begin(), t.block_indices_begins.end(), all.begin() + 2 * B + 1);
    std::copy(t.block_indices.begin(), t.block_indices.end(), all.begin() + 3 * B + 2);
    return cudaMemcpyAsync(tables_dev_, all.data(), tables_ints_ * sizeof(int32_t), cudaMemcpyHostToDevice, stream) ==
                   cudaSuccess
               ? B2A_OK
               : B2A_ERR_CUDA;
}

KvPoolState::Step KvPoolState::LastStep() const {
    std::lock_guard<std::mutex> lock(mutex_);
    const size_t B = static_cast<size_t>(batch_);
    Step s{};
    s.k_cache = k_pool_;
    s.v_cache = v_pool_;
    s.past_lens = tables_dev_;
    s.subsequence_begins = tables_dev_ + B;
    s.block_indices_begins = tables_dev_ + 2 * B + 1;
    s.block_indices = tables_dev_ + 3 * B + 2;
    s.num_seqs = batch_;
    s.num_tokens = last_.num_tokens;
    s.num_blocks_total = num_blocks_;
    s.max_context_len = last_.max_context_len;
    s.max_q_len = last_.max_q_len;
    s.prefill_row_blocks = last_.prefill_row_blocks;
    s.prefill_kv_tokens = last_.prefill_kv_tokens;
    return s;
}

int KvPoolState::append_locked(const void* k_new, const void* v_new, int q_len, int32_t* status, cudaStream_t stream) {
    if (k_new == nullptr || v_new == nullptr) return B2A_ERR_NULL;
    if (q_len <= 0 || q_len > max_step_tokens_) return B2A_ERR_DIM;
    std::vector<int64_t> ids(static_cast<size_t>(batch_));
    std::vector<int32_t> ql(static_cast<size_t>(batch_), q_len);
    for (int b = 0; b < batch_; ++b) ids[static_cast<size_t>(b)] = b;
    StepTables t;
    int rc = manager_.schedule_step(ids.data(), ql.data(), batch_, t);
    if (rc != B2A_OK) return rc;
    rc = upload_tables(t, stream);
    if (rc != B2A_OK) return rc;
    const void *rk = k_new, *rv = v_new;
    if (q_len > 1) {  // [B, Hkv, q, D] -> token-major rows; one new row per sequence is token-major as it is
        rc = kv_rows_from_bhsd_launch(x_dtype_, k_new, rows_k_, batch_, hkv_, q_len, d_, q_len, 0, stream);
        if (rc == B2A_OK) rc = kv_rows_from_bhsd_launch(x_dtype_, v_new, rows_v_, batch_, hkv_, q_len, d_, q_len, 0, stream);
        if (rc != B2A_OK) return rc;
        rk = rows_k_;
        rv = rows_v_;
    }
    const b2a_paged_desc d = desc(batch_ * q_len);
    const size_t B = static_cast<size_t>(batch_);
    rc = b2a_paged_kv_store(&d, rk, rv, k_pool_, v_pool_, tables_dev_, tables_dev_ + B, tables_dev_ + 3 * B + 2,
                            tables_dev_ + 2 * B + 1, status, reinterpret_cast<b2a_stream_t>(stream));
    if (rc == B2A_OK) last_ = std::move(t);
    return rc;
}

int KvPoolState::Append(const void* k_new, const void* v_new, int q_len, int32_t* status, cudaStream_t stream) {
    std::lock_guard<std::mutex> lock(mutex_);
    return append_locked(k_new, v_new, q_len, status, stream);
}

int KvPoolState::SetState(const void* k_host, const void* v_host, int T, cudaStream_t stream) {
    if (k_host == nullptr || v_host == nullptr) return B2A_ERR_NULL;
    if (T < 0) return B2A_ERR_DIM;
    int rc = Reset();
    if (rc != B2A_OK || T == 0) return rc;
    std::lock_guard<std::mutex> lock(mutex_);
    if ((static_cast<int64_t>(T) + bs_ - 1) / bs_ * batch_ > manager_.free_blocks()) return B2A_ERR_CAPACITY;
    const size_t bytes = static_cast<size_t>(batch_) * hkv_ * T * d_ * x_size_;
    DeviceTemp dk(bytes), dv(bytes);
    if (dk.p == nullptr || dv.p == nullptr) return B2A_ERR_CUDA;
    if (cudaMemcpyAsync(dk.p, k_host, bytes, cudaMemcpyHostToDevice, stream) != cudaSuccess ||
        cudaMemcpyAsync(dv.p, v_host, bytes, cudaMemcpyHostToDevice, stream) != cudaSuccess)
        return B2A_ERR_CUDA;
    // in slices of at most max_step_tokens positions: each slice is a step of the cache's own append path
    for (int t0 = 0; t0 < T && rc == B2A_OK; t0 += max_step_tokens_) {
        const int q = std::min(max_step_tokens_, T - t0);
        rc = kv_rows_from_bhsd_launch(x_dtype_, dk.p, rows_k_, batch_, hkv_, q, d_, T, t0, stream);
        if (rc == B2A_OK) rc = kv_rows_from_bhsd_launch(x_dtype_, dv.p, rows_v_, batch_, hkv_, q, d_, T, t0, stream);
        if (rc != B2A_OK) break;
        std::vector<int64_t> ids(static_cast<size_t>(batch_));
        std::vector<int32_t> ql(static_cast<size_t>(batch_), q);
        for (int b = 0; b < batch_; ++b) ids[static_cast<size_t>(b)] = b;
        StepTables t;
        rc = manager_.schedule_step(ids.data(), ql.data(), batch_, t);
        if (rc == B2A_OK) rc = upload_tables(t, stream);
        if (rc != B2A_OK) break;
        const b2a_paged_desc d = desc(batch_ * q);
        const size_t B = static_cast<size_t>(batch_);
        rc = b2a_paged_kv_store(&d, rows_k_, rows_v_, k_pool_, v_pool_, tables_dev_, tables_dev_ + B,
                                tables_dev_ + 3 * B + 2, tables_dev_ + 2 * B + 1, nullptr,
                                reinterpret_cast<b2a_stream_t>(stream));
        if (rc == B2A_OK) last_ = std::move(t);
    }
    if (cudaStreamSynchronize(stream) != cudaSuccess) return B2A_ERR_CUDA;  // the temporaries go away here
    return rc;
}

int KvPoolState::ReadDense(void* k_dev, void* v_dev, int T, int32_t* status, cudaStream_t stream) const {
    std::lock_guard<std::mutex> lock(mutex_);
    if (k_dev == nullptr || v_dev == nullptr) return B2A_ERR_NULL;
    if (T != manager_.sequence_len(0)) return B2A_ERR_DIM;
    const size_t B = static_cast<size_t>(batch_);
    int rc = kv_export_launch(kv_dtype_, x_dtype_, k_pool_, tables_dev_ + 3 * B + 2, tables_dev_ + 2 * B + 1, num_blocks_,
                              batch_, hkv_, T, d_, bs_, k_dev, status, stream);
    if (rc == B2A_OK)
        rc = kv_export_launch(kv_dtype_, x_dtype_, v_pool_, tables_dev_ + 3 * B + 2, tables_dev_ + 2 * B + 1, num_blocks_,
                              batch_, hkv_, T, d_, bs_, v_dev, status, stream);
    return rc;
}

int KvPoolState::GetState(void* k_host, void* v_host, int T, cudaStream_t stream) const {
    if (k_host == nullptr || v_host == nullptr) return B2A_ERR_NULL;
    if (T == 0) return length() == 0 ? B2A_OK : B2A_ERR_DIM;
    const size_t bytes = static_cast<size_t>(batch_) * hkv_ * T * d_ * x_size_;
    DeviceTemp dk(bytes), dv(bytes);
    if (dk.p == nullptr || dv.p == nullptr) return B2A_ERR_CUDA;
    const int rc = ReadDense(dk.p, dv.p, T, nullptr, stream);
    if (rc != B2A_OK) return rc;
    if (cudaMemcpyAsync(k_host, dk.p, bytes, cudaMemcpyDeviceToHost, stream) != cudaSuccess ||
        cudaMemcpyAsync(v_host, dv.p, bytes, cudaMemcpyDeviceToHost, stream) != cudaSuccess ||
        cudaStreamSynchronize(stream) != cudaSuccess)
        return B2A_ERR_CUDA;
    return B2A_OK;
}

// blob: [8 int32 header][per sequence, per logical block: the K chunks of all KV heads, then the V chunks]
size_t KvPoolState::ExportBytes() const {
    std::lock_guard<std::mutex> lock(mutex_);
    const size_t blocks = (static_cast<size_t>(manager_.sequence_len(0)) + bs_ - 1) / bs_;
    return kBlobHeaderInts * sizeof(int32_t) + static_cast<size_t>(batch_) * blocks * 2 * hkv_ * chunk_bytes_;
}

int KvPoolState::Export(void* host_blob, size_t bytes, cudaStream_t stream) const {
    if (host_blob == nullptr) return B2A_ERR_NULL;
    if (bytes < ExportBytes()) return B2A_ERR_CAPACITY;
    std::lock_guard<std::mutex> lock(mutex_);
    const int T = manager_.sequence_len(0);
    const int32_t header[kBlobHeaderInts] = {kBlobMagic, kv_dtype_, batch_, hkv_, d_, bs_, T, 0};
    std::memcpy(host_blob, header, sizeof header);
    char* at = static_cast<char*>(host_blob) + sizeof header;
    const size_t per_block = static_cast<size_t>(hkv_) * chunk_bytes_;
    for (int b = 0; b < batch_; ++b) {
        const std::vector<int32_t>* blocks = manager_.sequence_blocks(b);
        const size_t used = (static_cast<size_t>(T) + bs_ - 1) / bs_;
        for (size_t i = 0; i < used; ++i) {
            const size_t phys = static_cast<size_t>((*blocks)[i]);
            if (cudaMemcpyAsync(at, static_cast<const char*>(k_pool_) + phys * per_block, per_block, cudaMemcpyDeviceToHost, stream) != cudaSuccess ||
                cudaMemcpyAsync(at + per_block, static_cast<const char*>(v_pool_) + phys * per_block, per_block, cudaMemcpyDeviceToHost, stream) != cudaSuccess)
                return B2A_ERR_CUDA;
            at += 2 * per_block;
        }
    }
    return cudaStreamSynchronize(stream) == cudaSuccess ? B2A_OK : B2A_ERR_CUDA;
}

int KvPoolState::Import(const void* host_blob, size_t bytes, cudaStream_t stream) {
    if (host_blob == nullptr) return B2A_ERR_NULL;
    if (bytes < kBlobHeaderInts * sizeof(int32_t)) return B2A_ERR_DIM;
    int32_t header[kBlobHeaderInts];
    std::memcpy(header, host_blob, sizeof header);
    if (header[0] != kBlobMagic || header[1] != kv_dtype_ || header[2] != batch_ || header[3] != hkv_ || header[4] != d_ ||
        header[5] != bs_ || header[6] < 0)
        return B2A_ERR_DIM;  // an image of another geometry
    const int T = header[6];
    const size_t per_block = static_cast<size_t>(hkv_) * chunk_bytes_;
    const size_t used = (static_cast<size_t>(T) + bs_ - 1) / bs_;
    if (bytes < sizeof header + static_cast<size_t>(batch_) * used * 2 * per_block) return B2A_ERR_DIM;
    int rc = Reset();
    if (rc != B2A_OK || T == 0) return rc;
    std::lock_guard<std::mutex> lock(mutex_);
    std::vector<int64_t> ids(static_cast<size_t>(batch_));
    std::vector<int32_t> ql(static_cast<size_t>(batch_), T);
    for (int b = 0; b < batch_; ++b) ids[static_cast<size_t>(b)] = b;
    StepTables t;
    rc = manager_.schedule_step(ids.data(), ql.data(), batch_, t);  // reserves the blocks (all or nothing)
    if (rc != B2A_OK) return rc;
    const char* at = static_cast<const char*>(host_blob) + sizeof header;
    for (int b = 0; b < batch_; ++b) {
        const std::vector<int32_t>* blocks = manager_.sequence_blocks(b);
        for (size_t i = 0; i < used; ++i) {
            const size_t phys = static_cast<size_t>((*blocks)[i]);
            if (cudaMemcpyAsync(static_cast<char*>(k_pool_) + phys * per_block, at, per_block, cudaMemcpyHostToDevice, stream) != cudaSuccess ||
                cudaMemcpyAsync(static_cast<char*>(v_pool_) + phys * per_block, at + per_block, per_block, cudaMemcpyHostToDevice, stream) != cudaSuccess)
                return B2A_ERR_CUDA;
            at += 2 * per_block;
        }
    }
    // the tables now describe "every position present": the next Append continues from T
    rc = upload_tables(t, stream);
    if (rc == B2A_OK) last_ = std::move(t);
    if (cudaStreamSynchronize(stream) != cudaSuccess) return B2A_ERR_CUDA;
    return rc;
}

}  // namespace b2a

// ---- C ABI (declared in b2a.h) ----------------------------------------------------------------------------------
struct b2a_kvstate {
    b2a::KvPoolState* state;
};

extern "C" {

int b2a_kvstate_create(int32_t kv_dtype, int32_t x_dtype, int32_t batch, int32_t hkv, int32_t d, int32_t block_size,
                       int32_t num_blocks, int32_t max_step_tokens, b2a_kvstate** out) {
    if (out == nullptr) return B2A_ERR_NULL;
    try {
        auto* s = new b2a::KvPoolState(kv_dtype, x_dtype, batch, hkv, d, block_size, num_blocks, max_step_tokens);
        *out = new b2a_kvstate{s};
        return B2A_OK;
    } catch (const std::invalid_argument&) {
        return B2A_ERR_DIM;
    } catch (const std::bad_alloc&) {
        return B2A_ERR_CAPACITY;
    } catch (const std::exception&) {
        return B2A_ERR_CUDA;
    }
}

void b2a_kvstate_destroy(b2a_kvstate* s) {
    if (s == nullptr) return;
    delete s->state;
    delete s;
}

int32_t b2a_kvstate_length(const b2a_kvstate* s) { return s == nullptr ? -1 : s->state->length(); }
int b2a_kvstate_reset(b2a_kvstate* s) { return s == nullptr ? B2A_ERR_NULL : s->state->Reset(); }
int b2a_kvstate_set_state(b2a_kvstate* s, const void* k_host, const void* v_host, int32_t T, b2a_stream_t stream) {
    return s == nullptr ? B2A_ERR_NULL : s->state->SetState(k_host, v_host, T, reinterpret_cast<cudaStream_t>(stream));
}
int b2a_kvstate_get_state(const b2a_kvstate* s, void* k_host, void* v_host, int32_t T, b2a_stream_t stream) {
    return s == nullptr ? B2A_ERR_NULL : s->state->GetState(k_host, v_host, T, reinterpret_cast<cudaStream_t>(stream));
}
int b2a_kvstate_append(b2a_kvstate* s, const void* k_new, const void* v_new, int32_t q_len, int32_t* status,
                       b2a_stream_t stream) {
    return s == nullptr ? B2A_ERR_NULL : s->state->Append(k_new, v_new, q_len, status, reinterpret_cast<cudaStream_t>(stream));
}
int b2a_kvstate_read_dense(const b2a_kvstate* s, void* k_dev, void* v_dev, int32_t T, int32_t* status, b2a_stream_t stream) {
    return s == nullptr ? B2A_ERR_NULL : s->state->ReadDense(k_dev, v_dev, T, status, reinterpret_cast<cudaStream_t>(stream));
}
int b2a_kvstate_last_step(const b2a_kvstate* s, b2a_kvstate_step* out) {
    if (s == nullptr || out == nullptr) return B2A_ERR_NULL;
    const b2a::KvPoolState::Step st = s->state->LastStep();
    out->k_cache = st.k_cache;
    out->v_cache = st.v_cache;
    out->past_lens = st.past_lens;
    out->subsequence_begins = st.subsequence_begins;
    out->block_indices = st.block_indices;
    out->block_indices_begins = st.block_indices_begins;
    out->num_seqs = st.num_seqs;
    out->num_tokens = st.num_tokens;
    out->num_blocks_total = st.num_blocks_total;
    out->max_context_len = st.max_context_len;
    out->max_q_len = st.max_q_len;
    out->prefill_row_blocks = st.prefill_row_blocks;
    out->prefill_kv_tokens = st.prefill_kv_tokens;
    return B2A_OK;
}
size_t b2a_kvstate_export_bytes(const b2a_kvstate* s) { return s == nullptr ? 0 : s->state->ExportBytes(); }
int b2a_kvstate_export(const b2a_kvstate* s, void* host_blob, size_t bytes, b2a_stream_t stream) {
    return s == nullptr ? B2A_ERR_NULL : s->state->Export(host_blob, bytes, reinterpret_cast<cudaStream_t>(stream));
}
int b2a_kvstate_import(b2a_kvstate* s, const void* host_blob, size_t bytes, b2a_stream_t stream) {
    return s == nullptr ? B2A_ERR_NULL : s->state->Import(host_blob, bytes, reinterpret_cast<cudaStream_t>(stream));
}

}  // extern "C"
