#include "kv_block_manager.hpp"

#include <algorithm>
#include <cstring>
#include <new>

#include "b2a.h"

namespace b2a {

KvBlockManager::KvBlockManager(int32_t num_blocks, int32_t block_size, uint64_t shuffle_seed)
    : num_blocks_(num_blocks), block_size_(block_size) {
    free_.resize(static_cast<size_t>(num_blocks));
    // back() is handed out first: descending fill makes the unshuffled order 0, 1, 2, ...
    for (int32_t i = 0; i < num_blocks; ++i) free_[static_cast<size_t>(i)] = num_blocks - 1 - i;
    if (shuffle_seed != 0) {
        uint64_t s = shuffle_seed;
        auto next = [&s]() {
            s ^= s << 13;
            s ^= s >> 7;
            s ^= s << 17;
            return s;
        };
        for (size_t i = free_.size(); i > 1; --i) std::swap(free_[i - 1], free_[next() % i]);
    }
}

bool KvBlockManager::add_sequence(int64_t id) { return seqs_.emplace(id, Seq{}).second; }

bool KvBlockManager::free_sequence(int64_t id) {
    auto it = seqs_.find(id);
    if (it == seqs_.end()) return false;
    for (auto rit = it->second.blocks.rbegin(); rit != it->second.blocks.rend(); ++rit) free_.push_back(*rit);
    seqs_.erase(it);
    return true;
}

int32_t KvBlockManager::sequence_len(int64_t id) const {
    auto it = seqs_.find(id);
    return it == seqs_.end() ? -1 : it->second.len;
}

const std::vector<int32_t>* KvBlockManager::sequence_blocks(int64_t id) const {
    auto it = seqs_.find(id);
    return it == seqs_.end() ? nullptr : &it->second.blocks;
}

int64_t KvBlockManager::blocks_needed(const int64_t* ids, const int32_t* q_lens, int32_t n) const {
    int64_t need = 0;
    for (int32_t i = 0; i < n; ++i) {
        auto it = seqs_.find(ids[i]);
        if (it == seqs_.end() || q_lens[i] < 0) return -1;
        const int64_t new_len = static_cast<int64_t>(it->second.len) + q_lens[i];
        const int64_t blocks = (new_len + block_size_ - 1) / block_size_;
        need += std::max<int64_t>(0, blocks - static_cast<int64_t>(it->second.blocks.size()));
    }
    return need;
}

int KvBlockManager::schedule_step(const int64_t* ids, const int32_t* q_lens, int32_t n, StepTables& out) {
    if (n < 0 || (n > 0 && (ids == nullptr || q_lens == nullptr))) return B2A_ERR_DIM;
    for (int32_t i = 0; i < n; ++i) {
        if (seqs_.find(ids[i]) == seqs_.end()) return B2A_ERR_NOT_FOUND;
        if (q_lens[i] < 0) return B2A_ERR_DIM;
        for (int32_t j = 0; j < i; ++j)
            if (ids[j] == ids[i]) return B2A_ERR_DIM;  // a sequence appears once per step
    }
    const int64_t need = blocks_needed(ids, q_lens, n);
    if (need < 0) return B2A_ERR_DIM;
    if (need > static_cast<int64_t>(free_.size())) return B2A_ERR_CAPACITY;

    out = StepTables{};
    out.past_lens.resize(static_cast<size_t>(n));
    out.subsequence_begins.assign(static_cast<size_t>(n) + 1, 0);
    out.block_indices_begins.assign(static_cast<size_t>(n) + 1, 0);
    for (int32_t i = 0; i < n; ++i) {
        Seq& s = seqs_[ids[i]];
        out.past_lens[static_cast<size_t>(i)] = s.len;
        const int32_t new_len = s.len + q_lens[i];
        const size_t blocks = static_cast<size_t>((new_len + block_size_ - 1) / block_size_);
        while (s.blocks.size() < blocks) {
            s.blocks.push_back(free_.back());
            free_.pop_back();
        }
        s.len = new_len;
        out.block_indices.insert(out.block_indices.end(), s.blocks.begin(), s.blocks.begin() + static_cast<long>(blocks));
        out.subsequence_begins[static_cast<size_t>(i) + 1] = out.subsequence_begins[static_cast<size_t>(i)] + q_lens[i];
        out.block_indices_begins[static_cast<size_t>(i) + 1] = static_cast<int32_t>(out.block_indices.size());
        out.max_context_len = std::max(out.max_context_len, new_len);
        out.max_q_len = std::max(out.max_q_len, q_lens[i]);
        if (q_lens[i] >= 2) {
            out.prefill_row_blocks += (q_lens[i] + 127) / 128;
            out.prefill_kv_tokens += (new_len + 127) / 128 * 128;
        }
    }
    out.num_tokens = out.subsequence_begins[static_cast<size_t>(n)];
    last_prefill_row_blocks_ = out.prefill_row_blocks;
    last_prefill_kv_tokens_ = out.prefill_kv_tokens;
    return B2A_OK;
}

}  // namespace b2a

// ---- C ABI -------------------------------------------------------------------------------------------------
struct b2a_kvmgr {
    b2a::KvBlockManager impl;
    b2a_kvmgr(int32_t nb, int32_t bs, uint64_t seed) : impl(nb, bs, seed) {}
};

extern "C" {

int b2a_kvmgr_create(int32_t num_blocks, int32_t block_size, uint64_t shuffle_seed, b2a_kvmgr** out) {
    if (out == nullptr) return B2A_ERR_NULL;
    if (num_blocks < 0 || block_size <= 0) return B2A_ERR_DIM;
    *out = new (std::nothrow) b2a_kvmgr(num_blocks, block_size, shuffle_seed);
    return *out ? B2A_OK : B2A_ERR_CAPACITY;
}

void b2a_kvmgr_destroy(b2a_kvmgr* m) { delete m; }

int b2a_kvmgr_add_sequence(b2a_kvmgr* m, int64_t seq_id) {
    if (m == nullptr) return B2A_ERR_NULL;
    return m->impl.add_sequence(seq_id) ? B2A_OK : B2A_ERR_DIM;
}

int b2a_kvmgr_free_sequence(b2a_kvmgr* m, int64_t seq_id) {
    if (m == nullptr) return B2A_ERR_NULL;
    return m->impl.free_sequence(seq_id) ? B2A_OK : B2A_ERR_NOT_FOUND;
}

int32_t b2a_kvmgr_free_blocks(const b2a_kvmgr* m) { return m ? m->impl.free_blocks() : -1; }

int32_t b2a_kvmgr_sequence_len(const b2a_kvmgr* m, int64_t seq_id) { return m ? m->impl.sequence_len(seq_id) : -1; }

int32_t b2a_kvmgr_last_prefill_row_blocks(const b2a_kvmgr* m) { return m ? m->impl.last_prefill_row_blocks() : 0; }
int32_t b2a_kvmgr_last_prefill_kv_tokens(const b2a_kvmgr* m) { return m ? m->impl.last_prefill_kv_tokens() : 0; }

int b2a_kvmgr_schedule_step(b2a_kvmgr* m, const int64_t* seq_ids, const int32_t* q_lens, int32_t n,
                            int32_t* past_lens, int32_t* subsequence_begins, int32_t* block_indices,
                            int32_t block_indices_capacity, int32_t* block_indices_begins,
                            int32_t* num_block_indices, int32_t* max_context_len) {
    if (m == nullptr || past_lens == nullptr || subsequence_begins == nullptr || block_indices == nullptr ||
        block_indices_begins == nullptr)
        return B2A_ERR_NULL;
    // capacity is checked before any state changes: count the entries the step will emit
    int64_t entries = 0;
    for (int32_t i = 0; i < n; ++i) {
        const int32_t len = m->impl.sequence_len(seq_ids[i]);
        if (len < 0) return B2A_ERR_NOT_FOUND;
        if (q_lens[i] < 0) return B2A_ERR_DIM;
        entries += (static_cast<int64_t>(len) + q_lens[i] + m->impl.block_size() - 1) / m->impl.block_size();
    }
    if (entries > block_indices_capacity) return B2A_ERR_CAPACITY;
    b2a::StepTables t;
    const int rc = m->impl.schedule_step(seq_ids, q_lens, n, t);
    if (rc != B2A_OK) return rc;
    std::memcpy(past_lens, t.past_lens.data(), t.past_lens.size() * sizeof(int32_t));
    std::memcpy(subsequence_begins, t.subsequence_begins.data(), t.subsequence_begins.size() * sizeof(int32_t));
    std::memcpy(block_indices, t.block_indices.data(), t.block_indices.size() * sizeof(int32_t));
    std::memcpy(block_indices_begins, t.block_indices_begins.data(), t.block_indices_begins.size() * sizeof(int32_t));
    if (num_block_indices) *num_block_indices = static_cast<int32_t>(t.block_indices.size());
    if (max_context_len) *max_context_len = t.max_context_len;
    return B2A_OK;
}

}  // extern "C"
