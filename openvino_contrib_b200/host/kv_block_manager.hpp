// Host-side owner of a paged KV pool's bookkeeping: free list, per-sequence block lists, step tables.
//
// It has the role CudaVariableState has for the reference's contiguous cache
// (modules/nvidia_plugin/src/cuda_variable_state.hpp:31-183: reset, grow, hand the buffer to ReadValue/Assign),
// for a pool of fixed-size blocks shared by many sequences.  Pure host code: the pool bytes themselves live in
// device memory owned by whoever created the pool.
#pragma once

#include <cstdint>
#include <unordered_map>
#include <vector>

namespace b2a {

struct StepTables {
    std::vector<int32_t> past_lens;             // [n]
    std::vector<int32_t> subsequence_begins;    // [n+1]
    std::vector<int32_t> block_indices;         // [sum of blocks of the scheduled sequences]
    std::vector<int32_t> block_indices_begins;  // [n+1]
    int32_t max_context_len = 0;
    int32_t max_q_len = 0;
    int32_t prefill_row_blocks = 0;  // sum of ceil(q_len / 128) over the sequences with two or more new tokens
    int32_t prefill_kv_tokens = 0;   // sum of their context lengths, each rounded up to 128
    int32_t num_tokens = 0;
};

class KvBlockManager {
public:
    // shuffle_seed != 0 permutes the initial free list (xorshift, reproducible) so that tables are not monotone.
    KvBlockManager(int32_t num_blocks, int32_t block_size, uint64_t shuffle_seed = 0);

    int32_t num_blocks() const { return num_blocks_; }
    int32_t block_size() const { return block_size_; }
    int32_t free_blocks() const { return static_cast<int32_t>(free_.size()); }

    bool add_sequence(int64_t id);   // false if it exists
    bool free_sequence(int64_t id);  // false if unknown; its blocks return to the free list
    int32_t sequence_len(int64_t id) const;  // -1 if unknown
    int32_t last_prefill_row_blocks() const { return last_prefill_row_blocks_; }  // of the last scheduled step
    int32_t last_prefill_kv_tokens() const { return last_prefill_kv_tokens_; }
    const std::vector<int32_t>* sequence_blocks(int64_t id) const;

    // Blocks that scheduling q_lens[i] new tokens for ids[i] would take from the free list; -1 if an id is unknown
    // or a length negative.
    int64_t blocks_needed(const int64_t* ids, const int32_t* q_lens, int32_t n) const;

    // All-or-nothing: reserves the blocks, advances the lengths and fills `out`.  Returns 0, or
    // B2A_ERR_NOT_FOUND / B2A_ERR_CAPACITY / B2A_ERR_DIM with no state changed.
    int schedule_step(const int64_t* ids, const int32_t* q_lens, int32_t n, StepTables& out);

private:
    struct Seq {
        std::vector<int32_t> blocks;
        int32_t len = 0;
    };
    int32_t num_blocks_, block_size_;
    int32_t last_prefill_row_blocks_ = 0;
    int32_t last_prefill_kv_tokens_ = 0;
    std::vector<int32_t> free_;  // stack: back() is handed out next
    std::unordered_map<int64_t, Seq> seqs_;
};

}  // namespace b2a
