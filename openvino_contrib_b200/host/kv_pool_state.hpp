// KvPoolState: the KV cache of one attention layer of a STATEFUL model, kept in a paged pool.
//
// A stateful OpenVINO model carries its cache in two variables per layer, each a dense [B, Hkv, T, D] tensor:
// ReadValue hands the past to a Concat with the step's new rows and Assign stores the grown tensor back
// (modules/nvidia_plugin/src/ops/read_value.cpp:31-72, src/ops/assign.cpp:29-56, src/kernels/concat.cu:16-32), which
// copies the whole cache every step.  The reference keeps such a variable in CudaVariableState
// (modules/nvidia_plugin/src/cuda_variable_state.hpp:31-183).  This class has that class's shape - reset, set_state /
// get_state with host tensors for the user-facing API, and device-side fast paths for the operations - but the bytes
// live in the block pool the paged kernels read, so that
//   Assign(Concat(ReadValue, new))  becomes  Append(new)            (quantise the new rows into their blocks: no copy
//                                                                     of the past),
//   ReadValue -> attention          becomes  the step tables below  (the attention kernels walk the block table).
// One object holds the K and the V variable of a layer for a batch of B sequences, which, as in the dense variable,
// all have the same length T.  It owns the device pools, a KvBlockManager and the device copies of the step tables.
//
// Thread-safety as in the reference's class: every member function takes the object's mutex; host <-> device copies
// of the slow paths run on the caller's stream and are synchronised before they return.
#pragma once

#include <cuda_runtime_api.h>

#include <cstddef>
#include <cstdint>
#include <mutex>
#include <vector>

#include "b2a.h"
#include "kv_block_manager.hpp"

namespace b2a {

class KvPoolState {
public:
    // kv_dtype: element type of the pool (B2A_U8 with per-token f16 scale / zero-point, or B2A_F16 / B2A_BF16);
    // x_dtype: element type of the model's variable (what set_state / get_state / Append exchange: f32, f16, bf16).
    // max_step_tokens bounds q_len of one Append.  Throws std::runtime_error on a CUDA failure, std::invalid_argument
    // on bad dimensions.
    KvPoolState(int kv_dtype, int x_dtype, int batch, int hkv, int d, int block_size, int num_blocks, int max_step_tokens);
    ~KvPoolState();
    KvPoolState(const KvPoolState&) = delete;
    KvPoolState& operator=(const KvPoolState&) = delete;

    int batch() const { return batch_; }
    int length() const;  // T: positions held per sequence
    size_t element_size() const { return x_size_; }

    // ---- user-facing API, host tensors [B, Hkv, T, D] of x_dtype (CudaVariableState::reset / set_state / get_state)
    int Reset();                                                        // back to the empty cache; blocks return to the free list
    int SetState(const void* k_host, const void* v_host, int T, cudaStream_t stream);
    int GetState(void* k_host, void* v_host, int T, cudaStream_t stream) const;  // T must equal length()

    // ---- fast paths for the operations, device memory only, nothing synchronises
    // Concat + Assign: k_new / v_new are device tensors [B, Hkv, q_len, D] of x_dtype (what the model's Concat would
    // have appended).  Reserves blocks, uploads the step tables and stores the rows.  B2A_ERR_CAPACITY if the pool is
    // exhausted (nothing changes then).
    int Append(const void* k_new, const void* v_new, int q_len, int32_t* status, cudaStream_t stream);
    // ReadValue for the attention operation: the pools and the tables of the LAST Append, in PagedAttentionExtension's
    // operand order.  Valid until the next Append / SetState / Reset.
    struct Step {
        const void *k_cache, *v_cache;
        const int32_t *past_lens, *subsequence_begins, *block_indices, *block_indices_begins;  // device
        int32_t num_seqs, num_tokens, num_blocks_total, max_context_len, max_q_len;
        int32_t prefill_row_blocks, prefill_kv_tokens;
    };
    Step LastStep() const;
    // A dense copy for an operation that wants the variable itself (ReadValueOp's device copy): [B, Hkv, T, D].
    int ReadDense(void* k_dev, void* v_dev, int T, int32_t* status, cudaStream_t stream) const;

    // ---- exact image of the state, for fixtures and for moving a cache between processes: the pool bytes of the
    // blocks in use plus the block lists, bit for bit (a u8 pool is NOT re-quantised by the round trip)
    size_t ExportBytes() const;
    int Export(void* host_blob, size_t bytes, cudaStream_t stream) const;
    int Import(const void* host_blob, size_t bytes, cudaStream_t stream);

private:
    int append_locked(const void* k_new, const void* v_new, int q_len, int32_t* status, cudaStream_t stream);
    int upload_tables(const StepTables& t, cudaStream_t stream);
    b2a_paged_desc desc(int num_tokens) const;

    const int kv_dtype_, x_dtype_, batch_, hkv_, d_, bs_, num_blocks_, max_step_tokens_;
    size_t x_size_ = 0, chunk_bytes_ = 0;
    mutable std::mutex mutex_;
    KvBlockManager manager_;
    StepTables last_;
    void *k_pool_ = nullptr, *v_pool_ = nullptr, *rows_k_ = nullptr, *rows_v_ = nullptr;
    int32_t* tables_dev_ = nullptr;    // [past_lens | subsequence_begins | block_indices_begins | block_indices]
    int32_t* tables_host_ = nullptr;   // pinned staging of the same
    size_t tables_ints_ = 0;
};

}  // namespace b2a
