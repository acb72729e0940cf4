/*
 * b2a.h — C ABI of the B200 attention library (libb2a.so).
 *
 * The library replaces, for the attention path only, what OpenVINO's nvidia_plugin builds
 * out of a dozen elementary operations.  Each entry point names the reference interface
 * it stands in for (paths relative to modules/nvidia_plugin/ of openvino_contrib).
 *
 * Conventions
 *   - every pointer named q/k/v/o/..._cache/workspace/status and every i32 table is DEVICE memory
 *     unless the comment says "host";
 *   - every call only validates on the host and enqueues kernels on `stream`; none allocates,
 *     synchronises or copies across the host/device boundary, so all are legal inside stream capture
 *     (the plugin captures Execute() under cudaStreamCaptureModeThreadLocal, src/cuda/graph.cpp:76-78);
 *   - the return value is a b2a_status from host-side validation (0 = launched);
 *   - `status` (optional, may be NULL) is a device int32 the kernels OR error bits into when a bounded
 *     wait expires or an index check fails; the caller reads it whenever it synchronises.
 *
 * No function here has a CPU fallback: without a CUDA device the compute entry points return
 * B2A_ERR_CUDA.
 */
#ifndef B2A_H_
#define B2A_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* b2a_stream_t; /* == cudaStream_t */

typedef enum b2a_dtype { B2A_F32 = 0, B2A_F16 = 1, B2A_BF16 = 2, B2A_U8 = 3 } b2a_dtype;
typedef enum b2a_mask_kind { B2A_MASK_NONE = 0, B2A_MASK_BOOL = 1, B2A_MASK_ADD = 2 } b2a_mask_kind;

typedef enum b2a_status {
    B2A_OK = 0,
    B2A_ERR_NULL = 1,        /* a required pointer is NULL */
    B2A_ERR_DIM = 2,         /* a dimension is non-positive or inconsistent (Hq % Hkv, D limits, ...) */
    B2A_ERR_DTYPE = 3,       /* unsupported element type combination */
    B2A_ERR_ALIGN = 4,       /* a pointer or stride breaks the alignment the kernels need */
    B2A_ERR_WORKSPACE = 5,   /* workspace missing or too small */
    B2A_ERR_CUDA = 6,        /* a CUDA runtime call failed (no device, launch error) */
    B2A_ERR_UNSUPPORTED = 7, /* valid request this build has no kernel for */
    B2A_ERR_CAPACITY = 8,    /* block manager: pool exhausted / output array too small */
    B2A_ERR_NOT_FOUND = 9,   /* block manager: unknown sequence id */
    B2A_ERR_SCRATCH_LIMIT = 10 /* b2a_paged_attention_noalloc: the step needs more than the built-in scratch */
} b2a_status;

/* bits OR-ed into the device status word */
#define B2A_DEV_TIMEOUT 0x1u   /* a bounded wait (mbarrier / flag) gave up */
#define B2A_DEV_BAD_BLOCK 0x2u /* a block-table entry was outside [0, num_blocks_total) */
#define B2A_DEV_BAD_LEN 0x4u   /* a length/offset table was inconsistent */

/* ---------------------------------------------------------------------------------------------
 * ScaledDotProductAttention
 *
 * Replaces the chain the reference obtains from ov::pass::ScaledDotProductAttentionDecomposition
 * (src/transformer/cuda_graph_transformer.cpp:151-156): Multiply (src/ops/multiply.cpp:16-43),
 * Transpose (src/ops/transpose.cpp:58-135), MatMul via cublasGemmStridedBatchedEx
 * (src/ops/matmul.cpp:185-227), the causal-mask subgraph (src/kernels/comparison.cu:17-49,
 * src/kernels/select.cu:16-45, src/kernels/broadcast.cu:16-24), Add (src/ops/add.cpp:17-43),
 * Softmax via cudnnSoftmaxForward (src/ops/softmax.cpp:178-193) and the second MatMul.
 *
 * Layout: q [B,Hq,Sq,D], k [B,Hkv,Skv,D], v [B,Hkv,Skv,Dv], o [B,Hq,Sq,Dv]; strides in ELEMENTS,
 * innermost stride must be 1; an all-zero stride array means "contiguous".  Hq % Hkv == 0; query head h
 * reads KV head h / (Hq/Hkv).  causal != 0: query i keeps keys 0..i (top-left aligned) and the mask is
 * ignored.  mask: B2A_MASK_BOOL = u8, non-zero keeps; B2A_MASK_ADD = same dtype as q, added to the scaled
 * scores; mask_strides address a logical [B,Hq,Sq,Skv] tensor (stride 0 on broadcast dimensions).
 * scale == 0 selects 1/sqrt(D).
 * ------------------------------------------------------------------------------------------- */
typedef struct b2a_sdpa_desc {
    int32_t dtype; /* b2a_dtype of q, k, v and o */
    int32_t B, Hq, Hkv, Sq, Skv, D, Dv;
    int32_t causal;
    float scale;
    int64_t q_strides[4], k_strides[4], v_strides[4], o_strides[4];
    int32_t mask_kind; /* b2a_mask_kind */
    int32_t reserved;
    int64_t mask_strides[4];
} b2a_sdpa_desc;

/* Scratch bytes b2a_sdpa_forward needs for `desc` (0 is a valid answer).  Plays the part of
 * IOperationExec::GetWorkBufferRequest (src/cuda_operation_base.hpp:56, src/memory_manager/cuda_workbuffers.hpp:18-22). */
int b2a_sdpa_workspace_bytes(const b2a_sdpa_desc* desc, int sm_count, size_t* out_bytes);

/* Enqueue the fused attention.  Plays the part of the Execute() bodies listed above. */
int b2a_sdpa_forward(const b2a_sdpa_desc* desc, const void* q, const void* k, const void* v, const void* mask,
                     void* o, void* workspace, size_t workspace_bytes, int32_t* status, b2a_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * PagedAttentionExtension
 *
 * Replaces the reference's only KV-cache mechanism: ReadValueOp::Execute (src/ops/read_value.cpp:31-72),
 * the Concat of past and new K/V (src/kernels/concat.cu:16-32), AssignOp::Execute (src/ops/assign.cpp:29-56)
 * over CudaVariableState (src/cuda_variable_state.hpp:31-183), followed by the decomposed SDPA above.
 *
 * query [num_tokens, Hq*D], key [num_tokens, Hkv*D], value [num_tokens, Hkv*Dv], out [num_tokens, Hq*Dv],
 * row-major, dense.  Caches are block pools [num_blocks_total, Hkv, chunk]:
 *   kv_dtype == B2A_U8 : chunk = block_size*D u8 values (token-major), then block_size f16 scales, then
 *                        block_size f16 zero-points (per token, asymmetric: x = (u8 - zp) * scale);
 *                        chunk bytes = block_size*(D+4);
 *   kv_dtype == B2A_F16/B2A_BF16 : chunk = [block_size, D] elements of that type.
 * past_lens [num_seqs], subsequence_begins [num_seqs+1], block_indices [sum blocks],
 * block_indices_begins [num_seqs+1]: int32, device.  Token t of sequence s sits at cache position
 * past_lens[s] + (t - subsequence_begins[s]) and attends to positions 0..that, or only to the last
 * `sliding_window` of them when sliding_window > 0.
 * max_context_len bounds past_lens[s] + q_len[s] over all s; it sizes grids and the workspace so that the
 * same launch is valid for any lengths below it (graph replay with changed lengths).
 * max_q_len bounds q_len[s]; 1 selects the decode kernel.
 * ------------------------------------------------------------------------------------------- */
typedef struct b2a_paged_desc {
    int32_t q_dtype;  /* B2A_F16 | B2A_BF16 | B2A_F32: type of query, key, value and out */
    int32_t kv_dtype; /* B2A_U8 | B2A_F16 | B2A_BF16 */
    int32_t Hq, Hkv, D, Dv, block_size;
    int32_t num_seqs, num_tokens, num_blocks_total;
    int32_t max_context_len, max_q_len;
    float scale; /* 0 selects 1/sqrt(D) */
    int32_t sliding_window;
    /* Optional: sum over the sequences with two or more new tokens of ceil(q_len / 128), as the scheduler that
     * built the step knows it (b2a_kvmgr_last_prefill_row_blocks).  It only sizes the grid of the prefill kernel
     * more tightly; 0 = unknown, the bound num_tokens/128 + num_seqs is used.  A value that is too small makes the
     * kernel report B2A_DEV_BAD_LEN instead of computing a wrong answer. */
    int32_t prefill_row_blocks;
    /* Optional: an upper bound on the sum, over the sequences with two or more new tokens, of their context length
     * (past + new tokens) rounded up to 128 (b2a_kvmgr_last_prefill_kv_tokens).  With it (and room for it in the
     * workspace: b2a_paged_workspace_bytes counts 2 * Hkv * this * D * 2 bytes) those contexts are de-quantised once
     * into an f16 scratch and the prefill kernel stages K/V tiles by TMA; without it (0) every prefill CTA
     * de-quantises its own tiles.  A bound that is too small makes the step report B2A_DEV_BAD_LEN. */
    int32_t prefill_kv_tokens;
    /* Optional, decode rows only.  Non-zero: the caller promises that the kernel directly before this call on the stream
     * writes no cache row other than the rows of this step's new tokens (true when that kernel is this step's
     * b2a_paged_kv_store, or a kernel that does not touch the cache at all).  The decode kernel, which is launched
     * while that kernel still drains, then starts copying cache blocks that hold no new token before it waits for
     * it.  0 (the default): every cache read comes after the wait. */
    int32_t cache_rows_settled;
} b2a_paged_desc;

/* Bytes of one (block, KV head) chunk of a cache of `kv_dtype` with head size d. */
size_t b2a_paged_chunk_bytes(int32_t kv_dtype, int32_t block_size, int32_t d);

/* Scratch bytes b2a_paged_attention needs (split-K partials).  GetWorkBufferRequest counterpart. */
int b2a_paged_workspace_bytes(const b2a_paged_desc* desc, int sm_count, size_t* out_bytes);

/* Append this step's K/V rows to the pools through the block table, quantising to u8 when the cache is u8.
 * Counterpart of the Concat + Assign pair (src/kernels/concat.cu:16-32, src/ops/assign.cpp:29-56). */
int b2a_paged_kv_store(const b2a_paged_desc* desc, const void* key, const void* value, void* k_cache,
                       void* v_cache, const int32_t* past_lens, const int32_t* subsequence_begins,
                       const int32_t* block_indices, const int32_t* block_indices_begins, int32_t* status,
                       b2a_stream_t stream);

/* b2a_paged_kv_store with the rotary position embedding of the KEY rows fused in: the first rotary_dim values of a key
 * row at cache position p are rotated in pairs (i, i + rotary_dim/2) by the angle whose cosine and sine are
 * cos_table[p][i] and sin_table[p][i] (device float32 tables [table_positions][rotary_dim/2]; the "rotate-half" form of
 * the Llama family), each product and sum one float32 operation rounded to nearest, and the rotated float32 values are
 * what is quantised.  Values are stored as they are.  No counterpart in the reference: there the rotation reaches the
 * plugin decomposed into Multiply / Concat / Add nodes and costs a pass over K in memory (src/ops/multiply.cpp:16-43,
 * src/kernels/concat.cu:16-32); a model hands the un-rotated key projection to this call instead.  A position beyond
 * the table is reported (B2A_DEV_BAD_LEN) and its row left unwritten. */
int b2a_paged_kv_store_rope(const b2a_paged_desc* desc, const void* key, const void* value, void* k_cache,
                            void* v_cache, const int32_t* past_lens, const int32_t* subsequence_begins,
                            const int32_t* block_indices, const int32_t* block_indices_begins, const float* cos_table,
                            const float* sin_table, int32_t rotary_dim, int32_t table_positions, int32_t* status,
                            b2a_stream_t stream);

/* Attention of every query token over its sequence's cache (call after b2a_paged_kv_store of the same step).
 * Counterpart of ReadValue + decomposed SDPA (src/ops/read_value.cpp:31-72 and the SDPA chain above).
 * The four table arrays of a step must be complete before the step's kernels are launched: the kernels are launched
 * programmatically dependent on the kernel before them on the stream and read the tables while that kernel drains,
 * so that kernel must not be the one that writes them (tables uploaded from the host, or written by any earlier
 * kernel, are fine; so is replaying a captured step after changing them). */
int b2a_paged_attention(const b2a_paged_desc* desc, const void* query, const void* k_cache, const void* v_cache,
                        const int32_t* past_lens, const int32_t* subsequence_begins, const int32_t* block_indices,
                        const int32_t* block_indices_begins, void* out, void* workspace, size_t workspace_bytes,
                        int32_t* status, b2a_stream_t stream);

/* Decode attention for callers that cannot provide a workspace and must not allocate one.
 * No counterpart in the reference: there every operation declares its scratch through GetWorkBufferRequest and
 * the plugin's memory manager lays it out when the model is compiled.  Code that reaches this library some other
 * way has no such channel and often no way to call cudaMalloc at the point of the call either: an operator body
 * running under stream capture (an allocation there ends the capture with an error), a custom-operation
 * extension that only ever sees its input and output buffers, a serving loop that has handed the whole device
 * memory to its KV pool up front.  For them the split-K partials live in an array that is part of the library
 * image: B2A_BUILTIN_SCRATCH_BYTES on every GPU that loads libb2a.so, held until the process exits.
 *
 * Same arguments and results as b2a_paged_attention, minus the workspace, with these limits:
 *   - decode steps only: one query token per sequence, u8 cache, D = Dv = 128, block size 16, f16 or bf16
 *     queries (otherwise B2A_ERR_UNSUPPORTED);
 *   - the step's split-K partials (b2a_paged_workspace_bytes of the same descriptor) must fit the built-in
 *     array, otherwise B2A_ERR_SCRATCH_LIMIT and nothing is launched;
 *   - the first call on each device looks up the array's device address (no allocation, but a runtime query):
 *     make that first call before any stream capture begins;
 *   - all calls on one device share the one array, and it keeps whatever the previous call left in it (no part
 *     of it needs clearing between calls): calls that may run concurrently on the GPU race on it, so keep them
 *     on one stream or order them with events. */
#define B2A_BUILTIN_SCRATCH_BYTES (16u << 20)
int b2a_paged_attention_noalloc(const b2a_paged_desc* desc, const void* query, const void* k_cache,
                                const void* v_cache, const int32_t* past_lens, const int32_t* subsequence_begins,
                                const int32_t* block_indices, const int32_t* block_indices_begins, void* out,
                                int32_t* status, b2a_stream_t stream);

/* Score output of PagedAttentionExtension (its second output, which cache-eviction policies accumulate; the
 * reference's policy consumes such sums, modules/genai_optimizations/genai_opt/token_eviction.py:154-183): for every
 * sequence of the step, the attention probabilities of its LAST query token over the sequence's cached keys, summed
 * over the query heads.  Call after b2a_paged_kv_store of the step (the new tokens' keys are part of the context).
 *   scores        float32, flat: sequence s occupies [score_begins[s], score_begins[s+1]) with one value per context
 *                 position 0 .. past + new tokens - 1 (positions a sliding window leaves out: 0); a sequence without a
 *                 new token has no entries.  Every sequence's values sum to Hq.
 *   score_begins  int32 [num_seqs + 1], written by the call.
 *   scores_capacity  floats `scores` holds; a step that needs more reports B2A_DEV_BAD_LEN and writes nothing beyond.
 * u8 caches with D = 128, 16-token blocks, f16 / bf16 queries, at most eight query heads per KV head and 128 query
 * heads; anything else is B2A_ERR_UNSUPPORTED.  Only K is read, twice.  Enqueue-only, graph-capturable. */
int b2a_paged_scores_workspace_bytes(const b2a_paged_desc* desc, int sm_count, size_t* out_bytes);
int b2a_paged_last_token_scores(const b2a_paged_desc* desc, const void* query, const void* k_cache,
                                const int32_t* past_lens, const int32_t* subsequence_begins,
                                const int32_t* block_indices, const int32_t* block_indices_begins, float* scores,
                                int64_t scores_capacity, int32_t* score_begins, void* workspace, size_t workspace_bytes,
                                int32_t* status, b2a_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * Head-sharded attention over the GPUs of one node (one rank per GPU).
 *
 * No counterpart in the reference, which never spans devices (one independent plugin configuration per device
 * id, src/cuda_plugin.cpp:25-32).  Rank r of `world` owns KV heads [r*Hkv/world, (r+1)*Hkv/world) and their query
 * heads; K/V never cross NVLink.  The per-head outputs are exchanged by the kernels that produce them: they store
 * this rank's part of the result into the group's memory on EVERY rank (peer stores over NVLink); no collective
 * library is on the data path.
 *
 * Set-up (allocates; not for the hot path): every rank creates its group; when the ranks are processes, the 64-byte
 * handles of all ranks are exchanged by any host-side means (torch.distributed all_gather, MPI, a file), in rank
 * order, and passed to _connect; when one process drives several ranks (peer access enabled between their devices)
 * it passes every rank's b2a_shard_group_output pointer to _connect_pointers instead.
 * staging_bytes: decode steps into a caller's buffer need 2 * num_tokens * Hq_total * D * 2 of the largest step (the
 * values travel with the step number in 8-byte words that the receiver polls: no flag round trip), decode steps in
 * place num_tokens * Hq_total * D * 2, prefill steps the full output.
 *
 * Failure handling: every device-side wait on another rank is bounded in wall-clock time (one second unless
 * _set_wait_ms says otherwise).  When it runs out the kernel returns, the step's result is incomplete and the status
 * word carries B2A_DEV_TIMEOUT.  After a timeout the ranks' step counters no longer agree: every rank calls
 * b2a_shard_group_reset (between steps, with a host-side barrier of all ranks before the next step) or the group is
 * destroyed and rebuilt.
 * ------------------------------------------------------------------------------------------- */
typedef struct b2a_shard_group b2a_shard_group;
int b2a_shard_group_create(int rank, int world, size_t staging_bytes, b2a_shard_group** out);
int b2a_shard_group_handle(const b2a_shard_group* g, unsigned char handle[64]);
int b2a_shard_group_connect(b2a_shard_group* g, const unsigned char* handles /* world * 64 bytes, rank order */);
/* Same-process form of _connect: bases[r] = what b2a_shard_group_output returned for rank r's group (bases[rank] is
 * ignored).  The pointers must be usable from this rank's device (same device, or peer access enabled). */
int b2a_shard_group_connect_pointers(b2a_shard_group* g, void* const* bases /* world entries, rank order */);
/* Bound of every device-side wait on another rank for the calls that follow (default 1000 ms). */
int b2a_shard_group_set_wait_ms(b2a_shard_group* g, int milliseconds);
/* Synchronises this rank's device, clears the group's flags, counters and staging memory and forgets the kind of
 * step it served: the state of a fresh group.  Collective in effect, because peers store into this memory: every
 * rank first lets its own device go idle (cudaDeviceSynchronize), then - after a host-side barrier of all ranks -
 * calls this, and no rank enqueues a step before a second barrier. */
int b2a_shard_group_reset(b2a_shard_group* g);
void b2a_shard_group_destroy(b2a_shard_group* g);
/* The group's own memory on this rank (fixed for the group's life).  Passing it as `out_full` to
 * b2a_paged_attention_sharded selects the in-place step: the rows are stored straight into this buffer on EVERY
 * rank, the kernel's last CTA publishes the step and waits (bounded) for the other ranks - one launch, no copy,
 * capturable in a CUDA graph.  The rows are then read in place; they stay valid until this rank enqueues its next
 * step on the group. */
int b2a_shard_group_output(const b2a_shard_group* g, void** out);
/* Decode step on this rank's heads (`local_desc` carries the LOCAL Hq and Hkv; query [num_tokens, Hq_local*D];
 * caches hold the local KV heads), output exchanged as above: out_full [num_tokens, Hq_local*world*D] is complete
 * on every rank when the stream reaches the end of the call's work.  The decode kernel's last CTA of every
 * (sequence, KV head) merges the splits and sends the rows; with a caller's `out_full` a second small kernel polls
 * the arriving words and fills it (two launches per step, capturable).  Decode shapes only (as
 * b2a_paged_attention_noalloc); workspace as b2a_paged_workspace_bytes(local_desc).  All ranks must call it the
 * same number of times; a rank that never arrives makes the others report B2A_DEV_TIMEOUT when the wait bound
 * runs out. */
int b2a_paged_attention_sharded(b2a_shard_group* g, const b2a_paged_desc* local_desc, const void* query,
                                const void* k_cache, const void* v_cache, const int32_t* past_lens,
                                const int32_t* subsequence_begins, const int32_t* block_indices,
                                const int32_t* block_indices_begins, void* out_full, void* workspace,
                                size_t workspace_bytes, int32_t* status, b2a_stream_t stream);
/* Prefill SDPA on this rank's heads (`local_desc` carries the LOCAL Hq and Hkv and the strides of the local q, k, v;
 * o_strides and the mask fields are ignored: no mask operand, dense output).  The tensor-core kernel's epilogue
 * stores every finished output tile into the full-width buffer of EVERY rank (one TMA store per rank, so the
 * exchange overlaps the rest of the grid's computation), then the stream waits, bounded, for the other ranks.
 * *out_full points at this rank's complete [B, Hq_local*world, Sq, Dv] result inside the group's memory (the two
 * halves of the staging area alternate by step): it is valid once the stream has passed the call's work, and stays
 * so for work enqueued before the next call on this group.  Shapes: what the tensor-core kernel takes (f16/bf16,
 * D = Dv = 128, 16-byte aligned strides), else B2A_ERR_UNSUPPORTED; staging_bytes >= the full output.  A group
 * serves either decode steps or prefill steps (the first call decides), and a sharded prefill call is not
 * capturable in a CUDA graph (the buffer alternation is host state).  No counterpart in the reference. */
int b2a_sdpa_forward_sharded(b2a_shard_group* g, const b2a_sdpa_desc* local_desc, const void* q, const void* k,
                             const void* v, void** out_full, int32_t* status, b2a_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * KV block manager (host only; no CUDA calls).  Owns the free list of a pool of `num_blocks` physical
 * blocks and the per-sequence block lists, and emits the four int32 tables of a step.  It takes the place
 * CudaVariableState has for the contiguous cache (src/cuda_variable_state.hpp:31-183: reset / grow / hand
 * out the buffer), for a paged pool.
 * ------------------------------------------------------------------------------------------- */
typedef struct b2a_kvmgr b2a_kvmgr;

int b2a_kvmgr_create(int32_t num_blocks, int32_t block_size, uint64_t shuffle_seed, b2a_kvmgr** out);
void b2a_kvmgr_destroy(b2a_kvmgr* m);
int b2a_kvmgr_add_sequence(b2a_kvmgr* m, int64_t seq_id);
int b2a_kvmgr_free_sequence(b2a_kvmgr* m, int64_t seq_id);
int32_t b2a_kvmgr_free_blocks(const b2a_kvmgr* m);
int32_t b2a_kvmgr_sequence_len(const b2a_kvmgr* m, int64_t seq_id); /* -1 if unknown */
/* b2a_paged_desc.prefill_row_blocks of the step scheduled last */
int32_t b2a_kvmgr_last_prefill_row_blocks(const b2a_kvmgr* m);
/* b2a_paged_desc.prefill_kv_tokens of the step scheduled last */
int32_t b2a_kvmgr_last_prefill_kv_tokens(const b2a_kvmgr* m);
/* Reserve blocks for q_lens[i] new tokens of seq_ids[i] (all or nothing), fill the step tables (host arrays:
 * past_lens[n], subsequence_begins[n+1], block_indices[capacity], block_indices_begins[n+1]) and advance
 * the sequences' lengths.  *num_block_indices and *max_context_len receive the totals. */
int b2a_kvmgr_schedule_step(b2a_kvmgr* m, const int64_t* seq_ids, const int32_t* q_lens, int32_t n,
                            int32_t* past_lens, int32_t* subsequence_begins, int32_t* block_indices,
                            int32_t block_indices_capacity, int32_t* block_indices_begins,
                            int32_t* num_block_indices, int32_t* max_context_len);

/* ---------------------------------------------------------------------------------------------
 * ScaledDotProductAttention on HOST tensors: what the plugin does for a model whose inputs and outputs live in host
 * memory - ParameterOp uploads (src/ops/parameter.cpp:24-33), the operation runs, ResultOp downloads
 * (src/ops/result.cpp:28-43) - with the three overlapped: the problem is cut into pieces of a few KV heads of one batch entry,
 * and the upload of piece i+1, the operation on piece i and the download of piece i-1 run at the same time on three
 * streams.  The operation is the C++ SdpaOp, created through the operation registry, executed once per piece; called
 * again with the same four tensors, the whole step is captured into a CUDA graph once and replayed from then on.
 * _create allocates (device tensors for the shapes given, streams, events); _run only enqueues: q, k, v, out are
 * host pointers in [B, H, S, D] layout (pinned, or the copies serialise), the work is ordered after what `stream`
 * holds and `stream` waits for the last download.
 * ------------------------------------------------------------------------------------------- */
typedef struct b2a_host_sdpa b2a_host_sdpa;
/* kv_heads_per_piece: KV heads (with the query heads that read them) per piece, a divisor of Hkv; 0 = chosen so that a
 * piece uploads at least 8 MB (much smaller copies do not reach the bus's bandwidth). */
int b2a_host_sdpa_create(int32_t dtype, int32_t B, int32_t Hq, int32_t Hkv, int32_t Sq, int32_t Skv, int32_t D,
                         int32_t causal, int32_t kv_heads_per_piece, b2a_host_sdpa** out);
int b2a_host_sdpa_run(b2a_host_sdpa* h, const void* q, const void* k, const void* v, void* out, b2a_stream_t stream);
int b2a_host_sdpa_pieces(const b2a_host_sdpa* h);
void b2a_host_sdpa_destroy(b2a_host_sdpa* h);

/* ---------------------------------------------------------------------------------------------
 * KV cache of a STATEFUL model kept in the paged pool.
 *
 * Takes the place of CudaVariableState (src/cuda_variable_state.hpp:31-183) for the two variables - K and V, each a
 * dense [B, Hkv, T, D] tensor - that a ReadValue / Concat / Assign model keeps per attention layer
 * (src/ops/read_value.cpp:31-72, src/ops/assign.cpp:29-56, src/kernels/concat.cu:16-32), with the bytes living in the
 * block pool the paged kernels read: Assign(Concat(ReadValue, new)) becomes _append (the new rows are quantised into
 * their blocks; the past is not copied), ReadValue -> attention becomes _last_step (pools + step tables in
 * PagedAttentionExtension's operand order).  reset / set_state / get_state keep their meaning for the user-facing
 * API (src/cuda_variable_state.hpp:62-105); _export / _import move the exact pool image, for fixtures.
 * One object = one layer, B sequences of equal length.  _create, _set_state, _get_state, _export, _import allocate
 * and synchronise (slow paths); _append, _read_dense and _last_step only enqueue.
 * ------------------------------------------------------------------------------------------- */
typedef struct b2a_kvstate b2a_kvstate;
typedef struct b2a_kvstate_step {
    const void *k_cache, *v_cache;                                                           /* device pools */
    const int32_t *past_lens, *subsequence_begins, *block_indices, *block_indices_begins;   /* device tables */
    int32_t num_seqs, num_tokens, num_blocks_total, max_context_len, max_q_len;
    int32_t prefill_row_blocks, prefill_kv_tokens;                                           /* b2a_paged_desc hints */
} b2a_kvstate_step;
/* kv_dtype: pool element type (B2A_U8 | B2A_F16 | B2A_BF16); x_dtype: the variable's element type (B2A_F32 | B2A_F16 |
 * B2A_BF16); max_step_tokens bounds q_len of one _append. */
int b2a_kvstate_create(int32_t kv_dtype, int32_t x_dtype, int32_t batch, int32_t hkv, int32_t d, int32_t block_size,
                       int32_t num_blocks, int32_t max_step_tokens, b2a_kvstate** out);
void b2a_kvstate_destroy(b2a_kvstate* s);
int32_t b2a_kvstate_length(const b2a_kvstate* s); /* T: positions held per sequence */
int b2a_kvstate_reset(b2a_kvstate* s);
/* k_host / v_host: HOST tensors [B, Hkv, T, D] of x_dtype.  _get_state wants T == b2a_kvstate_length; a u8 pool
 * returns the de-quantised values (code - zp) * scale, i.e. what the attention kernels compute with. */
int b2a_kvstate_set_state(b2a_kvstate* s, const void* k_host, const void* v_host, int32_t T, b2a_stream_t stream);
int b2a_kvstate_get_state(const b2a_kvstate* s, void* k_host, void* v_host, int32_t T, b2a_stream_t stream);
/* k_new / v_new: DEVICE tensors [B, Hkv, q_len, D] of x_dtype.  B2A_ERR_CAPACITY (nothing changed) when the pool is
 * exhausted. */
int b2a_kvstate_append(b2a_kvstate* s, const void* k_new, const void* v_new, int32_t q_len, int32_t* status,
                       b2a_stream_t stream);
/* The variable itself as a dense DEVICE tensor [B, Hkv, T, D] (what ReadValueOp would have copied out). */
int b2a_kvstate_read_dense(const b2a_kvstate* s, void* k_dev, void* v_dev, int32_t T, int32_t* status,
                           b2a_stream_t stream);
/* Pools and tables of the last _append (valid until the next _append / _set_state / _reset / _import). */
int b2a_kvstate_last_step(const b2a_kvstate* s, b2a_kvstate_step* out);
size_t b2a_kvstate_export_bytes(const b2a_kvstate* s);
int b2a_kvstate_export(const b2a_kvstate* s, void* host_blob, size_t bytes, b2a_stream_t stream);
int b2a_kvstate_import(b2a_kvstate* s, const void* host_blob, size_t bytes, b2a_stream_t stream);

const char* b2a_status_string(int status);
int b2a_version(void);

#ifdef __cplusplus
}
#endif
#endif /* B2A_H_ */
