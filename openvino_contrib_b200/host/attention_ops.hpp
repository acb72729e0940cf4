// The two attention operators, written against the nvidia_plugin operation interface
// (OperationBase, modules/nvidia_plugin/src/cuda_operation_base.hpp:80-149) and registered under the OpenVINO
// type names with OPERATION_REGISTER (modules/nvidia_plugin/src/cuda_operation_registry.hpp:133-137).
//
// With these registered, GraphTransformer must no longer run ScaledDotProductAttentionDecomposition
// (modules/nvidia_plugin/src/transformer/cuda_graph_transformer.cpp:151-156): the node reaches
// SubGraph::initExecuteSequence whole and is built through the registry like any other operation.
#pragma once

#include "b2a.h"
#include "ov_shim.hpp"

namespace ov {
namespace nvidia_gpu {

// ov::op::v13::ScaledDotProductAttention: inputs query, key, value[, attention_mask[, scale]]; attribute causal.
// The scale operand is accepted when its producer is a Constant (its value is read at construction, the way the
// reference's operations read constant operands); a scale computed at run time is refused: it is a device scalar
// and reading it would need a synchronisation inside Execute.
class SdpaOp : public OperationBase {
public:
    using NodeOp = ov::op::v13::ScaledDotProductAttention;
    SdpaOp(const CreationContext& context, const NodeOp& node, IndexCollection&& inputIds, IndexCollection&& outputIds);
    void Execute(const InferenceRequestContext& context, Inputs inputTensors, Outputs outputTensors,
                 const Workbuffers& workbuffers) const override;
    CudaGraphCompatibility GetCudaGraphCompatibilityImpl() const override { return CudaGraphCompatibility::FULL; }
    WorkbufferRequest GetWorkBufferRequest() const override;
    const b2a_sdpa_desc& desc() const { return desc_; }

private:
    b2a_sdpa_desc desc_{};
    size_t workspace_bytes_ = 0;
    bool has_mask_ = false;
};

// PagedAttentionExtension.  The constructor depends only on what is static for a compiled model: head counts,
// head size, block size, element types and the capacity maxima.  The live token / sequence counts of a step come
// from the request's DynamicBufferContext when the operand shapes are dynamic, so one instance serves every step of
// a continuous-batching loop and never has to be re-created per shape the way DynamicOperation does
// (modules/nvidia_plugin/src/cuda_dynamic_operation.cpp:420-528).
// Nothing about the object changes after construction (operation objects are shared by concurrent requests,
// modules/nvidia_plugin/src/cuda_operation_base.hpp:41-44):
//   - capacity (grids and work buffers are sized for it) comes from the node's run-time information, keys
//     "b2a.max_seqs", "b2a.max_context_len", "b2a.max_step_tokens", "b2a.max_prefill_kv_tokens"; defaults: the
//     static operand shapes, the pool size, one full context plus a token per sequence, and no scratch for
//     de-quantised prefill contexts;
//   - what the scheduler knows about one step (AttentionStepHints) comes with the request context.  Without hints a
//     step with multi-token sequences is sized by the capacity, so a captured graph replays whatever the step holds.
// Operands 3 and 4 (the caches) are updated in place: they must be bound to device-resident pool memory
// (KvPoolState), not uploaded per inference like an ordinary Parameter
// (modules/nvidia_plugin/src/ops/parameter.cpp:24-33).
class PagedAttentionOp : public OperationBase {
public:
    using NodeOp = ov::op::PagedAttentionExtension;
    PagedAttentionOp(const CreationContext& context, const NodeOp& node, IndexCollection&& inputIds,
                     IndexCollection&& outputIds);
    void Execute(const InferenceRequestContext& context, Inputs inputTensors, Outputs outputTensors,
                 const Workbuffers& workbuffers) const override;
    CudaGraphCompatibility GetCudaGraphCompatibilityImpl() const override { return CudaGraphCompatibility::FULL; }
    WorkbufferRequest GetWorkBufferRequest() const override;
    const b2a_paged_desc& desc() const { return desc_; }
    int max_seqs() const { return max_seqs_; }
    int max_context_len() const { return max_context_len_; }
    int max_step_tokens() const { return max_step_tokens_; }
    // The node's second output (scores of every sequence's last query token, flat float32) is produced when the node
    // has one: the bound buffer must hold score_capacity() floats (run-time information "b2a.max_score_entries",
    // default max_seqs * max_context_len); the third work buffer then holds the score kernels' scratch followed by
    // the int32 [max_seqs + 1] offsets of the sequences in the output.
    bool has_scores() const { return score_capacity_ > 0; }
    int64_t score_capacity() const { return score_capacity_; }
    size_t score_begins_offset() const { return score_ws_bytes_; }
    // The descriptor Execute would launch for a step of these extents and hints (the checks Execute makes, without
    // the launch): what the capacity tests compare the work-buffer request against.
    b2a_paged_desc StepDesc(int num_tokens, int num_seqs, const AttentionStepHints& hints) const;

private:
    size_t WorkspaceBound() const;
    b2a_paged_desc desc_{};  // num_seqs / num_tokens hold the static extents (0 = dynamic)
    int max_seqs_ = 0, max_context_len_ = 0, max_step_tokens_ = 0, max_prefill_kv_tokens_ = 0;
    size_t workspace_bytes_ = 0;
    int64_t score_capacity_ = 0;   // 0: the node has no second output
    size_t score_ws_bytes_ = 0;
};

}  // namespace nvidia_gpu
}  // namespace ov
