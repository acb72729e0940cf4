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

// ov::op::v13::ScaledDotProductAttention: inputs query, key, value[, attention_mask]; attribute causal.
// A fifth (scale) operand is not accepted: it is a device scalar at run time and reading it would need a
// synchronisation inside Execute; constant-fold it into the query or leave it to the default 1/sqrt(E).
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
// head size, block size, element types and the capacity maxima (sequences per step, context length).  The live
// token / sequence counts of a step come from the request's DynamicBufferContext when the operand shapes are
// dynamic, so one instance serves every step of a continuous-batching loop and never has to be re-created per
// shape the way DynamicOperation does (modules/nvidia_plugin/src/cuda_dynamic_operation.cpp:420-528).
// Operands 3 and 4 (the caches) are updated in place: they must be bound to device-resident pool memory
// (the KvBlockManager's pool), not uploaded per inference like an ordinary Parameter
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
    // Capacity the grids and the workspace are sized for; defaults to the static operand shapes.
    // max_prefill_kv_tokens > 0 also reserves the f16 scratch that lets a step de-quantise the contexts of its
    // multi-token sequences once (up to that many context tokens, each sequence rounded up to 128).
    void SetCapacity(int max_seqs, int max_context_len, int max_prefill_kv_tokens = 0);
    // What the scheduler knows about the next step (KvBlockManager::StepTables carries both); zeros = unknown.
    // Hints beyond the reserved capacity are ignored.
    void SetStepHints(int32_t prefill_row_blocks, int32_t prefill_kv_tokens);
    const b2a_paged_desc& desc() const { return desc_; }

private:
    size_t WorkspaceBound() const;
    b2a_paged_desc desc_{};  // num_seqs / num_tokens hold the static extents (0 = dynamic)
    int max_seqs_ = 0, max_context_len_ = 0, max_prefill_kv_tokens_ = 0;
    int32_t hint_row_blocks_ = 0, hint_kv_tokens_ = 0;
    size_t workspace_bytes_ = 0;
};

}  // namespace nvidia_gpu
}  // namespace ov
