#include "attention_ops.hpp"

#include <algorithm>
#include <string>

namespace ov {
namespace nvidia_gpu {
namespace {

int dtype_of(const ov::element::Type& t) {
    switch (static_cast<ov::element::Type_t>(t)) {
        case ov::element::Type_t::f32: return B2A_F32;
        case ov::element::Type_t::f16: return B2A_F16;
        case ov::element::Type_t::bf16: return B2A_BF16;
        case ov::element::Type_t::u8: return B2A_U8;
        default: return -1;
    }
}

void throwIfError(int rc, const std::string& where) {
    if (rc != B2A_OK) ov::throw_ov_exception(where + ": " + b2a_status_string(rc));
}

// [.., H, S, E] -> (B, H, S, E); rank 3 is [N, S, E]
void split_bhse(const ov::Shape& s, int& b, int& h, int& l, int& e) {
    if (s.size() < 3) ov::throw_ov_exception("ScaledDotProductAttention: operand rank must be >= 3");
    e = static_cast<int>(s[s.size() - 1]);
    l = static_cast<int>(s[s.size() - 2]);
    if (s.size() == 3) {
        h = 1;
        b = static_cast<int>(s[0]);
    } else {
        h = static_cast<int>(s[s.size() - 3]);
        size_t bb = 1;
        for (size_t i = 0; i + 3 < s.size(); ++i) bb *= s[i];
        b = static_cast<int>(bb);
    }
}

}  // namespace

SdpaOp::SdpaOp(const CreationContext& context, const NodeOp& node, IndexCollection&& inputIds,
               IndexCollection&& outputIds)
    : OperationBase(context, node, std::move(inputIds), std::move(outputIds)) {
    const size_t n_in = node.get_input_size();
    if (n_in < 3 || n_in > 4)
        ov::throw_ov_exception("ScaledDotProductAttention: 3 or 4 inputs supported (a scale operand must be folded)");
    const int dt = dtype_of(node.get_input_element_type(0));
    if (dt < 0 || dt == B2A_U8) ov::throw_ov_exception("ScaledDotProductAttention: unsupported precision");
    for (size_t i = 1; i < 3; ++i)
        if (node.get_input_element_type(i) != node.get_input_element_type(0))
            ov::throw_ov_exception("ScaledDotProductAttention: q, k, v precisions differ");
    int bq, hq, sq, e, bk, hk, sk, ek, bv, hv, sv, ev;
    split_bhse(node.get_input_shape(0), bq, hq, sq, e);
    split_bhse(node.get_input_shape(1), bk, hk, sk, ek);
    split_bhse(node.get_input_shape(2), bv, hv, sv, ev);
    if (bq != bk || bq != bv || hk != hv || sk != sv || e != ek)
        ov::throw_ov_exception("ScaledDotProductAttention: inconsistent operand shapes");
    desc_.dtype = dt;
    desc_.B = bq; desc_.Hq = hq; desc_.Hkv = hk; desc_.Sq = sq; desc_.Skv = sk; desc_.D = e; desc_.Dv = ev;
    desc_.causal = node.get_causal() ? 1 : 0;
    desc_.scale = 0.f;  // 1/sqrt(E)
    desc_.mask_kind = B2A_MASK_NONE;
    if (n_in == 4 && !node.get_causal()) {
        has_mask_ = true;
        const auto& mt = node.get_input_element_type(3);
        if (mt == ov::element::boolean || mt == ov::element::u8) {
            desc_.mask_kind = B2A_MASK_BOOL;
        } else if (mt == node.get_input_element_type(0)) {
            desc_.mask_kind = B2A_MASK_ADD;
        } else {
            ov::throw_ov_exception("ScaledDotProductAttention: mask precision must be boolean or that of the query");
        }
        // numpy-broadcast the mask shape against [B, Hq, Sq, Skv]: stride 0 where its extent is 1 or missing
        const ov::Shape& ms = node.get_input_shape(3);
        if (ms.size() > 4) ov::throw_ov_exception("ScaledDotProductAttention: mask rank > 4");
        const int64_t full[4] = {bq, hq, sq, sk};
        int64_t stride = 1;
        for (int i = 3; i >= 0; --i) {
            const int mi = static_cast<int>(ms.size()) - (4 - i);
            const int64_t ext = mi >= 0 ? static_cast<int64_t>(ms[static_cast<size_t>(mi)]) : 1;
            if (ext != 1 && ext != full[i]) ov::throw_ov_exception("ScaledDotProductAttention: mask not broadcastable");
            desc_.mask_strides[i] = ext == 1 ? 0 : stride;
            stride *= ext;
        }
    }
    throwIfError(b2a_sdpa_workspace_bytes(&desc_, 0, &workspace_bytes_), "b2a_sdpa_workspace_bytes");
}

WorkbufferRequest SdpaOp::GetWorkBufferRequest() const {
    WorkbufferRequest r;
    if (workspace_bytes_ > 0) r.mutable_sizes.push_back(workspace_bytes_);
    return r;
}

void SdpaOp::Execute(const InferenceRequestContext& context, Inputs in, Outputs out, const Workbuffers& wb) const {
    if (in.size() < 3 || out.size() != 1) ov::throw_ov_exception("ScaledDotProductAttention: operand count");
    const void* mask = has_mask_ ? in[3].get() : nullptr;
    void* ws = (workspace_bytes_ > 0 && !wb.mutable_buffers.empty()) ? wb.mutable_buffers[0].get() : nullptr;
    throwIfError(b2a_sdpa_forward(&desc_, in[0].get(), in[1].get(), in[2].get(), mask, out[0].get(), ws,
                                  workspace_bytes_, nullptr,
                                  reinterpret_cast<b2a_stream_t>(context.getThreadContext().stream().get())),
                 "b2a_sdpa_forward");
}

PagedAttentionOp::PagedAttentionOp(const CreationContext& context, const NodeOp& node, IndexCollection&& inputIds,
                                   IndexCollection&& outputIds)
    : OperationBase(context, node, std::move(inputIds), std::move(outputIds)) {
    if (node.get_input_size() < 11) ov::throw_ov_exception("PagedAttentionExtension: at least 11 inputs expected");
    if (node.get_input_size() > 11 && node.get_input_shape(11).size() > 0 && node.get_input_shape(11)[0] != 0)
        ov::throw_ov_exception("PagedAttentionExtension: alibi slopes are not supported");
    const int qdt = dtype_of(node.get_input_element_type(0));
    const int kvdt = dtype_of(node.get_input_element_type(3));
    if (qdt < 0 || qdt == B2A_U8 || kvdt < 0 || kvdt == B2A_F32)
        ov::throw_ov_exception("PagedAttentionExtension: unsupported precision");
    // key_cache [num_blocks, Hkv, block_size, D (+4 bytes of f16 scale / zero-point per token when u8)]
    const ov::Shape& kc = node.get_input_shape(3);
    const ov::Shape& vc = node.get_input_shape(4);
    if (kc.size() != 4 || vc.size() != 4) ov::throw_ov_exception("PagedAttentionExtension: caches must be rank 4");
    const int meta = kvdt == B2A_U8 ? 4 : 0;
    desc_.q_dtype = qdt;
    desc_.kv_dtype = kvdt;
    desc_.num_blocks_total = static_cast<int>(kc[0]);
    desc_.Hkv = static_cast<int>(kc[1]);
    desc_.block_size = static_cast<int>(kc[2]);
    desc_.D = static_cast<int>(kc[3]) - meta;
    desc_.Dv = static_cast<int>(vc[3]) - meta;
    const ov::Shape& qs = node.get_input_shape(0);
    if (qs.size() != 2 || desc_.D <= 0 || qs[1] % static_cast<size_t>(desc_.D) != 0)
        ov::throw_ov_exception("PagedAttentionExtension: query must be [tokens, Hq*D]");
    desc_.Hq = static_cast<int>(qs[1]) / desc_.D;
    if (desc_.Hkv <= 0 || desc_.Hq % desc_.Hkv != 0) ov::throw_ov_exception("PagedAttentionExtension: Hq % Hkv != 0");
    desc_.scale = node.const_scale.value_or(0.f);  // 0 selects 1/sqrt(D)
    desc_.sliding_window = node.const_sliding_window.value_or(0);
    desc_.num_tokens = static_cast<int>(qs[0]);  // 0 = dynamic: read per step
    desc_.num_seqs = static_cast<int>(node.get_input_shape(5).empty() ? 0 : node.get_input_shape(5)[0]);
    max_seqs_ = desc_.num_seqs > 0 ? desc_.num_seqs : 256;
    max_context_len_ = std::max(1, desc_.num_blocks_total * desc_.block_size);
    has_dynamic_buffer_ = false;
    workspace_bytes_ = WorkspaceBound();
}

void PagedAttentionOp::SetCapacity(int max_seqs, int max_context_len, int max_prefill_kv_tokens) {
    if (max_seqs <= 0 || max_context_len <= 0 || max_prefill_kv_tokens < 0)
        ov::throw_ov_exception("PagedAttentionExtension: bad capacity");
    max_seqs_ = max_seqs;
    max_context_len_ = max_context_len;
    max_prefill_kv_tokens_ = max_prefill_kv_tokens;
    workspace_bytes_ = WorkspaceBound();
}

void PagedAttentionOp::SetStepHints(int32_t prefill_row_blocks, int32_t prefill_kv_tokens) {
    hint_row_blocks_ = prefill_row_blocks > 0 ? prefill_row_blocks : 0;
    hint_kv_tokens_ = prefill_kv_tokens > 0 && prefill_kv_tokens <= max_prefill_kv_tokens_ ? prefill_kv_tokens : 0;
}

size_t PagedAttentionOp::WorkspaceBound() const {
    // The split plan depends on the live sequence count, so take the largest request over 1..max_seqs.
    size_t worst = 16;
    for (int n = 1; n <= max_seqs_; ++n) {
        b2a_paged_desc d = desc_;
        d.num_seqs = n;
        // a mixed step: the decode partials for n sequences plus the prefill work list for the token capacity
        d.num_tokens = max_context_len_ + max_seqs_;
        d.max_context_len = max_context_len_;
        d.max_q_len = 2;
        d.prefill_kv_tokens = max_prefill_kv_tokens_;
        size_t bytes = 0;
        throwIfError(b2a_paged_workspace_bytes(&d, 0, &bytes), "b2a_paged_workspace_bytes");
        worst = std::max(worst, bytes);
    }
    return worst;
}

WorkbufferRequest PagedAttentionOp::GetWorkBufferRequest() const {
    // [0] split-K partials of the decode kernel, sized for the capacity; [1] the device status word
    WorkbufferRequest r;
    r.mutable_sizes.push_back(workspace_bytes_);
    r.mutable_sizes.push_back(16);
    return r;
}

void PagedAttentionOp::Execute(const InferenceRequestContext& context, Inputs in, Outputs out,
                               const Workbuffers& wb) const {
    if (in.size() < 11 || out.size() < 1) ov::throw_ov_exception("PagedAttentionExtension: operand count");
    b2a_paged_desc d = desc_;
    // live extents: dynamic shapes recorded for this request win over the static ones
    const auto& dyn = context.getDynamicBufferContext();
    if (auto s = dyn.getShape(input_ids_.at(0).GetId())) d.num_tokens = static_cast<int>(s->at(0));
    if (auto s = dyn.getShape(input_ids_.at(5).GetId())) d.num_seqs = static_cast<int>(s->at(0));
    if (d.num_tokens <= 0 || d.num_seqs <= 0) return;  // an empty step
    if (d.num_seqs > max_seqs_) ov::throw_ov_exception("PagedAttentionExtension: more sequences than the capacity");
    if (d.num_tokens > max_context_len_ + max_seqs_)
        ov::throw_ov_exception("PagedAttentionExtension: more tokens in one step than the capacity");
    d.max_context_len = max_context_len_;
    d.max_q_len = d.num_tokens == d.num_seqs ? 1 : d.num_tokens - d.num_seqs + 1;
    d.prefill_row_blocks = hint_row_blocks_;
    d.prefill_kv_tokens = hint_kv_tokens_;
    if (wb.mutable_buffers.size() < 2) ov::throw_ov_exception("PagedAttentionExtension: work buffers missing");
    auto stream = context.getThreadContext().stream().get();
    auto* status = static_cast<int32_t*>(wb.mutable_buffers[1].get());
    if (cudaMemsetAsync(status, 0, sizeof(int32_t), stream) != cudaSuccess)
        ov::throw_ov_exception("PagedAttentionExtension: cudaMemsetAsync failed");
    const auto* past_lens = static_cast<const int32_t*>(in[5].get());
    const auto* subseq = static_cast<const int32_t*>(in[6].get());
    const auto* bidx = static_cast<const int32_t*>(in[7].get());
    const auto* bbeg = static_cast<const int32_t*>(in[8].get());
    auto s = reinterpret_cast<b2a_stream_t>(stream);
    throwIfError(b2a_paged_kv_store(&d, in[1].get(), in[2].get(), in[3].as_mutable().get(), in[4].as_mutable().get(),
                                    past_lens, subseq, bidx, bbeg, status, s),
                 "b2a_paged_kv_store");
    throwIfError(b2a_paged_attention(&d, in[0].get(), in[3].get(), in[4].get(), past_lens, subseq, bidx, bbeg,
                                     out[0].get(), wb.mutable_buffers[0].get(), workspace_bytes_, status, s),
                 "b2a_paged_attention");
}

}  // namespace nvidia_gpu
}  // namespace ov

using ov::nvidia_gpu::PagedAttentionOp;
using ov::nvidia_gpu::SdpaOp;
OPERATION_REGISTER(SdpaOp, ScaledDotProductAttention)
OPERATION_REGISTER(PagedAttentionOp, PagedAttentionExtension)
