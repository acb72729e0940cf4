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

// integer entry of the node's run-time information, or `fallback`
int64_t rt_info_int(const ov::Node& node, const char* key, int64_t fallback) {
    const auto& rt = node.get_rt_info();
    const auto it = rt.find(key);
    if (it == rt.end()) return fallback;
#ifdef B2A_WITH_OPENVINO
    return it->second.as<int64_t>();
#else
    return it->second;
#endif
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
    if (n_in < 3 || n_in > 5) ov::throw_ov_exception("ScaledDotProductAttention: 3 to 5 inputs expected");
    if (n_in == 5 && !node.const_scale.has_value())
        ov::throw_ov_exception("ScaledDotProductAttention: the scale operand must be a Constant (a run-time scale "
                               "would need a synchronisation inside Execute)");
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
    if (n_in == 5) {
        desc_.scale = *node.const_scale;
        if (!(desc_.scale > 0.f)) ov::throw_ov_exception("ScaledDotProductAttention: scale must be positive");
    }
    desc_.mask_kind = B2A_MASK_NONE;
    // (an attention_mask operand of extent 0 means "no mask", as the op's specification has it)
    const bool mask_given = n_in >= 4 && !(node.get_input_shape(3).size() == 1 && node.get_input_shape(3)[0] == 0);
    if (mask_given && !node.get_causal()) {
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
    if (in.size() < (has_mask_ ? 4u : 3u) || out.size() != 1) ov::throw_ov_exception("ScaledDotProductAttention: operand count");
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
    if (!(desc_.scale >= 0.f) || desc_.sliding_window < 0)
        ov::throw_ov_exception("PagedAttentionExtension: scale / sliding_window out of range");
    desc_.num_tokens = static_cast<int>(qs[0]);  // 0 = dynamic: read per step
    desc_.num_seqs = static_cast<int>(node.get_input_shape(5).empty() ? 0 : node.get_input_shape(5)[0]);
    const int64_t pool_tokens = std::max<int64_t>(1, static_cast<int64_t>(desc_.num_blocks_total) * desc_.block_size);
    const int64_t ms = rt_info_int(node, "b2a.max_seqs", desc_.num_seqs > 0 ? desc_.num_seqs : 256);
    const int64_t mc = rt_info_int(node, "b2a.max_context_len", pool_tokens);
    const int64_t mp = rt_info_int(node, "b2a.max_prefill_kv_tokens", 0);
    const int64_t mt = rt_info_int(node, "b2a.max_step_tokens", mc + ms);
    if (ms <= 0 || ms > 65535 || mc <= 0 || mc > (1 << 30) || mp < 0 || mp > (1 << 30) || mt < ms || mt > (1 << 30))
        ov::throw_ov_exception("PagedAttentionExtension: bad capacity in the node's run-time information");
    max_seqs_ = static_cast<int>(ms);
    max_context_len_ = static_cast<int>(mc);
    max_step_tokens_ = static_cast<int>(mt);
    max_prefill_kv_tokens_ = static_cast<int>((mp + 127) / 128 * 128);
    workspace_bytes_ = WorkspaceBound();
    if (node.get_output_size() >= 2) {
        const int64_t cap = rt_info_int(node, "b2a.max_score_entries", ms * mc);
        if (cap <= 0) ov::throw_ov_exception("PagedAttentionExtension: bad b2a.max_score_entries");
        b2a_paged_desc d = desc_;
        d.max_context_len = max_context_len_;
        d.max_q_len = 1;
        size_t worst = 0;
        for (int n = 1; n <= max_seqs_; ++n) {  // (fewer sequences are cut into more chunks: not monotone)
            d.num_seqs = d.num_tokens = n;
            size_t bytes = 0;
            // (a configuration the score kernels do not take fails here, which query_model reads as "not supported")
            throwIfError(b2a_paged_scores_workspace_bytes(&d, 0, &bytes), "b2a_paged_scores_workspace_bytes");
            worst = std::max(worst, bytes);
        }
        score_capacity_ = cap;
        score_ws_bytes_ = (worst + 15) & ~static_cast<size_t>(15);
    }
}

b2a_paged_desc PagedAttentionOp::StepDesc(int num_tokens, int num_seqs, const AttentionStepHints& hints) const {
    if (num_seqs > max_seqs_) ov::throw_ov_exception("PagedAttentionExtension: more sequences than the capacity");
    if (num_tokens > max_step_tokens())
        ov::throw_ov_exception("PagedAttentionExtension: more tokens in one step than the capacity");
    if (num_tokens < num_seqs) ov::throw_ov_exception("PagedAttentionExtension: a scheduled sequence without a token");
    b2a_paged_desc d = desc_;
    d.num_tokens = num_tokens;
    d.num_seqs = num_seqs;
    d.max_context_len = max_context_len_;
    // every scheduled sequence has at least one token, so no sequence has more than this many
    d.max_q_len = num_tokens - num_seqs + 1;
    d.prefill_row_blocks = 0;
    d.prefill_kv_tokens = 0;
    // Execute launches the step's store directly before its attention: no other cache row changes in between
    d.cache_rows_settled = 1;
    if (d.max_q_len >= 2) {
        // The work list is reserved for the bound tokens/128 + sequences; a hint can only tighten it.  The scratch
        // of de-quantised contexts is reserved for max_prefill_kv_tokens; a step that says it needs more (or says
        // nothing when nothing is reserved) de-quantises inside the prefill kernel instead.
        const int32_t rb_bound = num_tokens / 128 + num_seqs;
        if (hints.prefill_row_blocks > 0 && hints.prefill_row_blocks <= rb_bound) d.prefill_row_blocks = hints.prefill_row_blocks;
        if (hints.prefill_kv_tokens > 0)
            d.prefill_kv_tokens = hints.prefill_kv_tokens <= max_prefill_kv_tokens_ ? hints.prefill_kv_tokens : 0;
        else
            d.prefill_kv_tokens = max_prefill_kv_tokens_;  // unknown: the whole reserve (the device lays it out)
    }
    return d;
}

size_t PagedAttentionOp::WorkspaceBound() const {
    // Largest request over every step the capacity admits.  The decode partials depend on the live sequence count
    // (the split plan does), so take the maximum over 1..max_seqs; the prefill work list and scratch are largest
    // for the largest token count, no hints (hints only tighten) and the whole scratch reserve.
    size_t worst = 16;
    for (int n = 1; n <= max_seqs_; ++n) {
        b2a_paged_desc d = desc_;
        d.num_seqs = n;
        d.num_tokens = max_step_tokens();
        d.max_context_len = max_context_len_;
        d.max_q_len = 2;
        d.prefill_row_blocks = 0;
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
    // [2] (nodes with a score output) scratch of the score kernels, then the sequences' offsets in the output
    if (has_scores()) r.mutable_sizes.push_back(score_ws_bytes_ + sizeof(int32_t) * (static_cast<size_t>(max_seqs_) + 1));
    return r;
}

void PagedAttentionOp::Execute(const InferenceRequestContext& context, Inputs in, Outputs out,
                               const Workbuffers& wb) const {
    if (in.size() < 11 || out.size() < 1) ov::throw_ov_exception("PagedAttentionExtension: operand count");
    // live extents: dynamic shapes recorded for this request win over the static ones
    int num_tokens = desc_.num_tokens, num_seqs = desc_.num_seqs;
    const auto& dyn = context.getDynamicBufferContext();
    if (auto s = dyn.getShape(input_ids_.at(0).GetId())) num_tokens = static_cast<int>(s->at(0));
    if (auto s = dyn.getShape(input_ids_.at(5).GetId())) num_seqs = static_cast<int>(s->at(0));
    if (num_tokens <= 0 || num_seqs <= 0) return;  // an empty step
    const b2a_paged_desc d = StepDesc(num_tokens, num_seqs, context.getAttentionStepHints());
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
    if (has_scores() && out.size() >= 2 && out[1].get() != nullptr) {
        if (wb.mutable_buffers.size() < 3) ov::throw_ov_exception("PagedAttentionExtension: score work buffer missing");
        // the score kernels split the longest admitted context the same way for every step, so the scratch reserved
        // at construction fits: the step's descriptor with the capacity's sequence count for the layout
        b2a_paged_desc sd = d;
        char* ws = static_cast<char*>(wb.mutable_buffers[2].get());
        size_t need = 0;
        throwIfError(b2a_paged_scores_workspace_bytes(&sd, 0, &need), "b2a_paged_scores_workspace_bytes");
        if (need > score_ws_bytes_) ov::throw_ov_exception("PagedAttentionExtension: score scratch too small");
        throwIfError(b2a_paged_last_token_scores(&sd, in[0].get(), in[3].get(), past_lens, subseq, bidx, bbeg,
                                                 static_cast<float*>(out[1].get()), score_capacity_,
                                                 reinterpret_cast<int32_t*>(ws + score_ws_bytes_), ws, score_ws_bytes_,
                                                 status, s),
                     "b2a_paged_last_token_scores");
    }
}

}  // namespace nvidia_gpu
}  // namespace ov

using ov::nvidia_gpu::PagedAttentionOp;
using ov::nvidia_gpu::SdpaOp;
OPERATION_REGISTER(SdpaOp, ScaledDotProductAttention)
OPERATION_REGISTER(PagedAttentionOp, PagedAttentionExtension)
