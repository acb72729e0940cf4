// ScaledDotProductAttention for a model whose inputs and outputs live in HOST memory.
//
// In the reference plugin a host tensor reaches an operation through ParameterOp (one cudaMemcpyAsync host -> device,
// modules/nvidia_plugin/src/ops/parameter.cpp:24-33) and leaves it through ResultOp (device -> host,
// modules/nvidia_plugin/src/ops/result.cpp:28-43), all on the request's one stream: upload, compute and download
// run one after the other.  HostSdpaRunner keeps those three roles but cuts the problem into independent pieces -
// a few KV heads of one batch entry each: the K/V rows of those heads and the query/output rows of the heads that
// read them, all contiguous in [B, H, S, D] tensors - and runs the upload of piece i+1, SdpaOp::Execute on piece i and the
// download of piece i-1 at the same time on three streams.  Only the first piece's upload and the last piece's
// download are exposed; the step costs about the longer of the two copy directions.
//
// The operation is created once through the OperationRegistry for the shape of ONE piece ([1, h*G, Sq, D] queries,
// [1, h, Skv, D] keys/values for h KV heads per piece) and executed on every piece with the piece's device pointers.
//
// A step is a few hundred runtime calls (three uploads, a launch, a download and their events per piece), which on a
// busy host take longer than the GPU needs for them.  So, like the plugin's graph runner
// (modules/nvidia_plugin/src/cuda_graph_topology_runner.cpp:13-141, which captures Parameter and Result copies with
// the operations), the runner captures the whole step into a CUDA graph the second time it is called with the same
// four host tensors and replays that graph from then on: one launch per step.
#pragma once

#include <memory>
#include <vector>

#include "attention_ops.hpp"

namespace ov {
namespace nvidia_gpu {

class HostSdpaRunner {
public:
    // dtype: b2a_dtype of q, k, v, o (B2A_F32 / B2A_F16 / B2A_BF16).  Allocates the device tensors, three streams
    // and two events per piece; throws through ov::throw_ov_exception.
    // kv_heads_per_piece: KV heads (with their query heads) per piece; must divide Hkv; 0 = the default (pieces of
    // at least 8 MB of upload: copies much smaller than that do not reach the bus's bandwidth).
    HostSdpaRunner(int dtype, int B, int Hq, int Hkv, int Sq, int Skv, int D, bool causal, int device = 0,
                   int kv_heads_per_piece = 0);
    ~HostSdpaRunner();
    HostSdpaRunner(const HostSdpaRunner&) = delete;
    HostSdpaRunner& operator=(const HostSdpaRunner&) = delete;

    // Enqueue one inference: q [B,Hq,Sq,D], k/v [B,Hkv,Skv,D] and out [B,Hq,Sq,D] are HOST pointers (pinned memory,
    // or the copies serialise).  The work is ordered after what `caller_stream` holds at the call and `caller_stream`
    // is made to wait for the last download, so events recorded on it bracket the whole step; `out` is complete
    // when `caller_stream` has been synchronised.  Nothing here synchronises; the second call in a row with the same
    // four tensors also captures and instantiates the step's graph (a one-off host-side cost).
    void Run(const void* q, const void* k, const void* v, void* out, cudaStream_t caller_stream);
    int pieces() const { return B_ * (Hkv_ / hpp_); }
    bool replaying() const { return graph_exec_ != nullptr; }  // the last Run launched a captured graph
    size_t h2d_bytes() const;
    size_t d2h_bytes() const;

private:
    void Enqueue(const void* q, const void* k, const void* v, void* out, cudaStream_t origin);
    bool Capture(const void* q, const void* k, const void* v, void* out);
    int B_, Hq_, Hkv_, Sq_, Skv_, D_, G_, hpp_;  // hpp_: KV heads per piece
    size_t esize_;
    CUDA::Device device_;
    ThreadContext thread_;          // its stream runs the kernels
    InferenceRequestContext request_;
    OperationBase::Ptr op_;         // SdpaOp for one piece
    void *dq_ = nullptr, *dk_ = nullptr, *dv_ = nullptr, *do_ = nullptr, *ws_ = nullptr;
    Workbuffers workbuffers_;
    cudaStream_t up_ = nullptr, down_ = nullptr, origin_ = nullptr;  // origin_: where a captured step begins and ends
    cudaEvent_t begin_ = nullptr, end_ = nullptr, caller_in_ = nullptr, caller_out_ = nullptr;
    const void* last_[4] = {nullptr, nullptr, nullptr, nullptr};  // host tensors of the previous Run
    cudaGraphExec_t graph_exec_ = nullptr;                        // the step over last_, once captured
    bool capture_failed_ = false;
    std::vector<cudaEvent_t> uploaded_, computed_;
};

}  // namespace nvidia_gpu
}  // namespace ov
