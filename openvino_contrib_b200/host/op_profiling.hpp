// Per-operation timing hook: an event pair and an NVTX range around one operation's Execute.
//
// The reference brackets every operation with CUDA events when profiling is enabled: Profiler::ProfileExecStep
// (modules/nvidia_plugin/src/cuda_profiler.hpp:127-160) wraps Execute / Capture / ExecuteGraph between
// PerformaceTiming::setStart and setStop (modules/nvidia_plugin/src/utils/perf_timing.hpp:24-40), and measure()
// accumulates the elapsed time of the pair once the stream has been synchronised.  ProfiledStep is that wrapper for
// the attention operations of this library, with one addition: the bracket is also an NVTX range named after the
// operation's type and node name, so a timeline tool shows which launches belong to which node.  As in the
// reference, timing an operation is for eager execution: events recorded inside a stream capture cannot be timed
// (the reference switches CUDA graphs off while profiling, modules/nvidia_plugin/src/cuda_compiled_model.cpp:61-62).
#pragma once

#include <nvtx3/nvToolsExt.h>

#include <string>
#include <utility>

#include "ov_shim.hpp"

namespace ov {
namespace nvidia_gpu {

class ProfiledStep {
public:
    explicit ProfiledStep(const OperationBase& op) : op_(op), label_(op.GetTypeName() + ": " + op.GetName()) {
        if (cudaEventCreate(&start_) != cudaSuccess || cudaEventCreate(&stop_) != cudaSuccess)
            ov::throw_ov_exception("ProfiledStep: cudaEventCreate failed");
    }
    ~ProfiledStep() {
        if (start_) cudaEventDestroy(start_);
        if (stop_) cudaEventDestroy(stop_);
    }
    ProfiledStep(const ProfiledStep&) = delete;
    ProfiledStep& operator=(const ProfiledStep&) = delete;

    // Execute between two events on the request's stream, inside an NVTX range.
    void execute(const InferenceRequestContext& context, IOperationExec::Inputs in, IOperationExec::Outputs out,
                 const Workbuffers& wb) {
        cudaStream_t stream = context.getThreadContext().stream().get();
        nvtxRangePushA(label_.c_str());
        const bool timed = cudaEventRecord(start_, stream) == cudaSuccess;
        try {
            op_.Execute(context, in, out, wb);
        } catch (...) {
            nvtxRangePop();
            throw;
        }
        pending_ = timed && cudaEventRecord(stop_, stream) == cudaSuccess;
        nvtxRangePop();
        ++calls_;
    }

    // Adds the last execute()'s elapsed milliseconds to the total (call after the stream has been synchronised;
    // PerformaceTiming::measure does the same) and returns the total.
    float measure() {
        if (pending_) {
            float ms = 0.f;
            if (cudaEventElapsedTime(&ms, start_, stop_) == cudaSuccess) duration_ms_ += ms;
            pending_ = false;
        }
        return duration_ms_;
    }
    float duration_ms() const noexcept { return duration_ms_; }
    unsigned calls() const noexcept { return calls_; }
    const std::string& label() const noexcept { return label_; }

private:
    const OperationBase& op_;
    std::string label_;
    cudaEvent_t start_ = nullptr, stop_ = nullptr;
    bool pending_ = false;
    float duration_ms_ = 0.f;
    unsigned calls_ = 0;
};

}  // namespace nvidia_gpu
}  // namespace ov
