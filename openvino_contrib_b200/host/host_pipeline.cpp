#include "host_pipeline.hpp"

#include <new>
#include <string>

namespace ov {
namespace nvidia_gpu {
namespace {

void cuda_ok(cudaError_t e, const char* what) {
    if (e != cudaSuccess) ov::throw_ov_exception(std::string("HostSdpaRunner: ") + what + ": " + cudaGetErrorString(e));
}

ov::element::Type element_of(int dtype) {
    switch (dtype) {
        case B2A_F32: return ov::element::f32;
        case B2A_F16: return ov::element::f16;
        case B2A_BF16: return ov::element::bf16;
        default: ov::throw_ov_exception("HostSdpaRunner: unsupported precision");
    }
}

std::vector<TensorID> tensor_ids(unsigned first, unsigned n) {
    std::vector<TensorID> v;
    for (unsigned i = 0; i < n; ++i) v.emplace_back(first + i);
    return v;
}

}  // namespace

HostSdpaRunner::HostSdpaRunner(int dtype, int B, int Hq, int Hkv, int Sq, int Skv, int D, bool causal, int device,
                               int kv_heads_per_piece)
    : B_(B), Hq_(Hq), Hkv_(Hkv), Sq_(Sq), Skv_(Skv), D_(D), G_(Hkv > 0 ? Hq / Hkv : 0), hpp_(kv_heads_per_piece),
      esize_(element_of(dtype).size()), device_(device), thread_(device_), request_(thread_) {
    if (B <= 0 || Hq <= 0 || Hkv <= 0 || Sq <= 0 || Skv <= 0 || D <= 0 || Hq % Hkv != 0)
        ov::throw_ov_exception("HostSdpaRunner: bad dimensions");
    if (hpp_ <= 0) {  // smallest divisor of Hkv that makes a piece's upload at least 8 MB
        const size_t per_head = (static_cast<size_t>(G_) * Sq + 2 * static_cast<size_t>(Skv)) * D * esize_;
        for (hpp_ = 1; hpp_ < Hkv && (Hkv % hpp_ != 0 || hpp_ * per_head < (8u << 20)); ++hpp_) {
        }
    }
    if (Hkv % hpp_ != 0) ov::throw_ov_exception("HostSdpaRunner: KV heads per piece must divide the KV heads");
    // the operation for ONE piece, built the way the plugin builds any operation: a node, the registry
    auto node = std::make_shared<ov::op::v13::ScaledDotProductAttention>(causal);
    const auto et = element_of(dtype);
    const auto z = [](int x) { return static_cast<size_t>(x); };
    node->add_input(et, {1, z(G_ * hpp_), z(Sq), z(D)});
    node->add_input(et, {1, z(hpp_), z(Skv), z(D)});
    node->add_input(et, {1, z(hpp_), z(Skv), z(D)});
    node->add_output(et, {1, z(G_ * hpp_), z(Sq), z(D)});
    CreationContext cc{device_, false};
    op_ = OperationRegistry::getInstance().createOperation(cc, node, tensor_ids(0, 3), tensor_ids(3, 1));
    const auto req = op_->GetWorkBufferRequest();
    if (!req.mutable_sizes.empty()) {
        cuda_ok(cudaMalloc(&ws_, req.mutable_sizes[0]), "cudaMalloc");
        workbuffers_.mutable_buffers.emplace_back(ws_);
    }
    const size_t nq = z(B) * Hq * Sq * D * esize_, nkv = z(B) * Hkv * Skv * D * esize_;
    cuda_ok(cudaMalloc(&dq_, nq), "cudaMalloc");
    cuda_ok(cudaMalloc(&dk_, nkv), "cudaMalloc");
    cuda_ok(cudaMalloc(&dv_, nkv), "cudaMalloc");
    cuda_ok(cudaMalloc(&do_, nq), "cudaMalloc");
    cuda_ok(cudaStreamCreateWithFlags(&up_, cudaStreamNonBlocking), "cudaStreamCreate");
    cuda_ok(cudaStreamCreateWithFlags(&down_, cudaStreamNonBlocking), "cudaStreamCreate");
    cuda_ok(cudaStreamCreateWithFlags(&origin_, cudaStreamNonBlocking), "cudaStreamCreate");
    for (cudaEvent_t* e : {&begin_, &end_, &caller_in_, &caller_out_})
        cuda_ok(cudaEventCreateWithFlags(e, cudaEventDisableTiming), "cudaEventCreate");
    uploaded_.resize(z(pieces()));
    computed_.resize(z(pieces()));
    for (auto& e : uploaded_) cuda_ok(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "cudaEventCreate");
    for (auto& e : computed_) cuda_ok(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "cudaEventCreate");
}

HostSdpaRunner::~HostSdpaRunner() {
    cudaDeviceSynchronize();
    for (auto e : uploaded_) cudaEventDestroy(e);
    for (auto e : computed_) cudaEventDestroy(e);
    if (graph_exec_) cudaGraphExecDestroy(graph_exec_);
    for (cudaEvent_t e : {begin_, end_, caller_in_, caller_out_})
        if (e) cudaEventDestroy(e);
    for (cudaStream_t s : {up_, down_, origin_})
        if (s) cudaStreamDestroy(s);
    for (void* p : {dq_, dk_, dv_, do_, ws_})
        if (p) cudaFree(p);
}

size_t HostSdpaRunner::h2d_bytes() const {
    return (static_cast<size_t>(B_) * Hq_ * Sq_ + 2 * static_cast<size_t>(B_) * Hkv_ * Skv_) * D_ * esize_;
}
size_t HostSdpaRunner::d2h_bytes() const { return static_cast<size_t>(B_) * Hq_ * Sq_ * D_ * esize_; }

void HostSdpaRunner::Run(const void* q, const void* k, const void* v, void* out, cudaStream_t caller_stream) {
    if (q == nullptr || k == nullptr || v == nullptr || out == nullptr) ov::throw_ov_exception("HostSdpaRunner: null tensor");
    const void* now[4] = {q, k, v, out};
    const bool same = now[0] == last_[0] && now[1] == last_[1] && now[2] == last_[2] && now[3] == last_[3];
    if (!same && graph_exec_ != nullptr) {  // other tensors: the captured step is of no use any more
        cudaGraphExecDestroy(graph_exec_);
        graph_exec_ = nullptr;
    }
    if (same && graph_exec_ == nullptr && !capture_failed_) capture_failed_ = !Capture(q, k, v, out);
    for (int i = 0; i < 4; ++i) last_[i] = now[i];
    if (graph_exec_ == nullptr) {
        Enqueue(q, k, v, out, caller_stream);
        return;
    }
    // the captured step, between the caller's earlier work and its later work
    cuda_ok(cudaEventRecord(caller_in_, caller_stream), "cudaEventRecord");
    cuda_ok(cudaStreamWaitEvent(origin_, caller_in_, 0), "cudaStreamWaitEvent");
    cuda_ok(cudaGraphLaunch(graph_exec_, origin_), "cudaGraphLaunch");
    cuda_ok(cudaEventRecord(caller_out_, origin_), "cudaEventRecord");
    cuda_ok(cudaStreamWaitEvent(caller_stream, caller_out_, 0), "cudaStreamWaitEvent");
}

bool HostSdpaRunner::Capture(const void* q, const void* k, const void* v, void* out) {
    // thread-local mode: other threads of the process may go on using the runtime meanwhile
    if (cudaStreamBeginCapture(origin_, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
        (void)cudaGetLastError();
        return false;
    }
    cudaGraph_t graph = nullptr;
    bool ok = true;
    try {
        Enqueue(q, k, v, out, origin_);
    } catch (const std::exception&) {
        ok = false;
    }
    if (cudaStreamEndCapture(origin_, &graph) != cudaSuccess || graph == nullptr) ok = false;
    if (ok && cudaGraphInstantiate(&graph_exec_, graph, 0) != cudaSuccess) {
        graph_exec_ = nullptr;
        ok = false;
    }
    if (graph != nullptr) cudaGraphDestroy(graph);
    if (!ok) (void)cudaGetLastError();
    return ok;
}

void HostSdpaRunner::Enqueue(const void* q, const void* k, const void* v, void* out, cudaStream_t caller_stream) {
    cudaStream_t main = thread_.stream().get();
    // everything below comes after what the caller has enqueued (earlier users of the device tensors included)
    cuda_ok(cudaEventRecord(begin_, caller_stream), "cudaEventRecord");
    for (cudaStream_t s : {up_, main, down_}) cuda_ok(cudaStreamWaitEvent(s, begin_, 0), "cudaStreamWaitEvent");
    const size_t q_piece = static_cast<size_t>(G_) * hpp_ * Sq_ * D_ * esize_;   // rows of the query heads of the piece's KV heads
    const size_t kv_piece = static_cast<size_t>(hpp_) * Skv_ * D_ * esize_;
    auto at = [](const void* p, size_t off) { return static_cast<const char*>(p) + off; };
    auto at_m = [](void* p, size_t off) { return static_cast<char*>(p) + off; };
    for (int i = 0; i < pieces(); ++i) {
        const size_t qo = static_cast<size_t>(i) * q_piece, kvo = static_cast<size_t>(i) * kv_piece;
        // ParameterOp's part: host -> device, K and V first (the kernel's first loads), then the queries
        cuda_ok(cudaMemcpyAsync(at_m(dk_, kvo), at(k, kvo), kv_piece, cudaMemcpyHostToDevice, up_), "cudaMemcpyAsync");
        cuda_ok(cudaMemcpyAsync(at_m(dv_, kvo), at(v, kvo), kv_piece, cudaMemcpyHostToDevice, up_), "cudaMemcpyAsync");
        cuda_ok(cudaMemcpyAsync(at_m(dq_, qo), at(q, qo), q_piece, cudaMemcpyHostToDevice, up_), "cudaMemcpyAsync");
        cuda_ok(cudaEventRecord(uploaded_[static_cast<size_t>(i)], up_), "cudaEventRecord");
        cuda_ok(cudaStreamWaitEvent(main, uploaded_[static_cast<size_t>(i)], 0), "cudaStreamWaitEvent");
        const std::vector<CUDA::DevicePointer<const void*>> in{CUDA::DevicePointer<const void*>{at(dq_, qo)},
                                                               CUDA::DevicePointer<const void*>{at(dk_, kvo)},
                                                               CUDA::DevicePointer<const void*>{at(dv_, kvo)}};
        const std::vector<CUDA::DevicePointer<void*>> outs{CUDA::DevicePointer<void*>{at_m(do_, qo)}};
        op_->Execute(request_, {in.data(), in.size()}, {outs.data(), outs.size()}, workbuffers_);
        cuda_ok(cudaEventRecord(computed_[static_cast<size_t>(i)], main), "cudaEventRecord");
        // ResultOp's part: device -> host
        cuda_ok(cudaStreamWaitEvent(down_, computed_[static_cast<size_t>(i)], 0), "cudaStreamWaitEvent");
        cuda_ok(cudaMemcpyAsync(at_m(out, qo), at(do_, qo), q_piece, cudaMemcpyDeviceToHost, down_), "cudaMemcpyAsync");
    }
    cuda_ok(cudaEventRecord(end_, down_), "cudaEventRecord");
    cuda_ok(cudaStreamWaitEvent(caller_stream, end_, 0), "cudaStreamWaitEvent");
}

}  // namespace nvidia_gpu
}  // namespace ov

// ---- C ABI (declared in b2a.h) ----------------------------------------------------------------------------------
using ov::nvidia_gpu::HostSdpaRunner;

struct b2a_host_sdpa {
    std::unique_ptr<HostSdpaRunner> runner;
};

extern "C" {

int b2a_host_sdpa_create(int32_t dtype, int32_t B, int32_t Hq, int32_t Hkv, int32_t Sq, int32_t Skv, int32_t D,
                         int32_t causal, int32_t kv_heads_per_piece, b2a_host_sdpa** out) {
    if (out == nullptr) return B2A_ERR_NULL;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return B2A_ERR_CUDA;
    try {
        auto* h = new b2a_host_sdpa();
        h->runner = std::make_unique<HostSdpaRunner>(dtype, B, Hq, Hkv, Sq, Skv, D, causal != 0, dev, kv_heads_per_piece);
        *out = h;
        return B2A_OK;
    } catch (const std::bad_alloc&) {
        return B2A_ERR_CAPACITY;
    } catch (const std::exception&) {
        return B2A_ERR_UNSUPPORTED;
    }
}

int b2a_host_sdpa_run(b2a_host_sdpa* h, const void* q, const void* k, const void* v, void* out, b2a_stream_t stream) {
    if (h == nullptr || !h->runner) return B2A_ERR_NULL;
    try {
        h->runner->Run(q, k, v, out, reinterpret_cast<cudaStream_t>(stream));
        return B2A_OK;
    } catch (const std::exception&) {
        return B2A_ERR_CUDA;
    }
}

int b2a_host_sdpa_pieces(const b2a_host_sdpa* h) { return h != nullptr && h->runner ? h->runner->pieces() : 0; }

void b2a_host_sdpa_destroy(b2a_host_sdpa* h) { delete h; }

}  // extern "C"
