// Stand-ins for the slice of OpenVINO and of the nvidia_plugin operation API that the attention operators touch.
//
// The attention operators (attention_ops.hpp) are written against the plugin's own interface:
//   IOperationExec / IOperationMeta / OperationBase   modules/nvidia_plugin/src/cuda_operation_base.hpp:33-149
//   OperationRegistry, OPERATION_REGISTER              modules/nvidia_plugin/src/cuda_operation_registry.hpp:48-143
//   CreationContext                                    modules/nvidia_plugin/src/cuda_creation_context.hpp:16-27
//   InferenceRequestContext::getThreadContext          modules/nvidia_plugin/src/cuda_inference_request_context.hpp:22-102
//     (+ one accessor the plugin's class has to gain: getAttentionStepHints, see AttentionStepHints below)
//   ThreadContext::stream                              modules/nvidia_plugin/src/cuda_thread_context.hpp:14-31
//   WorkbufferRequest / Workbuffers / WorkbufferIds    modules/nvidia_plugin/src/memory_manager/cuda_workbuffers.hpp:18-54
//   CUDA::DevicePointer                                modules/nvidia_plugin/src/cuda/device_pointers.hpp:21-43
// Inside the plugin those come from its headers and from the OpenVINO developer package; neither is available
// to a standalone build, so this header declares the same names with the same member signatures, reduced to what
// the two operators and their tests use.  Building with -DB2A_WITH_OPENVINO skips it and includes the real ones.
#pragma once

#ifdef B2A_WITH_OPENVINO
#include <cuda_operation_base.hpp>
#include <cuda_operation_registry.hpp>
#include <openvino/op/paged_attention.hpp>
#include <openvino/op/scaled_dot_product_attention.hpp>
#else

#include <cuda_runtime_api.h>

#include <cstddef>
#include <cstdint>
#include <functional>
#include <map>
#include <memory>
#include <optional>
#include <stdexcept>
#include <string>
#include <string_view>
#include <typeindex>
#include <unordered_map>
#include <vector>

namespace gsl {
template <typename T>
class span {
public:
    span() = default;
    span(T* p, std::size_t n) : p_(p), n_(n) {}
    template <typename C, typename = decltype(std::declval<C&>().data())>
    span(C& c) : p_(c.data()), n_(c.size()) {}
    T* data() const { return p_; }
    std::size_t size() const { return n_; }
    bool empty() const { return n_ == 0; }
    T& operator[](std::size_t i) const { return p_[i]; }
    T* begin() const { return p_; }
    T* end() const { return p_ + n_; }

private:
    T* p_ = nullptr;
    std::size_t n_ = 0;
};
}  // namespace gsl

namespace ov {

[[noreturn]] inline void throw_ov_exception(const std::string& msg) { throw std::runtime_error(msg); }

namespace element {
enum class Type_t { dynamic, boolean, u8, i32, i64, f16, bf16, f32 };
class Type {
public:
    constexpr Type(Type_t t = Type_t::dynamic) : t_(t) {}
    constexpr operator Type_t() const { return t_; }
    std::size_t size() const {
        switch (t_) {
            case Type_t::boolean:
            case Type_t::u8: return 1;
            case Type_t::f16:
            case Type_t::bf16: return 2;
            case Type_t::i32:
            case Type_t::f32: return 4;
            case Type_t::i64: return 8;
            default: return 0;
        }
    }
    bool operator==(const Type& o) const { return t_ == o.t_; }
    bool operator!=(const Type& o) const { return t_ != o.t_; }

private:
    Type_t t_;
};
constexpr Type dynamic{Type_t::dynamic}, boolean{Type_t::boolean}, u8{Type_t::u8}, i32{Type_t::i32},
    i64{Type_t::i64}, f16{Type_t::f16}, bf16{Type_t::bf16}, f32{Type_t::f32};
}  // namespace element

using Shape = std::vector<std::size_t>;

struct DiscreteTypeInfo {
    const char* name;
    const char* version_id;
};

// A graph node reduced to what operator constructors read: type name, friendly name, operand shapes and types.
class Node {
public:
    virtual ~Node() = default;
    virtual const DiscreteTypeInfo& get_type_info() const = 0;
    const std::string& get_friendly_name() const { return name_; }
    void set_friendly_name(const std::string& n) { name_ = n; }
    std::size_t get_input_size() const { return in_shapes_.size(); }
    std::size_t get_output_size() const { return out_shapes_.size(); }
    const Shape& get_input_shape(std::size_t i) const { return in_shapes_.at(i); }
    const Shape& get_output_shape(std::size_t i) const { return out_shapes_.at(i); }
    const element::Type& get_input_element_type(std::size_t i) const { return in_types_.at(i); }
    const element::Type& get_output_element_type(std::size_t i) const { return out_types_.at(i); }
    void add_input(const element::Type& t, const Shape& s) {
        in_types_.push_back(t);
        in_shapes_.push_back(s);
    }
    void add_output(const element::Type& t, const Shape& s) {
        out_types_.push_back(t);
        out_shapes_.push_back(s);
    }
    // Run-time information attached to the node by whoever built the model (ov::Node::get_rt_info; the real map
    // holds ov::Any values - the operators only read integers from it, through rt_info_int in attention_ops.cpp).
    using RTMap = std::map<std::string, int64_t>;
    RTMap& get_rt_info() { return rt_info_; }
    const RTMap& get_rt_info() const { return rt_info_; }

private:
    RTMap rt_info_;
    std::string name_;
    std::vector<Shape> in_shapes_, out_shapes_;
    std::vector<element::Type> in_types_, out_types_;
};

namespace op {
namespace v13 {
// inputs: query, key, value[, attention_mask[, scale]]; attribute: causal
class ScaledDotProductAttention : public Node {
public:
    explicit ScaledDotProductAttention(bool causal) : causal_(causal) {}
    const DiscreteTypeInfo& get_type_info() const override {
        static const DiscreteTypeInfo info{"ScaledDotProductAttention", "opset13"};
        return info;
    }
    bool get_causal() const { return causal_; }
    // Value of the scale operand (input 4) when its producer is a Constant, which is how exported models carry a
    // non-default scale; an operator reads it once, at construction.
    std::optional<float> const_scale;

private:
    bool causal_;
};
}  // namespace v13

// inputs 0..12 in the published order (query, key, value, key_cache, value_cache, past_lens, subsequence_begins,
// block_indices, block_indices_begins, scale, sliding_window, alibi_slopes, max_context_len)
class PagedAttentionExtension : public Node {
public:
    const DiscreteTypeInfo& get_type_info() const override {
        static const DiscreteTypeInfo info{"PagedAttentionExtension", "extension"};
        return info;
    }
    // Values of the scale (operand 9) and sliding_window (operand 10) operands when they are Constants, which is
    // how exported models carry them; an operator reads them once, at construction.
    std::optional<float> const_scale;
    std::optional<int> const_sliding_window;
};
}  // namespace op
}  // namespace ov

namespace CUDA {

template <typename T>
class DevicePointer {
public:
    explicit DevicePointer(T p) : p_(p) {
        if (p == nullptr) throw std::invalid_argument("DevicePointer: null");
    }
    T get() const noexcept { return p_; }
    template <typename U>
    DevicePointer<U> cast() const noexcept {
        return DevicePointer<U>{static_cast<U>(p_)};
    }
    auto as_mutable() const noexcept {
        using M = std::remove_const_t<std::remove_pointer_t<T>>*;
        return DevicePointer<M>{const_cast<M>(p_)};
    }

private:
    T p_;
};

class Device {
public:
    explicit Device(int id = 0) : id_(id) {}
    int id() const { return id_; }
    const Device& setCurrent() const {
        if (cudaSetDevice(id_) != cudaSuccess) ov::throw_ov_exception("cudaSetDevice failed");
        return *this;
    }

private:
    int id_;
};

class Stream {
public:
    Stream() {
        if (cudaStreamCreate(&s_) != cudaSuccess) ov::throw_ov_exception("cudaStreamCreate failed");
    }
    ~Stream() { cudaStreamDestroy(s_); }
    Stream(const Stream&) = delete;
    Stream& operator=(const Stream&) = delete;
    cudaStream_t get() const noexcept { return s_; }
    void synchronize() const {
        if (cudaStreamSynchronize(s_) != cudaSuccess) ov::throw_ov_exception("cudaStreamSynchronize failed");
    }

private:
    cudaStream_t s_{};
};

}  // namespace CUDA

namespace ov {
namespace nvidia_gpu {

using BufferID = unsigned;
class TensorID {
public:
    explicit TensorID(BufferID id) : id_(id) {}
    BufferID GetId() const { return id_; }

private:
    BufferID id_;
};

struct WorkbufferRequest {
    using size_in_bytes_t = std::size_t;
    std::vector<size_in_bytes_t> immutable_sizes;
    std::vector<size_in_bytes_t> mutable_sizes;
};
struct Workbuffers {
    using immutable_buffer = CUDA::DevicePointer<const void*>;
    using mutable_buffer = CUDA::DevicePointer<void*>;
    std::vector<immutable_buffer> immutable_buffers;
    std::vector<mutable_buffer> mutable_buffers;
};
struct WorkbufferIds {
    using vector_of_ids = std::vector<BufferID>;
    vector_of_ids immutableIds;
    vector_of_ids mutableIds;
};

class CreationContext {
public:
    // (set_current = false: the shim's own addition, for tests that build operations on a host without a GPU)
    explicit CreationContext(CUDA::Device d, bool opBenchOption, bool set_current = true)
        : device_(set_current ? d.setCurrent() : d), bench_(opBenchOption) {}
    CUDA::Device device() const { return device_; }
    bool opBenchOption() const noexcept { return bench_; }

private:
    CUDA::Device device_;
    bool bench_;
};

class ThreadContext {
public:
    explicit ThreadContext(CUDA::Device d) : device_(d.setCurrent()) {}
    CUDA::Device device() const { return device_; }
    const CUDA::Stream& stream() const noexcept { return stream_; }

private:
    CUDA::Device device_;
    CUDA::Stream stream_;
};

// Runtime extents of operands whose shape is dynamic at compile time (the plugin's DynamicBufferContext,
// modules/nvidia_plugin/src/cuda_dynamic_buffer_context.hpp:30-80, keyed by tensor id).
class DynamicBufferContext {
public:
    void setShape(BufferID id, Shape s) { shapes_[id] = std::move(s); }
    std::optional<Shape> getShape(BufferID id) const {
        auto it = shapes_.find(id);
        if (it == shapes_.end()) return std::nullopt;
        return it->second;
    }

private:
    std::map<BufferID, Shape> shapes_;
};

// What the scheduler that built a continuous-batching step knows about it and the device does not have to find out
// (b2a_paged_desc.prefill_row_blocks / prefill_kv_tokens; zeros = unknown).  It belongs to ONE inference request,
// like the dynamic shapes: operation objects are shared by concurrent requests and Execute is const, so per-step
// facts travel in the request context, never in the operation.
struct AttentionStepHints {
    int32_t prefill_row_blocks = 0;
    int32_t prefill_kv_tokens = 0;
};

class InferenceRequestContext {
public:
    explicit InferenceRequestContext(const ThreadContext& tc) : tc_(tc) {}
    const ThreadContext& getThreadContext() const noexcept { return tc_; }
    DynamicBufferContext& getDynamicBufferContext() { return dyn_; }
    const DynamicBufferContext& getDynamicBufferContext() const { return dyn_; }
    void setAttentionStepHints(const AttentionStepHints& h) { hints_ = h; }
    const AttentionStepHints& getAttentionStepHints() const noexcept { return hints_; }

private:
    const ThreadContext& tc_;
    DynamicBufferContext dyn_;
    AttentionStepHints hints_;
};

enum class CudaGraphCompatibility { NONE, FULL, SPECIAL };

class IOperationExec {
public:
    using Inputs = gsl::span<const CUDA::DevicePointer<const void*>>;
    using Outputs = gsl::span<const CUDA::DevicePointer<void*>>;
    using Buffers = std::vector<CUDA::DevicePointer<void*>>;
    enum class WorkbufferStatus { NoInitNeeded, InitNeeded };
    virtual ~IOperationExec() = default;
    virtual void Execute(const InferenceRequestContext& context, Inputs inputTensors, Outputs outputTensors,
                         const Workbuffers& workbuffers) const = 0;
    virtual CudaGraphCompatibility GetCudaGraphCompatibility() const = 0;
    virtual void Capture(InferenceRequestContext& context, Inputs inputTensors, Outputs outputTensors,
                         const Workbuffers& workbuffers) const = 0;
    virtual void ExecuteGraph(InferenceRequestContext& context, Inputs inputTensors, Outputs outputTensors,
                              const Workbuffers& workbuffers) const = 0;
    virtual void InitSharedImmutableWorkbuffers(const Buffers&) = 0;
    virtual WorkbufferRequest GetWorkBufferRequest() const = 0;
    virtual const WorkbufferIds& GetWorkbufferIds() const = 0;
    virtual WorkbufferStatus SetWorkbufferIds(WorkbufferIds&& workbufferIds) = 0;
};

class IOperationMeta {
public:
    struct Category {
        static constexpr std::string_view CUDA{"CUDA"};
    };
    virtual ~IOperationMeta() = default;
    virtual const std::string_view& GetCategory() const = 0;
    virtual const std::string& GetName() const = 0;
    virtual const std::string& GetTypeName() const = 0;
    virtual const ov::element::Type& GetRuntimePrecision() const = 0;
    virtual gsl::span<const TensorID> GetInputIds() const = 0;
    virtual gsl::span<const TensorID> GetOutputIds() const = 0;
};

class OperationBase : public IOperationExec, public IOperationMeta, public std::enable_shared_from_this<OperationBase> {
public:
    using Ptr = std::shared_ptr<OperationBase>;
    using IndexCollection = std::vector<TensorID>;
    OperationBase(const CreationContext&, const ov::Node& node, IndexCollection&& inputIds, IndexCollection&& outputIds)
        : node_name_(node.get_friendly_name()),
          type_name_(node.get_type_info().name),
          input_ids_(std::move(inputIds)),
          output_ids_(std::move(outputIds)) {
        if (node.get_output_size() > 0) runtime_precision_ = node.get_output_element_type(0);
    }
    CudaGraphCompatibility GetCudaGraphCompatibility() const final {
        return has_dynamic_buffer_ ? CudaGraphCompatibility::NONE : GetCudaGraphCompatibilityImpl();
    }
    virtual CudaGraphCompatibility GetCudaGraphCompatibilityImpl() const { return CudaGraphCompatibility::NONE; }
    void Capture(InferenceRequestContext& context, Inputs in, Outputs out, const Workbuffers& wb) const override {
        Execute(context, in, out, wb);
    }
    void ExecuteGraph(InferenceRequestContext&, Inputs, Outputs, const Workbuffers&) const override {}
    WorkbufferRequest GetWorkBufferRequest() const override { return {}; }
    void InitSharedImmutableWorkbuffers(const Buffers&) override {}
    const std::string_view& GetCategory() const override { return cuda_category_; }
    const std::string& GetName() const override { return node_name_; }
    const std::string& GetTypeName() const override { return type_name_; }
    const ov::element::Type& GetRuntimePrecision() const override { return runtime_precision_; }
    gsl::span<const TensorID> GetInputIds() const override { return {input_ids_.data(), input_ids_.size()}; }
    gsl::span<const TensorID> GetOutputIds() const override { return {output_ids_.data(), output_ids_.size()}; }
    const WorkbufferIds& GetWorkbufferIds() const override { return workbuffer_ids_; }
    WorkbufferStatus SetWorkbufferIds(WorkbufferIds&& ids) override {
        workbuffer_ids_ = ids;
        return workbuffer_ids_.immutableIds.empty() ? WorkbufferStatus::NoInitNeeded : WorkbufferStatus::InitNeeded;
    }

protected:
    std::string node_name_, type_name_;
    ov::element::Type runtime_precision_ = ov::element::dynamic;
    const IndexCollection input_ids_, output_ids_;
    WorkbufferIds workbuffer_ids_;
    bool has_dynamic_buffer_ = false;

private:
    static inline const std::string_view cuda_category_ = Category::CUDA;
};

// Name-keyed factory.  Same behaviour as the plugin's: a second registration of a name throws
// std::runtime_error, creating an unknown operation throws std::out_of_range.
class OperationRegistry final {
public:
    using IndexCollection = OperationBase::IndexCollection;
    using OperationBuilder = std::function<OperationBase::Ptr(const CreationContext&, const std::shared_ptr<ov::Node>&,
                                                              IndexCollection&&, IndexCollection&&)>;
    template <typename TOperation>
    class Register {
    public:
        explicit Register(const std::string& opName) {
            getInstance().registerOp(opName, [](const CreationContext& ctx, const std::shared_ptr<ov::Node>& node,
                                                IndexCollection&& in, IndexCollection&& out) -> OperationBase::Ptr {
                return std::make_shared<TOperation>(ctx, dynamic_cast<const typename TOperation::NodeOp&>(*node),
                                                    std::move(in), std::move(out));
            });
        }
    };
    static OperationRegistry& getInstance() {
        static OperationRegistry r;
        return r;
    }
    bool hasOperation(const std::shared_ptr<ov::Node>& node) const {
        return builders_.count(node->get_type_info().name) > 0;
    }
    OperationBase::Ptr createOperation(const CreationContext& ctx, const std::shared_ptr<ov::Node>& node,
                                       IndexCollection&& in, IndexCollection&& out) {
        return builders_.at(node->get_type_info().name)(ctx, node, std::move(in), std::move(out));
    }
    void registerOp(const std::string& opName, OperationBuilder&& b) {
        if (!builders_.try_emplace(opName, std::move(b)).second)
            throw std::runtime_error{"Operation " + opName + " is already registered !!"};
    }

private:
    std::unordered_map<std::string, OperationBuilder> builders_;
};

}  // namespace nvidia_gpu
}  // namespace ov

#define OPERATION_REGISTER(type, name)                                                                           \
    extern "C" {                                                                                                 \
    [[maybe_unused]] const ::ov::nvidia_gpu::OperationRegistry::Register<type> openvino_cuda_op_register_##name{ \
        #name};                                                                                                  \
    }

#endif  // B2A_WITH_OPENVINO
