// Tests of the C++ host side, in the shape of the reference's unit tests
// (modules/nvidia_plugin/tests/unit/relu.cpp:36-94): build a node, create the operation through the registry,
// allocate device buffers, Execute on a ThreadContext's stream, download, compare with an inline CPU loop.
//
//   host_tests --cpu     registry and block-manager tests only (no device needed)
//   host_tests           everything (needs a GPU)
#include <cmath>
#include <cstdio>
#include <cstring>
#include <random>
#include <vector>

#include "attention_ops.hpp"
#include "host_pipeline.hpp"
#include "op_profiling.hpp"
#include "kv_block_manager.hpp"

using namespace ov::nvidia_gpu;

static int g_failed = 0, g_run = 0;
#define CHECK(cond)                                                          \
    do {                                                                     \
        if (!(cond)) {                                                       \
            std::printf("  CHECK failed %s:%d: %s\n", __FILE__, __LINE__, #cond); \
            ++g_failed;                                                      \
            return;                                                          \
        }                                                                    \
    } while (0)
#define RUN(fn)                          \
    do {                                 \
        ++g_run;                         \
        const int before = g_failed;     \
        std::printf("[ RUN  ] %s\n", #fn); \
        fn();                            \
        std::printf("[ %s ] %s\n", g_failed == before ? " OK " : "FAIL", #fn); \
    } while (0)
#define CUDA_OK(x) CHECK((x) == cudaSuccess)

namespace {

struct DummyNode : ov::Node {
    const ov::DiscreteTypeInfo& get_type_info() const override {
        static const ov::DiscreteTypeInfo info{"NoSuchOperation", "test"};
        return info;
    }
};

std::vector<TensorID> ids(std::initializer_list<unsigned> l) {
    std::vector<TensorID> v;
    for (auto i : l) v.emplace_back(i);
    return v;
}

void test_registry() {
    auto& reg = OperationRegistry::getInstance();
    auto sdpa = std::make_shared<ov::op::v13::ScaledDotProductAttention>(true);
    auto pa = std::make_shared<ov::op::PagedAttentionExtension>();
    CHECK(reg.hasOperation(sdpa));
    CHECK(reg.hasOperation(pa));
    CHECK(!reg.hasOperation(std::make_shared<DummyNode>()));
    bool threw = false;
    try {
        OperationRegistry::Register<SdpaOp> again{"ScaledDotProductAttention"};
    } catch (const std::runtime_error&) {
        threw = true;
    }
    CHECK(threw);  // duplicate registration
}

void test_block_manager() {
    b2a::KvBlockManager m(8, 16, 0);
    CHECK(m.add_sequence(1) && m.add_sequence(2) && !m.add_sequence(1));
    int64_t idv[2] = {1, 2};
    int32_t ql[2] = {17, 1};
    b2a::StepTables t;
    CHECK(m.schedule_step(idv, ql, 2, t) == B2A_OK);
    CHECK(t.past_lens[0] == 0 && t.subsequence_begins[2] == 18 && t.block_indices.size() == 3);
    CHECK(t.block_indices_begins[1] == 2 && t.max_context_len == 17 && t.max_q_len == 17);
    CHECK(m.free_blocks() == 5);
    int32_t big[2] = {16 * 6, 1};
    CHECK(m.schedule_step(idv, big, 2, t) == B2A_ERR_CAPACITY);
    CHECK(m.free_blocks() == 5 && m.sequence_len(1) == 17);
    int64_t unknown[1] = {9};
    CHECK(m.schedule_step(unknown, ql, 1, t) == B2A_ERR_NOT_FOUND);
    CHECK(m.free_sequence(1) && m.free_blocks() == 7 && !m.free_sequence(1));
}

std::shared_ptr<ov::op::PagedAttentionExtension> paged_node(int Hq, int Hkv, int D, int bs, int nblocks) {
    auto node = std::make_shared<ov::op::PagedAttentionExtension>();
    const auto z = [](int x) { return static_cast<size_t>(x); };
    node->add_input(ov::element::bf16, {0, z(Hq * D)});
    node->add_input(ov::element::bf16, {0, z(Hkv * D)});
    node->add_input(ov::element::bf16, {0, z(Hkv * D)});
    node->add_input(ov::element::u8, {z(nblocks), z(Hkv), z(bs), z(D + 4)});
    node->add_input(ov::element::u8, {z(nblocks), z(Hkv), z(bs), z(D + 4)});
    for (int i = 0; i < 4; ++i) node->add_input(ov::element::i32, {0});
    node->add_input(ov::element::f32, {});
    node->add_input(ov::element::i32, {});
    node->add_output(ov::element::bf16, {0, z(Hq * D)});
    return node;
}

// The work-buffer request must cover every step the capacity admits.  Walks the edges: every sequence count with
// the longest contexts, the largest token count, hints present, absent, too large - and compares the request with
// what the library asks for the descriptor Execute would launch.  No device needed.
void test_paged_op_capacity_edges() {
    CreationContext cc{CUDA::Device{0}, false, /*set_current=*/false};
    const int Hq = 32, Hkv = 8, D = 128, bs = 16;
    for (int reserve : {0, 4096}) {
        auto node = paged_node(Hq, Hkv, D, bs, 4096);
        node->get_rt_info()["b2a.max_seqs"] = 48;
        node->get_rt_info()["b2a.max_context_len"] = 8192;
        node->get_rt_info()["b2a.max_prefill_kv_tokens"] = reserve;
        auto base = OperationRegistry::getInstance().createOperation(cc, node, ids({0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10}), ids({11}));
        auto op = std::dynamic_pointer_cast<const PagedAttentionOp>(base);
        CHECK(op != nullptr);
        const size_t have = op->GetWorkBufferRequest().mutable_sizes.at(0);
        size_t largest = 0;
        for (int n = 1; n <= op->max_seqs(); ++n)
            for (int tokens : {n, n + 1, n + 127, n + 1000, op->max_step_tokens()})
                for (AttentionStepHints h : {AttentionStepHints{}, AttentionStepHints{1, 128}, AttentionStepHints{9, 4096},
                                             AttentionStepHints{1 << 20, 1 << 20}}) {
                    const b2a_paged_desc d = op->StepDesc(tokens, n, h);
                    CHECK(d.max_q_len == tokens - n + 1);
                    CHECK(d.prefill_kv_tokens <= reserve);                  // never beyond the reserve
                    CHECK(d.prefill_row_blocks <= tokens / 128 + n);        // a hint can only tighten
                    size_t need = 0;
                    CHECK(b2a_paged_workspace_bytes(&d, 0, &need) == B2A_OK);
                    CHECK(need <= have);
                    largest = std::max(largest, need);
                }
        std::printf("  reserve %d: request %zu bytes, largest step %zu bytes\n", reserve, have, largest);
        CHECK(largest * 2 > have);  // and the request is not wildly more than the worst step
        // beyond the capacity: refused, as an exception (how the plugin reports an unusable request)
        for (auto bad : {std::pair<int, int>{op->max_step_tokens() + 1, 4}, std::pair<int, int>{60, 49}, std::pair<int, int>{3, 4}}) {
            bool threw = false;
            try {
                op->StepDesc(bad.first, bad.second, {});
            } catch (const std::exception&) {
                threw = true;
            }
            CHECK(threw);
        }
    }
}

void test_sdpa_scale_operand() {
    CreationContext cc{CUDA::Device{0}, false, /*set_current=*/false};
    auto make = [](bool constant_scale) {
        auto node = std::make_shared<ov::op::v13::ScaledDotProductAttention>(false);
        for (int i = 0; i < 3; ++i) node->add_input(ov::element::f16, {1, 4, 64, 128});
        node->add_input(ov::element::f16, {0});  // "no mask"
        node->add_input(ov::element::f16, {});   // scale
        node->add_output(ov::element::f16, {1, 4, 64, 128});
        if (constant_scale) node->const_scale = 0.25f;
        return node;
    };
    auto op = std::dynamic_pointer_cast<SdpaOp>(
        OperationRegistry::getInstance().createOperation(cc, make(true), ids({0, 1, 2, 3, 4}), ids({5})));
    CHECK(op != nullptr && op->desc().scale == 0.25f && op->desc().mask_kind == B2A_MASK_NONE);
    bool threw = false;
    try {
        OperationRegistry::getInstance().createOperation(cc, make(false), ids({0, 1, 2, 3, 4}), ids({5}));
    } catch (const std::exception&) {
        threw = true;  // a scale that is only known at run time
    }
    CHECK(threw);
}

// ---- GPU tests ------------------------------------------------------------------------------------------

void cpu_sdpa(const std::vector<float>& q, const std::vector<float>& k, const std::vector<float>& v,
              std::vector<float>& o, int B, int Hq, int Hkv, int Sq, int Skv, int D, bool causal) {
    const float scale = 1.0f / std::sqrt(static_cast<float>(D));
    const int g = Hq / Hkv;
    std::vector<float> s(static_cast<size_t>(Skv));
    for (int b = 0; b < B; ++b)
        for (int h = 0; h < Hq; ++h)
            for (int i = 0; i < Sq; ++i) {
                const float* qr = &q[((static_cast<size_t>(b) * Hq + h) * Sq + i) * D];
                const int lim = causal ? std::min(Skv, i + 1) : Skv;
                float mx = -INFINITY;
                for (int j = 0; j < lim; ++j) {
                    const float* kr = &k[((static_cast<size_t>(b) * Hkv + h / g) * Skv + j) * D];
                    float acc = 0.f;
                    for (int d = 0; d < D; ++d) acc += qr[d] * kr[d];
                    s[static_cast<size_t>(j)] = acc * scale;
                    mx = std::max(mx, s[static_cast<size_t>(j)]);
                }
                float den = 0.f;
                for (int j = 0; j < lim; ++j) {
                    s[static_cast<size_t>(j)] = std::exp(s[static_cast<size_t>(j)] - mx);
                    den += s[static_cast<size_t>(j)];
                }
                float* orow = &o[((static_cast<size_t>(b) * Hq + h) * Sq + i) * D];
                for (int d = 0; d < D; ++d) {
                    float acc = 0.f;
                    for (int j = 0; j < lim; ++j)
                        acc += s[static_cast<size_t>(j)] * v[((static_cast<size_t>(b) * Hkv + h / g) * Skv + j) * D + d];
                    orow[d] = acc / den;
                }
            }
}

template <typename T>
struct DevBuf {
    T* p = nullptr;
    size_t n = 0;
    explicit DevBuf(size_t count) : n(count) { cudaMalloc(reinterpret_cast<void**>(&p), std::max<size_t>(count, 1) * sizeof(T)); }
    ~DevBuf() { cudaFree(p); }
    void up(const std::vector<T>& h, cudaStream_t s) { cudaMemcpyAsync(p, h.data(), n * sizeof(T), cudaMemcpyHostToDevice, s); }
    void down(std::vector<T>& h, cudaStream_t s) {
        h.resize(n);
        cudaMemcpyAsync(h.data(), p, n * sizeof(T), cudaMemcpyDeviceToHost, s);
    }
};

void run_sdpa_case(int B, int H, int S, int D, bool causal, bool capture) {
    CreationContext cc{CUDA::Device{0}, false};
    ThreadContext tc{CUDA::Device{0}};
    InferenceRequestContext ctx{tc};
    auto node = std::make_shared<ov::op::v13::ScaledDotProductAttention>(causal);
    const ov::Shape shp{static_cast<size_t>(B), static_cast<size_t>(H), static_cast<size_t>(S), static_cast<size_t>(D)};
    for (int i = 0; i < 3; ++i) node->add_input(ov::element::f32, shp);
    node->add_output(ov::element::f32, shp);
    auto op = OperationRegistry::getInstance().createOperation(cc, node, ids({0, 1, 2}), ids({3}));
    CHECK(op->GetTypeName() == "ScaledDotProductAttention");
    CHECK(op->GetCudaGraphCompatibility() == CudaGraphCompatibility::FULL);
    const size_t n = static_cast<size_t>(B) * H * S * D;
    std::mt19937 rng(7);
    std::normal_distribution<float> nd;
    std::vector<float> q(n), k(n), v(n), o(n), ref(n);
    for (auto* vec : {&q, &k, &v})
        for (auto& x : *vec) x = nd(rng);
    DevBuf<float> dq(n), dk(n), dv(n), dout(n);
    auto s = tc.stream().get();
    dq.up(q, s); dk.up(k, s); dv.up(v, s);
    std::vector<CUDA::DevicePointer<const void*>> in{CUDA::DevicePointer<const void*>{dq.p},
                                                     CUDA::DevicePointer<const void*>{dk.p},
                                                     CUDA::DevicePointer<const void*>{dv.p}};
    std::vector<CUDA::DevicePointer<void*>> out{CUDA::DevicePointer<void*>{dout.p}};
    Workbuffers wb;
    if (!capture) {
        op->Execute(ctx, {in.data(), in.size()}, {out.data(), out.size()}, wb);
    } else {
        // capture Execute, instantiate, launch (tests/unit/cuda_graph_compatibility.cpp:38-60)
        tc.stream().synchronize();
        cudaGraph_t graph{};
        cudaGraphExec_t exec{};
        CUDA_OK(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
        op->Capture(ctx, {in.data(), in.size()}, {out.data(), out.size()}, wb);
        CUDA_OK(cudaStreamEndCapture(s, &graph));
        CUDA_OK(cudaGraphInstantiate(&exec, graph, 0));
        CUDA_OK(cudaGraphLaunch(exec, s));
        CUDA_OK(cudaGraphLaunch(exec, s));
        cudaGraphExecDestroy(exec);
        cudaGraphDestroy(graph);
    }
    dout.down(o, s);
    tc.stream().synchronize();
    CUDA_OK(cudaGetLastError());
    cpu_sdpa(q, k, v, ref, B, H, H, S, S, D, causal);
    float worst = 0.f;
    for (size_t i = 0; i < n; ++i) worst = std::max(worst, std::fabs(o[i] - ref[i]));
    std::printf("  sdpa B%d H%d S%d D%d causal=%d capture=%d max|diff|=%g\n", B, H, S, D, causal, capture, worst);
    CHECK(worst < 2e-5f);
}

void test_sdpa_op() {
    // the shapes of the reference's functional test, f32
    for (bool causal : {false, true}) {
        run_sdpa_case(1, 1, 4, 8, causal, false);
        run_sdpa_case(1, 4, 16, 32, causal, false);
        run_sdpa_case(1, 8, 32, 64, causal, false);
    }
}

void test_sdpa_op_graph_capture() { run_sdpa_case(1, 8, 32, 64, true, true); }

void test_sdpa_op_rejects() {
    CreationContext cc{CUDA::Device{0}, false};
    auto node = std::make_shared<ov::op::v13::ScaledDotProductAttention>(false);
    node->add_input(ov::element::f32, {1, 6, 8, 64});
    node->add_input(ov::element::f32, {1, 4, 8, 64});
    node->add_input(ov::element::f32, {1, 4, 8, 64});
    node->add_output(ov::element::f32, {1, 6, 8, 64});
    bool threw = false;
    try {
        OperationRegistry::getInstance().createOperation(cc, node, ids({0, 1, 2}), ids({3}));
    } catch (const std::exception&) {
        threw = true;  // how is_operation_supported learns "no" (src/cuda_plugin.cpp:171-188)
    }
    CHECK(threw);
    bool oor = false;
    try {
        OperationRegistry::getInstance().createOperation(cc, std::make_shared<DummyNode>(), ids({}), ids({}));
    } catch (const std::out_of_range&) {
        oor = true;
    }
    CHECK(oor);
}

float h2f(uint16_t h) {
    const uint32_t sign = (h >> 15) & 1, exp = (h >> 10) & 31, man = h & 1023;
    float v;
    if (exp == 0) v = std::ldexp(static_cast<float>(man), -24);
    else if (exp == 31) v = man ? NAN : INFINITY;
    else v = std::ldexp(static_cast<float>(man | 1024), static_cast<int>(exp) - 25);
    return sign ? -v : v;
}
uint16_t f2h(float f) {  // round to nearest even; inputs here are small normal numbers
    uint32_t x;
    std::memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000;
    int32_t exp = static_cast<int32_t>((x >> 23) & 255) - 127 + 15;
    uint32_t man = x & 0x7FFFFF;
    if (exp <= 0) return static_cast<uint16_t>(sign);
    if (exp >= 31) return static_cast<uint16_t>(sign | 0x7C00);
    uint32_t h = (static_cast<uint32_t>(exp) << 10) | (man >> 13);
    const uint32_t rem = man & 0x1FFF;
    if (rem > 0x1000 || (rem == 0x1000 && (h & 1))) ++h;
    return static_cast<uint16_t>(sign | h);
}

// Two decode steps through PagedAttentionOp with tables from the KvBlockManager; the second step replays a
// captured graph.  The CPU side reads the pool the GPU wrote (bytes, f16 scale, f16 zero-point) and attends
// over the de-quantised rows.
void test_paged_op_decode_with_block_manager() {
    const int Hq = 8, Hkv = 2, D = 128, bs = 16, nseq = 3, nblocks = 64;
    const int chunk = bs * (D + 4);
    CreationContext cc{CUDA::Device{0}, false};
    ThreadContext tc{CUDA::Device{0}};
    InferenceRequestContext ctx{tc};
    auto s = tc.stream().get();
    auto node = std::make_shared<ov::op::PagedAttentionExtension>();
    node->add_input(ov::element::f16, {0, static_cast<size_t>(Hq * D)});
    node->add_input(ov::element::f16, {0, static_cast<size_t>(Hkv * D)});
    node->add_input(ov::element::f16, {0, static_cast<size_t>(Hkv * D)});
    node->add_input(ov::element::u8, {nblocks, Hkv, bs, D + 4});
    node->add_input(ov::element::u8, {nblocks, Hkv, bs, D + 4});
    node->add_input(ov::element::i32, {0});
    node->add_input(ov::element::i32, {0});
    node->add_input(ov::element::i32, {0});
    node->add_input(ov::element::i32, {0});
    node->add_input(ov::element::f32, {});
    node->add_input(ov::element::i32, {});
    node->add_output(ov::element::f16, {0, static_cast<size_t>(Hq * D)});
    // capacity: part of the compiled model, carried by the node (room to de-quantise prefill contexts once)
    node->get_rt_info()["b2a.max_seqs"] = 4;
    node->get_rt_info()["b2a.max_context_len"] = nblocks * bs / 2;
    node->get_rt_info()["b2a.max_prefill_kv_tokens"] = 512;
    auto base = OperationRegistry::getInstance().createOperation(cc, node, ids({0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10}), ids({11}));
    auto op = std::dynamic_pointer_cast<const PagedAttentionOp>(base);  // const: nothing about it changes from here on
    CHECK(op != nullptr);
    const auto req = op->GetWorkBufferRequest();
    CHECK(req.mutable_sizes.size() == 2);
    DevBuf<uint8_t> ws(req.mutable_sizes[0]), st(req.mutable_sizes[1]);
    Workbuffers wb;
    wb.mutable_buffers = {CUDA::DevicePointer<void*>{ws.p}, CUDA::DevicePointer<void*>{st.p}};

    DevBuf<uint8_t> kc(static_cast<size_t>(nblocks) * Hkv * chunk), vc(static_cast<size_t>(nblocks) * Hkv * chunk);
    CUDA_OK(cudaMemsetAsync(kc.p, 0xFF, kc.n, s));
    CUDA_OK(cudaMemsetAsync(vc.p, 0xFF, vc.n, s));

    b2a::KvBlockManager mgr(nblocks, bs, 99);
    const int64_t seq_ids[nseq] = {10, 11, 12};
    for (auto id : seq_ids) mgr.add_sequence(id);
    std::mt19937 rng(3);
    std::normal_distribution<float> nd;

    // step 0: prefill of 37 / 16 / 5 tokens (tensor-core kernel over contexts de-quantised once, by the scheduler's
    // hints); steps 1..2: one token each (decode kernel)
    const int32_t prefill[nseq] = {37, 16, 5};
    const int32_t one[nseq] = {1, 1, 1};
    const int max_tok = 64;
    DevBuf<uint16_t> dq(static_cast<size_t>(max_tok) * Hq * D), dk(static_cast<size_t>(max_tok) * Hkv * D),
        dv(static_cast<size_t>(max_tok) * Hkv * D), dout(static_cast<size_t>(max_tok) * Hq * D);
    DevBuf<int32_t> d_past(nseq), d_sb(nseq + 1), d_bi(nblocks), d_bb(nseq + 1);
    cudaGraphExec_t exec{};
    for (int step = 0; step < 3; ++step) {
        b2a::StepTables t;
        CHECK(mgr.schedule_step(seq_ids, step == 0 ? prefill : one, nseq, t) == B2A_OK);
        const int ntok = t.num_tokens;
        if (step == 0) CHECK(t.prefill_row_blocks == 3 && t.prefill_kv_tokens == 3 * 128);
        // what the scheduler knows about this step travels with the request; the last step passes nothing and is
        // sized by the capacity
        ctx.setAttentionStepHints(step < 2 ? AttentionStepHints{t.prefill_row_blocks, t.prefill_kv_tokens} : AttentionStepHints{});
        std::vector<uint16_t> q(static_cast<size_t>(max_tok) * Hq * D, 0), k(static_cast<size_t>(max_tok) * Hkv * D, 0),
            v(static_cast<size_t>(max_tok) * Hkv * D, 0);
        for (size_t i = 0; i < static_cast<size_t>(ntok) * Hq * D; ++i) q[i] = f2h(nd(rng));
        for (size_t i = 0; i < static_cast<size_t>(ntok) * Hkv * D; ++i) {
            k[i] = f2h(nd(rng));
            v[i] = f2h(nd(rng));
        }
        dq.up(q, s); dk.up(k, s); dv.up(v, s);
        std::vector<int32_t> bi(static_cast<size_t>(nblocks), 0);
        std::copy(t.block_indices.begin(), t.block_indices.end(), bi.begin());
        d_past.up(t.past_lens, s); d_sb.up(t.subsequence_begins, s); d_bi.up(bi, s); d_bb.up(t.block_indices_begins, s);
        ctx.getDynamicBufferContext().setShape(0, {static_cast<size_t>(ntok), static_cast<size_t>(Hq * D)});
        ctx.getDynamicBufferContext().setShape(5, {static_cast<size_t>(nseq)});
        std::vector<CUDA::DevicePointer<const void*>> in;
        for (const void* p : {static_cast<const void*>(dq.p), static_cast<const void*>(dk.p), static_cast<const void*>(dv.p),
                              static_cast<const void*>(kc.p), static_cast<const void*>(vc.p),
                              static_cast<const void*>(d_past.p), static_cast<const void*>(d_sb.p),
                              static_cast<const void*>(d_bi.p), static_cast<const void*>(d_bb.p),
                              static_cast<const void*>(st.p), static_cast<const void*>(st.p)})
            in.emplace_back(p);
        std::vector<CUDA::DevicePointer<void*>> out{CUDA::DevicePointer<void*>{dout.p}};
        if (step < 2) {
            op->Execute(ctx, {in.data(), in.size()}, {out.data(), out.size()}, wb);
            if (step == 1) {  // capture the decode step for replay
                tc.stream().synchronize();
                cudaGraph_t graph{};
                CUDA_OK(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
                op->Capture(ctx, {in.data(), in.size()}, {out.data(), out.size()}, wb);
                CUDA_OK(cudaStreamEndCapture(s, &graph));
                CUDA_OK(cudaGraphInstantiate(&exec, graph, 0));
                cudaGraphDestroy(graph);
            }
        } else {
            CUDA_OK(cudaGraphLaunch(exec, s));  // same buffers, new contents, lengths one longer
        }
        std::vector<uint16_t> o;
        std::vector<uint8_t> hk, hv;
        std::vector<uint8_t> status;
        dout.down(o, s); kc.down(hk, s); vc.down(hv, s); st.down(status, s);
        tc.stream().synchronize();
        CUDA_OK(cudaGetLastError());
        int32_t st_word;
        std::memcpy(&st_word, status.data(), 4);
        CHECK(st_word == 0);
        // CPU attention over the de-quantised pool
        float worst = 0.f;
        const float scale = 1.0f / std::sqrt(static_cast<float>(D));
        for (int sq = 0; sq < nseq; ++sq) {
            const int b0 = t.subsequence_begins[static_cast<size_t>(sq)], b1 = t.subsequence_begins[static_cast<size_t>(sq) + 1];
            for (int tk = b0; tk < b1; ++tk) {
                const int pos = t.past_lens[static_cast<size_t>(sq)] + (tk - b0);
                for (int h = 0; h < Hq; ++h) {
                    const int hk_i = h / (Hq / Hkv);
                    std::vector<float> sc(static_cast<size_t>(pos) + 1);
                    float mx = -INFINITY;
                    auto deq = [&](const std::vector<uint8_t>& pool, int p, int d) {
                        const int blk = t.block_indices[static_cast<size_t>(t.block_indices_begins[static_cast<size_t>(sq)] + p / bs)];
                        const uint8_t* c = &pool[(static_cast<size_t>(blk) * Hkv + hk_i) * chunk];
                        uint16_t sc16, zp16;
                        std::memcpy(&sc16, c + bs * D + 2 * (p % bs), 2);
                        std::memcpy(&zp16, c + bs * D + 2 * bs + 2 * (p % bs), 2);
                        return (static_cast<float>(c[(p % bs) * D + d]) - h2f(zp16)) * h2f(sc16);
                    };
                    for (int p = 0; p <= pos; ++p) {
                        float acc = 0.f;
                        for (int d = 0; d < D; ++d) acc += h2f(q[(static_cast<size_t>(tk) * Hq + h) * D + d]) * deq(hk, p, d);
                        sc[static_cast<size_t>(p)] = acc * scale;
                        mx = std::max(mx, sc[static_cast<size_t>(p)]);
                    }
                    float den = 0.f;
                    for (auto& x : sc) {
                        x = std::exp(x - mx);
                        den += x;
                    }
                    for (int d = 0; d < D; ++d) {
                        float acc = 0.f;
                        for (int p = 0; p <= pos; ++p) acc += sc[static_cast<size_t>(p)] * deq(hv, p, d);
                        const float got = h2f(o[(static_cast<size_t>(tk) * Hq + h) * D + d]);
                        worst = std::max(worst, std::fabs(got - acc / den));
                    }
                }
            }
        }
        std::printf("  paged step %d (%d tokens%s) max|diff|=%g\n", step, ntok, step == 2 ? ", graph replay" : "", worst);
        CHECK(worst < 2e-3f);
    }
    cudaGraphExecDestroy(exec);
}

// The per-operation timing hook: an event pair (and an NVTX range) around Execute, accumulated over calls the way
// the reference's profiler accumulates them (src/utils/perf_timing.hpp:24-40).
// The node's second output: scores of every sequence's last query token (b2a_paged_last_token_scores through the
// operator).  One mixed step (20-token prefill, 5-token prefill, then the same sequences with one token each); the
// scores must be non-negative, sum to Hq per sequence, and sit at the cumulative contexts.
void test_paged_op_score_output() {
    const int Hq = 8, Hkv = 2, D = 128, bs = 16, nseq = 2, nblocks = 32;
    const int chunk = bs * (D + 4);
    CreationContext cc{CUDA::Device{0}, false};
    ThreadContext tc{CUDA::Device{0}};
    InferenceRequestContext ctx{tc};
    auto s = tc.stream().get();
    auto node = std::make_shared<ov::op::PagedAttentionExtension>();
    node->add_input(ov::element::f16, {0, static_cast<size_t>(Hq * D)});
    node->add_input(ov::element::f16, {0, static_cast<size_t>(Hkv * D)});
    node->add_input(ov::element::f16, {0, static_cast<size_t>(Hkv * D)});
    node->add_input(ov::element::u8, {nblocks, Hkv, bs, D + 4});
    node->add_input(ov::element::u8, {nblocks, Hkv, bs, D + 4});
    for (int i = 0; i < 4; ++i) node->add_input(ov::element::i32, {0});
    node->add_input(ov::element::f32, {});
    node->add_input(ov::element::i32, {});
    node->add_output(ov::element::f16, {0, static_cast<size_t>(Hq * D)});
    node->add_output(ov::element::f32, {0});
    node->get_rt_info()["b2a.max_seqs"] = 4;
    node->get_rt_info()["b2a.max_context_len"] = 128;
    auto base = OperationRegistry::getInstance().createOperation(cc, node, ids({0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10}), ids({11, 12}));
    auto op = std::dynamic_pointer_cast<const PagedAttentionOp>(base);
    CHECK(op != nullptr && op->has_scores() && op->score_capacity() == 4 * 128);
    const auto req = op->GetWorkBufferRequest();
    CHECK(req.mutable_sizes.size() == 3);
    DevBuf<uint8_t> ws(req.mutable_sizes[0]), st(req.mutable_sizes[1]), sws(req.mutable_sizes[2]);
    Workbuffers wb;
    wb.mutable_buffers = {CUDA::DevicePointer<void*>{ws.p}, CUDA::DevicePointer<void*>{st.p}, CUDA::DevicePointer<void*>{sws.p}};
    DevBuf<uint8_t> kc(static_cast<size_t>(nblocks) * Hkv * chunk), vc(static_cast<size_t>(nblocks) * Hkv * chunk);
    CUDA_OK(cudaMemsetAsync(kc.p, 0, kc.n, s));
    CUDA_OK(cudaMemsetAsync(vc.p, 0, vc.n, s));
    b2a::KvBlockManager mgr(nblocks, bs, 7);
    const int64_t seq_ids[nseq] = {1, 2};
    for (auto id : seq_ids) mgr.add_sequence(id);
    std::mt19937 rng(11);
    std::normal_distribution<float> nd;
    const int max_tok = 32;
    DevBuf<uint16_t> dq(static_cast<size_t>(max_tok) * Hq * D), dk(static_cast<size_t>(max_tok) * Hkv * D),
        dv(static_cast<size_t>(max_tok) * Hkv * D), dout(static_cast<size_t>(max_tok) * Hq * D);
    DevBuf<float> dscores(static_cast<size_t>(op->score_capacity()));
    DevBuf<int32_t> d_past(nseq), d_sb(nseq + 1), d_bi(nblocks), d_bb(nseq + 1);
    const int32_t first[nseq] = {20, 5}, one[nseq] = {1, 1};
    for (int step = 0; step < 2; ++step) {
        b2a::StepTables t;
        CHECK(mgr.schedule_step(seq_ids, step == 0 ? first : one, nseq, t) == B2A_OK);
        const int ntok = t.num_tokens;
        std::vector<uint16_t> q(static_cast<size_t>(max_tok) * Hq * D, 0), k(static_cast<size_t>(max_tok) * Hkv * D, 0),
            v(static_cast<size_t>(max_tok) * Hkv * D, 0);
        for (size_t i = 0; i < static_cast<size_t>(ntok) * Hq * D; ++i) q[i] = f2h(nd(rng));
        for (size_t i = 0; i < static_cast<size_t>(ntok) * Hkv * D; ++i) {
            k[i] = f2h(nd(rng));
            v[i] = f2h(nd(rng));
        }
        dq.up(q, s); dk.up(k, s); dv.up(v, s);
        std::vector<int32_t> bi(static_cast<size_t>(nblocks), 0);
        std::copy(t.block_indices.begin(), t.block_indices.end(), bi.begin());
        d_past.up(t.past_lens, s); d_sb.up(t.subsequence_begins, s); d_bi.up(bi, s); d_bb.up(t.block_indices_begins, s);
        ctx.getDynamicBufferContext().setShape(0, {static_cast<size_t>(ntok), static_cast<size_t>(Hq * D)});
        ctx.getDynamicBufferContext().setShape(5, {static_cast<size_t>(nseq)});
        std::vector<CUDA::DevicePointer<const void*>> in;
        for (const void* p : {static_cast<const void*>(dq.p), static_cast<const void*>(dk.p), static_cast<const void*>(dv.p),
                              static_cast<const void*>(kc.p), static_cast<const void*>(vc.p),
                              static_cast<const void*>(d_past.p), static_cast<const void*>(d_sb.p),
                              static_cast<const void*>(d_bi.p), static_cast<const void*>(d_bb.p),
                              static_cast<const void*>(st.p), static_cast<const void*>(st.p)})
            in.emplace_back(p);
        std::vector<CUDA::DevicePointer<void*>> out{CUDA::DevicePointer<void*>{dout.p}, CUDA::DevicePointer<void*>{dscores.p}};
        op->Execute(ctx, {in.data(), in.size()}, {out.data(), out.size()}, wb);
        std::vector<float> sc;
        std::vector<uint8_t> status, tail;
        dscores.down(sc, s); st.down(status, s); sws.down(tail, s);
        tc.stream().synchronize();
        CUDA_OK(cudaGetLastError());
        int32_t st_word;
        std::memcpy(&st_word, status.data(), 4);
        CHECK(st_word == 0);
        int32_t begins[nseq + 1];
        std::memcpy(begins, tail.data() + op->score_begins_offset(), sizeof begins);
        int expect = 0;
        for (int sq = 0; sq < nseq; ++sq) {
            CHECK(begins[sq] == expect);
            const int ctxlen = t.past_lens[static_cast<size_t>(sq)] + (step == 0 ? first[sq] : 1);
            float sum = 0.f;
            for (int i = 0; i < ctxlen; ++i) {
                CHECK(sc[static_cast<size_t>(expect + i)] >= 0.f);
                sum += sc[static_cast<size_t>(expect + i)];
            }
            CHECK(std::fabs(sum - Hq) < 0.05f);
            expect += ctxlen;
        }
        CHECK(begins[nseq] == expect);
    }
}

void test_profiled_step() {
    CreationContext cc{CUDA::Device{0}, false};
    ThreadContext tc{CUDA::Device{0}};
    InferenceRequestContext ctx{tc};
    auto node = std::make_shared<ov::op::v13::ScaledDotProductAttention>(true);
    node->set_friendly_name("layer0/attention");
    const ov::Shape shp{1, 8, 512, 128};
    for (int i = 0; i < 3; ++i) node->add_input(ov::element::f16, shp);
    node->add_output(ov::element::f16, shp);
    auto op = OperationRegistry::getInstance().createOperation(cc, node, ids({0, 1, 2}), ids({3}));
    const size_t n = 8 * 512 * 128;
    DevBuf<uint16_t> dq(n), dk(n), dv(n), dout(n);
    auto s = tc.stream().get();
    CUDA_OK(cudaMemsetAsync(dq.p, 0, n * 2, s));
    CUDA_OK(cudaMemsetAsync(dk.p, 0, n * 2, s));
    CUDA_OK(cudaMemsetAsync(dv.p, 0, n * 2, s));
    std::vector<CUDA::DevicePointer<const void*>> in{CUDA::DevicePointer<const void*>{dq.p},
                                                     CUDA::DevicePointer<const void*>{dk.p},
                                                     CUDA::DevicePointer<const void*>{dv.p}};
    std::vector<CUDA::DevicePointer<void*>> out{CUDA::DevicePointer<void*>{dout.p}};
    Workbuffers wb;
    ProfiledStep step(*op);
    CHECK(step.label() == "ScaledDotProductAttention: layer0/attention");
    float total = 0.f;
    for (int i = 0; i < 3; ++i) {
        step.execute(ctx, {in.data(), in.size()}, {out.data(), out.size()}, wb);
        tc.stream().synchronize();
        const float now = step.measure();
        CHECK(now > total);  // every call adds its own device time
        total = now;
    }
    CHECK(step.calls() == 3 && step.measure() == total);  // nothing pending: the total stays
    std::printf("  %s: %u calls, %.3f ms on the device\n", step.label().c_str(), step.calls(), total);
}

// Host tensors in, host tensor out, through HostSdpaRunner (upload / SdpaOp::Execute / download per piece on three
// streams), against the CPU loop; two runs in a row (the second finds the device tensors in use by the first).
void test_host_pipeline() {
    const int B = 2, Hq = 4, Hkv = 2, S = 48, D = 64;
    HostSdpaRunner runner(B2A_F32, B, Hq, Hkv, S, S, D, /*causal=*/true, /*device=*/0, /*kv_heads_per_piece=*/1);
    CHECK(runner.pieces() == B * Hkv);
    const size_t nq = static_cast<size_t>(B) * Hq * S * D, nkv = static_cast<size_t>(B) * Hkv * S * D;
    float *q = nullptr, *k = nullptr, *v = nullptr, *o = nullptr;
    CUDA_OK(cudaMallocHost(reinterpret_cast<void**>(&q), nq * 4));
    CUDA_OK(cudaMallocHost(reinterpret_cast<void**>(&k), nkv * 4));
    CUDA_OK(cudaMallocHost(reinterpret_cast<void**>(&v), nkv * 4));
    CUDA_OK(cudaMallocHost(reinterpret_cast<void**>(&o), nq * 4));
    std::mt19937 rng(11);
    std::normal_distribution<float> nd;
    cudaStream_t s{};
    CUDA_OK(cudaStreamCreate(&s));
    for (int run = 0; run < 3; ++run) {  // plain calls, then the captured step (same host tensors, new contents)
        for (size_t i = 0; i < nq; ++i) q[i] = nd(rng);
        for (size_t i = 0; i < nkv; ++i) { k[i] = nd(rng); v[i] = nd(rng); }
        runner.Run(q, k, v, o, s);
        CUDA_OK(cudaStreamSynchronize(s));
        std::vector<float> qv(q, q + nq), kv(k, k + nkv), vv(v, v + nkv), ref(nq);
        cpu_sdpa(qv, kv, vv, ref, B, Hq, Hkv, S, S, D, true);
        float worst = 0.f;
        for (size_t i = 0; i < nq; ++i) worst = std::max(worst, std::fabs(o[i] - ref[i]));
        std::printf("  host pipeline run %d: %d pieces, graph %d, max|diff|=%g\n", run, runner.pieces(), runner.replaying(), worst);
        CHECK(worst < 2e-5f);
        CHECK(runner.replaying() == (run >= 1));
    }
    cudaStreamDestroy(s);
    cudaFreeHost(q); cudaFreeHost(k); cudaFreeHost(v); cudaFreeHost(o);
}

}  // namespace

int main(int argc, char** argv) {
    const bool cpu_only = argc > 1 && std::strcmp(argv[1], "--cpu") == 0;
    RUN(test_registry);
    RUN(test_block_manager);
    RUN(test_paged_op_capacity_edges);
    RUN(test_sdpa_scale_operand);
    if (!cpu_only) {
        int n = 0;
        if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) {
            std::printf("no CUDA device: GPU tests cannot run\n");
            return 2;
        }
        RUN(test_sdpa_op);
        RUN(test_sdpa_op_graph_capture);
        RUN(test_sdpa_op_rejects);
        RUN(test_paged_op_decode_with_block_manager);
        RUN(test_paged_op_score_output);
        RUN(test_host_pipeline);
        RUN(test_profiled_step);
    }
    std::printf("%d test(s), %d failed\n", g_run, g_failed);
    return g_failed ? 1 : 0;
}
