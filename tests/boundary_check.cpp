// Compiles include/warpdecode_b200.hpp without CUDA and calls every wrapper the way the reference's decoder calls
// the functions they stand in for (src/qwen38_forward.cuh: routed MoE, shared expert, finish; src/qwen38_runtime.cuh:
// load). The CUDA names are small stand-ins, as in the reference's own syntax check
// (tests/qwen38_cuda_syntax_check.sh). Linked against the built library by tests/test_host_cpu.py; main() only calls
// entry points that need no GPU.
#include <cstdio>
#include <cstring>

typedef struct stub_stream *cudaStream_t;      // stands in for cuda_runtime.h
struct __half { unsigned short v; };

#include "warpdecode_b200.hpp"

namespace ref {                                // stand-ins for the reference's types that the signatures mention
struct TensorInfo { const void *data = nullptr; int type = 21; long long dims[4] = {0, 0, 0, 0}; };
struct GpuMatrix { int rows = 0, cols = 0; };
struct GgufFile {};
struct Qwen38SharedExpertWeights {};
}  // namespace ref

// one layer of the decoder's MoE part, written like the reference's call site
static void moe_layer(wd_b200::Qwen38Runtime &rt, wd_b200::Qwen38MoeScratch &scratch, int layer, const float *x, float *out,
                      cudaStream_t stream) {
    ref::GpuMatrix router;
    ref::TensorInfo gate, up, down;
    ref::Qwen38SharedExpertWeights shared;
    wd_b200::run_qwen38_routed_moe_separate_f32_x(layer, x, router, gate, up, down, rt.expert_cache, scratch, out,
                                                  rt.layout.w_scale, stream);
    wd_b200::run_qwen38_shared_expert_f32_x(x, shared, scratch, stream);
    wd_b200::q38_finish_moe_f32(scratch, out, stream, [](float *, const float *, size_t, cudaStream_t) {});
    const std::vector<int> ids = scratch.h_ids();
    const std::vector<float> w = scratch.h_weights();
    (void)ids;
    (void)w;
}

int main(int argc, char **argv) {
    std::printf("abi %d default_cache_mib(183359) %lld\n", wd_version(), static_cast<long long>(wd_default_cache_mib(183359)));
    // an unreadable model must surface as the reference's kind of failure: std::runtime_error with a message
    try {
        ref::GgufFile g;
        wd_b200::Qwen38Runtime rt = wd_b200::load_qwen38_runtime(g, argc > 1 ? argv[1] : "/nonexistent.gguf", 100, 183359);
        wd_b200::Qwen38MoeScratch scratch;
        scratch.attach(rt.engine.get(), rt.layout.n_experts, rt.layout.top_k, rt.layout.hidden);
        scratch.initialize(rt.layout.n_experts, rt.layout.top_k, rt.layout.hidden, rt.layout.expert_ffn);
        ref::TensorInfo t;
        rt.expert_cache.initialize(static_cast<size_t>(rt.layout.cache_mib), t, t, t);
        (void)rt.expert_cache.acquire(0, 0, t, t, t, static_cast<cudaStream_t>(nullptr));
        moe_layer(rt, scratch, 0, nullptr, nullptr, nullptr);
    } catch (const std::runtime_error &e) {
        std::printf("runtime_error: %s\n", e.what());
        if (!std::strstr(e.what(), "warpdecode_b200")) return 2;
    }
    // the dense path's load_model / Runtime / run / output_hash, written like the reference's bench loop
    // (src/warodecode.cu:2706-2758); an unreadable file is the same kind of failure
    try {
        ref::GgufFile g;
        wd_b200::Model model = wd_b200::load_model(g, argc > 2 ? argv[2] : "/nonexistent-dense.gguf");
        wd_b200::Runtime rt(model, 128);
        const double seconds = rt.run(64, true, 1);
        std::printf("dense: %d layers, %.3f ms, hash %llx\n", model.layers, seconds * 1e3,
                    static_cast<unsigned long long>(rt.output_hash(64)));
    } catch (const std::runtime_error &e) {
        std::printf("runtime_error: %s\n", e.what());
        return std::strstr(e.what(), "warpdecode_b200") ? 0 : 3;
    }
    return 0;
}
