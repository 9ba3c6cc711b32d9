// warpdecode_b200.hpp — the reference engine's C++ entry points for the MoE block, kept by name and
// argument list, over the C ABI of warpdecode_b200.h.
//
// The reference (one translation unit, namespace wd) calls its MoE path through inline C++ functions and
// classes; it has no C ABI. A maintainer who swaps that path for this library includes this header in
// place of the corresponding parts of src/qwen38_moe.cuh, src/expert_cache.cuh, src/qwen38_runtime.cuh and (the dense
// path at the end of this file) src/warodecode.cu:
// the functions below have the reference's names, parameter order and error behaviour (std::runtime_error
// carrying the library's message), and forward to the C ABI. Each one names the reference declaration it
// stands in for (paths inside the reference project).
//
// The reference's own types appear in these signatures (TensorInfo, GpuMatrix, ...). They enter as template
// parameters, so that this header compiles against the reference's definitions when it is included there, and
// against any stand-in with the same members elsewhere (tests/boundary_check.cpp does that without CUDA).
// What this library needs from them: TensorInfo::data (host pointer of the GGUF tensor); nothing from
// GpuMatrix (the engine keeps its own repacked router).
#ifndef WARPDECODE_B200_HPP
#define WARPDECODE_B200_HPP

#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

#include "warpdecode_b200.h"

namespace wd_b200 {

// Every failure of the C ABI becomes the exception the reference's callers expect
// (the reference throws std::runtime_error for every geometry, type and CUDA failure).
inline void check(int rc) {
    if (rc != WD_OK) throw std::runtime_error(std::string("warpdecode_b200: ") + wd_last_error());
}

// Owns one wd_engine (RAII, move-only like the reference's LowBitMatrix, src/lowbit.cuh:20-66).
class Engine {
public:
    Engine() = default;
    explicit Engine(const wd_config &cfg) { check(wd_engine_create(&cfg, &e_)); }
    Engine(const Engine &) = delete;
    Engine &operator=(const Engine &) = delete;
    Engine(Engine &&o) noexcept : e_(o.e_) { o.e_ = nullptr; }
    Engine &operator=(Engine &&o) noexcept {
        if (this != &o) {
            reset();
            e_ = o.e_;
            o.e_ = nullptr;
        }
        return *this;
    }
    ~Engine() { reset(); }
    void reset() {
        if (e_) wd_engine_destroy(e_);
        e_ = nullptr;
    }
    wd_engine *get() const { return e_; }
    explicit operator bool() const { return e_ != nullptr; }

private:
    wd_engine *e_ = nullptr;
};

// Stands in for wd::GpuExpertCache (src/expert_cache.cuh:2156-2536). The slot pool lives inside the engine;
// this object is the view of it that the reference's call sites hold.
class GpuExpertCache {
public:
    // What acquire() hands back: where the expert sits. The reference returns borrowed LowBitMatrix views
    // (ExpertDeviceWeights, owns = false) that stay valid until the slot is evicted; here the kernels index the
    // pool by slot themselves, so the slot number is all a caller can need.
    struct ExpertDeviceWeights {
        int slot = -1;
        bool owns = false;
    };

    void attach(wd_engine *e) { e_ = e; }

    // initialize(capacity_mib, sample tensors, ...) (src/expert_cache.cuh:2176): the pool was sized when the
    // engine was created (wd_config::cache_mib, same meaning as capacity_mib); this call checks that it holds at
    // least one selection, which is where the reference throws for a cache below one slot (:2207-2209).
    template <class TensorInfoT>
    void initialize(size_t capacity_mib, const TensorInfoT &, const TensorInfoT &, const TensorInfoT &, size_t = 0, size_t = 0,
                    size_t = 0) {
        if (!e_) throw std::runtime_error("expert cache is not attached to an engine");
        if (capacity_mib > 0 && slot_count() < 1) throw std::runtime_error("expert cache smaller than one slot");
    }

    // acquire(layer, expert, gate, up, down, stream) (src/expert_cache.cuh:2252)
    template <class TensorInfoT, class StreamT>
    ExpertDeviceWeights acquire(int layer, int expert, const TensorInfoT &, const TensorInfoT &, const TensorInfoT &, StreamT) {
        if (!e_) throw std::runtime_error("expert cache is not initialized");
        ExpertDeviceWeights w;
        check(wd_cache_acquire(e_, layer, expert, &w.slot));
        return w;
    }

    size_t slot_count() const { return e_ ? static_cast<size_t>(wd_cache_slot_count(e_)) : 0; }
    size_t slot_bytes() const { return e_ ? static_cast<size_t>(wd_cache_slot_bytes(e_)) : 0; }

private:
    wd_engine *e_ = nullptr;
};

// Stands in for wd::Qwen38MoeScratch (src/qwen38_moe.cuh:1701-2150) as far as callers read results from it after
// a forward call. The engine owns every buffer; the accessors copy the named result of the LAST forward call
// out (they synchronise, like the reference's h_ids()/h_weights() after its per-layer stream sync, :2363-2379).
class Qwen38MoeScratch {
public:
    void attach(wd_engine *e, int n_experts, int top_k, int hidden) {
        e_ = e;
        n_experts_ = n_experts;
        top_k_ = top_k;
        hidden_ = hidden;
    }
    // initialize(n_experts, k, hidden, expert_ffn) with the reference's limits (src/qwen38_moe.cuh:1709-1714)
    void initialize(int n_experts, int top_k, int hidden, int) {
        if (n_experts > 4096 || top_k > 16) throw std::runtime_error("Qwen3.8 MoE scratch: experts <= 4096, k <= 16");
        if (e_ && (n_experts != n_experts_ || top_k != top_k_ || hidden != hidden_))
            throw std::runtime_error("Qwen3.8 MoE scratch geometry differs from the engine's");
    }
    int hidden() const { return hidden_; }
    std::vector<int> h_ids() const { return tap<int>(WD_TAP_IDS, top_k_); }
    std::vector<float> h_weights() const { return tap<float>(WD_TAP_WEIGHTS, top_k_); }
    std::vector<float> logits() const { return tap<float>(WD_TAP_LOGITS, n_experts_); }
    std::vector<float> accum() const { return tap<float>(WD_TAP_ROUTED, hidden_); }         // d_accum(): the routed sum
    std::vector<float> shared_down() const { return tap<float>(WD_TAP_SHARED, hidden_); }   // down_f32()
    float shared_gate() const { return tap<float>(WD_TAP_SHARED_GATE, 1)[0]; }              // d_shared_gate()
    wd_engine *engine() const { return e_; }
    // where the fused block left its output until q38_finish_moe_f32 hands it on
    float *pending_out = nullptr;

private:
    template <class T>
    std::vector<T> tap(int which, int n) const {
        if (!e_) throw std::runtime_error("MoE scratch is not attached to an engine");
        std::vector<T> v(static_cast<size_t>(n));
        check(wd_read_tap(e_, which, -1, v.data(), v.size() * sizeof(T)));
        return v;
    }
    wd_engine *e_ = nullptr;
    int n_experts_ = 0, top_k_ = 0, hidden_ = 0;
};

// Stands in for the MoE part of wd::Qwen38Runtime (src/qwen38_runtime.cuh:27-65).
struct Qwen38Runtime {
    wd_config layout{};
    Engine engine;
    GpuExpertCache expert_cache;
    size_t expert_cache_slots = 0;
    wd_gguf *file = nullptr;       // the mapped GGUF: must outlive the engine, as the reference's GgufFile must
    Qwen38Runtime() = default;
    Qwen38Runtime(Qwen38Runtime &&o) noexcept { *this = std::move(o); }
    Qwen38Runtime &operator=(Qwen38Runtime &&o) noexcept {
        if (this != &o) {
            release();
            layout = o.layout;
            engine = std::move(o.engine);
            expert_cache = o.expert_cache;
            expert_cache_slots = o.expert_cache_slots;
            file = o.file;
            o.file = nullptr;
        }
        return *this;
    }
    ~Qwen38Runtime() { release(); }

private:
    void release() {
        engine.reset();
        if (file) wd_gguf_close(file);
        file = nullptr;
    }
};

// load_qwen38_runtime(g, model_path, sm, memory_mib) (src/qwen38_runtime.cuh:117): geometry from the file's
// qwen4exp.* keys, cache sized like qwen38_tuning_for_gpu (0.75 * memory - 8 GiB, clamped, or
// WARODECODE_EXPERT_CACHE_MIB; src/qwen38_tuning.hpp:88-116), every layer's router, shared expert and experts
// loaded. The GgufFile argument is accepted for the signature; the library maps the file itself.
template <class GgufFileT>
inline Qwen38Runtime load_qwen38_runtime(const GgufFileT &, const std::string &model_path, int sm, int memory_mib) {
    if (sm < 100) throw std::runtime_error("warpdecode_b200 is built for sm_100a only");
    Qwen38Runtime rt;
    check(wd_gguf_open(model_path.c_str(), &rt.file));
    rt.layout.ep_size = 1;
    rt.layout.max_tokens = 4;
    check(wd_gguf_config(rt.file, &rt.layout));
    rt.layout.cache_mib = wd_default_cache_mib(memory_mib);
    rt.engine = Engine(rt.layout);
    check(wd_engine_load_gguf(rt.engine.get(), rt.file));
    rt.expert_cache.attach(rt.engine.get());
    rt.expert_cache_slots = rt.expert_cache.slot_count();
    return rt;
}

// run_qwen38_routed_moe_separate_f32_x<Capture>(layer, x, router, gate_exps, up_exps, down_exps, cache, scratch,
// out, expert_scale, stream, preselected, trace) (src/qwen38_moe.cuh:3761-3779). Here ONE kernel launch computes
// the whole block (selection, routed experts, shared expert, finish); the routed sum the reference leaves in
// scratch.d_accum() is scratch.accum(), and `out` receives the finished block output already (the reference's
// callers overwrite it again through q38_finish_moe_f32, which is then a no-op). expert_scale must be the
// engine's w_scale; a preselected run and the F16 trace have no counterpart and are refused.
template <bool CaptureSelectedOutput = false, class GpuMatrixT, class TensorInfoT, class CacheT, class StreamT, class HalfT = void>
inline void run_qwen38_routed_moe_separate_f32_x(int layer, const float *x, const GpuMatrixT &, const TensorInfoT &, const TensorInfoT &,
                                                 const TensorInfoT &, CacheT &, Qwen38MoeScratch &scratch, float *out,
                                                 float expert_scale, StreamT stream, bool preselected = false,
                                                 HalfT *selected_output_trace = nullptr) {
    static_assert(!CaptureSelectedOutput, "the selected-output trace is not produced by this library");
    if (preselected || selected_output_trace != nullptr)
        throw std::runtime_error("warpdecode_b200: preselected experts and the selected-output trace are not supported");
    (void)expert_scale;
    check(wd_moe_forward(scratch.engine(), layer, x, out, 1, reinterpret_cast<void *>(stream)));
    scratch.pending_out = out;
}

// run_qwen38_shared_expert_f32_x(x, shared, scratch, stream) (src/qwen38_moe.cuh:3963): the shared expert ran inside
// the fused block; nothing is left to do.
template <class SharedWeightsT, class StreamT>
inline void run_qwen38_shared_expert_f32_x(const float *, const SharedWeightsT &, Qwen38MoeScratch &, StreamT) {}

// q38_finish_moe_f32(scratch, out, stream) (src/qwen38_moe.cuh:2442): out = routed + shared * gate. The fused block
// wrote exactly that into the `out` of the routed call; a different destination gets a device copy.
template <class StreamT, class CopyFn>
inline void q38_finish_moe_f32(Qwen38MoeScratch &scratch, float *out, StreamT stream, CopyFn device_copy) {
    if (scratch.pending_out == nullptr) throw std::runtime_error("q38_finish_moe_f32 without a routed MoE run");
    if (out != scratch.pending_out) device_copy(out, scratch.pending_out, static_cast<size_t>(scratch.hidden()) * sizeof(float), stream);
    scratch.pending_out = nullptr;
}

// ---- the dense (Llama-style Q4_0) path: Model / load_model / Runtime of src/warodecode.cu:1211-2150 -------------------

// Stands in for Model (src/warodecode.cu:1211-1248) as far as callers read it: the geometry. The tensors live in the
// decoder that Runtime builds, because this library sizes the KV cache when the decoder is created.
struct Model {
    std::string path;
    std::string arch;
    int hidden = 0, layers = 0, heads = 0, kv_heads = 0, head_dim = 0, ffn = 0, vocab = 0;
};

// load_model(const GgufFile &) (src/warodecode.cu:1255): here the file is named, the library maps it itself. The
// geometry is read at once (a file the dense path cannot run throws here, as in the reference); the weights are
// uploaded by Runtime.
template <class GgufFileT>
inline Model load_model(const GgufFileT &, const std::string &model_path, int device = 0) {
    Model m;
    m.path = model_path;
    wd_gguf *file = nullptr;
    check(wd_gguf_open(model_path.c_str(), &file));
    wd_dense_decoder *probe = nullptr;
    const int rc = wd_dense_decoder_load_gguf(file, /*max_ctx=*/32, device, &probe);
    wd_gguf_close(file);
    check(rc);
    wd_dense_config c{};
    check(wd_dense_decoder_config(probe, &c));
    wd_dense_decoder_destroy(probe);
    m.hidden = c.hidden; m.layers = c.n_layers; m.heads = c.n_heads; m.kv_heads = c.n_kv_heads; m.head_dim = c.head_dim;
    m.ffn = c.ffn; m.vocab = c.vocab;
    return m;
}

// Stands in for Runtime (src/warodecode.cu:2011-2150): Runtime(model, ctx), run(steps, use_graph, start_token) returning
// seconds, output_hash(steps) over the generated tokens (FNV-1a over their little-endian bytes, :2138-2147). One
// CUDA-graph replay per token either way; `use_graph` is accepted for the signature.
class Runtime {
public:
    Runtime(Model &model, int ctx, int device = 0) : max_ctx(ctx) {
        wd_gguf *file = nullptr;
        check(wd_gguf_open(model.path.c_str(), &file));
        const int rc = wd_dense_decoder_load_gguf(file, ctx, device, &d_);
        wd_gguf_close(file);
        check(rc);
    }
    Runtime(const Runtime &) = delete;
    Runtime &operator=(const Runtime &) = delete;
    ~Runtime() {
        if (d_) wd_dense_decoder_destroy(d_);
    }
    double run(int steps, bool /*use_graph*/, int start_token) {
        if (steps < 1 || steps + 1 > max_ctx) throw std::runtime_error("warpdecode_b200: steps must fit the context");
        tokens_.assign(static_cast<size_t>(steps) + 1, 0);
        float ms = 0.0f;
        check(wd_dense_decoder_decode(d_, &start_token, 1, steps, tokens_.data(), &ms));
        return static_cast<double>(ms) / 1000.0;
    }
    uint64_t output_hash(int steps) const {
        uint64_t h = 1469598103934665603ull;
        for (int i = 1; i <= steps && i < static_cast<int>(tokens_.size()); ++i) {
            const uint32_t x = static_cast<uint32_t>(tokens_[static_cast<size_t>(i)]);
            for (int b = 0; b < 4; ++b) {
                h ^= static_cast<uint8_t>(x >> (8 * b));
                h *= 1099511628211ull;
            }
        }
        return h;
    }
    const std::vector<int> &tokens() const { return tokens_; }      // the start token, then the generated ones
    int max_ctx = 0;

private:
    wd_dense_decoder *d_ = nullptr;
    std::vector<int> tokens_;
};

}  // namespace wd_b200

#endif
