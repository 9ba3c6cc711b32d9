// C-ABI shim over the reference project's own host MoE code (TEST INFRASTRUCTURE ONLY).
//
// This file contains no arithmetic of its own: it includes the reference's headers
// from where they lie (passed with -I by oracle/build_ref.sh) and forwards to them,
// so that tests can pin oracle/wd_oracle.c against the real thing and the bench can
// time the reference's CPU path. The built library lands in oracle/_ref/ and is never
// committed.
//
// Forwarded code: src/qwen38_cpu_moe.cuh (quantisers :220/:239, row dots :298-440 and
// :565-758, ggml exp/silu/sigmoid :816-842, dot_f32_avx2 :847, ThreadPool :877) and the
// router block of src/qwen38_moe.cuh (:693-831), extracted the way the reference's own
// tests/qwen38_router_host_check.sh:67-156 extracts it.
//
// The one composition written here, ref_moe_block(), runs those functions in the order
// the reference engine does (router -> selected experts -> ordered combine -> shared
// expert -> finish) with the reference's task split (one task per selected expert for
// gate/up, k * slices row ranges for down; src/qwen38_cpu_moe.cuh:1245-1291). The tasks run
// on the small pool below rather than on cpu_moe::ThreadPool: back-to-back parallel_for calls
// on that pool can lose a task index to a worker still draining the previous call (its
// index counter is shared between calls), which left this shim waiting forever. It differs from cpu_moe::run_layer in one place:
// the activation fed to the down projection is quantised with the quantiser ggml pairs
// with the down tensor's type (Q8_K for IQ2_S/IQ3_S, Q8_0 otherwise), because
// run_layer hard-wires Q8_0 for its IQ4_NL down tensors.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <memory>
#include <vector>

static inline float  __fadd_rn(float a, float b)   { return a + b; }
static inline float  __fsub_rn(float a, float b)   { return a - b; }
static inline float  __fmul_rn(float a, float b)   { return a * b; }
static inline float  __fdiv_rn(float a, float b)   { return a / b; }
static inline float  __fmaf_rn(float a, float b, float c) { return std::fma(a, b, c); }
static inline double __dadd_rn(double a, double b) { return a + b; }
static inline double __dsub_rn(double a, double b) { return a - b; }
static inline double __dmul_rn(double a, double b) { return a * b; }
static inline uint32_t __float_as_uint(float x) { uint32_t r; std::memcpy(&r, &x, 4); return r; }
static inline float __uint_as_float(uint32_t x) { float r; std::memcpy(&r, &x, 4); return r; }
static inline uint64_t __double_as_longlong(double x) { uint64_t r; std::memcpy(&r, &x, 8); return r; }
static inline double __longlong_as_double(uint64_t x) { double r; std::memcpy(&r, &x, 8); return r; }

#include "qwen38_cpu_moe.cuh"
#include "wd_ref_router_extract.h"   // generated into oracle/_ref by build_ref.sh

namespace cm = wd::cpu_moe;

// src/ggml_dequant.hpp is host code that asks its includer for __half / __float2half when there is no CUDA compiler
// (as tests/gemv_kquant_dequant_host_test.cpp of the reference does); the conversion is the reference's own.
struct __half { unsigned short bits; };
static inline __half __float2half(float v) { return __half{cm::f32_to_f16_bits(v)}; }
#include "ggml_dequant.hpp"

#include <atomic>
#include <condition_variable>
#include <functional>
#include <mutex>
#include <thread>

namespace {

// Fork-join pool. Each call owns its own Job object, so a worker that is late leaving one
// call can never take an index of the next.
class Pool {
public:
    explicit Pool(int threads) : threads_(std::max(1, threads)) {
        for (int i = 1; i < threads_; ++i) workers_.emplace_back([this] { loop(); });
    }
    ~Pool() {
        { std::lock_guard<std::mutex> l(m_); stop_ = true; }
        cv_.notify_all();
        for (auto & t : workers_) t.join();
    }
    int threads() const { return threads_; }
    void parallel_for(int count, const std::function<void(int)> & fn) {
        if (count <= 0) return;
        if (count == 1 || threads_ == 1) { for (int i = 0; i < count; ++i) fn(i); return; }
        auto job = std::make_shared<Job>();
        job->fn = &fn; job->count = count;
        { std::lock_guard<std::mutex> l(m_); job_ = job; ++gen_; }
        cv_.notify_all();
        run(*job);
        std::unique_lock<std::mutex> l(m_);
        done_.wait(l, [&] { return job->finished.load() == count; });
        job_.reset();
    }
private:
    struct Job { const std::function<void(int)> * fn; int count; std::atomic<int> next{0}, finished{0}; };
    void run(Job & j) {
        for (;;) {
            const int i = j.next.fetch_add(1);
            if (i >= j.count) return;
            (*j.fn)(i);
            if (j.finished.fetch_add(1) + 1 == j.count) { std::lock_guard<std::mutex> l(m_); done_.notify_all(); }
        }
    }
    void loop() {
        uint64_t seen = 0;
        for (;;) {
            std::shared_ptr<Job> j;
            {
                std::unique_lock<std::mutex> l(m_);
                cv_.wait(l, [&] { return stop_ || gen_ != seen; });
                if (stop_) return;
                seen = gen_; j = job_;
            }
            if (j) run(*j);
        }
    }
    int threads_;
    std::vector<std::thread> workers_;
    std::mutex m_;
    std::condition_variable cv_, done_;
    std::shared_ptr<Job> job_;
    uint64_t gen_ = 0;
    bool stop_ = false;
};

// Packed Q8_K as wd_oracle.h declares it: 292 bytes, no padding.
struct PackedQ8K {
    float d;
    int8_t qs[256];
    int16_t bsums[16];
};
static_assert(sizeof(PackedQ8K) == 292, "packed Q8_K layout");

std::vector<cm::q8_K> unpack_q8k(const void * packed, int n) {
    std::vector<cm::q8_K> out(static_cast<size_t>(n));
    const PackedQ8K * p = static_cast<const PackedQ8K *>(packed);
    for (int i = 0; i < n; ++i) {
        out[i].d = p[i].d;
        std::memcpy(out[i].qs, p[i].qs, 256);
        std::memcpy(out[i].bsums, p[i].bsums, 32);
    }
    return out;
}

bool uses_q8k(int ggml_type) { return ggml_type == 21 || ggml_type == 22; }

}  // namespace

extern "C" {

float ref_f16_to_f32(uint16_t h) { return cm::f16_to_f32(h); }
uint16_t ref_f32_to_f16(float v) { return cm::f32_to_f16_bits(v); }
uint32_t ref_iq3s_grid(int i) { return cm::kIq3sGrid[i & 511]; }
uint64_t ref_iq2s_grid(int i) { return cm::kIq2sGrid[i & 1023]; }

void ref_quantize_q8_0(const float * x, uint8_t * blocks, int n) {
    static_assert(sizeof(cm::q8_0) == 34, "Q8_0 block");
    cm::quantize_q8_0(x, reinterpret_cast<cm::q8_0 *>(blocks), n);
}

void ref_quantize_q8_K(const float * x, void * packed, int n) {
    std::vector<cm::q8_K> tmp(static_cast<size_t>(n));
    cm::quantize_q8_K(x, tmp.data(), n);
    PackedQ8K * p = static_cast<PackedQ8K *>(packed);
    for (int i = 0; i < n; ++i) {
        p[i].d = tmp[i].d;
        std::memcpy(p[i].qs, tmp[i].qs, 256);
        std::memcpy(p[i].bsums, tmp[i].bsums, 32);
    }
}

// variant 0: the AVX2 kernel the engine runs; 1: the reference's scalar twin.
float ref_row_iq3_s_q8_K(const uint8_t * w, const void * y, int cols, int variant) {
    auto yk = unpack_q8k(y, cols / 256);
    return variant ? cm::scalar_iq3_s_q8_K(w, yk.data(), cols) : cm::row_iq3_s_q8_K(w, yk.data(), cols);
}
float ref_row_iq2_s_q8_K(const uint8_t * w, const void * y, int cols, int variant) {
    auto yk = unpack_q8k(y, cols / 256);
    return variant ? cm::scalar_iq2_s_q8_K(w, yk.data(), cols) : cm::row_iq2_s_q8_K(w, yk.data(), cols);
}
float ref_row_q8_0_q8_0(const uint8_t * w, const uint8_t * y, int cols, int variant) {
    const cm::q8_0 * yb = reinterpret_cast<const cm::q8_0 *>(y);
    return variant ? cm::scalar_q8_0_q8_0(w, yb, cols) : cm::row_q8_0_q8_0(w, yb, cols);
}
float ref_row_iq4_nl_q8_0(const uint8_t * w, const uint8_t * y, int cols, int variant) {
    const cm::q8_0 * yb = reinterpret_cast<const cm::q8_0 *>(y);
    return variant ? cm::scalar_iq4_nl_q8_0(w, yb, cols) : cm::row_iq4_nl_q8_0(w, yb, cols);
}

// The dense loader's host requantiser (ggml_requantize_row_to_q8_0, src/ggml_dequant.hpp:362-392) and its Q6_K value.
int ref_requantize_row_to_q8_0(int type, const uint8_t * src, uint8_t * dst, int cols) {
    try {
        wd::ggml_requantize_row_to_q8_0(static_cast<wd::GgmlType>(type), src, dst, cols);
    } catch (const std::exception &) {
        return -1;
    }
    return 0;
}
float ref_q6_k_value(const uint8_t * blk, int i) { return wd::ggml_q6_k_value(blk, i); }

float ref_exp_ggml(float x) { return cm::ggml_avx2_exp_f32(x); }
float ref_silu_ggml(float x) { return cm::silu_ggml(x); }
float ref_sigmoid_ggml(float x) { return cm::sigmoid_ggml(x); }
float ref_dot_f32(const float * a, const float * b, int n) { return cm::dot_f32_avx2(a, b, n); }

// The device router functions of src/qwen38_moe.cuh compiled for the host.
void ref_router_exact(const float * logits, int n, int k, float w_scale, float * probs, int * ids,
                      float * weights) {
    wd::q38_moe_router_exact(logits, n, k, w_scale, probs, ids, weights);
}
float ref_router_exp(float x) { return wd::q38_exact_avx2_exp_f32(x); }

int ref_hardware_threads() { return cm::thread_count(); }

struct RefMoeWeights {
    int hidden, expert_ffn, shared_ffn, n_experts, top_k;
    int gate_type, up_type, down_type;
    float w_scale;
    const uint8_t * router;
    const float * router_bias;
    const uint8_t * gate;
    const uint8_t * up;
    const uint8_t * down;
    const float * shared_gate_vec;
    const uint8_t * shared_gate;
    const uint8_t * shared_up;
    const uint8_t * shared_down;
    const float * router_f32;   // F32 router [n_experts][hidden] (src/qwen38_moe.cuh:2252-2258); null: the Q8_0 one
};

// One MoE block on `threads` host threads. ids/weights/out are outputs; ids_in, when
// not null, skips the router and uses the given selection (routed experts only path).
int ref_moe_block(const RefMoeWeights * w, const float * x, int threads, int * ids, float * weights,
                  float * logits_out, float * out) {
    const int H = w->hidden, F = w->expert_ffn, SF = w->shared_ffn, E = w->n_experts, K = w->top_k;
    // q38_moe_expert_q8_act_geometry (src/qwen38_moe.cuh:2181-2183): hidden % 256, expert_ffn % 64; a Q8_K activation
    // for the down projection needs whole superblocks
    if (H % 256 || F % (uses_q8k(w->down_type) ? 256 : 64) || SF % 32 || K > 16 || K <= 0) return -1;
    const int gt = cm::block_type_from_ggml(w->gate_type);
    const int ut = cm::block_type_from_ggml(w->up_type);
    const int dt = cm::block_type_from_ggml(w->down_type);
    if (gt < 0 || ut < 0 || dt < 0) return -2;
    static std::unique_ptr<Pool> pool;
    if (!pool || pool->threads() != threads) pool.reset(new Pool(threads));

    const size_t q8_h = cm::row_bytes(cm::kQ8_0, H);
    std::vector<cm::q8_0> x_q80(static_cast<size_t>(H / 32));
    cm::quantize_q8_0(x, x_q80.data(), H / 32);
    std::vector<float> logits(static_cast<size_t>(E)), probs(static_cast<size_t>(E));
    pool->parallel_for(threads, [&](int t) {
        for (int e = t; e < E; e += threads) {
            float v = w->router_f32 ? cm::dot_f32_avx2(w->router_f32 + static_cast<size_t>(e) * H, x, H)
                                    : cm::row_q8_0_q8_0(w->router + static_cast<size_t>(e) * q8_h, x_q80.data(), H);
            if (w->router_bias) v = v + w->router_bias[e];
            logits[static_cast<size_t>(e)] = v;
        }
    });
    wd::q38_moe_router_exact(logits.data(), E, K, w->w_scale, probs.data(), ids, weights);
    if (logits_out) std::memcpy(logits_out, logits.data(), sizeof(float) * static_cast<size_t>(E));

    std::vector<cm::q8_K> x_q8k(static_cast<size_t>(H / 256));
    cm::quantize_q8_K(x, x_q8k.data(), H / 256);
    const size_t g_rb = cm::row_bytes(gt, H), u_rb = cm::row_bytes(ut, H), d_rb = cm::row_bytes(dt, F);
    std::vector<std::vector<float>> eo(static_cast<size_t>(K), std::vector<float>(static_cast<size_t>(H)));
    std::vector<std::vector<cm::q8_K>> a_k(static_cast<size_t>(K), std::vector<cm::q8_K>(static_cast<size_t>(F / 256 + 1)));
    std::vector<std::vector<cm::q8_0>> a_0(static_cast<size_t>(K), std::vector<cm::q8_0>(static_cast<size_t>(F / 32)));
    // stage 1: one pool task per selected expert (src/qwen38_cpu_moe.cuh:1259-1261)
    pool->parallel_for(K, [&](int j) {
        const int e = ids[j];
        const uint8_t * g0 = w->gate + static_cast<size_t>(e) * F * g_rb;
        const uint8_t * u0 = w->up + static_cast<size_t>(e) * F * u_rb;
        std::vector<float> act(static_cast<size_t>(F));
        for (int r = 0; r < F; ++r) {
            float g, u;
            if (gt == ut) {
                cm::dot_gate_up_row(gt, g0 + static_cast<size_t>(r) * g_rb, u0 + static_cast<size_t>(r) * u_rb,
                                    x_q8k.data(), H, &g, &u);
            } else {
                g = cm::dot_row(gt, g0 + static_cast<size_t>(r) * g_rb, x_q8k.data(), H);
                u = cm::dot_row(ut, u0 + static_cast<size_t>(r) * u_rb, x_q8k.data(), H);
            }
            act[static_cast<size_t>(r)] = cm::silu_ggml(g) * u;
        }
        if (uses_q8k(w->down_type)) cm::quantize_q8_K(act.data(), a_k[static_cast<size_t>(j)].data(), F / 256);
        else cm::quantize_q8_0(act.data(), a_0[static_cast<size_t>(j)].data(), F / 32);
    });
    // stage 2: k * slices row ranges (src/qwen38_cpu_moe.cuh:1264-1279)
    const int slices = std::max(1, std::min(pool->threads(), H / 64));
    const int rows_per = (H + slices - 1) / slices;
    pool->parallel_for(K * slices, [&](int t) {
        const int j = t / slices, s = t % slices;
        const int from = s * rows_per, to = std::min(H, from + rows_per);
        const uint8_t * d0 = w->down + static_cast<size_t>(ids[j]) * H * d_rb;
        const void * a = uses_q8k(w->down_type) ? static_cast<const void *>(a_k[static_cast<size_t>(j)].data())
                                                : static_cast<const void *>(a_0[static_cast<size_t>(j)].data());
        for (int r = from; r < to; ++r)
            eo[static_cast<size_t>(j)][static_cast<size_t>(r)] = cm::dot_row(dt, d0 + static_cast<size_t>(r) * d_rb, a, F);
    });
    std::vector<float> routed(static_cast<size_t>(H), 0.0f);
    for (int j = 0; j < K; ++j)
        for (int i = 0; i < H; ++i)
            routed[static_cast<size_t>(i)] = cm::add_rn(routed[static_cast<size_t>(i)],
                                                        cm::mul_rn(eo[static_cast<size_t>(j)][static_cast<size_t>(i)], weights[j]));

    if (SF <= 0) {
        std::memcpy(out, routed.data(), sizeof(float) * static_cast<size_t>(H));
        return 0;
    }
    const float sgate = cm::sigmoid_ggml(cm::dot_f32_avx2(w->shared_gate_vec, x, H));
    const size_t q8_f = cm::row_bytes(cm::kQ8_0, SF);
    std::vector<float> sact(static_cast<size_t>(SF));
    pool->parallel_for(threads, [&](int t) {
        for (int r = t; r < SF; r += threads) {
            const float g = cm::row_q8_0_q8_0(w->shared_gate + static_cast<size_t>(r) * q8_h, x_q80.data(), H);
            const float u = cm::row_q8_0_q8_0(w->shared_up + static_cast<size_t>(r) * q8_h, x_q80.data(), H);
            sact[static_cast<size_t>(r)] = cm::silu_ggml(g) * u;
        }
    });
    std::vector<cm::q8_0> s_q80(static_cast<size_t>(SF / 32));
    cm::quantize_q8_0(sact.data(), s_q80.data(), SF / 32);
    pool->parallel_for(threads, [&](int t) {
        for (int r = t; r < H; r += threads) {
            const float d = cm::row_q8_0_q8_0(w->shared_down + static_cast<size_t>(r) * q8_f, s_q80.data(), SF);
            out[r] = cm::add_rn(routed[static_cast<size_t>(r)], cm::mul_rn(d, sgate));
        }
    });
    return 0;
}

}  // extern "C"
