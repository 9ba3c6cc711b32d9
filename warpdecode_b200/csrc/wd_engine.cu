// Host side of the C ABI declared in include/warpdecode_b200.h: engine state, weight upload
// and repack, the expert slot cache, launches, CUDA-graph capture of the per-token stack.
#include "../../include/warpdecode_b200.h"

#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <list>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#include "wd_aux_kernels.cuh"
#include "wd_moe_batch.cuh"
#include "wd_dense.cuh"
#include "wd_dense_decoder.cuh"
#include "wd_dense_token.cuh"
#include "wd_plain_moe.cuh"
#include "wd_grids.h"

namespace {

thread_local std::string g_error;

int fail(int code, const std::string &msg) {
    g_error = msg;
    return code;
}

#define WD_CUDA(call)                                                                          \
    do {                                                                                       \
        cudaError_t e__ = (call);                                                              \
        if (e__ != cudaSuccess)                                                                \
            return fail(WD_E_CUDA, std::string(#call) + ": " + cudaGetErrorString(e__));       \
    } while (0)

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// A copy whose result a kernel on one of this library's NON-BLOCKING streams reads next. cudaMemcpy from pageable host
// memory may return as soon as the bytes sit in the driver's staging buffer, with the last chunk still on its way to the
// device, and a device-to-device cudaMemcpy does not wait on the host side at all; a non-blocking stream is not ordered
// behind either. Waiting for the legacy stream, on which both run, closes that window.
cudaError_t copy_sync(void *dst, const void *src, size_t bytes, cudaMemcpyKind kind) {
    cudaError_t ce = cudaMemcpy(dst, src, bytes, kind);
    if (ce == cudaSuccess) ce = cudaStreamSynchronize(cudaStreamLegacy);
    return ce;
}
cudaError_t upload_sync(void *dst, const void *src, size_t bytes) { return copy_sync(dst, src, bytes, cudaMemcpyHostToDevice); }

// Launch with the programmatic-serialization attribute: the kernel may be scheduled while its predecessor in the
// stream still runs; it orders itself behind it with grid_dep_wait() (wd_device.cuh).
template <class... KArgs, class... Args>
cudaError_t launch_dep(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}


bool pow2(int v) { return v > 0 && (v & (v - 1)) == 0; }

// Device buffers of a stand-alone entry point: released when the function returns, on every path.
struct ScopedDev {
    std::vector<void *> held;
    template <class T>
    cudaError_t alloc(T **out, size_t bytes) {
        const cudaError_t ce = cudaMalloc(reinterpret_cast<void **>(out), bytes);
        if (ce == cudaSuccess) held.push_back(*out);
        return ce;
    }
    ~ScopedDev() {
        for (void *q : held) cudaFree(q);
    }
};

struct Layer {
    uint8_t *router = nullptr;
    float *bias = nullptr;
    float *gate_vec = nullptr;
    uint8_t *sh_gate = nullptr, *sh_up = nullptr, *sh_down = nullptr;
    float *norm = nullptr;
    int *slot_of_expert = nullptr;              // device [E]
    std::vector<int> h_slot;                    // host mirror
    const uint8_t *h_gate = nullptr, *h_up = nullptr, *h_down = nullptr;   // retained host tensors
    bool have_router = false, have_shared = false, have_experts = false;
    bool host_pinned = false;                   // the retained host tensors are page-locked: no bounce copy
    // When the tensors came from a mapped file, misses are read with pread at these offsets instead of through the
    // mapping (no page faults on the copy threads; ExpertFileMap + ExpertPreadPool, src/expert_cache.cuh:204-508).
    int fd = -1;
    uint64_t file_gate = 0, file_up = 0, file_down = 0;
    uint8_t *owned_host = nullptr;              // page-locked copy of a generated layer's experts (capped cache only)
};

// A few host threads that copy missed experts from the caller's (pageable or mapped) tensors into the
// pinned ring, several experts at a time. The counterpart of the reference's ExpertPreadPool
// (src/expert_cache.cuh:357-508), minus the file offsets: the source here is memory.
class CopyPool {
public:
    explicit CopyPool(int n) {
        for (int i = 0; i < n; ++i) workers_.emplace_back([this] { run(); });
    }
    ~CopyPool() {
        {
            std::lock_guard<std::mutex> g(m_);
            stop_ = true;
        }
        cv_.notify_all();
        for (std::thread &t : workers_) t.join();
    }
    void submit(std::function<void()> f) {
        {
            std::lock_guard<std::mutex> g(m_);
            tasks_.push_back(std::move(f));
            ++pending_;
        }
        cv_.notify_one();
    }
    void wait_all() {
        std::unique_lock<std::mutex> g(m_);
        done_.wait(g, [this] { return pending_ == 0; });
    }

private:
    void run() {
        for (;;) {
            std::function<void()> f;
            {
                std::unique_lock<std::mutex> g(m_);
                cv_.wait(g, [this] { return stop_ || !tasks_.empty(); });
                if (tasks_.empty()) return;
                f = std::move(tasks_.front());
                tasks_.pop_front();
            }
            f();
            {
                std::lock_guard<std::mutex> g(m_);
                if (--pending_ == 0) done_.notify_all();
            }
        }
    }
    std::vector<std::thread> workers_;
    std::list<std::function<void()>> tasks_;
    std::mutex m_;
    std::condition_variable cv_, done_;
    int pending_ = 0;
    bool stop_ = false;
};

}  // namespace

struct wd_plain_moe;

struct wd_engine {
    wd_config cfg{};
    wd_plain_moe *plain = nullptr;          // set: the engine runs the plain-layout path (wd_plain_moe.inc) and nothing else
    int n_sm = 0;
    cudaStream_t stream = nullptr;
    int nsb_h = 0, nsb_f = 0, e_first = 0, e_count = 0;
    size_t gate_bytes = 0, down_bytes = 0, slot_bytes = 0;
    int64_t n_slots = 0;
    bool resident = false;
    uint8_t *pool = nullptr;
    std::vector<Layer> layers;
    // cache bookkeeping (used when not every owned expert fits)
    std::vector<int64_t> slot_key;                              // (layer << 32 | expert) or -1
    std::list<int> lru;                                         // front = most recent
    std::vector<std::list<int>::iterator> lru_pos;
    std::unordered_map<int64_t, int> key_slot;
    int64_t hits = 0, misses = 0, evictions = 0;
    int64_t h2d_bytes = 0, fill_host_ns = 0, acquires = 0;      // miss stream: bytes sent, host time spent placing experts
    // miss path of a capped cache: pinned ring and device staging of top_k experts, a copy stream
    cudaStream_t copy_stream = nullptr;
    cudaEvent_t fill_done = nullptr;
    uint8_t *miss_pinned = nullptr, *miss_staging = nullptr;
    int *pinned_ids = nullptr;
    int *miss_info = nullptr;               // page-locked: [0] layer a launch stopped at (-1 none), then [layer][top_k] picks
    // model load (all experts resident): two half-rings of kLoadBatch experts each, pinned and on the device
    uint8_t *load_pinned = nullptr, *load_staging = nullptr;
    cudaEvent_t load_done[2] = {nullptr, nullptr};
    unsigned *host_status = nullptr;  // pinned, device-visible: the last CTA of a launch leaves the status word here
    CopyPool *copy_pool = nullptr;
    // device scratch
    uint16_t *grid_packed = nullptr;        // IQ3_S codebook, packed
    uint16_t *grid2_packed = nullptr;       // IQ2_S codebook, packed
    uint16_t *synth_lut = nullptr;
    unsigned *sync = nullptr;
    unsigned long long *stamps = nullptr;   // [n_sm][16] phase timestamps when profiling is on
    bool profiling = false;
    int stamp_layer = 0;                    // offset of the profiled layer inside a launch
    wd::LayerDev *layer_table = nullptr;    // device copy of the per-layer pointers
    bool layer_table_dirty = true;
    // exchange buffers of the layer kernel: tagged words, two halves (by layer parity) per buffer
    wd::tagged_t *tagged = nullptr;
    size_t tagged_words = 0;
    int last_parity = 0;                    // half that holds the last launch's last layer (for the taps)
    uint32_t epoch = 0;                     // host mirror of the device's tag epoch (sync[8]): tags issued so far
    int last_tokens = 1;                    // tokens of the last forward call
    int *tok_ids = nullptr;                 // [max_tokens][top_k] selection of every token of the last call
    float *tok_weights = nullptr;
    size_t tagged_eo_offset = 0;            // word offset of the expert-output buffer inside `tagged`
    size_t tagged_left_offset = 0;          // word offset of the peers' "left layer" words
    // expert-parallel peers
    int n_peers = 0;
    void *peer_mapped[8] = {};              // bases opened from IPC handles (closed on disconnect); null for local peers
    float *weights = nullptr, *routed = nullptr, *x_buf = nullptr, *out_buf = nullptr, *residual_buf = nullptr;
    int *ids = nullptr;
    uint8_t *staging = nullptr;       // device, ggml-layout upload buffer
    size_t staging_bytes = 0;
    void *pinned = nullptr;           // host, for the *_host entry points and miss fills
    size_t pinned_bytes = 0;
    wd::MoeParams base{};
    size_t smem_bytes = 0;
    // the kernel for geometries compiled in (wd_moe_fast.cuh); null: the generic kernel runs
    const void *fast_fn = nullptr;
    wd::FastParams fbase{};
    size_t fast_smem = 0;
    // the batch kernel (wd_moe_batch.cuh): token batches of a resident single-GPU engine in one pass
    bool batch_ok = false;
    bool batch_single = false;              // one-token calls of wd_moe_forward run on the batch kernel as well
    bool last_batch = false;                // the last forward call ran on the batch kernel (it keeps fewer taps)
    wd::BatchParams bbase{};
    size_t batch_smem = 0;
    wd::tagged_t *btagged = nullptr;        // its exchange words
    float *eo_plain = nullptr, *shdown_plain = nullptr;     // inspection copies the fast kernel writes
    wd::tagged_t *xbuf = nullptr;                           // the compiled kernel's per-CTA mailboxes
    size_t xbuf_words = 0;
    unsigned *fallbacks = nullptr;                          // layers that took the exact rungs
    bool threshold_select = true;   // the generic kernel: ids from a threshold on the logits (WD_THRESHOLD_SELECT=0: the rungs)
};

namespace {

// Geometries the fast kernel is compiled for (IQ3_S experts, a Q8_0 shared expert). The first is the 48-layer
// model's block; the others are the small shapes the parity tests use, so that they exercise the same code.
template <int H, int F, int E, int K, int SF>
const void *fast_entry(const wd_config &c) {
    if (c.hidden == H && c.expert_ffn == F && c.n_experts == E && c.top_k == K && c.shared_ffn == SF)
        return reinterpret_cast<const void *>(&wd::moe_fast_kernel<wd::FastGeo<H, F, E, K, SF>>);
    return nullptr;
}

const void *find_fast_kernel(const wd_config &c) {
    if (c.gate_type != WD_TYPE_IQ3_S || c.down_type != WD_TYPE_IQ3_S) return nullptr;
    // The compiled kernel is opt-in: on the 48-layer model it measures about 10 % behind the generic kernel (see the
    // measurements beside its design notes), so engines run the generic one unless WD_COMPILED_KERNEL=1 is set when
    // they are created.
    const char *v = std::getenv("WD_COMPILED_KERNEL");
    if (v == nullptr || v[0] != '1') return nullptr;
    const void *f = nullptr;
    if (!f) f = fast_entry<2048, 512, 512, 10, 512>(c);
    if (!f) f = fast_entry<2048, 512, 32, 10, 512>(c);
    if (!f) f = fast_entry<512, 256, 32, 6, 256>(c);
    if (!f) f = fast_entry<512, 256, 64, 6, 256>(c);
    if (!f) f = fast_entry<512, 256, 32, 4, 256>(c);
    return f;
}

// Shared-memory plan and per-CTA shares of the fast kernel for this engine's grid.
int plan_fast(wd_engine *e) {
    wd::FastParams &p = e->fbase;
    const wd_config &c = e->cfg;
    const int ncta = e->n_sm;
    const int H = c.hidden, F = c.expert_ffn, E = c.n_experts, K = c.top_k, SF = c.shared_ffn;
    const int nsb_h = H / 256, nsb_f = F / 256, r2 = 32 / nsb_h, r3 = 32 / nsb_f;
    const int t2 = F / r2, t3 = H / r3;
    const size_t row_h = static_cast<size_t>(H / 32) * 34;
    const int n_router_ctas = E / 16, n_pair_ctas = ncta - n_router_ctas;
    if (n_pair_ctas < 1) return fail(WD_E_INVALID, "this grid is too small for the compiled layer kernel of this geometry");
    p.n_sp = (SF + n_pair_ctas - 1) / n_pair_ctas;
    p.p2_max = (K * t2 + ncta - 1) / ncta;
    p.b3_max = (t3 + ncta - 1) / ncta;
    p.act_pad = (p.p2_max * r2 + 15) / 16 * 16;
    if (wd::kFbTiles + 2 * p.p2_max + p.b3_max * K > static_cast<unsigned>(wd::kMaxBars) || p.b3_max * r3 > 80 ||
        p.n_sp > wd::kWarps || p.b3_max > 32)
        return fail(WD_E_INVALID, "this grid is too small for the compiled layer kernel of this geometry");
    size_t off = 0;
    auto take = [&](size_t bytes) {
        const size_t o = off;
        off = align_up(off + bytes, 128);
        return static_cast<unsigned>(o);
    };
    p.off_tab = take(wd::kGridTableBytes);
    p.off_xq0 = take(H);
    p.off_xd0 = take(H / 32 * 4);
    p.off_xk = take(static_cast<size_t>(nsb_h) * wd::kActSbStride);
    p.off_xdk = take(nsb_h * 4);
    p.off_actk = take(static_cast<size_t>(K) * nsb_f * wd::kActSbStride);
    p.off_actd = take(static_cast<size_t>(K) * nsb_f * 4);
    p.off_shq = take(SF);
    p.off_shd = take(SF / 32 * 4);
    p.off_misc = take(wd::kFmEnd * 4);
    p.off_bar = take(wd::kMaxBars * 8);
    p.off_slots = take(static_cast<size_t>(E) * 4);
    // tile accumulator; the F32 copy of x that the shared gate dot needs lives there during phases 0 and 1
    const size_t acc_tiles = std::max<size_t>(2 * p.p2_max, static_cast<size_t>(p.b3_max) * K);
    p.off_acc = take(std::max<size_t>(acc_tiles * wd::kFastAccStride * 4, static_cast<size_t>(H) * 4));
    p.off_xf = p.off_acc;
    p.off_rowbuf = take(static_cast<size_t>(2) * p.p2_max * r2 * 4);
    p.off_rows3 = take(static_cast<size_t>(p.b3_max) * (K + 1) * r3 * 4);
    p.off_push = take(std::max<size_t>(std::max<size_t>(p.act_pad, static_cast<size_t>(p.b3_max) * r3), 16) * 8);
    p.xstride = 2ull * E + 2ull * SF + 32 + 2ull * H + 2ull * K * F;
    p.off_a = take(std::max<size_t>(std::max<size_t>(16, 2 * p.n_sp) * row_h + static_cast<size_t>(H) * 4,
                                    static_cast<size_t>(2) * p.p2_max * wd::kIq3TileBytes));
    p.off_b = take(static_cast<size_t>(p.b3_max) * K * wd::kIq3TileBytes);
    p.off_c = take(static_cast<size_t>(p.b3_max) * r3 * (SF / 32) * 34);
    e->fast_smem = off;
    if (e->fast_smem > 227 * 1024) return fail(WD_E_INVALID, "the compiled layer kernel needs more shared memory than one SM has");
    return WD_OK;
}

int plan_shared_memory(wd_engine *e) {
    wd::MoeParams &p = e->base;
    const wd_config &c = e->cfg;
    const int ncta = e->n_sm;
    const int nbh = c.hidden / 32, nbs = c.shared_ffn / 32;
    size_t off = 0;
    auto take = [&](size_t bytes) {
        const size_t o = off;
        off = align_up(off + bytes, 128);
        return static_cast<unsigned>(o);
    };
    const bool any3 = c.gate_type == WD_TYPE_IQ3_S || c.down_type == WD_TYPE_IQ3_S;
    const bool any2 = c.gate_type == WD_TYPE_IQ2_S || c.down_type == WD_TYPE_IQ2_S;
    p.off_tab = take(any3 ? wd::kGridTableBytes : 128);
    p.off_tab2 = take(any2 ? wd::kIq2TableBytes : 128);
    p.off_xq0 = take(c.hidden);
    p.off_xd0 = take(nbh * 4);
    p.off_xk = take(e->nsb_h * wd::kActSbStride);
    p.off_xdk = take(e->nsb_h * 4);
    p.off_actk = take(static_cast<size_t>(c.top_k) * e->nsb_f * wd::kActSbStride);
    p.off_actd = take(static_cast<size_t>(c.top_k) * e->nsb_f * 4);
    p.off_shq = take(std::max(c.shared_ffn, 16));
    p.off_shd = take(std::max(nbs, 4) * 4);
    p.off_misc = take(4 * static_cast<size_t>(std::max(c.hidden, wd::kMiscSharedAct + c.shared_ffn)));
    const int r_h = 32 / e->nsb_h, r_f = 32 / e->nsb_f;
    const int scr_floats = std::max(r_h * (e->nsb_h * 8 + 8) + 32, r_f * (e->nsb_f * 8 + 8) + 32);
    p.scr_rows = static_cast<unsigned>(scr_floats);
    p.scr_bytes = static_cast<unsigned>(align_up((scr_floats + 64) * 4, 128));
    p.off_scr = take(static_cast<size_t>(p.scr_bytes) * wd::kWarps);
    const int n_rt = c.n_experts / 4, n_st = c.shared_ffn / 4;
    const int t2 = c.expert_ffn / r_h, t3 = c.hidden / r_f;
    p.n1r = (n_rt + ncta - 1) / ncta;
    p.n1s = (n_st + ncta - 1) / ncta;
    p.n2 = (c.top_k * t2 + ncta - 1) / ncta;
    const int n_sd = c.shared_ffn > 0 ? c.hidden / 4 : 0;
    // a CTA takes every ncta-th entry of [tiles | shared-down tasks]: at most ceil(len / ncta) of each part
    p.n3 = (c.top_k * t3 + ncta - 1) / ncta;
    p.nsd = (n_sd + ncta - 1) / ncta;
    if (p.n1r + p.n1s + p.n2 + p.n3 + p.nsd > wd::kMaxBars - 2)
        return fail(WD_E_INVALID, "geometry needs more staging slots per CTA than the kernel supports");
    p.off_bar = take(wd::kMaxBars * 8);
    p.off_slots = take(static_cast<size_t>(c.n_experts) * 4);
    p.off_rowbuf = take(static_cast<size_t>(2 * p.n2) * r_h * 4);
    const size_t rt_bytes = static_cast<size_t>(nbh) * 136;
    // stage A: phase-1 tasks, then gate/up tile pairs, then the selected experts' activations as floats
    const size_t stage_a = std::max(std::max(static_cast<size_t>(p.n1r + p.n1s) * 2 * rt_bytes,
                                             static_cast<size_t>(p.n2) * 2 * p.gu_tile),
                                    static_cast<size_t>(c.top_k) * c.expert_ffn * 4);
    p.off_stage_a = take(stage_a);
    // stage B also holds the F32 shared gate vector during phase 1
    p.off_stage_b = take(std::max(static_cast<size_t>(p.n3) * p.d_tile + static_cast<size_t>(p.nsd) * nbs * 136,
                                  static_cast<size_t>(c.hidden) * 4));
    e->smem_bytes = off;
    if (e->smem_bytes > 227 * 1024)
        return fail(WD_E_INVALID, "geometry needs " + std::to_string(e->smem_bytes) +
                                      " bytes of shared memory per CTA; the limit is 232448");
    return WD_OK;
}

// Shared-memory plan of the batch kernel for up to cfg.max_tokens tokens. Leaves e->batch_ok false (and the batch on
// the single-token kernel's token loop) when the geometry does not fit.
void plan_batch(wd_engine *e) {
    const wd_config &c = e->cfg;
    const wd::MoeParams &m = e->base;
    wd::BatchParams &p = e->bbase;
    e->batch_ok = false;
    const int ncta = e->n_sm, Tm = c.max_tokens, H = c.hidden, F = c.expert_ffn, SF = c.shared_ffn, E = c.n_experts, K = c.top_k;
    if (c.ep_size > 1 || E > wd::kMaxExperts || SF > 2 * wd::kThreads || Tm * K > 64) return;
    if (!e->resident && e->n_slots < static_cast<int64_t>(Tm) * K) return;      // a capped pool must hold one batch's picks
    if (const char *v = std::getenv("WD_BATCH_KERNEL")) if (std::atoi(v) == 0) return;
    // one-token calls take the batch kernel too (29 against 34 us per call at the 48-layer model's shape) unless told otherwise
    e->batch_single = true;
    if (const char *v = std::getenv("WD_BATCH_SINGLE")) e->batch_single = std::atoi(v) != 0;
    const int nbh = H / 32, nbs = SF / 32;
    p.H = H; p.F = F; p.SF = SF; p.E = E; p.K = K; p.T = Tm;
    p.nsb_h = m.nsb_h; p.nsb_f = m.nsb_f; p.t2_log2 = m.t2_log2; p.t3_log2 = m.t3_log2;
    p.w_scale = m.w_scale;
    p.pool = m.pool; p.slot_bytes = m.slot_bytes; p.gate_off = m.gate_off; p.up_off = m.up_off; p.down_off = m.down_off;
    p.grid_packed = m.grid_packed; p.grid2_packed = m.grid2_packed;
    p.gu_type = m.gu_type; p.d_type = m.d_type; p.gu_tile = m.gu_tile; p.d_tile = m.d_tile;
    p.sync = m.sync; p.host_status = m.host_status;
    size_t off = 0;
    auto take = [&](size_t bytes) {
        const size_t o = off;
        off = align_up(off + bytes, 128);
        return static_cast<unsigned>(o);
    };
    const bool any3 = c.gate_type == WD_TYPE_IQ3_S || c.down_type == WD_TYPE_IQ3_S;
    const bool any2 = c.gate_type == WD_TYPE_IQ2_S || c.down_type == WD_TYPE_IQ2_S;
    p.off_tab = take(any3 ? wd::kGridTableBytes : 128);
    p.off_tab2 = take(any2 ? wd::kIq2TableBytes : 128);
    {   // one token's region
        size_t t = 0;
        auto sub = [&](size_t bytes) { const size_t o = t; t = align_up(t + bytes, 16); return static_cast<unsigned>(o); };
        sub(std::max(H, SF * 4));                            // Q8_0 quants of x (offset 0); later the shared activation as floats
        p.tok_xd0 = sub(static_cast<size_t>(nbh) * 4);
        p.tok_xk = sub(static_cast<size_t>(m.nsb_h) * wd::kActSbStride);
        p.tok_xdk = sub(static_cast<size_t>(m.nsb_h) * 4);
        p.tok_shq = sub(std::max(SF, 16));
        p.tok_shd = sub(static_cast<size_t>(std::max(nbs, 4)) * 4);
        p.tok_sel = sub(wd::kMaxK * 8);
        p.tok_stride = static_cast<unsigned>(align_up(t, 128));
    }
    p.off_tok = take(static_cast<size_t>(p.tok_stride) * Tm);
    p.off_misc = take(4 * static_cast<size_t>(wd::kMiscSharedAct + std::max(SF, 32)));
    const int r_h = 32 / m.nsb_h, r_f = 32 / m.nsb_f;
    const int scr_floats = std::max(r_h * (m.nsb_h * 8 + 8) + 32, r_f * (m.nsb_f * 8 + 8) + 32);
    p.scr_rows = static_cast<unsigned>(scr_floats);
    p.scr_bytes = static_cast<unsigned>(align_up((scr_floats + 64) * 4, 128));
    p.off_scr = take(static_cast<size_t>(p.scr_bytes) * wd::kWarps);
    p.off_bar = take(wd::kBatchMaxBars * 8);
    p.off_slots = take(static_cast<size_t>(E) * 4);
    p.off_seq = take(wd::kBatchMaxRing * 4);
    p.off_seg = take(96 * 4 + static_cast<size_t>(wd::kMaxTokens) * K * m.nsb_f * 4);     // segments, pair counters, activation states
    {
        const int t2 = F / r_h, t3d = H / r_f;
        if (t2 > 4096 || t3d > 4096) return;
        p.max_tasks = static_cast<unsigned>(Tm * (2 * ((K * t2 + ncta - 1) / ncta) + (K * t3d + ncta - 1) / ncta + 1));
        p.off_tasks = take(static_cast<size_t>(p.max_tasks) * 16);
    }
    p.off_pairbuf = take(static_cast<size_t>(32) * 2 * r_h * 4);
    const int t3 = H / r_f;                                  // down tiles per pair
    const int max3 = (K * t3 + ncta - 1) / ncta;             // longest run of one token's down tiles in one CTA
    const int n_exp_tok = std::min(K, (max3 - 1) / t3 + 2);  // pairs such a run can touch
    p.n_act = static_cast<unsigned>(wd::kMaxTokens * n_exp_tok * m.nsb_f);
    if (p.n_act > 62) return;
    p.off_actk = take(static_cast<size_t>(p.n_act) * wd::kActSbStride);
    p.off_actd = take(static_cast<size_t>(p.n_act) * 4);
    const int n_rt = E / 4, n_st = SF / 4, n_sd = SF > 0 ? H / 4 : 0;
    p.n1r = (n_rt + ncta - 1) / ncta;
    p.n1s = (n_st + ncta - 1) / ncta;
    p.nsd = (n_sd + ncta - 1) / ncta;
    p.off_sd = take(static_cast<size_t>(p.nsd) * nbs * 136);
    p.off_ring = take(0);
    p.ring_slot = static_cast<unsigned>(align_up(std::max(p.gu_tile, p.d_tile), 16));
    const size_t limit = 227 * 1024;
    if (off >= limit) return;
    const size_t front = static_cast<size_t>(p.n1r + p.n1s) * 2 * nbh * 136 + static_cast<size_t>(H) * 4 * (1 + Tm);
    const int bars_fixed = static_cast<int>(p.n1r + p.n1s + 3 + p.nsd + wd::kMaxTokens + p.n_act);
    int ring = static_cast<int>((limit - off) / p.ring_slot);
    ring = std::min(ring, std::min(wd::kBatchMaxRing, wd::kBatchMaxBars - bars_fixed));
    if (const char *v = std::getenv("WD_BATCH_RING")) ring = std::min(ring, std::max(1, std::atoi(v)));
    // sixteen slots are being read at any time; the rest is how far ahead the copies run
    if (ring < wd::kWarps + 4 || static_cast<size_t>(ring) * p.ring_slot < front) return;
    const int rpc = (H + ncta - 1) / ncta;
    if (rpc * Tm > wd::kThreads) return;
    p.ring = static_cast<unsigned>(ring);
    e->batch_smem = off + static_cast<size_t>(ring) * p.ring_slot;
    e->batch_ok = true;
}

// ggml Q8_0 blocks -> the layout of the engine's layer kernel (4-row tasks, or single rows for the compiled kernel)
void launch_repack_q8(const wd_engine *e, const uint8_t *src, uint8_t *dst, int rows, int nb, cudaStream_t s) {
    const long long n = static_cast<long long>(rows) * nb;
    const unsigned grid = static_cast<unsigned>((n + 255) / 256);
    if (e->fast_fn) wd::repack_q8_0_rows_kernel<<<grid, 256, 0, s>>>(src, dst, rows, nb);
    else wd::repack_q8_0_kernel<<<grid, 256, 0, s>>>(src, dst, rows, nb);
}

int upload_repacked_q8(wd_engine *e, const void *host_ggml, int rows, int cols, uint8_t **dev_out) {
    const size_t bytes = static_cast<size_t>(rows) * (cols / 32) * 34;
    if (bytes > e->staging_bytes) return fail(WD_E_STATE, "staging buffer too small for a Q8_0 tensor");
    if (!*dev_out) WD_CUDA(cudaMalloc(dev_out, bytes));
    WD_CUDA(cudaMemcpyAsync(e->staging, host_ggml, bytes, cudaMemcpyHostToDevice, e->stream));
    launch_repack_q8(e, e->staging, *dev_out, rows, cols / 32, e->stream);
    WD_CUDA(cudaGetLastError());
    WD_CUDA(cudaStreamSynchronize(e->stream));
    return WD_OK;
}

int upload_f32(wd_engine *e, const float *host, size_t n, float **dev_out) {
    if (!*dev_out) WD_CUDA(cudaMalloc(dev_out, n * 4));
    WD_CUDA(upload_sync(*dev_out, host, n * 4));
    (void)e;
    return WD_OK;
}

// ggml blocks -> tiles for either expert format (grid.y batches of `src_stride` / `dst_stride` bytes)
static void launch_repack_iq(int type, const uint8_t *src, uint8_t *dst, long long nblocks, long long src_stride,
                             long long dst_stride, unsigned batches, cudaStream_t s) {
    const dim3 grid(static_cast<unsigned>((nblocks + 127) / 128), batches);
    if (type == WD_TYPE_IQ2_S) wd::repack_iq2s_kernel<<<grid, 128, 0, s>>>(src, dst, nblocks, src_stride, dst_stride);
    else wd::repack_iq3s_kernel<<<grid, 128, 0, s>>>(src, dst, nblocks, src_stride, dst_stride);
}

// Repack one expert's three ggml tensors (device pointers) into slot `slot`.
int repack_expert_into_slot(wd_engine *e, const uint8_t *g, const uint8_t *u, const uint8_t *d, int slot,
                            cudaStream_t s) {
    uint8_t *dst = e->pool + static_cast<size_t>(slot) * e->slot_bytes;
    const long long nb_gu = static_cast<long long>(e->cfg.expert_ffn) * e->nsb_h;
    const long long nb_d = static_cast<long long>(e->cfg.hidden) * e->nsb_f;
    launch_repack_iq(e->cfg.gate_type, g, dst, nb_gu, 0, 0, 1, s);
    launch_repack_iq(e->cfg.gate_type, u, dst + e->gate_bytes, nb_gu, 0, 0, 1, s);
    launch_repack_iq(e->cfg.down_type, d, dst + 2 * e->gate_bytes, nb_d, 0, 0, 1, s);
    WD_CUDA(cudaGetLastError());
    return WD_OK;
}

int check_layer(const wd_engine *e, int layer) {
    if (!e) return fail(WD_E_INVALID, "null engine");
    if (layer < 0 || layer >= e->cfg.n_layers) return fail(WD_E_STATE, "layer index out of range");
    return WD_OK;
}

void touch_slot(wd_engine *e, int slot) {
    e->lru.erase(e->lru_pos[slot]);
    e->lru.push_front(slot);
    e->lru_pos[slot] = e->lru.begin();
}

// Uploads the per-layer pointer table when any layer's pointers changed since the last launch.
int sync_layer_table(wd_engine *e, cudaStream_t s) {
    if (!e->layer_table_dirty) return WD_OK;
    std::vector<wd::LayerDev> host(e->layers.size());
    for (size_t i = 0; i < e->layers.size(); ++i) {
        const Layer &L = e->layers[i];
        host[i] = wd::LayerDev{L.router, L.bias, L.gate_vec, L.sh_gate, L.sh_up, L.sh_down, L.norm, L.slot_of_expert};
    }
    WD_CUDA(cudaMemcpyAsync(e->layer_table, host.data(), host.size() * sizeof(wd::LayerDev), cudaMemcpyHostToDevice, s));
    WD_CUDA(cudaStreamSynchronize(s));      // `host` goes out of scope
    e->layer_table_dirty = false;
    return WD_OK;
}

// Layers [begin, end) in one cooperative launch.
int launch_layers(wd_engine *e, int begin, int end, const float *x, float *residual, float *out, cudaStream_t s,
                  bool select_only = false, int n_tokens = 1, bool stop_on_miss = false) {
    for (int l = begin; l < end; ++l) {
        const Layer &L = e->layers[l];
        if (!L.have_router || !L.have_experts || (e->cfg.shared_ffn > 0 && !L.have_shared))
            return fail(WD_E_STATE, "layer " + std::to_string(l) + " has no weights yet");
    }
    int rc = sync_layer_table(e, s);
    if (rc) return rc;
    if (e->fast_fn) {
        wd::FastParams p = e->fbase;
        p.layers = e->layer_table;
        p.layer_begin = begin;
        p.layer_end = end;
        p.stamp_layer = std::min(end - 1, begin + e->stamp_layer);
        p.x = x;
        p.residual = residual;
        p.out = out;
        p.stamps = e->profiling ? e->stamps : nullptr;
        p.select_only = select_only ? 1 : 0;
        void *args[] = {&p};
        WD_CUDA(cudaLaunchCooperativeKernel(e->fast_fn, dim3(e->n_sm), dim3(wd::kThreads), args, e->fast_smem, s));
    } else {
        wd::MoeParams p = e->base;
        p.layers = e->layer_table;
        p.layer_begin = begin;
        p.layer_end = end;
        p.n_tokens = n_tokens;
        p.stop_on_miss = stop_on_miss ? 1 : 0;
        p.miss_info = e->miss_info;
        p.threshold_select = e->threshold_select ? 1 : 0;
        p.fallbacks = e->fallbacks;
        if (n_tokens > 1) {         // the selection of every token of the batch is kept
            p.ids = e->tok_ids;
            p.weights = e->tok_weights;
        }
        p.stamp_layer = std::min(end - 1, begin + e->stamp_layer);
        p.x = x;
        p.residual = residual;
        p.out = out;
        p.stamps = e->profiling ? e->stamps : nullptr;
        p.select_only = select_only ? 1 : 0;
        void *args[] = {&p};
        WD_CUDA(cudaLaunchCooperativeKernel(reinterpret_cast<void *>(wd::moe_layer_kernel), dim3(e->n_sm),
                                            dim3(wd::kThreads), args, e->smem_bytes, s));
    }
    // the kernel advances the device's epoch by the length of its sequence (layers, or the tokens of a batch)
    e->epoch += static_cast<uint32_t>(n_tokens > 1 && !e->fast_fn ? n_tokens : end - begin);
    e->last_parity = static_cast<int>(e->epoch & 1u);   // the last layer's tag is the new epoch; halves follow the tag
    e->last_tokens = 1;
    e->last_batch = false;
    return WD_OK;
}

int launch_layer(wd_engine *e, int layer, const float *x, float *residual, float *out, cudaStream_t s) {
    return launch_layers(e, layer, layer + 1, x, residual, out, s);
}

// A batch of n_tokens activations through one layer on the batch kernel (one cooperative launch).
int launch_batch(wd_engine *e, int layer, const float *x, float *out, int n_tokens, cudaStream_t s, bool stop_on_miss = false) {
    const Layer &L = e->layers[layer];
    if (!L.have_router || !L.have_experts || (e->cfg.shared_ffn > 0 && !L.have_shared))
        return fail(WD_E_STATE, "layer " + std::to_string(layer) + " has no weights yet");
    int rc = sync_layer_table(e, s);
    if (rc) return rc;
    wd::BatchParams p = e->bbase;
    p.layers = e->layer_table;
    p.layer = layer;
    p.T = n_tokens;
    p.threshold_select = e->threshold_select ? 1 : 0;
    p.fallbacks = e->fallbacks;
    p.stop_on_miss = stop_on_miss ? 1 : 0;
    p.miss_info = stop_on_miss ? e->miss_info : nullptr;
    p.x = x;
    p.out = out;
    p.ids = e->tok_ids;
    p.weights = e->tok_weights;
    p.routed = e->routed;
    p.stamps = e->profiling ? e->stamps : nullptr;
    void *args[] = {&p};
    WD_CUDA(cudaLaunchCooperativeKernel(reinterpret_cast<void *>(wd::moe_batch_kernel), dim3(e->n_sm), dim3(wd::kThreads), args,
                                        e->batch_smem, s));
    e->epoch += 1u;         // the whole batch carries one tag
    e->last_parity = static_cast<int>(e->epoch & 1u);
    e->last_tokens = n_tokens;
    e->last_batch = true;
    return WD_OK;
}

// Capped cache: one layer = a selection pass, the host's slot bookkeeping with the misses streamed in on
// the copy stream, then the full layer (which repeats the selection bit for bit and finds every slot).
// The flow of q38_moe_select_experts_f32_x + GpuExpertCache::acquire + ExpertStagePath
// (src/qwen38_moe.cuh:2323-2380, src/expert_cache.cuh:2252, :1166-1273).
int acquire_selected(wd_engine *e, int layer, cudaStream_t s, const int *host_ids = nullptr) {
    const wd_config &c = e->cfg;
    Layer &L = e->layers[layer];
    if (host_ids) {         // the picks are on the host already (a stopped launch left them there)
        memcpy(e->pinned_ids, host_ids, sizeof(int) * c.top_k);
    } else {
        WD_CUDA(cudaMemcpyAsync(e->pinned_ids, e->ids, sizeof(int) * c.top_k, cudaMemcpyDeviceToHost, s));
        WD_CUDA(cudaStreamSynchronize(s));
    }
    if (!L.h_gate) return fail(WD_E_STATE, "no host tensors to fill the slots from");
    std::vector<int> owned;
    for (int j = 0; j < c.top_k; ++j) {
        const int x = e->pinned_ids[j];
        if (x < 0 || x >= c.n_experts) return fail(WD_E_DEVICE, "the selection pass returned an expert id out of range");
        if (x >= e->e_first && x < e->e_first + e->e_count && std::find(owned.begin(), owned.end(), x) == owned.end())
            owned.push_back(x);
    }
    // hits first: they move to the front of the LRU list, so no victim below can be one of this layer's experts
    std::vector<int> missing;
    for (int x : owned) {
        if (L.h_slot[x] >= 0) {
            ++e->hits;
            touch_slot(e, L.h_slot[x]);
        } else {
            missing.push_back(x);
        }
    }
    if (missing.empty()) return WD_OK;
    const size_t gb = e->gate_bytes, db = e->down_bytes, one = 2 * gb + db;
    const auto t_begin = std::chrono::steady_clock::now();
    ++e->acquires;
    std::vector<int> changed_layers{layer};
    std::vector<int> slots(missing.size());
    // Pageable or file-backed sources: three read tasks per missed expert (gate, up, down) go to the copy threads at
    // once; each expert's DMA and repack are enqueued as soon as ITS three reads are done, while the threads keep
    // reading the next ones (ExpertPreadPool + ExpertStagePath::submit, src/expert_cache.cuh:357-508, :1166-1273).
    // A ring entry is free here because the previous layer's launch, which waited for its DMAs, has completed
    // (the ids this function works from were read after it).
    std::vector<std::atomic<int>> reads_left(missing.size());
    // whatever way this function is left, the read tasks (which point into this frame) have finished by then
    struct Drain {
        CopyPool *pool;
        ~Drain() {
            if (pool) pool->wait_all();
        }
    } drain{L.host_pinned ? nullptr : e->copy_pool};
    for (size_t m = 0; m < missing.size(); ++m) {
        const int x = missing[m], slot = e->lru.back();
        ++e->misses;
        const int64_t old = e->slot_key[slot];
        if (old >= 0) {
            const int ol = static_cast<int>(old >> 32);
            e->layers[ol].h_slot[static_cast<int>(old & 0xffffffff)] = -1;
            e->key_slot.erase(old);
            ++e->evictions;
            if (std::find(changed_layers.begin(), changed_layers.end(), ol) == changed_layers.end()) changed_layers.push_back(ol);
        }
        const int64_t key = (static_cast<int64_t>(layer) << 32) | static_cast<uint32_t>(x);
        e->slot_key[slot] = key;
        e->key_slot[key] = slot;
        L.h_slot[x] = slot;
        touch_slot(e, slot);
        slots[m] = slot;
        reads_left[m].store(L.host_pinned ? 0 : 3, std::memory_order_relaxed);
        if (!L.host_pinned) {
            uint8_t *pin = e->miss_pinned + m * one;
            const int fd = L.fd;
            std::atomic<int> *left = &reads_left[m];
            const struct { uint8_t *to; const uint8_t *from; uint64_t off; size_t n; } parts[3] = {
                {pin, L.h_gate + static_cast<size_t>(x) * gb, L.file_gate + static_cast<uint64_t>(x) * gb, gb},
                {pin + gb, L.h_up + static_cast<size_t>(x) * gb, L.file_up + static_cast<uint64_t>(x) * gb, gb},
                {pin + 2 * gb, L.h_down + static_cast<size_t>(x) * db, L.file_down + static_cast<uint64_t>(x) * db, db}};
            for (const auto &pt : parts) {
                uint8_t *to = pt.to;
                const uint8_t *from = pt.from;
                const uint64_t off = pt.off;
                const size_t n = pt.n;
                e->copy_pool->submit([=] {
                    // file-backed tensors: positional reads; a short or failed read falls back to the mapping
                    size_t done = 0;
                    while (fd >= 0 && done < n) {
                        const ssize_t r = pread(fd, to + done, n - done, static_cast<off_t>(off + done));
                        if (r <= 0) break;
                        done += static_cast<size_t>(r);
                    }
                    if (done < n) memcpy(to + done, from + done, n - done);
                    left->fetch_sub(1, std::memory_order_release);
                });
            }
        }
    }
    cudaStream_t cs = e->copy_stream;
    for (size_t m = 0; m < missing.size(); ++m) {
        uint8_t *st = e->miss_staging + m * one;
        if (L.host_pinned) {
            const int x = missing[m];
            WD_CUDA(cudaMemcpyAsync(st, L.h_gate + static_cast<size_t>(x) * gb, gb, cudaMemcpyHostToDevice, cs));
            WD_CUDA(cudaMemcpyAsync(st + gb, L.h_up + static_cast<size_t>(x) * gb, gb, cudaMemcpyHostToDevice, cs));
            WD_CUDA(cudaMemcpyAsync(st + 2 * gb, L.h_down + static_cast<size_t>(x) * db, db, cudaMemcpyHostToDevice, cs));
        } else {
            while (reads_left[m].load(std::memory_order_acquire) > 0) std::this_thread::yield();
            WD_CUDA(cudaMemcpyAsync(st, e->miss_pinned + m * one, one, cudaMemcpyHostToDevice, cs));
        }
        e->h2d_bytes += static_cast<int64_t>(one);
        int rc = repack_expert_into_slot(e, st, st + gb, st + 2 * gb, slots[m], cs);
        if (rc) return rc;
    }
    for (int l : changed_layers) {
        Layer &C = e->layers[l];      // pageable source: the runtime stages it before the call returns
        WD_CUDA(cudaMemcpyAsync(C.slot_of_expert, C.h_slot.data(), C.h_slot.size() * sizeof(int), cudaMemcpyHostToDevice, cs));
    }
    WD_CUDA(cudaEventRecord(e->fill_done, cs));
    WD_CUDA(cudaStreamWaitEvent(s, e->fill_done, 0));
    e->fill_host_ns += std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now() - t_begin).count();
    return WD_OK;
}

// Capped cache, optimistic: layers [begin, end) in ONE launch as long as every selected expert is resident. A launch
// that meets a missing expert stops at that layer; the host touches the finished layers' picks (recency order),
// places the stopped layer's experts and launches again from there. With a warm cache a token is one launch and one
// synchronisation, as with every expert resident. (The flow of GpuExpertCache::acquire + ExpertStagePath,
// src/expert_cache.cuh:2252, :1166-1273, without the per-layer host round trip of q38_moe_select_experts_f32_x,
// src/qwen38_moe.cuh:2363-2379.) Synchronises the stream.
int run_capped_optimistic(wd_engine *e, int begin, int end, const float *x, float *residual, float *out, cudaStream_t s) {
    const int K = e->cfg.top_k;
    int l = begin;
    bool relaunch = false;      // layer l was counted when its experts were placed
    int launches = 0;
    while (l < end) {
        // every launch either ends the range or places one more layer's experts: more launches than that is a fault
        if (++launches > 2 * (end - begin) + 2) return fail(WD_E_DEVICE, "the capped cache keeps stopping at the same layer");
        e->miss_info[0] = -1;
        int rc = launch_layers(e, l, end, x, residual, out, s, false, 1, true);
        if (rc) return rc;
        WD_CUDA(cudaStreamSynchronize(s));
        const int stopped = e->miss_info[0];
        const int done_end = stopped >= 0 ? stopped : end;       // layers [l, done_end) ran completely
        if (stopped >= 0) {
            // launch_layers counted end - l tags; the launch used stopped - l + 1
            e->epoch -= static_cast<uint32_t>(end - l);
            e->epoch += static_cast<uint32_t>(stopped - l + 1);
            e->last_parity = static_cast<int>(e->epoch & 1u);
        }
        for (int d = l; d < done_end; ++d) {                     // every pick of a finished layer was a hit
            for (int j = 0; j < K; ++j) {
                const int x_id = e->miss_info[1 + d * K + j];
                if (x_id >= e->e_first && x_id < e->e_first + e->e_count && e->layers[d].h_slot[x_id] >= 0) {
                    if (!(relaunch && d == l)) ++e->hits;
                    touch_slot(e, e->layers[d].h_slot[x_id]);
                }
            }
        }
        if (stopped < 0) break;
        if (stopped < l || stopped >= end) return fail(WD_E_DEVICE, "a stopped launch reported a layer outside its range");
        if (relaunch && stopped == l) return fail(WD_E_DEVICE, "a layer missed again right after its experts were placed");
        if ((rc = acquire_selected(e, stopped, s, e->miss_info + 1 + stopped * K))) return rc;
        l = stopped;
        relaunch = true;
    }
    return WD_OK;
}

int forward_capped(wd_engine *e, int layer, const float *x, float *residual, float *out, cudaStream_t s) {
    if (!e->fast_fn && e->n_peers == 0) return run_capped_optimistic(e, layer, layer + 1, x, residual, out, s);
    int rc = launch_layers(e, layer, layer + 1, x, residual, out, s, true);
    if (rc) return rc;
    if ((rc = acquire_selected(e, layer, s))) return rc;
    return launch_layers(e, layer, layer + 1, x, residual, out, s, false);
}

// A token batch on a capped cache: the batch kernel stops before its tile phase when a picked expert has no slot; the host
// then places every token's picks (hits are touched first, so one token's misses cannot evict another's picks as long as
// the pool holds a whole batch) and launches again.
int forward_capped_batch(wd_engine *e, int layer, const float *x, float *out, int n_tokens, cudaStream_t s) {
    const int K = e->cfg.top_k;
    for (int attempt = 0;; ++attempt) {
        e->miss_info[0] = -1;
        int rc = launch_batch(e, layer, x, out, n_tokens, s, true);
        if (rc) return rc;
        WD_CUDA(cudaStreamSynchronize(s));
        const int missed = e->miss_info[0];
        if (missed < 0) return fail(WD_E_DEVICE, "the batch kernel left no report of its picks");
        if (missed == 0) {
            if (attempt == 0) {         // every pick was a hit: count and touch them (a relaunch was counted when it was placed)
                for (int i = 0; i < n_tokens * K; ++i) {
                    const int x_id = e->miss_info[1 + i];
                    if (x_id >= 0 && x_id < e->cfg.n_experts && e->layers[layer].h_slot[x_id] >= 0) {
                        ++e->hits;
                        touch_slot(e, e->layers[layer].h_slot[x_id]);
                    }
                }
            }
            return WD_OK;
        }
        if (attempt >= 2) return fail(WD_E_DEVICE, "a token batch missed again right after its experts were placed");
        std::vector<int> picks(e->miss_info + 1, e->miss_info + 1 + n_tokens * K);   // acquire_selected reuses the pinned words
        for (int t = 0; t < n_tokens; ++t) {
            if ((rc = acquire_selected(e, layer, s, picks.data() + t * K))) return rc;
            // the next token's misses go through the same pinned ring and device staging: this token's copies must have left them
            WD_CUDA(cudaStreamSynchronize(e->copy_stream));
        }
    }
}

int check_device_status(wd_engine *e) {
    unsigned st = 0;
    WD_CUDA(cudaMemcpy(&st, e->sync + 2, sizeof(st), cudaMemcpyDeviceToHost));
    if (st != 0) {
        unsigned where[2] = {0, 0};     // shared-memory address of the first copy barrier that timed out, and of barrier 0
        cudaMemcpy(where, e->sync + 4, sizeof(where), cudaMemcpyDeviceToHost);
        const std::string bar = (st & 2u) ? " [copy barrier " + std::to_string((static_cast<long long>(where[0]) - where[1]) / 8) + "]" : "";
        // an interrupted launch leaves the tag epoch and the exchange words undefined: start over
        cudaMemset(e->sync, 0, 8192);
        cudaMemset(e->tagged, 0, e->tagged_words * sizeof(wd::tagged_t));
        if (e->xbuf) cudaMemset(e->xbuf, 0, e->xbuf_words * sizeof(wd::tagged_t));
        cudaDeviceSynchronize();                // the next launch runs on a stream that is not ordered behind these
        e->epoch = 0;
        return fail(WD_E_DEVICE, "kernel raised status " + std::to_string(st) +
                                     " (1 wait timeout, 2 copy timeout, 4 expert without slot, 8 geometry, "
                                     "16 exchange word overwritten before it was read)" + bar);
    }
    return WD_OK;
}

}  // namespace

#include "wd_plain_moe.inc"

#define WD_TILED_ONLY(e)                                                                                              \
    if ((e) && (e)->plain) return fail(WD_E_INVALID, "not available on an engine that runs the plain-layout path (wd_engine_create)")

extern "C" {

const char *wd_last_error(void) { return g_error.c_str(); }
int wd_version(void) { return (0 << 16) | 1; }

int64_t wd_default_cache_mib(int64_t memory_mib) {
    int64_t cache = memory_mib * 3 / 4 - 8 * 1024;
    cache = std::max<int64_t>(512, std::min<int64_t>(64 * 1024, cache));
    if (const char *v = std::getenv("WARODECODE_EXPERT_CACHE_MIB")) {
        const long mib = std::atol(v);
        if (mib > 0) cache = mib;
    }
    return cache;
}

int wd_engine_create(const wd_config *cfg, wd_engine **out) {
    if (!cfg || !out) return fail(WD_E_INVALID, "null argument");
    const wd_config &c = *cfg;
    const bool plain = plain_wanted(c);
    if (!plain && (c.hidden % 256 || !pow2(c.hidden / 256) || c.hidden / 256 > 32))
        return fail(WD_E_INVALID, "hidden must be 256 * 2^n, n <= 5");
    if (!plain && (c.expert_ffn % 256 || !pow2(c.expert_ffn / 256) || c.expert_ffn / 256 > 8))
        return fail(WD_E_INVALID, "expert_ffn must be 256 * 2^n, n <= 3");
    if (c.shared_ffn < 0 || c.shared_ffn % 128) return fail(WD_E_INVALID, "shared_ffn must be a multiple of 128");
    if (c.n_experts <= 0 || c.n_experts % 8 || c.n_experts > wd::kMaxExperts)
        return fail(WD_E_INVALID, "n_experts must be a multiple of 8, at most 1024");
    if (c.top_k < 1 || c.top_k > wd::kMaxK || c.top_k > c.n_experts) return fail(WD_E_INVALID, "top_k must be 1..16");
    if (c.n_layers < 1) return fail(WD_E_INVALID, "n_layers must be positive");
    auto iq = [](int t) { return t == WD_TYPE_IQ3_S || t == WD_TYPE_IQ2_S; };
    if (!plain && (!iq(c.gate_type) || !iq(c.down_type) || c.up_type != c.gate_type))
        return fail(WD_E_INVALID, "expert tensors must be IQ3_S or IQ2_S, gate and up of the same type");
    if (c.ep_size < 1 || c.ep_rank < 0 || c.ep_rank >= c.ep_size || c.n_experts % c.ep_size)
        return fail(WD_E_INVALID, "ep_rank/ep_size must partition n_experts evenly");
    if (c.max_tokens < 1 || c.max_tokens > 4) return fail(WD_E_INVALID, "max_tokens must be 1..4");
    int ndev = 0;
    WD_CUDA(cudaGetDeviceCount(&ndev));
    if (c.device < 0 || c.device >= ndev) return fail(WD_E_INVALID, "no such CUDA device");
    WD_CUDA(cudaSetDevice(c.device));
    cudaDeviceProp prop{};
    WD_CUDA(cudaGetDeviceProperties(&prop, c.device));
    if (prop.major < 10) return fail(WD_E_INVALID, "this library is built for sm_100a only");
    // geometries and tensor types outside the tiled kernels (the reference's own 2560 / 640 model, IQ4_NL down tensors,
    // an F32 router) run on ggml-layout tensors, one warp per row
    if (plain) return plain_create(c, prop, out);

    wd_engine *e = new wd_engine();
    e->cfg = c;
    e->n_sm = prop.multiProcessorCount;
    e->nsb_h = c.hidden / 256;
    e->nsb_f = c.expert_ffn / 256;
    e->e_count = c.n_experts / c.ep_size;
    e->e_first = c.ep_rank * e->e_count;
    e->gate_bytes = static_cast<size_t>(c.expert_ffn) * e->nsb_h * wd::iq_block_bytes(c.gate_type);
    e->down_bytes = static_cast<size_t>(c.hidden) * e->nsb_f * wd::iq_block_bytes(c.down_type);
    e->slot_bytes = align_up(2 * e->gate_bytes + e->down_bytes, 256);
    const int64_t owned = static_cast<int64_t>(e->e_count) * c.n_layers;
    if (c.cache_mib <= 0) {
        e->n_slots = owned;
    } else {
        e->n_slots = std::min<int64_t>(owned, (c.cache_mib << 20) / static_cast<int64_t>(e->slot_bytes));
        if (e->n_slots < c.top_k) {
            delete e;
            return fail(WD_E_INVALID, "expert cache smaller than one layer's selection");
        }
    }
    e->resident = e->n_slots == owned;
    if (const char *v = std::getenv("WD_THRESHOLD_SELECT")) e->threshold_select = v[0] != '0';
    int rc = WD_OK;
    auto bail = [&](int code) {
        wd_engine_destroy(e);
        return code;
    };
    cudaError_t ce;
#define WD_TRY(call)                                                                  \
    if ((ce = (call)) != cudaSuccess) {                                               \
        fail(WD_E_CUDA, std::string(#call) + ": " + cudaGetErrorString(ce));          \
        return bail(WD_E_CUDA);                                                       \
    }
    WD_TRY(cudaStreamCreateWithFlags(&e->stream, cudaStreamNonBlocking));
    WD_TRY(cudaMalloc(&e->pool, static_cast<size_t>(e->n_slots) * e->slot_bytes));
    e->layers.resize(c.n_layers);
    for (Layer &L : e->layers) {
        L.h_slot.assign(c.n_experts, -1);
        WD_TRY(cudaMalloc(&L.slot_of_expert, c.n_experts * sizeof(int)));
        WD_TRY(cudaMemset(L.slot_of_expert, 0xff, c.n_experts * sizeof(int)));
    }
    e->slot_key.assign(e->n_slots, -1);
    e->lru_pos.resize(e->n_slots);
    for (int64_t s = 0; s < e->n_slots; ++s) {
        e->lru.push_back(static_cast<int>(s));
        e->lru_pos[s] = std::prev(e->lru.end());
    }
    WD_TRY(cudaMalloc(&e->grid_packed, sizeof(wd_iq3s_grid_packed)));
    WD_TRY(upload_sync(e->grid_packed, wd_iq3s_grid_packed, sizeof(wd_iq3s_grid_packed)));
    WD_TRY(cudaMalloc(&e->grid2_packed, sizeof(wd_iq2s_grid_packed)));
    WD_TRY(upload_sync(e->grid2_packed, wd_iq2s_grid_packed, sizeof(wd_iq2s_grid_packed)));
    WD_TRY(cudaMalloc(&e->sync, 8192));
    WD_TRY(cudaMemset(e->sync, 0, 8192));
    const int H = c.hidden, F = c.expert_ffn, K = c.top_k, E = c.n_experts, SF = std::max(c.shared_ffn, 1);
    WD_TRY(cudaMalloc(&e->stamps, static_cast<size_t>(e->n_sm) * wd::kStampStride * 8));
    WD_TRY(cudaMemset(e->stamps, 0, static_cast<size_t>(e->n_sm) * wd::kStampStride * 8));
    WD_TRY(cudaMalloc(&e->layer_table, sizeof(wd::LayerDev) * c.n_layers));
    WD_TRY(cudaMalloc(&e->ids, K * 4));
    WD_TRY(cudaMalloc(&e->weights, K * 4));
    WD_TRY(cudaMalloc(&e->routed, H * 4));
    WD_TRY(cudaMalloc(&e->x_buf, static_cast<size_t>(c.max_tokens) * H * 4));
    WD_TRY(cudaMalloc(&e->out_buf, static_cast<size_t>(c.max_tokens) * H * 4));
    WD_TRY(cudaMalloc(&e->tok_ids, static_cast<size_t>(c.max_tokens) * K * 4));
    WD_TRY(cudaMalloc(&e->tok_weights, static_cast<size_t>(c.max_tokens) * K * 4));
    WD_TRY(cudaMalloc(&e->residual_buf, H * 4));
    WD_TRY(cudaMalloc(&e->fallbacks, 64));
    WD_TRY(cudaMemset(e->fallbacks, 0, 64));
    // tagged exchange words: logits, shared act, shared gate, act, expert out, shared down, residual (x2), progress
    // every region starts on a 128-byte line (16 words): lines that one CTA writes are then never shared with another's
    auto up16 = [](size_t w) { return (w + 15) / 16 * 16; };
    const size_t tw_logits = 0, tw_shact = up16(tw_logits + 2 * static_cast<size_t>(E)),
                 tw_shgate = up16(tw_shact + 2 * static_cast<size_t>(SF)), tw_act = tw_shgate + 32,
                 tw_eo = up16(tw_act + 2 * static_cast<size_t>(K) * F),
                 tw_shdown = up16(tw_eo + 2 * static_cast<size_t>(K) * H), tw_res = up16(tw_shdown + 2 * static_cast<size_t>(H)),
                 tw_prog = up16(tw_res + 2 * static_cast<size_t>(H)), tw_left = up16(tw_prog + static_cast<size_t>(e->n_sm)),
                 tw_end = tw_left + 16;
    e->tagged_words = tw_end;
    WD_TRY(cudaMalloc(&e->tagged, e->tagged_words * sizeof(wd::tagged_t)));
    WD_TRY(cudaMemset(e->tagged, 0, e->tagged_words * sizeof(wd::tagged_t)));
    // staging: one layer's routed experts in ggml layout (or a dense tensor, whichever is larger)
    const size_t dense = static_cast<size_t>(std::max(E, std::max(c.shared_ffn, H))) * (std::max(H, c.shared_ffn) / 32) * 34;
    const size_t one_expert = 2 * e->gate_bytes + e->down_bytes;
    e->staging_bytes = align_up(std::max(dense, one_expert * 8), 256);
    WD_TRY(cudaMalloc(&e->staging, e->staging_bytes));
    e->pinned_bytes = align_up(std::max<size_t>(one_expert, static_cast<size_t>(c.max_tokens) * H * 8), 256);
    WD_TRY(cudaMallocHost(&e->pinned, e->pinned_bytes));
    WD_TRY(cudaMallocHost(&e->host_status, 64));
    *e->host_status = 0u;
    if (!e->resident) {
        WD_TRY(cudaStreamCreateWithFlags(&e->copy_stream, cudaStreamNonBlocking));
        WD_TRY(cudaEventCreateWithFlags(&e->fill_done, cudaEventDisableTiming));
        WD_TRY(cudaMallocHost(&e->miss_pinned, one_expert * K));
        WD_TRY(cudaMalloc(&e->miss_staging, one_expert * K));
        WD_TRY(cudaMallocHost(&e->pinned_ids, sizeof(int) * K));
        WD_TRY(cudaMallocHost(&e->miss_info, sizeof(int) * (1 + static_cast<size_t>(std::max(c.n_layers, c.max_tokens)) * K)));
        e->copy_pool = new CopyPool(std::max(1, std::min(8, static_cast<int>(std::thread::hardware_concurrency()))));
    }
#undef WD_TRY

    wd::MoeParams &p = e->base;
    p.H = H; p.F = F; p.SF = c.shared_ffn; p.E = E; p.K = K;
    p.nsb_h = e->nsb_h; p.nsb_f = e->nsb_f;
    p.e_first = e->e_first; p.e_count = e->e_count;
    p.w_scale = c.w_scale; p.eps = c.rms_eps > 0 ? c.rms_eps : 1e-6f;
    p.inv_h = (H & (H - 1)) == 0 ? 1.0 / static_cast<double>(H) : 0.0;
    p.pool = e->pool; p.slot_bytes = e->slot_bytes;
    p.gate_off = 0; p.up_off = static_cast<unsigned>(e->gate_bytes); p.down_off = static_cast<unsigned>(2 * e->gate_bytes);
    p.grid_packed = e->grid_packed;
    p.grid2_packed = e->grid2_packed;
    p.gu_type = c.gate_type; p.d_type = c.down_type;
    p.gu_tile = wd::iq_tile_bytes(c.gate_type); p.d_tile = wd::iq_tile_bytes(c.down_type);
    p.ids = e->ids; p.weights = e->weights; p.routed = e->routed;
    p.t_logits = e->tagged + tw_logits; p.t_shared_act = e->tagged + tw_shact; p.t_shared_gate = e->tagged + tw_shgate;
    p.t_act = e->tagged + tw_act; p.t_expert_out = e->tagged + tw_eo; p.t_shared_down = e->tagged + tw_shdown;
    p.t_residual = e->tagged + tw_res; p.t_progress = e->tagged + tw_prog;
    e->tagged_eo_offset = tw_eo;
    e->tagged_left_offset = tw_left;
    p.t_peer_left = e->tagged + tw_left;
    p.n_peers = 0;
    p.sync = e->sync;
    p.host_status = e->host_status;
    { int t2 = F * e->nsb_h / 32, t3 = H * e->nsb_f / 32; p.t2_log2 = 0; while ((1 << p.t2_log2) < t2) ++p.t2_log2; p.t3_log2 = 0; while ((1 << p.t3_log2) < t3) ++p.t3_log2; }
    if ((rc = plan_shared_memory(e)) != WD_OK) return bail(rc);
    cudaError_t ae = cudaFuncSetAttribute(wd::moe_layer_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          static_cast<int>(e->smem_bytes));
    if (ae != cudaSuccess) {
        fail(WD_E_CUDA, std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(ae));
        return bail(WD_E_CUDA);
    }
    int occ = 0;
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, wd::moe_layer_kernel, wd::kThreads, e->smem_bytes);
    if (occ < 1) {
        fail(WD_E_INVALID, "the layer kernel does not fit one CTA per SM with this geometry");
        return bail(WD_E_INVALID);
    }
    if (c.shared_ffn > 0 && (e->fast_fn = find_fast_kernel(c)) != nullptr) {
        wd::FastParams &f = e->fbase;
        if ((rc = plan_fast(e)) != WD_OK) {
            e->fast_fn = nullptr;       // the generic kernel serves this grid
        } else {
            // CTAs per mailbox, measured on the 48-layer model (tok/s): 1 -> 827, 2 -> 865, 4 -> 894, 8 -> 907, 16 -> 914,
            // 37 -> 905, 148 (one shared copy that everybody polls) -> 845
            f.mbox_group = 16;
            if (const char *g = std::getenv("WD_MBOX_GROUP")) f.mbox_group = std::max(1, std::min(e->n_sm, std::atoi(g)));
            e->xbuf_words = static_cast<size_t>((e->n_sm + f.mbox_group - 1) / f.mbox_group) * f.xstride;
            cudaError_t fe = cudaMalloc(&e->xbuf, e->xbuf_words * sizeof(wd::tagged_t));
            if (fe == cudaSuccess) fe = cudaMemset(e->xbuf, 0, e->xbuf_words * sizeof(wd::tagged_t));
            if (fe == cudaSuccess) fe = cudaMalloc(&e->eo_plain, static_cast<size_t>(K) * H * 4);
            if (fe == cudaSuccess) fe = cudaMalloc(&e->shdown_plain, static_cast<size_t>(H) * 4);

            if (fe == cudaSuccess)
                fe = cudaFuncSetAttribute(e->fast_fn, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(e->fast_smem));
            if (fe != cudaSuccess) {
                fail(WD_E_CUDA, std::string("setting up the compiled layer kernel: ") + cudaGetErrorString(fe));
                return bail(WD_E_CUDA);
            }
            f.e_first = p.e_first; f.e_count = p.e_count; f.w_scale = p.w_scale; f.eps = p.eps;
            f.pool = p.pool; f.slot_bytes = p.slot_bytes; f.gate_off = p.gate_off; f.up_off = p.up_off; f.down_off = p.down_off;
            f.grid_packed = p.grid_packed;
            f.xbuf = e->xbuf;
            f.t_expert_out = p.t_expert_out; f.t_progress = p.t_progress;
            f.t_peer_left = p.t_peer_left; f.n_peers = 0;
            f.ids = p.ids; f.weights = p.weights; f.routed = p.routed;
            f.expert_out = e->eo_plain; f.shared_down = e->shdown_plain;
            f.sync = p.sync; f.host_status = p.host_status; f.fallbacks = e->fallbacks;
        }
        rc = WD_OK;
    }
    if (!e->fast_fn) plan_batch(e);
    if (e->batch_ok) {
        wd::BatchParams &b = e->bbase;
        const size_t Tm = static_cast<size_t>(c.max_tokens);
        auto up16 = [](size_t w) { return (w + 15) / 16 * 16; };
        const size_t w_logits = 0, w_shact = up16(w_logits + Tm * E), w_shgate = up16(w_shact + Tm * std::max(c.shared_ffn, 1)),
                     w_act = w_shgate + 16, w_eo = up16(w_act + Tm * K * F), w_shdown = up16(w_eo + Tm * K * H),
                     w_sel = up16(w_shdown + Tm * H), w_end = up16(w_sel + Tm * 2 * wd::kMaxK);
        cudaError_t be = cudaMalloc(&e->btagged, w_end * sizeof(wd::tagged_t));
        if (be == cudaSuccess) be = cudaMemset(e->btagged, 0, w_end * sizeof(wd::tagged_t));
        if (be == cudaSuccess)
            be = cudaFuncSetAttribute(wd::moe_batch_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(e->batch_smem));
        int bocc = 0;
        if (be == cudaSuccess) be = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&bocc, wd::moe_batch_kernel, wd::kThreads, e->batch_smem);
        if (be != cudaSuccess) {
            fail(WD_E_CUDA, std::string("setting up the batch kernel: ") + cudaGetErrorString(be));
            return bail(WD_E_CUDA);
        }
        if (bocc < 1) e->batch_ok = false;
        b.t_logits = e->btagged + w_logits; b.t_shact = e->btagged + w_shact; b.t_shgate = e->btagged + w_shgate;
        b.t_act = e->btagged + w_act; b.t_eo = e->btagged + w_eo; b.t_shdown = e->btagged + w_shdown;
        b.t_sel = e->btagged + w_sel;
    }
    *out = e;
    return WD_OK;
}

void wd_engine_destroy(wd_engine *e) {
    if (!e) return;
    cudaSetDevice(e->cfg.device);
    if (e->stream) cudaStreamSynchronize(e->stream);
    plain_destroy(e);
    wd_ep_disconnect(e);
    for (Layer &L : e->layers) {
        cudaFree(L.router); cudaFree(L.bias); cudaFree(L.gate_vec); cudaFree(L.sh_gate); cudaFree(L.sh_up);
        cudaFree(L.sh_down); cudaFree(L.norm); cudaFree(L.slot_of_expert);
        if (L.owned_host) cudaFreeHost(L.owned_host);
    }
    void *bufs[] = {e->pool, e->grid_packed, e->grid2_packed, e->synth_lut, e->sync, e->tagged, e->ids, e->weights, e->routed, e->tok_ids, e->tok_weights,
                    e->x_buf, e->out_buf, e->residual_buf, e->staging, e->stamps, e->layer_table, e->eo_plain, e->shdown_plain, e->fallbacks, e->xbuf, e->btagged};
    for (void *b : bufs) cudaFree(b);
    delete e->copy_pool;
    cudaFree(e->miss_staging);
    if (e->miss_pinned) cudaFreeHost(e->miss_pinned);
    if (e->pinned_ids) cudaFreeHost(e->pinned_ids);
    if (e->miss_info) cudaFreeHost(e->miss_info);
    if (e->fill_done) cudaEventDestroy(e->fill_done);
    if (e->copy_stream) cudaStreamDestroy(e->copy_stream);
    if (e->pinned) cudaFreeHost(e->pinned);
    if (e->host_status) cudaFreeHost(e->host_status);
    if (e->load_pinned) cudaFreeHost(e->load_pinned);
    cudaFree(e->load_staging);
    for (cudaEvent_t ev : e->load_done)
        if (ev) cudaEventDestroy(ev);
    if (e->stream) cudaStreamDestroy(e->stream);
    delete e;
}

int wd_set_router(wd_engine *e, int layer, const void *router_q8_0, const float *bias) {
    int rc = check_layer(e, layer);
    if (rc) return rc;
    if (!router_q8_0) return fail(WD_E_INVALID, "null router");
    if (e->cfg.router_f32) return fail(WD_E_STATE, "this engine was created for an F32 router: use wd_set_router_f32");
    WD_CUDA(cudaSetDevice(e->cfg.device));
    Layer &L = e->layers[layer];
    if ((rc = upload_repacked_q8(e, router_q8_0, e->cfg.n_experts, e->cfg.hidden, &L.router))) return rc;
    if (bias) {
        if ((rc = upload_f32(e, bias, e->cfg.n_experts, &L.bias))) return rc;
    }
    L.have_router = true;
    e->layer_table_dirty = true;
    return WD_OK;
}

int wd_set_router_f32(wd_engine *e, int layer, const float *router, const float *bias) {
    int rc = check_layer(e, layer);
    if (rc) return rc;
    if (!router) return fail(WD_E_INVALID, "null router");
    if (!e->plain || !e->cfg.router_f32) return fail(WD_E_STATE, "this engine was not created with router_f32 set");
    WD_CUDA(cudaSetDevice(e->cfg.device));
    if ((rc = upload_f32(e, router, static_cast<size_t>(e->cfg.n_experts) * e->cfg.hidden, &e->plain->layers[layer].router_f32))) return rc;
    if (bias && (rc = upload_f32(e, bias, e->cfg.n_experts, &e->layers[layer].bias))) return rc;
    e->layers[layer].have_router = true;
    return WD_OK;
}

int wd_set_shared(wd_engine *e, int layer, const float *gate_vec, const void *g, const void *u, const void *d) {
    int rc = check_layer(e, layer);
    if (rc) return rc;
    if (e->cfg.shared_ffn == 0) return fail(WD_E_STATE, "engine was created without a shared expert");
    if (!gate_vec || !g || !u || !d) return fail(WD_E_INVALID, "null shared expert tensor");
    WD_CUDA(cudaSetDevice(e->cfg.device));
    Layer &L = e->layers[layer];
    if ((rc = upload_f32(e, gate_vec, e->cfg.hidden, &L.gate_vec))) return rc;
    if ((rc = upload_repacked_q8(e, g, e->cfg.shared_ffn, e->cfg.hidden, &L.sh_gate))) return rc;
    if ((rc = upload_repacked_q8(e, u, e->cfg.shared_ffn, e->cfg.hidden, &L.sh_up))) return rc;
    if ((rc = upload_repacked_q8(e, d, e->cfg.hidden, e->cfg.shared_ffn, &L.sh_down))) return rc;
    L.have_shared = true;
    e->layer_table_dirty = true;
    return WD_OK;
}

int wd_set_norm(wd_engine *e, int layer, const float *weight) {
    int rc = check_layer(e, layer);
    if (rc) return rc;
    e->layer_table_dirty = true;
    WD_CUDA(cudaSetDevice(e->cfg.device));
    Layer &L = e->layers[layer];
    if (!weight) {
        cudaFree(L.norm);
        L.norm = nullptr;
        return WD_OK;
    }
    return upload_f32(e, weight, e->cfg.hidden, &L.norm);
}

static int fill_slot_from_host(wd_engine *e, int layer, int expert, int slot) {
    Layer &L = e->layers[layer];
    const size_t gb = e->gate_bytes, db = e->down_bytes;
    uint8_t *st = e->staging;
    // pageable or mapped host memory -> pinned bounce buffer -> device staging -> repack into the slot
    uint8_t *pin = static_cast<uint8_t *>(e->pinned);
    memcpy(pin, L.h_gate + static_cast<size_t>(expert) * gb, gb);
    memcpy(pin + gb, L.h_up + static_cast<size_t>(expert) * gb, gb);
    memcpy(pin + 2 * gb, L.h_down + static_cast<size_t>(expert) * db, db);
    WD_CUDA(cudaMemcpyAsync(st, pin, 2 * gb + db, cudaMemcpyHostToDevice, e->stream));
    int rc = repack_expert_into_slot(e, st, st + gb, st + 2 * gb, slot, e->stream);
    if (rc) return rc;
    WD_CUDA(cudaStreamSynchronize(e->stream));   // the bounce buffers are reused by the next fill
    return WD_OK;
}

static int bind_slot(wd_engine *e, int layer, int expert, int slot) {
    Layer &L = e->layers[layer];
    const int64_t old = e->slot_key[slot];
    if (old >= 0) {
        Layer &OL = e->layers[static_cast<int>(old >> 32)];
        const int oe = static_cast<int>(old & 0xffffffff);
        OL.h_slot[oe] = -1;
        const int minus1 = -1;
        WD_CUDA(cudaMemcpyAsync(OL.slot_of_expert + oe, &minus1, sizeof(int), cudaMemcpyHostToDevice, e->stream));
        e->key_slot.erase(old);
        ++e->evictions;
    }
    const int64_t key = (static_cast<int64_t>(layer) << 32) | static_cast<uint32_t>(expert);
    e->slot_key[slot] = key;
    e->key_slot[key] = slot;
    L.h_slot[expert] = slot;
    WD_CUDA(cudaMemcpyAsync(L.slot_of_expert + expert, &slot, sizeof(int), cudaMemcpyHostToDevice, e->stream));
    WD_CUDA(cudaStreamSynchronize(e->stream));
    return WD_OK;
}

// Every owned expert of a layer from host tensors (memory or file) into its slots, pipelined: host threads fill one
// pinned half-ring (memcpy, or pread for file-backed tensors) while the GPU copies and repacks the other
// (ExpertPreadPool + ExpertStagePath of the reference's load path, src/expert_cache.cuh:357-508, :1166-1254).
static constexpr int kLoadBatch = 8;

static int load_layer_resident(wd_engine *e, int layer) {
    Layer &L = e->layers[layer];
    const size_t gb = e->gate_bytes, db = e->down_bytes, one = 2 * gb + db;
    if (!e->load_pinned) {
        WD_CUDA(cudaMallocHost(&e->load_pinned, 2 * kLoadBatch * one));
        WD_CUDA(cudaMalloc(&e->load_staging, 2 * kLoadBatch * one));
        for (cudaEvent_t &ev : e->load_done) WD_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
        if (!e->copy_pool) e->copy_pool = new CopyPool(std::max(1, std::min(8, static_cast<int>(std::thread::hardware_concurrency()))));
    }
    cudaStream_t s = e->stream;
    const long long nb_gu = static_cast<long long>(e->cfg.expert_ffn) * e->nsb_h, nb_d = static_cast<long long>(e->cfg.hidden) * e->nsb_f;
    bool used[2] = {false, false};
    for (int x0 = 0, half = 0; x0 < e->e_count; x0 += kLoadBatch, half ^= 1) {
        const int n = std::min(kLoadBatch, e->e_count - x0);
        uint8_t *pin = e->load_pinned + static_cast<size_t>(half) * kLoadBatch * one;
        uint8_t *st = e->load_staging + static_cast<size_t>(half) * kLoadBatch * one;
        if (used[half]) WD_CUDA(cudaEventSynchronize(e->load_done[half]));     // the GPU is done with this half
        for (int m = 0; m < n; ++m) {
            const int x = e->e_first + x0 + m;
            uint8_t *to = pin + static_cast<size_t>(m) * one;
            const uint8_t *g = L.h_gate + static_cast<size_t>(x) * gb, *u = L.h_up + static_cast<size_t>(x) * gb,
                          *d = L.h_down + static_cast<size_t>(x) * db;
            const int fd = L.fd;
            const uint64_t fg = L.file_gate + static_cast<uint64_t>(x) * gb, fu = L.file_up + static_cast<uint64_t>(x) * gb,
                           fdn = L.file_down + static_cast<uint64_t>(x) * db;
            e->copy_pool->submit([=] {
                auto fetch = [&](uint8_t *dst, const uint8_t *from, uint64_t off, size_t bytes) {
                    size_t done = 0;
                    while (fd >= 0 && done < bytes) {
                        const ssize_t r = pread(fd, dst + done, bytes - done, static_cast<off_t>(off + done));
                        if (r <= 0) break;
                        done += static_cast<size_t>(r);
                    }
                    if (done < bytes) memcpy(dst + done, from + done, bytes - done);
                };
                fetch(to, g, fg, gb);
                fetch(to + gb, u, fu, gb);
                fetch(to + 2 * gb, d, fdn, db);
            });
        }
        e->copy_pool->wait_all();
        WD_CUDA(cudaMemcpyAsync(st, pin, static_cast<size_t>(n) * one, cudaMemcpyHostToDevice, s));
        uint8_t *dst = e->pool + static_cast<size_t>(layer * e->e_count + x0) * e->slot_bytes;
        const long long so = static_cast<long long>(one), sb = static_cast<long long>(e->slot_bytes);
        launch_repack_iq(e->cfg.gate_type, st, dst, nb_gu, so, sb, n, s);
        launch_repack_iq(e->cfg.gate_type, st + gb, dst + gb, nb_gu, so, sb, n, s);
        launch_repack_iq(e->cfg.down_type, st + 2 * gb, dst + 2 * gb, nb_d, so, sb, n, s);
        WD_CUDA(cudaGetLastError());
        WD_CUDA(cudaEventRecord(e->load_done[half], s));
        used[half] = true;
    }
    std::vector<int> slots(e->cfg.n_experts, -1);
    for (int x = 0; x < e->e_count; ++x) {
        const int expert = e->e_first + x, slot = layer * e->e_count + x;
        slots[expert] = slot;
        const int64_t key = (static_cast<int64_t>(layer) << 32) | static_cast<uint32_t>(expert);
        e->slot_key[slot] = key;
        e->key_slot[key] = slot;
    }
    L.h_slot = slots;
    WD_CUDA(cudaMemcpyAsync(L.slot_of_expert, slots.data(), slots.size() * sizeof(int), cudaMemcpyHostToDevice, s));
    WD_CUDA(cudaStreamSynchronize(s));
    return WD_OK;
}

static int set_experts_from(wd_engine *e, int layer, const void *gate, const void *up, const void *down, int fd,
                            uint64_t file_gate, uint64_t file_up, uint64_t file_down);

int wd_set_experts_typed(wd_engine *e, int layer, const void *gate, int gate_type, const void *up, int up_type,
                         const void *down, int down_type) {
    if (!e) return fail(WD_E_INVALID, "null engine");
    if (e->plain) return plain_set_experts(e, layer, gate, gate_type, up, up_type, down, down_type, cudaMemcpyHostToDevice);
    if (gate_type != e->cfg.gate_type || up_type != e->cfg.up_type || down_type != e->cfg.down_type)
        return fail(WD_E_INVALID, "this engine takes the tensor types it was created with in every layer");
    return wd_set_experts(e, layer, gate, up, down);
}

int wd_set_experts_fused(wd_engine *e, int layer, const void *gate_up, int gate_up_type, const void *down, int down_type) {
    if (!e) return fail(WD_E_INVALID, "null engine");
    if (!e->plain)
        return fail(WD_E_INVALID, "a fused gate_up tensor is taken by engines on the plain-layout path only; give the tiled kernels "
                                  "separate gate and up tensors");
    return plain_set_experts_fused(e, layer, gate_up, gate_up_type, down, down_type);
}

int wd_set_experts(wd_engine *e, int layer, const void *gate, const void *up, const void *down) {
    if (e && e->plain)
        return plain_set_experts(e, layer, gate, e->cfg.gate_type, up, e->cfg.up_type, down, e->cfg.down_type, cudaMemcpyHostToDevice);
    return set_experts_from(e, layer, gate, up, down, -1, 0, 0, 0);
}

// fd >= 0: the tensors are also readable from that file at the given offsets (positional reads instead of copies
// out of a mapping)
static int set_experts_from(wd_engine *e, int layer, const void *gate, const void *up, const void *down, int fd,
                            uint64_t file_gate, uint64_t file_up, uint64_t file_down) {
    int rc = check_layer(e, layer);
    if (rc) return rc;
    if (!gate || !up || !down) return fail(WD_E_INVALID, "null expert tensor");
    WD_CUDA(cudaSetDevice(e->cfg.device));
    Layer &L = e->layers[layer];
    L.h_gate = static_cast<const uint8_t *>(gate);
    L.h_up = static_cast<const uint8_t *>(up);
    L.h_down = static_cast<const uint8_t *>(down);
    L.have_experts = true;
    L.fd = fd;
    L.file_gate = file_gate;
    L.file_up = file_up;
    L.file_down = file_down;
    {
        cudaPointerAttributes at{};
        L.host_pinned = true;
        for (const void *q : {gate, up, down}) {
            if (cudaPointerGetAttributes(&at, q) != cudaSuccess || at.type != cudaMemoryTypeHost) L.host_pinned = false;
        }
        cudaGetLastError();
    }
    e->layer_table_dirty = true;
    if (e->resident) return load_layer_resident(e, layer);
    return WD_OK;
}

int wd_set_experts_device(wd_engine *e, int layer, const void *gate, const void *up, const void *down) {
    if (e && e->plain)
        return plain_set_experts(e, layer, gate, e->cfg.gate_type, up, e->cfg.up_type, down, e->cfg.down_type, cudaMemcpyDeviceToDevice);
    int rc = check_layer(e, layer);
    if (rc) return rc;
    if (!e->resident) return fail(WD_E_STATE, "device-side expert upload needs a pool that holds every owned expert");
    WD_CUDA(cudaSetDevice(e->cfg.device));
    Layer &L = e->layers[layer];
    const uint8_t *g = static_cast<const uint8_t *>(gate), *u = static_cast<const uint8_t *>(up),
                  *d = static_cast<const uint8_t *>(down);
    std::vector<int> slots(e->cfg.n_experts, -1);
    {
        // the owned experts of a layer occupy consecutive slots: three launches repack them all
        const int slot0 = layer * e->e_count;
        uint8_t *dst = e->pool + static_cast<size_t>(slot0) * e->slot_bytes;
        const long long nb_gu = static_cast<long long>(e->cfg.expert_ffn) * e->nsb_h;
        const long long nb_d = static_cast<long long>(e->cfg.hidden) * e->nsb_f;
        const long long gb = static_cast<long long>(e->gate_bytes), db = static_cast<long long>(e->down_bytes);
        const long long sb = static_cast<long long>(e->slot_bytes);
        launch_repack_iq(e->cfg.gate_type, g + e->e_first * gb, dst, nb_gu, gb, sb, e->e_count, e->stream);
        launch_repack_iq(e->cfg.gate_type, u + e->e_first * gb, dst + gb, nb_gu, gb, sb, e->e_count, e->stream);
        launch_repack_iq(e->cfg.down_type, d + e->e_first * db, dst + 2 * gb, nb_d, db, sb, e->e_count, e->stream);
        WD_CUDA(cudaGetLastError());
    }
    for (int x = 0; x < e->e_count; ++x) {
        const int expert = e->e_first + x, slot = layer * e->e_count + x;
        slots[expert] = slot;
        const int64_t key = (static_cast<int64_t>(layer) << 32) | static_cast<uint32_t>(expert);
        e->slot_key[slot] = key;
        e->key_slot[key] = slot;
    }
    L.h_slot = slots;
    WD_CUDA(cudaMemcpyAsync(L.slot_of_expert, slots.data(), slots.size() * sizeof(int), cudaMemcpyHostToDevice, e->stream));
    WD_CUDA(cudaStreamSynchronize(e->stream));
    L.have_experts = true;
    return WD_OK;
}

int64_t wd_cache_slot_count(const wd_engine *e) { return e ? e->n_slots : 0; }
int64_t wd_cache_slot_bytes(const wd_engine *e) { return e ? static_cast<int64_t>(e->slot_bytes) : 0; }

int wd_cache_acquire(wd_engine *e, int layer, int expert, int *slot_out) {
    WD_TILED_ONLY(e);
    int rc = check_layer(e, layer);
    if (rc) return rc;
    if (expert < e->e_first || expert >= e->e_first + e->e_count)
        return fail(WD_E_INVALID, "expert is not owned by this rank");
    WD_CUDA(cudaSetDevice(e->cfg.device));
    Layer &L = e->layers[layer];
    int slot = L.h_slot[expert];
    if (slot >= 0) {
        ++e->hits;
        touch_slot(e, slot);
    } else {
        if (!L.h_gate) return fail(WD_E_STATE, "no host tensors to fill the slot from");
        ++e->misses;
        slot = e->lru.back();
        if ((rc = fill_slot_from_host(e, layer, expert, slot))) return rc;
        if ((rc = bind_slot(e, layer, expert, slot))) return rc;
        touch_slot(e, slot);
    }
    if (slot_out) *slot_out = slot;
    return WD_OK;
}

int wd_cache_stream_stats(const wd_engine *e, int64_t stats[3]) {
    if (!e || !stats) return fail(WD_E_INVALID, "null argument");
    stats[0] = e->h2d_bytes; stats[1] = e->fill_host_ns; stats[2] = e->acquires;
    return WD_OK;
}

int wd_cache_stats(const wd_engine *e, int64_t stats[3]) {
    if (!e || !stats) return fail(WD_E_INVALID, "null argument");
    stats[0] = e->hits; stats[1] = e->misses; stats[2] = e->evictions;
    return WD_OK;
}

// A batch of tokens (speculative verify, Qwen38MoeTokenBatch::run, src/qwen38_moe.cuh:2955): pair (t, j) uses expert
// ids[t][j] on the activation of token t and each token's rows are combined in its own rank order, exactly as a
// single-token call. With every expert resident the whole batch is ONE launch of the layer kernel, which walks the
// tokens the way a stack launch walks layers (the next token's router and shared rows travel during the current
// token's down phase; router, shared expert and repeated experts of tokens 1.. come from L2). A capped cache still
// takes the tokens one at a time, because the host places each token's experts between its two passes.
int wd_moe_forward(wd_engine *e, int layer, const float *x_dev, float *out_dev, int n_tokens, void *stream) {
    int rc = check_layer(e, layer);
    if (rc) return rc;
    if (n_tokens < 1 || n_tokens > e->cfg.max_tokens) return fail(WD_E_INVALID, "n_tokens must be 1..max_tokens");
    if (!x_dev || !out_dev) return fail(WD_E_INVALID, "null buffer");
    WD_CUDA(cudaSetDevice(e->cfg.device));
    cudaStream_t s = stream ? static_cast<cudaStream_t>(stream) : e->stream;
    if (e->plain) return plain_forward(e, layer, x_dev, out_dev, n_tokens, s);
    const int H = e->cfg.hidden, K = e->cfg.top_k;
    // (with profiling on, a one-token call stays on the layer kernel, whose phase stamps the caller is asking for)
    if (e->batch_ok && e->n_peers == 0 && reinterpret_cast<uintptr_t>(x_dev) % 16 == 0) {
        if (!e->resident && n_tokens > 1) return forward_capped_batch(e, layer, x_dev, out_dev, n_tokens, s);
        if (e->resident && (n_tokens > 1 || (e->batch_single && !e->profiling))) return launch_batch(e, layer, x_dev, out_dev, n_tokens, s);
    }
    if (e->resident && !e->fast_fn && n_tokens > 1) {
        rc = launch_layers(e, layer, layer + 1, x_dev, nullptr, out_dev, s, false, n_tokens);
        if (rc) return rc;
        e->last_tokens = n_tokens;
        return WD_OK;
    }
    for (int t = 0; t < n_tokens; ++t) {
        const float *x = x_dev + static_cast<size_t>(t) * H;
        float *out = out_dev + static_cast<size_t>(t) * H;
        rc = e->resident ? launch_layer(e, layer, x, nullptr, out, s) : forward_capped(e, layer, x, nullptr, out, s);
        if (rc) return rc;
        WD_CUDA(cudaMemcpyAsync(e->tok_ids + t * K, e->ids, K * 4, cudaMemcpyDeviceToDevice, s));
        WD_CUDA(cudaMemcpyAsync(e->tok_weights + t * K, e->weights, K * 4, cudaMemcpyDeviceToDevice, s));
    }
    e->last_tokens = n_tokens;
    return WD_OK;
}

int wd_moe_forward_host(wd_engine *e, int layer, const float *x_host, float *out_host, int n_tokens) {
    int rc = check_layer(e, layer);
    if (rc) return rc;
    if (n_tokens < 1 || n_tokens > e->cfg.max_tokens) return fail(WD_E_INVALID, "n_tokens must be 1..max_tokens");
    if (!x_host || !out_host) return fail(WD_E_INVALID, "null buffer");
    const size_t n = static_cast<size_t>(e->cfg.hidden) * n_tokens, bytes = n * 4;
    WD_CUDA(cudaSetDevice(e->cfg.device));
    float *pin = static_cast<float *>(e->pinned);
    memcpy(pin, x_host, bytes);
    WD_CUDA(cudaMemcpyAsync(e->x_buf, pin, bytes, cudaMemcpyHostToDevice, e->stream));
    if ((rc = wd_moe_forward(e, layer, e->x_buf, e->out_buf, n_tokens, e->stream))) return rc;
    WD_CUDA(cudaMemcpyAsync(pin + n, e->out_buf, bytes, cudaMemcpyDeviceToHost, e->stream));
    WD_CUDA(cudaStreamSynchronize(e->stream));
    memcpy(out_host, pin + n, bytes);
    return check_device_status(e);
}

int wd_stack_step(wd_engine *e, float *residual_dev, void *stream) {
    if (!e || !residual_dev) return fail(WD_E_INVALID, "null argument");
    WD_CUDA(cudaSetDevice(e->cfg.device));
    cudaStream_t s = stream ? static_cast<cudaStream_t>(stream) : e->stream;
    if (e->plain) return plain_stack_step(e, residual_dev, s);
    if (!e->resident && !e->fast_fn && e->n_peers == 0)
        return run_capped_optimistic(e, 0, e->cfg.n_layers, nullptr, residual_dev, e->out_buf, s);
    if (!e->resident) {     // layer by layer: the host places the selected experts between the two passes
        for (int l = 0; l < e->cfg.n_layers; ++l) {
            int rc = forward_capped(e, l, nullptr, residual_dev, e->out_buf, s);
            if (rc) return rc;
        }
        return WD_OK;
    }
    return launch_layers(e, 0, e->cfg.n_layers, nullptr, residual_dev, e->out_buf, s);
}

int wd_stack_step_host(wd_engine *e, const float *in_host, float *out_host) {
    if (!e || !in_host || !out_host) return fail(WD_E_INVALID, "null argument");
    const size_t bytes = static_cast<size_t>(e->cfg.hidden) * 4;
    WD_CUDA(cudaSetDevice(e->cfg.device));
    float *pin = static_cast<float *>(e->pinned);
    memcpy(pin, in_host, bytes);
    WD_CUDA(cudaMemcpyAsync(e->residual_buf, pin, bytes, cudaMemcpyHostToDevice, e->stream));
    int rc = wd_stack_step(e, e->residual_buf, e->stream);
    if (rc) return rc;
    WD_CUDA(cudaMemcpyAsync(pin + e->cfg.hidden, e->residual_buf, bytes, cudaMemcpyDeviceToHost, e->stream));
    WD_CUDA(cudaStreamSynchronize(e->stream));
    memcpy(out_host, pin + e->cfg.hidden, bytes);
    // the last CTA of every launch leaves the status word in pinned host memory: no copy to read it.
    // (Letting the kernel read and write the residual in pinned memory directly was measured slower: every CTA
    // fetches the whole vector over PCIe.)
    if (!e->plain && *e->host_status == 0u) return WD_OK;
    return check_device_status(e);
}

// The compiled kernel's act values, from CTA 0's mailbox: row jl there is the jl-th OWNED selected expert. Rows of
// experts another rank owns come back as zeros.
static int read_fast_act(wd_engine *e, float *dst, size_t bytes) {
    const wd_config &c = e->cfg;
    const int K = c.top_k, F = c.expert_ffn;
    if (bytes < static_cast<size_t>(K) * F * 4) return fail(WD_E_INVALID, "tap buffer too small");
    WD_CUDA(cudaStreamSynchronize(e->stream));
    WD_CUDA(cudaDeviceSynchronize());
    const size_t words = static_cast<size_t>(K) * F;
    std::vector<wd::tagged_t> w(words);
    std::vector<int> ids(K);
    const size_t o_act = 2ull * c.n_experts + 2ull * c.shared_ffn + 32 + 2ull * c.hidden;       // inside a mailbox
    WD_CUDA(cudaMemcpy(w.data(), e->xbuf + o_act + static_cast<size_t>(e->last_parity) * words, words * sizeof(wd::tagged_t),
                       cudaMemcpyDeviceToHost));
    WD_CUDA(cudaMemcpy(ids.data(), e->ids, K * sizeof(int), cudaMemcpyDeviceToHost));
    int jl = 0;
    for (int j = 0; j < K; ++j) {
        const bool owned = ids[j] >= e->e_first && ids[j] < e->e_first + e->e_count;
        for (int f = 0; f < F; ++f) {
            const uint32_t v = owned ? static_cast<uint32_t>(w[static_cast<size_t>(jl) * F + f]) : 0u;
            memcpy(dst + static_cast<size_t>(j) * F + f, &v, 4);
        }
        jl += owned ? 1 : 0;
    }
    return WD_OK;
}

int wd_read_tap(wd_engine *e, int tap, int token, void *dst, size_t bytes) {
    if (!e || !dst) return fail(WD_E_INVALID, "null argument");
    if (token == -1) token = e->last_tokens - 1;     // the last token of the last call
    if (token < 0 || token >= e->last_tokens) return fail(WD_E_INVALID, "token out of range");
    if (e->plain) {
        WD_CUDA(cudaSetDevice(e->cfg.device));
        return plain_read_tap(e, tap, token, dst, bytes);
    }
    const bool per_launch = tap == WD_TAP_STAMPS || tap == WD_TAP_FALLBACKS;     // not tied to a token
    // the token walk of the layer kernel keeps ids and weights of every token and everything else of the last one; the batch
    // kernel keeps everything of every token except the routed sum (last token only)
    if (token != e->last_tokens - 1 && !per_launch &&
        (e->last_batch ? tap == WD_TAP_ROUTED : (tap != WD_TAP_IDS && tap != WD_TAP_WEIGHTS)))
        return fail(WD_E_STATE, "only the ids and weights of earlier tokens of a batch are kept; other taps show its last token");
    WD_CUDA(cudaSetDevice(e->cfg.device));
    const wd_config &c = e->cfg;
    const wd::MoeParams &p = e->base;
    const size_t par = static_cast<size_t>(e->last_parity);
    const void *src = nullptr;              // plain buffer
    const wd::tagged_t *tsrc = nullptr;     // or tagged words of the last layer's half
    size_t n = 0;
    if (e->last_batch && !per_launch && tap != WD_TAP_ROUTED) {       // the batch kernel's exchange words, [token][...]
        const wd::BatchParams &b = e->bbase;
        const size_t t = static_cast<size_t>(token);
        switch (tap) {
            case WD_TAP_LOGITS: tsrc = b.t_logits + t * c.n_experts; n = c.n_experts * 4; break;
            case WD_TAP_IDS: src = e->tok_ids + t * c.top_k; n = c.top_k * 4; break;
            case WD_TAP_WEIGHTS: src = e->tok_weights + t * c.top_k; n = c.top_k * 4; break;
            case WD_TAP_ACT: n = static_cast<size_t>(c.top_k) * c.expert_ffn * 4; tsrc = b.t_act + t * (n / 4); break;
            case WD_TAP_EXPERT_OUT: n = static_cast<size_t>(c.top_k) * c.hidden * 4; tsrc = b.t_eo + t * (n / 4); break;
            case WD_TAP_SHARED: tsrc = b.t_shdown + t * c.hidden; n = c.hidden * 4; break;
            case WD_TAP_SHARED_GATE: tsrc = b.t_shgate + t; n = 4; break;
            case WD_TAP_SHARED_ACT: tsrc = b.t_shact + t * c.shared_ffn; n = static_cast<size_t>(c.shared_ffn) * 4; break;
            default: return fail(WD_E_INVALID, "unknown tap");
        }
    } else
    switch (tap) {
        case WD_TAP_LOGITS:      // the compiled kernel: CTA 0's mailbox ([2][E] logits | [2][SF] shared act | [2][16] gate | ..)
            tsrc = e->fast_fn ? e->xbuf + par * c.n_experts : p.t_logits + par * c.n_experts;
            n = c.n_experts * 4;
            break;
        case WD_TAP_IDS:
            src = e->last_tokens > 1 ? e->tok_ids + token * c.top_k : e->ids;
            n = c.top_k * 4;
            break;
        case WD_TAP_WEIGHTS:
            src = e->last_tokens > 1 ? e->tok_weights + token * c.top_k : e->weights;
            n = c.top_k * 4;
            break;
        case WD_TAP_ACT:
            n = static_cast<size_t>(c.top_k) * c.expert_ffn * 4;
            if (e->fast_fn) return read_fast_act(e, static_cast<float *>(dst), bytes);
            tsrc = p.t_act + par * (n / 4);
            break;
        case WD_TAP_EXPERT_OUT:
            n = static_cast<size_t>(c.top_k) * c.hidden * 4;
            if (e->fast_fn) src = e->eo_plain;
            else tsrc = p.t_expert_out + par * (n / 4);
            break;
        case WD_TAP_ROUTED: src = e->routed; n = c.hidden * 4; break;
        case WD_TAP_SHARED:
            if (e->fast_fn) src = e->shdown_plain;
            else tsrc = p.t_shared_down + par * c.hidden;
            n = c.hidden * 4;
            break;
        case WD_TAP_FALLBACKS: src = e->fallbacks; n = 4; break;
        case WD_TAP_SHARED_GATE:
            tsrc = e->fast_fn ? e->xbuf + 2 * c.n_experts + 2 * c.shared_ffn + par * 16 : p.t_shared_gate + par;
            n = 4;
            break;
        case WD_TAP_SHARED_ACT:
            tsrc = e->fast_fn ? e->xbuf + 2 * c.n_experts + par * c.shared_ffn : p.t_shared_act + par * std::max(c.shared_ffn, 1);
            n = static_cast<size_t>(c.shared_ffn) * 4;
            break;
        case WD_TAP_STAMPS: src = e->stamps; n = static_cast<size_t>(e->n_sm) * wd::kStampStride * 8; break;
        default: return fail(WD_E_INVALID, "unknown tap");
    }
    if (bytes < n) return fail(WD_E_INVALID, "tap buffer too small");
    WD_CUDA(cudaStreamSynchronize(e->stream));
    WD_CUDA(cudaDeviceSynchronize());
    if (tsrc) {     // drop the tags
        std::vector<wd::tagged_t> words(n / 4);
        WD_CUDA(cudaMemcpy(words.data(), tsrc, words.size() * sizeof(wd::tagged_t), cudaMemcpyDeviceToHost));
        uint32_t *o = static_cast<uint32_t *>(dst);
        for (size_t i = 0; i < words.size(); ++i) o[i] = static_cast<uint32_t>(words[i]);
    } else {
        WD_CUDA(cudaMemcpy(dst, src, n, cudaMemcpyDeviceToHost));
    }
    return WD_OK;
}

int wd_set_profiling(wd_engine *e, int on) {
    WD_TILED_ONLY(e);
    if (!e) return fail(WD_E_INVALID, "null engine");
    e->profiling = on != 0;
    e->stamp_layer = on > 1 ? on - 1 : 0;   // on = 1 + offset of the profiled layer within a launch
    return WD_OK;
}

int wd_sm_count(const wd_engine *e) { return e ? e->n_sm : 0; }
// Cycles one SM needs for a round of `warps` IQ3_S tiles resident in shared memory (see iq3_decoder_rate_kernel).
int wd_measure_tile_decoder(int device, int nsb, int warps, int unroll, double *cycles_per_round) {
    if (!cycles_per_round || warps < 1 || warps > wd::kWarps || (unroll != 1 && unroll != 8) || nsb < 1 || nsb > 32 || (32 % nsb) != 0)
        return fail(WD_E_INVALID, "tile decoder measurement: warps 1..16, unroll 1 or 8, nsb a power of two up to 32");
    WD_CUDA(cudaSetDevice(device));
    int n_sm = 0;
    WD_CUDA(cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, device));
    ScopedDev hold;
    uint16_t *grid = nullptr;
    unsigned long long *cyc = nullptr;
    float *sink = nullptr;
    WD_CUDA(hold.alloc(&grid, sizeof(wd_iq3s_grid_packed)));
    WD_CUDA(hold.alloc(&cyc, static_cast<size_t>(n_sm) * sizeof(unsigned long long)));
    WD_CUDA(hold.alloc(&sink, static_cast<size_t>(n_sm) * wd::kThreads * sizeof(float)));
    WD_CUDA(upload_sync(grid, wd_iq3s_grid_packed, sizeof(wd_iq3s_grid_packed)));
    const size_t sm = wd::kGridTableBytes + 16 * wd::kIq3TileBytes + 32 * wd::kActSbStride + 128 + static_cast<size_t>(wd::kWarps) * 640 * 4;
    const int iters = 200;
    auto fn = unroll == 8 ? wd::iq3_decoder_rate_kernel<8> : wd::iq3_decoder_rate_kernel<1>;
    WD_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sm)));
    for (int rep = 0; rep < 2; ++rep) fn<<<n_sm, wd::kThreads, sm>>>(grid, nsb, iters, warps, cyc, sink);
    WD_CUDA(cudaDeviceSynchronize());
    std::vector<unsigned long long> h(n_sm);
    WD_CUDA(cudaMemcpy(h.data(), cyc, h.size() * sizeof(h[0]), cudaMemcpyDeviceToHost));
    std::sort(h.begin(), h.end());
    *cycles_per_round = static_cast<double>(h[h.size() / 2]) / iters;
    return WD_OK;
}

const char *wd_kernel_name(const wd_engine *e) {
    if (e && e->plain) return "plain_gate_up_kernel";     // the longest of the seven kernels of a plain-layout call
    return e && e->fast_fn ? "moe_fast_kernel" : "moe_layer_kernel";
}
const char *wd_last_kernel_name(const wd_engine *e) { return e && e->last_batch ? "moe_batch_kernel" : wd_kernel_name(e); }
const char *wd_batch_kernel_name(const wd_engine *e) { return e && e->batch_ok ? "moe_batch_kernel" : wd_kernel_name(e); }

// ---- expert parallelism ----------------------------------------------------------------------------
int wd_ep_handle_bytes(void) { return static_cast<int>(sizeof(cudaIpcMemHandle_t)); }

int wd_ep_export(wd_engine *e, void *handle_out) {
    WD_TILED_ONLY(e);
    if (!e || !handle_out) return fail(WD_E_INVALID, "null argument");
    WD_CUDA(cudaSetDevice(e->cfg.device));
    cudaIpcMemHandle_t h;
    WD_CUDA(cudaIpcGetMemHandle(&h, e->tagged));
    memcpy(handle_out, &h, sizeof(h));
    return WD_OK;
}

namespace {
// the compiled kernel's parameter block carries the same peer pointers
void mirror_peers(wd_engine *e) {
    for (int p = 0; p < 8; ++p) {
        e->fbase.peer_expert_out[p] = e->base.peer_expert_out[p];
        e->fbase.peer_left_out[p] = e->base.peer_left_out[p];
        e->fbase.peer_rank[p] = e->base.peer_rank[p];
    }
    e->fbase.n_peers = e->base.n_peers;
}

int ep_check_connect(wd_engine *e, int n_peers) {
    if (!e) return fail(WD_E_INVALID, "null engine");
    if (n_peers != e->cfg.ep_size - 1) return fail(WD_E_INVALID, "expected ep_size - 1 peers");
    if (n_peers > 7) return fail(WD_E_INVALID, "at most 8 expert-parallel ranks");
    if (e->n_peers) return fail(WD_E_STATE, "already connected");
    return WD_OK;
}
}  // namespace

int wd_ep_connect(wd_engine *e, int n_peers, const void *handles) {
    WD_TILED_ONLY(e);
    int rc = ep_check_connect(e, n_peers);
    if (rc) return rc;
    if (n_peers > 0 && !handles) return fail(WD_E_INVALID, "null handles");
    WD_CUDA(cudaSetDevice(e->cfg.device));
    WD_CUDA(cudaDeviceSynchronize());
    for (int p = 0; p < n_peers; ++p) {
        cudaIpcMemHandle_t h;
        memcpy(&h, static_cast<const uint8_t *>(handles) + static_cast<size_t>(p) * sizeof(h), sizeof(h));
        void *base = nullptr;
        cudaError_t ce = cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess);
        if (ce != cudaSuccess) {
            for (int q = 0; q < p; ++q) cudaIpcCloseMemHandle(e->peer_mapped[q]);
            return fail(WD_E_CUDA, std::string("cudaIpcOpenMemHandle: ") + cudaGetErrorString(ce));
        }
        e->peer_mapped[p] = base;
        e->base.peer_expert_out[p] = static_cast<wd::tagged_t *>(base) + e->tagged_eo_offset;
        // peers are the other ranks in rank order; each peer keeps one "left layer" word per global rank
        e->base.peer_rank[p] = p < e->cfg.ep_rank ? p : p + 1;
        e->base.peer_left_out[p] = static_cast<wd::tagged_t *>(base) + e->tagged_left_offset + e->cfg.ep_rank;
    }
    e->n_peers = e->base.n_peers = n_peers;
    mirror_peers(e);
    return WD_OK;
}

int wd_ep_connect_local(wd_engine *e, int n_peers, wd_engine *const *peers) {
    WD_TILED_ONLY(e);
    int rc = ep_check_connect(e, n_peers);
    if (rc) return rc;
    if (n_peers > 0 && !peers) return fail(WD_E_INVALID, "null peers");
    WD_CUDA(cudaSetDevice(e->cfg.device));
    for (int p = 0; p < n_peers; ++p) {
        const wd_engine *o = peers[p];
        if (!o || o == e || o->tagged_words != e->tagged_words || o->cfg.ep_size != e->cfg.ep_size)
            return fail(WD_E_INVALID, "peer engines must be distinct and share the geometry");
        if (o->cfg.device != e->cfg.device) {
            int can = 0;
            WD_CUDA(cudaDeviceCanAccessPeer(&can, e->cfg.device, o->cfg.device));
            if (!can) return fail(WD_E_STATE, "no peer access between the two devices");
            cudaError_t ce = cudaDeviceEnablePeerAccess(o->cfg.device, 0);
            if (ce == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();
            else if (ce != cudaSuccess) return fail(WD_E_CUDA, std::string("cudaDeviceEnablePeerAccess: ") + cudaGetErrorString(ce));
        }
        e->peer_mapped[p] = nullptr;
        e->base.peer_expert_out[p] = o->tagged + o->tagged_eo_offset;
        e->base.peer_rank[p] = o->cfg.ep_rank;
        e->base.peer_left_out[p] = o->tagged + o->tagged_left_offset + e->cfg.ep_rank;
    }
    e->n_peers = e->base.n_peers = n_peers;
    mirror_peers(e);
    return WD_OK;
}

int wd_ep_disconnect(wd_engine *e) {
    if (!e) return fail(WD_E_INVALID, "null engine");
    if (!e->n_peers) return WD_OK;
    cudaSetDevice(e->cfg.device);
    cudaDeviceSynchronize();
    for (int p = 0; p < e->n_peers; ++p) {
        if (e->peer_mapped[p]) cudaIpcCloseMemHandle(e->peer_mapped[p]);
        e->peer_mapped[p] = nullptr;
        e->base.peer_expert_out[p] = nullptr;
        e->base.peer_left_out[p] = nullptr;
    }
    e->n_peers = e->base.n_peers = 0;
    mirror_peers(e);
    return WD_OK;
}

int wd_reset_exchange(wd_engine *e) {
    WD_TILED_ONLY(e);
    if (!e) return fail(WD_E_INVALID, "null engine");
    WD_CUDA(cudaSetDevice(e->cfg.device));
    WD_CUDA(cudaDeviceSynchronize());
    WD_CUDA(cudaMemset(e->sync, 0, 8192));
    WD_CUDA(cudaMemset(e->tagged, 0, e->tagged_words * sizeof(wd::tagged_t)));
    if (e->xbuf) WD_CUDA(cudaMemset(e->xbuf, 0, e->xbuf_words * sizeof(wd::tagged_t)));
    WD_CUDA(cudaDeviceSynchronize());           // the next launch runs on a stream that is not ordered behind these
    e->epoch = 0;
    return WD_OK;
}

int wd_device_status(wd_engine *e, int *status) {
    if (!e || !status) return fail(WD_E_INVALID, "null argument");
    WD_CUDA(cudaSetDevice(e->cfg.device));
    WD_CUDA(cudaDeviceSynchronize());
    unsigned st = 0;
    WD_CUDA(cudaMemcpy(&st, e->sync + 2, sizeof(st), cudaMemcpyDeviceToHost));
    *status = static_cast<int>(st);
    if (st) {
        WD_CUDA(cudaMemset(e->sync, 0, 8192));
        WD_CUDA(cudaMemset(e->tagged, 0, e->tagged_words * sizeof(wd::tagged_t)));
        if (e->xbuf) WD_CUDA(cudaMemset(e->xbuf, 0, e->xbuf_words * sizeof(wd::tagged_t)));
        WD_CUDA(cudaDeviceSynchronize());       // the next launch runs on a stream that is not ordered behind these
        e->epoch = 0;
    }
    return WD_OK;
}

// ---- stand-alone pieces -------------------------------------------------------------------------
int wd_router_topk_host(const float *logits, int n_experts, int k, float w_scale, int *ids, float *weights,
                        float *probs) {
    if (!logits || !ids || !weights) return fail(WD_E_INVALID, "null argument");
    if (n_experts <= 0 || n_experts % 8 || n_experts > wd::kMaxExperts || k < 1 || k > wd::kMaxK)
        return fail(WD_E_INVALID, "n_experts must be a multiple of 8 up to 1024, k 1..16");
    ScopedDev bufs;
    float *d_l = nullptr, *d_w = nullptr, *d_p = nullptr;
    int *d_i = nullptr;
    WD_CUDA(bufs.alloc(&d_l, n_experts * 4));
    WD_CUDA(bufs.alloc(&d_p, n_experts * 4));
    WD_CUDA(bufs.alloc(&d_w, wd::kMaxK * 4));
    WD_CUDA(bufs.alloc(&d_i, wd::kMaxK * 4));
    WD_CUDA(upload_sync(d_l, logits, n_experts * 4));
    wd::test_router_kernel<<<1, wd::kThreads>>>(d_l, n_experts, k, w_scale, d_i, d_w, d_p);
    WD_CUDA(cudaGetLastError());
    WD_CUDA(cudaDeviceSynchronize());
    WD_CUDA(cudaMemcpy(ids, d_i, k * 4, cudaMemcpyDeviceToHost));
    WD_CUDA(cudaMemcpy(weights, d_w, k * 4, cudaMemcpyDeviceToHost));
    if (probs) WD_CUDA(cudaMemcpy(probs, d_p, n_experts * 4, cudaMemcpyDeviceToHost));
    return WD_OK;
}

static int quantize_host(const float *x, int n, void *q80, void *q8k) {
    if (!x || n <= 0 || n % 256 || n > 8192) return fail(WD_E_INVALID, "n must be a multiple of 256 up to 8192");
    ScopedDev bufs;
    float *d_x = nullptr;
    uint8_t *d_0 = nullptr, *d_k = nullptr;
    WD_CUDA(bufs.alloc(&d_x, n * 4));
    WD_CUDA(upload_sync(d_x, x, n * 4));
    if (q80) WD_CUDA(bufs.alloc(&d_0, n / 32 * 34));
    if (q8k) WD_CUDA(bufs.alloc(&d_k, n / 256 * 292));
    const size_t smem = n * 4 + n + n / 32 * 4 + (n / 256 + 1) * wd::kActSbStride + (n / 256 + 4) * 4 + 64;
    WD_CUDA(cudaFuncSetAttribute(wd::test_quantize_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024));
    wd::test_quantize_kernel<<<1, 512, smem>>>(d_x, n, d_0, d_k);
    WD_CUDA(cudaGetLastError());
    WD_CUDA(cudaDeviceSynchronize());
    if (q80) WD_CUDA(cudaMemcpy(q80, d_0, n / 32 * 34, cudaMemcpyDeviceToHost));
    if (q8k) WD_CUDA(cudaMemcpy(q8k, d_k, n / 256 * 292, cudaMemcpyDeviceToHost));
    return WD_OK;
}
int wd_quantize_q8_0_host(const float *x, int n, void *blocks) { return quantize_host(x, n, blocks, nullptr); }
int wd_quantize_q8_K_host(const float *x, int n, void *blocks) { return quantize_host(x, n, nullptr, blocks); }

int wd_matvec_host(int type, const void *w, int rows, int cols, const float *x, float *y, int32_t *partials) {
    if (!w || !x || !y) return fail(WD_E_INVALID, "null argument");
    ScopedDev bufs;
    float *d_x = nullptr, *d_y = nullptr;
    uint8_t *d_src = nullptr, *d_dst = nullptr;
    int *d_p = nullptr;
    uint16_t *d_grid = nullptr;
    if (type == WD_TYPE_IQ3_S || type == WD_TYPE_IQ2_S) {
        const int nsb = cols / 256;
        if (cols % 256 || !pow2(nsb) || nsb > 32 || rows % (32 / nsb))
            return fail(WD_E_INVALID, "IQ3_S / IQ2_S matvec: cols must be 256*2^n (n<=5), rows a multiple of 32/(cols/256)");
        const bool iq2 = type == WD_TYPE_IQ2_S;
        const size_t bytes = static_cast<size_t>(rows) * nsb * wd::iq_block_bytes(type);
        WD_CUDA(bufs.alloc(&d_src, bytes));
        WD_CUDA(bufs.alloc(&d_dst, bytes));
        WD_CUDA(bufs.alloc(&d_x, cols * 4));
        WD_CUDA(bufs.alloc(&d_y, rows * 4));
        WD_CUDA(bufs.alloc(&d_grid, sizeof(wd_iq2s_grid_packed)));      // the larger of the two codebooks
        if (iq2) WD_CUDA(upload_sync(d_grid, wd_iq2s_grid_packed, sizeof(wd_iq2s_grid_packed)));
        else WD_CUDA(upload_sync(d_grid, wd_iq3s_grid_packed, sizeof(wd_iq3s_grid_packed)));
        if (partials) WD_CUDA(bufs.alloc(&d_p, static_cast<size_t>(rows) * nsb * 8 * 4));
        WD_CUDA(upload_sync(d_src, w, bytes));
        WD_CUDA(upload_sync(d_x, x, cols * 4));
        const long long nblocks = static_cast<long long>(rows) * nsb;
        if (iq2) wd::repack_iq2s_kernel<<<static_cast<unsigned>((nblocks + 127) / 128), 128>>>(d_src, d_dst, nblocks, 0, 0);
        else wd::repack_iq3s_kernel<<<static_cast<unsigned>((nblocks + 127) / 128), 128>>>(d_src, d_dst, nblocks, 0, 0);
        const int nw = 8;
        const size_t smem = wd::kGridTableBytes + nsb * wd::kActSbStride + 32 * 4 + nw * wd::kIq3TileBytes + nw * 640 * 4 + 256;
        WD_CUDA(cudaFuncSetAttribute(wd::iq_matvec_tiles_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        wd::iq_matvec_tiles_kernel<<<64, nw * 32, smem>>>(d_dst, rows, nsb, d_x, d_y, d_p, d_grid, type);
        WD_CUDA(cudaGetLastError());
        WD_CUDA(cudaDeviceSynchronize());
        WD_CUDA(cudaMemcpy(y, d_y, rows * 4, cudaMemcpyDeviceToHost));
        if (partials) WD_CUDA(cudaMemcpy(partials, d_p, static_cast<size_t>(rows) * nsb * 8 * 4, cudaMemcpyDeviceToHost));
    } else if (type == WD_TYPE_Q8_0) {
        const int nb = cols / 32;
        if (cols % 128 || rows % 4 || cols > 8192) return fail(WD_E_INVALID, "Q8_0 matvec: cols % 128, rows % 4");
        const size_t bytes = static_cast<size_t>(rows) * nb * 34;
        WD_CUDA(bufs.alloc(&d_src, bytes));
        WD_CUDA(bufs.alloc(&d_dst, bytes));
        WD_CUDA(bufs.alloc(&d_x, cols * 4));
        WD_CUDA(bufs.alloc(&d_y, rows * 4));
        WD_CUDA(upload_sync(d_src, w, bytes));
        WD_CUDA(upload_sync(d_x, x, cols * 4));
        const long long n = static_cast<long long>(rows) * nb;
        wd::repack_q8_0_kernel<<<static_cast<unsigned>((n + 255) / 256), 256>>>(d_src, d_dst, rows, nb);
        const int nw = 8;
        const size_t smem = cols * 4 + cols + nb * 4 + nw * nb * 136 + 256;
        WD_CUDA(cudaFuncSetAttribute(wd::test_matvec_q8_0_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        wd::test_matvec_q8_0_kernel<<<64, nw * 32, smem>>>(d_dst, rows, nb, d_x, d_y);
        WD_CUDA(cudaGetLastError());
        WD_CUDA(cudaDeviceSynchronize());
        WD_CUDA(cudaMemcpy(y, d_y, rows * 4, cudaMemcpyDeviceToHost));
    } else if (type == WD_TYPE_Q4_0) {
        void *packed = nullptr;
        int rc = wd_dense_pack_q4_0(w, rows, cols, &packed);
        if (rc) return rc;
        WD_CUDA(bufs.alloc(&d_x, cols * 4));
        WD_CUDA(bufs.alloc(&d_y, rows * 4));
        WD_CUDA(upload_sync(d_x, x, cols * 4));
        rc = wd_dense_matvec_q4_0(packed, rows, cols, d_x, d_y, nullptr);
        if (rc == WD_OK) {
            WD_CUDA(cudaDeviceSynchronize());
            WD_CUDA(cudaMemcpy(y, d_y, rows * 4, cudaMemcpyDeviceToHost));
        }
        wd_dense_free(packed);
        if (rc) return rc;
    } else {
        return fail(WD_E_INVALID, "matvec supports IQ3_S, IQ2_S, Q8_0 and Q4_0");
    }
    return WD_OK;
}

// ---- dense Q4_0 path ---------------------------------------------------------------------------------
static int dense_check(int rows, int cols) {
    if (rows <= 0 || cols <= 0 || rows % 32 || cols % (32 * wd::kDenseUnroll) || cols > 32768)
        return fail(WD_E_INVALID, "Q4_0 matvec: rows must be a multiple of 32, cols a multiple of 256 up to 32768");
    return WD_OK;
}

int wd_dense_pack_q4_0_device(const void *w_ggml_dev, int rows, int cols, void **packed_dev, void *stream) {
    if (!w_ggml_dev || !packed_dev) return fail(WD_E_INVALID, "null argument");
    int rc = dense_check(rows, cols);
    if (rc) return rc;
    const int nb = cols / 32;
    uint8_t *dst = nullptr;
    WD_CUDA(cudaMalloc(&dst, static_cast<size_t>(rows) * nb * 18));
    const long long n = static_cast<long long>(rows) * nb;
    wd::repack_q4_0_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t *>(w_ggml_dev), dst, rows, nb);
    cudaError_t ce = cudaGetLastError();
    if (ce != cudaSuccess) {
        cudaFree(dst);
        return fail(WD_E_CUDA, std::string("repack_q4_0_kernel: ") + cudaGetErrorString(ce));
    }
    *packed_dev = dst;
    return WD_OK;
}

int wd_dense_pack_q4_0(const void *w_ggml_host, int rows, int cols, void **packed_dev) {
    if (!w_ggml_host || !packed_dev) return fail(WD_E_INVALID, "null argument");
    int rc = dense_check(rows, cols);
    if (rc) return rc;
    const size_t bytes = static_cast<size_t>(rows) * (cols / 32) * 18;
    uint8_t *src = nullptr;
    WD_CUDA(cudaMalloc(&src, bytes));
    cudaError_t ce = upload_sync(src, w_ggml_host, bytes);
    if (ce == cudaSuccess) {
        rc = wd_dense_pack_q4_0_device(src, rows, cols, packed_dev, nullptr);
        cudaDeviceSynchronize();
    }
    cudaFree(src);
    if (ce != cudaSuccess) return fail(WD_E_CUDA, std::string("cudaMemcpy: ") + cudaGetErrorString(ce));
    return rc;
}

int wd_dense_free(void *packed_dev) {
    if (packed_dev) cudaFree(packed_dev);
    return WD_OK;
}

int wd_dense_matvec_q4_0(const void *packed_dev, int rows, int cols, const float *x_dev, float *y_dev, void *stream) {
    if (!packed_dev || !x_dev || !y_dev) return fail(WD_E_INVALID, "null argument");
    int rc = dense_check(rows, cols);
    if (rc) return rc;
    const int nb = cols / 32;
    const size_t smem = static_cast<size_t>(cols) + static_cast<size_t>(nb) * 4;
    const size_t smem_tile = ((static_cast<size_t>(nb) * 36 + 15) & ~static_cast<size_t>(15)) + wd::kDenseSegSmem;
    static bool attr_set = false;
    if (!attr_set) {
        WD_CUDA(cudaFuncSetAttribute(wd::q4_0_gemv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 40 * 1024));
        WD_CUDA(cudaFuncSetAttribute(wd::q4_0_gemv_tile_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024));
        attr_set = true;
    }
    int dev = 0, n_sm = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
    const int warps = wd::kDenseThreads / 32;
    const int tiles = rows / 32;
    if (tiles <= n_sm * 4) {        // few rows: one CTA per tile, blocks of a row spread over the CTA's warps
        wd::q4_0_gemv_tile_kernel<<<tiles, wd::kDenseThreads, smem_tile, static_cast<cudaStream_t>(stream)>>>(
            static_cast<const uint8_t *>(packed_dev), rows, nb, x_dev, y_dev);
        WD_CUDA(cudaGetLastError());
        return WD_OK;
    }
    // one tile per warp while every CTA can be resident at once (8 per SM); beyond that, whole waves
    int grid = (tiles + warps - 1) / warps;
    if (grid > n_sm * 8) grid = n_sm * 8;
    wd::q4_0_gemv_kernel<<<grid, wd::kDenseThreads, smem, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t *>(packed_dev), rows, nb, x_dev, y_dev);
    WD_CUDA(cudaGetLastError());
    return WD_OK;
}

// ---- output head: Q8_0 matvec + arg-max ------------------------------------------------------------------
static int head_check(int rows, int cols) {
    if (rows <= 0 || cols <= 0 || rows % 32 || cols % (32 * wd::kHeadUnroll) || cols > 32768)
        return fail(WD_E_INVALID, "Q8_0 head: rows must be a multiple of 32, cols a multiple of 128 up to 32768");
    return WD_OK;
}

int wd_dense_pack_q8_0_device(const void *w_ggml_dev, int rows, int cols, void **packed_dev, void *stream) {
    if (!w_ggml_dev || !packed_dev) return fail(WD_E_INVALID, "null argument");
    int rc = head_check(rows, cols);
    if (rc) return rc;
    const int nb = cols / 32;
    uint8_t *dst = nullptr;
    // the packed matrix, then 16 bytes of arg-max state (key, flags)
    WD_CUDA(cudaMalloc(&dst, static_cast<size_t>(rows) * nb * 34 + 16 + 16));
    const long long n = static_cast<long long>(rows) * nb;
    wd::repack_q8_0_planar_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t *>(w_ggml_dev), dst, rows, nb);
    cudaError_t ce = cudaGetLastError();
    if (ce != cudaSuccess) {
        cudaFree(dst);
        return fail(WD_E_CUDA, std::string("repack_q8_0_planar_kernel: ") + cudaGetErrorString(ce));
    }
    *packed_dev = dst;
    return WD_OK;
}

int wd_dense_pack_q8_0(const void *w_ggml_host, int rows, int cols, void **packed_dev) {
    if (!w_ggml_host || !packed_dev) return fail(WD_E_INVALID, "null argument");
    int rc = head_check(rows, cols);
    if (rc) return rc;
    const size_t bytes = static_cast<size_t>(rows) * (cols / 32) * 34;
    uint8_t *src = nullptr;
    WD_CUDA(cudaMalloc(&src, bytes));
    cudaError_t ce = upload_sync(src, w_ggml_host, bytes);
    if (ce == cudaSuccess) {
        rc = wd_dense_pack_q8_0_device(src, rows, cols, packed_dev, nullptr);
        cudaDeviceSynchronize();
    }
    cudaFree(src);
    if (ce != cudaSuccess) return fail(WD_E_CUDA, std::string("cudaMemcpy: ") + cudaGetErrorString(ce));
    return rc;
}

int wd_head_argmax_q8_0(void *packed_dev, int rows, int cols, const float *x_dev, float *logits_dev, int *token_dev,
                        int *nonfinite_dev, void *stream) {
    if (!packed_dev || !x_dev || !token_dev) return fail(WD_E_INVALID, "null argument");
    int rc = head_check(rows, cols);
    if (rc) return rc;
    const int nb = cols / 32;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // state behind the packed matrix (16-byte aligned): u64 key, then the flags word
    uint8_t *state = static_cast<uint8_t *>(packed_dev) + ((static_cast<size_t>(rows) * nb * 34 + 15) & ~static_cast<size_t>(15));
    unsigned long long *key = reinterpret_cast<unsigned long long *>(state);
    int *flags = reinterpret_cast<int *>(state + 8);
    WD_CUDA(cudaMemsetAsync(state, 0, 16, s));
    static bool attr_set = false;
    if (!attr_set) {
        WD_CUDA(cudaFuncSetAttribute(wd::q8_0_head_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 40 * 1024));
        attr_set = true;
    }
    int dev = 0, n_sm = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
    const int warps = wd::kDenseThreads / 32, tiles = rows / 32;
    int grid = (tiles + warps - 1) / warps;
    if (grid > n_sm * 8) grid = n_sm * 8;
    const size_t smem = static_cast<size_t>(cols) + static_cast<size_t>(nb) * 4;
    wd::q8_0_head_kernel<<<grid, wd::kDenseThreads, smem, s>>>(static_cast<const uint8_t *>(packed_dev), rows, nb, x_dev,
                                                             logits_dev, key, flags);
    wd::head_finish_kernel<<<1, 1, 0, s>>>(key, token_dev);
    WD_CUDA(cudaGetLastError());
    if (nonfinite_dev) WD_CUDA(cudaMemcpyAsync(nonfinite_dev, flags, sizeof(int), cudaMemcpyDeviceToDevice, s));
    return WD_OK;
}

int wd_embed_q8_0(const void *table_ggml_dev, int rows, int cols, const int *token_dev, float *out_dev, void *stream) {
    if (!table_ggml_dev || !token_dev || !out_dev) return fail(WD_E_INVALID, "null argument");
    if (rows <= 0 || cols <= 0 || cols % 32) return fail(WD_E_INVALID, "embedding: cols must be a multiple of 32");
    wd::embed_q8_0_kernel<<<(cols + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t *>(table_ggml_dev), rows, cols / 32, token_dev, out_dev);
    WD_CUDA(cudaGetLastError());
    return WD_OK;
}

// ---- synthetic model ----------------------------------------------------------------------------------
static int ensure_lut(wd_engine *e, cudaStream_t s) {
    if (e->synth_lut) return WD_OK;
    WD_CUDA(cudaMalloc(&e->synth_lut, 65536 * 2));
    wd::synth_iq3s_lut_kernel<<<256, 256, 0, s>>>(e->grid_packed, e->synth_lut);
    WD_CUDA(cudaGetLastError());
    return WD_OK;
}

static int synth_into(wd_engine *e, int type, long long rows, int cols, float sigma, uint64_t seed, uint64_t sid,
                      void *dst, cudaStream_t s, long long first_row = 0) {
    if (type == WD_TYPE_Q8_0) {
        const long long nb = rows * (cols / 32);
        wd::synth_q8_0_kernel<<<static_cast<unsigned>((nb + 127) / 128), 128, 0, s>>>(static_cast<uint8_t *>(dst), nb,
                                                                                     sigma, seed, sid);
    } else if (type == WD_TYPE_IQ3_S) {
        int rc = ensure_lut(e, s);
        if (rc) return rc;
        const long long nb = rows * (cols / 256);
        wd::synth_iq3s_kernel<<<static_cast<unsigned>((nb + 63) / 64), 64, 0, s>>>(
            static_cast<uint8_t *>(dst), first_row * (cols / 256), nb, sigma, seed, sid, e->synth_lut);
    } else if (type == WD_TYPE_F32) {
        const long long n = rows * cols;
        wd::synth_f32_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, s>>>(static_cast<float *>(dst), n, sigma,
                                                                                   seed, sid);
    } else {
        return fail(WD_E_INVALID, "synthetic generator supports F32, Q8_0 and IQ3_S");
    }
    WD_CUDA(cudaGetLastError());
    return WD_OK;
}

int wd_synth_tensor_device(int type, int rows, int cols, float sigma, uint64_t seed, uint64_t stream_id,
                           void *dst_dev, void *stream) {
    if (!dst_dev || rows <= 0 || cols <= 0) return fail(WD_E_INVALID, "bad argument");
    if (type == WD_TYPE_IQ3_S)
        return fail(WD_E_STATE, "IQ3_S tensors come from wd_synth_model / wd_synth_expert_host (the engine owns the "
                                "codebook lookup table of that encoder)");
    if (type == WD_TYPE_Q8_0 && cols % 32) return fail(WD_E_INVALID, "Q8_0 needs cols % 32 == 0");
    return synth_into(nullptr, type, rows, cols, sigma, seed, stream_id, dst_dev, static_cast<cudaStream_t>(stream));
}

// stream ids of the tensors of layer l: l*16 + {0 router, 1 bias, 2 gate vec, 3..5 shared gate/up/down,
// 6 norm (unused), 8 gate exps, 9 up exps, 10 down exps}
static uint64_t sid(int layer, int which) { return static_cast<uint64_t>(layer) * 16 + which; }

int wd_synth_model(wd_engine *e, uint64_t seed, float sigma, float bias_sigma) {
    WD_TILED_ONLY(e);
    if (!e) return fail(WD_E_INVALID, "null engine");
    e->layer_table_dirty = true;
    if (e->cfg.gate_type != WD_TYPE_IQ3_S || e->cfg.down_type != WD_TYPE_IQ3_S)
        return fail(WD_E_STATE, "the device-side generator writes IQ3_S experts only");
    WD_CUDA(cudaSetDevice(e->cfg.device));
    const wd_config &c = e->cfg;
    cudaStream_t s = e->stream;
    const size_t gb = e->gate_bytes, db = e->down_bytes;
    const size_t need = static_cast<size_t>(c.n_experts) * (2 * gb + db);
    ScopedDev bufs;         // `big` is released on every path out of this function
    uint8_t *big = nullptr;
    WD_CUDA(bufs.alloc(&big, need));
    int rc = WD_OK;
    for (int l = 0; l < c.n_layers && rc == WD_OK; ++l) {
        Layer &L = e->layers[l];
        const size_t q8_eh = static_cast<size_t>(c.n_experts) * (c.hidden / 32) * 34;
        auto dense = [&](int which, int rows, int cols, uint8_t **dst) -> int {
            const size_t bytes = static_cast<size_t>(rows) * (cols / 32) * 34;
            if (!*dst) WD_CUDA(cudaMalloc(dst, bytes));
            int r = synth_into(e, WD_TYPE_Q8_0, rows, cols, sigma, seed, sid(l, which), e->staging, s);
            if (r) return r;
            launch_repack_q8(e, e->staging, *dst, rows, cols / 32, s);
            WD_CUDA(cudaGetLastError());
            return WD_OK;
        };
        (void)q8_eh;
        if ((rc = dense(0, c.n_experts, c.hidden, &L.router))) break;
        if (bias_sigma > 0) {
            if (!L.bias) WD_CUDA(cudaMalloc(&L.bias, c.n_experts * 4));
            if ((rc = synth_into(e, WD_TYPE_F32, 1, c.n_experts, bias_sigma, seed, sid(l, 1), L.bias, s))) break;
        }
        L.have_router = true;
        if (c.shared_ffn > 0) {
            if (!L.gate_vec) WD_CUDA(cudaMalloc(&L.gate_vec, c.hidden * 4));
            if ((rc = synth_into(e, WD_TYPE_F32, 1, c.hidden, sigma, seed, sid(l, 2), L.gate_vec, s))) break;
            if ((rc = dense(3, c.shared_ffn, c.hidden, &L.sh_gate))) break;
            if ((rc = dense(4, c.shared_ffn, c.hidden, &L.sh_up))) break;
            if ((rc = dense(5, c.hidden, c.shared_ffn, &L.sh_down))) break;
            L.have_shared = true;
        }
        uint8_t *g = big, *u = big + static_cast<size_t>(c.n_experts) * gb, *d = u + static_cast<size_t>(c.n_experts) * gb;
        if ((rc = synth_into(e, WD_TYPE_IQ3_S, static_cast<long long>(c.n_experts) * c.expert_ffn, c.hidden, sigma, seed,
                             sid(l, 8), g, s)))
            break;
        if ((rc = synth_into(e, WD_TYPE_IQ3_S, static_cast<long long>(c.n_experts) * c.expert_ffn, c.hidden, sigma, seed,
                             sid(l, 9), u, s)))
            break;
        if ((rc = synth_into(e, WD_TYPE_IQ3_S, static_cast<long long>(c.n_experts) * c.hidden, c.expert_ffn, sigma, seed,
                             sid(l, 10), d, s)))
            break;
        if (e->resident) {
            if ((rc = wd_set_experts_device(e, l, g, u, d))) break;
        } else {
            // a capped cache streams its misses from host memory: keep a page-locked copy of the layer's experts
            if (!L.owned_host) WD_CUDA(cudaMallocHost(&L.owned_host, need));
            WD_CUDA(cudaMemcpyAsync(L.owned_host, big, need, cudaMemcpyDeviceToHost, s));
            WD_CUDA(cudaStreamSynchronize(s));
            const size_t ge = static_cast<size_t>(c.n_experts) * gb;
            if ((rc = wd_set_experts(e, l, L.owned_host, L.owned_host + ge, L.owned_host + 2 * ge))) break;
        }
    }
    cudaStreamSynchronize(s);
    return rc;
}

int wd_synth_expert_host(wd_engine *e, uint64_t seed, float sigma, int layer, int expert, void *gate, void *up,
                         void *down) {
    WD_TILED_ONLY(e);
    int rc = check_layer(e, layer);
    if (rc) return rc;
    if (expert < 0 || expert >= e->cfg.n_experts || !gate || !up || !down) return fail(WD_E_INVALID, "bad argument");
    WD_CUDA(cudaSetDevice(e->cfg.device));
    const wd_config &c = e->cfg;
    const size_t gb = e->gate_bytes, db = e->down_bytes;
    // regenerate this expert's rows only: the generator indexes values by absolute block number
    cudaStream_t s = e->stream;
    uint8_t *st = e->staging;
    if (2 * gb + db > e->staging_bytes) return fail(WD_E_STATE, "staging buffer too small");
    const long long F = c.expert_ffn, H = c.hidden;
    if ((rc = synth_into(e, WD_TYPE_IQ3_S, F, c.hidden, sigma, seed, sid(layer, 8), st, s, expert * F))) return rc;
    if ((rc = synth_into(e, WD_TYPE_IQ3_S, F, c.hidden, sigma, seed, sid(layer, 9), st + gb, s, expert * F))) return rc;
    if ((rc = synth_into(e, WD_TYPE_IQ3_S, H, c.expert_ffn, sigma, seed, sid(layer, 10), st + 2 * gb, s, expert * H))) return rc;
    WD_CUDA(cudaMemcpyAsync(gate, st, gb, cudaMemcpyDeviceToHost, s));
    WD_CUDA(cudaMemcpyAsync(up, st + gb, gb, cudaMemcpyDeviceToHost, s));
    WD_CUDA(cudaMemcpyAsync(down, st + 2 * gb, db, cudaMemcpyDeviceToHost, s));
    WD_CUDA(cudaStreamSynchronize(s));
    return WD_OK;
}

int wd_synth_dense_host(wd_engine *e, uint64_t seed, float sigma, float bias_sigma, int layer, void *router,
                        float *bias, float *gate_vec, void *sh_gate, void *sh_up, void *sh_down) {
    WD_TILED_ONLY(e);
    int rc = check_layer(e, layer);
    if (rc) return rc;
    WD_CUDA(cudaSetDevice(e->cfg.device));
    const wd_config &c = e->cfg;
    cudaStream_t s = e->stream;
    auto q8 = [&](int which, int rows, int cols, void *dst) -> int {
        if (!dst) return WD_OK;
        int r = synth_into(e, WD_TYPE_Q8_0, rows, cols, sigma, seed, sid(layer, which), e->staging, s);
        if (r) return r;
        WD_CUDA(cudaMemcpyAsync(dst, e->staging, static_cast<size_t>(rows) * (cols / 32) * 34, cudaMemcpyDeviceToHost, s));
        WD_CUDA(cudaStreamSynchronize(s));
        return WD_OK;
    };
    auto f32 = [&](int which, int n, float sg, float *dst) -> int {
        if (!dst) return WD_OK;
        int r = synth_into(e, WD_TYPE_F32, 1, n, sg, seed, sid(layer, which), e->staging, s);
        if (r) return r;
        WD_CUDA(cudaMemcpyAsync(dst, e->staging, static_cast<size_t>(n) * 4, cudaMemcpyDeviceToHost, s));
        WD_CUDA(cudaStreamSynchronize(s));
        return WD_OK;
    };
    if ((rc = q8(0, c.n_experts, c.hidden, router))) return rc;
    if (bias_sigma > 0 && (rc = f32(1, c.n_experts, bias_sigma, bias))) return rc;
    if (c.shared_ffn > 0) {
        if ((rc = f32(2, c.hidden, sigma, gate_vec))) return rc;
        if ((rc = q8(3, c.shared_ffn, c.hidden, sh_gate))) return rc;
        if ((rc = q8(4, c.shared_ffn, c.hidden, sh_up))) return rc;
        if ((rc = q8(5, c.hidden, c.shared_ffn, sh_down))) return rc;
    }
    return WD_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------------
// Allocation-free matvec.
//
// Some callers must not trigger a device allocation: a decode loop that has already handed nearly all
// of HBM to the expert slot pool (a cudaMalloc there can fail, and even when it succeeds it synchronises
// the whole device), code running between the steps of a latency-critical token loop, or a host engine
// whose memory is owned by another allocator. For them this entry point computes y = W x for one IQ3_S
// matrix with the same repack + decode kernels as wd_matvec_host, but takes every buffer from the
// caller (device pointers) and keeps its only scratch - the packed codebook and the repacked tiles - in
// the fixed array below, which every GPU that loads this library holds until the process exits.
//
// The array's name is only a host-side handle; the device address the kernels need comes from
// cudaGetSymbolAddress, looked up once per device by the first call made with that device current. The same
// first call uploads the packed codebook into the front of the array with a blocking copy (later calls never
// write that region), so it should happen before any stream capture. All calls share the array: it keeps the previous
// call's tiles (each call overwrites every byte it later reads, so nothing has to be cleared), and two
// calls that overlap on the GPU - different streams, or one stream re-entered from two host threads -
// race on it.
// ---------------------------------------------------------------------------------------------------
namespace {

constexpr size_t kNoAllocScratchBytes = 8u << 20;            // 8 MiB per GPU
constexpr size_t kNoAllocGridBytes = 1024;                   // packed codebook at the front
static __device__ __align__(256) unsigned char wd_noalloc_scratch[kNoAllocScratchBytes];

constexpr int kNoAllocMaxDevices = 64;
// Set once per device, after the codebook is in place. Two threads that race through the set-up of one device
// both upload the same bytes and store the same address.
std::atomic<void *> g_noalloc_ptr[kNoAllocMaxDevices];

int noalloc_scratch_for_current_device(void **out) {
    int dev = -1;
    WD_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kNoAllocMaxDevices) return fail(WD_E_INVALID, "device ordinal out of range");
    void *p = g_noalloc_ptr[dev].load(std::memory_order_acquire);
    if (!p) {
        const cudaError_t ce = cudaGetSymbolAddress(&p, wd_noalloc_scratch);
        if (ce != cudaSuccess || p == nullptr)
            return fail(WD_E_CUDA, std::string("cudaGetSymbolAddress(wd_noalloc_scratch): ") + cudaGetErrorString(ce));
        static_assert(sizeof(wd_iq3s_grid_packed) == kNoAllocGridBytes, "packed codebook size");
        WD_CUDA(upload_sync(p, wd_iq3s_grid_packed, sizeof(wd_iq3s_grid_packed)));
        g_noalloc_ptr[dev].store(p, std::memory_order_release);
    }
    *out = p;
    return WD_OK;
}

}  // namespace

extern "C" int wd_matvec_iq3s_noalloc(const void *w_dev, int rows, int cols, const float *x_dev, float *y_dev,
                                      void *stream) {
    if (!w_dev || !x_dev || !y_dev) return fail(WD_E_INVALID, "null buffer");
    const int nsb = cols / 256;
    if (rows <= 0 || cols <= 0 || cols % 256 || !pow2(nsb) || nsb > 32 || rows % (32 / nsb))
        return fail(WD_E_INVALID, "cols must be 256*2^n (n<=5) and rows a multiple of 32/(cols/256)");
    const size_t tile_bytes = static_cast<size_t>(rows) * nsb * 110;
    if (tile_bytes > kNoAllocScratchBytes - kNoAllocGridBytes)
        return fail(WD_E_INVALID, "matrix of " + std::to_string(tile_bytes) + " bytes exceeds the fixed scratch of " +
                                      std::to_string(kNoAllocScratchBytes - kNoAllocGridBytes) +
                                      " bytes of the allocation-free matvec");
    void *base = nullptr;
    int rc = noalloc_scratch_for_current_device(&base);
    if (rc) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    uint16_t *grid = static_cast<uint16_t *>(base);
    uint8_t *tiles = static_cast<uint8_t *>(base) + kNoAllocGridBytes;
    const long long nblocks = static_cast<long long>(rows) * nsb;
    wd::repack_iq3s_kernel<<<static_cast<unsigned>((nblocks + 127) / 128), 128, 0, s>>>(
        static_cast<const uint8_t *>(w_dev), tiles, nblocks, 0, 0);
    const int nw = 8;
    const size_t smem = wd::kGridTableBytes + nsb * wd::kActSbStride + 32 * 4 + nw * wd::kIq3TileBytes + nw * 640 * 4 + 256;
    WD_CUDA(cudaFuncSetAttribute(wd::iq_matvec_tiles_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    wd::iq_matvec_tiles_kernel<<<64, nw * 32, smem, s>>>(tiles, rows, nsb, x_dev, y_dev, nullptr, grid);
    WD_CUDA(cudaGetLastError());
    return WD_OK;
}

#include "wd_gguf.inc"
#include "wd_dense_decoder.inc"
