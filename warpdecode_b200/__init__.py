"""warpdecode_b200: B200 (sm_100a) implementation of the batch-1 MoE decode hot path.

The product is the C-ABI shared library built from csrc/ (include/warpdecode_b200.h); this
module is the thin Python binding used by the tests, the bench and the smoke check. There is
no CPU fallback: loading fails loudly when the library is missing, and every call reports the
library's own error text.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
LIB_PATH = os.path.join(HERE, "libwarpdecode_b200.so")
SOURCES = [os.path.join(HERE, "csrc", f) for f in
           ("wd_engine.cu", "wd_aux_kernels.cuh", "wd_moe_kernel.cuh", "wd_moe_kernel_phases.inc", "wd_moe_fast.cuh", "wd_moe_batch.cuh", "wd_dense_decoder.cuh", "wd_dense_decoder.inc", "wd_dense_token.cuh",
            "wd_plain_moe.cuh", "wd_plain_moe.inc", "wd_blocks.cuh", "wd_router.cuh",
            "wd_formats.cuh", "wd_device.cuh", "wd_dense.cuh", "wd_gguf.inc",
            "wd_grids.h")] + [os.path.join(ROOT, "include", "warpdecode_b200.h")]

TYPE_F32, TYPE_Q4_0, TYPE_Q8_0, TYPE_IQ4_NL, TYPE_IQ3_S, TYPE_IQ2_S = 0, 2, 8, 20, 21, 22
TAPS = dict(logits=0, ids=1, weights=2, act=3, expert_out=4, routed=5, shared=6, shared_gate=7, shared_act=8)

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-diag-suppress", "1886", "-shared", "-Xcompiler", "-fPIC"]


def build(force=False, verbose=False):
    """Compile csrc/ into libwarpdecode_b200.so with nvcc (cross-compiles without a GPU)."""
    if not force and os.path.exists(LIB_PATH):
        newest = max(os.path.getmtime(s) for s in SOURCES)
        if os.path.getmtime(LIB_PATH) >= newest:
            return LIB_PATH
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", LIB_PATH, SOURCES[0]]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + r.stdout + r.stderr)
    if verbose:
        print(r.stderr)
    return LIB_PATH


class Config(C.Structure):
    _fields_ = [("hidden", C.c_int32), ("expert_ffn", C.c_int32), ("shared_ffn", C.c_int32),
                ("n_experts", C.c_int32), ("top_k", C.c_int32), ("n_layers", C.c_int32),
                ("gate_type", C.c_int32), ("up_type", C.c_int32), ("down_type", C.c_int32),
                ("w_scale", C.c_float), ("ep_rank", C.c_int32), ("ep_size", C.c_int32),
                ("max_tokens", C.c_int32), ("device", C.c_int32), ("cache_mib", C.c_int64),
                ("rms_eps", C.c_float), ("router_f32", C.c_int32)]


class DenseConfig(C.Structure):
    _fields_ = [("hidden", C.c_int32), ("n_heads", C.c_int32), ("n_kv_heads", C.c_int32), ("head_dim", C.c_int32),
                ("ffn", C.c_int32), ("vocab", C.c_int32), ("n_layers", C.c_int32), ("max_ctx", C.c_int32),
                ("rms_eps", C.c_float), ("rope_theta", C.c_float), ("device", C.c_int32)]


_lib = None


def lib():
    """The loaded C-ABI library. Raises if it has not been built (no fallback exists)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: run warpdecode_b200.build() (needs nvcc); "
                               "there is no CPU fallback")
        L = C.CDLL(LIB_PATH)
        L.wd_last_error.restype = C.c_char_p
        L.wd_default_cache_mib.restype = C.c_int64
        L.wd_default_cache_mib.argtypes = [C.c_int64]
        L.wd_cache_slot_count.restype = C.c_int64
        L.wd_cache_slot_bytes.restype = C.c_int64
        L.wd_cache_slot_count.argtypes = [C.c_void_p]
        L.wd_cache_slot_bytes.argtypes = [C.c_void_p]
        L.wd_engine_create.argtypes = [C.POINTER(Config), C.POINTER(C.c_void_p)]
        L.wd_engine_destroy.argtypes = [C.c_void_p]
        L.wd_engine_destroy.restype = None
        vp, i = C.c_void_p, C.c_int
        L.wd_set_router.argtypes = [vp, i, vp, vp]
        L.wd_set_router_f32.argtypes = [vp, i, vp, vp]
        L.wd_set_shared.argtypes = [vp, i, vp, vp, vp, vp]
        L.wd_set_norm.argtypes = [vp, i, vp]
        L.wd_set_experts.argtypes = [vp, i, vp, vp, vp]
        L.wd_set_experts_typed.argtypes = [vp, i, vp, i, vp, i, vp, i]
        L.wd_set_experts_fused.argtypes = [vp, i, vp, i, vp, i]
        L.wd_set_experts_device.argtypes = [vp, i, vp, vp, vp]
        L.wd_cache_acquire.argtypes = [vp, i, i, C.POINTER(C.c_int)]
        L.wd_cache_stats.argtypes = [vp, C.POINTER(C.c_int64)]
        L.wd_cache_stream_stats.argtypes = [vp, C.POINTER(C.c_int64)]
        L.wd_moe_forward.argtypes = [vp, i, vp, vp, i, vp]
        L.wd_moe_forward_host.argtypes = [vp, i, vp, vp, i]
        L.wd_stack_step.argtypes = [vp, vp, vp]
        L.wd_stack_step_host.argtypes = [vp, vp, vp]
        L.wd_read_tap.argtypes = [vp, i, i, vp, C.c_size_t]
        L.wd_device_status.argtypes = [vp, C.POINTER(C.c_int)]
        L.wd_set_profiling.argtypes = [vp, i]
        L.wd_sm_count.argtypes = [vp]
        L.wd_router_topk_host.argtypes = [vp, i, i, C.c_float, vp, vp, vp]
        L.wd_quantize_q8_0_host.argtypes = [vp, i, vp]
        L.wd_quantize_q8_K_host.argtypes = [vp, i, vp]
        L.wd_matvec_host.argtypes = [i, vp, i, i, vp, vp, vp]
        L.wd_synth_model.argtypes = [vp, C.c_uint64, C.c_float, C.c_float]
        L.wd_synth_tensor_device.argtypes = [i, i, i, C.c_float, C.c_uint64, C.c_uint64, vp, vp]
        L.wd_kernel_name.argtypes = [vp]
        L.wd_kernel_name.restype = C.c_char_p
        L.wd_batch_kernel_name.argtypes = [vp]
        L.wd_batch_kernel_name.restype = C.c_char_p
        L.wd_last_kernel_name.argtypes = [vp]
        L.wd_last_kernel_name.restype = C.c_char_p
        L.wd_measure_tile_decoder.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_double)]
        L.wd_dense_decoder_create.argtypes = [C.POINTER(DenseConfig), C.POINTER(C.c_void_p)]
        L.wd_dense_decoder_set_tensor_typed.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]
        L.wd_dense_decoder_tensor_type.argtypes = [C.c_void_p, C.c_int, C.c_int]
        L.wd_dense_decoder_load_gguf.argtypes = [C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_void_p)]
        L.wd_dense_decoder_config.argtypes = [C.c_void_p, C.POINTER(DenseConfig)]
        L.wd_dense_decoder_destroy.argtypes = [C.c_void_p]
        L.wd_dense_decoder_destroy.restype = None
        L.wd_dense_decoder_kernel_name.argtypes = [C.c_void_p]
        L.wd_dense_decoder_kernel_name.restype = C.c_char_p
        L.wd_dense_decoder_set_tensor.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p]
        L.wd_dense_decoder_get_tensor.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_size_t]
        L.wd_dense_decoder_synth.argtypes = [C.c_void_p, C.c_uint64, C.c_float]
        L.wd_dense_decoder_decode.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.POINTER(C.c_float)]
        L.wd_dense_decoder_read.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        L.wd_synth_expert_host.argtypes = [vp, C.c_uint64, C.c_float, i, i, vp, vp, vp]
        L.wd_synth_dense_host.argtypes = [vp, C.c_uint64, C.c_float, C.c_float, i, vp, vp, vp, vp, vp, vp]
        L.wd_ep_export.argtypes = [vp, vp]
        L.wd_ep_connect.argtypes = [vp, i, vp]
        L.wd_ep_connect_local.argtypes = [vp, i, C.POINTER(vp)]
        L.wd_ep_disconnect.argtypes = [vp]
        L.wd_reset_exchange.argtypes = [vp]
        L.wd_dense_pack_q4_0.argtypes = [vp, i, i, C.POINTER(vp)]
        L.wd_dense_pack_q4_0_device.argtypes = [vp, i, i, C.POINTER(vp), vp]
        L.wd_dense_matvec_q4_0.argtypes = [vp, i, i, vp, vp, vp]
        L.wd_dense_free.argtypes = [vp]
        L.wd_dense_pack_q8_0.argtypes = [vp, i, i, C.POINTER(vp)]
        L.wd_dense_pack_q8_0_device.argtypes = [vp, i, i, C.POINTER(vp), vp]
        L.wd_head_argmax_q8_0.argtypes = [vp, i, i, vp, vp, vp, vp, vp]
        L.wd_embed_q8_0.argtypes = [vp, i, i, vp, vp, vp]
        L.wd_gguf_open.argtypes = [C.c_char_p, C.POINTER(vp)]
        L.wd_gguf_close.argtypes = [vp]
        L.wd_gguf_close.restype = None
        L.wd_gguf_config.argtypes = [vp, C.POINTER(Config)]
        L.wd_gguf_tensor.argtypes = [vp, C.c_char_p, C.POINTER(vp), C.POINTER(i), C.POINTER(C.c_int64), C.POINTER(i)]
        L.wd_engine_load_gguf.argtypes = [vp, vp]
        _lib = L
    return _lib


class WdError(RuntimeError):
    pass


def _check(rc):
    if rc != 0:
        raise WdError(f"warpdecode_b200 error {rc}: {lib().wd_last_error().decode(errors='replace')}")


def _ptr(a):
    return None if a is None else a.ctypes.data


class Gguf:
    """A mapped GGUF file (wd_gguf): geometry and tensor lookup without a GPU; Engine.from_gguf loads it."""

    def __init__(self, path):
        self.h = C.c_void_p()
        _check(lib().wd_gguf_open(os.fsencode(path), C.byref(self.h)))

    def config(self):
        cfg = Config()
        cfg.ep_size, cfg.max_tokens = 1, 1
        _check(lib().wd_gguf_config(self.h, C.byref(cfg)))
        return cfg

    def tensor(self, name):
        """(numpy uint8 view into the mapping, ggml type id, dims in GGUF order)."""
        data, t, nd = C.c_void_p(), C.c_int(), C.c_int()
        dims = (C.c_int64 * 4)()
        _check(lib().wd_gguf_tensor(self.h, name.encode(), C.byref(data), C.byref(t), dims, C.byref(nd)))
        dims = list(dims)[:nd.value]
        n = int(np.prod(dims))
        per = {0: (4, 1), 1: (2, 1), 2: (18, 32), 8: (34, 32), 14: (210, 256), 20: (18, 32), 21: (110, 256), 22: (82, 256)}[t.value]
        nbytes = n // per[1] * per[0]
        buf = (C.c_uint8 * nbytes).from_address(data.value)
        return np.frombuffer(buf, np.uint8), t.value, dims

    def close(self):
        if self.h:
            lib().wd_gguf_close(self.h)
            self.h = C.c_void_p()


class Engine:
    """One MoE stack on one GPU (wd_engine)."""

    @classmethod
    def from_gguf(cls, gguf, **kw):
        """Engine with the file's geometry, every layer loaded (the Gguf must outlive the engine)."""
        c = gguf.config()
        eng = cls(c.hidden, c.expert_ffn, c.n_experts, c.top_k, c.shared_ffn, c.n_layers, expert_type=c.gate_type,
                  down_type=c.down_type, w_scale=c.w_scale, rms_eps=c.rms_eps, router_f32=bool(c.router_f32), **kw)
        _check(lib().wd_engine_load_gguf(eng.h, gguf.h))
        eng._keep.append(gguf)
        return eng

    def __init__(self, hidden, expert_ffn, n_experts, top_k, shared_ffn=0, n_layers=1, expert_type=TYPE_IQ3_S,
                 w_scale=1.0, ep_rank=0, ep_size=1, device=0, cache_mib=0, rms_eps=1e-6, max_tokens=1, down_type=None,
                 router_f32=False):
        self.cfg = Config(hidden, expert_ffn, shared_ffn, n_experts, top_k, n_layers, expert_type, expert_type,
                          expert_type if down_type is None else down_type, w_scale, ep_rank, ep_size, max_tokens,
                          device, cache_mib, rms_eps, int(router_f32))
        self.h = C.c_void_p()
        _check(lib().wd_engine_create(C.byref(self.cfg), C.byref(self.h)))
        self._keep = []

    def close(self):
        if self.h:
            lib().wd_engine_destroy(self.h)
            self.h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- weights -----------------------------------------------------------------------------
    def load_block(self, layer, m):
        """m: dict in the layout of synth.make_moe_block (ggml block bytes, host numpy arrays)."""
        u8 = lambda a: np.ascontiguousarray(a, np.uint8)
        f32 = lambda a: np.ascontiguousarray(a, np.float32)
        bias = f32(m["router_bias"]) if m.get("router_bias") is not None else None
        if self.cfg.router_f32:
            _check(lib().wd_set_router_f32(self.h, layer, _ptr(f32(m["router_f32"])), _ptr(bias)))
        else:
            _check(lib().wd_set_router(self.h, layer, _ptr(u8(m["router"])), _ptr(bias)))
        if self.cfg.shared_ffn:
            gv, sg, su, sd = f32(m["shared_gate_vec"]), u8(m["shared_gate"]), u8(m["shared_up"]), u8(m["shared_down"])
            _check(lib().wd_set_shared(self.h, layer, _ptr(gv), _ptr(sg), _ptr(su), _ptr(sd)))
        g, u, d = u8(m["gate"]), u8(m["up"]), u8(m["down"])
        self._keep += [g, u, d]           # the library retains these host pointers
        if (m["gate_type"], m["up_type"], m["down_type"]) != (self.cfg.gate_type, self.cfg.up_type, self.cfg.down_type):
            _check(lib().wd_set_experts_typed(self.h, layer, _ptr(g), m["gate_type"], _ptr(u), m["up_type"], _ptr(d),
                                              m["down_type"]))
        else:
            _check(lib().wd_set_experts(self.h, layer, _ptr(g), _ptr(u), _ptr(d)))

    def set_norm(self, layer, w):
        w = None if w is None else np.ascontiguousarray(w, np.float32)
        _check(lib().wd_set_norm(self.h, layer, _ptr(w)))

    def synth_model(self, seed, sigma=0.02, bias_sigma=0.0):
        _check(lib().wd_synth_model(self.h, seed, sigma, bias_sigma))

    def synth_expert_host(self, seed, sigma, layer, expert):
        c = self.cfg
        gb = c.expert_ffn * (c.hidden // 256) * 110
        db = c.hidden * (c.expert_ffn // 256) * 110
        g, u, d = np.zeros(gb, np.uint8), np.zeros(gb, np.uint8), np.zeros(db, np.uint8)
        _check(lib().wd_synth_expert_host(self.h, seed, sigma, layer, expert, _ptr(g), _ptr(u), _ptr(d)))
        return g, u, d

    def synth_dense_host(self, seed, sigma, bias_sigma, layer):
        c = self.cfg
        q8 = lambda r, cols: np.zeros(r * (cols // 32) * 34, np.uint8)
        out = dict(router=q8(c.n_experts, c.hidden))
        out["router_bias"] = np.zeros(c.n_experts, np.float32) if bias_sigma > 0 else None
        if c.shared_ffn:
            out.update(shared_gate_vec=np.zeros(c.hidden, np.float32), shared_gate=q8(c.shared_ffn, c.hidden),
                       shared_up=q8(c.shared_ffn, c.hidden), shared_down=q8(c.hidden, c.shared_ffn))
        _check(lib().wd_synth_dense_host(self.h, seed, sigma, bias_sigma, layer, _ptr(out["router"]),
                                         _ptr(out["router_bias"]), _ptr(out.get("shared_gate_vec")),
                                         _ptr(out.get("shared_gate")), _ptr(out.get("shared_up")),
                                         _ptr(out.get("shared_down"))))
        return out

    # -- forward -----------------------------------------------------------------------------
    def forward_host(self, layer, x):
        """x: [hidden], or [n_tokens][hidden] for a batch of up to max_tokens tokens."""
        x = np.ascontiguousarray(x, np.float32)
        n = 1 if x.ndim == 1 else x.shape[0]
        out = np.zeros_like(x)
        _check(lib().wd_moe_forward_host(self.h, layer, _ptr(x), _ptr(out), n))
        return out

    def forward_device(self, layer, x_ptr, out_ptr, stream=None, n_tokens=1):
        _check(lib().wd_moe_forward(self.h, layer, x_ptr, out_ptr, n_tokens, stream))

    def stack_step_host(self, residual):
        r = np.ascontiguousarray(residual, np.float32)
        out = np.zeros_like(r)
        _check(lib().wd_stack_step_host(self.h, _ptr(r), _ptr(out)))
        return out

    def stack_step_device(self, residual_ptr, stream=None):
        _check(lib().wd_stack_step(self.h, residual_ptr, stream))

    # expert parallelism (one engine per GPU, created with ep_rank / ep_size)
    def ep_export(self):
        """This engine's exchange-buffer handle, to be passed to the other ranks' ep_connect."""
        buf = C.create_string_buffer(lib().wd_ep_handle_bytes())
        _check(lib().wd_ep_export(self.h, buf))
        return buf.raw

    def ep_connect(self, handles):
        """handles: the other ranks' ep_export() results (another process each)."""
        blob = b"".join(handles)
        _check(lib().wd_ep_connect(self.h, len(handles), C.c_char_p(blob) if handles else None))

    def ep_connect_local(self, peers):
        """peers: the other ranks' Engine objects of this process (different devices)."""
        arr = (C.c_void_p * max(len(peers), 1))(*[p.h.value for p in peers])
        _check(lib().wd_ep_connect_local(self.h, len(peers), arr))

    def ep_disconnect(self):
        _check(lib().wd_ep_disconnect(self.h))

    def reset_exchange(self):
        _check(lib().wd_reset_exchange(self.h))

    def device_status(self):
        st = C.c_int()
        _check(lib().wd_device_status(self.h, C.byref(st)))
        return st.value

    def tap(self, name, token=None):
        """Intermediate of the last forward call; `token` picks a token of a batch (default: its last)."""
        c = self.cfg
        shapes = dict(logits=(c.n_experts,), ids=(c.top_k,), weights=(c.top_k,), act=(c.top_k, c.expert_ffn),
                      expert_out=(c.top_k, c.hidden), routed=(c.hidden,), shared=(c.hidden,), shared_gate=(1,),
                      shared_act=(max(c.shared_ffn, 1),))
        a = np.zeros(shapes[name], np.int32 if name == "ids" else np.float32)
        if token is None:
            token = -1
        _check(lib().wd_read_tap(self.h, TAPS[name], token, _ptr(a), a.nbytes))
        return a

    def fallbacks(self):
        """Layers so far whose expert ids came from the exact rungs instead of the logit threshold."""
        a = np.zeros(1, np.uint32)
        _check(lib().wd_read_tap(self.h, 10, -1, _ptr(a), 4))
        return int(a[0])

    def kernel_name(self):
        """Name of the kernel that this engine's stack step launches."""
        return lib().wd_kernel_name(self.h).decode()

    def last_kernel_name(self):
        """Name of the kernel the last forward call ran on."""
        return lib().wd_last_kernel_name(self.h).decode()

    def batch_kernel_name(self):
        """Name of the kernel a token batch (forward with several tokens) runs on."""
        return lib().wd_batch_kernel_name(self.h).decode()

    def set_profiling(self, on):
        _check(lib().wd_set_profiling(self.h, int(on)))

    def stamps(self):
        """[sm_count, 32] uint64 global-timer values of the last launch (profiling on): 0..15 the layer's phases,
        16..21 the stages of the selection, 24/25 the SM clock counter at stamps 0 and 10."""
        n = lib().wd_sm_count(self.h)
        a = np.zeros((n, 32), np.uint64)
        _check(lib().wd_read_tap(self.h, 9, 0, _ptr(a), a.nbytes))
        return a

    def slot_count(self):
        return lib().wd_cache_slot_count(self.h)

    def slot_bytes(self):
        return lib().wd_cache_slot_bytes(self.h)

    def cache_acquire(self, layer, expert):
        slot = C.c_int()
        _check(lib().wd_cache_acquire(self.h, layer, expert, C.byref(slot)))
        return slot.value

    def cache_stream_stats(self):
        """(bytes sent host -> device, host nanoseconds spent placing misses, layers placed) since creation."""
        st = (C.c_int64 * 3)()
        _check(lib().wd_cache_stream_stats(self.h, st))
        return tuple(st)

    def cache_stats(self):
        """(hits, misses, evictions) since creation."""
        st = (C.c_int64 * 3)()
        _check(lib().wd_cache_stats(self.h, st))
        return tuple(st)


# -- expert-parallel host helpers --------------------------------------------------------------
def ep_range(n_experts, rank, size):
    """Experts [first, first + count) that rank `rank` of `size` owns (contiguous, equal shares)."""
    if size < 1 or not 0 <= rank < size or n_experts % size:
        raise ValueError("ep_rank/ep_size must partition n_experts evenly")
    count = n_experts // size
    return rank * count, count


def ep_connect_all(engine, dist, rank, world):
    """Exchanges the ranks' exchange-buffer handles over an initialised torch.distributed group (any
    backend) and connects `engine` to every other rank. Collective: every rank must call it."""
    handles = [None] * world
    dist.all_gather_object(handles, engine.ep_export())
    engine.ep_connect([h for r, h in enumerate(handles) if r != rank])
    dist.barrier()
    return handles


# -- dense Q4_0 matvec -------------------------------------------------------------------------
class DenseQ4_0:
    """A Q4_0 matrix [rows][cols] packed on the device (wd_dense_pack_q4_0*); y = W x on device buffers."""

    def __init__(self, rows, cols, ggml_host=None, ggml_dev_ptr=None, stream=None):
        self.rows, self.cols, self.p = rows, cols, C.c_void_p()
        if ggml_host is not None:
            w = np.ascontiguousarray(ggml_host, np.uint8)
            assert w.size == rows * (cols // 32) * 18
            _check(lib().wd_dense_pack_q4_0(_ptr(w), rows, cols, C.byref(self.p)))
        else:
            _check(lib().wd_dense_pack_q4_0_device(ggml_dev_ptr, rows, cols, C.byref(self.p), stream))

    def matvec(self, x_ptr, y_ptr, stream=None):
        _check(lib().wd_dense_matvec_q4_0(self.p, self.rows, self.cols, x_ptr, y_ptr, stream))

    def close(self):
        if self.p:
            lib().wd_dense_free(self.p)
            self.p = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class HeadQ8_0:
    """Output head: a Q8_0 matrix [vocab][hidden] packed on the device; token = arg-max(W x) (wd_head_argmax_q8_0)."""

    def __init__(self, rows, cols, ggml_host=None, ggml_dev_ptr=None, stream=None):
        self.rows, self.cols, self.p = rows, cols, C.c_void_p()
        if ggml_host is not None:
            w = np.ascontiguousarray(ggml_host, np.uint8)
            assert w.size == rows * (cols // 32) * 34
            _check(lib().wd_dense_pack_q8_0(_ptr(w), rows, cols, C.byref(self.p)))
        else:
            _check(lib().wd_dense_pack_q8_0_device(ggml_dev_ptr, rows, cols, C.byref(self.p), stream))

    def argmax(self, x_ptr, token_ptr, logits_ptr=None, nonfinite_ptr=None, stream=None):
        _check(lib().wd_head_argmax_q8_0(self.p, self.rows, self.cols, x_ptr, logits_ptr, token_ptr, nonfinite_ptr, stream))

    def close(self):
        if self.p:
            lib().wd_dense_free(self.p)
            self.p = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


DT_TOKEN_EMBD, DT_OUTPUT_NORM, DT_OUTPUT, DT_ATTN_NORM, DT_WQKV, DT_WO, DT_FFN_NORM, DT_W_GATE_UP, DT_W_DOWN = range(9)
DT_BQKV, DT_Q_NORM, DT_K_NORM = 9, 10, 11          # optional F32 vectors: q/k/v biases, q and k head norms


class DenseDecoder:
    """The plain (dense) Q4_0 decoder (wd_dense_decoder_*): Llama-style layers, greedy decode on the device."""

    def __init__(self, hidden, n_heads, n_kv_heads, head_dim, ffn, vocab, n_layers, max_ctx, rms_eps=1e-5, rope_theta=500000.0,
                 device=0):
        self.cfg = DenseConfig(hidden, n_heads, n_kv_heads, head_dim, ffn, vocab, n_layers, max_ctx, rms_eps, rope_theta, device)
        self.h = C.c_void_p()
        _check(lib().wd_dense_decoder_create(C.byref(self.cfg), C.byref(self.h)))

    @classmethod
    def from_gguf(cls, gguf, max_ctx, device=0):
        """Decoder with the geometry and tensors of a Llama-style Q4_0 file (wd_dense_decoder_load_gguf)."""
        self = cls.__new__(cls)
        self.h = C.c_void_p()
        _check(lib().wd_dense_decoder_load_gguf(gguf.h, max_ctx, device, C.byref(self.h)))
        self.cfg = DenseConfig()
        _check(lib().wd_dense_decoder_config(self.h, C.byref(self.cfg)))
        return self

    def shape(self, which):
        c = self.cfg
        q = c.n_heads * c.head_dim
        kv = c.n_kv_heads * c.head_dim
        return {DT_TOKEN_EMBD: (c.vocab, c.hidden), DT_OUTPUT: (c.vocab, c.hidden), DT_WQKV: (q + 2 * kv, c.hidden),
                DT_WO: (c.hidden, q), DT_W_GATE_UP: (2 * c.ffn, c.hidden), DT_W_DOWN: (c.hidden, c.ffn)}.get(which)

    def vector_len(self, which):
        c = self.cfg
        return {DT_BQKV: (c.n_heads + 2 * c.n_kv_heads) * c.head_dim, DT_Q_NORM: c.head_dim, DT_K_NORM: c.head_dim}.get(which, c.hidden)

    def set_tensor(self, layer, which, data, type=TYPE_Q4_0):
        """A vector (F32) or a matrix in ggml blocks of `type` (Q4_0, or Q8_0 for what a model file holds in other types)."""
        shp = self.shape(which)
        a = np.ascontiguousarray(data, np.float32 if shp is None else np.uint8)
        assert a.size == (self.vector_len(which) if shp is None else shp[0] * (shp[1] // 32) * (34 if type == TYPE_Q8_0 else 18))
        _check(lib().wd_dense_decoder_set_tensor_typed(self.h, layer, which, type, _ptr(a)))

    def tensor_type(self, layer, which):
        t = lib().wd_dense_decoder_tensor_type(self.h, layer, which)
        if t < 0:
            _check(t)
        return t

    def get_tensor(self, layer, which):
        shp = self.shape(which)
        per = 34 if shp is not None and self.tensor_type(layer, which) == TYPE_Q8_0 else 18
        a = np.zeros(self.vector_len(which), np.float32) if shp is None else np.zeros(shp[0] * (shp[1] // 32) * per, np.uint8)
        _check(lib().wd_dense_decoder_get_tensor(self.h, layer, which, _ptr(a), a.nbytes))
        return a

    def kernel_name(self):
        return lib().wd_dense_decoder_kernel_name(self.h).decode()

    def synth(self, seed, sigma=0.02):
        _check(lib().wd_dense_decoder_synth(self.h, seed, sigma))

    def decode(self, prompt, n_gen):
        """Greedy decode; returns (tokens [len(prompt) + n_gen], device milliseconds of the whole run)."""
        pr = np.ascontiguousarray(prompt, np.int32)
        out = np.zeros(pr.size + n_gen, np.int32)
        ms = C.c_float()
        _check(lib().wd_dense_decoder_decode(self.h, _ptr(pr), pr.size, n_gen, _ptr(out), C.byref(ms)))
        return out, ms.value

    def read(self):
        logits = np.zeros(self.cfg.vocab, np.float32)
        hidden = np.zeros(self.cfg.hidden, np.float32)
        _check(lib().wd_dense_decoder_read(self.h, _ptr(logits), _ptr(hidden)))
        return logits, hidden

    def close(self):
        if self.h:
            lib().wd_dense_decoder_destroy(self.h)
            self.h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def measure_tile_decoder(nsb=8, warps=16, unroll=1, device=0):
    """SM clock cycles per round of `warps` IQ3_S tiles decoded from shared memory (the issue bound of the expert GEMVs)."""
    c = C.c_double()
    _check(lib().wd_measure_tile_decoder(device, nsb, warps, unroll, C.byref(c)))
    return c.value


def embed_q8_0(table_dev_ptr, rows, cols, token_ptr, out_ptr, stream=None):
    _check(lib().wd_embed_q8_0(table_dev_ptr, rows, cols, token_ptr, out_ptr, stream))


def synth_tensor_device(t, rows, cols, sigma, seed, stream_id, dst_ptr, stream=None):
    """rows x cols N(0, sigma) weights quantised to ggml type `t`, written to device memory at dst_ptr."""
    _check(lib().wd_synth_tensor_device(t, rows, cols, sigma, seed, stream_id, dst_ptr, stream))


# -- stand-alone pieces ------------------------------------------------------------------------
def router_topk(logits, k, w_scale=1.0):
    logits = np.ascontiguousarray(logits, np.float32)
    ids, w, p = np.zeros(k, np.int32), np.zeros(k, np.float32), np.zeros(logits.size, np.float32)
    _check(lib().wd_router_topk_host(_ptr(logits), logits.size, k, w_scale, _ptr(ids), _ptr(w), _ptr(p)))
    return p, ids, w


def quantize_q8_0(x):
    x = np.ascontiguousarray(x, np.float32)
    out = np.zeros(x.size // 32 * 34, np.uint8)
    _check(lib().wd_quantize_q8_0_host(_ptr(x), x.size, _ptr(out)))
    return out


def quantize_q8_K(x):
    x = np.ascontiguousarray(x, np.float32)
    out = np.zeros(x.size // 256 * 292, np.uint8)
    _check(lib().wd_quantize_q8_K_host(_ptr(x), x.size, _ptr(out)))
    return out


def matvec(t, w, rows, cols, x, partials=False):
    w = np.ascontiguousarray(w, np.uint8)
    x = np.ascontiguousarray(x, np.float32)
    y = np.zeros(rows, np.float32)
    p = np.zeros((rows, cols // 256, 8), np.int32) if partials else None
    _check(lib().wd_matvec_host(t, _ptr(w), rows, cols, _ptr(x), _ptr(y), _ptr(p)))
    return (y, p) if partials else y
