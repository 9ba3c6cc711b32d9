"""ctypes access to the CPU oracle (oracle/libwd_oracle.so) and, when it was built,
to the reference project's own host code (oracle/_ref/libwd_ref.so).

Test infrastructure only: nothing under warpdecode_b200/ imports this module.
"""
import ctypes as C
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")

TYPE_F32, TYPE_Q4_0, TYPE_Q8_0, TYPE_IQ4_NL, TYPE_IQ3_S, TYPE_IQ2_S = 0, 2, 8, 20, 21, 22
TYPE_Q6_K = 14
BLOCK_BYTES = {TYPE_Q8_0: 34, TYPE_Q4_0: 18, TYPE_IQ4_NL: 18, TYPE_IQ3_S: 110, TYPE_IQ2_S: 82}
BLOCK_ELEMS = {TYPE_Q8_0: 32, TYPE_Q4_0: 32, TYPE_IQ4_NL: 32, TYPE_IQ3_S: 256, TYPE_IQ2_S: 256}
Q8K_BYTES = 292

_f32p = C.POINTER(C.c_float)
_u8p = C.POINTER(C.c_uint8)
_i32p = C.POINTER(C.c_int32)


def row_bytes(t, cols):
    return cols // BLOCK_ELEMS[t] * BLOCK_BYTES[t]


def fbits(a):
    """float32 bit patterns with every NaN mapped to one pattern: NaN payload and sign are not
    part of any contract (x86 produces 0xffc00000, CUDA 0x7fffffff for the same operation)."""
    a = np.ascontiguousarray(a, np.float32)
    b = a.view(np.uint32).copy()
    b[np.isnan(a)] = 0x7fc00000
    return b


def _p(a, ty):
    return None if a is None else a.ctypes.data_as(ty)


class MoeWeightsC(C.Structure):
    _fields_ = [
        ("hidden", C.c_int), ("expert_ffn", C.c_int), ("shared_ffn", C.c_int),
        ("n_experts", C.c_int), ("top_k", C.c_int),
        ("gate_type", C.c_int), ("up_type", C.c_int), ("down_type", C.c_int),
        ("w_scale", C.c_float),
        ("router", _u8p), ("router_bias", _f32p),
        ("gate", _u8p), ("up", _u8p), ("down", _u8p),
        ("shared_gate_vec", _f32p),
        ("shared_gate", _u8p), ("shared_up", _u8p), ("shared_down", _u8p),
        ("router_f32", _f32p),
    ]


class MoeResultC(C.Structure):
    _fields_ = [
        ("logits", _f32p), ("probs", _f32p), ("ids", _i32p), ("weights", _f32p),
        ("act", _f32p), ("expert_out", _f32p), ("routed", _f32p), ("shared", _f32p),
        ("shared_gate", _f32p), ("out", _f32p),
    ]


def build_oracle():
    subprocess.run(["make", "-s", "-C", ORACLE_DIR], check=True)
    if os.path.isdir(os.environ.get("WD_REFERENCE", "/root/reference")):
        subprocess.run(["bash", os.path.join(ORACLE_DIR, "build_ref.sh")], check=True,
                       stdout=subprocess.DEVNULL)


class DenseLayerC(C.Structure):
    _fields_ = [("attn_norm", C.c_void_p), ("wqkv", C.c_void_p), ("wo", C.c_void_p), ("ffn_norm", C.c_void_p),
                ("w_gate_up", C.c_void_p), ("w_down", C.c_void_p),
                ("wqkv_type", C.c_int), ("wo_type", C.c_int), ("w_gate_up_type", C.c_int), ("w_down_type", C.c_int),
                ("bqkv", C.c_void_p), ("q_norm", C.c_void_p), ("k_norm", C.c_void_p)]


class DenseModelC(C.Structure):
    _fields_ = [("hidden", C.c_int), ("n_heads", C.c_int), ("n_kv_heads", C.c_int), ("head_dim", C.c_int), ("ffn", C.c_int),
                ("vocab", C.c_int), ("n_layers", C.c_int), ("max_ctx", C.c_int), ("rms_eps", C.c_float),
                ("token_embd", C.c_void_p), ("output_norm", C.c_void_p), ("output", C.c_void_p),
                ("layers", C.POINTER(DenseLayerC)), ("rope_table", C.c_void_p), ("hidden_out", C.c_void_p),
                ("token_embd_type", C.c_int), ("output_type", C.c_int)]


class DenseOracle:
    """The dense decoder of oracle/wd_oracle_dense.c over numpy tensors (ggml Q4_0 bytes, F32 norms)."""

    def __init__(self, oracle, cfg, tensors, layers, rope_theta):
        """cfg: dict(hidden, n_heads, n_kv_heads, head_dim, ffn, vocab, n_layers, max_ctx, rms_eps); tensors: dict with
        token_embd, output_norm, output; layers: list of dicts attn_norm, wqkv, wo, ffn_norm, w_gate_up, w_down. A
        matrix is Q4_0 unless the dict holds "<name>_type" = TYPE_Q8_0."""
        self.L = oracle.lib
        self.keep = []

        def ptr(a, dt):
            a = np.ascontiguousarray(a, dt)
            self.keep.append(a)
            return a.ctypes.data

        self.layers = (DenseLayerC * cfg["n_layers"])()
        for i, l in enumerate(layers):
            self.layers[i] = DenseLayerC(ptr(l["attn_norm"], np.float32), ptr(l["wqkv"], np.uint8), ptr(l["wo"], np.uint8),
                                         ptr(l["ffn_norm"], np.float32), ptr(l["w_gate_up"], np.uint8), ptr(l["w_down"], np.uint8),
                                         l.get("wqkv_type", 0), l.get("wo_type", 0), l.get("w_gate_up_type", 0), l.get("w_down_type", 0),
                                         ptr(l["bqkv"], np.float32) if l.get("bqkv") is not None else None,
                                         ptr(l["q_norm"], np.float32) if l.get("q_norm") is not None else None,
                                         ptr(l["k_norm"], np.float32) if l.get("k_norm") is not None else None)
        self.rope = np.zeros(cfg["max_ctx"] * (cfg["head_dim"] // 2) * 2, np.float32)
        self.L.wdo_rope_table.argtypes = [C.c_int, C.c_int, C.c_double, C.c_void_p]
        self.L.wdo_rope_table(cfg["max_ctx"], cfg["head_dim"], float(rope_theta), self.rope.ctypes.data)
        self.hidden = np.zeros(cfg["hidden"], np.float32)
        self.m = DenseModelC(cfg["hidden"], cfg["n_heads"], cfg["n_kv_heads"], cfg["head_dim"], cfg["ffn"], cfg["vocab"],
                             cfg["n_layers"], cfg["max_ctx"], cfg["rms_eps"], ptr(tensors["token_embd"], np.uint8),
                             ptr(tensors["output_norm"], np.float32), ptr(tensors["output"], np.uint8), self.layers,
                             self.rope.ctypes.data, self.hidden.ctypes.data, tensors.get("token_embd_type", 0),
                             tensors.get("output_type", 0))
        kv = cfg["n_layers"] * cfg["max_ctx"] * cfg["n_kv_heads"] * cfg["head_dim"]
        self.kc, self.vc = np.zeros(kv, np.float32), np.zeros(kv, np.float32)
        self.logits = np.zeros(cfg["vocab"], np.float32)
        self.L.wdo_dense_step.argtypes = [C.POINTER(DenseModelC), C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]
        self.L.wdo_dense_step.restype = C.c_int

    def step(self, token, pos):
        return int(self.L.wdo_dense_step(C.byref(self.m), self.kc.ctypes.data, self.vc.ctypes.data, int(token), int(pos),
                                         self.logits.ctypes.data))

    def decode(self, prompt, n_gen):
        toks = list(map(int, prompt))
        tok = toks[0]
        for pos in range(len(prompt) + n_gen - 1):
            nxt = self.step(tok, pos)
            if pos + 1 < len(prompt):
                nxt = toks[pos + 1]
            else:
                toks.append(nxt)
            tok = nxt
        return np.array(toks, np.int32)


class Oracle:
    """The plain-C restatement."""

    def __init__(self):
        path = os.path.join(ORACLE_DIR, "libwd_oracle.so")
        if not os.path.exists(path):
            build_oracle()
        L = self.lib = C.CDLL(path)
        L.wdo_f16_to_f32.restype = C.c_float
        L.wdo_f16_to_f32.argtypes = [C.c_uint16]
        L.wdo_f32_to_f16.restype = C.c_uint16
        L.wdo_f32_to_f16.argtypes = [C.c_float]
        L.wdo_iq3s_grid.restype = C.c_uint32
        L.wdo_iq2s_grid.restype = C.c_uint64
        L.wdo_requantize_row_to_q8_0.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int]
        L.wdo_q6_k_value.restype = C.c_float
        L.wdo_q6_k_value.argtypes = [C.c_void_p, C.c_int]
        for name in ("wdo_row_q8_0_q8_0", "wdo_row_iq4_nl_q8_0", "wdo_row_q4_0_q8_0", "wdo_row_q4_0_q8_0_lanes",
                     "wdo_row_q8_0_q8_0_lanes"):
            getattr(L, name).restype = C.c_float
            getattr(L, name).argtypes = [C.c_void_p, C.c_void_p, C.c_int]
        L.wdo_matvec_q8_0_argmax.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        for name in ("wdo_row_iq3_s_q8_K", "wdo_row_iq2_s_q8_K"):
            getattr(L, name).restype = C.c_float
            getattr(L, name).argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
        for name in ("wdo_exp_ggml", "wdo_silu_ggml", "wdo_sigmoid_ggml"):
            getattr(L, name).restype = C.c_float
            getattr(L, name).argtypes = [C.c_float]
        L.wdo_dot_f32.restype = C.c_float
        L.wdo_dot_f32.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
        L.wdo_router_exact.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_float, C.c_void_p,
                                       C.c_void_p, C.c_void_p]
        L.wdo_quantize_q8_0.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
        L.wdo_quantize_q8_K.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
        L.wdo_moe_block.argtypes = [C.POINTER(MoeWeightsC), C.c_void_p, C.POINTER(MoeResultC),
                                    C.c_int, C.c_int]
        L.wdo_rmsnorm.argtypes = [C.c_void_p, C.c_void_p, C.c_float, C.c_int, C.c_void_p]

    # -- elementwise -----------------------------------------------------
    def f16_to_f32(self, bits):
        return np.array([self.lib.wdo_f16_to_f32(int(b)) for b in np.asarray(bits).ravel()], np.float32)

    def f32_to_f16(self, vals):
        return np.array([self.lib.wdo_f32_to_f16(float(v)) for v in np.asarray(vals, np.float32).ravel()], np.uint16)

    def unary(self, name, vals):
        f = getattr(self.lib, "wdo_" + name)
        return np.array([f(float(v)) for v in np.asarray(vals, np.float32).ravel()], np.float32)

    def grids(self):
        g3 = np.array([self.lib.wdo_iq3s_grid(i) for i in range(512)], np.uint32)
        g2 = np.array([self.lib.wdo_iq2s_grid(i) for i in range(1024)], np.uint64)
        return g3, g2

    # -- quantisers ------------------------------------------------------
    def quantize_q8_0(self, x):
        x = np.ascontiguousarray(x, np.float32)
        out = np.zeros(x.size // 32 * 34, np.uint8)
        self.lib.wdo_quantize_q8_0(x.ctypes.data, out.ctypes.data, x.size // 32)
        return out

    def quantize_q8_K(self, x):
        x = np.ascontiguousarray(x, np.float32)
        out = np.zeros(x.size // 256 * Q8K_BYTES, np.uint8)
        self.lib.wdo_quantize_q8_K(x.ctypes.data, out.ctypes.data, x.size // 256)
        return out

    # -- rows --------------------------------------------------------------
    def row(self, t, w_row, y, cols, partials=False):
        w_row = np.ascontiguousarray(w_row, np.uint8)
        y = np.ascontiguousarray(y, np.uint8)
        if t in (TYPE_IQ3_S, TYPE_IQ2_S):
            f = self.lib.wdo_row_iq3_s_q8_K if t == TYPE_IQ3_S else self.lib.wdo_row_iq2_s_q8_K
            part = np.zeros(cols // 256 * 8, np.int32)
            v = f(w_row.ctypes.data, y.ctypes.data, cols, part.ctypes.data if partials else None)
            return (np.float32(v), part) if partials else np.float32(v)
        f = {TYPE_Q8_0: self.lib.wdo_row_q8_0_q8_0, TYPE_IQ4_NL: self.lib.wdo_row_iq4_nl_q8_0,
             TYPE_Q4_0: self.lib.wdo_row_q4_0_q8_0}[t]
        return np.float32(f(w_row.ctypes.data, y.ctypes.data, cols))

    def requantize_rows_to_q8_0(self, t, blob, rows, cols):
        """[rows][cols] of ggml type t (Q8_0 or Q6_K = 14) -> Q8_0 blocks, the dense loader's host rule."""
        blob = np.ascontiguousarray(blob, np.uint8)
        rb = cols // 32 * 34 if t == TYPE_Q8_0 else cols // 256 * 210
        out = np.zeros(rows * (cols // 32) * 34, np.uint8)
        for r in range(rows):
            rc = self.lib.wdo_requantize_row_to_q8_0(t, blob.ctypes.data + r * rb, out.ctypes.data + r * (cols // 32) * 34, cols)
            if rc != 0:
                raise RuntimeError("wdo_requantize_row_to_q8_0 refused the row")
        return out

    def head_argmax_q8_0(self, w, rows, cols, y, logits=False):
        """Greedy token of a Q8_0 head [rows][cols] (ggml blocks) for the Q8_0-quantised activation y:
        the row dot of every row, then the largest finite logit, lowest index first."""
        w = np.ascontiguousarray(w, np.uint8)
        y = np.ascontiguousarray(y, np.uint8)
        out = np.zeros(rows, np.float32) if logits else None
        tok = self.lib.wdo_matvec_q8_0_argmax(w.ctypes.data, rows, cols, y.ctypes.data, out.ctypes.data if logits else None)
        return (tok, out) if logits else tok

    def dot_f32(self, a, b):
        a = np.ascontiguousarray(a, np.float32)
        b = np.ascontiguousarray(b, np.float32)
        return np.float32(self.lib.wdo_dot_f32(a.ctypes.data, b.ctypes.data, a.size))

    def router(self, logits, k, w_scale=1.0):
        logits = np.ascontiguousarray(logits, np.float32)
        n = logits.size
        probs = np.zeros(n, np.float32)
        ids = np.zeros(k, np.int32)
        w = np.zeros(k, np.float32)
        self.lib.wdo_router_exact(logits.ctypes.data, n, k, w_scale, probs.ctypes.data,
                                  ids.ctypes.data, w.ctypes.data)
        return probs, ids, w

    def rmsnorm(self, x, weight, eps):
        x = np.ascontiguousarray(x, np.float32)
        y = np.zeros_like(x)
        wp = None if weight is None else np.ascontiguousarray(weight, np.float32).ctypes.data
        self.lib.wdo_rmsnorm(x.ctypes.data, wp, eps, x.size, y.ctypes.data)
        return y

    # -- whole block -------------------------------------------------------
    def moe_block(self, m, x, first_expert=0, n_local=None):
        """m: dict with the MoeWeightsC field names (numpy uint8/float32 arrays)."""
        keep = []

        def u8(a):
            if a is None:
                return None
            a = np.ascontiguousarray(a, np.uint8)
            keep.append(a)
            return a.ctypes.data_as(_u8p)

        def f32(a):
            if a is None:
                return None
            a = np.ascontiguousarray(a, np.float32)
            keep.append(a)
            return a.ctypes.data_as(_f32p)

        w = MoeWeightsC(m["hidden"], m["expert_ffn"], m.get("shared_ffn", 0), m["n_experts"], m["top_k"],
                        m["gate_type"], m["up_type"], m["down_type"], m.get("w_scale", 1.0),
                        u8(m.get("router")), f32(m.get("router_bias")), u8(m["gate"]), u8(m["up"]), u8(m["down"]),
                        f32(m.get("shared_gate_vec")), u8(m.get("shared_gate")), u8(m.get("shared_up")),
                        u8(m.get("shared_down")), f32(m.get("router_f32")))
        H, F, E, K = m["hidden"], m["expert_ffn"], m["n_experts"], m["top_k"]
        res = {
            "logits": np.zeros(E, np.float32), "probs": np.zeros(E, np.float32),
            "ids": np.zeros(K, np.int32), "weights": np.zeros(K, np.float32),
            "act": np.zeros((K, F), np.float32), "expert_out": np.zeros((K, H), np.float32),
            "routed": np.zeros(H, np.float32), "shared": np.zeros(H, np.float32),
            "shared_gate": np.zeros(1, np.float32), "out": np.zeros(H, np.float32),
        }
        r = MoeResultC(_p(res["logits"], _f32p), _p(res["probs"], _f32p), _p(res["ids"], _i32p),
                       _p(res["weights"], _f32p), _p(res["act"], _f32p), _p(res["expert_out"], _f32p),
                       _p(res["routed"], _f32p), _p(res["shared"], _f32p), _p(res["shared_gate"], _f32p),
                       _p(res["out"], _f32p))
        x = np.ascontiguousarray(x, np.float32)
        rc = self.lib.wdo_moe_block(C.byref(w), x.ctypes.data, C.byref(r), first_expert,
                                    E if n_local is None else n_local)
        if rc != 0:
            raise RuntimeError(f"wdo_moe_block failed: {rc}")
        return res


class Reference:
    """The reference project's own functions (oracle/_ref/libwd_ref.so)."""

    @staticmethod
    def available():
        return os.path.exists(os.path.join(ORACLE_DIR, "_ref", "libwd_ref.so"))

    def __init__(self):
        L = self.lib = C.CDLL(os.path.join(ORACLE_DIR, "_ref", "libwd_ref.so"))
        L.ref_f16_to_f32.restype = C.c_float
        L.ref_f16_to_f32.argtypes = [C.c_uint16]
        L.ref_f32_to_f16.restype = C.c_uint16
        L.ref_f32_to_f16.argtypes = [C.c_float]
        L.ref_iq3s_grid.restype = C.c_uint32
        L.ref_iq2s_grid.restype = C.c_uint64
        for name in ("ref_row_iq3_s_q8_K", "ref_row_iq2_s_q8_K", "ref_row_q8_0_q8_0", "ref_row_iq4_nl_q8_0"):
            getattr(L, name).restype = C.c_float
            getattr(L, name).argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int]
        for name in ("ref_exp_ggml", "ref_silu_ggml", "ref_sigmoid_ggml", "ref_router_exp"):
            getattr(L, name).restype = C.c_float
            getattr(L, name).argtypes = [C.c_float]
        L.ref_requantize_row_to_q8_0.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int]
        L.ref_q6_k_value.restype = C.c_float
        L.ref_q6_k_value.argtypes = [C.c_void_p, C.c_int]
        L.ref_dot_f32.restype = C.c_float
        L.ref_dot_f32.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
        L.ref_router_exact.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_float, C.c_void_p, C.c_void_p,
                                       C.c_void_p]
        L.ref_quantize_q8_0.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
        L.ref_quantize_q8_K.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
        L.ref_moe_block.argtypes = [C.POINTER(MoeWeightsC), C.c_void_p, C.c_int, C.c_void_p, C.c_void_p,
                                    C.c_void_p, C.c_void_p]
        L.ref_hardware_threads.restype = C.c_int

    def f16_to_f32(self, bits):
        return np.array([self.lib.ref_f16_to_f32(int(b)) for b in np.asarray(bits).ravel()], np.float32)

    def f32_to_f16(self, vals):
        return np.array([self.lib.ref_f32_to_f16(float(v)) for v in np.asarray(vals, np.float32).ravel()], np.uint16)

    def unary(self, name, vals):
        f = getattr(self.lib, "ref_" + name)
        return np.array([f(float(v)) for v in np.asarray(vals, np.float32).ravel()], np.float32)

    def grids(self):
        g3 = np.array([self.lib.ref_iq3s_grid(i) for i in range(512)], np.uint32)
        g2 = np.array([self.lib.ref_iq2s_grid(i) for i in range(1024)], np.uint64)
        return g3, g2

    def quantize_q8_0(self, x):
        x = np.ascontiguousarray(x, np.float32)
        out = np.zeros(x.size // 32 * 34, np.uint8)
        self.lib.ref_quantize_q8_0(x.ctypes.data, out.ctypes.data, x.size // 32)
        return out

    def quantize_q8_K(self, x):
        x = np.ascontiguousarray(x, np.float32)
        out = np.zeros(x.size // 256 * Q8K_BYTES, np.uint8)
        self.lib.ref_quantize_q8_K(x.ctypes.data, out.ctypes.data, x.size // 256)
        return out

    def row(self, t, w_row, y, cols, variant=0):
        w_row = np.ascontiguousarray(w_row, np.uint8)
        y = np.ascontiguousarray(y, np.uint8)
        f = {TYPE_IQ3_S: self.lib.ref_row_iq3_s_q8_K, TYPE_IQ2_S: self.lib.ref_row_iq2_s_q8_K,
             TYPE_Q8_0: self.lib.ref_row_q8_0_q8_0, TYPE_IQ4_NL: self.lib.ref_row_iq4_nl_q8_0}[t]
        return np.float32(f(w_row.ctypes.data, y.ctypes.data, cols, variant))

    def dot_f32(self, a, b):
        a = np.ascontiguousarray(a, np.float32)
        b = np.ascontiguousarray(b, np.float32)
        return np.float32(self.lib.ref_dot_f32(a.ctypes.data, b.ctypes.data, a.size))

    def requantize_rows_to_q8_0(self, t, blob, rows, cols):
        blob = np.ascontiguousarray(blob, np.uint8)
        rb = cols // 32 * 34 if t == TYPE_Q8_0 else cols // 256 * 210
        out = np.zeros(rows * (cols // 32) * 34, np.uint8)
        for r in range(rows):
            rc = self.lib.ref_requantize_row_to_q8_0(t, blob.ctypes.data + r * rb, out.ctypes.data + r * (cols // 32) * 34, cols)
            if rc != 0:
                raise RuntimeError("ggml_requantize_row_to_q8_0 threw")
        return out

    def router(self, logits, k, w_scale=1.0):
        logits = np.ascontiguousarray(logits, np.float32)
        n = logits.size
        probs = np.zeros(n, np.float32)
        ids = np.zeros(k, np.int32)
        w = np.zeros(k, np.float32)
        self.lib.ref_router_exact(logits.ctypes.data, n, k, w_scale, probs.ctypes.data, ids.ctypes.data,
                                  w.ctypes.data)
        return probs, ids, w

    def threads(self):
        return int(self.lib.ref_hardware_threads())

    def moe_block(self, m, x, threads=None):
        keep = []

        def u8(a):
            if a is None:
                return None
            a = np.ascontiguousarray(a, np.uint8)
            keep.append(a)
            return a.ctypes.data_as(_u8p)

        def f32(a):
            if a is None:
                return None
            a = np.ascontiguousarray(a, np.float32)
            keep.append(a)
            return a.ctypes.data_as(_f32p)

        w = MoeWeightsC(m["hidden"], m["expert_ffn"], m.get("shared_ffn", 0), m["n_experts"], m["top_k"],
                        m["gate_type"], m["up_type"], m["down_type"], m.get("w_scale", 1.0),
                        u8(m.get("router")), f32(m.get("router_bias")), u8(m["gate"]), u8(m["up"]), u8(m["down"]),
                        f32(m.get("shared_gate_vec")), u8(m.get("shared_gate")), u8(m.get("shared_up")),
                        u8(m.get("shared_down")), f32(m.get("router_f32")))
        H, E, K = m["hidden"], m["n_experts"], m["top_k"]
        ids = np.zeros(K, np.int32)
        wts = np.zeros(K, np.float32)
        logits = np.zeros(E, np.float32)
        out = np.zeros(H, np.float32)
        x = np.ascontiguousarray(x, np.float32)
        rc = self.lib.ref_moe_block(C.byref(w), x.ctypes.data, threads or self.threads(), ids.ctypes.data,
                                    wts.ctypes.data, logits.ctypes.data, out.ctypes.data)
        if rc != 0:
            raise RuntimeError(f"ref_moe_block failed: {rc}")
        return {"ids": ids, "weights": wts, "logits": logits, "out": out}


# ---------------------------------------------------------------------------
# seeded synthetic data shared by the CPU and GPU tests
# ---------------------------------------------------------------------------
def random_blocks(rng, t, nblocks):
    """Random block bytes with a normal f16 scale in [0.0005, 0.05], the way the reference's
    host tests fill rows (tests/qwen38_cpu_moe_host_test.cpp:72-119)."""
    bb = BLOCK_BYTES[t]
    raw = rng.integers(0, 256, size=(nblocks, bb), dtype=np.uint8)
    d = rng.uniform(0.0005, 0.05, size=nblocks).astype(np.float16)
    raw[:, 0:2] = d.view(np.uint8).reshape(nblocks, 2)
    return raw.reshape(-1)


def adversarial_logits(rng, n, kind):
    """Router rows aimed at the hard branches: the patterns of the reference's
    tests/router_parallel_exact_test.cu:36-76 and tests/qwen38_router_host_test.cpp:181-295."""
    u = lambda lo, hi, size=None: np.float32(rng.uniform(lo, hi, size))
    x = np.zeros(n, np.float32)
    if kind == "normal":
        x = rng.standard_normal(n).astype(np.float32)
    elif kind == "const":
        x[:] = 0.25
    elif kind == "alphabet":
        x = rng.integers(0, 4, n).astype(np.float32) - 1.5
    elif kind == "large":
        x = np.where(rng.random(n) < 0.5, -1, 1).astype(np.float32) * (80 + 60 * rng.random(n)).astype(np.float32)
    elif kind == "tiny":
        x = np.where(rng.random(n) < 0.5, -1, 1).astype(np.float32) * np.float32(1e-30)
    elif kind == "zeros_denormals":
        x = np.array([0.0, -0.0, 1e-38] * (n // 3 + 1), np.float32)[:n]
    elif kind == "some_neg_inf":
        x = rng.standard_normal(n).astype(np.float32)
        x[::7] = -np.inf
    elif kind == "all_pos_inf":
        x[:] = np.inf
    elif kind == "all_neg_inf":
        x[:] = -np.inf
    elif kind == "one_winner":
        x[:] = -120.0
        x[n // 3] = 0.5
    elif kind == "small_normal":
        x = (rng.standard_normal(n) * 0.1).astype(np.float32)
    elif kind == "model_range":
        x = u(-14, -1, n)
    elif kind == "near_tie":
        x = u(-30, -15, n)
        base = u(-6, -2)
        for i in range(min(24, n)):
            x[i] = base + u(-1e-6, 1e-6) * (1 + i % 5)
        for _ in range(24):
            a, b = rng.integers(0, min(24, n), 2)
            x[a] = x[b]
    elif kind == "extremes":
        for i in range(n):
            x[i] = [-np.inf, u(-100, -88), u(-1e30, -1e20), 0.0, u(0, 80), -0.0,
                    np.float32(2.0 ** -149), u(-20, -5)][i % 8]
    elif kind == "hot":
        x = u(-0.5, 60, n)
    elif kind == "max_first":
        x = u(-12, -4, n)
        x[0] = 0.0
    elif kind == "max_last":
        x = u(-12, -4, n)
        x[0] = -12.0
        x[n - 1] = 0.0
    elif kind == "one_finite":
        x[:] = -np.inf
        x[n // 2] = u(-5, -1)
    elif kind == "all_underflow":
        x[:] = -1.0e30
    elif kind == "prob_tie":
        x = u(-25, -18, n)
        for i in range(min(40, n)):
            x[i] = np.float32(-3.0) + np.float32(i % 3) * np.float32(1.1920929e-7 * 0.5)
    elif kind == "nan_mixed":
        x = rng.standard_normal(n).astype(np.float32)
        x[5::11] = np.nan
    else:
        raise ValueError(kind)
    return np.ascontiguousarray(x, np.float32)


ADVERSARIAL_KINDS = ["normal", "const", "alphabet", "large", "tiny", "zeros_denormals", "some_neg_inf",
                     "all_pos_inf", "all_neg_inf", "one_winner", "small_normal", "model_range", "near_tie",
                     "extremes", "hot", "max_first", "max_last", "one_finite", "all_underflow", "prob_tie",
                     "nan_mixed"]
