"""Seeded synthetic models in ggml block formats, and a minimal GGUF v3 writer.

The reference never quantises weights itself (its tests fill blocks with random
bytes, tests/qwen38_cpu_moe_host_test.cpp:72-119), and parity for the MoE path is
defined on the dot products *given the block bytes*. The encoders here are this
project's own deterministic ones: they produce valid Q8_0 / Q4_0 / IQ3_S / IQ2_S
blocks (layouts: src/gguf.hpp:293-306, src/lowbit.cuh:1359-1363, :1045-1048 of the
reference) from N(0, sigma) weights, so the CPU oracle and the CUDA path can be fed
the same bytes. They do not claim to reproduce ggml's own quantiser choices.

Host-side, numpy only; sized for test-scale models. Full-size models are generated
on the device by the wd_synth_* entry points of the C ABI.
"""
import os
import re
import struct

import numpy as np

TYPE_F32, TYPE_Q4_0, TYPE_Q8_0, TYPE_IQ4_NL, TYPE_IQ3_S, TYPE_IQ2_S = 0, 2, 8, 20, 21, 22
BLOCK_BYTES = {TYPE_Q8_0: 34, TYPE_Q4_0: 18, TYPE_IQ4_NL: 18, TYPE_IQ3_S: 110, TYPE_IQ2_S: 82}
BLOCK_ELEMS = {TYPE_Q8_0: 32, TYPE_Q4_0: 32, TYPE_IQ4_NL: 32, TYPE_IQ3_S: 256, TYPE_IQ2_S: 256}

_HERE = os.path.dirname(os.path.abspath(__file__))
_grid_cache = {}


def row_bytes(t, cols):
    if t == TYPE_F32:
        return cols * 4
    assert cols % BLOCK_ELEMS[t] == 0
    return cols // BLOCK_ELEMS[t] * BLOCK_BYTES[t]


def grids():
    """(iq3s [512,4] uint8 magnitudes, iq2s [1024,8] uint8 magnitudes) from csrc/wd_grids.h."""
    if "g" not in _grid_cache:
        txt = open(os.path.join(_HERE, "csrc", "wd_grids.h")).read()

        def arr(name):
            body = txt[txt.index(name + "["):]
            body = body[body.index("{") + 1:body.index("};")]
            return np.array([int(v, 16) for v in re.findall(r"0x[0-9a-fA-F]+", body)], np.uint32)

        p3, p2 = arr("wd_iq3s_grid_packed"), arr("wd_iq2s_grid_packed")
        g3 = np.stack([2 * ((p3 >> (3 * j)) & 7) + 1 for j in range(4)], 1).astype(np.uint8)
        c2 = np.stack([(p2 >> (2 * j)) & 3 for j in range(8)], 1)
        g2 = (8 + 17 * c2 + (c2 == 2)).astype(np.uint8)
        _grid_cache["g"] = (g3, g2)
    return _grid_cache["g"]


# ---------------------------------------------------------------------------
# encoders (weights [rows, cols] float32 -> uint8 [rows, row_bytes])
# ---------------------------------------------------------------------------
def quantize_q8_0(w):
    w = np.ascontiguousarray(w, np.float32)
    rows, cols = w.shape
    b = w.reshape(rows, cols // 32, 32)
    amax = np.abs(b).max(-1)
    d = (amax / np.float32(127)).astype(np.float16)
    df = d.astype(np.float32)
    inv = np.where(df > 0, np.float32(1) / np.where(df > 0, df, 1), 0).astype(np.float32)
    q = np.clip(np.rint(b * inv[..., None]), -127, 127).astype(np.int8)
    out = np.zeros((rows, cols // 32, 34), np.uint8)
    out[..., 0:2] = d.view(np.uint8).reshape(rows, cols // 32, 2)
    out[..., 2:] = q.view(np.uint8)
    return out.reshape(rows, -1)


def quantize_q4_0(w):
    w = np.ascontiguousarray(w, np.float32)
    rows, cols = w.shape
    b = w.reshape(rows, cols // 32, 32)
    idx = np.abs(b).argmax(-1)
    mx = np.take_along_axis(b, idx[..., None], -1)[..., 0]
    d = (mx / np.float32(-8)).astype(np.float16)
    df = d.astype(np.float32)
    inv = np.where(df != 0, np.float32(1) / np.where(df != 0, df, 1), 0).astype(np.float32)
    q = np.clip(np.floor(b * inv[..., None] + np.float32(8.5)), 0, 15).astype(np.uint8)
    out = np.zeros((rows, cols // 32, 18), np.uint8)
    out[..., 0:2] = d.view(np.uint8).reshape(rows, cols // 32, 2)
    out[..., 2:] = q[..., :16] | (q[..., 16:] << 4)
    return out.reshape(rows, -1)


def _iq3s_cell_lut():
    """Nearest codebook entry for each of 16^4 cells of the magnitude cube [0,16)^4."""
    if "lut3" not in _grid_cache:
        g3 = grids()[0].astype(np.float32)
        centres = np.stack(np.meshgrid(*[np.arange(16, dtype=np.float32) + 0.5] * 4, indexing="ij"), -1).reshape(-1, 4)
        lut = np.zeros(65536, np.uint16)
        for s in range(0, 65536, 4096):
            c = centres[s:s + 4096]
            d2 = ((c[:, None, :] - g3[None]) ** 2).sum(-1)
            lut[s:s + 4096] = d2.argmin(1)
        _grid_cache["lut3"] = lut
    return _grid_cache["lut3"]


def quantize_iq3_s(w):
    """value(ib32, c, j) = d * (1 + 2*s4[ib32]) * (+-grid[idx][j]); see the block layout in
    src/lowbit.cuh:1359-1363 of the reference: d(2) qs(64) qh(8) signs(32) scales(4)."""
    w = np.ascontiguousarray(w, np.float32)
    rows, cols = w.shape
    nb = cols // 256
    b = w.reshape(rows, nb, 8, 8, 4)                      # [row, sb, ib32, chunk, j]
    a = np.abs(b)
    sub_max = a.reshape(rows, nb, 8, 32).max(-1)          # per 32-value sub-block
    sigma = sub_max / np.float32(13.0)                    # target size of one magnitude unit
    d = (sigma.max(-1) / np.float32(31.0)).astype(np.float16)
    df = d.astype(np.float32)
    safe = np.where(df > 0, df, 1).astype(np.float32)
    s4 = np.clip(np.rint((sigma / safe[..., None] - 1) / 2), 0, 15).astype(np.uint8)
    s4 = np.where(df[..., None] > 0, s4, 0).astype(np.uint8)
    unit = safe[..., None] * (1 + 2 * s4.astype(np.float32))          # [row, sb, ib32]
    t = np.clip(a / unit[..., None, None], 0, np.float32(15.999))
    cell = np.floor(t).astype(np.uint32)
    code = (cell[..., 0] << 12) | (cell[..., 1] << 8) | (cell[..., 2] << 4) | cell[..., 3]
    idx = _iq3s_cell_lut()[code]                          # [row, sb, ib32, chunk] 9-bit
    neg = (b < 0).astype(np.uint8)                        # [row, sb, ib32, chunk, j]
    out = np.zeros((rows, nb, 110), np.uint8)
    out[..., 0:2] = d.view(np.uint8).reshape(rows, nb, 2)
    out[..., 2:66] = (idx & 0xff).astype(np.uint8).reshape(rows, nb, 64)
    hb = ((idx >> 8) & 1).astype(np.uint8)                # bit c of qh[ib32]
    out[..., 66:74] = (hb << np.arange(8, dtype=np.uint8)).sum(-1).astype(np.uint8)
    nib = (neg << np.arange(4, dtype=np.uint8)).sum(-1).astype(np.uint8)   # [row, sb, ib32, chunk]
    sg = nib[..., 0::2] | (nib[..., 1::2] << 4)           # byte g holds chunks 2g (low), 2g+1 (high)
    out[..., 74:106] = sg.reshape(rows, nb, 32)
    out[..., 106:110] = s4[..., 0::2] | (s4[..., 1::2] << 4)
    return out.reshape(rows, -1)


def _iq2s_cell_lut():
    if "lut2" not in _grid_cache:
        g2 = grids()[1].astype(np.float32)
        levels = np.array([8, 25, 43], np.float32)
        cells = np.stack(np.meshgrid(*[levels] * 8, indexing="ij"), -1).reshape(-1, 8)
        lut = np.zeros(cells.shape[0], np.uint16)
        for s in range(0, cells.shape[0], 729):
            c = cells[s:s + 729]
            lut[s:s + 729] = ((c[:, None, :] - g2[None]) ** 2).sum(-1).argmin(1)
        _grid_cache["lut2"] = lut
    return _grid_cache["lut2"]


def quantize_iq2_s(w):
    """value = d * (1 + 2*s4) * (+-grid[idx][j]) / 8; layout d(2) qs(32) signs(32) qh(8) scales(8)
    (src/lowbit.cuh:1045-1048 of the reference). Values 0..15 of a sub-block use the low scale
    nibble, values 16..31 the high one."""
    w = np.ascontiguousarray(w, np.float32)
    rows, cols = w.shape
    nb = cols // 256
    b = w.reshape(rows, nb, 8, 2, 2, 8)                   # [row, sb, ib32, half16, group, j8]
    a = np.abs(b)
    half_max = a.reshape(rows, nb, 8, 2, 16).max(-1)
    sigma = half_max / np.float32(43.0) * np.float32(8.0)
    d = (sigma.max((-1, -2)) / np.float32(31.0)).astype(np.float16)
    df = d.astype(np.float32)
    safe = np.where(df > 0, df, 1).astype(np.float32)
    s4 = np.clip(np.rint((sigma / safe[..., None, None] - 1) / 2), 0, 15).astype(np.uint8)
    s4 = np.where(df[..., None, None] > 0, s4, 0).astype(np.uint8)
    unit = safe[..., None, None] * (1 + 2 * s4.astype(np.float32)) / np.float32(8.0)
    t = a / unit[..., None, None]
    lvl = (t > 16.5).astype(np.uint32) + (t > 34.0).astype(np.uint32)     # nearest of 8 / 25 / 43
    code = np.zeros(lvl.shape[:-1], np.uint32)
    for j in range(8):
        code = code * 3 + lvl[..., j]
    idx = _iq2s_cell_lut()[code].reshape(rows, nb, 8, 4)  # group g = half16*2 + group
    neg = (b < 0).astype(np.uint8).reshape(rows, nb, 8, 4, 8)
    out = np.zeros((rows, nb, 82), np.uint8)
    out[..., 0:2] = d.view(np.uint8).reshape(rows, nb, 2)
    out[..., 2:34] = (idx & 0xff).astype(np.uint8).reshape(rows, nb, 32)
    out[..., 34:66] = (neg << np.arange(8, dtype=np.uint8)).sum(-1).astype(np.uint8).reshape(rows, nb, 32)
    hi = ((idx >> 8) & 3).astype(np.uint8)
    out[..., 66:74] = (hi << (2 * np.arange(4, dtype=np.uint8))).sum(-1).astype(np.uint8)
    out[..., 74:82] = s4[..., 0] | (s4[..., 1] << 4)
    return out.reshape(rows, -1)


IQ4_NL_VALUES = np.array([-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113], np.int8)


def quantize_iq4_nl(w):
    """IQ4_NL: per block of 32 an f16 scale d = max|w| / 127 and the nearest of the sixteen codebook values;
    byte j holds value j in its low nibble and value j + 16 in its high nibble (src/qwen38_cpu_moe.cuh:377-422)."""
    w = np.ascontiguousarray(w, np.float32)
    rows, cols = w.shape
    b = w.reshape(rows, cols // 32, 32)
    d = (np.abs(b).max(-1) / np.float32(127)).astype(np.float16)
    df = d.astype(np.float32)
    inv = np.where(df > 0, 1 / np.where(df > 0, df, 1), 0).astype(np.float32)
    idx = np.abs((b * inv[..., None])[..., None] - IQ4_NL_VALUES.astype(np.float32)).argmin(-1).astype(np.uint8)
    out = np.empty((rows, cols // 32, 18), np.uint8)
    out[..., 0:2] = d.view(np.uint8).reshape(rows, cols // 32, 2)
    out[..., 2:] = idx[..., :16] | (idx[..., 16:] << 4)
    return out.reshape(rows, -1)


QUANTIZERS = {TYPE_Q8_0: quantize_q8_0, TYPE_Q4_0: quantize_q4_0, TYPE_IQ3_S: quantize_iq3_s,
              TYPE_IQ2_S: quantize_iq2_s, TYPE_IQ4_NL: quantize_iq4_nl}


def random_blocks(rng, t, nblocks):
    """Random block bytes with an f16 scale in [0.0005, 0.05]: valid input for every row product, and the cheapest way
    to fill a full-size tensor of a type that has no encoder on the device."""
    raw = rng.integers(0, 256, size=(nblocks, BLOCK_BYTES[t]), dtype=np.uint8)
    raw[:, 0:2] = rng.uniform(0.0005, 0.05, size=nblocks).astype(np.float16).view(np.uint8).reshape(nblocks, 2)
    return raw.reshape(-1)


def dequantize(t, blob, rows, cols):
    """Reference decoder for the encoders' own tests."""
    blob = np.ascontiguousarray(blob, np.uint8).reshape(rows, cols // BLOCK_ELEMS[t], BLOCK_BYTES[t])
    d = blob[..., 0:2].copy().view(np.float16)[..., 0].astype(np.float32)
    if t == TYPE_Q8_0:
        return (blob[..., 2:].view(np.int8).astype(np.float32) * d[..., None]).reshape(rows, cols)
    if t == TYPE_Q4_0:
        q = blob[..., 2:]
        v = np.concatenate([(q & 15), (q >> 4)], -1).astype(np.float32) - 8
        return (v * d[..., None]).reshape(rows, cols)
    if t == TYPE_IQ4_NL:
        q = blob[..., 2:]
        v = IQ4_NL_VALUES[np.concatenate([(q & 15), (q >> 4)], -1)].astype(np.float32)
        return (v * d[..., None]).reshape(rows, cols)
    g3, g2 = grids()
    if t == TYPE_IQ3_S:
        qs = blob[..., 2:66].reshape(rows, -1, 8, 8).astype(np.uint32)
        qh = blob[..., 66:74].astype(np.uint32)
        idx = qs | (((qh[..., None] >> np.arange(8)) & 1) << 8)
        mag = g3[idx].astype(np.float32)                                       # [row, sb, ib, c, 4]
        sg = blob[..., 74:106].reshape(rows, -1, 8, 4)
        nib = np.stack([sg & 15, sg >> 4], -1).reshape(rows, -1, 8, 8)
        sign = 1 - 2 * ((nib[..., None] >> np.arange(4)) & 1).astype(np.float32)
        sc = blob[..., 106:110]
        s4 = np.stack([sc & 15, sc >> 4], -1).reshape(rows, -1, 8).astype(np.float32)
        return (mag * sign * (d[..., None] * (1 + 2 * s4))[..., None, None]).reshape(rows, cols)
    if t == TYPE_IQ2_S:
        qs = blob[..., 2:34].reshape(rows, -1, 8, 4).astype(np.uint32)
        sg = blob[..., 34:66].reshape(rows, -1, 8, 4)
        qh = blob[..., 66:74].astype(np.uint32)
        idx = qs | (((qh[..., None] >> (2 * np.arange(4))) & 3) << 8)
        mag = g2[idx].astype(np.float32)                                       # [row, sb, ib, g, 8]
        sign = 1 - 2 * ((sg[..., None] >> np.arange(8)) & 1).astype(np.float32)
        sc = blob[..., 74:82]
        s4 = np.stack([sc & 15, sc >> 4], -1).astype(np.float32)               # [row, sb, ib, half16]
        s4g = np.repeat(s4, 2, -1)                                             # per group
        return (mag * sign * (d[..., None, None] * (1 + 2 * s4g) / 8)[..., None]).reshape(rows, cols)
    raise ValueError(t)


# ---------------------------------------------------------------------------
# synthetic MoE block
# ---------------------------------------------------------------------------
def make_moe_block(seed, hidden, expert_ffn, n_experts, top_k, shared_ffn=None, expert_type=TYPE_IQ3_S,
                   down_type=None, sigma=0.02, bias_sigma=0.0, w_scale=1.0, router_f32=False):
    """One block's weights in ggml layout, N(0, sigma) from `seed`, in a fixed tensor order:
    router, gate, up, down, shared gate vector, shared gate/up/down, router bias. `router_f32`: the router stays
    F32 [E][H] under the key "router_f32" (the reference model's ffn_gate_inp) instead of Q8_0 under "router"."""
    rng = np.random.Generator(np.random.PCG64(seed))
    shared_ffn = expert_ffn if shared_ffn is None else shared_ffn
    down_type = expert_type if down_type is None else down_type
    H, F, E = hidden, expert_ffn, n_experts

    def normal(shape):
        return (rng.standard_normal(shape, dtype=np.float32) * np.float32(sigma))

    m = dict(hidden=H, expert_ffn=F, shared_ffn=shared_ffn, n_experts=E, top_k=top_k,
             gate_type=expert_type, up_type=expert_type, down_type=down_type, w_scale=w_scale)
    if router_f32:
        m["router_f32"] = normal((E, H)).reshape(-1)
    else:
        m["router"] = quantize_q8_0(normal((E, H))).reshape(-1)
    qe, qd = QUANTIZERS[expert_type], QUANTIZERS[down_type]
    m["gate"] = np.concatenate([qe(normal((F, H))).reshape(-1) for _ in range(E)])
    m["up"] = np.concatenate([qe(normal((F, H))).reshape(-1) for _ in range(E)])
    m["down"] = np.concatenate([qd(normal((H, F))).reshape(-1) for _ in range(E)])
    if shared_ffn:
        m["shared_gate_vec"] = normal((H,))
        m["shared_gate"] = quantize_q8_0(normal((shared_ffn, H))).reshape(-1)
        m["shared_up"] = quantize_q8_0(normal((shared_ffn, H))).reshape(-1)
        m["shared_down"] = quantize_q8_0(normal((H, shared_ffn))).reshape(-1)
    if bias_sigma > 0:
        m["router_bias"] = (rng.standard_normal(E, dtype=np.float32) * np.float32(bias_sigma))
    return m


# ---------------------------------------------------------------------------
# GGUF v3 writer (the subset the loader reads: scalar / string / int-array metadata, tensors)
# ---------------------------------------------------------------------------
_GGUF_U32, _GGUF_F32, _GGUF_STR, _GGUF_ARR, _GGUF_U64, _GGUF_I32 = 4, 6, 8, 9, 10, 5


def _gs(s):
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def write_gguf(path, metadata, tensors, alignment=32):
    """metadata: {key: int | float | str | list[int]}; tensors: list of (name, dims, type, uint8/float32 bytes)
    with dims in GGUF order [cols, rows(, experts)]."""
    head = struct.pack("<IIQQ", 0x46554747, 3, len(tensors), len(metadata))
    for k, v in metadata.items():
        head += _gs(k)
        if isinstance(v, bool):
            head += struct.pack("<IB", 7, int(v))
        elif isinstance(v, int):
            head += struct.pack("<II", _GGUF_U32, v) if 0 <= v < 2 ** 32 else struct.pack("<IQ", _GGUF_U64, v)
        elif isinstance(v, float):
            head += struct.pack("<If", _GGUF_F32, v)
        elif isinstance(v, str):
            head += struct.pack("<I", _GGUF_STR) + _gs(v)
        elif isinstance(v, (list, tuple)):
            head += struct.pack("<IIQ", _GGUF_ARR, _GGUF_I32, len(v)) + struct.pack(f"<{len(v)}i", *v)
        else:
            raise TypeError(k)
    offs, off = [], 0
    for name, dims, t, data in tensors:
        offs.append(off)
        off = (off + data.nbytes + alignment - 1) // alignment * alignment
    for (name, dims, t, data), o in zip(tensors, offs):
        head += _gs(name) + struct.pack("<I", len(dims)) + struct.pack(f"<{len(dims)}Q", *dims)
        head += struct.pack("<IQ", t, o)
    pad = (-len(head)) % alignment
    with open(path, "wb") as f:
        f.write(head + b"\0" * pad)
        for (name, dims, t, data), o in zip(tensors, offs):
            f.write(np.ascontiguousarray(data).tobytes())
            f.write(b"\0" * ((-data.nbytes) % alignment))


def moe_block_tensors(m, layer, fused=False):
    """GGUF tensor list for one block, named as the reference loader expects
    (src/qwen38_moe.cuh:569-573, :601-612). `fused`: gate and up as ONE tensor ffn_gate_up_exps [H, 2F, E], each
    expert's gate rows followed by its up rows."""
    p = f"blk.{layer}."
    H, F, E, SF = m["hidden"], m["expert_ffn"], m["n_experts"], m["shared_ffn"]
    router = (p + "ffn_gate_inp.weight", [H, E], TYPE_F32, m["router_f32"]) if "router_f32" in m else \
        (p + "ffn_gate_inp.weight", [H, E], TYPE_Q8_0, m["router"])
    t = [router,
         (p + "ffn_gate_exps.weight", [H, F, E], m["gate_type"], m["gate"]),
         (p + "ffn_up_exps.weight", [H, F, E], m["up_type"], m["up"]),
         (p + "ffn_down_exps.weight", [F, H, E], m["down_type"], m["down"])]
    if fused:
        assert m["gate_type"] == m["up_type"]
        g = np.ascontiguousarray(m["gate"], np.uint8).reshape(E, -1)
        u = np.ascontiguousarray(m["up"], np.uint8).reshape(E, -1)
        t[1:3] = [(p + "ffn_gate_up_exps.weight", [H, 2 * F, E], m["gate_type"], np.concatenate([g, u], 1).reshape(-1))]
    if SF:
        t += [(p + "ffn_gate_inp_shexp.weight", [H], TYPE_F32, m["shared_gate_vec"]),
              (p + "ffn_gate_shexp.weight", [H, SF], TYPE_Q8_0, m["shared_gate"]),
              (p + "ffn_up_shexp.weight", [H, SF], TYPE_Q8_0, m["shared_up"]),
              (p + "ffn_down_shexp.weight", [SF, H], TYPE_Q8_0, m["shared_down"])]
    if "router_bias" in m:
        t.append((p + "ffn_gate_inp.bias", [E], TYPE_F32, m["router_bias"]))
    return t
