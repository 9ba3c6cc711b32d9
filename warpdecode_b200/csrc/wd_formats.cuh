// Device-resident weight formats and their decoders.
//
// Weights arrive in ggml block layout (GGUF) and are repacked ONCE, when an expert enters a
// cache slot or a dense matrix is uploaded, into layouts whose shared-memory reads are
// conflict-free vector loads. The repack is a pure permutation of the same bits: a repacked
// IQ3_S block is still 110 bytes per 256 weights, a Q8_0 block 34 per 32.
//
// IQ3_S "tile" = 32 consecutive blocks of the row-major block sequence of a matrix (block
// index = row * nsb + sb, nsb = cols / 256), one block per lane, stored as planes:
//   QS  off    0: [sub-block i=0..7][lane][8 B]  the eight index bytes of sub-block i
//   SG  off 2048: [sub-block i][lane][4 B]       sign word: sign of (chunk c, value j) at bit 8j + 7 - c
//   HB  off 3072: [lane][8 B]                    byte i = ninth index bits of sub-block i (bit c = chunk c)
//   SC  off 3328: [lane][4 B]                    scale nibbles, unchanged
//   D   off 3456: [lane][2 B]                    f16 block scale
// (ggml's own layout of the same fields: src/lowbit.cuh:1359-1363 of the reference.)
// The decoder walks the eight sub-blocks in a loop, so its code stays a few KB: the kernel executes
// every instruction only a handful of times per launch and is otherwise bound by instruction fetch.
//
// IQ2_S tile (82 B per block, 2624 B per 32 blocks; ggml fields d(2) qs(32) signs(32) qh(8) scales(8),
// src/lowbit.cuh:1045-1048):
//   QS  off    0: [sub-block i][lane][4 B]  the four index bytes of sub-block i (one per pair of chunks)
//   SG  off 1024: [sub-block i][lane][4 B]  sign word, same arrangement as IQ3_S
//   QH  off 2048: [lane][8 B]               byte i = the four 2-bit index extensions of sub-block i
//   SC  off 2304: [lane][8 B]               byte i = scale nibbles of sub-block i (low: chunks 0-3, high: 4-7)
//   D   off 2560: [lane][2 B]               f16 block scale
// Its codebook (1024 entries of eight magnitudes) is a plain 8 KB shared-memory table.
//
// Q8_0 "task" = 4 consecutive rows of nb = cols / 32 blocks (nb a multiple of 4):
//   QS  [group g = b/4][row r][chunk-lane l][16 B], word i = values 4l..4l+3 of block 4g+i
//   D   off nb*128: [row r][nb] f16
#pragma once

#include "wd_device.cuh"
#include "wd_grids.h"

namespace wd {

constexpr int kIq3TileBytes = 3520;
constexpr int kIq3OffSG = 2048, kIq3OffHB = 3072, kIq3OffSC = 3328, kIq3OffD = 3456;
constexpr int kGridTableBytes = 65536;        // 512 entries x 32 lane-private copies x 4 B
constexpr int kIq2TileBytes = 2624;
constexpr int kIq2OffSG = 1024, kIq2OffQH = 2048, kIq2OffSC = 2304, kIq2OffD = 2560;
constexpr int kIq2TableBytes = 8192;          // 1024 entries x 8 B
constexpr int kTypeIq3s = 21, kTypeIq2s = 22; // ggml type ids (src/gguf.hpp:26-44)

__host__ __device__ constexpr int iq_tile_bytes(int type) { return type == kTypeIq2s ? kIq2TileBytes : kIq3TileBytes; }
__host__ __device__ constexpr int iq_block_bytes(int type) { return type == kTypeIq2s ? 82 : 110; }
__host__ __device__ constexpr int iq_tile_off_d(int type) { return type == kTypeIq2s ? kIq2OffD : kIq3OffD; }
// factor applied to a finished row sum (ggml's IQ2_S row dot ends with * 0.125, src/qwen38_cpu_moe.cuh:298-335)
__host__ __device__ constexpr float iq_row_post(int type) { return type == kTypeIq2s ? 0.125f : 1.0f; }
constexpr int kActSbStride = 272;             // 256 int8 + 16 pad: the 8 superblocks of a row hit 8 bank groups

// Lane-private copy of the IQ3_S codebook: entry idx = byte | h << 8 for lane L lives at byte
// offset byte*256 + h*128 + L*4, so the 32 lanes of a warp always hit 32 different banks.
// Each lane expands one entry; the warp then writes whole 128-byte rows (no bank conflicts).
__device__ __noinline__ void build_grid_table(uint8_t *tab, const uint16_t *packed_global) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    uint32_t *t = reinterpret_cast<uint32_t *>(tab);
    for (int base = warp * 32; base < 512; base += nw * 32) {
        const int e = base + lane;                               // e = byte*2 + h
        const uint32_t p = packed_global[(e >> 1) | ((e & 1) << 8)];
        uint32_t v = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) v |= (2u * ((p >> (3 * j)) & 7u) + 1u) << (8 * j);
#pragma unroll 8
        for (int i = 0; i < 32; ++i) t[(base + i) * 32 + lane] = __shfl_sync(0xffffffffu, v, i);
    }
}

// IQ2_S codebook, expanded from the packed table in global memory.
__device__ __noinline__ void build_iq2_table(uint8_t *tab2, const uint16_t *packed_global) {
    uint64_t *t = reinterpret_cast<uint64_t *>(tab2);
#pragma unroll 1
    for (int e = threadIdx.x; e < 1024; e += blockDim.x) t[e] = wd_iq2s_unpack(packed_global[e]);
}

// prmt.b32 with the full 4-bit selector nibbles: bit 3 of a nibble replicates the sign bit of the
// selected byte over the whole result byte (the __byte_perm intrinsic only documents 3 bits).
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}

__device__ __forceinline__ uint32_t word_of(const uint4 &v, int i) {
    return i == 0 ? v.x : (i == 1 ? v.y : (i == 2 ? v.z : v.w));
}

// One chunk (4 weights): table lookup, sign application, dp4a.
__device__ __forceinline__ int iq3_chunk_dot(uint32_t addr, uint32_t sword_shifted, int a_word,
                                             const uint8_t *tab) {
    const uint32_t g = *reinterpret_cast<const uint32_t *>(tab + addr);
    const uint32_t m = prmt(sword_shifted, 0u, 0xba98u);            // 0xff where the value is negative
    const uint32_t neg = 0x01010100u - g;                           // per-byte two's complement (g bytes >= 1)
    const uint32_t sgn = (g & ~m) | (neg & m);
    return dp4a_s8(a_word, static_cast<int>(sgn), 0);
}

// Per-block constants a lane keeps in registers while it walks the sub-blocks.
struct Iq3Head {
    uint2 hb;        // ninth index bits, one byte per sub-block
    uint32_t sc;     // scale nibbles
};

__device__ __forceinline__ void iq3_head(const uint8_t *tile, int lane, Iq3Head &h) {
    h.hb = *reinterpret_cast<const uint2 *>(tile + kIq3OffHB + lane * 8);
    h.sc = *reinterpret_cast<const uint32_t *>(tile + kIq3OffSC + lane * 4);
}

// Sub-block i of one block: partial[c] += ls * dot(a[chunk c], +-grid[idx c]) for the 8 chunks
// (the integer arithmetic of src/qwen38_cpu_moe.cuh:352-370).
__device__ __forceinline__ void iq3_subblock(const uint8_t *tile, const Iq3Head &h, int i, int lane,
                                             const uint4 a_lo, const uint4 a_hi, uint32_t lane4x2,
                                             const uint8_t *tab, int partial[8]) {
    const uint2 q = *reinterpret_cast<const uint2 *>(tile + i * 256 + lane * 8);     // .x chunks 0-3, .y chunks 4-7
    const uint32_t sw = *reinterpret_cast<const uint32_t *>(tile + kIq3OffSG + i * 128 + lane * 4);
    const uint32_t hbyte = ((i & 4) ? h.hb.y : h.hb.x) >> (8 * (i & 3));
    const uint32_t y = (hbyte & 0x0fu) | ((hbyte & 0xf0u) << 4);                     // bits 0-3 and 8-11
    const int ls = 1 + 2 * static_cast<int>((h.sc >> (4 * i)) & 15u);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const uint32_t qq = ((y << (7 - k)) & 0x8080u) | lane4x2;   // byte0: chunk k, byte1: chunk k+4
        const uint32_t addr_lo = prmt(q.x, qq, 0x7604u | (k << 4)); // = index byte * 256 + ninth bit * 128 + lane * 4
        const uint32_t addr_hi = prmt(q.y, qq, 0x7605u | (k << 4));
        const int d0 = iq3_chunk_dot(addr_lo, sw << k, static_cast<int>(word_of(a_lo, k)), tab);
        const int d1 = iq3_chunk_dot(addr_hi, sw << (k + 4), static_cast<int>(word_of(a_hi, k)), tab);
        partial[k] += d0 * ls;
        partial[k + 4] += d1 * ls;
    }
}

// Sub-blocks [i0, i1) of one block against the 256 int8 activations at `a` (shared memory, 16-byte aligned).
// UNROLL: sub-blocks decoded per loop iteration. 1 keeps the code small (the single-token kernel runs every instruction
// only a few times per layer and is sensitive to instruction fetch); 8 lets the loads of all sub-blocks run ahead.
template <int UNROLL = 1>
__device__ __forceinline__ void iq3_block_partials_range(const uint8_t *tile, int lane, const uint8_t *a,
                                                         uint32_t lane4x2, const uint8_t *tab, int partial[8], int i0,
                                                         int i1) {
    Iq3Head h;
    iq3_head(tile, lane, h);
#pragma unroll
    for (int c = 0; c < 8; ++c) partial[c] = 0;
    const uint4 *av = reinterpret_cast<const uint4 *>(a);
#pragma unroll(UNROLL)
    for (int i = i0; i < i1; ++i) iq3_subblock(tile, h, i, lane, av[2 * i], av[2 * i + 1], lane4x2, tab, partial);
}

// ---- IQ2_S --------------------------------------------------------------------------------------------
struct Iq2Head {
    uint2 qh;        // index extensions, one byte per sub-block
    uint2 sc;        // scale nibbles, one byte per sub-block
};

// Sub-block i of one IQ2_S block: partial[c] += ls(c) * dot(a[chunk c], +-grid[idx(c >> 1)] half (c & 1))
// (the integer arithmetic of src/qwen38_cpu_moe.cuh:298-335).
__device__ __forceinline__ void iq2_subblock(const uint8_t *tile, const Iq2Head &h, int i, int lane, const uint4 a_lo,
                                             const uint4 a_hi, const uint8_t *tab2, int partial[8]) {
    const uint32_t q = *reinterpret_cast<const uint32_t *>(tile + i * 128 + lane * 4);
    const uint32_t sw = *reinterpret_cast<const uint32_t *>(tile + kIq2OffSG + i * 128 + lane * 4);
    const uint32_t qhb = ((i & 4) ? h.qh.y : h.qh.x) >> (8 * (i & 3));
    const uint32_t scb = ((i & 4) ? h.sc.y : h.sc.x) >> (8 * (i & 3));
    const int ls_lo = 1 + 2 * static_cast<int>(scb & 15u), ls_hi = 1 + 2 * static_cast<int>((scb >> 4) & 15u);
#pragma unroll
    for (int grp = 0; grp < 4; ++grp) {
        const uint32_t idx = ((q >> (8 * grp)) & 0xffu) | (((qhb >> (2 * grp)) & 3u) << 8);
        const uint2 g = *reinterpret_cast<const uint2 *>(tab2 + idx * 8);
        const int c0 = 2 * grp, c1 = c0 + 1;
        const uint32_t a0 = word_of(c0 < 4 ? a_lo : a_hi, c0 & 3), a1 = word_of(c1 < 4 ? a_lo : a_hi, c1 & 3);
        const uint32_t m0 = prmt(sw << c0, 0u, 0xba98u), m1 = prmt(sw << c1, 0u, 0xba98u);
        const uint32_t s0 = (g.x & ~m0) | ((0x01010100u - g.x) & m0), s1 = (g.y & ~m1) | ((0x01010100u - g.y) & m1);
        partial[c0] += dp4a_s8(static_cast<int>(a0), static_cast<int>(s0), 0) * (c0 < 4 ? ls_lo : ls_hi);
        partial[c1] += dp4a_s8(static_cast<int>(a1), static_cast<int>(s1), 0) * (c1 < 4 ? ls_lo : ls_hi);
    }
}

__device__ __forceinline__ void iq2_block_partials_range(const uint8_t *tile, int lane, const uint8_t *a, const uint8_t *tab2,
                                                         int partial[8], int i0, int i1) {
    Iq2Head h;
    h.qh = *reinterpret_cast<const uint2 *>(tile + kIq2OffQH + lane * 8);
    h.sc = *reinterpret_cast<const uint2 *>(tile + kIq2OffSC + lane * 8);
#pragma unroll
    for (int c = 0; c < 8; ++c) partial[c] = 0;
    const uint4 *av = reinterpret_cast<const uint4 *>(a);
#pragma unroll 1
    for (int i = i0; i < i1; ++i) iq2_subblock(tile, h, i, lane, av[2 * i], av[2 * i + 1], tab2, partial);
}

// Full block.
template <int UNROLL = 1>
__device__ __forceinline__ void iq3_block_partials(const uint8_t *tile, int lane, const uint8_t *a, uint32_t lane4x2,
                                                   const uint8_t *tab, int partial[8]) {
    iq3_block_partials_range<UNROLL>(tile, lane, a, lane4x2, tab, partial, 0, 8);
}

}  // namespace wd
