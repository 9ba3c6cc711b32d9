// Device-resident weight formats and their decoders.
//
// Weights arrive in ggml block layout (GGUF) and are repacked ONCE, when an expert enters a
// cache slot or a dense matrix is uploaded, into layouts whose shared-memory reads are
// conflict-free 64/128-bit vector loads. The repack is a pure permutation of the same bits:
// a repacked IQ3_S block is still 110 bytes per 256 weights, a Q8_0 block 34 per 32.
//
// IQ3_S "tile" = 32 consecutive blocks of the row-major block sequence of a matrix (block
// index = row * nsb + sb, nsb = cols / 256), one block per lane, stored as planes:
//   QS  off    0: [pair p=0..3][lane][16 B]  bytes 0-7 = qs of sub-block 2p, 8-15 = of 2p+1
//   SG  off 2048: [quad q=0..1][lane][16 B]  word i = sign word of sub-block 4q+i,
//                                            sign of (chunk c, value j) at bit 8j + 7 - c
//   HB  off 3072: [lane][8 B]                word w covers sub-blocks 4w..4w+3; the 9th index
//                                            bit of (sub-block i, chunk c) sits at bit
//                                            16*((i&3)>>1) + 4*(i&1) + (c&3) + 8*(c>>2)
//   SC  off 3328: [lane][4 B]                scale nibbles, unchanged
//   D   off 3456: [lane][2 B]                f16 block scale
// (ggml's own layout of the same fields: src/lowbit.cuh:1359-1363 of the reference.)
//
// Q8_0 "task" = 4 consecutive rows of nb = cols / 32 blocks (nb a multiple of 4):
//   QS  [group g = b/4][row r][chunk-lane l][16 B], word i = values 4l..4l+3 of block 4g+i
//   D   off nb*128: [row r][nb] f16
#pragma once

#include "wd_device.cuh"

namespace wd {

constexpr int kIq3TileBytes = 3520;
constexpr int kIq3OffSG = 2048, kIq3OffHB = 3072, kIq3OffSC = 3328, kIq3OffD = 3456;
constexpr int kGridTableBytes = 65536;        // 512 entries x 32 lane-private copies x 4 B
constexpr int kActSbStride = 272;             // 256 int8 + 16 pad: the 8 superblocks of a row hit 8 bank groups

// Bit position of the 9th index bit inside its HB word (see the layout comment).
__host__ __device__ constexpr int iq3_hb_bit(int i, int c) {
    return 16 * ((i & 3) >> 1) + 4 * (i & 1) + (c & 3) + 8 * (c >> 2);
}

// Lane-private copy of the IQ3_S codebook: entry idx = byte | h << 8 for lane L lives at byte
// offset byte*256 + h*128 + L*4, so the 32 lanes of a warp always hit 32 different banks.
__device__ __forceinline__ void build_grid_table(uint8_t *tab, const uint16_t *packed_global) {
    for (int e = threadIdx.x; e < 512; e += blockDim.x) {       // e = byte*2 + h
        const int idx = (e >> 1) | ((e & 1) << 8);
        const uint32_t p = packed_global[idx];
        uint32_t v = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) v |= (2u * ((p >> (3 * j)) & 7u) + 1u) << (8 * j);
        uint4 *dst = reinterpret_cast<uint4 *>(tab + e * 128);
#pragma unroll
        for (int i = 0; i < 8; ++i) dst[i] = make_uint4(v, v, v, v);
    }
}

// Integer part of one IQ3_S block against one Q8_K superblock of activations:
// partial[c] = sum over the 8 sub-blocks of ls * dot(a[chunk c], +-grid) exactly as
// src/qwen38_cpu_moe.cuh:337-375 defines it. `tile` is the shared-memory tile, `a` the 256
// int8 activations of this block's superblock (16-byte aligned), `tab` the lane-private table.
struct Iq3Regs {
    uint4 qs[4];
    uint4 sg[2];
    uint2 hb;
    uint32_t sc;
};

__device__ __forceinline__ void iq3_load(const uint8_t *tile, int lane, Iq3Regs &r) {
#pragma unroll
    for (int p = 0; p < 4; ++p) r.qs[p] = *reinterpret_cast<const uint4 *>(tile + p * 512 + lane * 16);
#pragma unroll
    for (int q = 0; q < 2; ++q) r.sg[q] = *reinterpret_cast<const uint4 *>(tile + kIq3OffSG + q * 512 + lane * 16);
    r.hb = *reinterpret_cast<const uint2 *>(tile + kIq3OffHB + lane * 8);
    r.sc = *reinterpret_cast<const uint32_t *>(tile + kIq3OffSC + lane * 4);
}

__device__ __forceinline__ uint32_t word_of(const uint4 &v, int i) {
    return i == 0 ? v.x : (i == 1 ? v.y : (i == 2 ? v.z : v.w));
}

// prmt.b32 with the full 4-bit selector nibbles: bit 3 of a nibble replicates the sign bit of the
// selected byte over the whole result byte (the __byte_perm intrinsic only documents 3 bits).
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}

// One chunk: table lookup, sign application, dp4a.
__device__ __forceinline__ int iq3_chunk_dot(uint32_t addr, uint32_t sword_shifted, int a_word,
                                             const uint8_t *tab) {
    const uint32_t g = *reinterpret_cast<const uint32_t *>(tab + addr);
    const uint32_t m = prmt(sword_shifted, 0u, 0xba98u);      // 0xff where the value is negative
    const uint32_t neg = 0x01010100u - g;                           // per-byte two's complement (g bytes >= 1)
    const uint32_t sgn = (g & ~m) | (neg & m);
    return dp4a_s8(a_word, static_cast<int>(sgn), 0);
}

template <int I>
__device__ __forceinline__ void iq3_subblock(const Iq3Regs &r, const uint4 a_lo, const uint4 a_hi,
                                             uint32_t lane4x2, const uint8_t *tab, int partial[8]) {
    const uint4 &q4 = r.qs[I >> 1];
    const uint32_t qs_lo = (I & 1) ? q4.z : q4.x;     // chunks 0..3
    const uint32_t qs_hi = (I & 1) ? q4.w : q4.y;     // chunks 4..7
    const uint32_t sw = word_of(r.sg[I >> 2], I & 3);
    const uint32_t hw = (I >> 2) ? r.hb.y : r.hb.x;
    const int ls = 1 + 2 * static_cast<int>((r.sc >> (4 * I)) & 15u);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int p = iq3_hb_bit(I, k);               // bit of chunk k; chunk k+4 is 8 above
        const uint32_t sh = p >= 7 ? (hw >> (p - 7)) : (hw << (7 - p));
        const uint32_t q = (sh & 0x8080u) | lane4x2;  // byte0: chunk k, byte1: chunk k+4; bytes 2,3 zero
        const uint32_t addr_lo = prmt(qs_lo, q, 0x7604u | (k << 4));
        const uint32_t addr_hi = prmt(qs_hi, q, 0x7605u | (k << 4));
        const int a0 = static_cast<int>(word_of(a_lo, k));
        const int a1 = static_cast<int>(word_of(a_hi, k));
        const int d0 = iq3_chunk_dot(addr_lo, sw << k, a0, tab);
        const int d1 = iq3_chunk_dot(addr_hi, sw << (k + 4), a1, tab);
        partial[k] += d0 * ls;
        partial[k + 4] += d1 * ls;
    }
}

// Full block. `a` points at this block's superblock of activations in shared memory.
__device__ __forceinline__ void iq3_block_partials(const Iq3Regs &r, const uint8_t *a, uint32_t lane4x2,
                                                   const uint8_t *tab, int partial[8]) {
#pragma unroll
    for (int c = 0; c < 8; ++c) partial[c] = 0;
    const uint4 *av = reinterpret_cast<const uint4 *>(a);
    iq3_subblock<0>(r, av[0], av[1], lane4x2, tab, partial);
    iq3_subblock<1>(r, av[2], av[3], lane4x2, tab, partial);
    iq3_subblock<2>(r, av[4], av[5], lane4x2, tab, partial);
    iq3_subblock<3>(r, av[6], av[7], lane4x2, tab, partial);
    iq3_subblock<4>(r, av[8], av[9], lane4x2, tab, partial);
    iq3_subblock<5>(r, av[10], av[11], lane4x2, tab, partial);
    iq3_subblock<6>(r, av[12], av[13], lane4x2, tab, partial);
    iq3_subblock<7>(r, av[14], av[15], lane4x2, tab, partial);
}

// Two blocks (gate and up) against the same activations: the activation words are loaded once.
__device__ __forceinline__ void iq3_block_partials2(const Iq3Regs &r0, const Iq3Regs &r1, const uint8_t *a,
                                                    uint32_t lane4x2, const uint8_t *tab, int p0[8], int p1[8]) {
#pragma unroll
    for (int c = 0; c < 8; ++c) p0[c] = p1[c] = 0;
    const uint4 *av = reinterpret_cast<const uint4 *>(a);
#define WD_SB2(I)                                                          \
    {                                                                      \
        const uint4 lo = av[2 * I], hi = av[2 * I + 1];                    \
        iq3_subblock<I>(r0, lo, hi, lane4x2, tab, p0);                     \
        iq3_subblock<I>(r1, lo, hi, lane4x2, tab, p1);                     \
    }
    WD_SB2(0) WD_SB2(1) WD_SB2(2) WD_SB2(3) WD_SB2(4) WD_SB2(5) WD_SB2(6) WD_SB2(7)
#undef WD_SB2
}

}  // namespace wd
