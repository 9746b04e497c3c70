// Tuned step decoders for the codebook ("grid") types IQ2_XXS, IQ2_XS, IQ2_S, IQ3_XXS and IQ3_S.  See vqm_steps.cuh for
// the interface.
//
// A chunk of 8 weights is eight magnitude bytes out of the type's codebook (one 8-byte entry for the IQ2 types, two 4-byte
// entries for the IQ3 types), eight sign bits and a scale shared by 16 or 32 weights
// (engine/csrc/common/qwen_quant.cuh:221-270).  What the generic decoder spends per weight on signs and conversions is
// done here with one byte permute per weight:
//   * the eight sign bits are looked up in a 256-entry table of 8-byte words in shared memory whose byte i is 0x80 where
//     bit i is set (for the types that store 7 sign bits, entries 0..127 already carry the parity bit the format implies);
//   * one permute takes a magnitude byte into bits 8..15 and the matching sign byte into bits 24..31 of an otherwise zero
//     word: the signed subnormal float +-magnitude * 2^-141 (see bytes_to_subpair);
//   * one packed multiply per two weights with the chunk's scale db * 2^64 gives the dequantised weights times 2^-77 -
//     exact, every factor is a small integer or a power of two times the fp16 d.
// Index bytes, sign bytes and scale nibbles are fetched with 8- and 16-bit shared-memory loads at their natural
// alignment, so the 2-byte alignment of these blocks costs nothing.  Lane and chunk mapping are the generic decoder's
// (chunk j * 32 + lane of the segment), so the order of additions per output is the same for every M.
#pragma once

#include "vqm_steps.cuh"

namespace vqm {

__device__ __forceinline__ uint32_t lds8(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint2 lds64u(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}

__host__ __device__ constexpr bool is_grid_type(int type) {
    return type == kIQ2_XXS || type == kIQ2_XS || type == kIQ2_S || type == kIQ3_XXS || type == kIQ3_S;
}
// Types that store 7 sign bits per chunk; the eighth makes the parity even.
__host__ __device__ constexpr bool signs_have_parity(int type) { return type == kIQ2_XXS || type == kIQ2_XS || type == kIQ3_XXS; }
constexpr int kSignTableBytes = 256 * 8;

// Entry i of the sign table: byte k = 0x80 if bit k of the sign byte is set.  With `parity`, entries below 128 get bit 7
// from the parity of the seven bits below it (the c_ksigns table of engine/csrc/common/qwen_iq_tables.h, computed).
__device__ __forceinline__ uint2 sign_table_entry(uint32_t i, bool parity) {
    const uint32_t s = (parity && i < 128u) ? (i | ((__popc(i) & 1u) << 7)) : i;
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        lo |= ((s >> k) & 1u) << (8 * k + 7);
        hi |= ((s >> (4 + k)) & 1u) << (8 * k + 7);
    }
    return make_uint2(lo, hi);
}

// Magnitude byte K of `mags` and sign byte K of `signs` as the signed subnormal float: [sign][0][magnitude][0].  The zero
// bytes are the sign replication of a magnitude byte (magnitudes are below 128).
template <int K>
__device__ __forceinline__ uint32_t signed_sub(uint32_t mags, uint32_t signs) {
    constexpr uint32_t sel = ((4u + K) << 12) | ((8u | K) << 8) | (static_cast<uint32_t>(K) << 4) | (8u | K);
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(mags), "r"(signs), "n"(sel));
    return d;
}
__device__ __forceinline__ f32x2 pair_of(uint32_t lo, uint32_t hi) {
    f32x2 p;
    asm("mov.b64 %0, {%1, %2};" : "=l"(p) : "r"(lo), "r"(hi));
    return p;
}

// The eight weights of chunk c (0..31) of the block at shared address `blk`, times 2^-77, as four packed pairs.
// grid / signs: shared addresses of the codebook and of the sign table.
template <int TYPE>
__device__ __forceinline__ void grid_chunk(uint32_t blk, int c, uint32_t grid, uint32_t signs, f32x2 (&w)[4]) {
    const int ib = c >> 2, l = c & 3;
    const float d = half_bits_to_float(lds16(blk));
    uint32_t m0, m1, sbyte, scale;  // magnitudes of weights 0..3 and 4..7, sign table index, 4-bit scale
    if constexpr (TYPE == kIQ2_XXS) {
        // d @0, then per 32 weights: 4 grid index bytes and a word of 4 x 7 sign bits + 4-bit scale
        const uint32_t at = blk + 2 + 8 * ib;
        const uint32_t aux = lds16(at + 4) | (lds16(at + 6) << 16);
        const uint2 m = lds64u(grid + lds8(at + l) * 8);
        m0 = m.x, m1 = m.y;
        sbyte = (aux >> (7 * l)) & 127u;
        scale = aux >> 28;
    } else if constexpr (TYPE == kIQ2_XS) {
        // d @0, 32 x u16 (9-bit grid index, 7 sign bits) @2, 4-bit scale pairs @66 (8)
        const uint32_t q = lds16(blk + 2 + 2 * c);
        const uint2 m = lds64u(grid + (q & 511u) * 8);
        m0 = m.x, m1 = m.y;
        sbyte = q >> 9;
        scale = (lds8(blk + 66 + ib) >> (4 * (l >> 1))) & 15u;
    } else if constexpr (TYPE == kIQ2_S) {
        // d @0, index low bytes @2 (32), sign bytes @34 (32), index high bits @66 (8), scale pairs @74 (8)
        const uint32_t entry = lds8(blk + 2 + c) | ((lds8(blk + 66 + ib) << (8 - 2 * l)) & 0x300u);
        const uint2 m = lds64u(grid + entry * 8);
        m0 = m.x, m1 = m.y;
        sbyte = lds8(blk + 34 + c);
        scale = (lds8(blk + 74 + ib) >> (4 * (l >> 1))) & 15u;
    } else if constexpr (TYPE == kIQ3_XXS) {
        // d @0, grid index bytes @2 (64), per 32 weights a word of 4 x 7 sign bits + 4-bit scale @66
        const uint32_t at = blk + 66 + 4 * ib;
        const uint32_t aux = lds16(at) | (lds16(at + 2) << 16);
        const uint32_t idx = lds16(blk + 2 + 2 * c);
        m0 = lds32(grid + (idx & 0xFFu) * 4);
        m1 = lds32(grid + (idx >> 8) * 4);
        sbyte = (aux >> (7 * l)) & 127u;
        scale = aux >> 28;
    } else {
        static_assert(TYPE == kIQ3_S, "a codebook type");
        // d @0, grid index low bytes @2 (64), index high bits @66 (8), sign bytes @74 (32), 4-bit scales @106 (4)
        const uint32_t idx = lds16(blk + 2 + 2 * c);
        const uint32_t hb = lds8(blk + 66 + ib) >> (2 * l);
        m0 = lds32(grid + ((idx & 0xFFu) | ((hb & 1u) << 8)) * 4);
        m1 = lds32(grid + ((idx >> 8) | ((hb & 2u) << 7)) * 4);
        sbyte = lds8(blk + 74 + c);
        scale = (lds8(blk + 106 + (ib >> 1)) >> (4 * (ib & 1))) & 15u;
    }
    // db = d * (0.5 + scale) * 0.25 (IQ2), d * (0.5 + scale) * 0.5 (IQ3_XXS), d * (1 + 2 * scale) (IQ3_S): all d * (2 * scale + 1) * 2^k
    constexpr float kFactor = kSubScale * (TYPE == kIQ3_S ? 1.0f : TYPE == kIQ3_XXS ? 0.25f : 0.125f);
    const float db = d * kFactor * small_uint_to_float(2u * scale + 1u);
    const f32x2 db2 = pack2(db, db);
    const uint2 sg = lds64u(signs + sbyte * 8);
    w[0] = mul2(pair_of(signed_sub<0>(m0, sg.x), signed_sub<1>(m0, sg.x)), db2);
    w[1] = mul2(pair_of(signed_sub<2>(m0, sg.x), signed_sub<3>(m0, sg.x)), db2);
    w[2] = mul2(pair_of(signed_sub<0>(m1, sg.y), signed_sub<1>(m1, sg.y)), db2);
    w[3] = mul2(pair_of(signed_sub<2>(m1, sg.y), signed_sub<3>(m1, sg.y)), db2);
}

template <int TYPE, int M, int RW>
struct GridStep {
    static constexpr int kScratch = 0;
    static constexpr float kOutScale = kSubOutScale;
    // NR rows, all decoded (a chunk's missing rows are computed from whatever their slots hold - every index stays inside
    // its table - and dropped by the caller)
    template <int NR>
    struct Pass {
        static __device__ __forceinline__ void go(uint32_t stage, uint32_t d0, uint32_t rb16, uint32_t table, uint32_t xs, int cols,
                                                  f32x2 (&acc)[RW][M], int lane) {
            constexpr int SLOT = slot_bytes(TYPE), BB = chunk_block_bytes(TYPE);
            const uint32_t signs = table + (grid_bytes(TYPE) + 15) / 16 * 16;
            uint32_t row[NR];
#pragma unroll
            for (int r = 0; r < NR; ++r) row[r] = stage + r * SLOT + ((d0 + r * rb16) & 15u);
#pragma unroll 1
            for (int j = 0; j < kChunksPerLane; ++j) {
                const int chunk = j * 32 + lane;
                if (chunk * 8 < cols) {
                    X4 xa[M], xb[M];
#pragma unroll
                    for (int t = 0; t < M; ++t) {
                        xa[t] = lds_x4(xs + (t * kSegCols + chunk * 8) * 4);
                        xb[t] = lds_x4(xs + (t * kSegCols + chunk * 8 + 4) * 4);
                    }
                    const uint32_t boff = (chunk >> 5) * BB;
                    const int c = chunk & 31;
#pragma unroll
                    for (int r = 0; r < NR; ++r) {
                        f32x2 w[4];
                        grid_chunk<TYPE>(row[r] + boff, c, table, signs, w);
#pragma unroll
                        for (int t = 0; t < M; ++t)
                            acc[r][t] = fma2(w[3], xb[t].p23, fma2(w[2], xb[t].p01, fma2(w[1], xa[t].p23, fma2(w[0], xa[t].p01, acc[r][t]))));
                    }
                }
            }
        }
    };
    static __device__ __forceinline__ void run(uint32_t stage, uint32_t d0, uint32_t rb16, uint32_t, uint32_t table, uint32_t xs, int cols,
                                               int nrows, f32x2 (&acc)[RW][M], int lane) {
        dispatch_rows<Pass, RW>(nrows, stage, d0, rb16, table, xs, cols, acc, lane);
    }
};

template <int M, int RW>
struct Step<kIQ2_XXS, M, RW> : GridStep<kIQ2_XXS, M, RW> {};
template <int M, int RW>
struct Step<kIQ2_XS, M, RW> : GridStep<kIQ2_XS, M, RW> {};
template <int M, int RW>
struct Step<kIQ2_S, M, RW> : GridStep<kIQ2_S, M, RW> {};
template <int M, int RW>
struct Step<kIQ3_XXS, M, RW> : GridStep<kIQ3_XXS, M, RW> {};
template <int M, int RW>
struct Step<kIQ3_S, M, RW> : GridStep<kIQ3_S, M, RW> {};

}  // namespace vqm
