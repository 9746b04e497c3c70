// Tuned step decoders for IQ4_XS and IQ4_NL.  See vqm_steps.cuh for the interface.
//
// Both store 4-bit indices into 16 non-linear levels (engine/csrc/common/qwen_quant.cuh:60): byte k of a 16-byte run
// holds weight k in its low and weight 16 + k in its high nibble.
//   IQ4_XS block (136 B, 8-byte aligned): d (f16) @0 | scales_h (u16) @2 | scales_l[4] @4 | 128 bytes of nibbles @8;
//          group g (32 weights) owns bytes 16g..16g+15, its scale is d * (ls - 32) with a 6-bit ls (:211-220).
//   IQ4_NL block (18 B, 2-byte aligned): d (f16) @0 | 16 bytes of nibbles @2 (:159-164).
// Levels are looked up in registers: the 16 levels + 128 are 16 bytes in four registers, and three byte permutes turn
// four consecutive nibbles of a word into their four level bytes (two permutes look the low 3 index bits up in the lower
// and in the upper half of the table, a third picks between them with the indices' top bits).  A level byte becomes the
// subnormal (level + 128) * 2^-141 (bytes_to_subpair) and one FMA with (dl * 2^64, -128 * dl * 2^-77) yields the
// dequantised weight times 2^-77, exactly.  Lanes of odd groups take their high-nibble weights first, so that the eight
// lanes of a 16-byte activation load phase touch 32 different banks.
#pragma once

#include "vqm_steps.cuh"

namespace vqm {

// levels + 128, four per register (little endian): {-127,-104,-83,-65}, {-49,-35,-22,-10}, {1,13,25,38}, {53,69,89,113}
constexpr uint32_t kIq4T0 = 0x3F2D1801u, kIq4T1 = 0x766A5D4Fu, kIq4T2 = 0xA6998D81u, kIq4T3 = 0xF1D9C5B5u;

__device__ __forceinline__ uint32_t prmt_r(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
// Level bytes (+128) of the four nibbles in the low 16 bits of `n` (nibble j -> byte j).
__device__ __forceinline__ uint32_t iq4_levels4(uint32_t n) {
    const uint32_t low3 = n & 0x7777u;
    const uint32_t from_lower = prmt_r(kIq4T0, kIq4T1, low3), from_upper = prmt_r(kIq4T2, kIq4T3, low3);
    return prmt_r(from_lower, from_upper, ((n >> 1) & 0x4444u) | 0x3210u);  // selector nibble j: j, or 4 + j if index j >= 8
}
// Bytes sa and sb (selector words, see below) of `v` as a pair of subnormal floats.
__device__ __forceinline__ f32x2 sub_pair_sel(uint32_t v, uint32_t sa, uint32_t sb) {
    f32x2 p;
    const uint32_t lo = prmt_r(v, 0u, sa), hi = prmt_r(v, 0u, sb);
    asm("mov.b64 %0, {%1, %2};" : "=l"(p) : "r"(lo), "r"(hi));
    return p;
}

// The dot product of one nibble word per row: level bytes la = (lo0, hi0, lo1, hi1), lb = (lo2, hi2, lo3, hi3), where
// lo_k is weight 4q + k of the run and hi_k weight 16 + 4q + k.  `odd` lanes take the hi weights first.
template <int M, int RW, int NR>
struct Iq4Dot {
    // selectors: the byte goes to bits 8..15, byte 4 (of the zero operand) everywhere else
    static __device__ __forceinline__ void selectors(int odd, uint32_t (&sel)[4]) {
        sel[0] = 0x4404u | static_cast<uint32_t>(odd << 4);        // first,  k even: byte 0 (lo) or 1 (hi)
        sel[1] = 0x4404u | static_cast<uint32_t>((2 + odd) << 4);  // first,  k odd:  byte 2 or 3
        sel[2] = 0x4404u | static_cast<uint32_t>((1 - odd) << 4);  // second, k even
        sel[3] = 0x4404u | static_cast<uint32_t>((3 - odd) << 4);  // second, k odd
    }
    static __device__ __forceinline__ void go(const uint32_t (&w)[NR], const f32x2 (&ds)[NR], const uint32_t (&sel)[4], uint32_t x_first,
                                              uint32_t x_second, f32x2 (&acc)[RW][M]) {
        const f32x2 nbias = pack2(-128.0f * 0x1p-141f, -128.0f * 0x1p-141f);
        uint32_t la[NR], lb[NR];
        f32x2 c2[NR];
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            la[r] = iq4_levels4(w[r]);
            lb[r] = iq4_levels4(w[r] >> 16);
            c2[r] = mul2(ds[r], nbias);
        }
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            X4 x[M];
#pragma unroll
            for (int t = 0; t < M; ++t) x[t] = lds_x4((half ? x_second : x_first) + t * kSegCols * 4);
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                const f32x2 v01 = fma2(sub_pair_sel(la[r], sel[2 * half], sel[2 * half + 1]), ds[r], c2[r]);
                const f32x2 v23 = fma2(sub_pair_sel(lb[r], sel[2 * half], sel[2 * half + 1]), ds[r], c2[r]);
#pragma unroll
                for (int t = 0; t < M; ++t) acc[r][t] = fma2(v23, x[t].p23, fma2(v01, x[t].p01, acc[r][t]));
            }
        }
    }
};

template <int M, int RW>
struct Step<kIQ4_XS, M, RW> {
    static constexpr int kScratch = RW * 4 * 8 * 8;  // (dl, dl) * 2^64 per (row, block, group)
    static constexpr float kOutScale = kSubOutScale;

    template <int NR>
    struct Pass {
        static __device__ __forceinline__ void go(uint32_t stage, uint32_t d0, uint32_t rb16, uint32_t scratch, uint32_t xs, int nblk,
                                                  f32x2 (&acc)[RW][M], int lane) {
            constexpr int SLOT = slot_bytes(kIQ4_XS);
            // ---- scale pass: lane -> (block, group) of row r
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                const int blk = lane >> 3, g = lane & 7;
                const uint32_t bp = stage + r * SLOT + ((d0 + r * rb16) & 15u) + blk * 136;
                const uint2 h = make_uint2(lds32(bp), lds32(bp + 4));  // d | scales_h, scales_l
                const uint32_t ls = ((h.y >> (4 * g)) & 0x0Fu) | ((((h.x >> 16) >> (2 * g)) & 3u) << 4);
                const float dl = half_bits_to_float(h.x & 0xFFFFu) * kSubScale * (__uint_as_float(0x4B000000u | ls) - 8388640.0f);  // ls - 32
                const unsigned long long pair = pack2(dl, dl);
                asm volatile("st.shared.u64 [%0], %1;" ::"r"(scratch + (r * 32 + lane) * 8), "l"(pair) : "memory");
            }
            __syncwarp();
            // ---- dot pass: one block at a time, lane i -> 32-bit word i of the nibbles (group i / 4)
            const int g = lane >> 2, q = lane & 3, odd = g & 1;
            uint32_t sel[4];
            Iq4Dot<M, RW, NR>::selectors(odd, sel);
            const uint32_t x_first = xs + (g * 32 + 4 * q + 16 * odd) * 4, x_second = xs + (g * 32 + 4 * q + 16 * (1 - odd)) * 4;
            auto block_dot = [&](int blk) {
                uint32_t w[NR];
                f32x2 ds[NR];
#pragma unroll
                for (int r = 0; r < NR; ++r) {
                    w[r] = lds32(stage + r * SLOT + ((d0 + r * rb16) & 15u) + blk * 136 + 8 + 4 * lane);
                    ds[r] = lds64(scratch + (r * 32 + blk * 8 + g) * 8);
                }
                Iq4Dot<M, RW, NR>::go(w, ds, sel, x_first + blk * 1024, x_second + blk * 1024, acc);
            };
            if (nblk == 4) {  // a full segment: straight-line code
#pragma unroll
                for (int blk = 0; blk < 4; ++blk) block_dot(blk);
            } else {
#pragma unroll 1
                for (int blk = 0; blk < nblk; ++blk) block_dot(blk);
            }
            __syncwarp();  // the scratch table is rewritten by the next step
        }
    };

    static __device__ __forceinline__ void run(uint32_t stage, uint32_t d0, uint32_t rb16, uint32_t scratch, uint32_t, uint32_t xs, int cols,
                                               int nrows, f32x2 (&acc)[RW][M], int lane) {
        dispatch_rows<Pass, RW>(nrows, stage, d0, rb16, scratch, xs, cols >> 8, acc, lane);
    }
};

// IQ4_NL: lane -> (block b = lane / 4 of the 8 blocks of an iteration, nibble word q = lane % 4); a block's d is read by
// its four lanes directly.  cols is a multiple of 32 here, not of 256: blocks beyond the segment are skipped.
template <int M, int RW>
struct Step<kIQ4_NL, M, RW> {
    static constexpr int kScratch = 0;
    static constexpr float kOutScale = kSubOutScale;

    template <int NR>
    struct Pass {
        static __device__ __forceinline__ void go(uint32_t stage, uint32_t d0, uint32_t rb16, uint32_t xs, int nblocks, f32x2 (&acc)[RW][M],
                                                  int lane) {
            constexpr int SLOT = slot_bytes(kIQ4_NL);
            const int b = lane >> 2, q = lane & 3, odd = b & 1;
            uint32_t sel[4];
            Iq4Dot<M, RW, NR>::selectors(odd, sel);
#pragma unroll 1
            for (int b0 = 0; b0 < nblocks; b0 += 8) {
                const int blk = b0 + b;
                if (blk < nblocks) {
                    uint32_t w[NR];
                    f32x2 ds[NR];
#pragma unroll
                    for (int r = 0; r < NR; ++r) {
                        const uint32_t bp = stage + r * SLOT + ((d0 + r * rb16) & 15u) + blk * 18;
                        const float d = half_bits_to_float(lds16(bp)) * kSubScale;
                        ds[r] = pack2(d, d);
                        w[r] = lds32_a2(bp + 2 + 4 * q);
                    }
                    const uint32_t xl = xs + (blk * 32 + 4 * q) * 4;
                    Iq4Dot<M, RW, NR>::go(w, ds, sel, xl + 64 * odd, xl + 64 * (1 - odd), acc);
                }
            }
        }
    };

    static __device__ __forceinline__ void run(uint32_t stage, uint32_t d0, uint32_t rb16, uint32_t, uint32_t, uint32_t xs, int cols,
                                               int nrows, f32x2 (&acc)[RW][M], int lane) {
        dispatch_rows<Pass, RW>(nrows, stage, d0, rb16, xs, cols >> 5, acc, lane);
    }
};

}  // namespace vqm
