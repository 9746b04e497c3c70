// Tuned step decoder for IQ4_XS.  See vqm_steps.cuh for the interface.
//
// Block (136 B, 8-byte aligned): d (f16) @0 | scales_h (u16) @2 | scales_l[4] @4 | 128 bytes of nibbles @8; group g
// (32 weights) owns bytes 16g..16g+15: weights 0..15 are the low nibbles, 16..31 the high ones, each an index into the
// 16 non-linear levels; its scale is d * (ls - 32) with a 6-bit ls (engine/csrc/common/qwen_quant.cuh:211-220).
//   scale pass : lane -> (row, block, group): ls from the two packed fields, dl = d * (ls - 32), stored as a (dl, dl) pair.
//   dot pass   : one block at a time, lane i -> 32-bit word i of the nibbles (group i / 4): four low-nibble weights at
//                columns 32g + 4(i % 4) and four high-nibble weights 16 columns further.  A level is looked up as a
//                float in a 16-entry shared-memory table (16 entries = 16 banks: lookups never conflict), multiplied by
//                dl (exact: the dequantised weight) and accumulated with packed FMAs.
#pragma once

#include "vqm_steps.cuh"

namespace vqm {

template <int M, int RW>
struct Step<kIQ4_XS, M, RW> {
    static constexpr int kScratch = RW * 4 * 8 * 8;  // (dl, dl) per (row, block, group)
    static constexpr float kOutScale = 1.0f;

    template <int NR>
    struct Pass {
        static __device__ __forceinline__ float level(uint32_t table, uint32_t byte_off) {
            return __uint_as_float(lds32(table + byte_off));
        }

        static __device__ __forceinline__ void go(uint32_t stage, uint32_t d0, uint32_t rb16, uint32_t scratch, uint32_t table, uint32_t xs,
                                                  int nblk, f32x2 (&acc)[RW][M], int lane) {
            constexpr int SLOT = slot_bytes(kIQ4_XS);
            // ---- scale pass: lane -> (block, group) of row r
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                const int blk = lane >> 3, g = lane & 7;
                const uint32_t bp = stage + r * SLOT + ((d0 + r * rb16) & 15u) + blk * 136;
                const uint2 h = make_uint2(lds32(bp), lds32(bp + 4));  // d | scales_h, scales_l
                const uint32_t ls = ((h.y >> (4 * g)) & 0x0Fu) | ((((h.x >> 16) >> (2 * g)) & 3u) << 4);
                const float dl = half_bits_to_float(h.x & 0xFFFFu) * (__uint_as_float(0x4B000000u | ls) - 8388640.0f);  // ls - 32
                const unsigned long long pair = pack2(dl, dl);
                asm volatile("st.shared.u64 [%0], %1;" ::"r"(scratch + (r * 32 + lane) * 8), "l"(pair) : "memory");
            }
            __syncwarp();
            // ---- dot pass
            const int g = lane >> 2, q = lane & 3;
            const uint32_t xl = xs + (g * 32 + 4 * q) * 4;
#pragma unroll
            for (int blk = 0; blk < 4; ++blk) {
                if (blk < nblk) {
                    X4 xa[M], xb[M];
#pragma unroll
                    for (int t = 0; t < M; ++t) {
                        xa[t] = lds_x4(xl + (t * kSegCols + blk * 256) * 4);
                        xb[t] = lds_x4(xl + (t * kSegCols + blk * 256 + 16) * 4);
                    }
#pragma unroll
                    for (int r = 0; r < NR; ++r) {
                        const uint32_t w = lds32(stage + r * SLOT + ((d0 + r * rb16) & 15u) + blk * 136 + 8 + 4 * lane);
                        const f32x2 dl2 = lds64(scratch + (r * 32 + blk * 8 + g) * 8);
                        // byte k of w: low nibble -> weight k, high nibble -> weight 16 + k; table offsets are index * 4
                        const f32x2 a01 = mul2(pack2(level(table, (w << 2) & 0x3Cu), level(table, (w >> 6) & 0x3Cu)), dl2);
                        const f32x2 a23 = mul2(pack2(level(table, (w >> 14) & 0x3Cu), level(table, (w >> 22) & 0x3Cu)), dl2);
                        const f32x2 b01 = mul2(pack2(level(table, (w >> 2) & 0x3Cu), level(table, (w >> 10) & 0x3Cu)), dl2);
                        const f32x2 b23 = mul2(pack2(level(table, (w >> 18) & 0x3Cu), level(table, (w >> 26) & 0x3Cu)), dl2);
#pragma unroll
                        for (int t = 0; t < M; ++t)
                            acc[r][t] = fma2(b23, xb[t].p23, fma2(b01, xb[t].p01, fma2(a23, xa[t].p23, fma2(a01, xa[t].p01, acc[r][t]))));
                    }
                }
            }
            __syncwarp();  // the scratch table is rewritten by the next step
        }
    };

    static __device__ __forceinline__ void run(uint32_t stage, uint32_t d0, uint32_t rb16, uint32_t scratch, uint32_t table, uint32_t xs,
                                               int cols, int nrows, f32x2 (&acc)[RW][M], int lane) {
        dispatch_rows<Pass, RW>(nrows, stage, d0, rb16, scratch, table, xs, cols >> 8, acc, lane);
    }
};

}  // namespace vqm
