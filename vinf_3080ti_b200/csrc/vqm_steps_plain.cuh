// Tuned step decoders for Q8_0 and Q2_K.  See vqm_steps.cuh for the interface.
//
// Both are "scale times small integer (minus a minimum)" formats without sub-scale tables worth a pass of their own
// (engine/csrc/common/qwen_quant.cuh:163-170, 213-224):
//   Q8_0 block (34 B, 2-byte aligned): d (f16) @0 | 32 x int8 @2;                 weight = d * q
//   Q2_K block (84 B, 4-byte aligned): 16 x (4-bit scale | 4-bit min << 4) @0 | 64 bytes of 2-bit fields @16 | d @80 | dmin @82;
//        weights 128 h + 32 q + l (l < 32) are bit pair q of byte 32 h + l;       weight = d * sc * f - dmin * mn
// A chunk of 8 weights is two words of fields; each field byte becomes the subnormal float field * 2^-141 with one permute
// (bytes_to_subpair) and one packed FMA per two weights with (scale * 2^64, -offset * 2^-77) yields the dequantised weights
// times 2^-77 with the single rounding of the generic decoder (for Q8_0: int8 + 128 is the unsigned byte, the offset
// 128 * d; the result d * q is exact).  Lane and chunk mapping are the generic decoder's (chunk j * 32 + lane of the
// segment), so the order of additions per output is the same for every M.
#pragma once

#include "vqm_steps.cuh"

namespace vqm {

// The eight weights of chunk `chunk` of the segment whose row starts at shared address `row`, times 2^-77.
template <int TYPE>
__device__ __forceinline__ void plain_chunk(uint32_t row, int chunk, f32x2 (&w)[4]) {
    uint32_t w0, w1;
    f32x2 d2, c2;
    if constexpr (TYPE == kQ8_0) {
        const uint32_t at = row + (chunk >> 2) * 34;
        const float ds = half_bits_to_float(lds16(at)) * kSubScale;
        lds64_a2(at + 2 + 8 * (chunk & 3), w0, w1);
        w0 ^= 0x80808080u;
        w1 ^= 0x80808080u;
        d2 = pack2(ds, ds);
        c2 = mul2(d2, pack2(-128.0f * 0x1p-141f, -128.0f * 0x1p-141f));
    } else {
        static_assert(TYPE == kQ2_K, "Q8_0 or Q2_K");
        const int c = chunk & 31;
        const uint32_t at = row + (chunk >> 5) * 84;
        const uint32_t dd = lds32(at + 80), s = lds8(at + (c >> 1));
        const float dl = half_bits_to_float(dd & 0xFFFFu) * small_uint_to_float(s & 15u) * kSubScale;
        const float nml = half_bits_to_float(dd >> 16) * small_uint_to_float(s >> 4) * -kSubWeight;
        const uint32_t q = at + 16 + 32 * (c >> 4) + 8 * (c & 3);
        const int shift = 2 * ((c >> 2) & 3);
        w0 = (lds32(q) >> shift) & 0x03030303u;
        w1 = (lds32(q + 4) >> shift) & 0x03030303u;
        d2 = pack2(dl, dl);
        c2 = pack2(nml, nml);
    }
    w[0] = fma2(bytes_to_subpair<0, 1>(w0), d2, c2);
    w[1] = fma2(bytes_to_subpair<2, 3>(w0), d2, c2);
    w[2] = fma2(bytes_to_subpair<0, 1>(w1), d2, c2);
    w[3] = fma2(bytes_to_subpair<2, 3>(w1), d2, c2);
}

template <int TYPE, int M, int RW>
struct PlainStep {
    static constexpr int kScratch = 0;
    static constexpr float kOutScale = kSubOutScale;
    // NR rows, all decoded (a chunk's missing rows are computed from whatever their slots hold and dropped by the caller)
    template <int NR>
    struct Pass {
        static __device__ __forceinline__ void go(uint32_t stage, uint32_t d0, uint32_t rb16, uint32_t xs, int cols, f32x2 (&acc)[RW][M], int lane) {
            constexpr int SLOT = slot_bytes(TYPE);
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
#pragma unroll
                    for (int r = 0; r < NR; ++r) {
                        f32x2 w[4];
                        plain_chunk<TYPE>(row[r], chunk, w);
#pragma unroll
                        for (int t = 0; t < M; ++t)
                            acc[r][t] = fma2(w[3], xb[t].p23, fma2(w[2], xb[t].p01, fma2(w[1], xa[t].p23, fma2(w[0], xa[t].p01, acc[r][t]))));
                    }
                }
            }
        }
    };
    static __device__ __forceinline__ void run(uint32_t stage, uint32_t d0, uint32_t rb16, uint32_t, uint32_t, uint32_t xs, int cols, int nrows,
                                               f32x2 (&acc)[RW][M], int lane) {
        dispatch_rows<Pass, RW>(nrows, stage, d0, rb16, xs, cols, acc, lane);
    }
};

template <int M, int RW>
struct Step<kQ8_0, M, RW> : PlainStep<kQ8_0, M, RW> {};
template <int M, int RW>
struct Step<kQ2_K, M, RW> : PlainStep<kQ2_K, M, RW> {};

}  // namespace vqm
