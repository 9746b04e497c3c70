// Tuned step decoders for Q4_K, Q5_K, Q6_K and Q3_K (the types of the 27B layer set).  See vqm_steps.cuh for the interface.
//
// Common idea: the per-weight work is "raw field -> float" (one byte permute: the field becomes the subnormal
// field * 2^-141, see bytes_to_subpair), one packed multiply or FMA per two weights with the group scale dl * 2^64
// (exact: the result is the dequantised weight times 2^-77; the minimum of the types that carry one is the addend of
// that same multiply-add, field * dl - ml, so it costs nothing) and one FMA per activation row.
// Sub-scales are decoded once per step by a scale pass (word-wide mask arithmetic, four sub-scales per lane) into a
// per-warp table of (dl, dl) pairs.  The sequence of operations per output does not depend on the number of
// activation rows.
#pragma once

#include "vqm_steps.cuh"

namespace vqm {

// ---- Q4_K --------------------------------------------------------------------------------------------------
// Block (144 B, always 16-byte aligned): d, dmin (f16) | 12 bytes of 6-bit scales and mins | 128 bytes of nibbles;
// bytes 32p..32p+31 hold group 2p in their low and group 2p+1 in their high nibbles
// (engine/csrc/common/qwen_quant.cuh:165-175).
//   scale pass : lane -> (row, block, groups 4hh..4hh+3).  Per (row, block, pair of groups p) it leaves
//                {dl, dl, dl'/16, dl'/16} and {-ml, -ml, -ml', -ml'} (/16 because the high nibbles stay in place) in four
//                "piece" arrays indexed by lane, so that its stores and the dot pass's loads are conflict-free.
//   dot pass   : one block at a time, lane i -> 32-bit word i of the nibbles: 4 weights of group 2p (columns
//                64p + 4(i%8) ..) and 4 of group 2p+1 (32 columns further), p = i / 8.  Eight lanes read 128
//                contiguous bytes of activations per load, so the shared-memory reads are conflict-free.
// Q5_K (176 B, 16-byte aligned) is the same with a fifth bit: d, dmin | 12 bytes of scales and mins | 32 bytes of high
// bits (bit g of byte l belongs to weight 32g + l) | 128 bytes of nibbles (engine/csrc/common/qwen_quant.cuh:176-181).
// The lane that owns nibble word i also reads high-bit word i % 8; the high nibbles are shifted down so that the
// fifth bit fits into the byte.
template <int TYPE, int M, int RW>
struct K45Step {
    static_assert(TYPE == kQ4_K || TYPE == kQ5_K, "Q4_K or Q5_K");
    static constexpr bool kFive = TYPE == kQ5_K;
    static constexpr int kBlock = kFive ? 176 : 144, kNibbles = kFive ? 48 : 16;
    // piece 2w: scales, piece 2w + 1: mins of pair p = 2hh + w; slot (row * 4 + block) * 2 + hh of 16 bytes in each piece
    static constexpr int kPiece = RW * 4 * 2 * 16 + 32;  // + 32: consecutive pieces start 8 banks apart
    static constexpr int kScratch = 4 * kPiece;
    static constexpr float kOutScale = kSubOutScale;

    template <int NR>
    struct Pass {
        // One block of every row: lane i -> nibble word i (p = i / 8: groups 2p and 2p + 1).
        static __device__ __forceinline__ void block_dot(uint32_t wl, uint32_t hl, int p, uint32_t el, uint32_t xl, f32x2 (&acc)[RW][M]) {
            constexpr int SLOT = slot_bytes(TYPE);
            X4 xa[M], xb[M];
#pragma unroll
            for (int t = 0; t < M; ++t) {
                xa[t] = lds_x4(xl + t * kSegCols * 4);
                xb[t] = lds_x4(xl + (t * kSegCols + 32) * 4);
            }
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                const uint32_t w = lds32(wl + r * SLOT);
                uint32_t lo, hi;
                if constexpr (kFive) {
                    const uint32_t qh = lds32(hl + r * SLOT) >> (2 * p);
                    lo = (w & 0x0F0F0F0Fu) | ((qh << 4) & 0x10101010u);
                    hi = ((w >> 4) & 0x0F0F0F0Fu) | ((qh << 3) & 0x10101010u);
                } else {
                    lo = w & 0x0F0F0F0Fu;
                    hi = w & 0xF0F0F0F0u;  // 16 x the field; the scale table carries dl' / 16
                }
                const ulonglong2 dl = lds128(el + r * 128);            // (dl, dl), (dl', dl') [Q4_K: dl' / 16], each times 2^64
                const ulonglong2 nm = lds128(el + r * 128 + kPiece);   // (-ml, -ml), (-ml', -ml'), each times 2^-77
                // one fused multiply-add per pair: field * dl - ml, the dequantised weights times 2^-77 (the product is
                // exact, so this is the single rounding of the reference's dl * q - ml)
                const f32x2 a01 = fma2(bytes_to_subpair<0, 1>(lo), dl.x, nm.x), a23 = fma2(bytes_to_subpair<2, 3>(lo), dl.x, nm.x);
                const f32x2 b01 = fma2(bytes_to_subpair<0, 1>(hi), dl.y, nm.y), b23 = fma2(bytes_to_subpair<2, 3>(hi), dl.y, nm.y);
#pragma unroll
                for (int t = 0; t < M; ++t)
                    acc[r][t] = fma2(b23, xb[t].p23, fma2(b01, xb[t].p01, fma2(a23, xa[t].p23, fma2(a01, xa[t].p01, acc[r][t]))));
            }
        }

        static __device__ __forceinline__ void go(uint32_t stage, uint32_t scratch, uint32_t xs, int nblk, f32x2 (&acc)[RW][M], int lane) {
            constexpr int SLOT = slot_bytes(TYPE);
            const f32x2 neg_magic = pack2(-8388608.0f, -8388608.0f);
            // ---- scale pass
#pragma unroll
            for (int r0 = 0; r0 < NR; r0 += 4) {
                const int r = r0 + (lane >> 3), blk = (lane >> 1) & 3, hh = lane & 1;
                if (r < NR) {
                    const uint4 h = lds128u(stage + r * SLOT + blk * kBlock);
                    const float d = half_bits_to_float(h.x & 0xFFFFu) * kSubScale, ndmin = -half_bits_to_float(h.x >> 16) * kSubWeight;
                    // four 6-bit fields at a time (engine/csrc/common/qwen_quant.cuh:78-86)
                    const uint32_t scw = hh ? ((h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u)) : (h.y & 0x3F3F3F3Fu);
                    const uint32_t mnw = hh ? (((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u)) : (h.z & 0x3F3F3F3Fu);
                    const float dh = kFive ? d : d * 0.0625f;
                    const f32x2 dlo = pack2(d, d), dhi = pack2(dh, dh), mm = pack2(ndmin, ndmin);
                    const uint32_t dst = scratch + ((r * 4 + blk) * 2 + hh) * 16;
                    sts128(dst, mul2(bytes_to_pair<0, 0>(scw, neg_magic), dlo), mul2(bytes_to_pair<1, 1>(scw, neg_magic), dhi));
                    sts128(dst + kPiece, mul2(bytes_to_pair<0, 0>(mnw, neg_magic), mm), mul2(bytes_to_pair<1, 1>(mnw, neg_magic), mm));
                    sts128(dst + 2 * kPiece, mul2(bytes_to_pair<2, 2>(scw, neg_magic), dlo), mul2(bytes_to_pair<3, 3>(scw, neg_magic), dhi));
                    sts128(dst + 3 * kPiece, mul2(bytes_to_pair<2, 2>(mnw, neg_magic), mm), mul2(bytes_to_pair<3, 3>(mnw, neg_magic), mm));
                }
            }
            __syncwarp();
            // ---- dot pass
            const int p = lane >> 3;
            const uint32_t xl = xs + (p * 64 + 4 * (lane & 7)) * 4;
            const uint32_t el = scratch + (p & 1) * 2 * kPiece + (p >> 1) * 16;
            const uint32_t wl = stage + kNibbles + 4 * lane, hl = stage + 16 + 4 * (lane & 7);
            if (nblk == 4) {  // a full segment: straight-line code
#pragma unroll
                for (int blk = 0; blk < 4; ++blk) block_dot(wl + blk * kBlock, hl + blk * kBlock, p, el + blk * 32, xl + blk * 1024, acc);
            } else {
#pragma unroll 1
                for (int blk = 0; blk < nblk; ++blk) block_dot(wl + blk * kBlock, hl + blk * kBlock, p, el + blk * 32, xl + blk * 1024, acc);
            }
            __syncwarp();  // the scratch table is rewritten by the next step
        }
    };

    static __device__ __forceinline__ void run(uint32_t stage, uint32_t, uint32_t, uint32_t scratch, uint32_t, uint32_t xs, int cols,
                                               int nrows, f32x2 (&acc)[RW][M], int lane) {
        dispatch_rows<Pass, RW>(nrows, stage, scratch, xs, cols >> 8, acc, lane);
    }
};

template <int M, int RW>
struct Step<kQ4_K, M, RW> : K45Step<kQ4_K, M, RW> {};
template <int M, int RW>
struct Step<kQ5_K, M, RW> : K45Step<kQ5_K, M, RW> {};

// ---- Q6_K and Q3_K ---------------------------------------------------------------------------------------------
// Both share a block geometry: weight e = 128h + 32q + l (h: half, q: quarter, l < 32) takes its low bits from byte
// 32h + l of a 64-byte plane (Q6_K: two planes of nibbles, Q3_K: one plane of 2-bit fields) and its high bits from a
// second plane indexed by l, and weights 16k..16k+15 share sub-scale k = 8h + 2q + (l >> 4)
// (engine/csrc/common/qwen_quant.cuh:182-190,199-210).  Neither carries a minimum; both subtract a constant bias.
//   scale pass : lane -> (row, block, 4 sub-scales): integer sub-scale -> float, times d * 2^64, stored as (dl, dl)
//                pairs so that a dot-pass lane finds the sub-scales of its four quarters in one 32-byte slot
//                [h][l >> 4][q].
//   dot pass   : lane -> (block, half h, 8 consecutive l = 8jj..8jj+7): two words of each plane give 32 weights, 8 per
//                quarter, at columns 128h + 32q + 8jj, all eight under one sub-scale.  A quarter's fields are
//                turned into subnormal floats f * 2^-141 and one FMA with (dl, c = -bias * dl * 2^-77) yields the
//                dequantised weights times 2^-77 (exact).  Lanes with h = 1 take their second four columns first, so
//                that the eight lanes of a 16-byte shared-memory load phase of activations touch 32 different banks.
//                Blocks are only 2-byte aligned, so plane words are fetched with aligned loads + a funnel shift.
template <int TYPE>
struct QuarterFormat;

template <>
struct QuarterFormat<kQ6_K> {
    static constexpr int kBlockBytes = 210;
    static constexpr float kBias = 32.0f;       // field - 32
    static constexpr float kScaleBias = 128.0f;  // int8 sub-scale, read as (byte ^ 0x80) - 128
    struct Words {
        uint32_t ql0, ql1, qh;
    };
    // the lane's 8 bytes of the first nibble plane, and from there to its 8 bytes of the high-bit plane
    static __device__ __forceinline__ uint32_t lane_off(int h, int jj) { return 64 * h + 8 * jj; }
    static __device__ __forceinline__ uint32_t second_off(int h) { return 128 - 32 * h; }
    // bf / bs: 4-byte aligned addresses at or below the lane's first / second four bytes of the first nibble plane,
    // sh: 0 or 16 (the bytes start sh / 8 further)
    static __device__ __forceinline__ void load(uint32_t bf, uint32_t bs, uint32_t sh, uint32_t d2nd, int, Words &first, Words &second) {
        first = Words{__funnelshift_r(lds32(bf), lds32(bf + 4), sh), __funnelshift_r(lds32(bf + 32), lds32(bf + 36), sh),
                      __funnelshift_r(lds32(bf + d2nd), lds32(bf + d2nd + 4), sh)};
        second = Words{__funnelshift_r(lds32(bs), lds32(bs + 4), sh), __funnelshift_r(lds32(bs + 32), lds32(bs + 36), sh),
                       __funnelshift_r(lds32(bs + d2nd), lds32(bs + d2nd + 4), sh)};
    }
    // bytes = fields of quarter Q (4 weights), still carrying the bias; every byte is below 0x80
    template <int Q>
    static __device__ __forceinline__ uint32_t quarter(const Words &w) {
        const uint32_t ql = (Q & 1) ? w.ql1 : w.ql0;
        const uint32_t lo = (Q >= 2 ? (ql >> 4) : ql) & 0x0F0F0F0Fu;
        const uint32_t hi = Q == 0 ? (w.qh << 4) : Q == 1 ? (w.qh << 2) : Q == 2 ? w.qh : (w.qh >> 2);
        return lo | (hi & 0x30303030u);
    }
    // four sub-scales 4c..4c+3 as biased bytes, and d
    static __device__ __forceinline__ uint32_t scale_word(uint32_t bp, int c, float *d) {
        *d = half_bits_to_float(lds16(bp + 208));
        return lds32_a2(bp + 192 + 4 * c) ^ 0x80808080u;
    }
};

template <>
struct QuarterFormat<kQ3_K> {
    static constexpr int kBlockBytes = 110;
    static constexpr float kBias = 4.0f;        // (low2 | high << 2) - 4
    static constexpr float kScaleBias = 32.0f;  // 6-bit sub-scale - 32
    struct Words {
        uint32_t qs, hm;
    };
    static __device__ __forceinline__ uint32_t lane_off(int h, int jj) { return 32 + 32 * h + 8 * jj; }
    static __device__ __forceinline__ uint32_t second_off(int h) { return 0u - static_cast<uint32_t>(32 + 32 * h); }
    static __device__ __forceinline__ void load(uint32_t bf, uint32_t bs, uint32_t sh, uint32_t d2nd, int h, Words &first, Words &second) {
        // bit 4h + q of a mask byte belongs to quarter q of half h
        first = Words{__funnelshift_r(lds32(bf), lds32(bf + 4), sh), __funnelshift_r(lds32(bf + d2nd), lds32(bf + d2nd + 4), sh) >> (4 * h)};
        second = Words{__funnelshift_r(lds32(bs), lds32(bs + 4), sh), __funnelshift_r(lds32(bs + d2nd), lds32(bs + d2nd + 4), sh) >> (4 * h)};
    }
    template <int Q>
    static __device__ __forceinline__ uint32_t quarter(const Words &w) {
        const uint32_t lo = (Q == 0 ? w.qs : (w.qs >> (2 * Q))) & 0x03030303u;
        const uint32_t hb = Q == 0 ? (w.hm << 2) : Q == 1 ? (w.hm << 1) : Q == 2 ? w.hm : (w.hm >> 1);
        return lo | (hb & 0x04040404u);
    }
    static __device__ __forceinline__ uint32_t scale_word(uint32_t bp, int c, float *d) {
        *d = half_bits_to_float(lds16(bp + 108));
        // sub-scale k: low nibble from byte k % 8 (>> 4 for k >= 8), high 2 bits from byte 8 + k % 4 (>> 2 (k / 4))
        const uint32_t wl = lds32_a2(bp + 96 + 4 * (c & 1)), w2 = lds32_a2(bp + 104);
        const uint32_t lo = (wl >> (4 * (c >> 1))) & 0x0F0F0F0Fu;
        const uint32_t hi = static_cast<uint32_t>((static_cast<unsigned long long>(w2) << 4) >> (2 * c)) & 0x30303030u;
        return lo | hi;
    }
};

template <int TYPE, int M, int RW>
struct QuarterStep {
    using F = QuarterFormat<TYPE>;
    // per (row, block): 16 sub-scales x (dl, dl), as [h][l >> 4][quarter], 128 bytes + 16 of padding: the two blocks whose
    // lanes share a 64-bit load phase then read different banks
    static constexpr int kEntry = 144;
    static constexpr int kScratch = RW * 4 * kEntry;
    static constexpr float kOutScale = kSubOutScale;

    template <int NR>
    struct Pass {
        // Four of the lane's columns (xa: their activations) of one quarter, every row.
        static __device__ __forceinline__ void quad_dot(const uint32_t (&q)[NR], const f32x2 (&d2)[NR], uint32_t xa, f32x2 (&acc)[RW][M]) {
            const f32x2 nbias = pack2(-F::kBias * 0x1p-141f, -F::kBias * 0x1p-141f);
            X4 x[M];
#pragma unroll
            for (int t = 0; t < M; ++t) x[t] = lds_x4(xa + t * kSegCols * 4);
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                // exact: field * 2^-141 * dl * 2^64 - bias * dl * 2^-77, the dequantised weight times 2^-77
                // (c is recomputed per four columns rather than kept per row: a multiply is cheaper than the registers)
                const f32x2 c = mul2(d2[r], nbias);
                const f32x2 q01 = fma2(bytes_to_subpair<0, 1>(q[r]), d2[r], c), q23 = fma2(bytes_to_subpair<2, 3>(q[r]), d2[r], c);
#pragma unroll
                for (int t = 0; t < M; ++t) acc[r][t] = fma2(q23, x[t].p23, fma2(q01, x[t].p01, acc[r][t]));
            }
        }

        template <int Q>
        static __device__ __forceinline__ void quarter_dot(const typename F::Words (&first)[NR], const typename F::Words (&second)[NR],
                                                           uint32_t el, uint32_t x_first, uint32_t x_second, f32x2 (&acc)[RW][M]) {
            uint32_t q[NR];
            f32x2 d2[NR];
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                d2[r] = lds64(el + r * 4 * kEntry + Q * 8);
#ifdef VQM_X_NO_QUARTER
                q[r] = first[r].qh + Q;
#else
                q[r] = F::template quarter<Q>(first[r]);
#endif
            }
            quad_dot(q, d2, x_first + Q * 32 * 4, acc);
#pragma unroll
#ifdef VQM_X_NO_QUARTER
            for (int r = 0; r < NR; ++r) q[r] = second[r].qh + Q;
#else
            for (int r = 0; r < NR; ++r) q[r] = F::template quarter<Q>(second[r]);
#endif
            quad_dot(q, d2, x_second + Q * 32 * 4, acc);
        }

        static __device__ __forceinline__ void go(uint32_t stage, uint32_t d0, uint32_t rb16, uint32_t scratch, uint32_t xs, int nblk,
                                                  f32x2 (&acc)[RW][M], int lane) {
            constexpr int SLOT = slot_bytes(TYPE), BB = F::kBlockBytes;
            // ---- scale pass: task -> (row, block, scale word c)
            {
                const f32x2 neg_magic = pack2(-(8388608.0f + F::kScaleBias), -(8388608.0f + F::kScaleBias));
#pragma unroll
                for (int task0 = 0; task0 < 16 * NR; task0 += 32) {
                    const int task = task0 + lane, r = task >> 4, blk = (task >> 2) & 3, c = task & 3;
                    if (r < NR) {
                        const uint32_t bp = stage + r * SLOT + ((d0 + r * rb16) & 15u) + blk * BB;
                        float d;
                        const uint32_t sw = F::scale_word(bp, c, &d);
                        d *= kSubScale;
                        const f32x2 dd = pack2(d, d);
                        // sub-scale k = 4c + i belongs to half k >> 3, quarter (k >> 1) & 3, l >> 4 = k & 1
                        const uint32_t dst = scratch + (r * 4 + blk) * kEntry + (c >> 1) * 64 + (c & 1) * 16;
                        sts128(dst, mul2(bytes_to_pair<0, 0>(sw, neg_magic), dd), mul2(bytes_to_pair<2, 2>(sw, neg_magic), dd));       // l < 16
                        sts128(dst + 32, mul2(bytes_to_pair<1, 1>(sw, neg_magic), dd), mul2(bytes_to_pair<3, 3>(sw, neg_magic), dd));  // l >= 16
                    }
                }
            }
            __syncwarp();
            // ---- dot pass: all four blocks at once
            const int blk = lane >> 3, h = (lane >> 2) & 1, jj = lane & 3;
            if (blk < nblk) {
                const uint32_t lane_off = blk * BB + F::lane_off(h, jj), d2nd = F::second_off(h);
                typename F::Words first[NR], second[NR];
#pragma unroll
                for (int r = 0; r < NR; ++r) {
                    const uint32_t a = stage + r * SLOT + ((d0 + r * rb16) & 15u) + lane_off, b = a & ~3u;
#ifdef VQM_X_NO_LOAD
                    first[r] = typename F::Words{a, b, d0};
                    second[r] = typename F::Words{b, a, rb16};
#else
                    F::load(b + 4 * h, b + 4 - 4 * h, (a & 2u) << 3, d2nd, h, first[r], second[r]);
#endif
                }
                const uint32_t el = scratch + blk * kEntry + (h * 2 + (jj >> 1)) * 32;
                const uint32_t x_first = xs + (blk * 256 + 128 * h + 8 * jj + 4 * h) * 4;
                const uint32_t x_second = xs + (blk * 256 + 128 * h + 8 * jj + 4 * (1 - h)) * 4;
                quarter_dot<0>(first, second, el, x_first, x_second, acc);
                quarter_dot<1>(first, second, el, x_first, x_second, acc);
                quarter_dot<2>(first, second, el, x_first, x_second, acc);
                quarter_dot<3>(first, second, el, x_first, x_second, acc);
            }
            __syncwarp();  // the scratch table is rewritten by the next step
        }
    };

    static __device__ __forceinline__ void run(uint32_t stage, uint32_t d0, uint32_t rb16, uint32_t scratch, uint32_t, uint32_t xs,
                                               int cols, int nrows, f32x2 (&acc)[RW][M], int lane) {
        dispatch_rows<Pass, RW>(nrows, stage, d0, rb16, scratch, xs, cols >> 8, acc, lane);
    }
};

template <int M, int RW>
struct Step<kQ6_K, M, RW> : QuarterStep<kQ6_K, M, RW> {};
template <int M, int RW>
struct Step<kQ3_K, M, RW> : QuarterStep<kQ3_K, M, RW> {};

}  // namespace vqm
