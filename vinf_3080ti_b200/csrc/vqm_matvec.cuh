// Quantized matvec / small-M batched matmul for sm_100a:  y[t][r] = sum_k W[r][k] x[t][k],  t < M <= 8.
//
// Replaces the reference's vinf_qmatvec_kernel (engine/csrc/megakernel/qwen_runtime.cu:579-628).  W stays
// in raw GGUF block layout in HBM and is read exactly once for all M activation rows.
//
// Shape of the kernel
//   * One wave of blocks of 8 warps.  The rows are split evenly over all warps of the grid (a warp gets
//     a contiguous run of rows/warps or one more); a warp takes its run in chunks of at most RW rows and
//     walks each chunk in steps of kSegCols = 1024 columns.  All warps make the same number of steps.
//   * Weights: every WARP runs its own pipeline.  For each of its RW rows the byte range of the step's
//     segment (rounded out to 16-byte boundaries) is fetched by one non-multicast bulk copy
//     (cp.async.bulk global -> shared) into the warp's ring of S stages; completion is counted on an
//     mbarrier per stage.
//   * Activations: the step's segment x[t][seg] of all M rows is staged ONCE per block in a ring of XS
//     shared-memory stages, also by bulk copies.  The warp that is last to finish reading a stage
//     refills it, so nobody waits for the refill to be issued.
//   * Decoding runs from shared memory; the per-type decoders (Step<TYPE, M, RW>) choose the lane
//     mapping.  fp32 accumulation: per (row, activation row) an (even, odd) pair of partial sums updated
//     with packed fp32 FMAs, then a warp xor-shuffle tree.  The order of additions for an output does not
//     depend on M or RW, so an M-row pass equals M single-row passes bit for bit, as the reference
//     guarantees (engine/csrc/megakernel/qwen_runtime.cu:575-577).
//   * Optional fused argmax over the rows (the LM head): every warp keeps the best (value, row) per
//     activation row, blocks write partials, the last block to finish reduces them.  Ties go to the
//     lowest row and a column with no value above -inf yields 0x7fffffff, like the reference's
//     argmax_kernel (engine/csrc/megakernel/qwen_runtime.cu:851-876).
//   * Every wait on an mbarrier is bounded; on expiry the warp records a code in the status word and
//     leaves the loop.
#pragma once

#include "vqm_formats.cuh"
#include "vqm_kernels.h"

namespace vqm {

constexpr int kSegCols = 1024;                 // columns per pipeline step
constexpr int kChunksPerLane = kSegCols / 256;  // 8-weight chunks a lane decodes per row per step
constexpr int kWarps = 8;                      // warps per block
constexpr int kMaxTok = 8;                     // activation rows per launch
constexpr int kWarpSmemBudget = 5120;          // weight staging bytes a warp aims for (at least two stages are kept)
constexpr int kBarrierBytes = 1024;            // mbarriers and counters at the front of shared memory
constexpr int kXStageBudget = 49152;           // activation staging bytes a block aims for (at least two stages)

// Bytes of one row's segment and of the shared-memory slot that receives it (the copy is widened to
// 16-byte boundaries on both sides: up to 14 bytes in front, and the decoders' funnel loads may touch
// up to 4 bytes behind).
__host__ __device__ constexpr int seg_bytes(int type) { return kSegCols / chunk_block(type) * chunk_block_bytes(type); }
__host__ __device__ constexpr int slot_bytes(int type) { return (seg_bytes(type) + 14 + 8 + 15) / 16 * 16; }
__host__ __device__ constexpr int stages_for(int type, int rw) {
    const int s = kWarpSmemBudget / (rw * slot_bytes(type));
    return s < 2 ? 2 : s > 8 ? 8 : s;
}
__host__ __device__ constexpr int x_stages_for(int m) {
    const int s = kXStageBudget / (m * kSegCols * 4);
    return s < 2 ? 2 : s > 4 ? 4 : s;
}
__host__ __device__ constexpr int table_bytes_padded(int type) { return (grid_bytes(type) + 15) / 16 * 16; }
__host__ __device__ constexpr size_t matvec_smem_bytes(int type, int rw, int m) {
    return static_cast<size_t>(table_bytes_padded(type)) + kBarrierBytes +
           static_cast<size_t>(x_stages_for(m)) * m * kSegCols * 4 +
           static_cast<size_t>(kWarps) * stages_for(type, rw) * rw * slot_bytes(type);
}

// ---- mbarrier / bulk-copy primitives ---------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait: ~2^22 polls with a short sleep after the first few hundred.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity) {
    for (int i = 0; i < (1 << 22); ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (i > 256) __nanosleep(64);
    }
    return false;
}

// One contiguous global -> shared copy of `bytes` (multiple of 16; both addresses 16-byte aligned),
// completion counted in bytes on `bar`.  No multicast.
__device__ __forceinline__ void bulk_copy_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// ---- arithmetic helpers ------------------------------------------------------------------------------

// Two fp32 values in one 64-bit register pair; sm_100 executes add/mul/fma on both halves with one
// instruction (one issue slot for two FMAs), which is what lets a warp keep up with the weight stream.
using f32x2 = unsigned long long;

__device__ __forceinline__ f32x2 pack2(float lo, float hi) {
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(f32x2 v, float &lo, float &hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
    f32x2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
    f32x2 d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {
    f32x2 d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

// Bytes K0 and K1 of `w` as an exact (float, float) pair: each byte is dropped into the mantissa of 2^23
// and the pair is rebased with one packed add.  `neg_magic` = pack2(-(2^23 + bias), -(2^23 + bias)).
template <int K0, int K1>
__device__ __forceinline__ f32x2 bytes_to_pair(uint32_t w, f32x2 neg_magic) {
    const uint32_t lo = __byte_perm(w, 0x4B000000u, 0x7540 + K0), hi = __byte_perm(w, 0x4B000000u, 0x7540 + K1);
    f32x2 p;
    asm("mov.b64 %0, {%1, %2};" : "=l"(p) : "r"(lo), "r"(hi));
    return add2(p, neg_magic);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

__device__ __forceinline__ bool better(float v, int i, float bv, int bi) { return v > bv || (v == bv && i < bi); }

// Four consecutive staged activations (16-byte aligned, shared memory) as two packed pairs.
struct X4 {
    f32x2 p01, p23;
};
__device__ __forceinline__ X4 lds_x4(const float *xs) {
    const ulonglong2 v = *reinterpret_cast<const ulonglong2 *>(xs);
    return X4{v.x, v.y};
}
__device__ __forceinline__ float sum_x4(const X4 &x) {
    float lo, hi;
    unpack2(add2(x.p01, x.p23), lo, hi);
    return lo + hi;
}

// ---- per-type step decoders ------------------------------------------------------------------------------
// A "step" is kSegCols (1024) columns of the warp's RW rows, staged in shared memory.  Step<TYPE, M, RW>::run
// adds the step's contribution to acc[r][t] (an (even, odd) pair of partial sums per output).
//   stage  : RW slots of slot_bytes(TYPE); row r's segment starts at stage + r * slot + ((d0 + r * rb16) & 15)
//   scratch: kScratch bytes of per-warp shared memory (scale tables)
//   table  : the type's lookup table (block-wide shared memory)
//   xs     : the staged activations of the segment, [M][kSegCols] fp32 in shared memory
//   cols   : columns of this segment (1024, or less for the last one; a multiple of the block size)
//   nrows  : rows of this row group that exist (1..RW)

// Generic decoder: one 8-weight chunk per lane at a time through deq8<TYPE>, exact dequantised values
// multiplied straight into the sums.  Correct for every type; the tuned decoders below replace it for the
// types the 27B layer set is made of.
template <int TYPE, int M, int RW>
struct Step {
    static constexpr int kScratch = 0;
    static __device__ __forceinline__ void run(const uint8_t *stage, uint32_t d0, uint32_t rb16, uint8_t *, const uint8_t *table,
                                               const float *xs, int cols, int nrows, f32x2 (&acc)[RW][M], int lane) {
        constexpr int SLOT = slot_bytes(TYPE), CPB = chunk_block(TYPE) / 8, BB = chunk_block_bytes(TYPE);
#pragma unroll 1
        for (int j = 0; j < kChunksPerLane; ++j) {
            const int chunk = j * 32 + lane;
            if (chunk * 8 < cols) {
                X4 xa[M], xb[M];
#pragma unroll
                for (int t = 0; t < M; ++t) {
                    xa[t] = lds_x4(xs + t * kSegCols + chunk * 8);
                    xb[t] = lds_x4(xs + t * kSegCols + chunk * 8 + 4);
                }
                const int boff = (chunk / CPB) * BB, c = chunk % CPB;
#pragma unroll
                for (int r = 0; r < RW; ++r) {
                    if (r < nrows) {
                        float v[8];
                        deq8<TYPE>(stage + r * SLOT + ((d0 + r * rb16) & 15u) + boff, c, v, table);
                        const f32x2 v01 = pack2(v[0], v[1]), v23 = pack2(v[2], v[3]), v45 = pack2(v[4], v[5]), v67 = pack2(v[6], v[7]);
#pragma unroll
                        for (int t = 0; t < M; ++t)
                            acc[r][t] = fma2(v67, xb[t].p23, fma2(v45, xb[t].p01, fma2(v23, xa[t].p23, fma2(v01, xa[t].p01, acc[r][t]))));
                    }
                }
            }
        }
    }
};

// Q4_K.  Block (144 B, always 16-byte aligned): d, dmin (f16) | 12 bytes of 6-bit scales and mins | 128 bytes of
// nibbles; bytes 32p..32p+31 hold group 2p in their low and group 2p+1 in their high nibbles
// (engine/csrc/common/qwen_quant.cuh:165-175).  With q the raw nibble,
//     sum_i (dl q_i - ml) x_i  =  dl * sum_i q_i x_i  -  ml * sum_i x_i
// so the per-weight work is nibble -> float and one FMA; the group scale is applied to the partial sums.
//   scale pass : lane -> (row, block, half of the groups); decodes 4 scales and 4 mins with word-wide mask ops and
//                leaves, per pair of groups (2p, 2p+1), {dl, dl, dl'/16, dl'/16, -ml, -ml', 0, 0} in the warp's
//                scratch table (/16 because the high nibbles stay in place).
//   dot pass   : one block per pass, lane i -> 32-bit word i of the nibbles: 4 weights of group 2p (columns
//                64p + 4(i%8) ..) and 4 of group 2p+1 (32 columns further).  Eight lanes read 128 contiguous
//                bytes of activations per load, so the shared-memory reads are conflict-free.
template <int M, int RW>
struct Step<kQ4_K, M, RW> {
    // Scale table of the warp: for each (row, block, pair of groups) {dl, dl'/16, -ml, -ml'}, 16 bytes.  The
    // pairs with even and odd index live in two halves of the table so that consecutive lanes of the scale
    // pass store to consecutive 16-byte slots (no bank conflicts).
    static constexpr int kHalf = RW * 4 * 32 + 32;  // + 32: the two halves start 8 banks apart
    static constexpr int kScratch = 2 * kHalf;

    // Rows of the chunk that do not exist are skipped with warp-uniform branches.
    static __device__ __forceinline__ void run(const uint8_t *stage, uint32_t, uint32_t, uint8_t *scratch, const uint8_t *,
                                               const float *xs, int cols, int nrows, f32x2 (&acc)[RW][M], int lane) {
        constexpr int SLOT = slot_bytes(kQ4_K);
        const int nblk = cols >> 8;
        const f32x2 neg_magic = pack2(-8388608.0f, -8388608.0f);
        // ---- scale pass: lane -> (row, block, groups 4hh..4hh+3)
#pragma unroll
        for (int r0 = 0; r0 < RW; r0 += 4) {
            const int r = r0 + (lane >> 3), blk = (lane >> 1) & 3, hh = lane & 1;
            if (r < nrows) {
                const uint4 h = *reinterpret_cast<const uint4 *>(stage + r * SLOT + blk * 144);
                const float d = half_bits_to_float(h.x & 0xFFFFu), ndmin = -half_bits_to_float(h.x >> 16);
                // four 6-bit fields at a time (engine/csrc/common/qwen_quant.cuh:78-86)
                const uint32_t scw = hh ? ((h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u)) : (h.y & 0x3F3F3F3Fu);
                const uint32_t mnw = hh ? (((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u)) : (h.z & 0x3F3F3F3Fu);
                const f32x2 dd = pack2(d, d * 0.0625f), mm = pack2(ndmin, ndmin);
                ulonglong2 e0, e1;
                e0.x = mul2(bytes_to_pair<0, 1>(scw, neg_magic), dd);
                e0.y = mul2(bytes_to_pair<0, 1>(mnw, neg_magic), mm);
                e1.x = mul2(bytes_to_pair<2, 3>(scw, neg_magic), dd);
                e1.y = mul2(bytes_to_pair<2, 3>(mnw, neg_magic), mm);
                uint8_t *dst = scratch + (r * 4 + blk) * 32 + hh * 16;
                *reinterpret_cast<ulonglong2 *>(dst) = e0;          // pair 2hh
                *reinterpret_cast<ulonglong2 *>(dst + kHalf) = e1;  // pair 2hh + 1
            }
        }
        __syncwarp();
        // ---- dot pass: one block at a time, lane -> 32-bit word `lane` of the block's nibbles
        const int p = lane >> 3;
        const float *xl = xs + p * 64 + 4 * (lane & 7);
        const uint8_t *el = scratch + (p & 1) * kHalf + (p >> 1) * 16;
#pragma unroll
        for (int blk = 0; blk < 4; ++blk) {
            if (blk < nblk) {
                X4 xa[M], xb[M];
                f32x2 sx[M];
#pragma unroll
                for (int t = 0; t < M; ++t) {
                    xa[t] = lds_x4(xl + t * kSegCols + blk * 256);
                    xb[t] = lds_x4(xl + t * kSegCols + blk * 256 + 32);
                    sx[t] = pack2(sum_x4(xa[t]), sum_x4(xb[t]));
                }
#pragma unroll
                for (int r = 0; r < RW; ++r) {
                    if (r >= nrows) break;
                    const uint32_t w = *reinterpret_cast<const uint32_t *>(stage + r * SLOT + blk * 144 + 16 + 4 * lane);
                    const uint32_t lo = w & 0x0F0F0F0Fu, hi = w & 0xF0F0F0F0u;
                    const f32x2 a01 = bytes_to_pair<0, 1>(lo, neg_magic), a23 = bytes_to_pair<2, 3>(lo, neg_magic);
                    const f32x2 b01 = bytes_to_pair<0, 1>(hi, neg_magic), b23 = bytes_to_pair<2, 3>(hi, neg_magic);
                    const ulonglong2 e = *reinterpret_cast<const ulonglong2 *>(el + (r * 4 + blk) * 32);
                    float dl, dlh;
                    unpack2(e.x, dl, dlh);
                    const f32x2 dl2 = pack2(dl, dl), dlh2 = pack2(dlh, dlh);
#pragma unroll
                    for (int t = 0; t < M; ++t) {
                        const f32x2 sa = fma2(a23, xa[t].p23, mul2(a01, xa[t].p01));
                        const f32x2 sb = fma2(b23, xb[t].p23, mul2(b01, xb[t].p01));
                        acc[r][t] = fma2(e.y, sx[t], fma2(dlh2, sb, fma2(dl2, sa, acc[r][t])));
                    }
                }
            }
        }
        __syncwarp();  // the scratch table is rewritten by the next step
    }
};

// Q6_K and Q3_K share a block geometry: weight e = 128h + 32q + l (h: half, q: quarter, l < 32) takes its low bits from
// byte 32h + l of a 64-byte plane (Q6_K: two planes of nibbles, Q3_K: one plane of 2-bit fields) and its high bits
// from a second plane indexed by l, and weights 16k..16k+15 share sub-scale k = 8h + 2q + (l >> 4)
// (engine/csrc/common/qwen_quant.cuh:182-190,199-210).  Neither carries a minimum, so
//     sum_i dl q_i x_i = dl * sum_i q_i x_i      with q the raw field minus a constant (32 / 4).
//   scale pass : lane -> (row, block, 4 sub-scales): integer sub-scale -> float, times d, stored so that a dot-pass
//                lane finds the sub-scales of its four quarters in one 16-byte slot.
//   dot pass   : lane -> (block, half h, 4 consecutive l = 4j..4j+3): one word of each plane gives 16 weights, 4 per
//                quarter, at columns 128h + 32q + 4j.  Eight lanes read 128 contiguous bytes of activations.
//                Blocks are only 2-byte aligned, so plane words are fetched with aligned loads + a funnel shift;
//                a pass takes the blocks of equal parity, which have the same alignment in every lane.
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
    static __device__ __forceinline__ Words load(const uint8_t *bp, int h, int j) {
        return Words{ld32<2>(bp + 64 * h + 4 * j), ld32<2>(bp + 64 * h + 32 + 4 * j), ld32<2>(bp + 128 + 32 * h + 4 * j)};
    }
    // bytes = fields of quarter Q (4 weights), still carrying the bias
    template <int Q>
    static __device__ __forceinline__ uint32_t quarter(const Words &w, int) {
        const uint32_t ql = (Q & 1) ? w.ql1 : w.ql0;
        const uint32_t lo = (Q >= 2 ? (ql >> 4) : ql) & 0x0F0F0F0Fu;
        const uint32_t hi = Q == 0 ? (w.qh << 4) : Q == 1 ? (w.qh << 2) : Q == 2 ? w.qh : (w.qh >> 2);
        return lo | (hi & 0x30303030u);
    }
    // four sub-scales 4c..4c+3 as biased bytes, and d
    static __device__ __forceinline__ uint32_t scale_word(const uint8_t *bp, int c, float *d) {
        *d = half_bits_to_float(ld16(bp + 208));
        return ld32<2>(bp + 192 + 4 * c) ^ 0x80808080u;
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
    static __device__ __forceinline__ Words load(const uint8_t *bp, int h, int j) {
        return Words{ld32<2>(bp + 32 + 32 * h + 4 * j), ld32<2>(bp + 4 * j) >> (4 * h)};
    }
    template <int Q>
    static __device__ __forceinline__ uint32_t quarter(const Words &w, int) {
        const uint32_t lo = (Q == 0 ? w.qs : (w.qs >> (2 * Q))) & 0x03030303u;
        const uint32_t hb = Q == 0 ? (w.hm << 2) : Q == 1 ? (w.hm << 1) : Q == 2 ? w.hm : (w.hm >> 1);
        return lo | (hb & 0x04040404u);
    }
    static __device__ __forceinline__ uint32_t scale_word(const uint8_t *bp, int c, float *d) {
        *d = half_bits_to_float(ld16(bp + 108));
        // sub-scale k: low nibble from byte k % 8 (>> 4 for k >= 8), high 2 bits from byte 8 + k % 4 (>> 2 (k / 4))
        const uint32_t wl = ld32<2>(bp + 96 + 4 * (c & 1)), w2 = ld32<2>(bp + 104);
        const uint32_t lo = (wl >> (4 * (c >> 1))) & 0x0F0F0F0Fu;
        const uint32_t hi = static_cast<uint32_t>((static_cast<unsigned long long>(w2) << 4) >> (2 * c)) & 0x30303030u;
        return lo | hi;
    }
};

template <int TYPE, int M, int RW>
struct QuarterStep {
    using F = QuarterFormat<TYPE>;
    static constexpr int kEntry = 64;  // per (row, block): 16 sub-scales x d, as [h][l >> 4][quarter]
    static constexpr int kScratch = RW * 4 * kEntry;

    static __device__ __forceinline__ void run(const uint8_t *stage, uint32_t d0, uint32_t rb16, uint8_t *scratch, const uint8_t *,
                                               const float *xs, int cols, int nrows, f32x2 (&acc)[RW][M], int lane) {
        constexpr int SLOT = slot_bytes(TYPE), BB = F::kBlockBytes;
        const int nblk = cols >> 8;
        // ---- scale pass: task -> (row, block, scale word c)
        {
            const f32x2 neg_magic = pack2(-(8388608.0f + F::kScaleBias), -(8388608.0f + F::kScaleBias));
#pragma unroll
            for (int task0 = 0; task0 < 16 * RW; task0 += 32) {
                const int task = task0 + lane, r = task >> 4, blk = (task >> 2) & 3, c = task & 3;
                if (r < nrows) {
                    const uint8_t *bp = stage + r * SLOT + ((d0 + r * rb16) & 15u) + blk * BB;
                    float d;
                    const uint32_t sw = F::scale_word(bp, c, &d);
                    const f32x2 dd = pack2(d, d);
                    // sub-scale k = 4c + i belongs to half k >> 3, quarter (k >> 1) & 3, l >> 4 = k & 1
                    float *dst = reinterpret_cast<float *>(scratch + (r * 4 + blk) * kEntry) + (c >> 1) * 8 + 2 * (c & 1);
                    *reinterpret_cast<f32x2 *>(dst) = mul2(bytes_to_pair<0, 2>(sw, neg_magic), dd);      // l < 16: quarters 2(c&1), +1
                    *reinterpret_cast<f32x2 *>(dst + 4) = mul2(bytes_to_pair<1, 3>(sw, neg_magic), dd);  // l >= 16
                }
            }
        }
        __syncwarp();
        // ---- dot pass
        const f32x2 neg_magic = pack2(-(8388608.0f + F::kBias), -(8388608.0f + F::kBias));
        const int bsel = lane >> 4, h = (lane >> 3) & 1, j = lane & 7;
#pragma unroll
        for (int s = 0; s < 2; ++s) {
            const int blk = s + 2 * bsel;
            if (blk < nblk) {
                typename F::Words w[RW];
                float4 dl[RW];
#pragma unroll
                for (int r = 0; r < RW; ++r) {
                    if (r >= nrows) break;
                    w[r] = F::load(stage + r * SLOT + ((d0 + r * rb16) & 15u) + blk * BB, h, j);
                    dl[r] = *reinterpret_cast<const float4 *>(scratch + (r * 4 + blk) * kEntry + (h * 2 + (j >> 2)) * 16);
                }
                const float *xq = xs + blk * 256 + h * 128 + 4 * j;
                quarter_dot<0>(w, dl, xq, neg_magic, nrows, acc);
                quarter_dot<1>(w, dl, xq, neg_magic, nrows, acc);
                quarter_dot<2>(w, dl, xq, neg_magic, nrows, acc);
                quarter_dot<3>(w, dl, xq, neg_magic, nrows, acc);
            }
        }
        __syncwarp();  // the scratch table is rewritten by the next step
    }

    template <int Q>
    static __device__ __forceinline__ void quarter_dot(const typename F::Words (&w)[RW], const float4 (&dl)[RW], const float *xq,
                                                       f32x2 neg_magic, int nrows, f32x2 (&acc)[RW][M]) {
        X4 x[M];
#pragma unroll
        for (int t = 0; t < M; ++t) x[t] = lds_x4(xq + t * kSegCols + Q * 32);
#pragma unroll
        for (int r = 0; r < RW; ++r) {
            if (r >= nrows) break;
            const uint32_t q = F::template quarter<Q>(w[r], 0);
            const f32x2 q01 = bytes_to_pair<0, 1>(q, neg_magic), q23 = bytes_to_pair<2, 3>(q, neg_magic);
            const float d = Q == 0 ? dl[r].x : Q == 1 ? dl[r].y : Q == 2 ? dl[r].z : dl[r].w;
            const f32x2 d2 = pack2(d, d);
#pragma unroll
            for (int t = 0; t < M; ++t) acc[r][t] = fma2(d2, fma2(q23, x[t].p23, mul2(q01, x[t].p01)), acc[r][t]);
        }
    }
};

template <int M, int RW>
struct Step<kQ6_K, M, RW> : QuarterStep<kQ6_K, M, RW> {};
template <int M, int RW>
struct Step<kQ3_K, M, RW> : QuarterStep<kQ3_K, M, RW> {};

// ---- the kernel ------------------------------------------------------------------------------------------

template <int TYPE, int RW, int M>
__host__ __device__ constexpr size_t matvec_smem_bytes_for() {
    return matvec_smem_bytes(TYPE, RW, M) + static_cast<size_t>(kWarps) * Step<TYPE, M, RW>::kScratch;
}

template <int TYPE, int M, int RW>
__global__ void __launch_bounds__(kWarps * 32, (M <= 4 ? 2 : 1)) qmv_kernel(const MatvecArgs a) {
    using StepT = Step<TYPE, M, RW>;
    constexpr int S = stages_for(TYPE, RW);
    constexpr int XS = x_stages_for(M);
    constexpr int SLOT = slot_bytes(TYPE);
    constexpr int SEG = seg_bytes(TYPE);
    constexpr int TABLE = table_bytes_padded(TYPE);
    constexpr int XSTAGE = M * kSegCols * 4;
    constexpr bool kAligned = block_align(TYPE) >= 16;  // every segment starts on a 16-byte boundary
    static_assert(RW * M <= 32, "one lane per (row, activation row) output");
    static_assert(kWarps * 8 * 8 + 8 * 8 + 8 * 4 <= kBarrierBytes, "barrier area");

    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t *table = smem;
    uint64_t *wbars = reinterpret_cast<uint64_t *>(smem + TABLE);          // [kWarps][8] weight stages
    uint64_t *xfull = wbars + kWarps * 8;                                    // [XS] activation stages
    int *xdone = reinterpret_cast<int *>(xfull + 8);                         // [XS] warps done with the stage
    uint8_t *xbuf = smem + TABLE + kBarrierBytes;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint64_t *bar = wbars + warp * 8;
    uint8_t *buf = xbuf + XS * XSTAGE + static_cast<size_t>(warp) * (S * RW * SLOT);
    uint8_t *scratch = xbuf + XS * XSTAGE + static_cast<size_t>(kWarps) * (S * RW * SLOT) + warp * StepT::kScratch;

    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < S; ++s) mbar_init(bar + s, 1);
    }
    if (threadIdx.x == 0) {
#pragma unroll
        for (int s = 0; s < XS; ++s) {
            mbar_init(xfull + s, 1);
            xdone[s] = 0;
        }
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();

    // Even split of the rows over all warps of the grid: warp gw gets `my_count` consecutive rows from
    // `my_begin`, taken in `n_chunks` chunks of at most RW rows (chunk sizes differ by at most one).
    // n_chunks is the same for every warp, so the warps of a block share the activation stages.
    const int total_warps = gridDim.x * kWarps, gw = blockIdx.x * kWarps + warp;
    const int base = a.rows / total_warps, rem = a.rows % total_warps;
    const int my_count = base + (gw < rem ? 1 : 0), my_begin = gw * base + (gw < rem ? gw : rem);
    const int n_chunks = (base + (rem > 0 ? 1 : 0) + RW - 1) / RW;
    const int chunk_base = my_count / n_chunks, chunk_rem = my_count % n_chunks;  // chunk c has chunk_base + (c < chunk_rem) rows
    const int n_seg = (a.cols + kSegCols - 1) / kSegCols;
    const int n_steps = n_chunks * n_seg;
    const uintptr_t wbase = reinterpret_cast<uintptr_t>(a.w);
    const uint32_t rb16 = static_cast<uint32_t>(a.row_bytes) & 15u;

    // Activation stage for step `step` (segment `seg`): one bulk copy per activation row.  Called by one thread.
    auto issue_x = [&](int xstage, int seg) {
        const int cols_here = a.cols - seg * kSegCols < kSegCols ? a.cols - seg * kSegCols : kSegCols;
        mbar_expect_tx(xfull + xstage, static_cast<uint32_t>(M * cols_here * 4));
#pragma unroll
        for (int t = 0; t < M; ++t)
            bulk_copy_g2s(xbuf + xstage * XSTAGE + t * (kSegCols * 4), a.x + static_cast<size_t>(t) * a.cols + seg * kSegCols,
                          static_cast<uint32_t>(cols_here * 4), xfull + xstage);
    };

    // Weight issue side: lane r (< rows of the chunk) walks the byte range of row `i_row0 + r`, one segment per step.
    int i_chunk = 0, i_row0 = my_begin, i_nrows = chunk_base + (0 < chunk_rem ? 1 : 0), i_seg = 0, i_stage = 0;
    auto issue_w = [&]() {
        if (i_nrows > 0) {  // warp-uniform
            uint32_t bytes = 0;
            uintptr_t src = 0;
            if (lane < i_nrows) {
                const long long off = static_cast<long long>(i_seg) * SEG;
                const long long len = a.row_bytes - off < SEG ? a.row_bytes - off : SEG;
                const uintptr_t p = wbase + static_cast<uintptr_t>(i_row0 + lane) * static_cast<uintptr_t>(a.row_bytes) + off;
                src = p & ~static_cast<uintptr_t>(15);
                bytes = static_cast<uint32_t>((p - src + len + 15) & ~static_cast<uintptr_t>(15));
            }
            const uint32_t total = __reduce_add_sync(0xffffffffu, bytes);
            if (lane == 0) mbar_expect_tx(bar + i_stage, total);
            __syncwarp();
            if (bytes) bulk_copy_g2s(buf + (i_stage * RW + lane) * SLOT, reinterpret_cast<const void *>(src), bytes, bar + i_stage);
            if (++i_stage == S) i_stage = 0;
        }
        if (++i_seg == n_seg) {
            i_seg = 0;
            i_row0 += i_nrows;
            ++i_chunk;
            i_nrows = chunk_base + (i_chunk < chunk_rem ? 1 : 0);
        }
    };

    // The weights never depend on an earlier kernel, so their first copies go out at once; everything that reads the
    // activations or writes outputs comes after griddepcontrol.wait.  With programmatic dependent launch this block
    // may have started while the previous kernel of the stream was still draining, which hides the launch latency
    // and the first-byte latency of the weight stream (without that launch attribute both instructions are no-ops).
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    int issued = 0;
    for (; issued < S && issued < n_steps; ++issued) issue_w();
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (threadIdx.x == 0) {
        const int n = n_steps < XS ? n_steps : XS;
        for (int s = 0; s < n; ++s) issue_x(s, s % n_seg);
    }

    if constexpr (TABLE > 0) {
        if constexpr (grid_is_codebook(TYPE)) {
            const uint32_t *src = reinterpret_cast<const uint32_t *>(a.codebook);
            for (int i = threadIdx.x; i < grid_bytes(TYPE) / 4; i += blockDim.x) reinterpret_cast<uint32_t *>(table)[i] = src[i];
        } else {
            if (threadIdx.x < 16) reinterpret_cast<float *>(table)[threadIdx.x] = kIq4Levels[threadIdx.x];
        }
        __syncthreads();
    }

    f32x2 acc[RW][M];
#pragma unroll
    for (int r = 0; r < RW; ++r)
#pragma unroll
        for (int t = 0; t < M; ++t) acc[r][t] = 0ull;
    float best_v = -INFINITY;
    int best_i = 0x7fffffff;
    const bool want_argmax = a.out_idx != nullptr;
    bool expired = false;

    int stage = 0, xstage = 0, seg = 0, chunk = 0, row0 = my_begin, nrows = chunk_base + (0 < chunk_rem ? 1 : 0);
    uint32_t phase = 0, xphase = 0;
    for (int step = 0; step < n_steps; ++step) {
        if (!mbar_wait_bounded(xfull + xstage, xphase)) {
            expired = true;
            break;
        }
        const bool active = nrows > 0;
        if (active) {
            if (!mbar_wait_bounded(bar + stage, phase)) {
                expired = true;
                break;
            }
            const uint8_t *stage_buf = buf + stage * RW * SLOT;
            // where row 0's segment starts inside its slot (the copy began at the 16-byte boundary below it)
            const uint32_t d0 = kAligned ? 0u : (static_cast<uint32_t>(wbase & 15u) + static_cast<uint32_t>(row0) * rb16 +
                                                 static_cast<uint32_t>(seg) * (SEG & 15)) & 15u;
            const int cols_here = a.cols - seg * kSegCols < kSegCols ? a.cols - seg * kSegCols : kSegCols;
#ifdef VQM_PROBE_NO_COMPUTE  // experiment: stream the weights through the pipeline without decoding them
            acc[0][0] += static_cast<unsigned long long>(stage_buf[d0 + lane]);
#else
            StepT::run(stage_buf, d0, kAligned ? 0u : rb16, scratch, table, reinterpret_cast<const float *>(xbuf + xstage * XSTAGE),
                       cols_here, nrows, acc, lane);
#endif
        }
        __syncwarp();
        // Done with the activation stage; the last warp of the block to get here refills it.
        if (lane == 0) {
            __threadfence_block();
            if (atomicAdd(xdone + xstage, 1) == kWarps - 1) {
                xdone[xstage] = 0;
                __threadfence_block();
                if (step + XS < n_steps) {
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    issue_x(xstage, (seg + XS) % n_seg);
                }
            }
        }
        if (issued < n_steps) {
            issue_w();
            ++issued;
        }

        if (seg == n_seg - 1) {
            if (active) {
                // lane r*M + t ends up holding y[t][row0 + r]
                float mine = 0.0f;
#pragma unroll
                for (int r = 0; r < RW; ++r)
#pragma unroll
                    for (int t = 0; t < M; ++t) {
                        float lo, hi;
                        unpack2(acc[r][t], lo, hi);
                        const float s = warp_sum(lo + hi);
                        if (lane == r * M + t) mine = s;
                        acc[r][t] = 0ull;
                    }
                if (lane < RW * M) {
                    const int r = lane / M, t = lane % M, row = row0 + r;
                    if (r < nrows) {
                        if (a.y != nullptr) a.y[static_cast<size_t>(t) * a.rows + row] = mine;
                        if (want_argmax && better(mine, row, best_v, best_i)) {
                            best_v = mine;
                            best_i = row;
                        }
                    }
                }
            }
            seg = 0;
            row0 += nrows;
            ++chunk;
            nrows = chunk_base + (chunk < chunk_rem ? 1 : 0);
        } else {
            ++seg;
        }
        if (active && ++stage == S) {
            stage = 0;
            phase ^= 1u;
        }
        if (++xstage == XS) {
            xstage = 0;
            xphase ^= 1u;
        }
    }

    if (expired) {
        if (lane == 0) atomicExch(a.status, kStatusWaitExpired);
        // give the copies still in flight into this warp's buffers one more bounded chance to land
        for (int s = 0; s < S; ++s) (void)mbar_wait_bounded(bar + s, 0);
    }

    if (want_argmax) {
        // block partial per activation row, then the last block reduces all partials
        __shared__ float s_val[kWarps][32];
        __shared__ int s_idx[kWarps][32];
        __shared__ bool s_last;
        s_val[warp][lane] = best_v;
        s_idx[warp][lane] = best_i;
        __syncthreads();
        if (threadIdx.x < M) {
            const int t = threadIdx.x;
            float bv = -INFINITY;
            int bi = 0x7fffffff;
            for (int w = 0; w < kWarps; ++w)
                for (int r = 0; r < RW; ++r)
                    if (better(s_val[w][r * M + t], s_idx[w][r * M + t], bv, bi)) {
                        bv = s_val[w][r * M + t];
                        bi = s_idx[w][r * M + t];
                    }
            a.part_val[t * gridDim.x + blockIdx.x] = bv;
            a.part_idx[t * gridDim.x + blockIdx.x] = bi;
        }
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) s_last = atomicAdd(a.done_counter, 1u) == gridDim.x - 1;
        __syncthreads();
        if (s_last) {
            __threadfence();
            if (warp < M) {
                const int t = warp;
                float bv = -INFINITY;
                int bi = 0x7fffffff;
                for (int b = lane; b < static_cast<int>(gridDim.x); b += 32) {
                    const float v = __ldcg(a.part_val + t * gridDim.x + b);
                    const int i = __ldcg(a.part_idx + t * gridDim.x + b);
                    if (better(v, i, bv, bi)) {
                        bv = v;
                        bi = i;
                    }
                }
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) {
                    const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
                    const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
                    if (better(ov, oi, bv, bi)) {
                        bv = ov;
                        bi = oi;
                    }
                }
                if (lane == 0) {
                    a.out_idx[t] = bi == 0x7fffffff ? bi : bi + a.row_base;
                    if (a.out_val != nullptr) a.out_val[t] = bv;
                }
            }
            if (threadIdx.x == 0) *a.done_counter = 0;
        }
    }
}

}  // namespace vqm
