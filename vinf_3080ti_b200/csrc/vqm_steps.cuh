// Per-type step decoders of the quantized matvec kernel (vqm_matvec.cuh).
//
// A "step" is kSegCols (1024) columns of a warp's rows, staged in shared memory.  Step<TYPE, M, RW>::run adds the
// step's contribution to acc[r][t], an (even, odd) pair of fp32 partial sums per (row, activation row).  Everything
// here addresses shared memory through 32-bit shared-space addresses and explicit ld.shared / st.shared, which keeps
// the address arithmetic in 32 bits.
//   stage  : RW slots of slot_bytes(TYPE); row r's segment starts at stage + r * slot + ((d0 + r * rb16) & 15)
//   scratch: kScratch bytes of per-warp shared memory (scale tables)
//   table  : the type's lookup table (block-wide shared memory)
//   xs     : the staged activations of the segment, [M][kSegCols] fp32
//   cols   : columns of this segment (1024, or less for the last one; a multiple of the block size)
//   nrows  : rows of the chunk that exist (1..RW); the tuned decoders are compiled for a fixed row count NR and
//            run the smallest NR >= nrows they have (extra rows decode stale bytes and are dropped by the caller)
#pragma once

#include "vqm_formats.cuh"

namespace vqm {

constexpr int kSegCols = 1024;                 // columns per pipeline step
constexpr int kChunksPerLane = kSegCols / 256;  // 8-weight chunks a lane decodes per row per step (generic decoder)

__host__ __device__ constexpr int seg_bytes(int type) { return kSegCols / chunk_block(type) * chunk_block_bytes(type); }
// Slot that receives one row's segment: the copy is widened to 16-byte boundaries on both sides (up to 14 bytes in
// front), and the decoders' funnel loads may touch up to 4 bytes behind.
__host__ __device__ constexpr int slot_bytes(int type) { return (seg_bytes(type) + 14 + 8 + 15) / 16 * 16; }

// ---- shared-memory access ------------------------------------------------------------------------------

__device__ __forceinline__ uint32_t lds32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ unsigned long long lds64(uint32_t a) {
    unsigned long long v;
    asm volatile("ld.shared.u64 %0, [%1];" : "=l"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ ulonglong2 lds128(uint32_t a) {
    ulonglong2 v;
    asm volatile("ld.shared.v2.u64 {%0, %1}, [%2];" : "=l"(v.x), "=l"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ uint4 lds128u(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ void sts128(uint32_t a, unsigned long long x, unsigned long long y) {
    asm volatile("st.shared.v2.u64 [%0], {%1, %2};" ::"r"(a), "l"(x), "l"(y) : "memory");
}
// 32-bit word at a 2-byte aligned shared address: two aligned loads and a funnel shift.
__device__ __forceinline__ uint32_t lds32_a2(uint32_t a) {
    const uint32_t b = a & ~3u;
    return __funnelshift_r(lds32(b), lds32(b + 4), (a & 2u) * 8u);
}

// Eight bytes at a 2-byte aligned shared address: three aligned words and two funnel shifts.
__device__ __forceinline__ void lds64_a2(uint32_t a, uint32_t &lo, uint32_t &hi) {
    const uint32_t b = a & ~3u, sh = (a & 2u) * 8u;
    const uint32_t w0 = lds32(b), w1 = lds32(b + 4), w2 = lds32(b + 8);
    lo = __funnelshift_r(w0, w1, sh);
    hi = __funnelshift_r(w1, w2, sh);
}

// ---- packed fp32 arithmetic ------------------------------------------------------------------------------

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

// Byte K of `w` as the subnormal float byte * 2^-141 (the byte sits in bits 8..15 of an otherwise zero word): the
// cheapest exact integer -> float there is, one byte permute and no rebasing add.  fp32 multiplies and FMAs take
// subnormal inputs at full rate.  The tuned decoders multiply it by a group scale carrying an extra 2^64, which yields
// the dequantised weight times 2^-77 (exact, a power-of-two factor); sums are kept in that scale and the kernel
// multiplies each finished output by kOutScale = 2^77.  With fp16 block scales the scaled terms stay inside the normal
// fp32 range (largest group scale 65504 * 128 * 2^64 < 2^88; a weight of 2^-24 times 2^-77 is 2^-101).
constexpr float kSubScale = 0x1p64f;     // folded into the group scales
constexpr float kSubWeight = 0x1p-77f;   // dequantised weight -> value held in the sums (2^-141 * 2^64)
constexpr float kSubOutScale = 0x1p77f;  // applied once per output
template <int K0, int K1>
__device__ __forceinline__ f32x2 bytes_to_subpair(uint32_t w) {
    const uint32_t lo = __byte_perm(w, 0u, 0x4404 | (K0 << 4)), hi = __byte_perm(w, 0u, 0x4404 | (K1 << 4));
    f32x2 p;
    asm("mov.b64 %0, {%1, %2};" : "=l"(p) : "r"(lo), "r"(hi));
    return p;
}

// Four consecutive staged activations (16-byte aligned) as two packed pairs.
struct X4 {
    f32x2 p01, p23;
};
__device__ __forceinline__ X4 lds_x4(uint32_t a) {
    const ulonglong2 v = lds128(a);
    return X4{v.x, v.y};
}
__device__ __forceinline__ float sum_x4(const X4 &x) {
    float lo, hi;
    unpack2(add2(x.p01, x.p23), lo, hi);
    return lo + hi;
}

// Row counts a tuned decoder is compiled for, given the chunk height RW: RW/2 .. RW (the launcher picks the smallest
// RW that covers a warp's share of the rows, so fewer than RW/2 rows only occur in a tensor's last chunks).
template <template <int> class Pass, int RW, typename... Args>
__device__ __forceinline__ void dispatch_rows(int nrows, Args &&...args) {
    if constexpr (RW == 1) {
        Pass<1>::go(args...);
    } else if constexpr (RW == 2) {
        if (nrows <= 1) Pass<1>::go(args...);
        else Pass<2>::go(args...);
    } else if constexpr (RW == 4) {
        if (nrows <= 2) Pass<2>::go(args...);
        else if (nrows == 3) Pass<3>::go(args...);
        else Pass<4>::go(args...);
    } else {
        static_assert(RW == 8, "chunk heights are 1, 2, 4 or 8");
        if (nrows <= 4) Pass<4>::go(args...);
        else if (nrows == 5) Pass<5>::go(args...);
        else if (nrows == 6) Pass<6>::go(args...);
        else if (nrows == 7) Pass<7>::go(args...);
        else Pass<8>::go(args...);
    }
}

// ---- generic decoder ---------------------------------------------------------------------------------------
// One 8-weight chunk per lane at a time through deq8<TYPE>: exact dequantised values multiplied straight into the
// sums.  Correct for every type; the tuned decoders below replace it for the types the 27B layer set is made of.
template <int TYPE, int M, int RW>
struct Step {
    static constexpr int kScratch = 0;
    static constexpr float kOutScale = 1.0f;  // factor between the sums and the outputs
    static __device__ __forceinline__ void run(uint32_t stage, uint32_t d0, uint32_t rb16, uint32_t, uint32_t table, uint32_t xs,
                                               int cols, int nrows, f32x2 (&acc)[RW][M], int lane) {
        constexpr int SLOT = slot_bytes(TYPE), CPB = chunk_block(TYPE) / 8, BB = chunk_block_bytes(TYPE);
        const uint8_t *stage_p = static_cast<const uint8_t *>(__cvta_shared_to_generic(stage));
        const uint8_t *table_p = static_cast<const uint8_t *>(__cvta_shared_to_generic(table));
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
                const int boff = (chunk / CPB) * BB, c = chunk % CPB;
#pragma unroll
                for (int r = 0; r < RW; ++r) {
                    if (r < nrows) {
                        float v[8];
                        deq8<TYPE>(stage_p + r * SLOT + ((d0 + r * rb16) & 15u) + boff, c, v, table_p);
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

}  // namespace vqm
