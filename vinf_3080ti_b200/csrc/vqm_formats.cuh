// GGUF block formats for the quantized matvec: type ids, block traits and the per-chunk decoders.
//
// A "chunk" is 8 consecutive weights of one block (chunk c = weights 8c..8c+7), the same unit the
// reference's decoder works in (engine/csrc/common/qwen_quant.cuh:151-279).  The decoders here read the
// block from SHARED memory, where the matvec kernel has staged it with a bulk copy that keeps the
// block's global alignment modulo 16; blocks of most types are only 2-byte aligned, so multi-byte
// fields are fetched with aligned 32-bit loads and a funnel shift.
//
// Every product formed while dequantising (fp16 super-scale x integer sub-scale x integer quant or
// codebook value, and the 0.5 / 0.25 factors of the IQ2/IQ3 types) has at most 24 significant bits,
// so it is exact in fp32 in any order; the only rounding is the final `dl * q - ml` of the types
// that carry a minimum, done as one fused multiply-add.  The values are therefore bit-identical to
// the reference's double-precision dequantiser (engine/src/vinf/gguf/dequant.py:121-500) rounded to fp32.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace vqm {

// GGUF tensor type ids (engine/csrc/common/qwen_quant.cuh:17-33).
enum : int {
    kF32 = 0, kF16 = 1, kQ8_0 = 8, kQ2_K = 10, kQ3_K = 11, kQ4_K = 12, kQ5_K = 13, kQ6_K = 14,
    kIQ2_XXS = 16, kIQ2_XS = 17, kIQ3_XXS = 18, kIQ4_NL = 20, kIQ3_S = 21, kIQ2_S = 22, kIQ4_XS = 23,
};

struct Traits {
    int block;  // weights per block
    int size;   // bytes per block
};

// engine/csrc/common/qwen_quant.cuh:40-58
__host__ __device__ constexpr Traits traits_of(int type) {
    switch (type) {
        case kF32: return {1, 4};
        case kF16: return {1, 2};
        case kQ8_0: return {32, 34};
        case kQ2_K: return {256, 84};
        case kQ3_K: return {256, 110};
        case kQ4_K: return {256, 144};
        case kQ5_K: return {256, 176};
        case kQ6_K: return {256, 210};
        case kIQ4_NL: return {32, 18};
        case kIQ3_S: return {256, 110};
        case kIQ4_XS: return {256, 136};
        case kIQ2_XXS: return {256, 66};
        case kIQ2_XS: return {256, 74};
        case kIQ2_S: return {256, 82};
        case kIQ3_XXS: return {256, 98};
        default: return {0, 0};
    }
}

// Unquantised types are handled as pseudo-blocks of 8 weights (one chunk each).
__host__ __device__ constexpr int chunk_block(int type) { return traits_of(type).block >= 8 ? traits_of(type).block : 8; }
__host__ __device__ constexpr int chunk_block_bytes(int type) {
    return traits_of(type).block >= 8 ? traits_of(type).size : 8 * traits_of(type).size;
}

// Bytes of the lookup table a type's decoder indexes in shared memory (0 = none): the codebook of the
// IQ2/IQ3 types (engine/csrc/common/qwen_quant.cuh:142-144), or the 16 fp32 levels of IQ4_NL / IQ4_XS.
__host__ __device__ constexpr int grid_bytes(int type) {
    return type == kIQ3_S ? 2048 : type == kIQ2_XXS ? 2048 : type == kIQ2_XS ? 4096 : type == kIQ2_S ? 8192
         : type == kIQ3_XXS ? 1024 : (type == kIQ4_NL || type == kIQ4_XS) ? 64 : 0;
}
// True when the table comes from the caller (a GGUF codebook), false when it is built in.
__host__ __device__ constexpr bool grid_is_codebook(int type) { return grid_bytes(type) > 64; }

// Guaranteed alignment (bytes) of every block of a type when the tensor base is 16-byte aligned.
__host__ __device__ constexpr int block_align(int type) {
    const int s = chunk_block_bytes(type);
    return s % 16 == 0 ? 16 : s % 8 == 0 ? 8 : s % 4 == 0 ? 4 : 2;
}

// The 16 non-linear levels of IQ4_NL / IQ4_XS (engine/csrc/common/qwen_quant.cuh:60).
static __device__ __constant__ float kIq4Levels[16] = {-127.f, -104.f, -83.f, -65.f, -49.f, -35.f, -22.f, -10.f,
                                                      1.f, 13.f, 25.f, 38.f, 53.f, 69.f, 89.f, 113.f};

// ---- byte access ---------------------------------------------------------------------------------

__device__ __forceinline__ float half_bits_to_float(uint32_t h) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(h)));
}

// 16-bit little-endian field at a 2-byte aligned address.
__device__ __forceinline__ uint32_t ld16(const uint8_t *p) { return *reinterpret_cast<const uint16_t *>(p); }

// 32-bit little-endian word at an address with alignment A (A >= 4: one load; A == 2: two aligned
// loads and a funnel shift; reads up to 2 bytes past the word, which the staging slot pads for).
template <int A>
__device__ __forceinline__ uint32_t ld32(const uint8_t *p) {
    if constexpr (A >= 4) {
        return *reinterpret_cast<const uint32_t *>(p);
    } else {
        const uintptr_t a = reinterpret_cast<uintptr_t>(p);
        const uint32_t *q = reinterpret_cast<const uint32_t *>(a & ~static_cast<uintptr_t>(3));
        return __funnelshift_r(q[0], q[1], static_cast<uint32_t>(a & 2u) * 8u);
    }
}

// Two consecutive words (8 bytes).
template <int A>
__device__ __forceinline__ uint2 ld64(const uint8_t *p) {
    if constexpr (A >= 8) {
        return *reinterpret_cast<const uint2 *>(p);
    } else if constexpr (A >= 4) {
        const uint32_t *q = reinterpret_cast<const uint32_t *>(p);
        return make_uint2(q[0], q[1]);
    } else {
        const uintptr_t a = reinterpret_cast<uintptr_t>(p);
        const uint32_t *q = reinterpret_cast<const uint32_t *>(a & ~static_cast<uintptr_t>(3));
        const uint32_t sh = static_cast<uint32_t>(a & 2u) * 8u;
        const uint32_t w0 = q[0], w1 = q[1], w2 = q[2];
        return make_uint2(__funnelshift_r(w0, w1, sh), __funnelshift_r(w1, w2, sh));
    }
}

// Byte k of `w` as an exact float: the byte is dropped into the mantissa of 2^23 and 2^23 (+ bias) is
// subtracted, which avoids an integer-to-float conversion.  bias lets "q - 32" style offsets ride along.
template <int K>
__device__ __forceinline__ float byte_to_float(uint32_t w, float bias = 0.0f) {
    return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540 + K)) - (8388608.0f + bias);
}

__device__ __forceinline__ void bytes_to_floats(uint32_t w, float bias, float *v) {
    v[0] = byte_to_float<0>(w, bias);
    v[1] = byte_to_float<1>(w, bias);
    v[2] = byte_to_float<2>(w, bias);
    v[3] = byte_to_float<3>(w, bias);
}

// Small unsigned integer (< 2^23) to float without a conversion instruction.
__device__ __forceinline__ float small_uint_to_float(uint32_t v) { return __uint_as_float(0x4B000000u | v) - 8388608.0f; }

// (scale, min) pair g of the 12 packed bytes of Q4_K / Q5_K (engine/csrc/common/qwen_quant.cuh:78-86).
__device__ __forceinline__ void k4_scale_min(const uint8_t *s, int g, uint32_t *sc, uint32_t *mn) {
    if (g < 4) {
        *sc = s[g] & 63u;
        *mn = s[g + 4] & 63u;
    } else {
        *sc = (s[g + 4] & 0x0Fu) | ((s[g - 4] >> 6) << 4);
        *mn = (s[g + 4] >> 4) | ((s[g] >> 6) << 4);
    }
}

// Sign byte for a 7-bit index of IQ2_XXS / IQ2_XS / IQ3_XXS: bit 7 makes the parity even
// (the table c_ksigns_iq2xs of engine/csrc/common/qwen_iq_tables.h, computed instead of stored).
__device__ __forceinline__ uint32_t ksign(uint32_t s7) { return s7 | ((__popc(s7) & 1u) << 7); }

// v[i] = scale * mag_i with the sign bit taken from bit i of `signs` (bit set = negative).
__device__ __forceinline__ void signed_scaled4(uint32_t mags, float scale, uint32_t signs, float *v) {
    float m[4];
    bytes_to_floats(mags, 0.0f, m);
#pragma unroll
    for (int i = 0; i < 4; ++i)
        v[i] = __uint_as_float(__float_as_uint(scale * m[i]) ^ (((signs >> i) & 1u) << 31));
}

// ---- chunk decoders --------------------------------------------------------------------------------
// deq8<TYPE>(blk, c, v, grid): v[0..7] = weights 8c..8c+7 of the block at `blk` (shared memory).
// `grid` is the type's lookup table in shared memory (see grid_bytes), unused by the other types.

template <int TYPE>
__device__ __forceinline__ void deq8(const uint8_t *blk, int c, float v[8], const uint8_t *grid) {
    constexpr int A = block_align(TYPE);
    if constexpr (TYPE == kF32) {
        const float4 a = *reinterpret_cast<const float4 *>(blk), b = *reinterpret_cast<const float4 *>(blk + 16);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else if constexpr (TYPE == kF16) {
        const uint4 h = *reinterpret_cast<const uint4 *>(blk);
        const uint32_t w[4] = {h.x, h.y, h.z, h.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[2 * i] = half_bits_to_float(w[i] & 0xFFFFu);
            v[2 * i + 1] = half_bits_to_float(w[i] >> 16);
        }
    } else if constexpr (TYPE == kQ8_0) {
        // d (f16) @0, 32 x int8 @2
        const float d = half_bits_to_float(ld16(blk));
        const uint2 q = ld64<A>(blk + 2 + 8 * c);
        float f[8];
        bytes_to_floats(q.x ^ 0x80808080u, 128.0f, f);  // int8 + 128 is the unsigned byte
        bytes_to_floats(q.y ^ 0x80808080u, 128.0f, f + 4);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = d * f[i];
    } else if constexpr (TYPE == kIQ4_NL) {
        // d @0, 16 bytes of nibbles @2: weights 0..15 are the low nibbles, 16..31 the high ones
        const float d = half_bits_to_float(ld16(blk));
        const uint2 q = ld64<A>(blk + 2 + 8 * (c & 1));
        const int shift = (c >> 1) * 4;
        const uint32_t w[2] = {(q.x >> shift) & 0x0F0F0F0Fu, (q.y >> shift) & 0x0F0F0F0Fu};
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = d * reinterpret_cast<const float *>(grid)[(w[i >> 2] >> (8 * (i & 3))) & 0xFFu];
    } else if constexpr (TYPE == kQ4_K || TYPE == kQ5_K) {
        // d, dmin @0,2; 12 bytes of 6-bit scales/mins @4; Q4_K: nibbles @16; Q5_K: high bits @16, nibbles @48
        const uint32_t dd = ld32<A>(blk);
        const float d = half_bits_to_float(dd & 0xFFFFu), dmin = half_bits_to_float(dd >> 16);
        const int g = c >> 2, l0 = 8 * (c & 3);
        uint32_t sc, mn;
        k4_scale_min(blk + 4, g, &sc, &mn);
        const float dl = d * small_uint_to_float(sc), ml = dmin * small_uint_to_float(mn);
        const int shift = 4 * (g & 1);
        const uint2 q = ld64<A>(blk + (TYPE == kQ4_K ? 16 : 48) + 32 * (g >> 1) + l0);
        uint32_t w0 = (q.x >> shift) & 0x0F0F0F0Fu, w1 = (q.y >> shift) & 0x0F0F0F0Fu;
        if constexpr (TYPE == kQ5_K) {
            const uint2 h = ld64<A>(blk + 16 + l0);
            w0 |= ((h.x >> g) & 0x01010101u) << 4;
            w1 |= ((h.y >> g) & 0x01010101u) << 4;
        }
        float f[8];
        bytes_to_floats(w0, 0.0f, f);
        bytes_to_floats(w1, 0.0f, f + 4);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = fmaf(dl, f[i], -ml);
    } else if constexpr (TYPE == kQ6_K) {
        // low nibbles @0 (128), high 2 bits @128 (64), int8 scales @192 (16), d @208
        const int chunk = c >> 4, quarter = (c >> 2) & 3, l0 = 8 * (c & 3);
        const uint2 ql = ld64<A>(blk + chunk * 64 + (quarter & 1) * 32 + l0);
        const uint2 qh = ld64<A>(blk + 128 + chunk * 32 + l0);
        const float d = half_bits_to_float(ld16(blk + 208));
        const int sc = static_cast<int8_t>(blk[192 + (c >> 1)]);
        const float dl = d * static_cast<float>(sc);
        const int ls = (quarter >> 1) * 4, hs = 2 * quarter;
        const uint32_t w0 = ((ql.x >> ls) & 0x0F0F0F0Fu) | (((qh.x >> hs) & 0x03030303u) << 4);
        const uint32_t w1 = ((ql.y >> ls) & 0x0F0F0F0Fu) | (((qh.y >> hs) & 0x03030303u) << 4);
        float f[8];
        bytes_to_floats(w0, 32.0f, f);
        bytes_to_floats(w1, 32.0f, f + 4);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = dl * f[i];
    } else if constexpr (TYPE == kQ2_K) {
        // 16 scale/min bytes @0, 2-bit quants @16 (64), d @80, dmin @82
        const uint32_t dd = ld32<A>(blk + 80);
        const uint32_t s = blk[c >> 1];
        const float dl = half_bits_to_float(dd & 0xFFFFu) * small_uint_to_float(s & 15u);
        const float ml = half_bits_to_float(dd >> 16) * small_uint_to_float(s >> 4);
        const uint2 q = ld64<A>(blk + 16 + 32 * (c >> 4) + 8 * (c & 3));
        const int shift = 2 * ((c >> 2) & 3);
        float f[8];
        bytes_to_floats((q.x >> shift) & 0x03030303u, 0.0f, f);
        bytes_to_floats((q.y >> shift) & 0x03030303u, 0.0f, f + 4);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = fmaf(dl, f[i], -ml);
    } else if constexpr (TYPE == kQ3_K) {
        // high-bit mask @0 (32), 2-bit quants @32 (64), 12 bytes of 6-bit scales @96, d @108
        const int k = c >> 1;
        const uint8_t *s = blk + 96;
        const int lo = (s[k & 7] >> (4 * (k >> 3))) & 0x0F;
        const int hi = (s[8 + (k & 3)] >> (2 * (k >> 2))) & 0x03;
        const float dl = half_bits_to_float(ld16(blk + 108)) * static_cast<float>((lo | (hi << 4)) - 32);
        const uint2 q = ld64<A>(blk + 32 + 32 * (c >> 4) + 8 * (c & 3));
        const uint2 hm = ld64<A>(blk + 8 * (c & 3));
        const int shift = 2 * ((c >> 2) & 3), hbit = c >> 2;
        // q = low - (high bit set ? 0 : 4) = (low | high << 2) - 4
        const uint32_t w0 = ((q.x >> shift) & 0x03030303u) | (((hm.x >> hbit) & 0x01010101u) << 2);
        const uint32_t w1 = ((q.y >> shift) & 0x03030303u) | (((hm.y >> hbit) & 0x01010101u) << 2);
        float f[8];
        bytes_to_floats(w0, 4.0f, f);
        bytes_to_floats(w1, 4.0f, f + 4);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = dl * f[i];
    } else if constexpr (TYPE == kIQ4_XS) {
        // d @0, scales_h (u16) @2, scales_l @4 (4), nibbles @8 (128): group g = 16 bytes, low then high nibbles
        const uint32_t hdr = ld32<A>(blk);
        const float d = half_bits_to_float(hdr & 0xFFFFu);
        const int g = c >> 2;
        const int ls = ((blk[4 + (g >> 1)] >> (4 * (g & 1))) & 0x0F) | ((((hdr >> 16) >> (2 * g)) & 3) << 4);
        const float dl = d * static_cast<float>(ls - 32);
        const uint2 q = ld64<A>(blk + 8 + 16 * g + 8 * (c & 1));
        const int shift = ((c >> 1) & 1) * 4;
        const uint32_t w[2] = {(q.x >> shift) & 0x0F0F0F0Fu, (q.y >> shift) & 0x0F0F0F0Fu};
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = dl * reinterpret_cast<const float *>(grid)[(w[i >> 2] >> (8 * (i & 3))) & 0xFFu];
    } else if constexpr (TYPE == kIQ3_S) {
        // d @0, grid index low bytes @2 (64), index high bits @66 (8), sign bytes @74 (32), 4-bit scales @106 (4)
        const int g = c >> 2;
        const float db = half_bits_to_float(ld16(blk)) *
                         small_uint_to_float(1u + 2u * ((blk[106 + (g >> 1)] >> (4 * (g & 1))) & 0x0Fu));
        const uint32_t signs = blk[74 + c];
        const uint32_t idx = ld16(blk + 2 + 2 * c);  // two index bytes: entries 2c and 2c + 1
        const uint32_t hb = blk[66 + (c >> 2)] >> (2 * (c & 3));
        const uint32_t e0 = (idx & 0xFFu) | ((hb & 1u) << 8), e1 = (idx >> 8) | ((hb & 2u) << 7);
        const uint32_t *g32 = reinterpret_cast<const uint32_t *>(grid);
        signed_scaled4(g32[e0], db, signs, v);
        signed_scaled4(g32[e1], db, signs >> 4, v + 4);
    } else if constexpr (TYPE == kIQ2_XXS) {
        // d @0, then per 32 weights: 4 grid index bytes and a word of 4 x 7 sign bits + 4-bit scale
        const int ib = c >> 2, l = c & 3;
        const uint2 aux = ld64<A>(blk + 2 + 8 * ib);
        const float db = half_bits_to_float(ld16(blk)) * (0.5f + small_uint_to_float(aux.y >> 28)) * 0.25f;
        const uint32_t signs = ksign((aux.y >> (7 * l)) & 127u);
        const uint2 m = reinterpret_cast<const uint2 *>(grid)[(aux.x >> (8 * l)) & 0xFFu];
        signed_scaled4(m.x, db, signs, v);
        signed_scaled4(m.y, db, signs >> 4, v + 4);
    } else if constexpr (TYPE == kIQ2_XS) {
        // d @0, 32 x u16 (9-bit grid index, 7 sign bits) @2, 4-bit scale pairs @66 (8)
        const int ib = c >> 2, l = c & 3;
        const uint32_t q = ld16(blk + 2 + 2 * c);
        const float db = half_bits_to_float(ld16(blk)) *
                         (0.5f + small_uint_to_float((blk[66 + ib] >> (4 * (l >> 1))) & 0x0Fu)) * 0.25f;
        const uint32_t signs = ksign(q >> 9);
        const uint2 m = reinterpret_cast<const uint2 *>(grid)[q & 511u];
        signed_scaled4(m.x, db, signs, v);
        signed_scaled4(m.y, db, signs >> 4, v + 4);
    } else if constexpr (TYPE == kIQ2_S) {
        // d @0, index low bytes @2 (32), sign bytes @34 (32), index high bits @66 (8), scale pairs @74 (8)
        const int ib = c >> 2, l = c & 3;
        const uint32_t entry = blk[2 + c] | ((static_cast<uint32_t>(blk[66 + ib]) << (8 - 2 * l)) & 0x300u);
        const uint32_t signs = blk[34 + c];
        const float db = half_bits_to_float(ld16(blk)) *
                         (0.5f + small_uint_to_float((blk[74 + ib] >> (4 * (l >> 1))) & 0x0Fu)) * 0.25f;
        const uint2 m = reinterpret_cast<const uint2 *>(grid)[entry];
        signed_scaled4(m.x, db, signs, v);
        signed_scaled4(m.y, db, signs >> 4, v + 4);
    } else if constexpr (TYPE == kIQ3_XXS) {
        // d @0, grid index bytes @2 (64), per 32 weights a word of 4 x 7 sign bits + 4-bit scale @66
        const int ib = c >> 2, l = c & 3;
        const uint32_t aux = ld32<A>(blk + 66 + 4 * ib);
        const float db = half_bits_to_float(ld16(blk)) * (0.5f + small_uint_to_float(aux >> 28)) * 0.5f;
        const uint32_t signs = ksign((aux >> (7 * l)) & 127u);
        const uint32_t idx = ld16(blk + 2 + 2 * c);
        const uint32_t *g32 = reinterpret_cast<const uint32_t *>(grid);
        signed_scaled4(g32[idx & 0xFFu], db, signs, v);
        signed_scaled4(g32[idx >> 8], db, signs >> 4, v + 4);
    }
}

}  // namespace vqm
