// Prompt-pass GEMM on the 5th-generation tensor cores:  Y[t][r] = sum_k W[r][k] X[t][k]  for hundreds of activation rows.
//
// Same contract as the warp-level kernel in vqm_gemm.cu (replaces the reference's vinf_qgemm_kernel,
// engine/csrc/megakernel/qwen_runtime.cu:655-769: fp16 operands, fp32 accumulation), built on tcgen05:
//   * a block owns 128 weight rows per MMA M-half and 256 activation rows per accumulator, as one or two accumulators of
//     128 x 256 fp32 in tensor memory (at most 512 columns, the whole TMEM of an SM: one block per SM); the shapes are
//     listed at stage_bytes below;
//   * two blocks of a cluster work as a pair (tcgen05.mma.cta_group::2, M = 256): each decodes its own 128 weight rows
//     per accumulator and holds half of the accumulator's 256 activation rows in its shared memory, which halves what a
//     block reads of the activations from L2; the first block issues the MMAs for both and commits to the barriers of
//     both (multicast commit), the second block forwards its "full" slots to the first with one remote arrive per slot,
//     each block drains its own 128 lanes of tensor memory;
//   * the raw weight bytes come in by bulk copies (1-D TMA, no multicast), 256 columns of the block's rows at a time
//     into a ring of two shared-memory buffers, one copy per row issued by the row's first decoder thread, so that the
//     decoders never wait for global memory (F16 and F32, whose 256 columns are too wide for the ring, are decoded
//     straight from global memory);
//   * K is walked in stages of 64 (two to four stage buffers, as many as fit), each weight stage filled and consumed as
//     two halves of 32 (the pipeline's slots): warps 0-15 dequantise the weight half-tiles - warps 0-7 the first half
//     of every stage, warps 8-15 the second; four threads per row, one chunk of 8 weights each, two rows per thread -
//     with the exact block decoders (Q4_K, Q5_K, Q6_K, Q3_K and Q8_0 with a per-block header and constant shifts, see
//     FastHeader), store them as fp16 in the K-major 128-byte-swizzled layout the tensor core reads, make the writes
//     visible to the async proxy and arrive, once per warp, on the slot's "full" mbarrier;
//   * one thread of warp 16 feeds the activations: per stage one TMA tile copy (cp.async.bulk.tensor.2d, 64 columns x
//     the block's activation rows of an accumulator, written by the hardware in the same 128-byte swizzle; no
//     multicast) that completes on the stage's own mbarrier; a stage is refilled once the MMAs of its second half are done;
//   * one thread of warp 17 issues, per slot, 2 K-steps x the accumulators of tcgen05.mma (kind::f16, N = 256, K = 16)
//     from shared-memory descriptors and commits them to the slot's "empty" mbarrier, which hands the slot back to the
//     producers, so tile production runs up to a ring's length ahead of the MMAs;
//   * after the last commit, warps 0-15 read the accumulators with tcgen05.ld (warp w reads lanes 32 (w % 4) onwards, one
//     weight row per thread; the four warps of a lane group share the columns) and store y; a warp stores 32
//     consecutive rows of one activation row, 128 bytes.
// Where the time goes: profiles/prompt_gemm_tc5_Q4_K_17408x5120x512.md has the step-by-step history, the ablation builds
// (VQM_TC5_ABLATE) and the ncu figures.
// Every mbarrier wait is bounded: on expiry the block records a status code, everybody falls through to the end, and
// the tensor memory is released before the block returns.
#include <cuda.h>  // CUtensorMap and the driver entry point that encodes one (types only; nothing links against the driver)
#include <cuda_fp16.h>

#include "vqm_formats.cuh"
#include "vqm_kernels.h"
#include "vqm_steps.cuh"

#ifndef VQM_TC5_SHAPE
#define VQM_TC5_SHAPE 0  // experiment builds: block shape for more than 256 activation rows, see launch_t
#endif
#ifndef VQM_TC5_ABLATE
#define VQM_TC5_ABLATE 0  // experiment builds (wrong results): 1 = fast decoders store zeros, 2 = no activation copies,
                         // 4 = no proxy fence by the producers, 8 = only the MMA issue loop runs, without waiting
#endif

namespace vqm {
namespace {

// A block computes kTM * MR weight rows by kTNH * NH activation rows: MR x NH accumulators of 128 x 256 in tensor memory
// (MR * NH <= 2: 512 columns), alone or as a pair of blocks (see stage_bytes).  In use: 1 x 1 pairs up to 256 activation
// rows, 1 x 2 pairs above; 2 x 1 (256 weight rows per block halve what the blocks together read of the activations from
// L2, at the price of decoding every weight twice as often) and single blocks are kept for experiment builds, launch_t
// has the measurements.
constexpr int kTM = 128, kTNH = 256, kTK = 64;
constexpr int kMaxStages = 4;  // stages of the tile ring: as many as fit into shared memory, see stages_for
constexpr int kTA1 = kTM * kTK * 2, kTB1 = kTNH * kTK * 2;  // 16 KB per 128 weight rows, 32 KB per 256 activation rows
// With PAIR two blocks of a cluster (two SMs) work as one: tcgen05.mma.cta_group::2 multiplies the 256 weight rows of the
// two blocks (128 each, M = 256) by 256 activation rows of which each block holds one half in its shared memory, so a
// block pulls only half of the activation tile out of L2 - the traffic that bounds this kernel.  Accumulator rows stay
// with the block that decoded them (its 128 lanes of tensor memory).
__host__ __device__ constexpr int stage_bytes(int mr, int nh, bool pair) { return mr * kTA1 + nh * (pair ? kTB1 / 2 : kTB1); }
constexpr int kAThreads = 512;           // decoder warps 0-15
constexpr int kTThreads = kAThreads + 64;  // warp 16: one thread feeds the activation tiles (TMA); warp 17: one thread issues the MMAs
constexpr int kLoadWarp = kAThreads / 32;  // the MMA warp is the one after it
// Raw-block ring: a "column" is 256 weight columns of the 128 rows; a row's bytes of one column are contiguous.
constexpr int kRawCols = 256;
__host__ __device__ constexpr int raw_run_bytes(int type) { return kRawCols / chunk_block(type) * chunk_block_bytes(type); }
// slot of one row: the run, up to 14 bytes in front (the copy starts at the 16-byte boundary below), the decoders' reads
// of up to 8 bytes behind, rounded to 16
__host__ __device__ constexpr int raw_slot_bytes(int type) { return (raw_run_bytes(type) + 14 + 8 + 15) / 16 * 16; }
__host__ __device__ constexpr int table_bytes16(int type) { return grid_bytes(type) > 0 ? (grid_bytes(type) + 15) / 16 * 16 : 16; }
// Staged where the ring fits beside two stages of tiles: every quantised type in the shapes in use (Q8_0 only beside a
// pair's smaller stages); F16 and F32 never.
__host__ __device__ constexpr size_t smem_without_ring(int type, int mr, int nh, bool pair, int stages) {
    return table_bytes16(type) + 1024 + static_cast<size_t>(stages) * stage_bytes(mr, nh, pair);
}
__host__ __device__ constexpr bool raw_staged(int type, int mr, int nh, bool pair) {
    return raw_run_bytes(type) <= 272 && smem_without_ring(type, mr, nh, pair, 2) + 2 * mr * kTM * raw_slot_bytes(type) <= 227 * 1024;
}
__host__ __device__ constexpr int raw_ring_bytes(int type, int mr, int nh, bool pair) {
    return raw_staged(type, mr, nh, pair) ? 2 * mr * kTM * raw_slot_bytes(type) : 0;
}
__host__ __device__ constexpr size_t tc5_smem_bytes(int type, int mr, int nh, bool pair, int stages) {
    return smem_without_ring(type, mr, nh, pair, stages) + raw_ring_bytes(type, mr, nh, pair);
}
// The ring is what hides the refill round trip of a slot (MMAs done -> "empty" -> copies from L2 / decode -> "full"),
// which is several times longer than a slot's MMAs: every stage that fits is used.
__host__ __device__ constexpr int stages_for(int type, int mr, int nh, bool pair) {
    int s = kMaxStages;
    while (s > 2 && tc5_smem_bytes(type, mr, nh, pair, s) > 227 * 1024) --s;
    return s;
}
// 256 weight rows per block need the raw ring for 256 rows (reading them from global memory per chunk is too slow there)
[[maybe_unused]] __host__ __device__ constexpr bool fits_two_row_halves(int type, bool pair) { return raw_staged(type, 2, 1, pair); }

__device__ __forceinline__ uint32_t s32(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void bar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void bar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool bar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// try_wait that acquires at cluster scope: pairs with the other block's arrive of cluster scope
__device__ __forceinline__ bool bar_try_cluster(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait; also gives up as soon as another thread of the block has (`failed` is a shared flag).
__device__ __forceinline__ bool bar_wait(uint32_t bar, uint32_t parity, volatile int *failed) {
#pragma unroll 1
    for (int i = 0; i < (1 << 22); ++i) {  // a second or so
        // plain try_wait: measured against a suspend-time hint of 2 us (4 us slower on 125) and a test_wait spin (6 us slower)
        if (bar_try(bar, parity)) return true;
        if (*failed) return false;
        if (i > 4096) __nanosleep(200);  // only a wait that is already far beyond a pipeline step backs off
    }
    *failed = 1;
    return false;
}
__device__ __forceinline__ bool bar_wait_cluster(uint32_t bar, uint32_t parity, volatile int *failed) {
#pragma unroll 1
    for (int i = 0; i < (1 << 22); ++i) {
        if (bar_try_cluster(bar, parity)) return true;
        if (*failed) return false;
        if (i > 4096) __nanosleep(200);
    }
    *failed = 1;
    return false;
}

// Warp-wide forms (every lane of the warp calls them together).
//   warp_wait: every lane polls and the warp votes, so that it takes one branch even when a wait gives up.  (Polling by
//              lane 0 alone with a broadcast was measured: slower, 204 instead of 141 us for Q4_K 17408 x 5120 x 512.)
//   warp_arrive: one arrive per warp instead of 32 atomics on the barrier word, after the warp's own writes (and proxy
//              fences); __syncwarp orders them before lane 0's arrive.
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, volatile int *failed) {
    return __all_sync(0xFFFFFFFFu, bar_wait(bar, parity, failed) ? 1 : 0) != 0;
}
__device__ __forceinline__ void warp_arrive(uint32_t bar) {
    __syncwarp();
    if ((threadIdx.x & 31) == 0) bar_arrive(bar);
}

// Shared-memory matrix descriptor of a K-major tile in the 128-byte swizzle: rows of 64 fp16 = 128 bytes, groups of 8
// rows 1024 bytes apart (stride byte offset), tile base 1024-byte aligned; version 1 (sm_100), layout type 2.
__device__ __forceinline__ uint64_t sw128_desc(uint32_t addr) {
    return static_cast<uint64_t>((addr & 0x3FFFFu) >> 4) | (1ull << 16) | (static_cast<uint64_t>(1024 >> 4) << 32) | (1ull << 46) |
           (2ull << 61);
}
// Instruction descriptor, kind::f16: D fp32, A and B fp16, both K-major, N = 256, M = 128.
constexpr uint32_t kIdesc = (1u << 4) | ((256u >> 3) << 17) | ((128u >> 4) << 24);

__device__ __forceinline__ void mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(kIdesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// ---- fast chunk decoders of the producer warps --------------------------------------------------------------------------
// The generic block decoder (deq8) unpacks the block header for every chunk of 8 weights.  A producer thread stays on one
// row and walks a block's eight 32-column slots in order, so for the types below the header is unpacked once per block
// and a chunk is a load of 8 bytes, one byte permute per weight and packed fp32 arithmetic - the same operations in the
// same order as deq8, so the fp16 tiles are bit-identical to what the generic path stores.
template <int N>
struct Int {
    static constexpr int value = N;
};
__host__ __device__ constexpr bool has_fast_chunk(int type) { return type == kQ4_K || type == kQ5_K || type == kQ6_K || type == kQ3_K || type == kQ8_0; }

__device__ __forceinline__ uint32_t f16x2_of(f32x2 v) {  // (lo, hi) -> two fp16 in one word, round to nearest even
    float lo, hi;
    unpack2(v, lo, hi);
    uint32_t h;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(h) : "f"(hi), "f"(lo));
    return h;
}
// the four bytes of `w` times dl plus nml (packed), as fp16
__device__ __forceinline__ void bytes_fma_f16(uint32_t w, f32x2 neg_magic, f32x2 dl, f32x2 nml, uint32_t &h0, uint32_t &h1) {
    h0 = f16x2_of(fma2(bytes_to_pair<0, 1>(w, neg_magic), dl, nml));
    h1 = f16x2_of(fma2(bytes_to_pair<2, 3>(w, neg_magic), dl, nml));
}

template <int TYPE>
struct FastHeader;

// Q4_K / Q5_K (engine/csrc/common/qwen_quant.cuh:78-86, 171-196): d, dmin, 12 bytes of 6-bit scales and minimums; slot G of
// the block is its sub-block G (32 weights with one scale and one minimum), weight = d * sc * q - dmin * mn.
template <int TYPE>
struct FastHeaderK45 {
    uint32_t sc_lo, sc_hi, mn_lo, mn_hi;  // scales / minimums of sub-blocks 0..3 and 4..7, one per byte
    float d, ndmin;
    uint32_t qh0, qh1;  // Q5_K: the thread's 8 bytes of fifth bits (bit G belongs to slot G)
    __device__ __forceinline__ void load(uint32_t blk, int quarter) {
        const uint4 h = lds128u(blk);  // blocks of these types are 16-byte aligned
        d = half_bits_to_float(h.x & 0xFFFFu);
        ndmin = -half_bits_to_float(h.x >> 16);
        sc_lo = h.y & 0x3F3F3F3Fu;
        mn_lo = h.z & 0x3F3F3F3Fu;
        sc_hi = (h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u);
        mn_hi = ((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u);
        if constexpr (TYPE == kQ5_K) {
            const unsigned long long q = lds64(blk + 16 + 8 * quarter);
            qh0 = static_cast<uint32_t>(q), qh1 = static_cast<uint32_t>(q >> 32);
        }
    }
    template <int G>
    __device__ __forceinline__ void chunk(uint32_t blk, int quarter, uint32_t (&h)[4]) const {
        const float dl = d * byte_to_float<G & 3>(G < 4 ? sc_lo : sc_hi);
        const float nml = ndmin * byte_to_float<G & 3>(G < 4 ? mn_lo : mn_hi);  // -(dmin * mn), exactly
        const unsigned long long q = lds64(blk + (TYPE == kQ4_K ? 16 : 48) + 32 * (G >> 1) + 8 * quarter);
        uint32_t w0 = static_cast<uint32_t>(q), w1 = static_cast<uint32_t>(q >> 32);
        if constexpr (G & 1) w0 >>= 4, w1 >>= 4;
        w0 &= 0x0F0F0F0Fu, w1 &= 0x0F0F0F0Fu;
        if constexpr (TYPE == kQ5_K) {
            w0 |= (G <= 4 ? qh0 << (4 - G) : qh0 >> (G - 4)) & 0x10101010u;
            w1 |= (G <= 4 ? qh1 << (4 - G) : qh1 >> (G - 4)) & 0x10101010u;
        }
        const f32x2 neg_magic = pack2(-8388608.0f, -8388608.0f), dl2 = pack2(dl, dl), nml2 = pack2(nml, nml);
        bytes_fma_f16(w0, neg_magic, dl2, nml2, h[0], h[1]);
        bytes_fma_f16(w1, neg_magic, dl2, nml2, h[2], h[3]);
    }
};
template <>
struct FastHeader<kQ4_K> : FastHeaderK45<kQ4_K> {};
template <>
struct FastHeader<kQ5_K> : FastHeaderK45<kQ5_K> {};
// the four bytes of `w` (minus the bias inside neg_magic) times dl (packed), as fp16
__device__ __forceinline__ void bytes_mul_f16(uint32_t w, f32x2 neg_magic, f32x2 dl, uint32_t &h0, uint32_t &h1) {
    h0 = f16x2_of(mul2(bytes_to_pair<0, 1>(w, neg_magic), dl));
    h1 = f16x2_of(mul2(bytes_to_pair<2, 3>(w, neg_magic), dl));
}

// Q6_K (engine/csrc/common/qwen_quant.cuh:197-212): low nibbles @0 (128), high 2 bits @128 (64), int8 scales @192 (16),
// d @208; weight = d * sc * (q - 32).  Chunk c = 4 G + quarter of the block: low nibbles at 64 (G / 4) + 32 (G % 2) +
// 8 quarter, nibble (G % 4) / 2; high bits at 128 + 32 (G / 4) + 8 quarter, bit pair G % 4; scale c / 2.  The thread's six
// 8-byte fields of the block are loaded once (the blocks are only 2-byte aligned).
template <>
struct FastHeader<kQ6_K> {
    uint32_t ql[4][2], qh[2][2];  // [G / 4 * 2 + G % 2], [G / 4]
    uint32_t sc[2];               // the thread's eight scales (slots 0..3, 4..7), one per byte, as int8 + 128
    float d;
    __device__ __forceinline__ void load(uint32_t blk, int quarter) {
#pragma unroll
        for (int i = 0; i < 4; ++i) lds64_a2(blk + (i >> 1) * 64 + (i & 1) * 32 + 8 * quarter, ql[i][0], ql[i][1]);
#pragma unroll
        for (int i = 0; i < 2; ++i) lds64_a2(blk + 128 + 32 * i + 8 * quarter, qh[i][0], qh[i][1]);
        uint32_t s0, s1, s2, s3;  // the 16 scales; the thread's are the even or the odd bytes
        lds64_a2(blk + 192, s0, s1);
        lds64_a2(blk + 200, s2, s3);
        const uint32_t sel = (quarter >> 1) ? 0x7531u : 0x6420u;
        sc[0] = __byte_perm(s0, s1, sel) ^ 0x80808080u;
        sc[1] = __byte_perm(s2, s3, sel) ^ 0x80808080u;
        d = half_bits_to_float(lds16(blk + 208));
    }
    template <int G>
    __device__ __forceinline__ void chunk(uint32_t, int, uint32_t (&h)[4]) const {
        const float dl = d * byte_to_float<G & 3>(sc[G >> 2], 128.0f);
        constexpr int LS = ((G & 3) >> 1) * 4, HS = 2 * (G & 3);
        uint32_t w[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const uint32_t lo = ql[(G >> 2) * 2 + (G & 1)][i], hi = qh[G >> 2][i];
            w[i] = ((lo >> LS) & 0x0F0F0F0Fu) | ((HS <= 4 ? hi << (4 - HS) : hi >> (HS - 4)) & 0x30303030u);
        }
        const f32x2 neg_magic = pack2(-(8388608.0f + 32.0f), -(8388608.0f + 32.0f)), dl2 = pack2(dl, dl);
        bytes_mul_f16(w[0], neg_magic, dl2, h[0], h[1]);
        bytes_mul_f16(w[1], neg_magic, dl2, h[2], h[3]);
    }
};

// Q3_K (engine/csrc/common/qwen_quant.cuh:225-246): high-bit mask @0 (32), 2-bit quants @32 (64), 12 bytes of 6-bit
// scales @96, d @108; weight = d * (sc - 32) * ((q2 | hbit << 2) - 4).  Chunk c = 4 G + quarter: quants at 32 + 32 (G / 4) +
// 8 quarter, bit pair G % 4; mask at 8 quarter, bit G; scale c / 2.
template <>
struct FastHeader<kQ3_K> {
    uint32_t hm[2], qs[2][2];
    uint32_t sc[4];  // sc[G / 2]: the scale of slot G in byte 2 (G % 2), as the 6-bit field (32 too large)
    float d;
    __device__ __forceinline__ void load(uint32_t blk, int quarter) {
        lds64_a2(blk + 8 * quarter, hm[0], hm[1]);
#pragma unroll
        for (int i = 0; i < 2; ++i) lds64_a2(blk + 32 + 32 * i + 8 * quarter, qs[i][0], qs[i][1]);
        uint32_t s0, s1;
        lds64_a2(blk + 96, s0, s1);
        const uint32_t s2 = lds32_a2(blk + 104);
        d = half_bits_to_float(lds16(blk + 108));
        // scales k = 0..15, four per word: low nibbles of bytes 0..7 (k < 8) or their high nibbles, two more bits from
        // byte 8 + k % 4 at bit pair k / 4
        const uint32_t k0 = (s0 & 0x0F0F0F0Fu) | ((s2 << 4) & 0x30303030u), k1 = (s1 & 0x0F0F0F0Fu) | ((s2 << 2) & 0x30303030u);
        const uint32_t k2 = ((s0 >> 4) & 0x0F0F0F0Fu) | (s2 & 0x30303030u), k3 = ((s1 >> 4) & 0x0F0F0F0Fu) | ((s2 >> 2) & 0x30303030u);
        // the thread's scale of slot G is k = 2 G + quarter / 2: byte 2 (G % 2) + quarter / 2 of word G / 2
        const uint32_t sh = (quarter >> 1) * 8;
        sc[0] = k0 >> sh, sc[1] = k1 >> sh, sc[2] = k2 >> sh, sc[3] = k3 >> sh;
    }
    template <int G>
    __device__ __forceinline__ void chunk(uint32_t, int, uint32_t (&h)[4]) const {
        const float dl = d * byte_to_float<2 * (G & 1)>(sc[G >> 1], 32.0f);
        constexpr int QS = 2 * (G & 3);
        uint32_t w[2];
#pragma unroll
        for (int i = 0; i < 2; ++i)
            w[i] = ((qs[G >> 2][i] >> QS) & 0x03030303u) | ((G <= 2 ? hm[i] << (2 - G) : hm[i] >> (G - 2)) & 0x04040404u);
        const f32x2 neg_magic = pack2(-(8388608.0f + 4.0f), -(8388608.0f + 4.0f)), dl2 = pack2(dl, dl);
        bytes_mul_f16(w[0], neg_magic, dl2, h[0], h[1]);
        bytes_mul_f16(w[1], neg_magic, dl2, h[2], h[3]);
    }
};

// Q8_0 (engine/csrc/common/qwen_quant.cuh:163-170): blocks of 32 weights, d @0 and 32 int8 @2; slot G of a 256-column run is
// its block G, the thread's chunk the 8 bytes at 2 + 8 * quarter of it.  Nothing to unpack per run.
template <>
struct FastHeader<kQ8_0> {
    __device__ __forceinline__ void load(uint32_t, int) {}
    template <int G>
    __device__ __forceinline__ void chunk(uint32_t blk, int quarter, uint32_t (&h)[4]) const {
        const uint32_t at = blk + G * 34;
        const float d = half_bits_to_float(lds16(at));
        uint32_t w0, w1;
        lds64_a2(at + 2 + 8 * quarter, w0, w1);
        const f32x2 neg_magic = pack2(-(8388608.0f + 128.0f), -(8388608.0f + 128.0f)), d2 = pack2(d, d);
        bytes_mul_f16(w0 ^ 0x80808080u, neg_magic, d2, h[0], h[1]);  // int8 + 128 is the unsigned byte
        bytes_mul_f16(w1 ^ 0x80808080u, neg_magic, d2, h[2], h[3]);
    }
};

// (types without a fast decoder never instantiate this)
template <int TYPE>
struct FastHeader {
    __device__ __forceinline__ void load(uint32_t, int) {}
    template <int G>
    __device__ __forceinline__ void chunk(uint32_t, int, uint32_t (&)[4]) const {}
};

// ---- the two blocks of a pair ----------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// the address, in the cluster's shared window, of the same variable in block `rank`
__device__ __forceinline__ uint32_t in_block(uint32_t local, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
    return r;
}
__device__ __forceinline__ void bar_arrive_cluster(uint32_t cluster_addr) {
    // default semantics, as for a consumer's release of a remote slot; with .release.cluster every slot took 0.2 us longer
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Instruction descriptor of the pair MMA: M = 256 (128 rows from each block), N = 256.
constexpr uint32_t kIdescPair = (1u << 4) | ((256u >> 3) << 17) | ((256u >> 4) << 24);
__device__ __forceinline__ void mma_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(kIdescPair), "r"(accumulate)
        : "memory");
}
// arrives on the barrier at this address in both blocks of the pair once the MMAs issued so far are done
__device__ __forceinline__ void mma_commit_pair(uint32_t bar) {
    const uint16_t both = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar), "h"(both)
                 : "memory");
}

template <int TYPE, int MR, int NH, bool PAIR>
__global__ void __launch_bounds__(kTThreads, 1) qgemm_tc5_kernel(const __grid_constant__ CUtensorMap x_map, const uint8_t *w, float *y, int rows,
                                                                 int cols, long long row_bytes, int ntok, const uint8_t *codebook,
                                                                 unsigned *status) {
    constexpr int CPB = chunk_block(TYPE) / 8, BB = chunk_block_bytes(TYPE);
    constexpr int TABLE = table_bytes16(TYPE);
    constexpr int kTStage = stage_bytes(MR, NH, PAIR), kTA = MR * kTA1, kTN = NH * kTNH;
    constexpr int kBN = PAIR ? kTNH / 2 : kTNH;       // activation rows of an accumulator's tile that this block holds
    constexpr int kRowsPerAcc = PAIR ? 2 * kTM : kTM;  // weight rows of an accumulator (both blocks of a pair)
    constexpr int kTStages = stages_for(TYPE, MR, NH, PAIR), kTSlots = 2 * kTStages;  // slots: half stages
    constexpr uint32_t kTmemCols = 256 * MR * NH;
    static_assert(MR * NH <= 2, "512 columns of tensor memory");
    extern __shared__ uint8_t tc5_raw[];
    __shared__ __align__(8) uint64_t s_full[2 * kMaxStages], s_empty[2 * kMaxStages], s_xfull[kMaxStages], s_done, s_raw_full[2], s_raw_empty[2];
    __shared__ uint32_t s_tmem;
    __shared__ int s_failed;
    // table first, then the stages on a 1024-byte boundary (the swizzle works on absolute shared-memory address bits)
    uint8_t *table = tc5_raw;
    const uint32_t tiles = (s32(tc5_raw) + TABLE + 1023u) & ~1023u;
    constexpr bool kStaged = raw_staged(TYPE, MR, NH, PAIR);
    constexpr int RSLOT = raw_slot_bytes(TYPE), RUN = raw_run_bytes(TYPE);
    const uint32_t raw_ring = tiles + kTStages * kTStage;  // two buffers of MR * kTM row slots
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // a pair is two consecutive blocks of the grid's x; block `rank` of it owns rows rank * 128 .. + 127 of each accumulator
    const uint32_t rank = PAIR ? cluster_rank() : 0u;
    const int row0 = static_cast<int>(PAIR ? blockIdx.x >> 1 : blockIdx.x) * (kRowsPerAcc * MR) + static_cast<int>(rank) * kTM;
    const int tok0 = blockIdx.y * kTN;
    const int n_k = cols / kTK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kTSlots; ++s) {
            // one arrive per decoder warp of the group that owns the slot, and in the first block of a pair one more for the
            // second block's slot
            bar_init(s32(&s_full[s]), kAThreads / 64 + ((PAIR && rank == 0) ? 1 : 0));
            bar_init(s32(&s_empty[s]), 1);
        }
        for (int s = 0; s < kTStages; ++s) bar_init(s32(&s_xfull[s]), 1);  // the feeding thread's arrive with the stage's byte count
        bar_init(s32(&s_done), 1);
        for (int b = 0; b < 2; ++b) {
            bar_init(s32(&s_raw_full[b]), kTM / 2);     // one arrive (with its byte count) per copy-issuing thread
            bar_init(s32(&s_raw_empty[b]), kAThreads / 32);  // every decoder warp is done with the buffer
        }
        s_failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if constexpr (grid_bytes(TYPE) > 0) {
        if constexpr (grid_is_codebook(TYPE)) {
            for (int i = threadIdx.x; i < grid_bytes(TYPE) / 4; i += blockDim.x)
                reinterpret_cast<uint32_t *>(table)[i] = reinterpret_cast<const uint32_t *>(codebook)[i];
        } else {
            if (threadIdx.x < 16) reinterpret_cast<float *>(table)[threadIdx.x] = kIq4Levels[threadIdx.x];
        }
    }
    if (warp == 0) {  // tensor memory: 256 columns per accumulator (one block per SM)
        if constexpr (PAIR) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(&s_tmem)), "r"(kTmemCols) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(&s_tmem)), "r"(kTmemCols) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if constexpr (PAIR) cluster_sync_all();  // the other block's barriers and tensor memory exist before anybody signals or multiplies
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;
    volatile int *failed = &s_failed;
    // "full" is counted per block; the second block of a pair forwards each completed slot to the first block, which
    // issues the MMAs, with one arrive of cluster scope (such an arrive per producer warp made every slot take a
    // microsecond)
    auto full_arrive = [&](int slot) { warp_arrive(s32(&s_full[slot])); };

    const int n_slots = 2 * n_k;  // slot q of the pipeline: stage (q / 2) % 2, K half q % 2
#if VQM_TC5_ABLATE & 8
    if (warp <= kLoadWarp) {
    } else
#endif
    if (warp < 16) {
        // ---- weight half-tile: four threads per row, one chunk each; chunk c of the stage (8 weights, 16 bytes of fp16)
        //      goes to 16-byte slot c ^ (row % 8) of the row.
        // What a warp does for a slot is one chain of dependent steps (wait for "empty", load, decode, store, proxy fence,
        // arrive), so the warps are split into two groups that take the slots in turn - warps 0-7 the first K half of
        // every stage, warps 8-15 the second - and a thread decodes two rows (r and r + 64) of each row half instead of
        // one: twice the independent work per chain, half as many chains per warp (measured on one GPU with the TMA-fed
        // activation tiles, 17408 x 5120 x 512: IQ4_XS with the generic decoder 103-105 instead of 108-113 us, the types
        // with a fast decoder unchanged within the spread between runs).
        // The rows of a warp go 0, 4, 1, 5, ...: the 8 lanes the store unit serves together then hit 8 different 16-byte
        // columns of the swizzle (rows r and r + 4 use opposite halves).
        constexpr int NR = 2 * MR;  // rows per thread: i -> row half i / 2, row r + 64 * (i % 2) of it
        const int grp = warp >> 3;
        const int quarter = threadIdx.x & 3, r8 = (threadIdx.x >> 2) & 7;
        const int r = (warp & 7) * 8 + ((r8 >> 1) | ((r8 & 1) << 2));
        bool valid[NR];
        const uint8_t *w_row[NR];
#pragma unroll
        for (int i = 0; i < NR; ++i) {
            const int row = row0 + (i >> 1) * kRowsPerAcc + r + 64 * (i & 1);
            valid[i] = row < rows;
            w_row[i] = w + static_cast<size_t>(valid[i] ? row : 0) * row_bytes;
        }
        // One slot of this thread: wait until the MMAs that read the slot's previous contents are done, store the 8 fp16
        // weights of chunk `quarter` of the half stage for each of its rows (swizzled), make them visible to the tensor
        // core, arrive.
        auto slot_wait = [&](int q) -> bool { return warp_wait(s32(&s_empty[q % kTSlots]), ((q / kTSlots) & 1) ^ 1, failed); };
        auto slot_put = [&](int q, int i, const uint32_t (&h)[4]) {
            const int slot = q % kTSlots, c = (slot & 1) * 4 + quarter;  // chunk within the stage
            const int row = (i >> 1) * kTM + r + 64 * (i & 1);          // row of the block's weight tile
            asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(tiles + (slot >> 1) * kTStage + row * 128 + ((c ^ (r & 7)) << 4)),
                         "r"(h[0]), "r"(h[1]), "r"(h[2]), "r"(h[3])
                         : "memory");
        };
        auto slot_done = [&](int q) {
#if !(VQM_TC5_ABLATE & 4)
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
#endif
            full_arrive(q % kTSlots);
        };
        auto to_f16 = [](const float (&v)[8], uint32_t (&h)[4]) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const __half2 p = __floats2half2_rn(v[2 * e], v[2 * e + 1]);
                h[e] = *reinterpret_cast<const uint32_t *>(&p);
            }
        };
        if constexpr (!kStaged) {
            static_assert(kStaged || MR == 1, "two row halves only with the raw ring");
            for (int q = grp; q < n_slots; q += 2) {
                if (!slot_wait(q)) break;
                const int kc = (q >> 1) * (kTK / 8) + (q & 1) * 4 + quarter;  // chunk within the row
#pragma unroll
                for (int i = 0; i < NR; ++i) {
                    uint32_t h[4] = {0u, 0u, 0u, 0u};
                    if (valid[i]) {
                        float v[8];
                        deq8<TYPE>(w_row[i] + static_cast<size_t>(kc / CPB) * BB, kc % CPB, v, table);
                        to_f16(v, h);
                    }
                    slot_put(q, i, h);
                }
                slot_done(q);
            }
        } else {
            // Raw ring: column `col` (256 weight columns) of the block's rows goes to buffer col % 2.  The first thread of a
            // row in the first group issues the copies of its rows; the bytes keep their position inside their 16-byte line.
            constexpr int kSlotsPerCol = 2 * kRawCols / kTK;  // 8
            const int n_raw = (cols + kRawCols - 1) / kRawCols;
            int raw_issued = 0;  // columns this thread has queued copies for
            int raw_taken = 0;   // columns whose bytes this thread has waited for
            auto issue_raw = [&](int col) -> bool {  // the whole warp calls it (first group only); true unless a wait gave up
                const int b = col & 1;
                if (col >= 2 && !warp_wait(s32(&s_raw_empty[b]), ((col >> 1) - 1) & 1, failed)) return false;
                if (quarter == 0) {
                    raw_issued = col + 1;
                    const long long at = static_cast<long long>(col) * RUN;
                    const uint32_t run = row_bytes - at < RUN ? static_cast<uint32_t>(row_bytes - at) : static_cast<uint32_t>(RUN);
                    const uint32_t bar = s32(&s_raw_full[b]);
                    uintptr_t p[NR];
                    uint32_t bytes[NR], total = 0;
#pragma unroll
                    for (int i = 0; i < NR; ++i) {
                        p[i] = reinterpret_cast<uintptr_t>(w_row[i]) + static_cast<uintptr_t>(at);
                        bytes[i] = valid[i] ? ((static_cast<uint32_t>(p[i]) & 15u) + run + 15u) & ~15u : 0u;
                        total += bytes[i];
                    }
                    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(total) : "memory");
#pragma unroll
                    for (int i = 0; i < NR; ++i)
                        if (bytes[i])
                            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                                             raw_ring + ((b * MR + (i >> 1)) * kTM + r + 64 * (i & 1)) * RSLOT),
                                         "l"(p[i] & ~static_cast<uintptr_t>(15)), "r"(bytes[i]), "r"(bar)
                                         : "memory");
                }
                return true;
            };
            // Before slot g of column col.  Column col + 1 goes into the buffer column col - 1 left a little earlier: by the
            // first group's second slot every decoder warp has normally handed it back, so the wait inside holds nobody up.
            auto slot_begin = [&](int col, int g) -> bool {
                if (g == 2 && col >= 1 && col + 1 < n_raw && !issue_raw(col + 1)) return false;
                return slot_wait(col * kSlotsPerCol + g);
            };
            bool alive = grp != 0 || (issue_raw(0) && (n_raw < 2 || issue_raw(1)));
            for (int col = 0; alive && col < n_raw; ++col) {
                if (!warp_wait(s32(&s_raw_full[col & 1]), (col >> 1) & 1, failed)) break;  // every lane: it reads the bytes
                raw_taken = col + 1;
                uint32_t blk[NR];  // the rows' blocks of this column
#pragma unroll
                for (int i = 0; i < NR; ++i)
                    blk[i] = raw_ring + (((col & 1) * MR + (i >> 1)) * kTM + r + 64 * (i & 1)) * RSLOT +
                             (static_cast<uint32_t>(reinterpret_cast<uintptr_t>(w_row[i]) + static_cast<uintptr_t>(col) * RUN) & 15u);
                if constexpr (has_fast_chunk(TYPE)) {
                    // one block per column; the block header is unpacked once, the group's four slots are unrolled so that
                    // every shift and byte position is a constant
                    FastHeader<TYPE> hdr[NR];
#pragma unroll
                    for (int i = 0; i < NR; ++i) hdr[i].load(blk[i], quarter);
                    auto one = [&](auto g_tag) -> bool {
                        constexpr int G = decltype(g_tag)::value;
                        if (col * kSlotsPerCol + G >= n_slots) return true;  // the last run of a 32-weight-block type may be short
                        if (!slot_begin(col, G)) return false;
#pragma unroll
                        for (int i = 0; i < NR; ++i) {
                            uint32_t h[4] = {0u, 0u, 0u, 0u};
#if !(VQM_TC5_ABLATE & 1)
                            if (valid[i]) hdr[i].template chunk<G>(blk[i], quarter, h);
#endif
                            slot_put(col * kSlotsPerCol + G, i, h);
                        }
                        slot_done(col * kSlotsPerCol + G);
                        return true;
                    };
                    if (grp == 0) alive = one(Int<0>{}) && one(Int<2>{}) && one(Int<4>{}) && one(Int<6>{});
                    else alive = one(Int<1>{}) && one(Int<3>{}) && one(Int<5>{}) && one(Int<7>{});
                } else {
                    const int slots_here = n_slots - col * kSlotsPerCol < kSlotsPerCol ? n_slots - col * kSlotsPerCol : kSlotsPerCol;
#pragma unroll 1
                    for (int g = grp; g < slots_here; g += 2) {
                        if (!slot_begin(col, g)) {
                            alive = false;
                            break;
                        }
                        const int in_col = g * 4 + quarter;  // chunk within the column
#pragma unroll
                        for (int i = 0; i < NR; ++i) {
                            uint32_t h[4] = {0u, 0u, 0u, 0u};
                            if (valid[i]) {
                                float v[8];
                                deq8<TYPE>(static_cast<const uint8_t *>(__cvta_shared_to_generic(blk[i] + (in_col / CPB) * BB)), in_col % CPB, v, table);
                                to_f16(v, h);
                            }
                            slot_put(col * kSlotsPerCol + g, i, h);
                        }
                        slot_done(col * kSlotsPerCol + g);
                    }
                }
                if (alive) warp_arrive(s32(&s_raw_empty[col & 1]));  // hand the buffer back
            }
            // Only after a wait gave up: copies this thread queued and nobody waited for must land before the block may
            // leave (bounded; the columns complete in order).
            for (int col = raw_taken; col < raw_issued; ++col) {
#pragma unroll 1
                for (int i = 0; i < (1 << 16) && !bar_try(s32(&s_raw_full[col & 1]), (col >> 1) & 1); ++i) __nanosleep(64);
            }
        }
    } else if (warp == kLoadWarp) {
        // ---- activation tiles: one thread, one TMA tile copy per accumulator column block and stage (64 columns x kBN rows,
        //      written in the same 128-byte swizzle; no multicast; rows beyond ntok exist in the buffer and are zero).  A stage
        //      is refilled once the MMAs of its second half are done (MMAs complete in order).
        if (lane == 0) {
            // The kernel is launched while the conversion of the activations may still run (programmatic stream
            // serialization); this thread is the only reader of its output.
            asm volatile("griddepcontrol.wait;" ::: "memory");
            for (int k = 0; k < n_k; ++k) {
                const int stage = k % kTStages, use = k / kTStages;
                if (!bar_wait(s32(&s_empty[2 * stage + 1]), (use & 1) ^ 1, failed)) break;
                const uint32_t bar = s32(&s_xfull[stage]);
#if VQM_TC5_ABLATE & 2
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
#else
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(NH * kBN * 128) : "memory");
#pragma unroll
                for (int nh = 0; nh < NH; ++nh)
                    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                                     tiles + stage * kTStage + kTA + nh * kBN * 128),
                                 "l"(&x_map), "r"(k * kTK), "r"(tok0 + nh * kTNH + static_cast<int>(rank) * kBN), "r"(bar)
                                 : "memory");
#endif
            }
        }
    } else if (lane == 0 && rank != 0) {
        // ---- second block of a pair: tell the first block about every slot that is full here
        for (int q = 0; q < n_slots; ++q) {
            const int slot = q % kTSlots;
            if (!bar_wait(s32(&s_full[slot]), (q / kTSlots) & 1, failed)) break;
            if ((q & 1) == 0 && !bar_wait(s32(&s_xfull[slot >> 1]), (q / kTSlots) & 1, failed)) break;  // this block's activation tile too
            bar_arrive_cluster(in_block(s32(&s_full[slot]), 0));
        }
    } else if (lane == 0) {
        // ---- MMA issue (the first block of a pair issues for both): accumulator (mr, nh) at column (mr * NH + nh) * 256
        for (int q = 0; q < n_slots; ++q) {
            const int slot = q % kTSlots;
#if !(VQM_TC5_ABLATE & 8)
            if (!(PAIR ? bar_wait_cluster(s32(&s_full[slot]), (q / kTSlots) & 1, failed) : bar_wait(s32(&s_full[slot]), (q / kTSlots) & 1, failed))) break;
            if ((q & 1) == 0 && !bar_wait(s32(&s_xfull[slot >> 1]), (q / kTSlots) & 1, failed)) break;  // the stage's activation tile
#endif
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint64_t a_desc = sw128_desc(tiles + (slot >> 1) * kTStage), b_desc = sw128_desc(tiles + (slot >> 1) * kTStage + kTA);
#pragma unroll
            for (int jj = 0; jj < 2; ++jj) {  // 32 bytes further along K inside the swizzled rows per step
                const int j = (slot & 1) * 2 + jj;
                const uint32_t acc = (q | jj) != 0;
#pragma unroll
                for (int mr = 0; mr < MR; ++mr)
#pragma unroll
                    for (int nh = 0; nh < NH; ++nh) {  // accumulator (mr, nh): 128 weight rows (per block) x 256 activation rows
                        const uint64_t a = a_desc + 2 * j + ((mr * kTM * 128) >> 4), bd = b_desc + 2 * j + ((nh * kBN * 128) >> 4);
                        if constexpr (PAIR) mma_f16_pair(tmem + (mr * NH + nh) * 256, a, bd, acc);
                        else mma_f16(tmem + (mr * NH + nh) * 256, a, bd, acc);
                    }
            }
            // the slot is free again, in both blocks of a pair, once these MMAs have read it
            if constexpr (PAIR) mma_commit_pair(s32(&s_empty[slot]));
            else mma_commit(s32(&s_empty[slot]));
        }
        if constexpr (PAIR) mma_commit_pair(s32(&s_done));
        else mma_commit(s32(&s_done));
    }

    if (warp < 16) {
        // ---- epilogue: thread = weight row (TMEM lane) of each row half, loads of 32 columns.  A warp may read the 32 lanes
        //      (warp % 4) * 32 onwards, so the sixteen decoder warps work as four groups that share the column chunks.
        const bool ok = bar_wait(s32(&s_done), 0, failed);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int lane_group = warp & 3, col_group = warp >> 2;
        if (ok) {
#pragma unroll 1
            for (int cc = col_group; cc < MR * (kTN / 32); cc += 4) {
                const int mr = cc / (kTN / 32), c = cc % (kTN / 32);
                const int row = row0 + mr * kRowsPerAcc + lane_group * 32 + lane;
                uint32_t v[32];
                const uint32_t at = tmem + (static_cast<uint32_t>(lane_group * 32) << 16) + mr * kTN + c * 32;
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, "
                    "%18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
                      "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
                      "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
                      "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                    : "r"(at)
                    : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (row < rows) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int tok = tok0 + c * 32 + j;
                        if (tok < ntok) y[static_cast<size_t>(tok) * rows + row] = __uint_as_float(v[j]);
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if constexpr (PAIR) cluster_sync_all();  // neither block's shared or tensor memory goes away under the other
    if (warp == 0) {
        if constexpr (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
        else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
        if (lane == 0 && s_failed) atomicExch(status, kStatusWaitExpired);
    }
}

using PFN_encodeTiled = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                     const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

template <int TYPE, int MR, int NH, bool PAIR>
cudaError_t launch_shape(const uint8_t *w, const __half *xh, float *y, int rows, int cols, long long row_bytes, int ntok, const uint8_t *codebook,
                         unsigned *status, cudaStream_t stream) {
    constexpr size_t smem = tc5_smem_bytes(TYPE, MR, NH, PAIR, stages_for(TYPE, MR, NH, PAIR));
    static_assert(smem <= 227 * 1024, "shared memory of the tcgen05 GEMM");
    static bool configured = false;
    if (!configured) {
        const cudaError_t err =
            cudaFuncSetAttribute(qgemm_tc5_kernel<TYPE, MR, NH, PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (err != cudaSuccess) return err;
        configured = true;
    }
    constexpr int kRowsPerUnit = kTM * MR * (PAIR ? 2 : 1);  // weight rows of a block, or of a pair of blocks
    // The activations as a 2-D tensor [padded activation rows][cols] of fp16; a tile is 64 columns (one 128-byte swizzled
    // row each) of the activation rows one block holds of an accumulator.
    CUtensorMap x_map;
    {
        static PFN_encodeTiled encode = nullptr;
        if (encode == nullptr) {
            void *fn = nullptr;
            cudaDriverEntryPointQueryResult found;
            const cudaError_t err = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &found);
            if (err != cudaSuccess) return err;
            if (fn == nullptr || found != cudaDriverEntryPointSuccess) return cudaErrorNotSupported;
            encode = reinterpret_cast<PFN_encodeTiled>(fn);
        }
        const int tile = 2 * kTNH, padded = (ntok + tile - 1) / tile * tile;  // the runtime pads the buffer to gemm_tc5_token_tile()
        const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(padded)};
        const cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * 2};
        const cuuint32_t box[2] = {kTK, PAIR ? kTNH / 2 : kTNH}, elem[2] = {1, 1};
        if (encode(&x_map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half *>(xh), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((rows + kRowsPerUnit - 1) / kRowsPerUnit * (PAIR ? 2 : 1), (ntok + kTNH * NH - 1) / (kTNH * NH));
    cfg.blockDim = dim3(kTThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    // May start while the kernel before it in the stream (the fp32 -> fp16 conversion of the activations) still runs: the
    // set-up, the first weight copies and the first decoded tiles overlap it; the thread that feeds the activations waits for it.
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    int n_attr = 1;
    if constexpr (PAIR) {  // the two blocks of a pair form a cluster
        attr[n_attr].id = cudaLaunchAttributeClusterDimension;
        attr[n_attr].val.clusterDim.x = 2;
        attr[n_attr].val.clusterDim.y = 1;
        attr[n_attr].val.clusterDim.z = 1;
        ++n_attr;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    return cudaLaunchKernelEx(&cfg, qgemm_tc5_kernel<TYPE, MR, NH, PAIR>, x_map, w, y, rows, cols, row_bytes, ntok, codebook, status);
}

template <int TYPE>
cudaError_t launch_t(const uint8_t *w, const __half *xh, float *y, int rows, int cols, long long row_bytes, int ntok, const uint8_t *codebook,
                     unsigned *status, cudaStream_t stream) {
    // Which shape for which case was measured on 17408 x 5120 weights with 512 activation rows (times with the conversion
    // of the activations; VQM_TC5_SHAPE selects the alternatives in an experiment build):
    //   0  pairs of 1 x 2 blocks: 99-101 us for the four K-quants with a fast decoder, IQ4_XS 106, Q8_0 133 - the default
    //   1  single 1 x 2 blocks: the same for the K-quants, IQ4_XS 123, Q8_0 137
    //   2  2 x 1 (256 weight rows per block; pairs where the raw ring only fits beside a pair's smaller stages): 114-122;
    //      every weight is decoded once per 256 instead of once per 512 activation rows, which costs more than the halved
    //      activation traffic saves now that TMA feeds the activation tiles
    // Up to 256 activation rows: a pair of 1 x 1 blocks (90 us).
    if (ntok <= kTNH) return launch_shape<TYPE, 1, 1, true>(w, xh, y, rows, cols, row_bytes, ntok, codebook, status, stream);
#if VQM_TC5_SHAPE == 1
    return launch_shape<TYPE, 1, 2, false>(w, xh, y, rows, cols, row_bytes, ntok, codebook, status, stream);
#elif VQM_TC5_SHAPE == 2
    if constexpr (has_fast_chunk(TYPE) && fits_two_row_halves(TYPE, false)) {
        return launch_shape<TYPE, 2, 1, false>(w, xh, y, rows, cols, row_bytes, ntok, codebook, status, stream);
    } else if constexpr (has_fast_chunk(TYPE) && fits_two_row_halves(TYPE, true)) {
        return launch_shape<TYPE, 2, 1, true>(w, xh, y, rows, cols, row_bytes, ntok, codebook, status, stream);
    } else {
        return launch_shape<TYPE, 1, 2, true>(w, xh, y, rows, cols, row_bytes, ntok, codebook, status, stream);
    }
#else
    return launch_shape<TYPE, 1, 2, true>(w, xh, y, rows, cols, row_bytes, ntok, codebook, status, stream);
#endif
}

}  // namespace

int gemm_tc5_token_tile() { return 2 * kTNH; }  // the activation buffer is padded to the largest tile
bool gemm_tc5_supports(int cols) { return cols % kTK == 0; }

cudaError_t launch_qgemm_tc5(int type, const uint8_t *w, const void *xh, float *y, int rows, int cols, long long row_bytes, int ntok,
                             const uint8_t *codebook, unsigned *status, cudaStream_t stream) {
    const __half *x = static_cast<const __half *>(xh);
    switch (type) {
#define VQM_CASE(id, name) \
    case id: return launch_t<id>(w, x, y, rows, cols, row_bytes, ntok, codebook, status, stream);
        VQM_FOR_EACH_TYPE(VQM_CASE)
#undef VQM_CASE
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace vqm
