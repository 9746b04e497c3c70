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
//   * One launch can cover up to four tensors that share x, the type and the columns (q/k/v, gate/up): the launch
//     numbers their rows consecutively and a chain of selects maps a row to its tensor's weights and outputs.
//   * Short launches (the rows would leave more than half of the warps idle) are split by columns: the blocks of a
//     thread-block cluster share a group of rows, one row per warp, and a share of the columns each; partial sums go
//     to the first block's shared memory (distributed shared memory), one cluster barrier, and that block adds them in
//     column order.  The split depends on the rows and columns only, never on M.
//   * Row-sharded launches (several GPUs) store every output into the gathered vector inside each rank's exchange
//     region as well (plain remote stores) and the last block to finish raises this rank's flag in every region; a
//     consumer launch waits, bounded, for the flags of its producer.
//   * Optional fused argmax over the rows (the LM head): every warp keeps the best (value, row) per
//     activation row, blocks write partials, the last block to finish reduces them.  Ties go to the
//     lowest row and a column with no value above -inf yields 0x7fffffff, like the reference's
//     argmax_kernel (engine/csrc/megakernel/qwen_runtime.cu:851-876).
//   * Every wait on an mbarrier is bounded; on expiry the warp records a code in the status word and
//     leaves the loop.
#pragma once

#include "vqm_kernels.h"
#include "vqm_steps.cuh"
#include "vqm_steps_kquants.cuh"
#include "vqm_steps_iq4.cuh"
#include "vqm_steps_grid.cuh"
#include "vqm_steps_plain.cuh"

namespace vqm {

constexpr int kWarps = 8;                      // warps per block
constexpr int kMaxTok = 8;                     // activation rows per launch
constexpr int kBarrierBytes = 1024;            // mbarriers and counters at the front of shared memory
// The kernels with the fused prologues and the residual add are separate instantiations (a second set of translation
// units, -DVQM_FUSED=1), so that the plain matvec carries none of their code.
#ifndef VQM_FUSED
#define VQM_FUSED 0
#endif
constexpr bool kFusedBuild = VQM_FUSED != 0;

// lookup tables at the front of shared memory: the type's codebook or level table, then (codebook types) the sign table
__host__ __device__ constexpr int table_bytes_padded(int type) {
    return (grid_bytes(type) + 15) / 16 * 16 + (grid_is_codebook(type) ? kSignTableBytes : 0);
}

// Blocks per SM the register allocation aims for: two, except for the tall chunks of wide passes (their sums alone
// take RW * M register pairs).  One-row chunks always get two, which the column split of short launches counts on.
#ifndef VQM_BLOCKS_SMALL_M
#define VQM_BLOCKS_SMALL_M 2
#endif
#ifndef VQM_BLOCKS_MID_M
#define VQM_BLOCKS_MID_M 2
#endif
#ifndef VQM_MIN_BLOCKS
#define VQM_MIN_BLOCKS(M, RW) ((RW) == 1 ? 2 : (M) <= 2 ? VQM_BLOCKS_SMALL_M : (M) <= 4 ? VQM_BLOCKS_MID_M : 1)
#endif
#ifndef VQM_MAX_STAGES
#define VQM_MAX_STAGES 4
#endif
#ifndef VQM_X_STAGES
#define VQM_X_STAGES 2
#endif

// Shared memory goes to the HBM stream first: two activation stages (the activations are small and sit in L2), then as
// many weight stages per warp (2..VQM_MAX_STAGES) as fit beside them when the kernel's blocks share an SM
// (228 KB per SM, 1 KB of it reserved per block, ~5 KB of static arrays per block).
template <int TYPE, int M, int RW>
__host__ __device__ constexpr int x_stages() {
    return VQM_X_STAGES;
}
template <int TYPE, int M, int RW>
__host__ __device__ constexpr int w_stages() {
    constexpr int fixed = table_bytes_padded(TYPE) + kBarrierBytes + x_stages<TYPE, M, RW>() * M * kSegCols * 4 + kWarps * Step<TYPE, M, RW>::kScratch;
    constexpr int budget = (VQM_MIN_BLOCKS(M, RW) >= 3 ? 70 : VQM_MIN_BLOCKS(M, RW) == 2 ? 108 : 200) * 1024;
    constexpr int s = (budget - fixed) / (kWarps * RW * slot_bytes(TYPE));
    return s < 2 ? 2 : s > VQM_MAX_STAGES ? VQM_MAX_STAGES : s;
}
template <int TYPE, int RW, int M>
__host__ __device__ constexpr size_t matvec_smem_bytes_for() {
    return static_cast<size_t>(table_bytes_padded(TYPE)) + kBarrierBytes + static_cast<size_t>(x_stages<TYPE, M, RW>()) * M * kSegCols * 4 +
           static_cast<size_t>(kWarps) * w_stages<TYPE, M, RW>() * RW * slot_bytes(TYPE) + static_cast<size_t>(kWarps) * Step<TYPE, M, RW>::kScratch;
}

// ---- mbarrier / bulk-copy primitives ---------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

// (barriers and staging buffers are named by their 32-bit shared-space addresses)
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

// One poll.  The instruction itself may suspend the thread for up to `hint_ns` nanoseconds while the phase is still open,
// so a waiting warp issues a handful of instructions instead of spinning.
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(hint_ns)
        : "memory");
    return ok != 0;
}

// Both kinds of bounded wait measure their limit in time (the global nanosecond timer), not in polls: how long a poll takes
// varies by orders of magnitude (the suspend-time hint is only an upper bound), and the order of the two limits matters -
// the wait for another rank's push comes first in a kernel, has the shorter limit and must be the one that reports.
constexpr unsigned long long kPeerWaitNs = 1000000000ull;   // 1 s
constexpr unsigned long long kMbarWaitNs = 4000000000ull;   // 4 s
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Bounded wait on an mbarrier: polls of up to ~20 microseconds each until kMbarWaitNs have passed (and at most 2^26 polls,
// whatever the timer says), then the caller reports the expiry.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity, 2000u)) return true;
    const unsigned long long t0 = global_ns();
#pragma unroll 1
    for (int i = 0; i < (1 << 26); ++i) {
        if (mbar_try_wait(bar, parity, 20000u)) return true;
        if ((i & 63) == 63 && global_ns() - t0 > kMbarWaitNs) break;
    }
    return false;
}

// One contiguous global -> shared copy of `bytes` (multiple of 16; both addresses 16-byte aligned),
// completion counted in bytes on `bar`.  No multicast.
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes),
                 "r"(bar)
                 : "memory");
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

__device__ __forceinline__ bool better(float v, int i, float bv, int bi) { return v > bv || (v == bv && i < bi); }

// Warp sums of N values at once: returns, in lane j < N, the sum over all lanes of v[j] - the same xor tree
// (offsets 16, 8, 4, 2, 1, in that order) as warp_sum for every value, so the result is bit-identical to N separate
// warp_sum calls, but while more than one value is left a step exchanges HALF of them: lanes whose offset bit is set keep
// the upper half and hand over the lower, the others the reverse.  P = N rounded up to a power of two; about 2P
// shuffles and adds instead of 5N.
template <int N>
__device__ __forceinline__ float warp_sums(float (&v)[N], int lane) {
    constexpr int P = N <= 1 ? 1 : N <= 2 ? 2 : N <= 4 ? 4 : N <= 8 ? 8 : N <= 16 ? 16 : 32;
    float w[P];
#pragma unroll
    for (int i = 0; i < P; ++i) w[i] = i < N ? v[i] : 0.0f;
    int count = P;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        if (count > 1) {
            const bool upper = (lane & off) != 0;
#pragma unroll
            for (int i = 0; i < count / 2; ++i) {
                const float keep = upper ? w[i + count / 2] : w[i], send = upper ? w[i] : w[i + count / 2];
                w[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
            }
            count /= 2;
        } else {
            w[0] += __shfl_xor_sync(0xffffffffu, w[0], off);
        }
    }
    // value j has ended up in the lanes whose top log2(P) bits spell j
    return __shfl_sync(0xffffffffu, w[0], (lane * (32 / P)) & 31);
}

// Where launch row g lives: the tensor's output vector and the row inside the tensor, plus the tensor's place in the
// gathered vectors of a row-sharded launch.  A chain of selects over the (at most kMaxParts) tensors; kernel
// parameters are only indexed with constants.
struct RowHome {
    float *y;
    int local, rows, rows_total, row_begin;
    long long dst_off;
};
__device__ __forceinline__ RowHome home_of(const MatvecArgs &a, int g) {
    RowHome h{a.part[0].y, g, a.part[0].rows, a.push.rows_total[0], a.push.row_begin[0], a.push.dst_off[0]};
#pragma unroll
    for (int i = 1; i < kMaxParts; ++i)
        if (g >= a.part[i - 1].row_end) h = RowHome{a.part[i].y, g - a.part[i - 1].row_end, a.part[i].rows, a.push.rows_total[i],
                                                     a.push.row_begin[i], a.push.dst_off[i]};
    return h;
}
// Address of the first byte of launch row g.
__device__ __forceinline__ uintptr_t row_address(const MatvecArgs &a, int g) {
    const uint8_t *w = a.part[0].w;
    int local = g;
#pragma unroll
    for (int i = 1; i < kMaxParts; ++i)
        if (g >= a.part[i - 1].row_end) {
            w = a.part[i].w;
            local = g - a.part[i - 1].row_end;
        }
    return reinterpret_cast<uintptr_t>(w) + static_cast<uintptr_t>(local) * static_cast<uintptr_t>(a.row_bytes);
}

// ---- the kernel ------------------------------------------------------------------------------------------

// FUSED: with the activation prologues and the residual add compiled in (kFusedBuild of the translation unit; a template
// parameter so that the two builds of a kernel are two different functions).
template <int TYPE, int M, int RW, bool FUSED>
__global__ void __launch_bounds__(kWarps * 32, VQM_MIN_BLOCKS(M, RW)) qmv_kernel(const MatvecArgs a) {
    using StepT = Step<TYPE, M, RW>;
    constexpr int S = w_stages<TYPE, M, RW>();
    constexpr int XS = x_stages<TYPE, M, RW>();
    constexpr int SLOT = slot_bytes(TYPE);
    constexpr int SEG = seg_bytes(TYPE);
    constexpr int TABLE = table_bytes_padded(TYPE);
    constexpr int XSTAGE = M * kSegCols * 4;
    constexpr bool kAligned = block_align(TYPE) >= 16;  // every segment starts on a 16-byte boundary
    static_assert(RW * M <= 32, "one lane per (row, activation row) output");
    static_assert(kWarps * 8 * 8 + 8 * 8 + 8 * 4 + 8 * 8 + kMaxTok * 4 <= kBarrierBytes, "barrier area");

    __shared__ float s_split[kMaxSplit][kWarps][kMaxTok];  // column split: partial sums of the cluster's blocks (first block's copy)
    extern __shared__ __align__(128) uint8_t smem[];
    // layout: lookup table | barriers: [kWarps][8] weight stages, [8] activation stages, [XS] "warps done" counters |
    //         XS activation stages | per warp S x RW weight slots | per warp decoder scratch
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t smem0 = smem_u32(smem);
    uint8_t *table = smem;
    int *xdone = reinterpret_cast<int *>(smem + TABLE + (kWarps * 8 + 8) * 8);
    const uint32_t xfull = smem0 + TABLE + kWarps * 8 * 8;
    const uint32_t xready = xfull + 8 * 8 + 8 * 4;  // fused prologue: "every thread has transformed its share of the stage"
    float *norm_scale = reinterpret_cast<float *>(smem + TABLE + (kWarps * 8 + 8) * 8 + 8 * 4 + 8 * 8);  // [kMaxTok]
    const uint32_t xbuf = smem0 + TABLE + kBarrierBytes;
    const uint32_t bar = smem0 + TABLE + warp * 64;
    const uint32_t buf = xbuf + XS * XSTAGE + warp * (S * RW * SLOT);
    const uint32_t scratch = xbuf + XS * XSTAGE + kWarps * (S * RW * SLOT) + warp * StepT::kScratch;

    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < S; ++s) mbar_init(bar + s * 8, 1);
    }
    if (threadIdx.x == 0) {
#pragma unroll
        for (int s = 0; s < XS; ++s) {
            mbar_init(xfull + s * 8, 1);
            mbar_init(xready + s * 8, kWarps * 32);
            xdone[s] = 0;
        }
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();

    // Even split of the rows over the warps: warp gw gets `my_count` consecutive rows from `my_begin`, taken in
    // `n_chunks` chunks of at most RW rows (chunk sizes differ by at most one).  n_chunks is the same for every warp,
    // so the warps of a block share the activation stages.  With a column split, the k_split blocks of a thread-block
    // cluster form a group that shares its rows (one per warp) and block `kpart` of the cluster takes its share of the
    // columns.
    const int k_split = a.k_split, n_groups = gridDim.x / k_split, group = blockIdx.x / k_split, kpart = blockIdx.x % k_split;
    const int total_warps = n_groups * kWarps, gw = group * kWarps + warp;
    const int base = a.rows / total_warps, rem = a.rows % total_warps;
    const int my_count = base + (gw < rem ? 1 : 0), my_begin = gw * base + (gw < rem ? gw : rem);
    const int n_chunks = (base + (rem > 0 ? 1 : 0) + RW - 1) / RW;
    const int chunk_base = my_count / n_chunks, chunk_rem = my_count % n_chunks;  // chunk c has chunk_base + (c < chunk_rem) rows
    // columns [col_begin, col_end) in n_seg segments of kSegCols (the last one may be shorter); the split is even in
    // units of 256 columns
    const int n_units = (a.cols + 255) / 256;
    const int col_begin = kpart * n_units / k_split * 256;
    const int col_end = (kpart + 1) * n_units / k_split * 256 < a.cols ? (kpart + 1) * n_units / k_split * 256 : a.cols;
    const int n_seg = (col_end - col_begin + kSegCols - 1) / kSegCols;
    constexpr int CB = chunk_block(TYPE), CBB = chunk_block_bytes(TYPE);
    const uint32_t byte_begin = static_cast<uint32_t>(col_begin / CB * CBB), byte_end = static_cast<uint32_t>(col_end / CB * CBB);
    const int cols_last = col_end - col_begin - (n_seg - 1) * kSegCols;                       // columns of the last segment
    const uint32_t len_last = byte_end - byte_begin - static_cast<uint32_t>(n_seg - 1) * SEG;  // and its bytes
    const uint32_t w_align = static_cast<uint32_t>(reinterpret_cast<uintptr_t>(a.part[0].w) & 15u);
    const uint32_t rb16 = static_cast<uint32_t>(a.row_bytes) & 15u;

    // Activation stage of segment `seg`: one bulk copy per activation row.  Called by one thread.
    auto issue_x = [&](int xstage, int seg) {
        const int col0 = col_begin + seg * kSegCols;
        const int cols_here = seg == n_seg - 1 ? cols_last : kSegCols;
        mbar_expect_tx(xfull + xstage * 8, static_cast<uint32_t>(M * cols_here * 4));
#pragma unroll
        for (int t = 0; t < M; ++t)
            bulk_copy_g2s(xbuf + xstage * XSTAGE + t * (kSegCols * 4), a.x + static_cast<size_t>(t) * a.cols + col0,
                          static_cast<uint32_t>(cols_here * 4), xfull + xstage * 8);
    };

    // Weight issue side, S stages ahead of the consumer: lane r (< rows of the chunk) owns row `i_row0 + r` and walks its
    // bytes one segment per call; `i_at` is where the lane's next segment starts in global memory.
    int i_chunk = 0, i_row0 = my_begin, i_nrows = chunk_base + (0 < chunk_rem ? 1 : 0), i_seg = 0;
    uintptr_t i_at = row_address(a, i_row0 + (lane < RW ? lane : 0)) + byte_begin;
    auto issue_w = [&](uint32_t stage_at, uint32_t i_bar) {  // the stage to fill and its barrier
        const uint32_t i_slot = stage_at + lane * SLOT;
        const uint32_t len = i_seg == n_seg - 1 ? len_last : static_cast<uint32_t>(SEG);
        if constexpr (kAligned) {
            if (lane == 0) mbar_expect_tx(i_bar, static_cast<uint32_t>(i_nrows) * len);
            __syncwarp();
            if (lane < i_nrows) bulk_copy_g2s(i_slot, reinterpret_cast<const void *>(i_at), len, i_bar);
        } else {
            // the copy is widened to 16-byte boundaries and keeps the segment's offset inside its 16-byte line
            const uint32_t lead = static_cast<uint32_t>(i_at) & 15u;
            const uint32_t bytes = lane < i_nrows ? (lead + len + 15u) & ~15u : 0u;
            const uint32_t total = __reduce_add_sync(0xffffffffu, bytes);
            if (lane == 0) mbar_expect_tx(i_bar, total);
            __syncwarp();
            if (bytes) bulk_copy_g2s(i_slot, reinterpret_cast<const void *>(i_at - lead), bytes, i_bar);
        }
        i_at += SEG;
        if (++i_seg == n_seg) {
            i_seg = 0;
            i_row0 += i_nrows;
            ++i_chunk;
            i_nrows = chunk_base + (i_chunk < chunk_rem ? 1 : 0);
            i_at = row_address(a, i_row0 + (lane < RW ? lane : 0)) + byte_begin;
        }
    };

    // The weights never depend on an earlier kernel, so their first copies go out at once; everything that reads the
    // activations or writes outputs comes after griddepcontrol.wait.  With programmatic dependent launch this block
    // may have started while the previous kernel of the stream was still draining, which hides the launch latency
    // and the first-byte latency of the weight stream (without that launch attribute both instructions are no-ops).
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // (chunks that hold rows come first: once a chunk without rows is reached, or the last chunk is passed, nothing is left)
#ifndef VQM_PURE_COMPUTE  // (experiment switch: no copies and no waits, the decoders run on whatever shared memory holds)
#pragma unroll 1
    for (int s = 0; s < S && i_chunk < n_chunks && i_nrows > 0; ++s) issue_w(buf + s * (RW * SLOT), bar + s * 8);
#endif
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (warp == 0 && a.push.wait_slot > 0) {
        // Row-sharded input: x was assembled by pushes from every rank.  Lane p waits (bounded) until rank p has pushed
        // the slot as often as this rank has - the flags are polled in parallel, one L2 round trip when they are
        // already up - then the ranks' stores are made visible to the bulk copies below.
        bool ok = *reinterpret_cast<volatile unsigned *>(a.status) == 0;  // after one expiry later kernels do not wait again
        if (lane < a.push.n_ranks && ok) {
            const volatile unsigned *flag = reinterpret_cast<const volatile unsigned *>(a.push.region[a.push.rank] + a.push.flag_off) +
                                            (a.push.wait_slot - 1) * 8 + lane;
            const unsigned target = *reinterpret_cast<const volatile unsigned *>(a.push.pushes + (a.push.wait_slot - 1));
            int spins = 0;
            auto acquire = [](const volatile unsigned *p) {
                unsigned v;
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
                return v;
            };
            unsigned long long t0 = 0;
            while (static_cast<int>(acquire(flag) - target) < 0) {
                ++spins;
                if (spins == 64) t0 = global_ns();  // a push that is merely in flight is seen long before this
                if ((spins > 64 && (spins & 255) == 0 && global_ns() - t0 > kPeerWaitNs) || spins > (1 << 26)) {
                    ok = false;
                    break;
                }
                __nanosleep(40);
            }
        }
        ok = __all_sync(0xffffffffu, ok);
        if (lane == 0) {
            if (!ok) atomicCAS(a.status, 0u, kStatusPeerWaitExpired);
            asm volatile("fence.proxy.async;" ::: "memory");  // the acquired stores, before the bulk copies read them
        }
        __syncwarp();
    }
    const int n_steps = n_chunks * n_seg;  // activation stages every warp of the block walks through
#ifndef VQM_PURE_COMPUTE
    if (threadIdx.x == 0) {
        const int n = n_steps < XS ? n_steps : XS;
        for (int s = 0; s < n; ++s) issue_x(s, s % n_seg);
    }
#endif

    if constexpr (TABLE > 0) {
        if constexpr (grid_is_codebook(TYPE)) {
            const uint32_t *src = reinterpret_cast<const uint32_t *>(a.codebook);
            for (int i = threadIdx.x; i < grid_bytes(TYPE) / 4; i += blockDim.x) reinterpret_cast<uint32_t *>(table)[i] = src[i];
            uint2 *sign_table = reinterpret_cast<uint2 *>(table + (grid_bytes(TYPE) + 15) / 16 * 16);
            for (int i = threadIdx.x; i < 256; i += blockDim.x) sign_table[i] = sign_table_entry(static_cast<uint32_t>(i), signs_have_parity(TYPE));
        } else {
            if (threadIdx.x < 16) reinterpret_cast<float *>(table)[threadIdx.x] = kIq4Levels[threadIdx.x];
        }
        __syncthreads();
    }

    // Fused prologue (engine/csrc/megakernel/qwen_megakernel.cu:486-550): v = silu(x) * x2 or x, then with rmsnorm
    // v * rsqrt(mean(v^2) + eps) * norm_w.  Every block computes the M scales over all columns once; the staged
    // segments are then transformed in place by all threads of the block before anyone reads them.
    const bool transform = FUSED && (a.fuse & (kFuseNorm | kFuseSiluMul)) != 0;
    auto activation = [&](int t, int col) {
        const float v = a.x[static_cast<size_t>(t) * a.cols + col];
        return (a.fuse & kFuseSiluMul) ? v / (1.0f + expf(-v)) * a.x2[static_cast<size_t>(t) * a.cols + col] : v;
    };
    if (FUSED && (a.fuse & kFuseNorm)) {
        __shared__ float s_part[kWarps];
        for (int t = 0; t < M; ++t) {
            float local = 0.0f;
            for (int col = threadIdx.x; col < a.cols; col += kWarps * 32) {
                const float v = activation(t, col);
                local = fmaf(v, v, local);
            }
            local = warp_sum(local);
            if (lane == 0) s_part[warp] = local;
            __syncthreads();
            if (threadIdx.x == 0) {
                float total = 0.0f;
                for (int w = 0; w < kWarps; ++w) total += s_part[w];
                norm_scale[t] = 1.0f / sqrtf(total / static_cast<float>(a.cols) + a.eps);
            }
            __syncthreads();
        }
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

    uint32_t c_stage = buf, c_bar = bar, phase = 0;  // the weight stage the consumer is at
    int xstage = 0;
    uint32_t xphase = 0;
    int row0 = my_begin;
    for (int chunk = 0; chunk < n_chunks && !expired; ++chunk) {
        const int nrows = chunk_base + (chunk < chunk_rem ? 1 : 0);  // warp-uniform; chunks without rows come last
        // d0: where row 0's segment starts inside its slot (the copy began at the 16-byte boundary below it)
        uint32_t d0 = kAligned ? 0u : (w_align + static_cast<uint32_t>(row0) * rb16 + byte_begin) & 15u;
        for (int seg = 0; seg < n_seg; ++seg) {
#ifndef VQM_PURE_COMPUTE
            if (!mbar_wait_bounded(xfull + xstage * 8, xphase)) {
                expired = true;
                break;
            }
#endif
            if (transform) {
                // this thread's share of the stage: columns 4 * tid .. 4 * tid + 3 of every activation row
                const int col0 = col_begin + seg * kSegCols, cols_here = seg == n_seg - 1 ? cols_last : kSegCols;
                const int c = 4 * static_cast<int>(threadIdx.x);
                if (c < cols_here) {
#pragma unroll
                    for (int t = 0; t < M; ++t) {
                        const uint32_t at = xbuf + xstage * XSTAGE + (t * kSegCols + c) * 4;
                        float v[4];
                        asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]) : "r"(at));
                        if (a.fuse & kFuseSiluMul) {
                            const float4 g = *reinterpret_cast<const float4 *>(a.x2 + static_cast<size_t>(t) * a.cols + col0 + c);
                            v[0] = v[0] / (1.0f + expf(-v[0])) * g.x;
                            v[1] = v[1] / (1.0f + expf(-v[1])) * g.y;
                            v[2] = v[2] / (1.0f + expf(-v[2])) * g.z;
                            v[3] = v[3] / (1.0f + expf(-v[3])) * g.w;
                        }
                        if (a.fuse & kFuseNorm) {
                            const float4 nw = *reinterpret_cast<const float4 *>(a.norm_w + col0 + c);
                            const float sc = norm_scale[t];
                            v[0] *= sc * nw.x;
                            v[1] *= sc * nw.y;
                            v[2] *= sc * nw.z;
                            v[3] *= sc * nw.w;
                        }
                        asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(at), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]) : "memory");
                    }
                }
                // a bounded block-wide rendezvous: everybody has written its share before anybody reads the stage
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(xready + xstage * 8) : "memory");
                if (!mbar_wait_bounded(xready + xstage * 8, xphase)) {
                    expired = true;
                    break;
                }
            }
            if (nrows > 0) {
#ifndef VQM_PURE_COMPUTE
                if (!mbar_wait_bounded(c_bar, phase)) {
                    expired = true;
                    break;
                }
#endif
#ifndef VQM_ABLATE_STEP
                StepT::run(c_stage, d0, kAligned ? 0u : rb16, scratch, smem0, xbuf + xstage * XSTAGE, seg == n_seg - 1 ? cols_last : kSegCols, nrows,
                           acc, lane);
#endif
            }
            __syncwarp();
            // Done with the activation stage; the last warp of the block to get here refills it.
#ifndef VQM_PURE_COMPUTE
            if (lane == 0) {
                __threadfence_block();
                if (atomicAdd(xdone + xstage, 1) == kWarps - 1) {
                    xdone[xstage] = 0;
                    __threadfence_block();
                    if (chunk * n_seg + seg + XS < n_steps) {
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                        issue_x(xstage, (seg + XS) % n_seg);
                    }
                }
            }
#endif
            if (++xstage == XS) {
                xstage = 0;
                xphase ^= 1u;
            }
            if (nrows > 0) {
#ifndef VQM_PURE_COMPUTE
                if (i_chunk < n_chunks && i_nrows > 0) issue_w(c_stage, c_bar);  // refill the stage just consumed
#endif
                c_stage += RW * SLOT;
                c_bar += 8;
                if (c_bar == bar + S * 8) {
                    c_bar = bar;
                    c_stage = buf;
                    phase ^= 1u;
                }
                if constexpr (!kAligned) d0 = (d0 + SEG) & 15u;
            }
        }
        if (expired) break;
#ifdef VQM_NO_EPILOGUE
        if (nrows > 1000) {
#else
        if (nrows > 0) {
#endif
            // lane r*M + t ends up holding y[t][row0 + r]
            float sums[RW * M];
#pragma unroll
            for (int r = 0; r < RW; ++r)
#pragma unroll
                for (int t = 0; t < M; ++t) {
                    float lo, hi;
                    unpack2(acc[r][t], lo, hi);
                    sums[r * M + t] = lo + hi;
                    acc[r][t] = 0ull;
                }
            float mine = 0.0f;
            if constexpr (RW * M > 16) {
                mine = warp_sums(sums, lane);  // (measured: pays above 16 sums; below, its selects cost registers)
            } else {
#pragma unroll
                for (int i = 0; i < RW * M; ++i) {
                    const float s = warp_sum(sums[i]);
                    if (lane == i) mine = s;
                }
            }
            if (lane < RW * M) {
                const int r = lane / M, t = lane % M, row = row0 + r;
                if (r < nrows) {
                    if (k_split > 1) {
                        // this block's share of the columns only: it goes into the shared memory of the cluster's first
                        // block, which adds the shares up (one-row chunks: r = 0, lane = t)
                        uint32_t remote;
                        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(&s_split[kpart][warp][t])), "r"(0));
                        asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(mine) : "memory");
                    } else {
                        mine *= StepT::kOutScale;  // exact: 1 or a power of two (see bytes_to_subpair)
                        const RowHome h = home_of(a, row);
                        if (FUSED && (a.fuse & kFuseAdd) && h.y != nullptr) mine += h.y[static_cast<size_t>(t) * h.rows + h.local];  // y += W x
                        if (h.y != nullptr) h.y[static_cast<size_t>(t) * h.rows + h.local] = mine;
                        if (a.push.push_slot > 0) {
                            // row-sharded: the value also goes straight into every rank's gathered [M][rows_total] vector
                            const size_t at = static_cast<size_t>(t) * h.rows_total + h.row_begin + h.local;
                            for (int p = 0; p < a.push.n_ranks; ++p) reinterpret_cast<float *>(a.push.region[p] + h.dst_off)[at] = mine;
                        }
                        if (want_argmax && better(mine, row, best_v, best_i)) {
                            best_v = mine;
                            best_i = row;
                        }
                    }
                }
            }
        }
        row0 += nrows;
    }

    if (expired) {
        if (lane == 0) atomicCAS(a.status, 0u, kStatusWaitExpired);  // the first cause stays
        // give the copies still in flight into this warp's buffers one more bounded chance to land
        for (int s = 0; s < S; ++s) (void)mbar_wait_bounded(bar + s * 8, 0);
    }

    if (k_split > 1) {
        // Every block of the cluster has left its partial sums in the first block's shared memory once the cluster
        // barrier completes; that block adds them in the order of the column ranges and owns the outputs.
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        if (kpart == 0 && threadIdx.x < kWarps * kMaxTok) {
            const int w = threadIdx.x / kMaxTok, t = threadIdx.x % kMaxTok, g = group * kWarps + w;
            const int row = g * base + (g < rem ? g : rem);
            if (t < M && base + (g < rem ? 1 : 0) > 0) {
                float sum = 0.0f;
                for (int k = 0; k < k_split; ++k) sum += s_split[k][w][t];
                sum *= StepT::kOutScale;
                const RowHome h = home_of(a, row);
                if (FUSED && (a.fuse & kFuseAdd) && h.y != nullptr) sum += h.y[static_cast<size_t>(t) * h.rows + h.local];
                if (h.y != nullptr) h.y[static_cast<size_t>(t) * h.rows + h.local] = sum;
                if (a.push.push_slot > 0) {
                    const size_t at = static_cast<size_t>(t) * h.rows_total + h.row_begin + h.local;
                    for (int p = 0; p < a.push.n_ranks; ++p) reinterpret_cast<float *>(a.push.region[p] + h.dst_off)[at] = sum;
                }
            }
        }
    }

    const bool want_push = a.push.push_slot > 0;
    if (want_argmax || want_push) {
        // block partials of the argmax, then the last block to finish reduces them and / or signals the push
        __shared__ float s_val[kWarps][32];
        __shared__ int s_idx[kWarps][32];
        __shared__ bool s_last;
        if (want_argmax) {
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
        }
        // Release at GPU scope: this block's stores (remote ones included) happen before its count below; the last
        // block's system-scope fence is cumulative over everything it has observed through the counter.
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence();  // after the barrier, cumulative over the stores of the whole block
            s_last = atomicAdd(a.done_counter, 1u) == gridDim.x - 1;
        }
        __syncthreads();
        if (s_last) {
            if (want_push) __threadfence_system();
            else __threadfence();
            if (want_argmax && warp < M) {
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
            if (want_push) {
                // every block made its remote stores visible (system-wide fence above) before it counted itself done:
                // write this rank's new push count of the slot into every rank's table, then remember it here
                const unsigned count = a.push.pushes[a.push.push_slot - 1] + 1u;
                if (threadIdx.x < a.push.n_ranks) {
                    volatile unsigned *flag = reinterpret_cast<volatile unsigned *>(a.push.region[threadIdx.x] + a.push.flag_off) +
                                              (a.push.push_slot - 1) * 8 + a.push.rank;
                    *flag = count;
                }
                __syncthreads();
                if (threadIdx.x == 0) a.push.pushes[a.push.push_slot - 1] = count;
            }
            if (threadIdx.x == 0) *a.done_counter = 0;
        }
    }
}

}  // namespace vqm
