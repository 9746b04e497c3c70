// Quantized matvec / small-M batched matmul for sm_100a:  y[t][r] = sum_k W[r][k] x[t][k],  t < M <= 8.
//
// Replaces the reference's vinf_qmatvec_kernel (engine/csrc/megakernel/qwen_runtime.cu:579-628).  W stays
// in raw GGUF block layout in HBM and is read exactly once for all M activation rows.
//
// Shape of the kernel
//   * Persistent grid; every WARP runs its own pipeline and owns row groups of RW consecutive rows.
//     Nothing is shared between warps except the read-only lookup table, so there is no block-wide
//     synchronisation in the steady state.
//   * A pipeline step covers kSegCols = 1024 columns of the warp's RW rows.  For each row the byte range
//     of that segment (rounded out to 16-byte boundaries) is fetched by one non-multicast bulk copy
//     (cp.async.bulk global -> shared) into a ring of S stages; completion is signalled on an mbarrier
//     per stage.  S stages of RW x ~0.3-4 KB per warp keep 100-190 KB per SM in flight.
//   * Decoding runs from shared memory, 8 weights (one "chunk") per lane at a time: lane l takes chunk
//     j*32 + l of the segment, so the activations are read fully coalesced (and once per RW rows) with
//     two 16-byte loads per activation row, and the staged bytes are read conflict-free.
//   * fp32 accumulation: per (row, activation row) an (even, odd) pair of partial sums updated with
//     packed fp32 FMAs, then a warp xor-shuffle tree.  The order of additions for an output does not
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
constexpr int kWarpSmemBudget = 12288;         // staging bytes a warp aims for

// Bytes of one row's segment and of the shared-memory slot that receives it (the copy is widened to
// 16-byte boundaries on both sides: up to 14 bytes in front, and the decoders' funnel loads may touch
// up to 4 bytes behind).
__host__ __device__ constexpr int seg_bytes(int type) { return kSegCols / chunk_block(type) * chunk_block_bytes(type); }
__host__ __device__ constexpr int slot_bytes(int type) { return (seg_bytes(type) + 14 + 8 + 15) / 16 * 16; }
__host__ __device__ constexpr int stages_for(int type, int rw) {
    const int s = kWarpSmemBudget / (rw * slot_bytes(type));
    return s < 2 ? 2 : s > 8 ? 8 : s;
}
__host__ __device__ constexpr int table_bytes_padded(int type) { return (grid_bytes(type) + 15) / 16 * 16; }
__host__ __device__ constexpr size_t matvec_smem_bytes(int type, int rw) {
    return static_cast<size_t>(table_bytes_padded(type)) + kWarps * 8 * 8 +
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

// acc.{x,y} += a.{x,y} * b.{x,y} as one packed instruction (two fp32 FMAs per lane per issue slot).
__device__ __forceinline__ void ffma2(float2 &acc, float a0, float a1, float b0, float b1) {
#ifdef VQM_NO_F32X2
    acc.x = fmaf(a0, b0, acc.x);
    acc.y = fmaf(a1, b1, acc.y);
#else
    unsigned long long c, a, b;
    asm("mov.b64 %0, {%1, %2};" : "=l"(c) : "f"(acc.x), "f"(acc.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(a) : "f"(a0), "f"(a1));
    asm("mov.b64 %0, {%1, %2};" : "=l"(b) : "f"(b0), "f"(b1));
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(c) : "l"(a), "l"(b));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(acc.x), "=f"(acc.y) : "l"(c));
#endif
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

__device__ __forceinline__ bool better(float v, int i, float bv, int bi) { return v > bv || (v == bv && i < bi); }

// ---- the kernel ------------------------------------------------------------------------------------------

template <int TYPE, int M, int RW>
__global__ void __launch_bounds__(kWarps * 32, (M <= 4 ? 2 : 1)) qmv_kernel(const MatvecArgs a) {
    constexpr int S = stages_for(TYPE, RW);
    constexpr int SLOT = slot_bytes(TYPE);
    constexpr int SEG = seg_bytes(TYPE);
    constexpr int CPB = chunk_block(TYPE) / 8;  // chunks per block
    constexpr int BB = chunk_block_bytes(TYPE);
    constexpr int TABLE = table_bytes_padded(TYPE);
    static_assert(RW * M <= 32, "one lane per (row, activation row) output");

    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t *table = smem;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + TABLE);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint64_t *bar = bars + warp * 8;
    uint8_t *buf = smem + TABLE + kWarps * 8 * 8 + static_cast<size_t>(warp) * (S * RW * SLOT);

    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < S; ++s) mbar_init(bar + s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp();

    // This warp's row groups: first, first + total_warps, ...  (warps of one block are spread over the
    // row range so that a short tensor still touches every SM).
    const int total_warps = gridDim.x * kWarps;
    const int first = warp * gridDim.x + blockIdx.x;
    const int n_rg = (a.rows + RW - 1) / RW;
    const int my_rg = first < n_rg ? (n_rg - first + total_warps - 1) / total_warps : 0;
    const int n_seg = (a.cols + kSegCols - 1) / kSegCols;
    const int n_steps = my_rg * n_seg;
    const uintptr_t wbase = reinterpret_cast<uintptr_t>(a.w);

    auto issue = [&](int step) {
        const int rg = first + (step / n_seg) * total_warps, seg = step % n_seg, stage = step % S;
        const int row = rg * RW + lane;
        uint32_t bytes = 0;
        uintptr_t src = 0;
        if (lane < RW && row < a.rows) {
            const long long off = static_cast<long long>(seg) * SEG;
            const long long len = a.row_bytes - off < SEG ? a.row_bytes - off : SEG;
            const uintptr_t p = wbase + static_cast<uintptr_t>(row) * a.row_bytes + off;
            src = p & ~static_cast<uintptr_t>(15);
            bytes = static_cast<uint32_t>((p - src + len + 15) & ~static_cast<uintptr_t>(15));
        }
        const uint32_t total = __reduce_add_sync(0xffffffffu, bytes);
        if (lane == 0) mbar_expect_tx(bar + stage, total);
        __syncwarp();
        if (bytes) bulk_copy_g2s(buf + (stage * RW + lane) * SLOT, reinterpret_cast<const void *>(src), bytes, bar + stage);
    };

    const int prologue = n_steps < S ? n_steps : S;
    for (int s = 0; s < prologue; ++s) issue(s);

    if constexpr (TABLE > 0) {
        if constexpr (grid_is_codebook(TYPE)) {
            const uint32_t *src = reinterpret_cast<const uint32_t *>(a.codebook);
            for (int i = threadIdx.x; i < grid_bytes(TYPE) / 4; i += blockDim.x) reinterpret_cast<uint32_t *>(table)[i] = src[i];
        } else {
            if (threadIdx.x < 16) reinterpret_cast<float *>(table)[threadIdx.x] = kIq4Levels[threadIdx.x];
        }
        __syncthreads();
    }

    float2 acc[RW][M];
#pragma unroll
    for (int r = 0; r < RW; ++r)
#pragma unroll
        for (int t = 0; t < M; ++t) acc[r][t] = make_float2(0.0f, 0.0f);
    float best_v = -INFINITY;
    int best_i = 0x7fffffff;
    const bool want_argmax = a.out_idx != nullptr;
    bool expired = false;

    for (int step = 0; step < n_steps; ++step) {
        const int stage = step % S;
        if (!mbar_wait_bounded(bar + stage, (step / S) & 1)) {
            expired = true;
            break;
        }
        const int rg = first + (step / n_seg) * total_warps, seg = step % n_seg;
        const int row0 = rg * RW;
        const uint8_t *stage_buf = buf + stage * RW * SLOT;
        // where each row's segment starts inside its slot (the copy began at the 16-byte boundary below it)
        uint32_t delta[RW];
#pragma unroll
        for (int r = 0; r < RW; ++r)
            delta[r] = static_cast<uint32_t>((wbase + static_cast<uintptr_t>(row0 + r) * a.row_bytes +
                                              static_cast<uintptr_t>(seg) * SEG) & 15u);
#pragma unroll 1
        for (int j = 0; j < kChunksPerLane; ++j) {
            const int chunk = j * 32 + lane;
            const int col = seg * kSegCols + chunk * 8;
            if (col < a.cols) {
                float4 xa[M], xb[M];
#pragma unroll
                for (int t = 0; t < M; ++t) {
                    const float4 *xp = reinterpret_cast<const float4 *>(a.x + static_cast<size_t>(t) * a.cols + col);
                    xa[t] = __ldg(xp);
                    xb[t] = __ldg(xp + 1);
                }
                const int boff = (chunk / CPB) * BB, c = chunk % CPB;
#pragma unroll
                for (int r = 0; r < RW; ++r) {
                    if (row0 + r < a.rows) {
                        float v[8];
                        deq8<TYPE>(stage_buf + r * SLOT + delta[r] + boff, c, v, table);
#pragma unroll
                        for (int t = 0; t < M; ++t) {
                            ffma2(acc[r][t], v[0], v[1], xa[t].x, xa[t].y);
                            ffma2(acc[r][t], v[2], v[3], xa[t].z, xa[t].w);
                            ffma2(acc[r][t], v[4], v[5], xb[t].x, xb[t].y);
                            ffma2(acc[r][t], v[6], v[7], xb[t].z, xb[t].w);
                        }
                    }
                }
            }
        }
        __syncwarp();
        if (step + S < n_steps) issue(step + S);

        if (seg == n_seg - 1) {
            // lane r*M + t ends up holding y[t][row0 + r]
            float mine = 0.0f;
#pragma unroll
            for (int r = 0; r < RW; ++r)
#pragma unroll
                for (int t = 0; t < M; ++t) {
                    const float s = warp_sum(acc[r][t].x + acc[r][t].y);
                    if (lane == r * M + t) mine = s;
                    acc[r][t] = make_float2(0.0f, 0.0f);
                }
            if (lane < RW * M) {
                const int r = lane / M, t = lane % M, row = row0 + r;
                if (row < a.rows) {
                    if (a.y != nullptr) a.y[static_cast<size_t>(t) * a.rows + row] = mine;
                    if (want_argmax && better(mine, row, best_v, best_i)) {
                        best_v = mine;
                        best_i = row;
                    }
                }
            }
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
