// Prompt-pass GEMM on the 5th-generation tensor cores:  Y[t][r] = sum_k W[r][k] X[t][k]  for hundreds of activation rows.
//
// Same contract as the warp-level kernel in vqm_gemm.cu (replaces the reference's vinf_qgemm_kernel,
// engine/csrc/megakernel/qwen_runtime.cu:655-769: fp16 operands, fp32 accumulation), built on tcgen05:
//   * a block owns 128 weight rows (the MMA's M) and 512 activation rows (two accumulators of N = 256); the fp32
//     accumulators live in tensor memory (128 lanes x 512 columns, the whole TMEM of an SM, so one block per SM);
//   * K is walked in stages of 64, each filled and consumed as two halves of 32 (four pipeline slots in two stage
//     buffers): warps 0-15 dequantise the 128 x 32 weight half-tile with the exact block decoders (four threads per
//     row, one chunk of 8 weights each) and store it as fp16 in the K-major 128-byte-swizzled layout the tensor core
//     reads; warps 16-18 copy the 512 x 32 fp16 activation half-tile into the same layout with cp.async (the copies of
//     three slots in flight per thread); both sides make their writes visible to the async proxy and arrive on the
//     slot's "full" mbarrier;
//   * one thread of warp 19 issues, per slot, 2 K-steps x 2 accumulators of tcgen05.mma (kind::f16, M = 128, N = 256,
//     K = 16) from shared-memory descriptors and commits them to the slot's "empty" mbarrier, which hands the slot
//     back to the producers, so tile production runs up to three slots ahead of the MMAs;
//   * after the last commit, warps 0-3 read the accumulators with tcgen05.ld (warp w owns lanes 32w..32w+31, one
//     weight row per thread) and store y; a warp stores 32 consecutive rows of one activation row, 128 bytes.
// Every mbarrier wait is bounded: on expiry the block records a status code, everybody falls through to the end, and
// the tensor memory is released before the block returns.
#include <cuda_fp16.h>

#include "vqm_formats.cuh"
#include "vqm_kernels.h"

namespace vqm {
namespace {

constexpr int kTM = 128, kTN = 512, kTK = 64, kTStages = 2;
constexpr int kTA = kTM * kTK * 2, kTB = kTN * kTK * 2, kTStage = kTA + kTB;  // 16 KB + 64 KB
constexpr int kTSlots = 2 * kTStages;  // half stages
constexpr int kTThreads = 640;
constexpr int kAThreads = 512, kBThreads = 96;
constexpr uint32_t kTmemCols = 512;

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
// Bounded wait; also gives up as soon as another thread of the block has (`failed` is a shared flag).
__device__ __forceinline__ bool bar_wait(uint32_t bar, uint32_t parity, volatile int *failed) {
#pragma unroll 1
    for (int i = 0; i < (1 << 22); ++i) {
        if (bar_try(bar, parity)) return true;
        if (*failed) return false;
        if (i > 64) __nanosleep(32);
    }
    *failed = 1;
    return false;
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

template <int TYPE>
__global__ void __launch_bounds__(kTThreads, 1) qgemm_tc5_kernel(const uint8_t *w, const __half *xh, float *y, int rows, int cols,
                                                                 long long row_bytes, int ntok, const uint8_t *codebook,
                                                                 unsigned *status) {
    constexpr int CPB = chunk_block(TYPE) / 8, BB = chunk_block_bytes(TYPE);
    constexpr int TABLE = grid_bytes(TYPE) > 0 ? (grid_bytes(TYPE) + 15) / 16 * 16 : 16;
    extern __shared__ uint8_t tc5_raw[];
    __shared__ __align__(8) uint64_t s_full[kTSlots], s_empty[kTSlots], s_done;
    __shared__ uint32_t s_tmem;
    __shared__ int s_failed;
    // table first, then the stages on a 1024-byte boundary (the swizzle works on absolute shared-memory address bits)
    uint8_t *table = tc5_raw;
    const uint32_t tiles = (s32(tc5_raw) + TABLE + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = blockIdx.x * kTM, tok0 = blockIdx.y * kTN;
    const int n_k = cols / kTK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kTSlots; ++s) {
            bar_init(s32(&s_full[s]), kAThreads + kBThreads);
            bar_init(s32(&s_empty[s]), 1);
        }
        bar_init(s32(&s_done), 1);
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
    if (warp == 0) {  // tensor memory: all 512 columns (one block per SM)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(&s_tmem)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;
    volatile int *failed = &s_failed;

    const int n_slots = 2 * n_k;  // slot q of the pipeline: stage (q / 2) % 2, K half q % 2
    if (warp < 16) {
        // ---- weight half-tile: four threads per row, one chunk each; chunk c of the stage (8 weights, 16 bytes of fp16)
        //      goes to 16-byte slot c ^ (row % 8) of the row
        //      (the four threads of a row are neighbours in a warp: their global loads fall into the same sectors)
        const int r = threadIdx.x >> 2, quarter = threadIdx.x & 3;
        const bool valid = row0 + r < rows;
        const uint8_t *w_row = w + static_cast<size_t>(valid ? row0 + r : 0) * row_bytes;
        for (int q = 0; q < n_slots; ++q) {
            const int slot = q % kTSlots;
            if (!bar_wait(s32(&s_empty[slot]), ((q / kTSlots) & 1) ^ 1, failed)) break;
            const uint32_t a_row = tiles + (slot >> 1) * kTStage + r * 128;
            {
                const int c = (slot & 1) * 4 + quarter;   // chunk within the stage
                const int kc = (q >> 1) * (kTK / 8) + c;   // chunk within the row
                float v[8];
                if (valid) {
                    const uint8_t *blk = w_row + static_cast<size_t>(kc / CPB) * BB;
                    deq8<TYPE>(blk, kc % CPB, v, table);
                    // the row's bytes of the next stages: into L2 -> L1 ahead of use (hint only)
                    constexpr int kAhead = CPB == 32 ? BB : 4 * BB;
                    if (quarter == 0 && static_cast<long long>(kc / CPB) * BB + kAhead < row_bytes)
                        asm volatile("prefetch.global.L1 [%0];" ::"l"(blk + kAhead));
                } else {
#pragma unroll
                    for (int e = 0; e < 8; ++e) v[e] = 0.0f;
                }
                __half2 h[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) h[e] = __floats2half2_rn(v[2 * e], v[2 * e + 1]);
                const uint4 pk = *reinterpret_cast<const uint4 *>(h);
                asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(a_row + ((c ^ (r & 7)) << 4)), "r"(pk.x), "r"(pk.y), "r"(pk.z),
                             "r"(pk.w)
                             : "memory");
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            bar_arrive(s32(&s_full[slot]));
        }
    } else if (warp < 19) {
        // ---- activation half-tile: 512 rows x 4 chunks of 16 bytes, same swizzle; rows beyond ntok exist and are zero.
        //      The copies of up to three slots are in flight per thread (one cp.async group per slot).
        const int b = threadIdx.x - kAThreads;
        int issued = 0;
        bool alive = true;
        auto issue = [&]() {  // copies of slot `issued`, once the MMAs that read its previous contents are done
            const int slot = issued % kTSlots;
            if (!bar_wait(s32(&s_empty[slot]), ((issued / kTSlots) & 1) ^ 1, failed)) {
                alive = false;
                return;
            }
            const uint32_t b_tile = tiles + (slot >> 1) * kTStage + kTA;
            const __half *src = xh + static_cast<size_t>(tok0) * cols + (issued >> 1) * kTK + (slot & 1) * 32;
            for (int i = b; i < kTN * 4; i += kBThreads) {
                const int n = i >> 2, c = (slot & 1) * 4 + (i & 3);
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(b_tile + n * 128 + ((c ^ (n & 7)) << 4)),
                             "l"(src + static_cast<size_t>(n) * cols + (i & 3) * 8)
                             : "memory");
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
            ++issued;
        };
        while (alive && issued < n_slots && issued < 3) issue();
        for (int q = 0; alive && q < n_slots; ++q) {
            // groups complete in order: slot q has landed once at most (issued - q - 1) groups are still pending
            const int pending = issued - q - 1;
            if (pending >= 2) asm volatile("cp.async.wait_group 2;" ::: "memory");
            else if (pending == 1) asm volatile("cp.async.wait_group 1;" ::: "memory");
            else asm volatile("cp.async.wait_group 0;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            bar_arrive(s32(&s_full[q % kTSlots]));
            if (issued < n_slots) issue();
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
    } else if (lane == 0) {
        // ---- MMA issue: accumulator 0 (activation rows 0..255) at column 0, accumulator 1 at column 256
        for (int q = 0; q < n_slots; ++q) {
            const int slot = q % kTSlots;
            if (!bar_wait(s32(&s_full[slot]), (q / kTSlots) & 1, failed)) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint64_t a_desc = sw128_desc(tiles + (slot >> 1) * kTStage), b_desc = sw128_desc(tiles + (slot >> 1) * kTStage + kTA);
#pragma unroll
            for (int jj = 0; jj < 2; ++jj) {  // 32 bytes further along K inside the swizzled rows per step
                const int j = (slot & 1) * 2 + jj;
                const uint32_t acc = (q | jj) != 0;
                mma_f16(tmem, a_desc + 2 * j, b_desc + 2 * j, acc);
                mma_f16(tmem + 256, a_desc + 2 * j, b_desc + 2 * j + ((256 * 128) >> 4), acc);
            }
            mma_commit(s32(&s_empty[slot]));  // the slot is free again once these MMAs have read it
        }
        mma_commit(s32(&s_done));
    }

    if (warp < 4) {
        // ---- epilogue: thread = weight row (TMEM lane), 16 loads of 32 columns
        const bool ok = bar_wait(s32(&s_done), 0, failed);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int row = row0 + threadIdx.x;
        if (ok) {
#pragma unroll 1
            for (int c = 0; c < kTN / 32; ++c) {
                uint32_t v[32];
                const uint32_t at = tmem + (static_cast<uint32_t>(warp * 32) << 16) + c * 32;
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
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
        if (lane == 0 && s_failed) atomicExch(status, kStatusWaitExpired);
    }
}

template <int TYPE>
cudaError_t launch_t(const uint8_t *w, const __half *xh, float *y, int rows, int cols, long long row_bytes, int ntok, const uint8_t *codebook,
                     unsigned *status, cudaStream_t stream) {
    constexpr size_t smem = (grid_bytes(TYPE) > 0 ? (grid_bytes(TYPE) + 15) / 16 * 16 : 16) + 1024 + static_cast<size_t>(kTStages) * kTStage;
    static bool configured = false;
    if (!configured) {
        const cudaError_t err = cudaFuncSetAttribute(qgemm_tc5_kernel<TYPE>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (err != cudaSuccess) return err;
        configured = true;
    }
    const dim3 grid((rows + kTM - 1) / kTM, (ntok + kTN - 1) / kTN);
    qgemm_tc5_kernel<TYPE><<<grid, kTThreads, smem, stream>>>(w, xh, y, rows, cols, row_bytes, ntok, codebook, status);
    return cudaGetLastError();
}

}  // namespace

int gemm_tc5_token_tile() { return kTN; }
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
