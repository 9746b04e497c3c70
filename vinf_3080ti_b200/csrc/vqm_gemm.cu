// Prompt-pass GEMM: Y[t][r] = sum_k W[r][k] X[t][k] for many activation rows (prefill), on the tensor cores.
//
// Replaces the reference's vinf_qgemm_kernel + f32_to_f16_rows_kernel (engine/csrc/megakernel/qwen_runtime.cu:655-769):
// W stays in raw GGUF blocks; a block of 8 warps owns 64 weight rows x 256 activation rows, dequantises a
// 64 x 32 tile of weights to fp16 in shared memory with the exact block decoders (each weight is decoded once per 256
// activation rows), brings the matching 256 x 32 tile of fp16 activations in with cp.async, and accumulates in fp32
// with mma.sync m16n8k16.  Like the reference's wmma kernel the operands are fp16 (weights and activations are
// rounded to fp16, products are exact, sums are fp32), and every output is a dot product in the same K order
// whatever the tiling.  Two shared-memory stages overlap the next tile's decode and copies with the MMAs.
//
// This is the warp-level tensor-core path (below tcgen05 throughput).  Passes of 64 activation rows or more take the
// tcgen05 kernel in vqm_gemm_tc5.cu; this one serves fewer rows and column counts that are not multiples of 64.  It is
// only used when the caller asks for it (set_gemm_min_rows), as in the reference; decode and verification passes always
// take the fp32 matvec.
#include <cuda_fp16.h>

#include "vqm_formats.cuh"
#include "vqm_kernels.h"

namespace vqm {
namespace {

constexpr int kBM = 64, kBN = 256, kBK = 32, kLd = kBK + 8;  // +8 halves: conflict-free ldmatrix rows
constexpr int kGemmThreads = 256;

// The GEMM that follows is launched with programmatic stream serialization: its blocks may set themselves up while this
// kernel still runs (they wait for its completion before they read xh), so the trigger comes first.
__global__ void __launch_bounds__(256) f32_to_f16_rows_kernel(const float *x, __half *xh, long long n_valid, long long n_total) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n_total) xh[i] = __float2half_rn(i < n_valid ? x[i] : 0.0f);
}
// Eight elements per thread: two 16-byte loads, one 16-byte store (x 16-byte aligned, both counts multiples of 8).
__global__ void __launch_bounds__(256) f32_to_f16_rows8_kernel(const float4 *x, uint4 *xh, long long n_valid8, long long n_total8) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n_total8) return;
    uint4 out = make_uint4(0u, 0u, 0u, 0u);
    if (i < n_valid8) {
        const float4 a = x[2 * i], b = x[2 * i + 1];
        const __half2 h0 = __floats2half2_rn(a.x, a.y), h1 = __floats2half2_rn(a.z, a.w), h2 = __floats2half2_rn(b.x, b.y),
                      h3 = __floats2half2_rn(b.z, b.w);
        out = make_uint4(*reinterpret_cast<const uint32_t *>(&h0), *reinterpret_cast<const uint32_t *>(&h1),
                         *reinterpret_cast<const uint32_t *>(&h2), *reinterpret_cast<const uint32_t *>(&h3));
    }
    xh[i] = out;
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int TYPE>
__global__ void __launch_bounds__(kGemmThreads) qgemm_kernel(const uint8_t *w, const __half *xh, float *y, int rows, int cols,
                                                              long long row_bytes, int ntok, const uint8_t *codebook) {
    constexpr int CPB = chunk_block(TYPE) / 8, BB = chunk_block_bytes(TYPE);
    constexpr int TABLE = grid_bytes(TYPE) > 0 ? grid_bytes(TYPE) : 16;
    extern __shared__ __align__(16) uint8_t gemm_smem[];
    uint8_t *table = gemm_smem;
    __half(*a_tile)[kBM * kLd] = reinterpret_cast<__half(*)[kBM * kLd]>(gemm_smem + TABLE);
    __half(*b_tile)[kBN * kLd] = reinterpret_cast<__half(*)[kBN * kLd]>(gemm_smem + TABLE + 2 * kBM * kLd * 2);
    if constexpr (grid_bytes(TYPE) > 0) {
        if constexpr (grid_is_codebook(TYPE)) {
            for (int i = threadIdx.x; i < grid_bytes(TYPE) / 4; i += blockDim.x)
                reinterpret_cast<uint32_t *>(table)[i] = reinterpret_cast<const uint32_t *>(codebook)[i];
        } else {
            if (threadIdx.x < 16) reinterpret_cast<float *>(table)[threadIdx.x] = kIq4Levels[threadIdx.x];
        }
        __syncthreads();
    }
    const int row0 = blockIdx.x * kBM, tok0 = blockIdx.y * kBN;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int wm = (warp >> 2) * 32, wn = (warp & 3) * 64;  // this warp's 32 rows x 64 activation rows

    // A: thread -> (row, 8-weight chunk) of the 64 x 32 tile; B: thread -> 4 x 16 bytes of the 256 x 32 tile
    const int a_row = threadIdx.x >> 2, a_kc = threadIdx.x & 3;
    const bool a_valid = row0 + a_row < rows;
    const uint8_t *w_row = w + static_cast<size_t>(a_valid ? row0 + a_row : 0) * row_bytes;

    auto fill = [&](int stage, int k0) {
        // dequantise 8 weights exactly, round to fp16, one 16-byte store
        float v[8];
        const int kc = (k0 >> 3) + a_kc;
        if (a_valid) {
            deq8<TYPE>(w_row + static_cast<size_t>(kc / CPB) * BB, kc % CPB, v, table);
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = 0.0f;
        }
        __half2 h[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
        *reinterpret_cast<uint4 *>(&a_tile[stage][a_row * kLd + a_kc * 8]) = *reinterpret_cast<const uint4 *>(h);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int piece = threadIdx.x + i * kGemmThreads, tok = piece >> 2, part = piece & 3;
            // rows of xh beyond ntok exist and are zero (the activation buffer is padded to a multiple of kBN)
            cp_async16(static_cast<uint32_t>(__cvta_generic_to_shared(&b_tile[stage][tok * kLd + part * 8])),
                       xh + static_cast<size_t>(tok0 + tok) * cols + k0 + part * 8);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    float acc[2][8][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.0f;

    const int n_k = cols / kBK;
    fill(0, 0);
    for (int it = 0; it < n_k; ++it) {
        const int stage = it & 1;
        if (it + 1 < n_k) {
            fill(stage ^ 1, (it + 1) * kBK);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const uint32_t a_base = static_cast<uint32_t>(__cvta_generic_to_shared(&a_tile[stage][0]));
        const uint32_t b_base = static_cast<uint32_t>(__cvta_generic_to_shared(&b_tile[stage][0]));
#pragma unroll
        for (int kk = 0; kk < kBK; kk += 16) {
            uint32_t a[2][4];
#pragma unroll
            for (int i = 0; i < 2; ++i)  // rows lane % 16, k half lane / 16
                ldmatrix_x4(a_base + ((wm + 16 * i + (lane & 15)) * kLd + kk + (lane >> 4) * 8) * 2, a[i][0], a[i][1], a[i][2], a[i][3]);
#pragma unroll
            for (int j = 0; j < 8; j += 2) {
                // two n8 tiles per ldmatrix.x4: matrices (n 0-7, k 0-7), (n 0-7, k 8-15), (n 8-15, k 0-7), (n 8-15, k 8-15)
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4(b_base + ((wn + 8 * j + (lane & 7) + ((lane >> 4) << 3)) * kLd + kk + ((lane >> 3) & 1) * 8) * 2, b0, b1, b2, b3);
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    mma_16816(acc[i][j], a[i], b0, b1);
                    mma_16816(acc[i][j + 1], a[i], b2, b3);
                }
            }
        }
        __syncthreads();  // the stage is refilled in the next iteration
    }
    // C fragment: rows lane / 4 (+8), activation rows (lane % 4) * 2 (+1)
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int row = row0 + wm + 16 * i + (lane >> 2) + (e >> 1) * 8;
                const int tok = tok0 + wn + 8 * j + (lane & 3) * 2 + (e & 1);
                if (row < rows && tok < ntok) y[static_cast<size_t>(tok) * rows + row] = acc[i][j][e];
            }
}

template <int TYPE>
cudaError_t launch_t(const uint8_t *w, const __half *xh, float *y, int rows, int cols, long long row_bytes, int ntok,
                     const uint8_t *codebook, cudaStream_t stream) {
    const dim3 grid((rows + kBM - 1) / kBM, (ntok + kBN - 1) / kBN);
    constexpr size_t smem = (grid_bytes(TYPE) > 0 ? grid_bytes(TYPE) : 16) + 2 * (kBM + kBN) * kLd * sizeof(__half);
    static bool configured = false;
    if (!configured) {
        const cudaError_t err = cudaFuncSetAttribute(qgemm_kernel<TYPE>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (err != cudaSuccess) return err;
        configured = true;
    }
    qgemm_kernel<TYPE><<<grid, kGemmThreads, smem, stream>>>(w, xh, y, rows, cols, row_bytes, ntok, codebook);
    return cudaGetLastError();
}

}  // namespace

int gemm_token_tile() { return kBN; }

cudaError_t launch_f32_to_f16_rows(const float *x, void *xh, long long n_valid, long long n_total, cudaStream_t stream) {
    if (n_valid % 8 == 0 && n_total % 8 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(xh) % 16 == 0) {
        const long long blocks = (n_total / 8 + 255) / 256;
        f32_to_f16_rows8_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(reinterpret_cast<const float4 *>(x), static_cast<uint4 *>(xh),
                                                                                   n_valid / 8, n_total / 8);
    } else {
        const long long blocks = (n_total + 255) / 256;
        f32_to_f16_rows_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(x, static_cast<__half *>(xh), n_valid, n_total);
    }
    return cudaGetLastError();
}

cudaError_t launch_qgemm(int type, const uint8_t *w, const void *xh, float *y, int rows, int cols, long long row_bytes, int ntok,
                         const uint8_t *codebook, cudaStream_t stream) {
    const __half *x = static_cast<const __half *>(xh);
    switch (type) {
#define VQM_CASE(id, name) \
    case id: return launch_t<id>(w, x, y, rows, cols, row_bytes, ntok, codebook, stream);
        VQM_FOR_EACH_TYPE(VQM_CASE)
#undef VQM_CASE
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace vqm
